"""Stream-K launches of the grouped-head 8-bit kernel (equal ranges of the batch's token groups per CTA, rows cut
into pieces wherever a range ends): parity against the CPU oracle on shapes small enough for the oracle, with the
threshold lowered so that they take the stream-K path."""
import dataclasses

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL, gpu_step_and_compare

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _force(monkeypatch):
    monkeypatch.setenv("DX_ATTN_SK_MIN_UNITS", "1")
    monkeypatch.setenv("DX_ATTN_SK_ROW_FACTOR", "1000000")
    monkeypatch.setenv("DX_ATTN_STREAMK_16BIT", "1")


@pytest.mark.parametrize("cache", ["fp8", "int8", "none"])
@pytest.mark.parametrize("heads,dh", [((8, 1), 128), ((64, 8), 128), ((16, 1), 128), ((24, 1), 64), ((8, 2), 64)])
def test_ragged_batches(pkg, cache, heads, dh):
    cfg = workloads.DecodeConfig("sk", 7, heads[0], heads[1], dh, torch.bfloat16, cache, 64, 20, 3000, True, 77)
    r = gpu_step_and_compare(pkg, cfg)
    # (24 heads on one kv head with an FP8 cache run on the wide-group kernel, which has no stream-K form)
    if cache == "none":
        assert r["plan"].get("stream_k_ctas", 0) > 0, r["plan"]
    assert r["plan"]["kernel"] != "gqa_tensor_core" or r["plan"].get("stream_k_ctas", 0) > 0, r["plan"]


def test_many_short_rows_and_boundary_lengths(pkg):
    lens = [0, 1, 31, 32, 33, 63, 64, 65, 95, 96, 127, 128, 129, 255, 256, 257, 517, 1023, 1024, 1025, 2047, 2048]
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=len(lens))
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"].get("stream_k_ctas", 0) > 0


def test_one_long_row_cut_into_many_pieces(pkg):
    cfg = workloads.DecodeConfig("sk1", 1, 8, 1, 128, torch.bfloat16, "fp8", 128, 30000, 30000, True, 5)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"].get("stream_k_ctas", 0) > 100


def test_host_lengths_may_be_upper_bounds(pkg):
    """A captured graph replays with the host lengths it was planned with while the device lengths are the real
    (shorter) ones: pieces scheduled beyond the real length are empty, the result is that of the real length."""
    wl = workloads
    cfg = wl.DecodeConfig("skub", 6, 32, 4, 128, torch.bfloat16, "fp8", 64, 100, 1500, True, 9)
    w_cpu = wl.build_workload(cfg, "cpu")
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        bound = w_cpu.host_past_key_value_lengths + torch.tensor([0, 5, 40, 333, 1000, 64], dtype=torch.int32)
        M = w.kv_cache_block_pointers.shape[-1]
        bound = torch.clamp(bound, max=M * cfg.tokens_per_block - 1)
        assert plugin.plan(cfg.batch, int(bound.max()), bound).get("stream_k_ctas", 0) > 0
        out = plugin.enqueue_generation(w.qkv, w.sequence_length, bound, w.kv_cache_block_pointers,
                                        w.kv_orig_quant_scale, w.kv_quant_orig_scale)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
        pool_ref = w_cpu.pool.clone()
        ref = oracle.decode_attention_reference(
            w_cpu.qkv, w_cpu.sequence_length, pool_ref, w_cpu.offset_table, num_heads=cfg.num_heads,
            num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block,
            cache_mode=CACHE_MODE[cfg.cache], kv_scale_orig_quant=w_cpu.scale_orig_quant,
            kv_scale_quant_orig=w_cpu.scale_quant_orig)
        assert torch.equal(w.pool.cpu(), pool_ref)
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL
    finally:
        plugin.close()


def test_switch_and_threshold_keep_the_classic_plan(pkg, monkeypatch):
    cfg = workloads.DecodeConfig("skoff", 4, 8, 1, 128, torch.bfloat16, "fp8", 64, 200, 900, True, 3)
    monkeypatch.setenv("DX_ATTN_STREAMK", "0")
    r = gpu_step_and_compare(pkg, cfg, check_twice=False)
    assert "stream_k_ctas" not in r["plan"]
    monkeypatch.delenv("DX_ATTN_STREAMK")
    monkeypatch.delenv("DX_ATTN_SK_MIN_UNITS")  # default thresholds: this batch is far too small
    monkeypatch.delenv("DX_ATTN_SK_ROW_FACTOR")
    monkeypatch.delenv("DX_ATTN_STREAMK_16BIT")
    r = gpu_step_and_compare(pkg, cfg, check_twice=False)
    assert "stream_k_ctas" not in r["plan"]


@pytest.mark.parametrize("heads,tpb", [((8, 1), 64), ((64, 8), 128), ((16, 1), 32), ((12, 2), 64)])
def test_token_major_kernel_ragged_batches(pkg, monkeypatch, heads, tpb):
    """The tcgen05 token-major kernel under the same schedule (unit: its 128-token tile)."""
    monkeypatch.setenv("DX_ATTN_TOK", "1")
    cfg = workloads.DecodeConfig("sktok", 7, heads[0], heads[1], 128, torch.bfloat16, "fp8", tpb, 20, 3000, True, 78)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"]["kernel"] == "token_major_tcgen05" and r["plan"].get("stream_k_ctas", 0) > 0, r["plan"]


def test_token_major_kernel_boundary_lengths_and_long_row(pkg, monkeypatch):
    monkeypatch.setenv("DX_ATTN_TOK", "1")
    lens = [0, 1, 31, 32, 33, 63, 64, 65, 95, 96, 127, 128, 129, 255, 256, 257, 517, 1023, 1024, 1025, 2047, 2048]
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=len(lens))
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"].get("stream_k_ctas", 0) > 0
    cfg = workloads.DecodeConfig("sktok1", 1, 8, 1, 128, torch.bfloat16, "fp8", 128, 30000, 30000, True, 5)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"].get("stream_k_ctas", 0) > 100


@pytest.mark.parametrize("heads,tpb", [((8, 1), 64), ((64, 8), 128), ((16, 2), 32), ((6, 2), 64)])
def test_six_warp_form_ragged_batches(pkg, monkeypatch, heads, tpb):
    """The form with two six-warp CTAs per SM (FP8, Dh 128, up to 8 heads per kv head), which launches with long
    ranges use: forced here on small ragged batches, boundary lengths and one long row."""
    monkeypatch.setenv("DX_ATTN_SK_SIX_MIN_TOKENS", "1")
    cfg = workloads.DecodeConfig("sk6", 7, heads[0], heads[1], 128, torch.bfloat16, "fp8", tpb, 20, 3000, True, 79)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"].get("stream_k_ctas", 0) > 0 and r["plan"]["stream_k_ctas"] <= 2 * 148, r["plan"]
    lens = [0, 1, 31, 32, 33, 63, 64, 65, 95, 96, 127, 128, 129, 255, 256, 257, 517, 1023, 1024, 1025, 2047, 2048]
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=len(lens), tokens_per_block=tpb if tpb >= 32 else 64)
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert 0 < r["plan"].get("stream_k_ctas", 0) <= 2 * 148
    cfg = workloads.DecodeConfig("sk6l", 1, heads[0] // heads[1], 1, 128, torch.float16, "fp8", 128, 30000, 30000, True, 6)
    r = gpu_step_and_compare(pkg, cfg)
    assert 100 < r["plan"].get("stream_k_ctas", 0) <= 2 * 148
