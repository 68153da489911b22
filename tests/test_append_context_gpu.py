"""Context-phase KV append (the writer that fills the paged cache before decoding starts): CUDA path
through the C ABI against the oracle, bit-exact, and a prompt -> decode round trip that uses the
library's own writer for the cache the decode step then reads."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL, REPORT_DIR

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _setup(pkg, cfg, lens, seed=11, scale=None):
    wl = workloads
    w = wl.build_workload(cfg, "cpu", lengths=lens)  # only for the pool geometry and the page table
    g = torch.Generator().manual_seed(seed)
    L = int(lens.max())
    k = torch.randn(cfg.batch, cfg.num_kv_heads, L, cfg.head_size, generator=g).to(cfg.dtype)
    v = torch.randn(cfg.batch, cfg.num_kv_heads, L, cfg.head_size, generator=g).to(cfg.dtype)
    return w, k, v, L


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cache", ["none", "int8", "fp8"])
@pytest.mark.parametrize("dh,tpb", [(64, 16), (128, 64), (128, 128)])
def test_append_matches_oracle_bit_exact(pkg, dtype, cache, dh, tpb):
    wl = workloads
    cfg = wl.DecodeConfig("ctx", 4, 6, 3, dh, dtype, cache, tpb, 1, 300, True, 17)
    lens = torch.tensor([1, tpb, tpb + 1, 300], dtype=torch.int32)
    w, k, v, L = _setup(pkg, cfg, lens)
    pool_ref = torch.zeros_like(w.pool)
    oracle.append_context_reference(k, v, lens, pool_ref, w.offset_table, tokens_per_block=tpb,
                                    cache_mode=CACHE_MODE[cache], kv_scale_orig_quant=w.scale_orig_quant)
    wd = wl.to_device(w, "cuda:0")
    wd.pool.zero_()
    plugin = wl.make_plugin(cfg, 0)
    try:
        plugin.append_context(k.cuda(), v.cuda(), lens.cuda(), wd.kv_cache_block_pointers, wd.kv_orig_quant_scale)
        torch.cuda.synchronize()
        assert torch.equal(wd.pool.cpu(), pool_ref)  # bytes and positions; nothing else touched (pool was zero)
    finally:
        plugin.close()


@pytest.mark.parametrize("cache", ["none", "int8", "fp8"])
@pytest.mark.parametrize("tpb,blocks,window,sink", [
    (64, 8, 512, 0),    # table exactly as long as the window: slot = t % 512
    (64, 9, 512, 0),    # spare block: 576 slots cycle
    (64, 7, 448, 64),   # one whole sink block kept in place, 384 slots cycle behind it
    (64, 8, 300, 4),    # sink tokens end inside a block: the rest of that block stays unused
    (16, 8, 100, 5),
])
def test_append_with_a_window_shorter_than_the_prompt(pkg, cache, tpb, blocks, window, sink):
    """Cyclic cache in the context phase (unfusedAttentionKernels.cu:1591-1600 with the slots of
    kvCacheUtils.h:109-117): only the last `window` tokens are stored, at their cyclic slots; bit-exact against the
    oracle, whose slot arithmetic is pinned against the reference header (test_oracle_golden)."""
    wl = workloads
    cfg = wl.DecodeConfig("ctxw", 4, 6, 3, 128, torch.bfloat16, cache, tpb, 1, blocks * tpb, True, 19)
    # shorter than the window, exactly the window, a little longer, several times around
    lens = torch.tensor([max(1, window // 3), window, window + tpb + 3, 3 * window + 7], dtype=torch.int32)
    w = wl.build_workload(cfg, "cpu", lengths=torch.full((4,), blocks * tpb - 1, dtype=torch.int32))
    g = torch.Generator().manual_seed(23)
    L = int(lens.max())
    k = torch.randn(cfg.batch, cfg.num_kv_heads, L, cfg.head_size, generator=g).to(cfg.dtype)
    v = torch.randn(cfg.batch, cfg.num_kv_heads, L, cfg.head_size, generator=g).to(cfg.dtype)
    pool_ref = torch.zeros_like(w.pool)
    oracle.append_context_reference(k, v, lens, pool_ref, w.offset_table, tokens_per_block=tpb,
                                    cache_mode=CACHE_MODE[cache], kv_scale_orig_quant=w.scale_orig_quant,
                                    attention_window_size=window, sink_token_length=sink)
    wd = wl.to_device(w, "cuda:0")
    wd.pool.zero_()
    plugin = wl.make_plugin(cfg, 0)
    try:
        plugin.append_context(k.cuda(), v.cuda(), lens.cuda(), wd.kv_cache_block_pointers, wd.kv_orig_quant_scale,
                              attention_window_size=window, sink_token_length=sink)
        torch.cuda.synchronize()
        assert torch.equal(wd.pool.cpu(), pool_ref)
    finally:
        plugin.close()


def test_append_refuses_a_table_shorter_than_the_cycle(pkg):
    wl = workloads
    cfg = wl.DecodeConfig("ctxw", 1, 4, 2, 128, torch.bfloat16, "fp8", 64, 1, 256, True, 19)
    w = wl.to_device(wl.build_workload(cfg, "cpu", lengths=torch.tensor([255], dtype=torch.int32)), "cuda:0")
    k = torch.zeros(1, 2, 600, 128, dtype=torch.bfloat16, device="cuda:0")
    lens = torch.tensor([600], dtype=torch.int32, device="cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        table = w.kv_cache_block_pointers  # 4 blocks = 256 slots
        with pytest.raises(pkg.DecodeAttnError) as e:  # a window of 512 tokens cannot cycle in 256 slots
            plugin.append_context(k, k, lens, table, w.kv_orig_quant_scale, attention_window_size=512)
        assert e.value.status == pkg.plugin.DX_ERR_BAD_ARG
        with pytest.raises(pkg.DecodeAttnError) as e:  # the sink tokens must leave room in the window
            plugin.append_context(k, k, lens, table, w.kv_orig_quant_scale, attention_window_size=128, sink_token_length=128)
        assert e.value.status == pkg.plugin.DX_ERR_BAD_ARG
        plugin.append_context(k, k, lens, table, w.kv_orig_quant_scale, attention_window_size=256)  # fits exactly
        torch.cuda.synchronize()
    finally:
        plugin.close()


def test_append_known_answer_inputs(pkg):
    """Inputs of the reference known-answer test (srand(42), values in [0, 10], scale 0.1;
    cpp/tests/runtime/transposeKVKernelTest.cpp:152-225) through the product writer, fp16 activations:
    INT8 bytes equal the test's expectation exactly; FP8 bytes equal the kernel chain (oracle) exactly and the
    test's float-product expectation on all but a few ties of the half product."""
    wl = workloads
    qg = np.load(GOLDEN / "quant_golden.npz")
    x = torch.from_numpy(qg["kat_x"]).to(torch.float16)  # 4096 values = [B 2, H 1, L 16, Dh 128]
    for cache, key in (("int8", "kat_int8"), ("fp8", "kat_fp8")):
        cfg = wl.DecodeConfig("kat", 2, 1, 1, 128, torch.float16, cache, 16, 16, 16, True, 3)
        lens = torch.tensor([16, 16], dtype=torch.int32)
        w = wl.build_workload(cfg, "cpu", lengths=lens, shuffle_pages=True)
        k = x.view(2, 1, 16, 128).contiguous()
        wd = wl.to_device(w, "cuda:0")
        wd.pool.zero_()
        scale = torch.tensor([0.1], dtype=torch.float32, device="cuda:0")
        plugin = wl.make_plugin(cfg, 0)
        try:
            plugin.append_context(k.cuda(), k.cuda(), lens.cuda(), wd.kv_cache_block_pointers, scale)
            torch.cuda.synchronize()
        finally:
            plugin.close()
        pool = wd.pool.cpu()
        got = []
        for b in range(2):
            off = int(w.offset_table[b, 0, 0])
            got.append(pool[off: off + 16 * 128])
        got = torch.cat(got)
        want_chain = oracle.quantize_kv(x, 0.1, CACHE_MODE[cache])
        assert torch.equal(got, want_chain)
        kat = torch.from_numpy(qg[key]).view(torch.uint8)
        # the KAT multiplies in fp32 from the fp16-rounded input; fp16 inputs differ from its fp32 ones
        # only by the input rounding, so compare on the inputs the fp16 rounding left unchanged enough
        agree = (got == kat).float().mean().item()
        assert agree > (0.995 if cache == "int8" else 0.98), (cache, agree)


def test_prompt_then_decode_round_trip(pkg):
    """Fill the cache with the product writer from un-quantised K/V, then run a decode step and compare
    with attention computed directly from the prompt tensors (dequantised through the oracle's quantiser)."""
    wl = workloads
    cfg = wl.DecodeConfig("rt", 3, 16, 2, 128, torch.bfloat16, "fp8", 64, 90, 400, True, 23)
    lens = wl.draw_lengths(cfg)
    w, k, v, L = _setup(pkg, cfg, lens, seed=5)
    # scale from the prompt itself
    amax = max(float(k.abs().max()), float(v.abs().max()))
    s_qo = amax / 448.0
    s_oq = 1.0 / s_qo
    wd = wl.to_device(w, "cuda:0")
    sq = torch.tensor([s_oq], dtype=torch.float32, device="cuda:0")
    sd = torch.tensor([s_qo], dtype=torch.float32, device="cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        plugin.append_context(k.cuda(), v.cuda(), lens.cuda(), wd.kv_cache_block_pointers, sq)
        out = plugin.enqueue_generation(wd.qkv, wd.sequence_length, lens, wd.kv_cache_block_pointers, sq, sd)
        torch.cuda.synchronize()
    finally:
        plugin.close()
    # oracle: same two steps on the CPU copy
    pool_ref = w.pool.clone()
    oracle.append_context_reference(k, v, lens, pool_ref, w.offset_table, tokens_per_block=64,
                                    cache_mode=oracle.CACHE_FP8, kv_scale_orig_quant=s_oq)
    ref = oracle.decode_attention_reference(
        w.qkv, w.sequence_length, pool_ref, w.offset_table, num_heads=16, num_kv_heads=2, head_size=128,
        tokens_per_block=64, cache_mode=oracle.CACHE_FP8, kv_scale_orig_quant=s_oq, kv_scale_quant_orig=s_qo)
    assert torch.equal(wd.pool.cpu(), pool_ref)
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL
    # and against attention over the un-quantised prompt: only quantisation noise apart
    H, Hkv, Dh, G = 16, 2, 128, 8
    for b in range(cfg.batch):
        n = int(lens[b])
        q = w.qkv[b, : H * Dh].view(Hkv, G, Dh).float()
        kn = w.qkv[b, H * Dh:(H + Hkv) * Dh].view(Hkv, 1, Dh).float()
        vn = w.qkv[b, (H + Hkv) * Dh:].view(Hkv, 1, Dh).float()
        K = torch.cat([k[b, :, :n].float(), kn], 1)
        V = torch.cat([v[b, :, :n].float(), vn], 1)
        p = torch.softmax(q @ K.transpose(1, 2) / Dh ** 0.5, -1)
        o = (p @ V).reshape(-1)
        assert (out[b].float().cpu() - o).abs().max().item() < 0.1


def test_report_append_bandwidth(pkg):
    """Times the writer on a c4-shaped prompt batch (32 sequences x 4096 tokens, 8 kv heads, FP8) and records
    bytes moved per second in append_context.jsonl of the report directory; asserts only that it ran."""
    import json
    import os
    wl = workloads
    cfg = wl.DecodeConfig("ctxbw", 32, 64, 8, 128, torch.bfloat16, "fp8", 64, 4095, 4095, True, 9)
    lens = torch.full((32,), 4095, dtype=torch.int32)
    w = wl.build_workload(cfg, "cuda:0", lengths=lens)
    k = torch.randn(32, 8, 4096, 128, device="cuda:0", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    n = torch.full((32,), 4096, dtype=torch.int32, device="cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        for _ in range(3):
            plugin.append_context(k, v, n, w.kv_cache_block_pointers, w.kv_orig_quant_scale)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            plugin.append_context(k, v, n, w.kv_cache_block_pointers, w.kv_orig_quant_scale)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / 20 * 1e3
    finally:
        plugin.close()
    moved = 2 * k.numel() * (2 + 1)  # read 2 B, write 1 B per element, K and V
    rec = {"kernel": "kv_append_context_kernel", "us": us, "bytes": moved, "GBps": moved / us / 1e3}
    os.makedirs(REPORT_DIR, exist_ok=True)
    with open(os.path.join(REPORT_DIR, "append_context.jsonl"), "a") as f:
        f.write(json.dumps(rec) + "\n")
    print(rec)
    assert us > 0
