"""Remaining enqueueGeneration features on the GPU: beam search through the cache indirection table, cyclic
(sliding-window) cache with sink tokens, ALiBi.  Product (C ABI) against the CPU oracle - pool bytes bit-exact,
outputs within the fp32-oracle tolerance - and the oracle against the reference's own MMHA kernel
(oracle/_ref/libref_mmha.so, when the reference tree was present at build time)."""
import ctypes
import dataclasses
from pathlib import Path

import pytest
import torch

import workloads

import oracle
from oracle.attention_general_ref import decode_attention_general_reference
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL, REPORT_DIR

pytestmark = pytest.mark.gpu
LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_mmha.so"


@dataclasses.dataclass
class Case:
    heads: tuple
    dh: int
    dtype: torch.dtype
    cache: str
    tpb: int
    requests: int
    beam: int = 1
    window: int = 0          # 0: no sliding window
    sink: int = 0
    alibi: bool = False
    past_lo: int = 40
    past_hi: int = 300
    seed: int = 1


def _build(pkg, c: Case):
    """Workload with every cache slot filled; returns (cpu workload, extras dict)."""
    wl = workloads
    g = torch.Generator().manual_seed(c.seed)
    nseq = c.requests * c.beam
    past_req = torch.randint(c.past_lo, c.past_hi + 1, (c.requests,), generator=g, dtype=torch.int32)
    past = past_req.repeat_interleave(c.beam)  # beams of a request have the same length
    # slots the table must hold: the whole history, or the window when the cache is cyclic
    held = past.clone() if c.window == 0 else torch.clamp(past, max=c.window - 1)
    cfg = wl.DecodeConfig("feat", nseq, c.heads[0], c.heads[1], c.dh, c.dtype, c.cache, c.tpb, c.past_lo, c.past_hi,
                          False, 5000 + c.seed)
    w = wl.build_workload(cfg, "cpu", lengths=held)
    w = dataclasses.replace(w, sequence_length=(past + 1).to(torch.int32), host_past_key_value_lengths=past.clone())
    M = w.max_blocks_per_seq
    maw = M * c.tpb
    ex = {"beam_width": c.beam, "max_attention_window": maw,
          "cyclic_attention_window_size": c.window if c.window else maw, "sink_token_length": c.sink}
    if c.beam > 1:
        ex["cache_indirection"] = torch.randint(0, c.beam, (nseq, maw), generator=g, dtype=torch.int32)
        ctx = torch.stack([torch.randint(1, int(p) + 1, (1,), generator=g, dtype=torch.int32)[0] for p in past_req])
        ex["context_lengths"] = ctx.repeat_interleave(c.beam).to(torch.int32)
    if c.alibi:
        H = c.heads[0]
        ex["alibi_slopes"] = (2.0 ** (-8.0 * torch.arange(1, H + 1, dtype=torch.float32) / H)).to(c.dtype)
    return w, ex


def _oracle(w, ex, pool=None):
    cfg = w.cfg
    pool = w.pool.clone() if pool is None else pool
    out = decode_attention_general_reference(
        w.qkv, w.sequence_length, pool, w.offset_table, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
        head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block, cache_mode=CACHE_MODE[cfg.cache],
        kv_scale_orig_quant=w.scale_orig_quant, kv_scale_quant_orig=w.scale_quant_orig,
        beam_width=ex["beam_width"], cache_indirection=ex.get("cache_indirection"),
        context_lengths=ex.get("context_lengths"), max_attention_window=ex["max_attention_window"],
        cyclic_attention_window_size=ex["cyclic_attention_window_size"], sink_token_length=ex["sink_token_length"],
        alibi_slopes=ex.get("alibi_slopes"))
    return out, pool


def _plugin(pkg, c: Case):
    P = pkg.plugin
    return P.GPTAttentionPlugin(
        num_heads=c.heads[0], num_kv_heads=c.heads[1], head_size=c.dh, kv_cache_quant_mode=workloads.DecodeConfig(
            "q", 1, 1, 1, c.dh, c.dtype, c.cache, c.tpb, 1, 1, False, 0).quant_mode,
        tokens_per_block=c.tpb, multi_block_mode=True, type_id=c.dtype,
        position_embedding_type=P.PositionEmbeddingType.alibi if c.alibi else P.PositionEmbeddingType.learned_absolute)


def _run_product(pkg, c, w_cpu, ex):
    wl = workloads
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = _plugin(pkg, c)
    dev = lambda t: None if t is None else t.to("cuda:0")
    try:
        out = plugin.enqueue_generation(
            w.qkv, w.sequence_length, w.host_past_key_value_lengths, w.kv_cache_block_pointers,
            w.kv_orig_quant_scale, w.kv_quant_orig_scale, max_attention_window=ex["max_attention_window"],
            cache_indirection=dev(ex.get("cache_indirection")), beam_width=ex["beam_width"],
            sink_token_length=ex["sink_token_length"],
            cyclic_attention_window_size=ex["cyclic_attention_window_size"],
            context_lengths=dev(ex.get("context_lengths")), alibi_slopes=dev(ex.get("alibi_slopes")))
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
        return out.float().cpu(), w.pool.cpu()
    finally:
        plugin.close()


CASES = {
    "beam4_mha_fp16": Case((4, 4), 64, torch.float16, "none", 64, 3, beam=4),
    "beam2_gqa_int8": Case((8, 2), 128, torch.bfloat16, "int8", 64, 3, beam=2),
    "beam3_mqa_fp8": Case((8, 1), 128, torch.bfloat16, "fp8", 32, 2, beam=3),
    "window_wrapped_int8": Case((8, 2), 128, torch.bfloat16, "int8", 64, 4, window=256, past_lo=200, past_hi=900),
    "window_wrapped_fp16": Case((4, 4), 64, torch.float16, "none", 64, 4, window=192, past_lo=150, past_hi=700),
    "window_sink_fp8": Case((8, 1), 64, torch.float16, "fp8", 64, 4, window=256, sink=64, past_lo=100, past_hi=900),
    "window_exact_fill": Case((4, 2), 128, torch.bfloat16, "int8", 64, 3, window=128, past_lo=128, past_hi=128),
    "alibi_mha_bf16": Case((8, 8), 128, torch.bfloat16, "none", 64, 3, alibi=True),
    "alibi_gqa_int8": Case((8, 2), 64, torch.float16, "int8", 128, 3, alibi=True),
    "beam2_alibi_fp8": Case((4, 2), 128, torch.bfloat16, "fp8", 64, 2, beam=2, alibi=True),
    "beam2_window_wrapped": Case((4, 2), 64, torch.float16, "int8", 64, 2, beam=2, window=128, past_lo=100, past_hi=400),
    # grouped heads over an 8-bit cache without a wrapped window: the feature form of the tensor-core kernel
    "beam4_gqa_fp8_split": Case((16, 2), 128, torch.bfloat16, "fp8", 64, 2, beam=4, past_lo=3000, past_hi=5000, seed=7),
    "beam2_group16_int8": Case((32, 2), 128, torch.bfloat16, "int8", 64, 2, beam=2, past_lo=200, past_hi=900, seed=8),
    "alibi_group71_fp8": Case((71, 1), 64, torch.float16, "fp8", 64, 2, alibi=True, past_lo=100, past_hi=700, seed=9),
    "beam3_alibi_group12_int8": Case((24, 2), 64, torch.float16, "int8", 32, 2, beam=3, alibi=True, past_lo=1, past_hi=300, seed=10),
    "alibi_gqa_fp8_split": Case((8, 1), 128, torch.bfloat16, "fp8", 128, 2, alibi=True, past_lo=4000, past_hi=6000, seed=11),
    "window_wrapped_fp8_split": Case((16, 2), 128, torch.bfloat16, "fp8", 64, 2, window=4096, past_lo=3000, past_hi=9000, seed=12),
    "window_sink_alibi_int8": Case((8, 2), 64, torch.float16, "int8", 32, 3, window=256, sink=32, alibi=True, past_lo=100, past_hi=800, seed=13),
    "beam2_window_sink_fp8": Case((8, 2), 128, torch.bfloat16, "fp8", 64, 2, beam=2, window=256, sink=64, past_lo=100, past_hi=700, seed=14),
    # ... and over a 16-bit cache: the feature form of the 16-bit grouped-head kernel
    "beam2_gqa_bf16": Case((8, 2), 128, torch.bfloat16, "none", 64, 2, beam=2, seed=15),
    "alibi_gqa_fp16_split": Case((8, 2), 64, torch.float16, "none", 32, 2, alibi=True, past_lo=3000, past_hi=5000, seed=16),
    "window_wrapped_gqa_bf16": Case((16, 4), 128, torch.bfloat16, "none", 64, 3, window=256, past_lo=200, past_hi=900, seed=17),
    "beam3_window_sink_alibi_fp16": Case((12, 3), 64, torch.float16, "none", 16, 2, beam=3, window=128, sink=32, alibi=True, past_lo=50, past_hi=400, seed=18),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_features_against_oracle(pkg, name):
    c = CASES[name]
    w_cpu, ex = _build(pkg, c)
    ref, pool_ref = _oracle(w_cpu, ex)
    out, pool_gpu = _run_product(pkg, c, w_cpu, ex)
    diff = pool_gpu != pool_ref
    assert not bool(diff.any()), f"{int(diff.sum())} pool bytes differ from the oracle"
    err = (out - ref).abs()
    assert torch.isfinite(out).all()
    print(name, "max", err.max().item(), "mean", err.mean().item())
    assert err.max().item() < MAX_ABS_TOL, f"max-abs {err.max().item():.3e}"
    assert err.mean().item() < MEAN_ABS_TOL, f"mean-abs {err.mean().item():.3e}"


@pytest.mark.parametrize("name", ["beam4_gqa_fp8_split", "beam2_group16_int8", "beam2_alibi_fp8", "window_wrapped_int8",
                                  "window_sink_fp8", "beam2_window_wrapped", "window_wrapped_fp8_split", "beam2_gqa_bf16",
                                  "window_wrapped_gqa_bf16"])
def test_grouped_feature_kernel_agrees_with_the_per_head_kernel(pkg, name, monkeypatch):
    """The same call on the feature form of the grouped-head kernel (default) and, with DX_ATTN_FEATURE_GQA=0, on
    the per-head feature kernel: identical pool bytes, outputs within the output tolerance of each other."""
    c = CASES[name]
    w_cpu, ex = _build(pkg, c)
    out_a, pool_a = _run_product(pkg, c, w_cpu, ex)
    monkeypatch.setenv("DX_ATTN_FEATURE_GQA", "0")
    out_b, pool_b = _run_product(pkg, c, w_cpu, ex)
    assert torch.equal(pool_a, pool_b)
    err = (out_a - out_b).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


def test_features_off_equals_plain_oracle(pkg):
    """With every feature off the general oracle is the plain one (same outputs, same pool)."""
    c = Case((8, 2), 128, torch.bfloat16, "fp8", 64, 4)
    w_cpu, ex = _build(pkg, c)
    a, pa = _oracle(w_cpu, ex)
    pb = w_cpu.pool.clone()
    cfg = w_cpu.cfg
    b = oracle.decode_attention_reference(
        w_cpu.qkv, w_cpu.sequence_length, pb, w_cpu.offset_table, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block,
        cache_mode=CACHE_MODE[cfg.cache], kv_scale_orig_quant=w_cpu.scale_orig_quant,
        kv_scale_quant_orig=w_cpu.scale_quant_orig)
    assert torch.equal(pa, pb)
    assert (a - b).abs().max().item() < 1e-5


def test_unsupported_geometries_are_refused(pkg):
    """A sink that ends inside a block, and a wrapped window over a table with the spare block, need the
    reference's position shift: refused before anything is launched."""
    P = pkg.plugin
    c = Case((4, 4), 64, torch.float16, "none", 64, 2, window=128, sink=16, past_lo=100, past_hi=120)
    w_cpu, ex = _build(pkg, c)
    with pytest.raises(P.DecodeAttnError) as e:
        _run_product(pkg, c, w_cpu, ex)
    assert e.value.status == P.DX_ERR_UNSUPPORTED
    c = Case((4, 4), 64, torch.float16, "none", 64, 2, window=100, past_lo=300, past_hi=300)
    w_cpu, ex = _build(pkg, c)  # 100-token window in 2 blocks: (M-1)*64 = 64 < 100, fine ...
    ex["cyclic_attention_window_size"] = 64  # ... but a 64-token window leaves a spare block
    with pytest.raises(P.DecodeAttnError) as e:
        _run_product(pkg, c, w_cpu, ex)
    assert e.value.status == P.DX_ERR_UNSUPPORTED


# ----------------------------------------------------------------------------------------------------------
# the oracle against the reference kernel
# ----------------------------------------------------------------------------------------------------------
def _run_reference_ext(w, ex):
    cfg = w.cfg
    lib = ctypes.CDLL(str(LIB))
    fn = lib.ref_mmha_ext_bf16_128 if (cfg.dtype == torch.bfloat16 and cfg.head_size == 128) else lib.ref_mmha_ext_fp16_64
    fn.restype = ctypes.c_int
    out = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device=w.qkv.device)
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    P = ctypes.c_void_p
    keep = {k: v.to(w.qkv.device) for k, v in ex.items() if isinstance(v, torch.Tensor)}
    ptr = lambda k: P(keep[k].data_ptr() if k in keep else 0)
    st = fn(P(w.qkv.data_ptr()), P(out.data_ptr()), P(w.sequence_length.data_ptr()),
            P(w.kv_cache_block_pointers.data_ptr()), cfg.batch, cfg.num_heads, cfg.num_kv_heads,
            w.max_blocks_per_seq, cfg.tokens_per_block, ex["max_attention_window"],
            int(w.host_past_key_value_lengths.max()), ctypes.c_float(1.0),
            P(w.kv_orig_quant_scale.data_ptr() if w.kv_orig_quant_scale is not None else 0),
            P(w.kv_quant_orig_scale.data_ptr() if w.kv_quant_orig_scale is not None else 0),
            int(cfg.cache == "int8"), int(cfg.cache == "fp8"), sm, P(torch.cuda.current_stream().cuda_stream),
            ex["beam_width"], ptr("cache_indirection"), ptr("context_lengths"), ex["cyclic_attention_window_size"],
            ex["sink_token_length"], ptr("alibi_slopes"))
    assert st == 0, f"reference launcher returned {st}"
    torch.cuda.synchronize()
    return out.float().cpu()


# One kv head per q head, so that no other CTA of the reference reads a slot while it is being overwritten,
# and an INT8 or 16-bit... the reference accumulates q.k in fp32 only for the INT8 cache: tight tolerance there.
REF_CASES = {
    "beam4_int8": (Case((4, 4), 128, torch.bfloat16, "int8", 64, 3, beam=4), 3e-2),
    "beam2_fp16": (Case((4, 4), 64, torch.float16, "none", 64, 3, beam=2), 0.5),
    "window_wrapped_int8": (Case((4, 4), 128, torch.bfloat16, "int8", 64, 4, window=256, past_lo=200, past_hi=900), 3e-2),
    "window_sink_int8": (Case((4, 4), 64, torch.float16, "int8", 64, 4, window=256, sink=64, past_lo=100, past_hi=900), 3e-2),
    "alibi_int8": (Case((8, 8), 128, torch.bfloat16, "int8", 64, 3, alibi=True), 3e-2),
}


@pytest.mark.skipif(not LIB.exists(), reason="oracle/_ref/libref_mmha.so not built (needs the reference tree)")
@pytest.mark.parametrize("name", sorted(REF_CASES))
def test_oracle_matches_reference_kernel_features(pkg, name):
    c, tol = REF_CASES[name]
    w_cpu, ex = _build(pkg, c)
    ref, pool_ref = _oracle(w_cpu, ex)
    w = workloads.to_device(w_cpu, "cuda:0")
    out = _run_reference_ext(w, ex)
    # bit-exact: the bytes the reference kernel stored, and the (cyclic) slots it stored them in
    assert torch.equal(w.pool.cpu(), pool_ref)
    err = (out - ref).abs()
    print(name, "reference-kernel deviation from the oracle: max", err.max().item(), "mean", err.mean().item())
    assert err.max().item() < tol and err.mean().item() < tol / 10


def test_beams_with_bias_and_rotary_embedding(pkg):
    """The in-step pre-processing (bias add, GPT-NeoX rotary embedding) in front of the feature path:
    the rotated k of every beam is what gets stored, and the indirection table still picks the beams."""
    P = pkg.plugin
    c = Case((8, 2), 128, torch.bfloat16, "int8", 64, 2, beam=2, seed=11)
    w_cpu, ex = _build(pkg, c)
    cfg = w_cpu.cfg
    rope = dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0)
    g = torch.Generator().manual_seed(5)
    bias = (0.1 * torch.randn((cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size, generator=g)).to(cfg.dtype)
    qkv_pre = oracle.apply_bias_rope(w_cpu.qkv, w_cpu.sequence_length, num_heads=cfg.num_heads,
                                     num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, qkv_bias=bias, **rope)
    ref, pool_ref = _oracle(dataclasses.replace(w_cpu, qkv=qkv_pre), ex)
    w = workloads.to_device(w_cpu, "cuda:0")
    plugin = P.GPTAttentionPlugin(num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size,
                                  kv_cache_quant_mode=cfg.quant_mode, tokens_per_block=cfg.tokens_per_block,
                                  multi_block_mode=True, type_id=cfg.dtype, qkv_bias=True, **rope)
    try:
        out = plugin.enqueue_generation(
            w.qkv, w.sequence_length, w.host_past_key_value_lengths, w.kv_cache_block_pointers,
            w.kv_orig_quant_scale, w.kv_quant_orig_scale, max_attention_window=ex["max_attention_window"],
            cache_indirection=ex["cache_indirection"].cuda(), beam_width=2,
            context_lengths=ex["context_lengths"].cuda(), qkv_bias=bias.cuda())
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
        # the rotation is fp32 cos / sin / pow: allow the odd one-ulp difference in the stored bytes
        same = (w.pool.cpu() == pool_ref).double().mean().item()
        assert same > 0.9999, same
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL
    finally:
        plugin.close()


FEATURE_TIMING = {
    "beam 4 x 16 requests, 64 q / 8 kv heads, Dh 128, FP8, past 2048-4096":
        Case((64, 8), 128, torch.bfloat16, "fp8", 64, 16, beam=4, past_lo=2048, past_hi=4096, seed=3),
    "sliding window 4096 wrapped, 64 sequences, 32 q / 8 kv heads, Dh 128, FP8, past 5000-12000":
        Case((32, 8), 128, torch.bfloat16, "fp8", 64, 64, window=4096, past_lo=5000, past_hi=12000, seed=4),
}


@pytest.mark.parametrize("label", sorted(FEATURE_TIMING))
def test_report_feature_path_time(pkg, label):
    """Times the feature path on a beam-search batch of c4's shape and on a wrapped sliding window (recorded in
    feature_path.jsonl of the report directory)."""
    import json
    import os
    c = FEATURE_TIMING[label]
    w_cpu, ex = _build(pkg, c)
    w = workloads.to_device(w_cpu, "cuda:0")
    plugin = _plugin(pkg, c)
    try:
        dev = lambda t: None if t is None else t.cuda()
        ci, cl = dev(ex.get("cache_indirection")), dev(ex.get("context_lengths"))
        out = torch.empty(w.cfg.batch, c.heads[0] * c.dh, dtype=c.dtype, device="cuda:0")

        def step():
            plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                      w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale, out=out,
                                      max_attention_window=ex["max_attention_window"], cache_indirection=ci,
                                      beam_width=c.beam, context_lengths=cl,
                                      cyclic_attention_window_size=ex["cyclic_attention_window_size"])
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            step()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / 10 * 1e3
        walked = torch.clamp(w_cpu.host_past_key_value_lengths, max=c.window) if c.window else w_cpu.host_past_key_value_lengths
        kv = float(walked.double().sum() * c.heads[1] * c.dh * 2)
        rec = {"case": label, "us": us, "unique_kv_GBps": kv / us / 1e3}
        os.makedirs(REPORT_DIR, exist_ok=True)
        with open(os.path.join(REPORT_DIR, "feature_path.jsonl"), "a") as f:
            f.write(json.dumps(rec) + "\n")
        print(rec)
    finally:
        plugin.close()
