"""In-step QKV bias and rotary position embedding (GPT-J and GPT-NeoX style, with linear / dynamic scaling):
CUDA path through the C ABI against the CPU oracle and against the reference's own MMHA kernel recompiled
for sm_100a.  The rotation is fp32 arithmetic with cos / sin / pow, so the quantised K bytes are compared with
a stated allowance for one-ulp differences between math libraries; everything else stays bit-exact."""
import dataclasses
from pathlib import Path

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu
LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_mmha.so"

ROPES = {
    "gptj": dict(position_embedding_type=1, rotary_embedding_dim=64, rotary_embedding_base=10000.0),
    "neox": dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0),
    "neox_partial": dict(position_embedding_type=2, rotary_embedding_dim=32, rotary_embedding_base=500.0),
    "neox_linear": dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0,
                        rotary_embedding_scale_type=1, rotary_embedding_scale=4.0),
    "neox_dynamic": dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0,
                         rotary_embedding_scale_type=2, rotary_embedding_scale=2.0,
                         rotary_embedding_max_positions=256),
}


def _plugin(pkg, cfg, rope, bias):
    return pkg.GPTAttentionPlugin(num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size,
                                  multi_block_mode=cfg.multi_block_mode, kv_cache_quant_mode=cfg.quant_mode,
                                  tokens_per_block=cfg.tokens_per_block, type_id=cfg.dtype, device=0,
                                  qkv_bias=bias, **rope)


def _oracle(w_cpu, rope, bias):
    cfg = w_cpu.cfg
    qkv = oracle.apply_bias_rope(w_cpu.qkv, w_cpu.sequence_length, num_heads=cfg.num_heads,
                                 num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, qkv_bias=bias, **rope)
    pool = w_cpu.pool.clone()
    out = oracle.decode_attention_reference(
        qkv, w_cpu.sequence_length, pool, w_cpu.offset_table, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
        head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block, cache_mode=CACHE_MODE[cfg.cache],
        kv_scale_orig_quant=w_cpu.scale_orig_quant, kv_scale_quant_orig=w_cpu.scale_quant_orig)
    return out, pool


def _byte_agreement(a, b, changed_mask):
    return (a[changed_mask] == b[changed_mask]).double().mean().item()


@pytest.mark.parametrize("rope_name", list(ROPES))
@pytest.mark.parametrize("dtype,cache,heads,with_bias", [
    (torch.bfloat16, "fp8", (8, 1), False),
    (torch.bfloat16, "int8", (4, 4), True),
    (torch.float16, "none", (4, 2), True),
    (torch.float16, "fp8", (32, 2), False),
])
def test_rope_bias_against_oracle(pkg, rope_name, dtype, cache, heads, with_bias):
    wl = workloads
    rope = ROPES[rope_name]
    dh = 128
    if rope["rotary_embedding_dim"] > dh:
        pytest.skip("rotary dim larger than head size")
    cfg = wl.DecodeConfig("rope", 4, heads[0], heads[1], dh, dtype, cache, 64, 30, 700, True, 77)
    w_cpu = wl.build_workload(cfg, "cpu")
    g = torch.Generator().manual_seed(3)
    bias = (torch.randn((heads[0] + 2 * heads[1]) * dh, generator=g) * 0.5).to(dtype) if with_bias else None
    ref, pool_ref = _oracle(w_cpu, rope, bias)
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = _plugin(pkg, cfg, rope, with_bias)
    try:
        out = plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                        w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                        qkv_bias=None if bias is None else bias.cuda())
        torch.cuda.synchronize()
    finally:
        plugin.close()
    pool = w.pool.cpu()
    changed = pool_ref != w_cpu.pool
    # V bytes and everything not rotated: exact.  Rotated K bytes: cos/sin/pow may differ in the last bit
    # between the CUDA math library and the CPU, which after rounding to T and quantising flips a few bytes.
    assert not bool(((pool != w_cpu.pool) & ~((pool_ref != w_cpu.pool) | (pool != pool_ref))).any())
    agree = _byte_agreement(pool, pool_ref, changed | (pool != w_cpu.pool))
    assert agree > 0.99, agree
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


@pytest.mark.skipif(not LIB.exists(), reason="oracle/_ref/libref_mmha.so not built (needs the reference tree)")
@pytest.mark.parametrize("rope_name", list(ROPES))
@pytest.mark.parametrize("cache", ["int8", "none"])
def test_rope_bias_against_reference_kernel(pkg, rope_name, cache):
    """Same device math library on both sides: the K/V bytes the reference kernel appends after bias + RoPE
    must equal ours exactly."""
    from test_reference_kernel_gpu import _run_reference
    wl = workloads
    rope = ROPES[rope_name]
    cfg = wl.DecodeConfig("roperef", 4, 8, 2, 128, torch.bfloat16, cache, 64, 30, 700, False, 78)
    w_cpu = wl.build_workload(cfg, "cpu")
    g = torch.Generator().manual_seed(4)
    bias = (torch.randn((8 + 4) * 128, generator=g) * 0.5).to(torch.bfloat16).cuda()
    w_ours = wl.to_device(w_cpu, "cuda:0")
    w_ref = wl.to_device(w_cpu, "cuda:0")
    plugin = _plugin(pkg, cfg, rope, True)
    try:
        out = plugin.enqueue_generation(w_ours.qkv, w_ours.sequence_length, w_ours.host_past_key_value_lengths,
                                        w_ours.kv_cache_block_pointers, w_ours.kv_orig_quant_scale,
                                        w_ours.kv_quant_orig_scale, qkv_bias=bias)
        torch.cuda.synchronize()
    finally:
        plugin.close()
    out_ref = _run_reference(w_ref, qkv_bias=bias, rope=rope)
    same = (w_ours.pool == w_ref.pool)
    touched = (w_ours.pool != w_cpu.pool.cuda()) | (w_ref.pool != w_cpu.pool.cuda())
    n_diff = int((~same[touched]).sum())
    print(rope_name, cache, "bytes touched:", int(touched.sum()), "different from the reference kernel's:", n_diff)
    assert n_diff == 0
    d = (out.float() - out_ref.float()).abs()
    assert d.max().item() < 0.5 and d.mean().item() < 0.05
