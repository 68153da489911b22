"""Relative attention bias of the generation step (T5-style; the reference's relative_attention_bias input with the
relative position embedding type): explicit table [H, S, S] and the implicit bucket table [H, buckets], through the
C ABI against the CPU oracle, and the oracle against the reference's own MMHA kernel recompiled for sm_100a."""
import ctypes
from pathlib import Path

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu
LIB = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_mmha.so"


def _bias(cfg, stride, implicit, seed):
    g = torch.Generator().manual_seed(seed)
    shape = (cfg.num_heads, stride) if implicit else (cfg.num_heads, stride, stride)
    return torch.randn(*shape, generator=g).to(cfg.dtype)


def _oracle(w, bias, max_distance):
    cfg = w.cfg
    pool = w.pool.clone()
    out = oracle.attention_general_ref.decode_attention_general_reference(
        w.qkv, w.sequence_length, pool, w.offset_table, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
        head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block, cache_mode=CACHE_MODE[cfg.cache],
        kv_scale_orig_quant=w.scale_orig_quant, kv_scale_quant_orig=w.scale_quant_orig,
        relative_attention_bias=bias, max_distance=max_distance)
    return out, pool


def _product(pkg, w_cpu, bias, max_distance, position_embedding_type=5):
    cfg = w_cpu.cfg
    w = workloads.to_device(w_cpu, "cuda:0")
    plugin = pkg.GPTAttentionPlugin(num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size,
                                    multi_block_mode=True, kv_cache_quant_mode=cfg.quant_mode,
                                    tokens_per_block=cfg.tokens_per_block, type_id=cfg.dtype, device=0,
                                    position_embedding_type=position_embedding_type)
    try:
        out = plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                        w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                        relative_attention_bias=bias.cuda(), max_distance=max_distance)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
    finally:
        plugin.close()
    return out.float().cpu(), w.pool.cpu()


SHAPES = [
    ((8, 8), 64, torch.float16, "none", 64),
    ((8, 2), 128, torch.bfloat16, "fp8", 64),
    ((4, 4), 128, torch.bfloat16, "int8", 32),
    ((12, 1), 64, torch.float16, "fp8", 128),
]


@pytest.mark.parametrize("implicit,max_distance", [(False, 0), (True, 100), (True, 50)])
@pytest.mark.parametrize("heads,dh,dtype,cache,tpb", SHAPES)
def test_relative_bias_against_oracle(pkg, heads, dh, dtype, cache, tpb, implicit, max_distance):
    cfg = workloads.DecodeConfig("rel", 4, heads[0], heads[1], dh, dtype, cache, tpb, 0, 300, True, 41)
    w = workloads.build_workload(cfg, "cpu")
    stride = 32 if implicit else int(w.host_past_key_value_lengths.max()) + 3
    bias = _bias(cfg, stride, implicit, 7)
    ref, pool_ref = _oracle(w, bias, max_distance)
    out, pool = _product(pkg, w, bias, max_distance)
    assert torch.equal(pool, pool_ref)
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())
    # the bias matters: without it the result is a different one
    plain, _ = _oracle(w, None, 0)
    assert (plain - ref).abs().max().item() > 10 * MAX_ABS_TOL


def _reference_kernel(w, bias, max_distance):
    cfg = w.cfg
    lib = ctypes.CDLL(str(LIB))
    fn = lib.ref_mmha_relbias_bf16_128 if (cfg.dtype == torch.bfloat16 and cfg.head_size == 128) else lib.ref_mmha_relbias_fp16_64
    fn.restype = ctypes.c_int
    out = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device=w.qkv.device)
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    P = ctypes.c_void_p
    b = bias.to(w.qkv.device)
    st = fn(P(w.qkv.data_ptr()), P(out.data_ptr()), P(w.sequence_length.data_ptr()),
            P(w.kv_cache_block_pointers.data_ptr()), cfg.batch, cfg.num_heads, cfg.num_kv_heads,
            w.max_blocks_per_seq, cfg.tokens_per_block, w.max_blocks_per_seq * cfg.tokens_per_block,
            int(w.host_past_key_value_lengths.max()), ctypes.c_float(1.0),
            P(w.kv_orig_quant_scale.data_ptr() if w.kv_orig_quant_scale is not None else 0),
            P(w.kv_quant_orig_scale.data_ptr() if w.kv_quant_orig_scale is not None else 0),
            int(cfg.cache == "int8"), int(cfg.cache == "fp8"), sm, P(torch.cuda.current_stream().cuda_stream),
            P(b.data_ptr()), int(bias.shape[1]), max_distance)
    assert st == 0, f"reference launcher returned {st}"
    torch.cuda.synchronize()
    return out.float().cpu()


@pytest.mark.skipif(not LIB.exists(), reason="oracle/_ref/libref_mmha.so not built (needs the reference tree)")
@pytest.mark.parametrize("implicit,max_distance", [(False, 0), (True, 100), (True, 128)])
@pytest.mark.parametrize("heads,dh,dtype", [((4, 4), 128, torch.bfloat16), ((8, 8), 64, torch.float16)])
def test_oracle_and_product_match_the_reference_kernel(pkg, heads, dh, dtype, implicit, max_distance):
    """INT8 cache and one kv head per q head: the reference kernel then accumulates q.k in fp32 and no other CTA
    reads the slot it writes.  With max_distance 128 some positions sit exactly on a bucket boundary of the
    float formula; the product evaluates the same expression on the same GPU, so product and reference kernel
    must still agree there (the CPU oracle is compared where no boundary is hit)."""
    lib = ctypes.CDLL(str(LIB))
    if not hasattr(lib, "ref_mmha_relbias_bf16_128"):
        pytest.skip("oracle/_ref/libref_mmha.so predates the relative-bias entry point")
    cfg = workloads.DecodeConfig("relref", 3, heads[0], heads[1], dh, dtype, "int8", 64, 10, 300, False, 42)
    w_cpu = workloads.build_workload(cfg, "cpu")
    stride = 32 if implicit else int(w_cpu.host_past_key_value_lengths.max()) + 1
    bias = _bias(cfg, stride, implicit, 8)
    w = workloads.to_device(w_cpu, "cuda:0")
    ref_kernel = _reference_kernel(w, bias, max_distance)
    out, pool = _product(pkg, w_cpu, bias, max_distance)
    assert torch.equal(w.pool.cpu(), pool)  # the same bytes stored at the same place
    d = (out - ref_kernel).abs()
    print("product vs reference kernel: max", d.max().item(), "mean", d.mean().item())
    assert d.max().item() < 3e-2 and d.mean().item() < 3e-3
    if max_distance != 128:
        ref, _ = _oracle(w_cpu, bias, max_distance)
        e = (ref_kernel - ref).abs()
        print("reference kernel vs oracle: max", e.max().item(), "mean", e.mean().item())
        assert e.max().item() < 3e-2 and e.mean().item() < 3e-3


def test_argument_errors(pkg):
    P = pkg.plugin
    cfg = workloads.DecodeConfig("relerr", 2, 4, 4, 64, torch.float16, "none", 64, 50, 90, True, 43)
    w = workloads.build_workload(cfg, "cpu")
    bias = _bias(cfg, 128, False, 1)
    with pytest.raises(P.DecodeAttnError) as e:  # a table needs the relative position embedding type
        _product(pkg, w, bias, 0, position_embedding_type=0)
    assert e.value.status == P.DX_ERR_BAD_ARG
    with pytest.raises(P.DecodeAttnError) as e:  # explicit table shorter than the sequences
        _product(pkg, w, _bias(cfg, 40, False, 1), 0)
    assert e.value.status == P.DX_ERR_BAD_ARG
    with pytest.raises(P.DecodeAttnError) as e:  # implicit form: max_distance must exceed a quarter of the buckets
        _product(pkg, w, _bias(cfg, 32, True, 1), 8)
    assert e.value.status == P.DX_ERR_BAD_ARG
