"""Head sizes of the reference's MMHA switch other than 64 and 128
(cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention.cu:68-85: 32, 48, 80, 96, 104, 112, 144, 160, 192, 224,
256) through the C ABI: decode step, beam search / ALiBi / wrapped window, several new tokens per step and the
context-phase writer, each against the CPU oracle - pool bytes bit-exact, outputs within the output tolerance."""
import dataclasses

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL, gpu_step_and_compare
from test_generation_features_gpu import Case, _build, _oracle, _run_product

pytestmark = pytest.mark.gpu

OTHER_SIZES = [32, 48, 80, 96, 112, 144, 160, 192, 224, 256]


@pytest.mark.parametrize("cache", ["none", "int8", "fp8"])
@pytest.mark.parametrize("dh", OTHER_SIZES + [104])
def test_decode_step_matches_oracle(pkg, dh, cache):
    if dh == 104 and cache != "none":
        pytest.skip("a 104-byte cache row is not a multiple of 16 bytes: refused at creation (tested below)")
    wl = workloads
    dtype = torch.bfloat16 if dh % 32 == 0 else torch.float16
    cfg = wl.DecodeConfig(f"dh{dh}", 5, 8, 2, dh, dtype, cache, 64, 1, 700, True, 3000 + dh)
    lens = torch.tensor([0, 1, 63, 64, 700], dtype=torch.int32)
    gpu_step_and_compare(pkg, cfg, lengths=lens)


def test_head_size_104_needs_a_16_bit_cache(pkg):
    P = pkg.plugin
    for mode in (P.QuantMode.INT8_KV_CACHE, P.QuantMode.FP8_KV_CACHE):
        with pytest.raises(P.DecodeAttnError) as e:
            P.GPTAttentionPlugin(num_heads=4, num_kv_heads=4, head_size=104, kv_cache_quant_mode=mode,
                                 tokens_per_block=64, multi_block_mode=True, type_id=torch.float16)
        assert e.value.status == P.DX_ERR_UNSUPPORTED
    with pytest.raises(P.DecodeAttnError) as e:  # not in the reference's switch either
        P.GPTAttentionPlugin(num_heads=4, num_kv_heads=4, head_size=72, kv_cache_quant_mode=P.QuantMode.NONE,
                             tokens_per_block=64, multi_block_mode=True, type_id=torch.float16)
    assert e.value.status == P.DX_ERR_UNSUPPORTED


def test_plan_reports_the_feature_complete_kernel(pkg):
    wl = workloads
    cfg = wl.DecodeConfig("dh96", 2, 8, 2, 96, torch.float16, "fp8", 64, 1, 100, True, 7)
    plugin = wl.make_plugin(cfg, 0)
    try:
        plan = plugin.plan(2, 500)
        assert plan["kernel"] == "general_cuda_core" and plan["num_partitions"] == 1
        assert plugin.get_workspace_size(2, 500) == 0
    finally:
        plugin.close()


FEATURE_CASES = {
    "beam3_dh96_fp8": Case((8, 2), 96, torch.float16, "fp8", 64, 2, beam=3),
    "beam2_dh256_bf16": Case((4, 2), 256, torch.bfloat16, "none", 32, 2, beam=2),
    "window_wrapped_dh80_int8": Case((4, 4), 80, torch.float16, "int8", 64, 3, window=192, past_lo=150, past_hi=600),
    "window_sink_dh160_fp8": Case((8, 1), 160, torch.bfloat16, "fp8", 64, 3, window=256, sink=64, past_lo=100, past_hi=700),
    "alibi_dh48_fp16": Case((6, 6), 48, torch.float16, "none", 64, 3, alibi=True),
    "alibi_dh224_int8": Case((4, 2), 224, torch.bfloat16, "int8", 64, 2, alibi=True),
}


@pytest.mark.parametrize("name", sorted(FEATURE_CASES))
def test_features_on_other_head_sizes(pkg, name):
    c = FEATURE_CASES[name]
    w_cpu, ex = _build(pkg, c)
    ref, pool_ref = _oracle(w_cpu, ex)
    out, pool_gpu = _run_product(pkg, c, w_cpu, ex)
    assert torch.equal(pool_gpu, pool_ref)
    err = (out - ref).abs()
    assert torch.isfinite(out).all()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("dh,cache,dtype", [(32, "int8", torch.float16), (80, "fp8", torch.float16),
                                            (104, "none", torch.float16), (192, "fp8", torch.bfloat16),
                                            (256, "int8", torch.bfloat16), (256, "none", torch.bfloat16)])
def test_context_append_on_other_head_sizes(pkg, dh, cache, dtype):
    wl = workloads
    tpb = 32
    cfg = wl.DecodeConfig("ctxdh", 3, 4, 2, dh, dtype, cache, tpb, 1, 200, True, 29)
    lens = torch.tensor([1, tpb + 1, 200], dtype=torch.int32)
    w = wl.build_workload(cfg, "cpu", lengths=lens)
    g = torch.Generator().manual_seed(31)
    k = torch.randn(3, 2, 200, dh, generator=g).to(dtype)
    v = torch.randn(3, 2, 200, dh, generator=g).to(dtype)
    pool_ref = torch.zeros_like(w.pool)
    oracle.append_context_reference(k, v, lens, pool_ref, w.offset_table, tokens_per_block=tpb,
                                    cache_mode=CACHE_MODE[cache], kv_scale_orig_quant=w.scale_orig_quant)
    wd = wl.to_device(w, "cuda:0")
    wd.pool.zero_()
    plugin = wl.make_plugin(cfg, 0)
    try:
        plugin.append_context(k.cuda(), v.cuda(), lens.cuda(), wd.kv_cache_block_pointers, wd.kv_orig_quant_scale)
        torch.cuda.synchronize()
        assert torch.equal(wd.pool.cpu(), pool_ref)
    finally:
        plugin.close()


@pytest.mark.parametrize("dh,cache,dtype,heads", [(96, "fp8", torch.float16, (8, 2)), (256, "none", torch.bfloat16, (4, 4)),
                                                  (80, "int8", torch.float16, (6, 3))])
def test_several_new_tokens_on_other_head_sizes(pkg, dh, cache, dtype, heads):
    import test_multi_token_gpu as mt
    cfg = workloads.DecodeConfig("mtdh", 3, heads[0], heads[1], dh, dtype, cache, 32, 0, 400, True, 303)
    packed, _ = mt._tree("small", cfg.batch)
    q_len = packed.shape[1]
    pasts = workloads.draw_lengths(cfg)
    pasts[0] = 0
    w = mt._workload(pkg, cfg, q_len, pasts)
    ref, pool_ref = mt._oracle(w, packed)
    out, pool = mt._run(pkg, w, packed)
    assert torch.equal(pool, pool_ref)
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("dh,rope", [
    (256, dict(position_embedding_type=1, rotary_embedding_dim=64, rotary_embedding_base=10000.0)),   # GPT-J shape
    (96, dict(position_embedding_type=2, rotary_embedding_dim=96, rotary_embedding_base=10000.0)),
    (80, dict(position_embedding_type=2, rotary_embedding_dim=32, rotary_embedding_base=10000.0)),
])
def test_rope_and_bias_on_other_head_sizes(pkg, dh, rope):
    import test_rope_bias_gpu as rb
    wl = workloads
    dtype = torch.float16
    cfg = wl.DecodeConfig("ropedh", 3, 8, 2, dh, dtype, "fp8", 64, 30, 500, True, 79)
    w_cpu = wl.build_workload(cfg, "cpu")
    g = torch.Generator().manual_seed(3)
    bias = (torch.randn((8 + 2 * 2) * dh, generator=g) * 0.5).to(dtype)
    ref, pool_ref = rb._oracle(w_cpu, rope, bias)
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = rb._plugin(pkg, cfg, rope, True)
    try:
        ws = torch.empty(max(plugin.get_workspace_size(cfg.batch, 600), 128), dtype=torch.uint8, device="cuda:0")
        out = plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                        w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                        qkv_bias=bias.cuda(), workspace=ws)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
    finally:
        plugin.close()
    pool = w.pool.cpu()
    changed = pool_ref != w_cpu.pool
    agree = rb._byte_agreement(pool, pool_ref, changed | (pool != w_cpu.pool))
    assert agree > 0.99, agree
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("cache,heads,tpb", [("fp8", (16, 16), 64), ("int8", (8, 2), 32), ("none", (16, 16), 16),
                                             ("fp8", (4, 1), 128)])
def test_head_size_256_on_the_streaming_kernel_with_split_k(pkg, cache, heads, tpb):
    """Head size 256 (GPT-J- / Gemma-shaped) runs on the streaming per-head kernel: long sequences in a small batch are
    split into partitions and merged (the merge kernel's 8-floats-per-lane form)."""
    wl = workloads
    cfg = wl.DecodeConfig("dh256", 2, heads[0], heads[1], 256, torch.bfloat16, cache, tpb, 1, 9000, True, 3256)
    lens = torch.tensor([5000, 9000], dtype=torch.int32)
    res = gpu_step_and_compare(pkg, cfg, lengths=lens)
    assert res["plan"]["kernel"] == "mha_cuda_core" and res["plan"]["num_partitions"] > 1, res["plan"]


@pytest.mark.parametrize("heads,tpb,lens", [((8, 1), 64, [1, 300, 5000]), ((16, 4), 16, [0, 63, 900]),
                                            ((24, 2), 128, [17, 2000, 7000])])
def test_head_size_256_grouped_heads_over_a_16_bit_cache(pkg, heads, tpb, lens):
    """Gemma-shaped grouped heads (Dh 256, bf16 cache): the tensor-core grouped-head kernel, split-K and merge."""
    wl = workloads
    cfg = wl.DecodeConfig("dh256g", len(lens), heads[0], heads[1], 256, torch.bfloat16, "none", tpb, 0, max(lens), True, 3257)
    res = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert res["plan"]["kernel"] == "gqa_tensor_core", res["plan"]


def test_head_size_256_draft_tokens_over_a_16_bit_cache(pkg):
    import test_multi_token_gpu as mt
    cfg = workloads.DecodeConfig("mt256", 2, 8, 1, 256, torch.bfloat16, "none", 32, 0, 600, True, 3258)
    packed, _ = mt._tree("small", cfg.batch)
    w = mt._workload(pkg, cfg, packed.shape[1])
    ref, pool_ref = mt._oracle(w, packed)
    out, pool = mt._run(pkg, w, packed)
    assert torch.equal(pool, pool_ref)
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())
