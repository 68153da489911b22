"""The callers either side of the path, together: prompt written by the context append, block tables from
the product's host manager (new blocks allocated as sequences cross block boundaries), 20 decode steps checked
against the oracle every step; and one decode step captured in a CUDA graph and replayed (the per-step launch
cost dominates small batches - the reference runtime pays it every step, generation.py:2175-2387)."""
import pytest
import torch

import workloads

import oracle
from helpers import MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu


def test_prompt_and_twenty_decode_steps_with_block_manager(pkg):
    H, Hkv, Dh, tpb, B = 8, 2, 128, 16, 3
    blocks, M = 64, 12
    blk_bytes = Hkv * tpb * Dh
    pool = torch.zeros(2 * blocks * blk_bytes, dtype=torch.uint8, device="cuda:0")
    g = torch.Generator().manual_seed(42)
    order = torch.randperm(blocks, generator=g).tolist()
    mgr = pkg.KVCacheManager(pool, blocks, tpb, M, free_order=order)
    ctx = [5, 16, 31]
    for i, l in enumerate(ctx):
        mgr.add_sequence(pkg.GenerationSequence(i, i), l)
    L = max(ctx)
    k = torch.randn(B, Hkv, L, Dh, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Hkv, L, Dh, generator=g).to(torch.bfloat16)
    s_qo = 6.0 / 448.0
    s_oq = 1.0 / s_qo
    sq = torch.tensor([s_oq], dtype=torch.float32, device="cuda:0")
    sd = torch.tensor([s_qo], dtype=torch.float32, device="cuda:0")
    plugin = pkg.GPTAttentionPlugin(num_heads=H, num_kv_heads=Hkv, head_size=Dh, multi_block_mode=True,
                                    kv_cache_quant_mode=pkg.QuantMode.FP8_KV_CACHE, tokens_per_block=tpb,
                                    type_id=torch.bfloat16)
    base = pool.data_ptr()
    pool_ref = torch.zeros(pool.numel(), dtype=torch.uint8)
    try:
        table = mgr.get_block_pointers()
        lens = torch.tensor(ctx, dtype=torch.int32)
        plugin.append_context(k.cuda(), v.cuda(), lens.cuda(), table.cuda(), sq)
        off = torch.where(table != 0, table - base, torch.full_like(table, -1))
        oracle.append_context_reference(k, v, lens, pool_ref, off, tokens_per_block=tpb, cache_mode=oracle.CACHE_FP8,
                                        kv_scale_orig_quant=s_oq)
        for step in range(20):
            mgr.step([False] * B)  # may allocate a block for the token about to be written
            table = mgr.get_block_pointers()
            past = mgr.host_past_key_value_lengths() - 1
            qkv = torch.randn(B, (H + 2 * Hkv) * Dh, generator=g).to(torch.bfloat16)
            seq = (past + 1).to(torch.int32)
            out = plugin.enqueue_generation(qkv.cuda(), seq.cuda(), past, table.cuda(), sq, sd)
            torch.cuda.synchronize()
            off = torch.where(table != 0, table - base, torch.full_like(table, -1))
            ref = oracle.decode_attention_reference(
                qkv, seq, pool_ref, off, num_heads=H, num_kv_heads=Hkv, head_size=Dh, tokens_per_block=tpb,
                cache_mode=oracle.CACHE_FP8, kv_scale_orig_quant=s_oq, kv_scale_quant_orig=s_qo)
            assert torch.equal(pool.cpu(), pool_ref), f"step {step}"
            err = (out.float().cpu() - ref).abs()
            assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, f"step {step}"
        assert mgr.lens == [c + 20 for c in ctx]
    finally:
        plugin.close()


def test_step_replayed_from_a_cuda_graph(pkg):
    wl = workloads
    cfg = wl.DecodeConfig("graph", 6, 16, 2, 128, torch.bfloat16, "fp8", 64, 900, 2500, True, 31)
    w = wl.to_device(wl.build_workload(cfg, "cpu"), "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        eager = wl.run_step(plugin, w).clone()
        torch.cuda.synchronize()
        out = torch.zeros_like(eager)
        max_past = int(w.host_past_key_value_lengths.max())
        ws = torch.empty(max(plugin.get_workspace_size(cfg.batch, max_past), 256), dtype=torch.uint8, device="cuda:0")
        s = torch.cuda.Stream()
        call = plugin.bind_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                      w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                      out=out, workspace=ws, stream=s,
                                      max_attention_window=w.max_blocks_per_seq * cfg.tokens_per_block)
        with torch.cuda.stream(s):
            call()  # warm-up outside capture
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            call()
        out.zero_()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
        assert plugin.device_status() == 0
    finally:
        plugin.close()
