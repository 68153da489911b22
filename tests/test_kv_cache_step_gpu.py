"""Device-resident per-step cache bookkeeping (dx_kv_cache_step): the same tables and lengths as the host block
manager, step by step; an exhausted free list is reported through the status word; and a CUDA graph of
{bookkeeping, decode step} replays generation steps with no host work in between, checked against the oracle."""
import pytest
import torch

import oracle
from helpers import MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu


def _free_list(pool, blocks, block_bytes, order):
    base = pool.data_ptr()
    return torch.tensor([[base + i * block_bytes, base + (i + blocks) * block_bytes] for i in order], dtype=torch.int64)


def _setup(pkg, B, ctx, tpb, M, blocks, H=8, Hkv=2, Dh=128, seed=3):
    blk_bytes = Hkv * tpb * Dh
    pool = torch.zeros(2 * blocks * blk_bytes, dtype=torch.uint8, device="cuda:0")
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(blocks, generator=g).tolist()
    mgr = pkg.KVCacheManager(pool, blocks, tpb, M, free_order=order)
    for i, l in enumerate(ctx):
        mgr.add_sequence(pkg.GenerationSequence(i, i), l)
    plugin = pkg.GPTAttentionPlugin(num_heads=H, num_kv_heads=Hkv, head_size=Dh, multi_block_mode=True,
                                    kv_cache_quant_mode=pkg.QuantMode.FP8_KV_CACHE, tokens_per_block=tpb,
                                    type_id=torch.bfloat16)
    used = blocks - len(mgr.free_blocks)
    free = _free_list(pool, blocks, blk_bytes, mgr.free_blocks).cuda()
    return pool, mgr, plugin, free, used, g


def test_device_step_builds_the_host_managers_tables(pkg):
    B, tpb, M, blocks = 37, 16, 10, 400
    g0 = torch.Generator().manual_seed(9)
    ctx = torch.randint(1, 80, (B,), generator=g0).tolist()
    pool, mgr, plugin, free, _, _ = _setup(pkg, B, ctx, tpb, M, blocks)
    try:
        table = mgr.get_block_pointers().cuda()
        lens = torch.tensor(ctx, dtype=torch.int32, device="cuda:0")
        cursor = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        for step in range(40):
            mgr.step([False] * B)
            plugin.kv_cache_step(lens, table, free, cursor)
            torch.cuda.synchronize()
            assert torch.equal(table.cpu(), mgr.get_block_pointers()), f"step {step}"
            assert lens.cpu().tolist() == mgr.lens, f"step {step}"
        assert int(cursor) == blocks - len(mgr.free_blocks) - (blocks - free.shape[0])
        assert plugin.device_status() == 0
    finally:
        plugin.close()


def test_exhausted_free_list_is_reported(pkg):
    B, tpb, M, blocks = 4, 16, 4, 8
    pool, mgr, plugin, free, _, _ = _setup(pkg, B, [16, 16, 16, 16], tpb, M, blocks)  # 4 blocks used, 4 free
    P = pkg.plugin
    try:
        table = mgr.get_block_pointers().cuda()
        lens = torch.full((B,), 16, dtype=torch.int32, device="cuda:0")
        cursor = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        plugin.kv_cache_step(lens, table, free[:2].contiguous(), cursor)  # 4 sequences need a block, 2 are left
        torch.cuda.synchronize()
        assert plugin.device_status() == P.DX_ERR_BOUNDS
        assert plugin.device_status() == P.DX_OK  # reading the status clears it
        t = table.cpu()
        assert (t[:2, :, 1] != 0).all() and (t[2:, :, 1] == 0).all()
        assert int(cursor) == 2
    finally:
        plugin.close()


def test_graph_of_bookkeeping_and_decode_step_replays_without_host_work(pkg):
    H, Hkv, Dh, tpb, B, M, blocks, steps = 8, 2, 128, 16, 3, 12, 64, 24
    ctx = [5, 16, 31]
    pool, mgr, plugin, free, _, g = _setup(pkg, B, ctx, tpb, M, blocks, H, Hkv, Dh, seed=42)
    s_qo = 6.0 / 448.0
    s_oq = 1.0 / s_qo
    sq = torch.tensor([s_oq], dtype=torch.float32, device="cuda:0")
    sd = torch.tensor([s_qo], dtype=torch.float32, device="cuda:0")
    base = pool.data_ptr()
    pool_ref = torch.zeros(pool.numel(), dtype=torch.uint8)
    try:
        L = max(ctx)
        k = torch.randn(B, Hkv, L, Dh, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Hkv, L, Dh, generator=g).to(torch.bfloat16)
        table = mgr.get_block_pointers().cuda()
        lens = torch.tensor(ctx, dtype=torch.int32, device="cuda:0")
        plugin.append_context(k.cuda(), v.cuda(), lens, table, sq)
        off = torch.where(table.cpu() != 0, table.cpu() - base, torch.full_like(table.cpu(), -1))
        oracle.append_context_reference(k, v, lens.cpu(), pool_ref, off, tokens_per_block=tpb,
                                        cache_mode=oracle.CACHE_FP8, kv_scale_orig_quant=s_oq)
        cursor = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        qkv = torch.zeros(B, (H + 2 * Hkv) * Dh, dtype=torch.bfloat16, device="cuda:0")
        out = torch.empty(B, H * Dh, dtype=torch.bfloat16, device="cuda:0")
        # the launch plan is fixed at capture: size it for the longest sequence the replays will reach
        final_past = torch.tensor([c + steps for c in ctx], dtype=torch.int32)
        ws = torch.empty(plugin.get_workspace_size(B, int(final_past.max())) + 256, dtype=torch.uint8, device="cuda:0")
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            # warm-up outside the capture must not change the state: run on copies
            plugin.kv_cache_step(lens.clone(), table.clone(), free, cursor.clone(), stream=side)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                plugin.kv_cache_step(lens, table, free, cursor, stream=side)
                plugin.enqueue_generation(qkv, lens, final_past, table, sq, sd, out=out, workspace=ws, stream=side)
        for step in range(steps):
            x = torch.randn(B, (H + 2 * Hkv) * Dh, generator=g).to(torch.bfloat16)
            qkv.copy_(x)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            mgr.step([False] * B)
            t_host = mgr.get_block_pointers()
            assert torch.equal(table.cpu(), t_host), f"step {step}"
            seq = torch.tensor(mgr.lens, dtype=torch.int32)
            assert torch.equal(lens.cpu(), seq)
            off = torch.where(t_host != 0, t_host - base, torch.full_like(t_host, -1))
            ref = oracle.decode_attention_reference(
                x, seq, pool_ref, off, num_heads=H, num_kv_heads=Hkv, head_size=Dh, tokens_per_block=tpb,
                cache_mode=oracle.CACHE_FP8, kv_scale_orig_quant=s_oq, kv_scale_quant_orig=s_qo)
            assert torch.equal(pool.cpu(), pool_ref), f"step {step}"
            err = (out.float().cpu() - ref).abs()
            assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, f"step {step}"
        assert plugin.device_status() == 0
    finally:
        plugin.close()
