"""The allocation-free entry point against the regular one.

Some hosts of this library may not allocate device memory around a decode step: a plugin whose
scratch request was fixed when its engine was built and cannot grow with the live batch, a step that
runs while the device allocator is frozen, or an embedding that has no allocator at all (cudaMalloc is
off limits there).  For them dx_attn_enqueue_generation_static_scratch keeps the split-K partial
results in a fixed 8 MiB array inside the library instead of a caller-provided workspace.  This test
drives both entry points through the C ABI on the same inputs, twice in a row, and expects the same
output: the array keeps the previous call's contents, so the second call shows that nothing stale
leaks into a result.  It also checks that a batch whose partials do not fit is refused on the host.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from helpers import MAX_ABS_TOL, MEAN_ABS_TOL, oracle_step

pytestmark = pytest.mark.gpu


def _params(P, plugin, w, out, workspace):
    cfg = w.cfg
    p, _ = plugin._params(w.qkv, w.sequence_length, w.host_past_key_value_lengths.to(torch.int32).contiguous(),
                          w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale, out, workspace,
                          w.max_blocks_per_seq * cfg.tokens_per_block)
    return p


def test_static_scratch_matches_workspace_entry_point(pkg):
    wl, P = pkg.workloads, pkg.plugin
    lib = pkg.load_library()
    # long sequences, few rows: the plan splits every sequence into several partitions
    cfg = wl.DecodeConfig("noalloc", 3, 16, 2, 128, torch.bfloat16, "fp8", 64, 3000, 5000, True, 321)
    w_cpu = wl.build_workload(cfg, "cpu")
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    try:
        max_past = int(w.host_past_key_value_lengths.max())
        plan = plugin.plan(cfg.batch, max_past)
        assert plan["num_partitions"] > 1, plan
        need = plugin.get_workspace_size(cfg.batch, max_past)
        assert 0 < need <= lib.dx_attn_static_scratch_bytes()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        # regular entry point with a caller-owned workspace
        ws = torch.empty(need, dtype=torch.uint8, device="cuda:0")
        out_ref = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device="cuda:0")
        p = _params(P, plugin, w, out_ref, ws)
        assert lib.dx_attn_enqueue_generation(plugin._h, ctypes.byref(p), stream) == P.DX_OK
        torch.cuda.synchronize()
        pool_after = w.pool.clone()

        # allocation-free entry point: no workspace passed at all, two calls in a row
        for call in range(2):
            out = torch.full_like(out_ref, float("nan"))
            q = _params(P, plugin, w, out, None)
            before = torch.cuda.memory_allocated()
            st = lib.dx_attn_enqueue_generation_static_scratch(plugin._h, ctypes.byref(q), stream)
            assert st == P.DX_OK, (call, st)
            assert torch.cuda.memory_allocated() == before
            torch.cuda.synchronize()
            assert plugin.device_status() == 0
            d = (out.float() - out_ref.float()).abs()
            assert torch.isfinite(out.float()).all()
            assert d.max().item() < MAX_ABS_TOL and d.mean().item() < MEAN_ABS_TOL, (call, d.max().item())
            assert torch.equal(out, out_ref), f"call {call}: same kernels, same order -> same bits expected"
            assert torch.equal(w.pool, pool_after)

        # and both agree with the oracle
        ref, _ = oracle_step(w_cpu)
        e = (out.float().cpu() - ref).abs()
        assert e.max().item() < MAX_ABS_TOL and e.mean().item() < MEAN_ABS_TOL
    finally:
        plugin.close()


def test_static_scratch_refuses_what_does_not_fit(pkg):
    wl, P = pkg.workloads, pkg.plugin
    lib = pkg.load_library()
    # 49 short sequences and one very long one: the long one is cut into many partitions and the
    # dense [rows, partitions] partial buffer outgrows the fixed array; nothing may be launched
    cfg = wl.DecodeConfig("toolarge", 50, 64, 8, 128, torch.bfloat16, "fp8", 64, 128, 60000, True, 5)
    plugin = wl.make_plugin(cfg, 0)
    try:
        lens = torch.tensor([128] * 49 + [60000], dtype=torch.int32)
        blocks = (60000 + 1 + 63) // 64
        dummy = torch.zeros(16, dtype=torch.uint8, device="cuda:0")
        p = P._GenParams()
        p.struct_size = ctypes.sizeof(P._GenParams)
        p.attention_input = dummy.data_ptr()
        p.sequence_lengths = dummy.data_ptr()
        p.host_past_key_value_lengths = lens.data_ptr()
        p.beam_width, p.num_requests, p.max_blocks_per_sequence = 1, cfg.batch, blocks
        p.max_attention_window = p.cyclic_attention_window_size = blocks * 64
        p.block_pointers = dummy.data_ptr()
        p.kv_scale_orig_quant = p.kv_scale_quant_orig = dummy.data_ptr()
        p.context_buf = dummy.data_ptr()
        n0 = plugin.launch_count()
        st = lib.dx_attn_enqueue_generation_static_scratch(plugin._h, ctypes.byref(p), None)
        assert st == P.DX_ERR_WORKSPACE, st
        assert plugin.launch_count() == n0
        # the regular entry point asks for the same memory through its workspace argument
        assert lib.dx_attn_enqueue_generation(plugin._h, ctypes.byref(p), None) == P.DX_ERR_WORKSPACE
        assert plugin.get_workspace_size(cfg.batch, 60000) > lib.dx_attn_static_scratch_bytes()
    finally:
        plugin.close()
