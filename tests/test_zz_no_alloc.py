"""The allocation-free entry point against the regular one.

Some hosts of this library may not allocate device memory around a decode step: a plugin whose
scratch request was fixed when its engine was built and cannot grow with the live batch, a step that
runs while the device allocator is frozen, or an embedding that has no allocator at all (cudaMalloc is
off limits there).  For them dx_attn_enqueue_generation_static_scratch keeps the split-K partial
results in a fixed 8 MiB array inside the library instead of a caller-provided workspace.  This test
drives both entry points through the C ABI on the same inputs, twice in a row, and expects the same
output: the array keeps the previous call's contents, so the second call shows that nothing stale
leaks into a result.  It also checks that a batch whose partials do not fit is refused on the host,
and that the feature paths (beams, several new tokens per sequence), which need no partials at all,
are served like the regular entry point serves them.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

import workloads

from helpers import MAX_ABS_TOL, MEAN_ABS_TOL, oracle_step

pytestmark = pytest.mark.gpu


def _params(P, plugin, w, out, workspace):
    cfg = w.cfg
    p, _ = plugin._params(w.qkv, w.sequence_length, w.host_past_key_value_lengths.to(torch.int32).contiguous(),
                          w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale, out, workspace,
                          w.max_blocks_per_seq * cfg.tokens_per_block)
    return p


def test_static_scratch_matches_workspace_entry_point(pkg):
    wl, P = workloads, pkg.plugin
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

        # allocation-free entry point: no workspace passed at all, two calls in a row.  The first call on a device
        # looks the array's address up (which may load the library's device code: a driver-side allocation), so
        # the free-memory comparison is made around the second call, through cudaMemGetInfo.
        for call in range(2):
            out = torch.full_like(out_ref, float("nan"))
            q = _params(P, plugin, w, out, None)
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            st = lib.dx_attn_enqueue_generation_static_scratch(plugin._h, ctypes.byref(q), stream)
            assert st == P.DX_OK, (call, st)
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            if call == 1:
                assert free_after == free_before, "device memory was allocated (or freed) during the call"
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
    """A batch whose partial results outgrow the fixed array is refused before anything is launched.  Every
    argument is real and valid - lengths on the device, QKV and output of the right size, a table whose every entry
    points at one real block - so that a refusal that went missing would fail an assertion here instead of
    sending a kernel to wild addresses."""
    wl, P = workloads, pkg.plugin
    lib = pkg.load_library()
    # 49 short sequences and one very long one: the long one is cut into many partitions and the
    # dense [rows, partitions] partial buffer outgrows the fixed array
    cfg = wl.DecodeConfig("toolarge", 50, 64, 8, 128, torch.bfloat16, "fp8", 64, 128, 60000, True, 5)
    plugin = wl.make_plugin(cfg, 0)
    try:
        dev = "cuda:0"
        lens = torch.tensor([128] * 49 + [60000], dtype=torch.int32)
        blocks = (60000 + 1 + 63) // 64
        block = torch.zeros(cfg.num_kv_heads * 64 * cfg.head_size, dtype=torch.uint8, device=dev)  # one K/V block
        table = torch.full((cfg.batch, 2, blocks), block.data_ptr(), dtype=torch.int64, device=dev)
        qkv = torch.zeros(cfg.batch, (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size, dtype=cfg.dtype, device=dev)
        out = torch.zeros(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device=dev)
        seq = (lens + 1).to(dev)
        scale = torch.ones(1, dtype=torch.float32, device=dev)
        # the plan of exactly this call splits, and its partials do not fit the fixed array
        plan = plugin.plan(cfg.batch, 60000, lens)
        assert plan["num_partitions"] > 1 or plan.get("stream_k_ctas", 0) > 1, plan
        assert plugin.get_workspace_size(cfg.batch, 60000) > lib.dx_attn_static_scratch_bytes()
        p, _ = plugin._params(qkv, seq, lens, table, scale, scale, out, None, blocks * 64)
        n0 = plugin.launch_count()
        st = lib.dx_attn_enqueue_generation_static_scratch(plugin._h, ctypes.byref(p), None)
        assert st == P.DX_ERR_WORKSPACE, st
        assert plugin.launch_count() == n0
        # the regular entry point asks for the same memory through its workspace argument
        assert lib.dx_attn_enqueue_generation(plugin._h, ctypes.byref(p), None) == P.DX_ERR_WORKSPACE
        assert plugin.launch_count() == n0
        torch.cuda.synchronize()
        assert not bool(out.any())
    finally:
        plugin.close()


def test_static_scratch_serves_beams_like_the_regular_entry_point(pkg):
    """Beam search goes to the kernel that needs no split-K partials: the fixed array is not a limit there, however
    long the sequences are."""
    import test_generation_features_gpu as feat
    c = feat.Case((8, 2), 128, torch.bfloat16, "int8", 64, 2, beam=2, past_lo=300, past_hi=900, seed=11)
    w_cpu, ex = feat._build(pkg, c)
    w = workloads.to_device(w_cpu, "cuda:0")
    dev = lambda t: None if t is None else t.to("cuda:0")
    outs = []
    for static in (False, True, True):
        plugin = feat._plugin(pkg, c)
        try:
            out = plugin.enqueue_generation(
                w.qkv, w.sequence_length, w.host_past_key_value_lengths, w.kv_cache_block_pointers,
                w.kv_orig_quant_scale, w.kv_quant_orig_scale, max_attention_window=ex["max_attention_window"],
                cache_indirection=dev(ex["cache_indirection"]), beam_width=ex["beam_width"],
                context_lengths=dev(ex["context_lengths"]), static_scratch=static)
            torch.cuda.synchronize()
            assert plugin.device_status() == 0
            outs.append(out.clone())
        finally:
            plugin.close()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref, _ = feat._oracle(w_cpu, ex)
    e = (outs[1].float().cpu() - ref).abs()
    assert e.max().item() < MAX_ABS_TOL and e.mean().item() < MEAN_ABS_TOL


def test_static_scratch_serves_several_new_tokens_per_sequence(pkg):
    import test_multi_token_gpu as mt
    wl = workloads
    cfg = wl.DecodeConfig("mt_noalloc", 3, 8, 2, 128, torch.bfloat16, "fp8", 64, 100, 400, True, 77)
    q_len = 4
    w_cpu = mt._workload(pkg, cfg, q_len)
    packed = torch.tensor([[(1 << (t + 1)) - 1] for t in range(q_len)], dtype=torch.int32)  # chain: token t sees 0..t
    packed = packed.view(1, q_len, 1).repeat(cfg.batch, 1, 1).contiguous()
    out_a, pool_a = mt._run(pkg, w_cpu, packed)
    out_b, pool_b = mt._run(pkg, w_cpu, packed, static_scratch=True)
    out_c, pool_c = mt._run(pkg, w_cpu, packed, static_scratch=True)
    assert torch.equal(out_a, out_b) and torch.equal(out_a, out_c)
    assert torch.equal(pool_a, pool_b) and torch.equal(pool_a, pool_c)
    ref, pool_ref = mt._oracle(w_cpu, packed)
    assert torch.equal(pool_b, pool_ref)
    e = (out_b - ref).abs()
    assert e.max().item() < MAX_ABS_TOL and e.mean().item() < MEAN_ABS_TOL
