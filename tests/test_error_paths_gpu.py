"""Host-side failure detection on a live GPU: every bad call must come back with a status code and
ZERO kernels launched (the reference throws or exits; nothing here may fault, trap or hang a GPU)."""
import ctypes
import dataclasses

import pytest
import torch

import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture()
def setup(pkg):
    wl = workloads
    cfg = wl.DecodeConfig("err", 3, 16, 2, 128, torch.bfloat16, "fp8", 64, 2000, 3000, True, 1)
    w = wl.to_device(wl.build_workload(cfg, "cpu"), "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    out = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device="cuda:0")
    need = plugin.get_workspace_size(cfg.batch, int(w.host_past_key_value_lengths.max()))
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda:0")
    yield pkg, cfg, w, plugin, out, ws
    plugin.close()


def _call(pkg, plugin, w, out, ws, **over):
    P = pkg.plugin
    p, _ = plugin._params(w.qkv, w.sequence_length, w.host_past_key_value_lengths.contiguous(),
                          w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale, out, ws,
                          w.max_blocks_per_seq * w.cfg.tokens_per_block)
    for k, v in over.items():
        setattr(p, k, v)
    n0 = plugin.launch_count()
    st = plugin.lib.dx_attn_enqueue_generation(plugin._h, ctypes.byref(p),
                                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, plugin.launch_count() - n0


def test_good_call_launches_and_bad_calls_do_not(setup):
    pkg, cfg, w, plugin, out, ws = setup
    P = pkg.plugin
    st, n = _call(pkg, plugin, w, out, ws)
    assert st == P.DX_OK and n >= 1
    torch.cuda.synchronize()
    assert plugin.device_status() == P.DX_OK
    bad = [
        (dict(attention_input=None), P.DX_ERR_BAD_ARG),
        (dict(sequence_lengths=None), P.DX_ERR_BAD_ARG),
        (dict(block_pointers=None), P.DX_ERR_BAD_ARG),
        (dict(context_buf=None), P.DX_ERR_BAD_ARG),
        (dict(attention_input=w.qkv.data_ptr() + 2), P.DX_ERR_BAD_ARG),          # misaligned
        (dict(kv_scale_orig_quant=None), P.DX_ERR_BAD_ARG),                       # quantised cache needs scales
        (dict(num_requests=-1), P.DX_ERR_BAD_ARG),
        (dict(max_blocks_per_sequence=0), P.DX_ERR_BAD_ARG),
        (dict(max_blocks_per_sequence=2), P.DX_ERR_BAD_ARG),                      # table cannot hold the tokens
        (dict(beam_width=0), P.DX_ERR_BAD_ARG),
        (dict(beam_width=3), P.DX_ERR_BAD_ARG),                                   # beams without an indirection table
        (dict(sink_token_length=4), P.DX_ERR_UNSUPPORTED),                        # sink ends inside a block
        (dict(cyclic_attention_window_size=512), P.DX_ERR_UNSUPPORTED),          # wrapped window, table with spare blocks
        (dict(cyclic_attention_window_size=0), P.DX_ERR_BAD_ARG),
        (dict(alibi_slopes=w.qkv.data_ptr()), P.DX_ERR_BAD_ARG),                  # slopes without an ALiBi plugin
        (dict(struct_size=8), P.DX_ERR_BAD_ARG),
    ]
    for over, want in bad:
        st, n = _call(pkg, plugin, w, out, ws, **over)
        assert st == want, (over, st)
        assert n == 0, over
    # workspace: missing, too small, misaligned - only checked when the plan splits
    if plugin.plan(cfg.batch, int(w.host_past_key_value_lengths.max()))["num_partitions"] > 1:
        for over in (dict(workspace=None, workspace_bytes=0), dict(workspace_bytes=64)):
            st, n = _call(pkg, plugin, w, out, ws, **over)
            assert st == P.DX_ERR_WORKSPACE and n == 0, over
        st, n = _call(pkg, plugin, w, out, ws, workspace=ws.data_ptr() + 8)
        assert st == P.DX_ERR_BAD_ARG and n == 0
    # an empty batch is a successful no-op
    st, n = _call(pkg, plugin, w, out, ws, num_requests=0)
    assert st == P.DX_OK and n == 0
    torch.cuda.synchronize()
    assert plugin.device_status() == P.DX_OK


def test_validate_catches_corrupted_tables(setup):
    pkg, cfg, w, plugin, out, ws = setup
    P = pkg.plugin
    base, size = w.pool.data_ptr(), w.pool.numel()
    host = w.host_kv_cache_block_pointers.clone()
    lens = w.host_past_key_value_lengths
    assert plugin.validate(host, lens, base, size) == P.DX_OK
    t = host.clone(); t[1, 0, 0] = base + size            # one block past the pool
    assert plugin.validate(t, lens, base, size) == P.DX_ERR_BOUNDS
    t = host.clone(); t[0, 1, 2] = base - 64               # before the pool
    assert plugin.validate(t, lens, base, size) == P.DX_ERR_BOUNDS
    t = host.clone(); t[2, 0, 1] += 4                      # misaligned block
    assert plugin.validate(t, lens, base, size) == P.DX_ERR_BAD_ARG
    t = host.clone(); t[0, 0, 0] = 0                       # null pointer for a needed block
    assert plugin.validate(t, lens, base, size) == P.DX_ERR_BOUNDS
    long = lens.clone(); long[0] = w.max_blocks_per_seq * cfg.tokens_per_block + 5
    assert plugin.validate(host, long, base, size) == P.DX_ERR_BOUNDS


def test_guard_bytes_around_pool_and_workspace_stay_intact(pkg):
    """Poisoned guard regions before and after the KV pool, the output and the workspace: a step must
    not write outside its buffers (stand-in for compute-sanitizer, which is closed on this pool)."""
    wl = workloads
    cfg = wl.DecodeConfig("guard", 5, 8, 2, 128, torch.bfloat16, "int8", 32, 900, 1500, True, 12)
    w_cpu = wl.build_workload(cfg, "cpu")
    G = 4096
    big = torch.full((w_cpu.pool.numel() + 2 * G,), 0xA5, dtype=torch.uint8, device="cuda:0")
    big[G:-G] = w_cpu.pool.cuda()
    base = big.data_ptr() + G
    ptrs = torch.where(w_cpu.offset_table >= 0, w_cpu.offset_table + base, torch.zeros_like(w_cpu.offset_table)).cuda()
    plugin = wl.make_plugin(cfg, 0)
    try:
        need = plugin.get_workspace_size(cfg.batch, int(w_cpu.host_past_key_value_lengths.max()))
        wsb = torch.full((need + 2 * G,), 0x5A, dtype=torch.uint8, device="cuda:0")
        nout = cfg.batch * cfg.num_heads * cfg.head_size
        outb = torch.full((nout + 2 * G,), -7.0, dtype=cfg.dtype, device="cuda:0")
        plugin.enqueue_generation(w_cpu.qkv.cuda(), w_cpu.sequence_length.cuda(), w_cpu.host_past_key_value_lengths,
                                  ptrs, w_cpu.kv_orig_quant_scale.cuda(), w_cpu.kv_quant_orig_scale.cuda(),
                                  out=outb[G:G + nout].view(cfg.batch, -1), workspace=wsb[G:G + need] if need else None)
        torch.cuda.synchronize()
        assert bool((big[:G] == 0xA5).all()) and bool((big[-G:] == 0xA5).all())
        assert bool((wsb[:G] == 0x5A).all()) and bool((wsb[-G:] == 0x5A).all())
        assert bool((outb[:G] == -7.0).all()) and bool((outb[-G:] == -7.0).all())
        assert torch.isfinite(outb[G:G + nout].float()).all()
    finally:
        plugin.close()


# ---------------------------------------------------------------------------------------------------------
# Device-side failure reporting.  Every wait in the kernels has a poll limit; when one runs out the kernel
# records a time-out in the handle's status word and returns.  The tests below make that happen without
# hanging or faulting anything: a self-test kernel waits (a few hundred polls) on a barrier that nothing ever
# arrives on, and the attention kernels are then launched while the word still holds that report, which makes
# every wait in them give up after at most 256 polls.
# ---------------------------------------------------------------------------------------------------------
TIMEOUT_CONFIGS = {
    "gqa_fp8": ("t_gqa", 4, 16, 2, 128, torch.bfloat16, "fp8", 64, 1500, 2500, True, 31),
    "gqa_int8_16heads": ("t_gqa16h", 3, 32, 2, 128, torch.bfloat16, "int8", 128, 700, 1400, True, 32),
    "gqa_bf16_cache": ("t_gqa16", 3, 8, 2, 128, torch.bfloat16, "none", 64, 600, 1200, True, 33),
    "mha_int8": ("t_mha8", 4, 8, 8, 128, torch.bfloat16, "int8", 64, 500, 900, False, 34),
    "mha_fp16": ("t_mha", 4, 6, 6, 64, torch.float16, "none", 64, 300, 800, True, 35),
    "wide_mqa_fp8": ("t_wide", 4, 71, 1, 64, torch.float16, "fp8", 64, 300, 1200, True, 36),
}


@pytest.mark.parametrize("name", sorted(TIMEOUT_CONFIGS))
def test_bounded_wait_expiry_is_reported_and_cleared(pkg, name):
    from helpers import MAX_ABS_TOL, MEAN_ABS_TOL, oracle_step
    wl, P = workloads, pkg.plugin
    cfg = wl.DecodeConfig(*TIMEOUT_CONFIGS[name])
    w_cpu = wl.build_workload(cfg, "cpu")
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        assert plugin.lib.dx_attn_selftest_wait_timeout(plugin._h, 0, stream) == P.DX_ERR_BAD_ARG
        # (1) a wait that nothing satisfies runs out after 300 polls; the kernel records it and returns
        assert plugin.lib.dx_attn_selftest_wait_timeout(plugin._h, 300, stream) == P.DX_OK
        # (2) a real step enqueued while the report is pending: its waits give up early, the kernels take their
        #     time-out exits (rings drained, tensor memory freed) and the stream stays usable
        out_bad = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        del out_bad  # undefined by contract
        # (3) the report is read once, then the word is clear again
        assert plugin.device_status() == P.DX_ERR_TIMEOUT
        assert plugin.device_status() == P.DX_OK
        # (4) the next step is a normal one: pool bytes and output as the oracle has them
        w.pool.copy_(w_cpu.pool.cuda())
        out = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        assert plugin.device_status() == P.DX_OK
        ref, pool_ref = oracle_step(w_cpu)
        assert torch.equal(w.pool.cpu(), pool_ref)
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL
    finally:
        plugin.close()


@pytest.mark.parametrize("streamk", [False, True])
def test_device_length_beyond_the_planned_length_is_reported(pkg, streamk, monkeypatch):
    """host_past_key_value_lengths are what a step is planned with.  A device length that needs more partitions
    than that plan has cannot be served (the surplus tokens have no CTA); it is reported as DX_ERR_BOUNDS instead
    of being dropped silently, the merge stays inside its own rows, and nothing outside the buffers is touched."""
    wl, P = workloads, pkg.plugin
    if streamk:
        cfg = wl.DecodeConfig("exceed_sk", 32, 32, 8, 128, torch.bfloat16, "fp8", 64, 3800, 4000, True, 41)
        host_len = 3000
    else:
        monkeypatch.setenv("DX_ATTN_STREAMK", "0")
        monkeypatch.setenv("DX_ATTN_FORCE_CHUNK", "512")
        cfg = wl.DecodeConfig("exceed", 3, 16, 2, 128, torch.bfloat16, "fp8", 64, 2800, 3000, True, 42)
        host_len = 1000
    w = wl.to_device(wl.build_workload(cfg, "cpu"), "cuda:0")   # tables and pool hold the (long) device lengths
    plugin = wl.make_plugin(cfg, 0)
    try:
        short = torch.full((cfg.batch,), host_len, dtype=torch.int32)
        plan = plugin.plan(cfg.batch, host_len, short)
        assert ("stream_k_ctas" in plan) == streamk, plan
        G = 4096
        need = plugin.get_workspace_size(cfg.batch, host_len)
        wsb = torch.full((need + 2 * G,), 0x5A, dtype=torch.uint8, device="cuda:0")
        out = plugin.enqueue_generation(w.qkv, w.sequence_length, short, w.kv_cache_block_pointers,
                                        w.kv_orig_quant_scale, w.kv_quant_orig_scale, workspace=wsb[G:G + need],
                                        max_attention_window=w.max_blocks_per_seq * cfg.tokens_per_block)
        torch.cuda.synchronize()
        assert plugin.device_status() == P.DX_ERR_BOUNDS
        assert plugin.device_status() == P.DX_OK
        assert bool((wsb[:G] == 0x5A).all()) and bool((wsb[-G:] == 0x5A).all())
        del out
        # with the true lengths the same handle serves the step
        out = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        assert plugin.device_status() == P.DX_OK and torch.isfinite(out.float()).all()
    finally:
        plugin.close()
