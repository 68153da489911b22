"""Shared helpers of the parity tests: run one decode step through the C ABI on the GPU and through
the CPU oracle on identical seeded inputs, and compare bytes and outputs."""
from __future__ import annotations

import os

import torch

import workloads

import oracle

# Where the timing reports of the GPU tests go.
REPORT_DIR = os.environ.get("DX_TEST_REPORT_DIR", "test_reports")

# Tolerances of the attention output against the fp32 oracle (bf16/fp16 outputs).
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3

CACHE_MODE = {"none": oracle.CACHE_T, "int8": oracle.CACHE_INT8, "fp8": oracle.CACHE_FP8}


def oracle_step(w_cpu, pool=None):
    cfg = w_cpu.cfg
    pool = w_cpu.pool.clone() if pool is None else pool
    out = oracle.decode_attention_reference(
        w_cpu.qkv, w_cpu.sequence_length, pool, w_cpu.offset_table, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block,
        cache_mode=CACHE_MODE[cfg.cache], kv_scale_orig_quant=w_cpu.scale_orig_quant,
        kv_scale_quant_orig=w_cpu.scale_quant_orig)
    return out, pool


def expected_changed_positions(w_cpu):
    """Byte positions of the pool that the append may touch: (b, K|V, kv head, Dh*elem) at the new token."""
    cfg = w_cpu.cfg
    row = cfg.head_size * cfg.elem_bytes
    mask = torch.zeros_like(w_cpu.pool, dtype=torch.bool)
    for b in range(cfg.batch):
        pos = int(w_cpu.host_past_key_value_lengths[b])
        bi, li = pos // cfg.tokens_per_block, pos % cfg.tokens_per_block
        for kv in range(2):
            base = int(w_cpu.offset_table[b, kv, bi])
            for h in range(cfg.num_kv_heads):
                o = base + (h * cfg.tokens_per_block + li) * row
                mask[o:o + row] = True
    return mask


def gpu_step_and_compare(pkg, cfg, *, lengths=None, multi_block_mode=None, device="cuda:0", check_twice=True):
    wl = workloads
    w_cpu = wl.build_workload(cfg, "cpu", lengths=lengths)
    w = wl.to_device(w_cpu, device)
    plugin = wl.make_plugin(cfg, torch.device(device).index or 0, multi_block_mode=multi_block_mode)
    try:
        out = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        st = plugin.device_status()
        assert st == 0, f"device status {st} ({pkg.plugin._strerror(st)})"
        ref, pool_ref = oracle_step(w_cpu)
        pool_gpu = w.pool.cpu()
        # (1) the KV bytes written and where: whole pool identical to the oracle's pool
        diff = pool_gpu != pool_ref
        assert not bool(diff.any()), f"{int(diff.sum())} pool bytes differ from the oracle"
        # (2) nothing outside the new token's rows was touched
        touched = pool_gpu != w_cpu.pool
        assert not bool((touched & ~expected_changed_positions(w_cpu)).any())
        # (3) attention output within tolerance of the fp32 oracle
        err = (out.float().cpu() - ref).abs()
        assert torch.isfinite(out.float()).all()
        assert err.max().item() < MAX_ABS_TOL, f"max-abs {err.max().item():.3e}"
        assert err.mean().item() < MEAN_ABS_TOL, f"mean-abs {err.mean().item():.3e}"
        if check_twice:
            # (4) run-to-run determinism (same inputs -> identical bytes): cheap race detector
            out2 = wl.run_step(plugin, w)
            torch.cuda.synchronize()
            assert torch.equal(out, out2)
            assert torch.equal(w.pool.cpu(), pool_ref)
        return {"max_abs": err.max().item(), "mean_abs": err.mean().item(),
                "plan": plugin.plan(cfg.batch, int(w_cpu.host_past_key_value_lengths.max()),
                                    w_cpu.host_past_key_value_lengths)}
    finally:
        plugin.close()
