"""The benchmark configurations at their FULL sizes (c2, c3, c4, c5: up to 805 MB of KV), where the CPU oracle
cannot be run over the whole batch.  Checked instead:
  * the pool: exactly the new token's rows changed, and they hold the oracle's quantised bytes (bit-exact);
  * a sample of sequences against the CPU oracle at full length (output tolerance);
  * split invariance: stream-K / split-K on, off, and the classic partitions agree within tolerance;
  * idempotence: the same step again gives bit-identical output and pool;
  * convexity: every output channel lies inside the range of the (dequantised) V values it averages."""
import dataclasses

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu


def _run(pkg, cfg, w, multi_block=None):
    wl = workloads
    plugin = wl.make_plugin(cfg, 0, multi_block_mode=multi_block)
    try:
        out = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
        return out.clone()
    finally:
        plugin.close()


# (config, tensor-parallel degree): the whole job on one GPU, and one rank's shard of the 4- and 8-way jobs (the
# 8-way shards of c4 and c5 run classic equal partitions at full length, the others stream-K ranges)
CASES = [("c2", 1), ("c3", 1), ("c4", 1), ("c5", 1), ("c4", 4), ("c4", 8), ("c5", 4), ("c5", 8)]


@pytest.mark.parametrize("name,tp", CASES)
def test_full_size_properties(pkg, name, tp, monkeypatch):
    wl = workloads
    cfg = wl.shard_config(wl.CONFIGS[name], tp)
    w = wl.build_workload(cfg, "cuda:0")
    B, H, Hkv, Dh, tpb = cfg.batch, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, cfg.tokens_per_block
    row = Dh * cfg.elem_bytes
    pool_before = w.pool.clone()
    out = _run(pkg, cfg, w)
    assert torch.isfinite(out.float()).all()

    # ---- pool: only the new token's rows changed, with the oracle's bytes ----
    mode = CACHE_MODE[cfg.cache]
    qkv_cpu = w.qkv.cpu()
    k_new = qkv_cpu[:, H * Dh:(H + Hkv) * Dh].view(B, Hkv, Dh)
    v_new = qkv_cpu[:, (H + Hkv) * Dh:].view(B, Hkv, Dh)
    kq = oracle.quantize_kv(k_new, w.scale_orig_quant, mode).cuda()  # [B, Hkv, row] uint8
    vq = oracle.quantize_kv(v_new, w.scale_orig_quant, mode).cuda()
    past = w.host_past_key_value_lengths
    expect = pool_before.clone()
    blocks = expect.view(-1, Hkv, tpb, row)
    blk = Hkv * tpb * row
    for b in range(B):
        pos = int(past[b])
        ko, vo = int(w.offset_table[b, 0, pos // tpb]), int(w.offset_table[b, 1, pos // tpb])
        blocks[ko // blk, :, pos % tpb] = kq[b]
        blocks[vo // blk, :, pos % tpb] = vq[b]
    assert torch.equal(w.pool, expect), "pool differs from (old pool + the oracle's bytes of the new token)"

    # ---- idempotence ----
    out2 = _run(pkg, cfg, w)
    assert torch.equal(out, out2) and torch.equal(w.pool, expect)

    # ---- split invariance ----
    variants = {"multi_block off": _run(pkg, cfg, w, multi_block=False)}
    monkeypatch.setenv("DX_ATTN_STREAMK", "0")
    variants["classic partitions"] = _run(pkg, cfg, w, multi_block=True)
    monkeypatch.delenv("DX_ATTN_STREAMK")
    for what, o in variants.items():
        d = (o.float() - out.float()).abs()
        assert d.max().item() < MAX_ABS_TOL and d.mean().item() < MEAN_ABS_TOL, (what, d.max().item())
    assert torch.equal(w.pool, expect)

    # ---- a sample of sequences against the CPU oracle, at full length ----
    idx = [0, B // 2, B - 1]
    pool_cpu = w.pool.cpu()
    ref = oracle.decode_attention_reference(
        qkv_cpu[idx], w.sequence_length.cpu()[idx], pool_cpu, w.offset_table[idx], num_heads=H, num_kv_heads=Hkv,
        head_size=Dh, tokens_per_block=tpb, cache_mode=mode, kv_scale_orig_quant=w.scale_orig_quant,
        kv_scale_quant_orig=w.scale_quant_orig, append=False)  # the new token is in the pool already
    err = (out[idx].float().cpu() - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())

    # ---- convexity: min_t V <= out <= max_t V per (sequence, kv head, channel), for the sampled sequences ----
    G = H // Hkv
    deq = 1.0 if mode == oracle.CACHE_T else w.scale_quant_orig
    for j, b in enumerate(idx):
        total = int(past[b]) + 1
        nb = (total + tpb - 1) // tpb
        voffs = w.offset_table[b, 1, :nb]
        vraw = pool_cpu.view(-1, Hkv, tpb, row)[voffs // blk].permute(1, 0, 2, 3).reshape(Hkv, nb * tpb, row)[:, :total]
        V = oracle.dequantize_kv(vraw, mode, cfg.dtype) * deq  # [Hkv, total, Dh]
        lo, hi = V.amin(dim=1), V.amax(dim=1)                   # [Hkv, Dh]
        o = out[b].float().cpu().view(Hkv, G, Dh)
        eps = 2e-2
        assert bool((o >= lo[:, None, :] - eps).all()) and bool((o <= hi[:, None, :] + eps).all())



def test_c5_with_at_least_16_partitions_per_kv_head(pkg, monkeypatch):
    """The long-context configuration with its sequences cut into 1024-token partitions (16 to 33 CTAs per
    (sequence, kv head)) merged by the log-sum-exp kernel, at full size: pool bit-exact, three sequences against
    the oracle at full length, and agreement with the default plan."""
    wl = workloads
    cfg = wl.CONFIGS["c5"]
    w = wl.build_workload(cfg, "cuda:0")
    pool_before = w.pool.clone()
    out_default = _run(pkg, cfg, w)
    pool_default = w.pool.clone()
    w.pool.copy_(pool_before)
    monkeypatch.setenv("DX_ATTN_STREAMK", "0")
    monkeypatch.setenv("DX_ATTN_FORCE_CHUNK", "1024")
    plugin = wl.make_plugin(cfg, 0)
    try:
        plan = plugin.plan(cfg.batch, int(w.host_past_key_value_lengths.max()), w.host_past_key_value_lengths)
        assert plan["tokens_per_partition"] == 1024 and plan["num_partitions"] >= 16, plan
        assert int(w.host_past_key_value_lengths.min()) + 1 >= 16 * 1024
        out = wl.run_step(plugin, w)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
    finally:
        plugin.close()
    assert torch.equal(w.pool, pool_default)
    d = (out.float() - out_default.float()).abs()
    assert d.max().item() < MAX_ABS_TOL and d.mean().item() < MEAN_ABS_TOL
    idx = [0, cfg.batch // 2, cfg.batch - 1]
    ref = oracle.decode_attention_reference(
        w.qkv.cpu()[idx], w.sequence_length.cpu()[idx], w.pool.cpu(), w.offset_table[idx], num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block,
        cache_mode=CACHE_MODE[cfg.cache], kv_scale_orig_quant=w.scale_orig_quant,
        kv_scale_quant_orig=w.scale_quant_orig, append=False)
    err = (out[idx].float().cpu() - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())
