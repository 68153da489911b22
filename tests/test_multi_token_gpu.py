"""Several new tokens per sequence in one generation step (the reference's Medusa mode) through the C ABI, against
the CPU oracle: cache bytes of all new tokens bit-exact, outputs within the stated tolerance, for the draft trees
whose masks and position offsets the reference's medusa_utils.py produced (tests/golden)."""
import dataclasses
import json
from pathlib import Path

import pytest
import torch

import workloads

import oracle
from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu
GOLDEN = json.loads((Path(__file__).parent / "golden" / "medusa_mask_golden.json").read_text())


def _workload(pkg, cfg, q_len, pasts=None):
    """A single-token workload whose page tables have room for q_len new tokens, re-labelled: past lengths, lengths
    that include the new tokens, QKV of batch * q_len rows."""
    wl = workloads
    if pasts is None:
        pasts = wl.draw_lengths(cfg)
    pasts = torch.as_tensor(pasts, dtype=torch.int32)
    w = wl.build_workload(cfg, "cpu", lengths=pasts + (q_len - 1))
    g = torch.Generator().manual_seed(cfg.seed + 991)
    width = (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size
    qkv = torch.randn(cfg.batch * q_len, width, generator=g).to(cfg.dtype)
    return dataclasses.replace(w, qkv=qkv, host_past_key_value_lengths=pasts.clone())


def _oracle(w, packed, rope=None, offsets=None):
    cfg = w.cfg
    q_len = packed.shape[1]
    qkv = w.qkv
    if rope:
        qkv = oracle.apply_bias_rope(qkv, w.sequence_length, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                                     head_size=cfg.head_size, q_len=q_len, position_offsets=offsets, **rope)
    pool = w.pool.clone()
    out = oracle.multi_token_attention_reference(
        qkv, w.sequence_length, pool, w.offset_table, packed, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block,
        cache_mode=CACHE_MODE[cfg.cache], kv_scale_orig_quant=w.scale_orig_quant,
        kv_scale_quant_orig=w.scale_quant_orig)
    return out, pool


def _run(pkg, w_cpu, packed, rope=None, offsets=None, **kw):
    cfg = w_cpu.cfg
    w = workloads.to_device(w_cpu, "cuda:0")
    plugin = pkg.GPTAttentionPlugin(num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size,
                                    multi_block_mode=cfg.multi_block_mode, kv_cache_quant_mode=cfg.quant_mode,
                                    tokens_per_block=cfg.tokens_per_block, type_id=cfg.dtype, device=0, **(rope or {}))
    try:
        out = plugin.enqueue_generation(
            w.qkv, w.sequence_length, w.host_past_key_value_lengths, w.kv_cache_block_pointers,
            w.kv_orig_quant_scale, w.kv_quant_orig_scale, medusa_packed_mask=packed.cuda(),
            medusa_position_offsets=None if offsets is None else offsets.cuda(), **kw)
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
    finally:
        plugin.close()
    return out.float().cpu(), w.pool.cpu()


def _tree(name, batch):
    g = GOLDEN[name]
    packed = torch.tensor(g["packed_mask"], dtype=torch.int32).unsqueeze(0).expand(batch, -1, -1).contiguous()
    offsets = torch.tensor(g["position_offsets"], dtype=torch.int32).unsqueeze(0).expand(batch, -1).contiguous()
    return packed, offsets


@pytest.mark.parametrize("tree", sorted(GOLDEN))
@pytest.mark.parametrize("dtype,cache,heads,dh,tpb", [
    (torch.bfloat16, "fp8", (16, 2), 128, 64),
    (torch.bfloat16, "int8", (4, 4), 128, 32),
    (torch.float16, "none", (8, 2), 64, 16),
    (torch.float16, "fp8", (12, 1), 64, 128),
    (torch.bfloat16, "none", (8, 8), 128, 64),
])
def test_draft_trees_against_oracle(pkg, tree, dtype, cache, heads, dh, tpb):
    cfg = workloads.DecodeConfig("mt", 5, heads[0], heads[1], dh, dtype, cache, tpb, 0, 700, True, 301)
    packed, _ = _tree(tree, cfg.batch)
    q_len = packed.shape[1]
    pasts = workloads.draw_lengths(cfg)
    pasts[0] = 0  # a sequence with nothing but the new tokens
    pasts[1] = tpb - 1  # the new tokens straddle a block boundary
    w = _workload(pkg, cfg, q_len, pasts)
    ref, pool_ref = _oracle(w, packed)
    out, pool = _run(pkg, w, packed)
    assert torch.equal(pool, pool_ref)
    changed = int((pool != w.pool).sum())
    assert 0 < changed <= cfg.batch * q_len * 2 * cfg.num_kv_heads * dh * cfg.elem_bytes
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


def test_masks_may_differ_between_sequences(pkg):
    cfg = workloads.DecodeConfig("mtb", 4, 8, 2, 128, torch.bfloat16, "fp8", 64, 10, 300, True, 302)
    q_len = 9
    g = torch.Generator().manual_seed(5)
    dense = torch.tril(torch.rand(cfg.batch, q_len, q_len, generator=g) > 0.5) | torch.eye(q_len, dtype=torch.bool)
    dense[:, :, 0] = True
    packed = torch.stack([oracle.pack_mask(d) for d in dense])
    w = _workload(pkg, cfg, q_len)
    ref, pool_ref = _oracle(w, packed)
    out, pool = _run(pkg, w, packed)
    assert torch.equal(pool, pool_ref)
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL


@pytest.mark.parametrize("rope", [
    dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0),
    dict(position_embedding_type=1, rotary_embedding_dim=64, rotary_embedding_base=10000.0),
    dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_base=10000.0,
         rotary_embedding_scale_type=1, rotary_embedding_scale=4.0),
])
@pytest.mark.parametrize("with_offsets", [True, False])
def test_rotary_positions_follow_the_tree_depth(pkg, rope, with_offsets):
    cfg = workloads.DecodeConfig("mtr", 3, 8, 2, 128, torch.bfloat16, "fp8", 64, 10, 500, True, 303)
    packed, offsets = _tree("small", cfg.batch)
    if not with_offsets:
        offsets = None  # the default: token t at offset t (a chain of draft tokens)
    w = _workload(pkg, cfg, packed.shape[1])
    ref, pool_ref = _oracle(w, packed, rope, offsets)
    out, pool = _run(pkg, w, packed, rope, offsets)
    touched = (pool != w.pool) | (pool_ref != w.pool)
    agree = (pool[touched] == pool_ref[touched]).double().mean().item()
    assert agree > 0.99, agree  # cos / sin / pow of two math libraries: a few last-bit differences in the rotated K
    assert not bool(((pool != w.pool) & ~touched).any())
    err = (out - ref).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL


def test_what_the_mode_does_not_cover_is_refused(pkg):
    P = pkg.plugin
    cfg = workloads.DecodeConfig("mtu", 2, 8, 2, 128, torch.bfloat16, "fp8", 64, 100, 200, True, 304)
    packed, _ = _tree("chain3", cfg.batch)
    w = _workload(pkg, cfg, packed.shape[1], [150, 199])
    for kw in (dict(sink_token_length=64), dict(cyclic_attention_window_size=64)):
        with pytest.raises(P.DecodeAttnError) as e:
            _run(pkg, w, packed, **kw)
        assert e.value.status == P.DX_ERR_UNSUPPORTED
    dyn = dict(position_embedding_type=2, rotary_embedding_dim=128, rotary_embedding_scale_type=2,
               rotary_embedding_scale=2.0, rotary_embedding_max_positions=64)
    with pytest.raises(P.DecodeAttnError) as e:
        _run(pkg, w, packed, rope=dyn)
    assert e.value.status == P.DX_ERR_UNSUPPORTED
    # a table without room for the new tokens
    short = dataclasses.replace(w, offset_table=w.offset_table[:, :, :2].contiguous())
    with pytest.raises(P.DecodeAttnError) as e:
        _run(pkg, short, packed, max_attention_window=4096)
    assert e.value.status == P.DX_ERR_BAD_ARG


@pytest.mark.parametrize("tree", ["small", "wide"])
@pytest.mark.parametrize("dtype,cache,heads,dh,tpb,lo,hi", [
    (torch.bfloat16, "fp8", (16, 2), 128, 64, 3000, 6000),    # split-K partitions, 8 heads per kv head
    (torch.bfloat16, "int8", (8, 1), 128, 32, 0, 500),        # MQA: all rows on one kv head
    (torch.float16, "fp8", (24, 2), 64, 128, 0, 900),         # 12 heads per kv head: tokens straddle the 16-row slices
    (torch.float16, "int8", (4, 2), 64, 64, 0, 200),          # 2 heads per kv head
    (torch.bfloat16, "none", (16, 2), 128, 64, 3000, 6000),   # 16-bit cache (the one case the reference's XQA serves)
    (torch.float16, "none", (8, 2), 64, 16, 0, 300),
])
def test_grouped_rows_kernel_against_oracle_and_the_per_row_kernel(pkg, tree, dtype, cache, heads, dh, tpb, lo, hi,
                                                                   monkeypatch):
    """Grouped heads run on the grouped-head kernels with (token, head) rows (the default); the
    same call with DX_ATTN_FEATURE_GQA=0 runs one CTA per row.  Both against the oracle; identical pool bytes."""
    cfg = workloads.DecodeConfig("mtg", 3, heads[0], heads[1], dh, dtype, cache, tpb, lo, hi, True, 311)
    packed, _ = _tree(tree, cfg.batch)
    q_len = packed.shape[1]
    pasts = workloads.draw_lengths(cfg)
    pasts[0] = lo  # (0 where lo is 0: a sequence with nothing but the new tokens)
    w = _workload(pkg, cfg, q_len, pasts)
    ref, pool_ref = _oracle(w, packed)
    out, pool = _run(pkg, w, packed)
    assert torch.equal(pool, pool_ref)
    err = (out - ref).abs()
    assert torch.isfinite(out).all()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())
    monkeypatch.setenv("DX_ATTN_FEATURE_GQA", "0")
    out_b, pool_b = _run(pkg, w, packed)
    assert torch.equal(pool_b, pool_ref)
    err = (out - out_b).abs()
    assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL, (err.max().item(), err.mean().item())


@pytest.mark.parametrize("cache", ["fp8", "none"])
@pytest.mark.parametrize("grouped", [True, False])
def test_report_multi_token_time(pkg, grouped, cache, monkeypatch):
    """Times a 37-token draft tree on a batch of c4's shape (32 sequences) on the grouped-rows kernel and on the per-row
    kernel; recorded in feature_path.jsonl of the report directory."""
    import json
    import os
    from helpers import REPORT_DIR
    if not grouped:
        monkeypatch.setenv("DX_ATTN_FEATURE_GQA", "0")
    cfg = workloads.DecodeConfig("mtt", 32, 64, 8, 128, torch.bfloat16, cache, 64, 2048, 4096, True, 312)
    packed, _ = _tree("wide", cfg.batch)
    q_len = packed.shape[1]
    w_cpu = _workload(pkg, cfg, q_len)
    w = workloads.to_device(w_cpu, "cuda:0")
    plugin = pkg.GPTAttentionPlugin(num_heads=64, num_kv_heads=8, head_size=128, multi_block_mode=True,
                                    kv_cache_quant_mode=cfg.quant_mode, tokens_per_block=64, type_id=cfg.dtype, device=0)
    try:
        pm = packed.cuda()
        out = torch.empty(cfg.batch * q_len, 64 * 128, dtype=cfg.dtype, device="cuda:0")

        def step():
            plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                      w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale, out=out,
                                      medusa_packed_mask=pm)
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            step()
        b.record()
        torch.cuda.synchronize()
        assert plugin.device_status() == 0
        us = a.elapsed_time(b) / 10 * 1e3
        kv = float(w_cpu.sequence_length.double().sum() * 8 * 128 * 2 * cfg.elem_bytes)
        rec = {"case": f"{q_len} draft tokens x 32 sequences, 64 q / 8 kv heads, Dh 128, {cache} cache, past 2048-4096, "
                       + ("grouped rows" if grouped else "one CTA per row"), "us": us, "unique_kv_GBps": kv / us / 1e3}
        os.makedirs(REPORT_DIR, exist_ok=True)
        with open(os.path.join(REPORT_DIR, "feature_path.jsonl"), "a") as f:
            f.write(json.dumps(rec) + "\n")
        print(rec)
    finally:
        plugin.close()
