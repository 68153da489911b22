"""The partition bound the host picks in front of every enqueue (classic split-K launches) against a plain
restatement of its cost model.  The library's search counts the lengths into 128-token buckets; the restatement
below divides every length by every candidate, so the two must agree on every length vector."""
import math

import pytest
import torch

import workloads

pytestmark = pytest.mark.gpu

SMS, WAVES, MIN_CHUNK, FIXED, SLACK_FROM = 148, 8, 256, 400.0, 2.0


def _expected_bound(lengths, rows_per_seq, resident):
    max_total = int(max(lengths)) + 1
    t_max = (max_total + 127) // 128 * 128
    slots = SMS * resident
    best, target = float("inf"), t_max
    t = min(max(128, MIN_CHUNK), t_max)
    while True:
        cnt = sum((int(l) + 1 + t - 1) // t for l in lengths) * rows_per_seq
        fill = cnt / slots
        waves = max(1.0, math.ceil(fill - (0.05 if fill > SLACK_FROM else 0.0)))
        cost = waves * FIXED + 0.5 * min(t, max_total)
        if (t == t_max or cnt <= WAVES * slots) and cost < best:
            best, target = cost, t
        if t == t_max:
            break
        step = 128 if t < 2048 else ((t // 16) + 127) // 128 * 128
        t = min(t + step, t_max)
    return target


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("shape", ["mha_int8", "wide_fp8", "gqa_small_shard"])
def test_partition_bound_matches_the_cost_model(pkg, monkeypatch, seed, shape):
    wl = workloads
    monkeypatch.setenv("DX_ATTN_STREAMK", "0")  # classic launches only: this is about the partition search
    if shape == "mha_int8":  # one CTA row per q head, 3 CTAs per SM
        cfg = wl.DecodeConfig("p", 1, 32, 32, 128, torch.bfloat16, "int8", 64, 1, 1, True, 1)
        rows_per_seq, resident = 32, 3
    elif shape == "wide_fp8":  # 71 heads on one kv head: one CTA row per sequence
        cfg = wl.DecodeConfig("p", 1, 71, 1, 64, torch.float16, "fp8", 64, 1, 1, True, 1)
        rows_per_seq, resident = 1, 3
    else:  # 8 q heads on one kv head, FP8: the grouped-head kernel, 3 CTAs per SM
        cfg = wl.DecodeConfig("p", 1, 8, 1, 128, torch.bfloat16, "fp8", 64, 1, 1, True, 1)
        rows_per_seq, resident = 1, 3
    plugin = wl.make_plugin(cfg, 0)
    try:
        g = torch.Generator().manual_seed(seed)
        batch = int(torch.randint(1, 200, (1,), generator=g))
        hi = int(torch.randint(300, 20000, (1,), generator=g))
        lens = torch.randint(0, hi, (batch,), generator=g, dtype=torch.int64).to(torch.int32)
        plan = plugin.plan(batch, int(lens.max()), lens)
        assert "stream_k_ctas" not in plan
        assert plan["tokens_per_partition"] == _expected_bound(lens.tolist(), rows_per_seq, resident), (plan, batch, hi)
    finally:
        plugin.close()
