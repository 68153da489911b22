"""world_size-2 CPU test (gloo) of the multi-GPU host logic: every rank derives its shard of the same
seeded workload without talking to the others, the only communication is the timing/work reduction
outside the step, and the per-rank results concatenate to the single-rank result."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__ as g
        import bench
        from helpers import oracle_step
        import workloads as wl
        cfg = wl.DecodeConfig("tp", 3, 16, 4, 64, torch.bfloat16, "fp8", 16, 20, 90, True, 8)
        w = wl.build_workload(cfg, "cpu")          # same seed on every rank -> same lengths and tables
        ws = wl.shard_workload(w, world, rank)     # this rank's heads only
        assert ws.cfg.num_heads == cfg.num_heads // world and ws.cfg.num_kv_heads == cfg.num_kv_heads // world
        assert torch.equal(ws.host_past_key_value_lengths, w.host_past_key_value_lengths)
        o, _ = oracle_step(ws)                     # stands in for the GPU step: no data-path collective
        # the two ranks time their calibration loops differently and must still agree on the number of repetitions
        reps = bench.agreed_repeats(dist, torch.device("cpu"), 0.020 if rank == 0 else 0.140, 20, 0)
        all_reps = [None] * world
        dist.all_gather_object(all_reps, reps)
        assert all_reps == [25] * world, all_reps  # 70 ms / (20 steps x 0.140 ms) = 25; rank 0 alone would say 175
        maxima, sums = bench.reduce_over_ranks(dist, torch.device("cpu"), [10.0 + rank, 3.0 - rank],
                                               [float(ws.kv_bytes), 1.0])
        gathered = [torch.empty_like(o) for _ in range(world)] if rank == 0 else None
        dist.gather(o, gathered, dst=0)
        if rank == 0:
            full, _ = oracle_step(w)
            B, H, Dh = cfg.batch, cfg.num_heads, cfg.head_size
            cat = torch.cat([x.view(B, H // world, Dh) for x in gathered], 1).reshape(B, H * Dh)
            q.put({"equal": bool(torch.equal(cat, full)), "maxima": maxima, "sums": sums, "kv_full": float(w.kv_bytes)})
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_by_kv_head_without_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    res = q.get(timeout=10)
    assert res["equal"]
    assert res["maxima"] == [11.0, 3.0]            # max over ranks
    assert res["sums"] == [res["kv_full"], 2.0]    # work adds up to the full job
