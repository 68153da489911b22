#!/usr/bin/env python
"""Decode-attention benchmark: one "step" = one generation-phase attention call (append the new
token, attend over the paged FP8 KV cache) for the whole batch of the Llama-2-70B-shaped GQA
config, sharded by KV head over N GPUs exactly like tensor parallelism (no collective on the
timed path; total work is fixed, so scaling is "strong").

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c4] [--impl reference]

Prints ONE JSON line (rank 0).  `value` is KV-bytes-read GB/s aggregated over all ranks with
inputs resident in HBM; `e2e` is the same metric through the host-buffer C-ABI call
(host->device copies of the step inputs and the device->host copy of the output inside the
timed region); `roofline` compares the attention kernel(s) with the measured HBM copy bandwidth;
`cpu_baseline` is the CPU oracle (a PyTorch fp32 port of the reference's algorithm) on a bounded
sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

METRIC = "decode_attn_kv_read_bandwidth"
UNIT = "GB/s"
L2_BYTES = 126 * 1024 * 1024
EVENT_EVERY = 4


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (gqa_decode_fp8_c4.md, gqa_decode_int8_c5.md, mha_int8_decode_c2.md,
# wide_decode_fp8_c3.md, gqa_decode_fp8_c4_tp8_shard.md, gqa16_decode_bf16_c4kv16.md).  Captured at full size: each fits the capture rule.
PROFILED_TRAFFIC = {
    "c4_llama2_70b_gqa_fp8_tp1": 805493504,
    "c5_mixtral_long_gqa_int8_tp1": 379214080,
    "c2_llama2_7b_mha_int8_tp1": 813841664,
    "c3_falcon_7b_mqa_fp8_tp1": 20091392,
    "c4_llama2_70b_gqa_fp8_tp8": 103479808,
    "c4kv16_llama2_70b_gqa_bf16_cache_tp1": 799406592,
}


def profiled_traffic(workload_key: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    return PROFILED_TRAFFIC.get(workload_key)


def agreed_repeats(dist, dev, est_ms_per_step: float, steps: int, requested: int) -> int:
    """Repetitions of the timed loop, the same number on every rank: the ranks meet at a barrier around every
    repetition, so a count derived from a per-rank timing would leave the faster rank waiting for ever.  The
    estimate is reduced to its maximum over the ranks first.  At least 25 repetitions and 70 ms of GPU work; not
    more: a timed region of several hundred ms of this kernel runs into the board's power cap and is measured at
    a lower SM clock."""
    t = torch.tensor([est_ms_per_step], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    est = float(t.item())
    if requested > 0:
        return requested
    return int(min(400, max(25, -(-70.0 // max(1e-6, steps * est)))))


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while running."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        if self.ok and not self.samples:  # a timed region shorter than one period: sample once, right after it
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            except Exception:
                pass
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def load_workloads():
    """The seeded synthetic workloads live beside the tests (tests/workloads.py)."""
    tests_dir = str(ROOT / "tests")
    if tests_dir not in sys.path:
        sys.path.insert(0, tests_dir)
    import workloads
    return workloads


def workload_config(full_cfg, cfg, tp, world, replicas, pool_bytes):
    """`config` of the JSON line: what is measured.  Both arms print exactly this."""
    return {"workload": full_cfg.name, "batch": full_cfg.batch, "q_heads": full_cfg.num_heads,
            "kv_heads": full_cfg.num_kv_heads, "head_size": full_cfg.head_size, "kv_cache": full_cfg.cache,
            "tokens_per_block": full_cfg.tokens_per_block, "past_len": [full_cfg.len_lo, full_cfg.len_hi],
            "parallelism": f"tp{tp} by kv head" + (" (one shard emulated on 1 GPU)" if tp != world else ""),
            "per_gpu_heads": [cfg.num_heads, cfg.num_kv_heads],
            "l2": f"KV footprint per GPU {replicas} x {pool_bytes / 1e6:.0f} MB rotated (> L2 {L2_BYTES / 1e6:.0f} MB)"}


def pool_replicas(cfg):
    """Distinct KV pools a GPU rotates over so that consecutive steps never find their KV in L2: one when the
    pool alone is larger than 3 x L2, else enough of them to get there (at most 16)."""
    blocks = 0
    wl = load_workloads()
    past = wl.draw_lengths(cfg)
    tpb = cfg.tokens_per_block
    blocks = sum((int(l) + 1 + tpb - 1) // tpb for l in past) + 3
    pool_bytes = 2 * blocks * cfg.block_bytes
    return min(16, max(1, -(-3 * L2_BYTES // max(1, pool_bytes)))), pool_bytes


def cpu_oracle_sample(cfg, sample_batch: int, repeats: int):
    """Times the CPU oracle on `sample_batch` sequences of the config.  Returns (workload, list of seconds)."""
    import oracle
    wl = load_workloads()
    scfg = wl.scaled_config(cfg, batch=sample_batch)
    w = wl.build_workload(scfg, "cpu")
    mode = {"none": oracle.CACHE_T, "int8": oracle.CACHE_INT8, "fp8": oracle.CACHE_FP8}[cfg.cache]

    def once():
        pool = w.pool  # append rewrites the same bytes every time
        t0 = time.perf_counter()
        oracle.decode_attention_reference(
            w.qkv, w.sequence_length, pool, w.offset_table, num_heads=scfg.num_heads,
            num_kv_heads=scfg.num_kv_heads, head_size=scfg.head_size, tokens_per_block=scfg.tokens_per_block,
            cache_mode=mode, kv_scale_orig_quant=w.scale_orig_quant, kv_scale_quant_orig=w.scale_quant_orig)
        return time.perf_counter() - t0

    times = [once() for _ in range(repeats)]
    return w, times


def reduce_over_ranks(dist, device, maxima, sums):
    """Whole-job aggregation: times are the max over ranks, work counters the sum over ranks."""
    stats = torch.tensor(list(maxima), dtype=torch.float64, device=device)
    tot = torch.tensor(list(sums), dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    return [float(x) for x in stats.tolist()], [float(x) for x in tot.tolist()]


def run_reference_arm(args):
    """The reference's algorithm on the host CPU cores: the oracle port (the reference has no CPU
    implementation of this path and its plugin needs TensorRT).  Rank 0 only.  A step is the decode step of a
    bounded sample of the batch's sequences (full lengths), sized so that warm-up + steps end within minutes."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    wl = load_workloads()
    full_cfg = wl.CONFIGS[args.config]
    cfg = wl.shard_config(full_cfg, world)
    torch.set_num_threads(os.cpu_count() or 1)
    # calibrate on two sequences, then size the sample: about 100 s for the whole run, at most --cpu-sample sequences
    _, cal = cpu_oracle_sample(full_cfg, 2, 2)
    per_seq = min(cal) / 2
    n_steps = args.warmup + args.steps
    sample_batch = int(max(1, min(full_cfg.batch, args.cpu_sample, 100.0 / max(1e-9, n_steps * per_seq))))
    w, times = cpu_oracle_sample(full_cfg, sample_batch, n_steps)
    timed = times[args.warmup:]
    sec = sum(timed) / len(timed)
    gbs = w.kv_bytes / sec / 1e9
    replicas, pool_bytes = pool_replicas(cfg)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3 * full_cfg.batch / sample_batch,
        "ms_per_step_measured_sample": sec * 1e3,
        "ms_per_step_note": f"ms_per_step is the measured sample time ({sample_batch} sequences) scaled to the full "
                            f"batch of {full_cfg.batch}; value is bytes of the sample / its measured time",
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE_OF[full_cfg.cache], "data": "synthetic",
        "config": workload_config(full_cfg, cfg, world, world, replicas, pool_bytes),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample_batch} of {full_cfg.batch} sequences per step, full lengths, "
                                   f"whole job (all kv heads) on the host cores"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "sequences_per_s": sample_batch / sec,
    }
    print(json.dumps(line), flush=True)


DTYPE_OF = {"fp8": "fp8_e4m3 KV, bf16 q/out, fp32 accumulate", "int8": "int8 KV, bf16 q/out, fp32 accumulate",
            "none": "f16"}


class Timed:
    """One configuration on this rank: resident inputs, pre-marshalled C calls, and the timing loops."""

    def __init__(self, wl, full_cfg, tp, rank, local_rank, dev):
        self.wl, self.full_cfg, self.tp, self.dev = wl, full_cfg, tp, dev
        self.cfg = cfg = wl.shard_config(full_cfg, tp)
        self.replicas, _ = pool_replicas(cfg)
        self.ws = [wl.build_workload(cfg, dev, seed_offset=1000 * rank + i) for i in range(self.replicas)]
        w0 = self.ws[0]
        self.plugin = wl.make_plugin(cfg, local_rank, tp_size=tp, tp_rank=rank % tp)
        max_past = int(w0.host_past_key_value_lengths.max())
        wsize = self.plugin.get_workspace_size(cfg.batch, max_past)
        self.workspace = torch.empty(max(wsize, 1), dtype=torch.uint8, device=dev) if wsize else None
        self.out = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device=dev)
        self.plan = self.plugin.plan(cfg.batch, max_past, w0.host_past_key_value_lengths)
        self.stream = torch.cuda.current_stream(dev)
        # one pre-marshalled C call per replica: the timed loop does nothing but the C-ABI call
        self.bound = [self.plugin.bind_generation(
            w.qkv, w.sequence_length, w.host_past_key_value_lengths, w.kv_cache_block_pointers,
            w.kv_orig_quant_scale, w.kv_quant_orig_scale, out=self.out, workspace=self.workspace,
            max_attention_window=w.max_blocks_per_seq * cfg.tokens_per_block) for w in self.ws]
        self.kv_bytes = float(sum(w.kv_bytes for w in self.ws)) / self.replicas
        self.flops = float(w0.flops)
        self.pool_bytes = w0.pool.numel()

    def kernel_name(self):
        split = self.plan["num_partitions"] > 1 or "stream_k_ctas" in self.plan
        return self.plan["kernel"] + ("+lse_merge" if split else "")

    def warm(self, n):
        for i in range(n):
            self.bound[i % self.replicas]()
        torch.cuda.synchronize()
        assert self.plugin.device_status() == 0

    def repetition(self, steps, barrier, events=None):
        """`steps` back-to-back steps bracketed by barrier + synchronize; returns the CUDA-event time in ms.  With
        `events`, every EVENT_EVERY-th step is also bracketed by its own pair (per-launch device time)."""
        barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(self.stream)
        for i in range(steps):
            if events is not None and i % EVENT_EVERY == 0:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(self.stream)
                self.bound[i % self.replicas]()
                b.record(self.stream)
                events.append((a, b))
            else:
                self.bound[i % self.replicas]()
        t1.record(self.stream)
        torch.cuda.synchronize()
        barrier()
        return t0.elapsed_time(t1)

    def close(self):
        self.plugin.close()


def run_own_arm(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    entry.load_package()
    wl = load_workloads()
    full_cfg = wl.CONFIGS[args.config]
    tp = world
    if world == 1 and args.emulate_tp > 1:
        tp = args.emulate_tp  # one rank's shard of a tp-way job on a single GPU (tuning aid)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(values):
        t = torch.tensor(list(values), dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    # ---- inputs resident in HBM; rotate over replicas when one shard would fit in L2 ----
    m = Timed(wl, full_cfg, tp, rank, local_rank, dev)
    cfg, plugin, plan, replicas, ws = m.cfg, m.plugin, m.plan, m.replicas, m.ws
    warmup = max(args.warmup, 3)
    m.warm(warmup)

    # ---- the timed region: `repeats` repetitions of a `steps`-long loop, each bracketed by barrier + synchronize
    # and timed with CUDA events; every repetition is reduced to the max over ranks, the line reports the median
    # repetition.  The repetitions only make the figure rest on more GPU time (and give the clock sampler
    # something to sample); `steps` and `ms_per_step` mean what they always meant. ----
    est = m.repetition(min(args.steps, 20), barrier) / min(args.steps, 20)  # untimed: sizes the repetitions
    repeats = agreed_repeats(dist, dev, est, args.steps, args.repeats)
    sampler = ClockSampler(physical_gpu_index(local_rank), period_s=0.005)
    ev = []
    l0 = plugin.launch_count()
    sampler.start()
    rep_ms_local = [m.repetition(args.steps, barrier, ev) for _ in range(repeats)]
    clocks = sampler.stop()
    launches = plugin.launch_count() - l0
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in ev)
    rep_ms = max_over_ranks(rep_ms_local)  # per repetition: the slowest rank
    per_step = sorted(x / args.steps for x in rep_ms)
    ms = statistics.median(per_step)

    # ---- end to end through the host-buffer entry point ----
    out, workspace, stream = m.out, m.workspace, m.stream
    e2e_steps = max(10, min(args.steps, 300))
    pin = lambda t: t.cpu().pin_memory()
    h_qkv = [pin(w.qkv) for w in ws]
    h_len = [pin(w.sequence_length) for w in ws]
    h_tbl = [pin(w.kv_cache_block_pointers) for w in ws]
    h_out = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(5)]

    def bind_host(sync):
        return [plugin.bind_generation(h_qkv[j % replicas], h_len[j % replicas],
                                       ws[j % replicas].host_past_key_value_lengths, h_tbl[j % replicas],
                                       ws[j % replicas].kv_orig_quant_scale, ws[j % replicas].kv_quant_orig_scale,
                                       out=h_out[j % 5], workspace=workspace, host=True, sync=sync,
                                       max_attention_window=ws[j % replicas].max_blocks_per_seq * cfg.tokens_per_block)
                for j in range(5 * replicas)]

    def time_e2e(calls, drain):
        for i in range(3):
            calls[i % len(calls)]()
        drain()
        times = []
        for _ in range(5):
            barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(e2e_steps):
                calls[i % len(calls)]()
            drain()  # the last results are in host memory; e1 is recorded behind that point
            e1.record(stream)
            torch.cuda.synchronize()
            barrier()
            times.append(e0.elapsed_time(e1) / e2e_steps)
        return times

    # Two figures through the host-buffer entry point, every step copying its inputs from pinned host memory
    # and its result back: (a) pipelined - sync=0, the copies of a step overlap the kernels of the steps
    # before it (four staging slots in the library), results waited for with host_sync(); (b) strictly synchronous.
    # Each is the median of five repetitions of an e2e_steps-long loop (max over ranks per repetition).
    e2e_ms = e2e_sync_ms = float("nan")
    if not args.no_e2e:
        e2e_ms = statistics.median(max_over_ranks(time_e2e(bind_host(False), plugin.host_sync)))
        e2e_sync_ms = statistics.median(max_over_ranks(time_e2e(bind_host(True), lambda: None)))
    h2d = h_qkv[0].numel() * 2 + h_len[0].numel() * 4 + h_tbl[0].numel() * 8
    d2h = h_out[0].numel() * 2
    torch.cuda.synchronize()

    _, (kv_bytes_total, flops_total, launches_total) = reduce_over_ranks(
        dist, dev, [0.0], [m.kv_bytes, m.flops, float(launches)])
    kv_bytes_local, pool_bytes, kernel_name = m.kv_bytes, m.pool_bytes, m.kernel_name()
    del h_qkv, h_len, h_tbl, h_out, ws
    m.close()
    del m
    torch.cuda.empty_cache()

    # ---- the other configurations of the benchmark, measured the same way (fewer repetitions): c2 and c3 on one
    # GPU, c5 on one GPU and sharded by kv head like the headline when this is a multi-GPU job ----
    peak, peak_src = measured_peak_gbs()
    others = {}
    if not args.no_configs and args.config == "c4" and tp == world:
        for name in (["c2", "c3", "c5"] if world == 1 else ["c5"]):
            oc = wl.CONFIGS[name]
            if world > 1 and oc.num_kv_heads % world != 0:
                continue
            t = Timed(wl, oc, world, rank, local_rank, dev)
            t.warm(5)
            k = 50
            reps = max_over_ranks([t.repetition(k, barrier) for _ in range(7)])
            o_ms = statistics.median(reps) / k
            _, (o_bytes,) = reduce_over_ranks(dist, dev, [0.0], [t.kv_bytes])
            others[name] = {"workload": oc.name, "parallelism": f"tp{world} by kv head", "us_per_step": o_ms * 1e3,
                            "kv_gbs": o_bytes / (o_ms * 1e-3) / 1e9, "sequences_per_s": oc.batch / (o_ms * 1e-3),
                            "frac_of_measured_hbm_peak": o_bytes / (o_ms * 1e-3) / 1e9 / (peak * world),
                            "kernel": t.kernel_name(), "plan": t.plan, "steps": k, "repeats": 7,
                            "l2": f"{t.replicas} x {t.pool_bytes / 1e6:.0f} MB rotated"}
            t.close()
            del t
            torch.cuda.empty_cache()

    if rank == 0:
        value = kv_bytes_total / (ms * 1e-3) / 1e9
        # roofline of the dominant kernel on one GPU: this rank's algorithmic bytes / its event time
        achieved = kv_bytes_local / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE_OF[cfg.cache], "data": "synthetic",
            "config": workload_config(full_cfg, cfg, tp, world, replicas, pool_bytes),
            "launch_plan": {"kernel": plan["kernel"], "split_k_partitions": plan["num_partitions"],
                            "tokens_per_partition": plan["tokens_per_partition"],
                            "stream_k_ctas": plan.get("stream_k_ctas")},
            "repeats": repeats, "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1],
            "timed_gpu_ms": sum(rep_ms),
            "us_per_step": ms * 1e3, "sequences_per_s": full_cfg.batch / (ms * 1e-3),
            "kv_bytes_per_step": kv_bytes_total, "tflops_algorithmic": flops_total / (ms * 1e-3) / 1e12,
            "hbm_frac_of_measured_peak": value / (peak * world), "hbm_frac_of_8TBps_nominal": value / (8000.0 * world),
            "e2e": None if args.no_e2e else {"value": kv_bytes_total / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "us_per_step": e2e_ms * 1e3, "steps": e2e_steps, "repeats": 5,
                    "mode": "host-buffer C-ABI call with sync=0: the copies of a step overlap the kernels of the "
                            "steps before it (four staging slots), every result read back to pinned host memory",
                    "synchronous_value": kv_bytes_total / (e2e_sync_ms * 1e-3) / 1e9,
                    "synchronous_us_per_step": e2e_sync_ms * 1e3},
            "gpu_launches": int(launches_total), "gpu_launches_per_step": launches_total / (repeats * args.steps * world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": profiled_traffic(f"{full_cfg.name}_tp{tp}"),
                         "peak_source": peak_src, "kernel": kernel_name,
                         "algorithmic_bytes_per_launch": kv_bytes_local, "avg_launch_ms": kern_ms,
                         "launches_timed": len(ev)},
            "clocks": clocks,
        }
        if others:
            line["configs"] = others
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            sb = min(full_cfg.batch, args.cpu_sample)
            wc, times = cpu_oracle_sample(full_cfg, sb, 3)
            sec = statistics.median(times)
            line["cpu_baseline"] = {"value": wc.kv_bytes / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
                                    "kind": "port", "us_per_step_full_batch": sec * 1e6 * full_cfg.batch / sb,
                                    "sample": f"{sb} of {full_cfg.batch} sequences, full lengths, median of 3"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--config", default="c4", choices=["c1", "c2", "c3", "c4", "c5", "c4kv16"])
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=32, help="sequences per CPU-oracle step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-configs", action="store_true", help="skip the table of the other configurations")
    ap.add_argument("--repeats", type=int, default=0,
                    help="repetitions of the steps-long timed loop (0: at least 25, more until ~250 ms of GPU time)")
    ap.add_argument("--emulate-tp", type=int, default=1,
                    help="with --gpus 1: run ONE rank's shard of a tp-way job (tuning aid; value is that shard's)")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", str(Path(__file__).resolve())] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_own_arm(args)


if __name__ == "__main__":
    main()
