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
    "c4_llama2_70b_gqa_fp8_tp1": 805277440,
    "c5_mixtral_long_gqa_int8_tp1": 376647680,
    "c2_llama2_7b_mha_int8_tp1": 813736448,
    "c3_falcon_7b_mqa_fp8_tp1": 20090880,
    "c4_llama2_70b_gqa_fp8_tp8": 103483904,
    "c4kv16_llama2_70b_gqa_bf16_cache_tp1": 798216960,
}


def profiled_traffic(workload_key: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any."""
    return PROFILED_TRAFFIC.get(workload_key)


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


def cpu_oracle_sample(cfg, sample_batch: int, repeats: int):
    """Times the CPU oracle on `sample_batch` sequences of the config.  Returns (GB/s, seconds, bytes)."""
    import oracle
    pkg = entry.load_package()
    wl = pkg.workloads
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
    implementation of this path and its plugin needs TensorRT).  Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pkg = entry.load_package()
    wl = pkg.workloads
    cfg = wl.CONFIGS[args.config]
    torch.set_num_threads(os.cpu_count() or 1)
    sample_batch = min(cfg.batch, args.cpu_sample)
    w, times = cpu_oracle_sample(cfg, sample_batch, args.warmup + args.steps)
    timed = times[args.warmup:]
    sec = sum(timed) / len(timed)
    gbs = w.kv_bytes / sec / 1e9
    full_ms = sec * 1e3 * cfg.batch / sample_batch
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": full_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": cfg.cache if cfg.cache != "none" else "f16", "data": "synthetic",
        "config": {"workload": cfg.name, "note": "CPU oracle port of the reference algorithm; ms_per_step is the "
                   f"sample time scaled to the full batch ({cfg.batch} sequences)"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample_batch} of {cfg.batch} sequences per step, full lengths"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "sequences_per_s": sample_batch / sec,
    }
    print(json.dumps(line), flush=True)


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
    pkg = entry.load_package()
    wl = pkg.workloads
    full_cfg = wl.CONFIGS[args.config]
    tp = world
    if world == 1 and args.emulate_tp > 1:
        tp = args.emulate_tp  # one rank's shard of a tp-way job on a single GPU (tuning aid)
    cfg = wl.shard_config(full_cfg, tp)

    # ---- inputs resident in HBM; rotate over replicas when one shard would fit in L2 ----
    w0 = wl.build_workload(cfg, dev, seed_offset=1000 * rank)
    replicas = max(1, -(-3 * L2_BYTES // max(1, w0.pool.numel())))
    replicas = min(replicas, 16)
    ws = [w0] + [wl.build_workload(cfg, dev, seed_offset=1000 * rank + 1 + i) for i in range(replicas - 1)]
    plugin = wl.make_plugin(cfg, local_rank, tp_size=tp, tp_rank=rank)
    max_past = int(w0.host_past_key_value_lengths.max())
    wsize = plugin.get_workspace_size(cfg.batch, max_past)
    workspace = torch.empty(max(wsize, 1), dtype=torch.uint8, device=dev) if wsize else None
    out = torch.empty(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype, device=dev)
    plan = plugin.plan(cfg.batch, max_past, w0.host_past_key_value_lengths)
    stream = torch.cuda.current_stream(dev)

    # one pre-marshalled C call per replica: the timed loop does nothing but the C-ABI call
    bound = [plugin.bind_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                    w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                    out=out, workspace=workspace,
                                    max_attention_window=w.max_blocks_per_seq * cfg.tokens_per_block)
             for w in ws]

    def step(i):
        bound[i % replicas]()

    def barrier():
        if dist is not None:
            dist.barrier()

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    assert plugin.device_status() == 0

    sampler = ClockSampler(physical_gpu_index(local_rank))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    l0 = plugin.launch_count()
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for i in range(args.steps):
        if i % EVENT_EVERY == 0:  # per-launch device time of a sample of the steps (events cost host time)
            ev[i][0].record(stream)
            step(i)
            ev[i][1].record(stream)
        else:
            step(i)
    t_end.record(stream)
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    launches = plugin.launch_count() - l0
    ms_local = t_start.elapsed_time(t_end) / args.steps
    kern_ms = statistics.mean(a.elapsed_time(b) for i, (a, b) in enumerate(ev) if i % EVENT_EVERY == 0)

    # ---- end to end through the host-buffer entry point ----
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
        return e0.elapsed_time(e1) / e2e_steps

    # Two figures through the host-buffer entry point, every step copying its inputs from pinned host memory
    # and its result back: (a) pipelined - sync=0, the copies of a step overlap the kernels of the steps
    # before it (four staging slots in the library), results waited for with host_sync(); (b) strictly synchronous.
    e2e_ms_local = e2e_sync_ms_local = float("nan")
    if not args.no_e2e:
        e2e_ms_local = time_e2e(bind_host(False), plugin.host_sync)
        e2e_sync_ms_local = time_e2e(bind_host(True), lambda: None)
    h2d = h_qkv[0].numel() * 2 + h_len[0].numel() * 4 + h_tbl[0].numel() * 8
    d2h = h_out[0].numel() * 2
    # the device result of the e2e path equals the resident path's
    torch.cuda.synchronize()

    kv_bytes_local = float(sum(w.kv_bytes for w in ws)) / replicas
    flops_local = float(w0.flops)
    (ms, e2e_ms, _, e2e_sync_ms), (kv_bytes_total, flops_total, launches_total) = reduce_over_ranks(
        dist, dev, [ms_local, e2e_ms_local, kern_ms, e2e_sync_ms_local], [kv_bytes_local, flops_local, float(launches)])

    if rank == 0:
        peak, peak_src = measured_peak_gbs()
        value = kv_bytes_total / (ms * 1e-3) / 1e9
        # roofline of the dominant kernel on one GPU: this rank's algorithmic bytes / its event time
        achieved = kv_bytes_local / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": {"fp8": "fp8_e4m3 KV, bf16 q/out, fp32 accumulate",
                                           "int8": "int8 KV, bf16 q/out, fp32 accumulate",
                                           "none": "f16"}[cfg.cache],
            "data": "synthetic",
            "config": {"workload": full_cfg.name, "batch": full_cfg.batch, "q_heads": full_cfg.num_heads,
                       "kv_heads": full_cfg.num_kv_heads, "head_size": full_cfg.head_size,
                       "kv_cache": full_cfg.cache, "tokens_per_block": full_cfg.tokens_per_block,
                       "past_len": [full_cfg.len_lo, full_cfg.len_hi], "parallelism": f"tp{tp} by kv head" + (" (one shard emulated on 1 GPU)" if tp != world else ""),
                       "per_gpu_heads": [cfg.num_heads, cfg.num_kv_heads], "kernel": plan["kernel"],
                       "split_k_partitions": plan["num_partitions"],
                       "tokens_per_partition": plan["tokens_per_partition"],
                       "l2": f"KV footprint per GPU {replicas} x {w0.pool.numel() / 1e6:.0f} MB rotated "
                             f"(> L2 {L2_BYTES / 1e6:.0f} MB)"},
            "us_per_step": ms * 1e3, "sequences_per_s": full_cfg.batch / (ms * 1e-3),
            "kv_bytes_per_step": kv_bytes_total, "tflops_algorithmic": flops_total / (ms * 1e-3) / 1e12,
            "hbm_frac_of_measured_peak": value / (peak * world), "hbm_frac_of_8TBps_nominal": value / (8000.0 * world),
            "e2e": None if args.no_e2e else {"value": kv_bytes_total / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "us_per_step": e2e_ms * 1e3, "steps": e2e_steps,
                    "mode": "host-buffer C-ABI call with sync=0: the copies of a step overlap the kernels of the "
                            "steps before it (four staging slots), every result read back to pinned host memory",
                    "synchronous_value": kv_bytes_total / (e2e_sync_ms * 1e-3) / 1e9,
                    "synchronous_us_per_step": e2e_sync_ms * 1e3},
            "gpu_launches": int(launches_total),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": profiled_traffic(f"{full_cfg.name}_tp{tp}"),
                         "peak_source": peak_src,
                         "kernel": plan["kernel"] + ("+lse_merge" if plan["num_partitions"] > 1 else ""),
                         "algorithmic_bytes_per_launch": kv_bytes_local, "avg_launch_ms": kern_ms},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            sb = min(full_cfg.batch, args.cpu_sample)
            wc, times = cpu_oracle_sample(full_cfg, sb, 3)
            sec = statistics.median(times)
            line["cpu_baseline"] = {"value": wc.kv_bytes / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
                                    "kind": "port", "us_per_step_full_batch": sec * 1e6 * full_cfg.batch / sb,
                                    "sample": f"{sb} of {full_cfg.batch} sequences, full lengths, median of 3"}
        print(json.dumps(line), flush=True)
    plugin.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--config", default="c4", choices=["c1", "c2", "c3", "c4", "c5", "c4kv16"])
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=32, help="sequences per CPU-oracle step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--emulate-tp", type=int, default=1,
                    help="with --gpus 1: run ONE rank's shard of a tp-way job (tuning aid; value is that shard's)")
    args = ap.parse_args()

    if args.impl == "reference":
        if args.steps > 20:  # bounded: each step is seconds of CPU work
            args.steps = 20
        args.warmup = min(args.warmup, 3)
        run_reference_arm(args)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", str(Path(__file__).resolve())] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_own_arm(args)


if __name__ == "__main__":
    main()
