"""Cases of the bounds-checked build (libdecode_attn_checked.so), run in a process of their own by
test_bounds_checked_build_gpu.py with DX_DECODE_ATTN_LIB pointing at that library.  Prints one JSON object.

Every case is harmless even for a library without the checks (an index beyond a table row lands on the neighbouring
row's valid entries; the foreign pointer is a valid allocation), and nothing runs unless the loaded library says that
it has them."""
import dataclasses
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import workloads as wl  # noqa: E402
from helpers import MAX_ABS_TOL, MEAN_ABS_TOL, oracle_step  # noqa: E402


def _status(plugin):
    torch.cuda.synchronize()
    return plugin.device_status()


def _clean_step_ok(plugin, cfg, lens):
    w_cpu = wl.build_workload(cfg, "cpu", lengths=lens)
    w = wl.to_device(w_cpu, "cuda:0")
    out = wl.run_step(plugin, w)
    st = _status(plugin)
    ref, pool_ref = oracle_step(w_cpu)
    err = (out.float().cpu() - ref).abs()
    return bool(st == 0 and torch.equal(w.pool.cpu(), pool_ref) and err.max().item() < MAX_ABS_TOL
                and err.mean().item() < MEAN_ABS_TOL)


def main():
    pkg = wl._pkg
    P = pkg.plugin
    lib = pkg.load_library()
    res = {"has_checks": int(lib.dx_build_has_bounds_check())}
    if not res["has_checks"]:
        print(json.dumps(res))
        return
    shapes = {
        "gqa_fp8": wl.DecodeConfig("bc_gqa", 3, 16, 2, 128, torch.bfloat16, "fp8", 64, 1, 900, True, 41),
        "mha_int8": wl.DecodeConfig("bc_mha", 3, 4, 4, 128, torch.bfloat16, "int8", 64, 1, 900, False, 42),
        "gqa16": wl.DecodeConfig("bc_g16", 3, 8, 2, 64, torch.float16, "none", 32, 1, 900, True, 43),
        "wide_fp8": wl.DecodeConfig("bc_wide", 3, 71, 1, 64, torch.float16, "fp8", 64, 1, 900, True, 44),
        "general_dh96": wl.DecodeConfig("bc_gen", 3, 8, 2, 96, torch.float16, "fp8", 64, 1, 900, True, 45),
    }
    lens = torch.tensor([5, 300, 900], dtype=torch.int32)
    for name, cfg in shapes.items():
        r = {}
        plugin = wl.make_plugin(cfg, 0, multi_block_mode=False)
        try:
            # (1) checks compiled in do not change results
            r["clean_parity"] = _clean_step_ok(plugin, cfg, lens)
            # (2) a device length beyond the table row of sequence 0 (the host length says it fits; multi_block off,
            # so the kernels walk the whole device length): index out of the row
            w_cpu = wl.build_workload(cfg, "cpu", lengths=lens)
            w = wl.to_device(w_cpu, "cuda:0")
            cap = w.max_blocks_per_seq * cfg.tokens_per_block
            bad_len = w.sequence_length.clone()
            bad_len[0] = cap + 200
            w_bad = dataclasses.replace(w, sequence_length=bad_len)
            out = wl.run_step(plugin, w_bad)
            r["index_beyond_row"] = _status(plugin)
            r["index_beyond_row_cleared"] = _status(plugin)
            # (3) a block pointer outside the registered pool (a valid allocation of its own)
            w_cpu = wl.build_workload(cfg, "cpu", lengths=lens)
            w = wl.to_device(w_cpu, "cuda:0")
            plugin.set_pool_range(w.pool)
            out = wl.run_step(plugin, w)
            r["inside_pool"] = _status(plugin)
            foreign = torch.zeros(cfg.block_bytes + 256, dtype=torch.uint8, device="cuda:0")
            table = w.kv_cache_block_pointers.clone()
            table[2, 0, 1] = (foreign.data_ptr() + 255) // 256 * 256
            w_bad = dataclasses.replace(w, kv_cache_block_pointers=table)
            out = wl.run_step(plugin, w_bad)
            r["pointer_outside_pool"] = _status(plugin)
            r["foreign_untouched"] = bool((foreign == 0).all().item())
            plugin.set_pool_range(None)
            # (4) and afterwards everything is as before
            r["clean_parity_after"] = _clean_step_ok(plugin, cfg, lens)
        finally:
            plugin.close()
        res[name] = r
    print(json.dumps(res))


if __name__ == "__main__":
    main()
