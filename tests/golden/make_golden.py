"""Generates the committed golden fixtures of the oracle tests.  Run in a container that has the
reference tree (DX_REFERENCE_DIR) and the built checker (make -C oracle quant_check):

    python tests/golden/make_golden.py

Outputs (small, committed):
  page_table_golden.json  - pointer tables produced by the reference's own Python block manager
                            (tensorrt_llm/runtime/kv_cache_manager.py, imported by file path) for a
                            few allocate/step scenarios, as byte offsets from the pool base.
  quant_golden.npz        - quantise-on-write bytes from the CUDA toolkit's host conversions
                            (cuda_fp8.h, the header the reference kernels use) for EVERY fp16 and
                            bf16 bit pattern, int8 vectors including ties and saturation, and the
                            reference known-answer test's inputs (srand(42), scale 0.1;
                            cpp/tests/runtime/transposeKVKernelTest.cpp:152, :213-225) with the
                            expectations of its castTo<> functions (:76-88).
  medusa_mask_golden.json - for a few draft trees: the dense attention mask, the packed mask and the position
                            offsets that the reference's tensorrt_llm/runtime/medusa_utils.py builds (loaded by
                            file path; only its CPU functions are called).
"""
import ctypes
import importlib.util
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if not os.environ.get("DX_REFERENCE_DIR"):
    raise SystemExit("set DX_REFERENCE_DIR to the root of a TensorRT-LLM source tree")
REF = Path(os.environ["DX_REFERENCE_DIR"])


def load_ref_manager():
    path = REF / "tensorrt_llm" / "runtime" / "kv_cache_manager.py"
    spec = importlib.util.spec_from_file_location("ref_kv_cache_manager", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def page_tables():
    m = load_ref_manager()
    scenarios = []
    for (blocks, tpb, max_blocks, ctx_lens, steps, elts) in [
        (16, 8, 6, [5, 8, 17], 10, 64),
        (40, 64, 4, [1, 63, 64, 65, 130], 3, 128),
        (12, 16, 5, [30, 31], 20, 32),
    ]:
        pool = torch.zeros(2 * blocks * elts, dtype=torch.int8)
        mgr = m.KVCacheManager([pool], blocks, tpb, max_blocks, max_attention_window_size=max_blocks * tpb,
                               sink_token_len=0)
        for i, l in enumerate(ctx_lens):
            mgr.add_sequence(m.GenerationSequence(seq_idx=i, batch_idx=i), l)
        base = pool.data_ptr()
        snaps = []

        def snap():
            arr = mgr.get_block_pointers(1)  # [pools, B, beam, 2, M]
            a = arr[0, :, 0]
            off = torch.where(a != 0, a - base, torch.full_like(a, -1))
            return off.tolist()

        snaps.append({"lens": list(mgr.lens), "offsets": snap()})
        for _ in range(steps):
            mgr.step([False] * len(ctx_lens))
            snaps.append({"lens": list(mgr.lens), "offsets": snap()})
        scenarios.append({"blocks": blocks, "tokens_per_block": tpb, "max_blocks_per_seq": max_blocks,
                          "context_lens": ctx_lens, "block_bytes": elts, "snapshots": snaps})
    (HERE / "page_table_golden.json").write_text(json.dumps(scenarios))


def quant_vectors():
    lib = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libquant_check.so"))
    u16 = np.arange(65536, dtype=np.uint16)
    out = {}
    for name, fn, scale in [("fp16", lib.qc_fp8_from_fp16, 42.5390625), ("bf16", lib.qc_fp8_from_bf16, 42.5390625),
                            ("fp16_s1", lib.qc_fp8_from_fp16, 1.0), ("bf16_s1", lib.qc_fp8_from_bf16, 1.0)]:
        res = np.zeros(65536, dtype=np.uint8)
        fn(u16.ctypes.data_as(ctypes.c_void_p), 65536, ctypes.c_float(scale), res.ctypes.data_as(ctypes.c_void_p))
        out[f"fp8_from_{name}"] = res
        out[f"scale_{name}"] = np.float32(scale)
    # int8: dense grid with exact .5 ties, saturation on both sides, and a typical scale
    x = np.concatenate([np.arange(-140, 140, 0.25, dtype=np.float32), np.float32([1e6, -1e6, 127.5, -128.5, 0.0])])
    r = np.zeros(x.size, dtype=np.int8)
    lib.qc_int8_from_f32(x.ctypes.data_as(ctypes.c_void_p), x.size, ctypes.c_float(1.0), r.ctypes.data_as(ctypes.c_void_p))
    out["int8_x"], out["int8_q"] = x, r
    # the reference known-answer test's inputs: srand(42); 10 * rand() / RAND_MAX ; scale 0.1
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    n = 4096
    rmax = 2147483647
    kat = np.array([np.float32(10.0) * np.float32(libc.rand()) / np.float32(rmax) for _ in range(n)], dtype=np.float32)
    k8 = np.zeros(n, dtype=np.int8)
    kf = np.zeros(n, dtype=np.uint8)
    lib.qc_kat_int8(kat.ctypes.data_as(ctypes.c_void_p), n, ctypes.c_float(0.1), k8.ctypes.data_as(ctypes.c_void_p))
    lib.qc_kat_fp8(kat.ctypes.data_as(ctypes.c_void_p), n, ctypes.c_float(0.1), kf.ctypes.data_as(ctypes.c_void_p))
    out["kat_x"], out["kat_int8"], out["kat_fp8"] = kat, k8, kf
    # e4m3 byte -> float table
    b = np.arange(256, dtype=np.uint8)
    f = np.zeros(256, dtype=np.float32)
    lib.qc_fp8_to_f32(b.ctypes.data_as(ctypes.c_void_p), 256, f.ctypes.data_as(ctypes.c_void_p))
    out["fp8_to_f32"] = f
    np.savez_compressed(HERE / "quant_golden.npz", **out)


def medusa_masks():
    import types
    # the module's only package import is the reference logger: a stand-in keeps the import self-contained
    pkg = types.ModuleType("tensorrt_llm")
    log = types.ModuleType("tensorrt_llm.logger")
    log.logger = types.SimpleNamespace(warning=lambda *a, **k: None, info=lambda *a, **k: None)
    pkg.logger = log
    sys.modules.setdefault("tensorrt_llm", pkg)
    sys.modules.setdefault("tensorrt_llm.logger", log)
    path = REF / "tensorrt_llm" / "runtime" / "medusa_utils.py"
    spec = importlib.util.spec_from_file_location("ref_medusa_utils", path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    import copy
    trees = {
        "chain3": [[0], [0, 0], [0, 0, 0]],
        "small": [[0], [1], [0, 0], [0, 1], [1, 0], [0, 0, 0]],
        "wide": [[i] for i in range(6)] + [[i, j] for i in range(4) for j in range(3)]
                + [[i, j, 0] for i in range(3) for j in range(2)] + [[0, 0, 0, k] for k in range(12)],
    }
    out = {}
    for name, choices in trees.items():
        sorted_choices = sorted(copy.deepcopy(choices), key=m.path_sorting_key)
        heads = max(len(c) for c in sorted_choices)
        paths, level_counts, _, _ = m.choices_2_paths(heads, sorted_choices)
        paths = sorted(paths, key=m.path_sorting_key)
        topks = m.get_medusa_topks(heads, paths)
        tree_ids, pos_off, tree_paths = m.get_medusa_tree(heads, topks, level_counts, paths)
        n = len(tree_ids)
        mpaths = torch.stack([torch.tensor([-1] + p + ([-2] * (heads - len(p)))) for p in tree_paths]) + 1
        ids = torch.tensor([-1] + list(tree_ids)) + 1
        offsets = torch.tensor([-1] + list(pos_off)) + 1
        dense = m.get_medusa_mask(ids, mpaths)           # [n + 1, n + 1], row t: tokens token t attends to
        packed = m.get_packed_mask(n, dense[1:, 1:])     # int32 [n + 1, ceil((n + 1) / 32)]
        out[name] = {"choices": choices, "num_medusa_tokens": n, "dense_mask": dense.to(torch.int32).tolist(),
                     "packed_mask": packed.tolist(), "position_offsets": offsets.tolist()}
    (HERE / "medusa_mask_golden.json").write_text(json.dumps(out))


def kv_slots():
    """Slot of every token under the reference's KVBlockArray (kvCacheUtils.h:71-117), from the reference header
    itself compiled as a host program (make -C oracle kv_slots REF=...)."""
    import subprocess
    exe = ROOT / "oracle" / "_ref" / "ref_kv_slots"
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "kv_slots", f"REF={REF}"], check=True, stdout=subprocess.DEVNULL)
    cases = [  # tokens_per_block, max_blocks_per_seq, attention_window, sink_tokens, tokens listed
        (64, 8, 512, 0, 1400),     # plain cyclic window, table exactly as long as the window
        (64, 9, 512, 0, 1400),     # spare block: window + tokens_per_block slots cycle
        (64, 8, 448, 64, 1200),    # whole sink block, no spare block... (8 - 1) * 64 >= 448: spare block
        (64, 7, 448, 64, 1200),    # whole sink block, no spare block
        (64, 8, 300, 4, 900),      # sink tokens end inside a block: bubble of 60
        (16, 8, 100, 5, 400),      # bubble of 11, spare block or not by the constructor's rule
        (128, 4, 384, 0, 1000),
        (32, 40, 1024, 32, 3000),
    ]
    out = []
    for c in cases:
        res = subprocess.run([str(exe)] + [str(x) for x in c], check=True, capture_output=True, text=True)
        out.append(json.loads(res.stdout))
    (HERE / "kv_slot_golden.json").write_text(json.dumps(out))


if __name__ == "__main__":
    page_tables()
    quant_vectors()
    medusa_masks()
    kv_slots()
    print("written:", [p.name for p in HERE.iterdir()])
