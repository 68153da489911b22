"""CPU tests: the oracle against the committed golden vectors and against an independent,
loop-level restatement on small cases."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import workloads

import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def qg():
    return np.load(GOLDEN / "quant_golden.npz")


def _not_nan16(bits: torch.Tensor, dtype):
    return ~torch.isnan(bits.view(dtype).float())


@pytest.mark.parametrize("name,dtype", [("fp16", torch.float16), ("bf16", torch.bfloat16),
                                        ("fp16_s1", torch.float16), ("bf16_s1", torch.bfloat16)])
def test_fp8_bytes_every_16bit_pattern(qg, name, dtype):
    """quantise-on-write, FP8: every fp16 / bf16 bit pattern against the toolkit's host conversion."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    x = bits.view(dtype)
    got = oracle.quantize_kv(x, float(qg[f"scale_{name}"]), oracle.CACHE_FP8)
    want = torch.from_numpy(qg[f"fp8_from_{name}"])
    ok = _not_nan16(bits, dtype)
    assert torch.equal(got[ok], want[ok])


def test_int8_bytes_ties_and_saturation(qg):
    x = torch.from_numpy(qg["int8_x"])
    assert torch.equal(oracle.int8_from_f32(x), torch.from_numpy(qg["int8_q"]))
    # spot values: ties go to even, both ends saturate
    t = oracle.int8_from_f32(torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 127.5, 1e9, -1e9]))
    assert t.tolist() == [0, 2, 2, 0, -2, 127, 127, -128]


def test_reference_known_answer_vectors(qg):
    """Inputs and expectations of the reference's transposeKVKernelTest (srand(42), scale 0.1)."""
    x = torch.from_numpy(qg["kat_x"])
    prod = x * torch.tensor(0.1, dtype=torch.float32)
    assert torch.equal(oracle.int8_from_f32(prod), torch.from_numpy(qg["kat_int8"]))
    assert torch.equal(oracle.fp8_from_f32(prod), torch.from_numpy(qg["kat_fp8"]))


def test_fp8_dequant_table(qg):
    b = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    got = oracle.dequantize_kv(b, oracle.CACHE_FP8, torch.float16)
    want = torch.from_numpy(qg["fp8_to_f32"])
    ok = ~torch.isnan(want)
    assert torch.equal(got[ok], want[ok])
    assert int((~ok).sum()) == 2  # 0x7f and 0xff


def test_int8_dequant_and_roundtrip():
    b = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    f = oracle.dequantize_kv(b, oracle.CACHE_INT8, torch.float16)
    assert f.tolist() == [float(i) if i < 128 else float(i - 256) for i in range(256)]
    assert torch.equal(oracle.int8_from_f32(f).view(torch.uint8), b)


def test_page_tables_match_reference_manager():
    """Pointer tables of the oracle's pool model vs the reference's Python block manager."""
    scenarios = json.loads((GOLDEN / "page_table_golden.json").read_text())
    assert len(scenarios) >= 3
    for sc in scenarios:
        tpb = sc["tokens_per_block"]
        m = oracle.PagedPoolModel(sc["blocks"], sc["block_bytes"], sc["max_blocks_per_seq"])
        for l in sc["context_lens"]:
            m.add_sequence(l, tpb)
        for i, snap in enumerate(sc["snapshots"]):
            if i > 0:
                m.step(tpb)
            assert m.lens == snap["lens"]
            assert m.offset_table().tolist() == snap["offsets"], f"snapshot {i}"


def test_local_index_layout():
    Hkv, tpb, Dh = 3, 8, 16
    blk = torch.arange(Hkv * tpb * Dh).view(Hkv, tpb, Dh)
    for tok in (0, 5, 8, 13, 64 + 7):
        for h in range(Hkv):
            for c in (0, 7, 15):
                assert oracle.kv_local_index(tok, h, Dh, c, tpb) == int(blk[h, tok % tpb, c])
    assert oracle.kv_token_block(63, 64) == 0 and oracle.kv_token_block(64, 64) == 1
    with pytest.raises(AssertionError):
        oracle.kv_token_block(5, 48)


def _loop_reference(w, cache_mode):
    """Element-by-element restatement (no vectorised gather) of the same step, for tiny cases."""
    cfg = w.cfg
    H, Hkv, Dh, tpb = cfg.num_heads, cfg.num_kv_heads, cfg.head_size, cfg.tokens_per_block
    G, esz = H // Hkv, cfg.elem_bytes
    pool = w.pool.clone()
    out = torch.zeros(cfg.batch, H * Dh, dtype=torch.float64)
    deq = 1.0 if cache_mode == oracle.CACHE_T else w.scale_quant_orig

    def elem(off_row, tok, h):
        base = int(off_row[oracle.kv_token_block(tok, tpb)])
        i0 = oracle.kv_local_index(tok, h, Dh, 0, tpb) * esz
        raw = pool[base + i0: base + i0 + Dh * esz]
        return oracle.dequantize_kv(raw, cache_mode, cfg.dtype).double() * deq

    for b in range(cfg.batch):
        total = int(w.sequence_length[b])
        pos = total - 1
        for hk in range(Hkv):
            for kv in range(2):
                src = w.qkv[b, (H + kv * Hkv + hk) * Dh:(H + kv * Hkv + hk + 1) * Dh]
                q = oracle.quantize_kv(src, w.scale_orig_quant, cache_mode)
                base = int(w.offset_table[b, kv, oracle.kv_token_block(pos, tpb)])
                i0 = oracle.kv_local_index(pos, hk, Dh, 0, tpb) * esz
                pool[base + i0: base + i0 + Dh * esz] = q
        for h in range(H):
            hk = h // G
            q = w.qkv[b, h * Dh:(h + 1) * Dh].double()
            s = torch.stack([(q * elem(w.offset_table[b, 0], t, hk)).sum() for t in range(total)]) / math.sqrt(Dh)
            p = torch.softmax(s, 0)
            o = sum(p[t] * elem(w.offset_table[b, 1], t, hk) for t in range(total))
            out[b, h * Dh:(h + 1) * Dh] = o
    return out, pool


@pytest.mark.parametrize("cache,dtype", [("none", torch.float16), ("int8", torch.bfloat16), ("fp8", torch.float16),
                                         ("fp8", torch.bfloat16)])
def test_oracle_against_loop_restatement(pkg, cache, dtype):
    wl = workloads
    cfg = wl.DecodeConfig("tiny", 3, 4, 2, 64, dtype, cache, 16, 1, 40, False, 31)
    w = wl.build_workload(cfg, "cpu")
    mode = {"none": oracle.CACHE_T, "int8": oracle.CACHE_INT8, "fp8": oracle.CACHE_FP8}[cache]
    pool = w.pool.clone()
    got = oracle.decode_attention_reference(
        w.qkv, w.sequence_length, pool, w.offset_table, num_heads=4, num_kv_heads=2, head_size=64,
        tokens_per_block=16, cache_mode=mode, kv_scale_orig_quant=w.scale_orig_quant,
        kv_scale_quant_orig=w.scale_quant_orig)
    want, pool2 = _loop_reference(w, mode)
    assert torch.equal(pool, pool2)
    assert (got.double() - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("cache", ["none", "int8", "fp8"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_workload_fill_uses_the_same_bytes_as_the_oracle(pkg, cache, dtype):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(4096, generator=g) * 3).to(dtype)
    mode = {"none": oracle.CACHE_T, "int8": oracle.CACHE_INT8, "fp8": oracle.CACHE_FP8}[cache]
    s = 448.0 / 7.3 if cache == "fp8" else 127.0 / 7.3
    assert torch.equal(workloads.quantize_for_cache(x, s, cache), oracle.quantize_kv(x, s, mode))


def test_tp_shards_concatenate_to_the_full_result(pkg):
    """Sharding by kv head needs no exchange: per-rank oracle outputs concatenate to the full output."""
    wl = workloads
    cfg = wl.DecodeConfig("tp", 3, 16, 4, 64, torch.bfloat16, "fp8", 16, 20, 90, True, 8)
    w = wl.build_workload(cfg, "cpu")
    from helpers import oracle_step
    full, pool_full = oracle_step(w)
    full = full.view(cfg.batch, cfg.num_heads, cfg.head_size)
    for tp in (2, 4):
        parts = []
        for r in range(tp):
            ws = wl.shard_workload(w, tp, r)
            o, _ = oracle_step(ws)
            parts.append(o.view(cfg.batch, cfg.num_heads // tp, cfg.head_size))
        assert torch.equal(torch.cat(parts, 1), full)


def test_kv_slot_arithmetic_matches_the_reference_header():
    """oracle.kv_slot_of_token against slots printed by the reference's own KVBlockArray::getKVTokenIdx
    (kvCacheUtils.h, compiled from the reference tree by oracle/ref_kv_slots.cu; tests/golden/make_golden.py):
    plain cyclic windows, tables with the spare block, whole sink blocks, sink tokens that end inside a block."""
    import json
    cases = json.loads((GOLDEN / "kv_slot_golden.json").read_text())
    assert len(cases) >= 8
    seen_bubble = seen_spare = False
    for c in cases:
        seen_bubble |= c["bubble_len"] > 0
        seen_spare |= bool(c["one_more_block"])
        got = [oracle.kv_slot_of_token(t, tokens_per_block=c["tokens_per_block"],
                                       max_blocks_per_seq=c["max_blocks_per_seq"],
                                       attention_window_size=c["attention_window"],
                                       sink_token_length=c["sink_tokens"]) for t in range(len(c["slots"]))]
        assert got == c["slots"], c
    assert seen_bubble and seen_spare
