"""Parity of the persistent warp-specialised tcgen05 kernel (FP8 cache, Dh 128, up to 16 q heads per kv head;
DX_ATTN_TOKWS=1) against the CPU oracle: pool bytes bit-exact, output within the fp32-oracle tolerance, on
single-level schedules (one static range per CTA) and on two-level ones (static ranges + short ranges drawn from
the device counter)."""
import dataclasses

import pytest
import torch

import workloads

from helpers import gpu_step_and_compare

pytestmark = pytest.mark.gpu

KERNEL = "token_major_tcgen05_persistent"


@pytest.fixture(autouse=True)
def _enable(monkeypatch):
    monkeypatch.setenv("DX_ATTN_TOKWS", "1")


CASES = [
    # name, batch, H, Hkv, dtype, tokens/block, past lo, past hi
    ("one_partial_tile", 2, 8, 1, torch.bfloat16, 64, 40, 63),
    ("two_tiles", 2, 8, 1, torch.bfloat16, 64, 130, 250),
    ("long_rows", 3, 16, 2, torch.bfloat16, 64, 300, 900),
    ("llama70b_group", 3, 64, 8, torch.bfloat16, 64, 300, 2900),
    ("group4_block128", 2, 8, 2, torch.float16, 128, 300, 1900),
    ("group2_block32", 2, 4, 2, torch.bfloat16, 32, 300, 900),
    ("group12", 2, 24, 2, torch.bfloat16, 64, 300, 900),
    ("group16_block256", 2, 16, 1, torch.float16, 256, 300, 900),
    ("many_rows", 40, 32, 4, torch.bfloat16, 64, 10, 700),
]


@pytest.mark.parametrize("two_level", [False, True])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_persistent_cases(pkg, case, two_level, monkeypatch):
    name, batch, heads, kv_heads, dtype, tpb, lo, hi = case
    if two_level:
        # every schedule two-level, whatever its size: half of the tiles in dynamic ranges of at least one tile
        monkeypatch.setenv("DX_ATTN_WS_MIN_U1", "1")
        monkeypatch.setenv("DX_ATTN_WS_MIN_U2", "1")
        monkeypatch.setenv("DX_ATTN_WS_TAIL_PCT", "50")
        monkeypatch.setenv("DX_ATTN_WS_TAIL_DIV", "2")
    else:
        monkeypatch.setenv("DX_ATTN_WS_TAIL_PCT", "0")
    cfg = workloads.DecodeConfig(name, batch, heads, kv_heads, 128, dtype, "fp8", tpb, lo, hi, True, 7100 + heads)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"]["kernel"] == KERNEL, r["plan"]
    print(name, r)


@pytest.mark.parametrize("two_level", [False, True])
def test_persistent_boundary_lengths(pkg, two_level, monkeypatch):
    """Past lengths around block (64) and tile (128) boundaries, and an empty past."""
    if two_level:
        monkeypatch.setenv("DX_ATTN_WS_MIN_U1", "1")
        monkeypatch.setenv("DX_ATTN_WS_MIN_U2", "1")
    lens = [0, 1, 63, 64, 65, 127, 31, 32, 33, 126, 128, 129, 192, 517, 255, 256, 257, 1024]
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=len(lens))
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"]["kernel"] == KERNEL


def test_persistent_long_ranges(pkg):
    """Ranges of many tiles per CTA with several rows each: ring stages, S / P / O buffers and tickets wrap many
    times (32 sequences x 8 kv heads x 17 to 32 tiles over 148 CTAs)."""
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=32)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"]["kernel"] == KERNEL
