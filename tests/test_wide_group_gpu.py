"""Parity of the tcgen05 wide-group kernel (FP8 cache, more than 16 q heads per kv head) against the CPU
oracle: same checks as every other kernel (pool bytes bit-exact, output within the fp32-oracle tolerance)."""
import dataclasses

import pytest
import torch

import workloads

from helpers import gpu_step_and_compare

pytestmark = pytest.mark.gpu

WIDE = "wide_group_tcgen05"


def _cfg(pkg, name, batch, heads, kv_heads, dh, dtype, tpb, lo, hi, multi_block, seed):
    return workloads.DecodeConfig(name, batch, heads, kv_heads, dh, dtype, "fp8", tpb, lo, hi, multi_block, seed)


@pytest.mark.parametrize("case", [
    # name, batch, H, Hkv, Dh, dtype, tokens/block, past lo, past hi, split-K
    ("one_partial_tile", 2, 32, 1, 64, torch.bfloat16, 64, 40, 63, False),
    ("two_tiles", 2, 32, 1, 64, torch.bfloat16, 64, 100, 127, False),
    ("falcon_group_no_split", 3, 71, 1, 64, torch.bfloat16, 64, 300, 900, False),
    ("falcon_group_split", 3, 71, 1, 64, torch.float16, 64, 300, 2900, True),
    ("dh128_short", 2, 32, 1, 128, torch.bfloat16, 64, 40, 63, False),
    ("dh128_two_kv_heads", 3, 40, 2, 128, torch.float16, 128, 300, 1900, True),
    ("two_128_head_slices", 2, 160, 1, 64, torch.bfloat16, 64, 300, 900, True),
    ("exactly_128_heads", 2, 128, 1, 128, torch.bfloat16, 256, 200, 700, True),
    ("seventeen_heads", 2, 34, 2, 64, torch.float16, 64, 10, 400, True),
])
def test_wide_group_cases(pkg, case):
    name, batch, heads, kv_heads, dh, dtype, tpb, lo, hi, mb = case
    r = gpu_step_and_compare(pkg, _cfg(pkg, name, batch, heads, kv_heads, dh, dtype, tpb, lo, hi, mb, 9000 + heads))
    assert r["plan"]["kernel"] == WIDE
    print(name, r)


def test_wide_group_boundary_lengths(pkg):
    """Past lengths around tile (64 tokens), block and partition (128 tokens) boundaries, and an empty past."""
    lens = [0, 1, 62, 63, 64, 65, 126, 127, 128, 129, 191, 192, 255, 256, 257, 517, 1023, 1024]
    cfg = dataclasses.replace(workloads.CONFIGS["c3"], batch=len(lens))
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"]["kernel"] == WIDE


def test_small_blocks_and_switch_fall_back(pkg, monkeypatch):
    """Blocks shorter than one 64-token tile, and DX_ATTN_WIDE=0, keep the 16-head-slice kernel."""
    r = gpu_step_and_compare(pkg, _cfg(pkg, "tpb32", 2, 71, 1, 64, torch.bfloat16, 32, 100, 500, True, 1), check_twice=False)
    assert r["plan"]["kernel"] == "gqa_tensor_core"
    monkeypatch.setenv("DX_ATTN_WIDE", "0")
    r = gpu_step_and_compare(pkg, _cfg(pkg, "off", 2, 71, 1, 64, torch.bfloat16, 64, 100, 500, True, 2), check_twice=False)
    assert r["plan"]["kernel"] == "gqa_tensor_core"
