"""Parity of the opt-in token-major tcgen05 kernel (FP8 cache, Dh 128, up to 16 q heads per kv head;
DX_ATTN_TOK=1) against the CPU oracle: pool bytes bit-exact, output within the fp32-oracle tolerance."""
import dataclasses

import pytest
import torch

import workloads

from helpers import gpu_step_and_compare

pytestmark = pytest.mark.gpu

TOK = "token_major_tcgen05"


@pytest.fixture(autouse=True)
def _enable(monkeypatch):
    monkeypatch.setenv("DX_ATTN_TOK", "1")


@pytest.mark.parametrize("case", [
    # name, batch, H, Hkv, dtype, tokens/block, past lo, past hi, split-K
    ("one_partial_tile", 2, 8, 1, torch.bfloat16, 64, 40, 63, False),
    ("two_tiles", 2, 8, 1, torch.bfloat16, 64, 130, 250, False),
    ("long_no_split", 3, 16, 2, torch.bfloat16, 64, 300, 900, False),
    ("llama70b_group_split", 3, 64, 8, torch.bfloat16, 64, 300, 2900, True),
    ("group4_block128", 2, 8, 2, torch.float16, 128, 300, 1900, True),
    ("group2_block32", 2, 4, 2, torch.bfloat16, 32, 300, 900, True),
    ("group12", 2, 24, 2, torch.bfloat16, 64, 300, 900, True),
    ("group16_block256", 2, 16, 1, torch.float16, 256, 300, 900, False),
])
def test_token_major_cases(pkg, case):
    name, batch, heads, kv_heads, dtype, tpb, lo, hi, mb = case
    cfg = workloads.DecodeConfig(name, batch, heads, kv_heads, 128, dtype, "fp8", tpb, lo, hi, mb, 7000 + heads)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"]["kernel"] == TOK
    print(name, r)


def test_token_major_boundary_lengths(pkg):
    """Past lengths around block (64), tile and partition (128) boundaries, and an empty past."""
    lens = [0, 1, 63, 64, 65, 127, 31, 32, 33, 126, 128, 129, 192, 517, 255, 256, 257, 1024]
    cfg = dataclasses.replace(workloads.CONFIGS["c4"], batch=len(lens))
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"]["kernel"] == TOK


def test_token_major_is_opt_in(pkg, monkeypatch):
    monkeypatch.delenv("DX_ATTN_TOK")
    cfg = workloads.scaled_config(workloads.CONFIGS["c4"], batch=2, len_div=8)
    r = gpu_step_and_compare(pkg, cfg, check_twice=False)
    assert r["plan"]["kernel"] == "gqa_tensor_core"
