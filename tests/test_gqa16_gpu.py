"""Parity of the grouped-head tensor-core kernel for a 16-bit (fp16 / bf16) cache against the CPU oracle:
pool bytes bit-exact, output within the fp32-oracle tolerance; and the switch back to the per-head kernel."""
import dataclasses

import pytest
import torch

import workloads

from helpers import gpu_step_and_compare

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads", [(4, 2), (8, 1), (12, 1), (16, 1), (24, 1), (64, 8)])
@pytest.mark.parametrize("dh,tpb", [(64, 16), (64, 128), (128, 32), (128, 64), (128, 256)])
def test_group_sizes_head_dims_and_block_sizes(pkg, dtype, heads, dh, tpb):
    cfg = workloads.DecodeConfig("g16", 3, heads[0], heads[1], dh, dtype, "none", tpb, 30, 700, True, 31 + heads[0])
    r = gpu_step_and_compare(pkg, cfg, check_twice=False)
    assert r["plan"]["kernel"] == "gqa_tensor_core"


@pytest.mark.parametrize("multi_block", [False, True])
def test_boundary_lengths(pkg, multi_block):
    """Past lengths around group (16 tokens), block and partition (128 tokens) boundaries, and an empty past."""
    lens = [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 517, 1023, 1024, 1025]
    cfg = dataclasses.replace(workloads.CONFIGS["c4kv16"], batch=len(lens), multi_block_mode=multi_block)
    r = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))
    assert r["plan"]["kernel"] == "gqa_tensor_core"


def test_long_split_sequences(pkg):
    cfg = workloads.scaled_config(workloads.CONFIGS["c4kv16"], batch=3, len_div=1)
    r = gpu_step_and_compare(pkg, cfg)
    assert r["plan"]["num_partitions"] > 1


def test_switch_keeps_the_per_head_kernel(pkg, monkeypatch):
    monkeypatch.setenv("DX_ATTN_GQA16", "0")
    cfg = workloads.DecodeConfig("g16off", 2, 8, 2, 128, torch.bfloat16, "none", 64, 100, 500, True, 5)
    r = gpu_step_and_compare(pkg, cfg, check_twice=False)
    assert r["plan"]["kernel"] == "mha_cuda_core"
