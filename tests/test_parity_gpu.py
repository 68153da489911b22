"""GPU parity tests proper: CUDA path through the C ABI vs the CPU oracle on the same seeded inputs."""
import dataclasses

import pytest
import torch

import workloads

from helpers import gpu_step_and_compare

pytestmark = pytest.mark.gpu


def _cfg(pkg, name, **kw):
    return dataclasses.replace(workloads.CONFIGS[name], **kw)


@pytest.mark.parametrize("name,batch,len_div", [
    ("c1", 4, 1),     # config 1 at full size
    ("c2", 4, 4),     # Llama-2-7B MHA INT8, shortened
    ("c3", 6, 2),     # Falcon MQA FP8 (71 q heads on one kv head)
    ("c4", 4, 8),     # Llama-2-70B GQA FP8
    ("c5", 2, 16),    # Mixtral long GQA INT8, split-K
])
def test_config_shapes(pkg, name, batch, len_div):
    cfg = workloads.scaled_config(workloads.CONFIGS[name], batch=batch, len_div=len_div)
    r = gpu_step_and_compare(pkg, cfg)
    print(name, r)


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("name", ["c4", "c5"])
def test_tp_shards(pkg, name, tp):
    wl = workloads
    cfg = wl.scaled_config(wl.shard_config(wl.CONFIGS[name], tp), batch=3, len_div=16)
    gpu_step_and_compare(pkg, cfg)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c5"])
def test_block_boundary_lengths(pkg, name):
    """Past lengths around block and tile boundaries, including an empty past (first generated token)."""
    base = workloads.CONFIGS[name]
    tpb = base.tokens_per_block
    lens = [0, 1, tpb - 1, tpb, tpb + 1, 2 * tpb - 1, 31, 32, 33, 127, 128, 129, 3 * tpb, 517]
    cfg = dataclasses.replace(base, batch=len(lens))
    gpu_step_and_compare(pkg, cfg, lengths=torch.tensor(lens, dtype=torch.int32))


@pytest.mark.parametrize("name", ["c2", "c4", "c5"])
@pytest.mark.parametrize("multi_block", [False, True])
def test_multi_block_on_off(pkg, name, multi_block):
    cfg = workloads.scaled_config(workloads.CONFIGS[name], batch=2, len_div=4)
    r = gpu_step_and_compare(pkg, cfg, multi_block_mode=multi_block)
    if not multi_block:
        assert r["plan"]["num_partitions"] == 1


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cache", ["none", "int8", "fp8"])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2), (8, 1), (32, 2), (24, 2)])
@pytest.mark.parametrize("dh", [64, 128])
def test_dtype_cache_head_matrix(pkg, dtype, cache, heads, dh):
    wl = workloads
    cfg = wl.DecodeConfig("matrix", 3, heads[0], heads[1], dh, dtype, cache, 32, 40, 300, True, 4242)
    gpu_step_and_compare(pkg, cfg, check_twice=False)


@pytest.mark.parametrize("tpb", [16, 32, 64, 128, 256])
def test_tokens_per_block(pkg, tpb):
    wl = workloads
    cfg = wl.DecodeConfig("tpb", 3, 8, 2, 128, torch.bfloat16, "fp8", tpb, 100, 700, True, 77)
    gpu_step_and_compare(pkg, cfg, check_twice=False)


def test_eight_generation_steps(pkg):
    """Step the cache 8 times like the reference op test (tests/attention/test_gpt_attention.py:665, :1016):
    every step appends one token per sequence and must keep matching the oracle."""
    import oracle
    from helpers import CACHE_MODE, MAX_ABS_TOL, MEAN_ABS_TOL
    wl = workloads
    cfg = wl.DecodeConfig("steps", 4, 16, 2, 128, torch.bfloat16, "fp8", 64, 56, 70, True, 99)
    start = wl.draw_lengths(cfg)
    # blocks are allocated for 8 more tokens than the starting past lengths
    w_cpu = wl.build_workload(cfg, "cpu", lengths=start + 8)
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    pool_ref = w_cpu.pool.clone()
    g = torch.Generator().manual_seed(5)
    past = start.clone()
    for step in range(8):
        qkv = torch.randn(cfg.batch, (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_size, generator=g).to(cfg.dtype)
        seq = (past + 1).to(torch.int32)
        out = plugin.enqueue_generation(qkv.cuda(), seq.cuda(), past, w.kv_cache_block_pointers,
                                        w.kv_orig_quant_scale, w.kv_quant_orig_scale)
        torch.cuda.synchronize()
        ref = oracle.decode_attention_reference(
            qkv, seq, pool_ref, w_cpu.offset_table, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
            head_size=cfg.head_size, tokens_per_block=cfg.tokens_per_block, cache_mode=CACHE_MODE[cfg.cache],
            kv_scale_orig_quant=w_cpu.scale_orig_quant, kv_scale_quant_orig=w_cpu.scale_quant_orig)
        assert torch.equal(w.pool.cpu(), pool_ref), f"step {step}"
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() < MAX_ABS_TOL and err.mean().item() < MEAN_ABS_TOL
        past = past + 1
    plugin.close()


@pytest.mark.parametrize("cache,heads,dh", [("fp8", (8, 2), 128), ("int8", (4, 4), 64), ("none", (8, 2), 128)])
def test_many_partitions_per_row_are_merged_by_a_cta_per_row(pkg, cache, heads, dh, monkeypatch):
    """With 32 or more partitions the merge runs one CTA per q row (four warps share the partitions): forced here
    with 128-token partitions over sequences of up to 6000 tokens, a ragged batch, against the oracle."""
    monkeypatch.setenv("DX_ATTN_FORCE_CHUNK", "128")
    wl = workloads
    cfg = wl.DecodeConfig("many", 3, heads[0], heads[1], dh, torch.bfloat16 if dh == 128 else torch.float16, cache, 64,
                          1, 6000, True, 4321)
    res = gpu_step_and_compare(pkg, cfg, lengths=torch.tensor([130, 4200, 6000], dtype=torch.int32))
    assert res["plan"]["num_partitions"] >= 32, res["plan"]
