"""The oracle of the step with several new tokens per sequence (the reference's Medusa mode), on the CPU:
its mask format against vectors from the reference's own medusa_utils.py, and its attention against the
single-token oracle, which is pinned against the reference kernel."""
import json
from pathlib import Path

import pytest
import torch

import oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "medusa_mask_golden.json").read_text())


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_mask_packing_matches_the_reference_vectors(name):
    g = GOLDEN[name]
    q_len = g["num_medusa_tokens"] + 1
    dense = torch.tensor(g["dense_mask"], dtype=torch.bool)
    packed = torch.tensor(g["packed_mask"], dtype=torch.int32)
    assert dense.shape == (q_len, q_len) and packed.shape == (q_len, (q_len + 31) // 32)
    assert torch.equal(oracle.unpack_mask(packed, q_len), dense)
    assert torch.equal(oracle.pack_mask(dense), packed)
    # a draft token sees the token of the original head, itself and its ancestors only: one per tree depth
    off = torch.tensor(g["position_offsets"])
    assert torch.equal(dense.sum(dim=1), off + 1)
    assert bool(torch.equal(torch.diagonal(dense), torch.ones(q_len, dtype=torch.bool)))
    assert not bool(torch.triu(dense, diagonal=1).any())


def _case(cache, dtype, B, H, Hkv, Dh, tpb, pasts, q_len, seed):
    """Pool with random past, page table with room for the new tokens, QKV of B * q_len rows."""
    g = torch.Generator().manual_seed(seed)
    mode = {"none": oracle.CACHE_T, "int8": oracle.CACHE_INT8, "fp8": oracle.CACHE_FP8}[cache]
    esz = 2 if cache == "none" else 1
    blk = Hkv * tpb * Dh * esz
    need = [(p + q_len + tpb - 1) // tpb for p in pasts]
    blocks = sum(need) + 2
    order = torch.randperm(blocks, generator=g).tolist()
    offs = torch.full((B, 2, max(need)), -1, dtype=torch.int64)
    it = iter(order)
    for b in range(B):
        for i in range(need[b]):
            idx = next(it)
            offs[b, 0, i] = idx * blk
            offs[b, 1, i] = (idx + blocks) * blk
    x = torch.randn(2 * blocks * Hkv * tpb * Dh, generator=g).to(dtype)
    s_qo = {"none": 1.0, "int8": float(x.abs().max()) / 127.0, "fp8": float(x.abs().max()) / 448.0}[cache]
    s_oq = 1.0 / s_qo
    pool = oracle.quantize_kv(x, s_oq, mode).reshape(-1).contiguous()
    qkv = torch.randn(B * q_len, (H + 2 * Hkv) * Dh, generator=g).to(dtype)
    lens = torch.tensor([p + q_len for p in pasts], dtype=torch.int32)
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_size=Dh, tokens_per_block=tpb, cache_mode=mode,
              kv_scale_orig_quant=s_oq, kv_scale_quant_orig=s_qo)
    return qkv, lens, pool, offs, kw


@pytest.mark.parametrize("cache,dtype", [("none", torch.float16), ("int8", torch.bfloat16), ("fp8", torch.bfloat16)])
def test_chain_mask_equals_single_token_steps(cache, dtype):
    """Under a causal (chain) mask, Q tokens in one step are Q single-token steps."""
    B, H, Hkv, Dh, tpb, q_len = 3, 4, 2, 64, 16, 5
    pasts = [0, 17, 44]
    qkv, lens, pool, offs, kw = _case(cache, dtype, B, H, Hkv, Dh, tpb, pasts, q_len, 11)
    chain = oracle.pack_mask(torch.tril(torch.ones(q_len, q_len, dtype=torch.bool)))
    pool_m = pool.clone()
    out = oracle.multi_token_attention_reference(qkv, lens, pool_m, offs, chain.unsqueeze(0).expand(B, -1, -1), **kw)
    pool_s = pool.clone()
    for t in range(q_len):
        step_lens = torch.tensor([p + t + 1 for p in pasts], dtype=torch.int32)
        o = oracle.decode_attention_reference(qkv.view(B, q_len, -1)[:, t].contiguous(), step_lens, pool_s, offs, **kw)
        assert torch.allclose(out.view(B, q_len, -1)[:, t], o, atol=1e-5, rtol=1e-5)
    assert torch.equal(pool_m, pool_s)


@pytest.mark.parametrize("name", ["small", "wide"])
def test_tree_mask_equals_single_token_step_over_the_visible_tokens(name):
    """Token t under a tree mask = one single-token step over a cache that holds the past and the new tokens t may
    see (its ancestors), in order."""
    g = GOLDEN[name]
    q_len = g["num_medusa_tokens"] + 1
    dense = torch.tensor(g["dense_mask"], dtype=torch.bool)
    packed = torch.tensor(g["packed_mask"], dtype=torch.int32)
    B, H, Hkv, Dh, tpb = 2, 4, 2, 64, 16
    pasts = [5, 23]
    qkv, lens, pool, offs, kw = _case("fp8", torch.bfloat16, B, H, Hkv, Dh, tpb, pasts, q_len, 12)
    out = oracle.multi_token_attention_reference(qkv, lens, pool.clone(), offs, packed.unsqueeze(0).expand(B, -1, -1), **kw)
    rows = qkv.view(B, q_len, -1)
    for t in (0, 1, q_len // 2, q_len - 1):
        visible = [j for j in range(q_len) if bool(dense[t, j])]
        assert visible[-1] == t
        pool_s = pool.clone()
        for i, j in enumerate(visible):  # append the visible tokens one by one; the last step is token t itself
            step_lens = torch.tensor([p + i + 1 for p in pasts], dtype=torch.int32)
            o = oracle.decode_attention_reference(rows[:, j].contiguous(), step_lens, pool_s, offs, **kw)
        assert torch.allclose(out.view(B, q_len, -1)[:, t], o, atol=1e-5, rtol=1e-5)


def test_rope_positions_follow_the_offsets():
    B, q_len, H, Hkv, Dh = 2, 4, 2, 1, 64
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B * q_len, (H + 2 * Hkv) * Dh, generator=g).to(torch.float16)
    lens = torch.tensor([10, 33], dtype=torch.int32)
    off = torch.tensor([[0, 1, 1, 2], [0, 1, 2, 2]], dtype=torch.int32)
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_size=Dh, position_embedding_type=2, rotary_embedding_dim=Dh)
    got = oracle.apply_bias_rope(qkv, lens, q_len=q_len, position_offsets=off, **kw)
    for b in range(B):
        for t in range(q_len):
            r = b * q_len + t
            pos = int(lens[b]) - q_len + int(off[b, t])
            one = oracle.apply_bias_rope(qkv[r:r + 1], torch.tensor([pos + 1], dtype=torch.int32), **kw)
            assert torch.equal(got[r:r + 1], one)
