"""CPU checks of the oracle for the remaining enqueueGeneration features (beam search, cyclic window, sink
tokens, ALiBi): the cache geometry against values worked out by hand from KVBlockArray's constructor
(cpp/tensorrt_llm/kernels/kvCacheUtils.h:74-117), and the attention against a direct per-token evaluation."""
import math

import torch

import oracle
from oracle.attention_general_ref import cyclic_geometry, decode_attention_general_reference, kv_token_slot


def test_cyclic_geometry_matches_the_constructor_by_hand():
    # (max blocks, tokens per block, window, sink) -> (bubble, one more block, cyclic length)
    assert cyclic_geometry(4, 64, 256, 0) == (0, False, 256)      # (4-1)*64 = 192 < 256
    assert cyclic_geometry(5, 64, 256, 0) == (0, True, 320)       # spare block: 256 + 64 slots cycle
    assert cyclic_geometry(4, 64, 256, 64) == (0, False, 192)     # one sink block never cycles
    assert cyclic_geometry(5, 64, 256, 4) == (60, False, 252)     # 4 sink tokens leave a 60-token bubble: 256 < 256+60
    assert cyclic_geometry(6, 64, 256, 4) == (60, True, 316)


def test_token_slots_wrap_behind_the_sink():
    sink, bubble, cyc = 64, 0, 192
    assert [kv_token_slot(t, sink, bubble, cyc) for t in (0, 63, 64, 255, 256, 257, 447, 448)] == \
        [0, 63, 64, 255, 64, 65, 255, 64]
    assert kv_token_slot(300, 0, 0, 256) == 44


def _tiny(beam, tpb=4, hkv=1, g=2, dh=8, past=(5, 5), seed=0):
    gen = torch.Generator().manual_seed(seed)
    nseq = len(past)
    M = max((p + 1 + tpb - 1) // tpb for p in past)
    blocks = nseq * M
    row = dh * 2
    blk = hkv * tpb * row
    pool = torch.randn(2 * blocks * hkv * tpb * dh, generator=gen).to(torch.float16).view(torch.uint8).clone()
    offs = torch.empty(nseq, 2, M, dtype=torch.int64)
    for b in range(nseq):
        for i in range(M):
            offs[b, 0, i] = (b * M + i) * blk
            offs[b, 1, i] = (blocks + b * M + i) * blk
    qkv = torch.randn(nseq, (hkv * g + 2 * hkv) * dh, generator=gen).to(torch.float16)
    seq = torch.tensor([p + 1 for p in past], dtype=torch.int32)
    return qkv, seq, pool, offs, dict(num_heads=hkv * g, num_kv_heads=hkv, head_size=dh, tokens_per_block=tpb,
                                      cache_mode=oracle.CACHE_T)


def _direct(qkv, pool, offs, bb, h, slots_src, tlength, kw, slope=0.0):
    """softmax(q.k / sqrt(dh) + slope * (s - tlength)) v evaluated token by token."""
    H, Hkv, dh, tpb = kw["num_heads"], kw["num_kv_heads"], kw["head_size"], kw["tokens_per_block"]
    hk = h // (H // Hkv)
    cache = pool.view(torch.float16).view(-1, Hkv, tpb, dh)
    blk_elems = Hkv * tpb * dh * 2
    q = qkv[bb, h * dh:(h + 1) * dh].float()
    ks, vs, bias = [], [], []
    for s, src in slots_src:
        ks.append(cache[int(offs[src, 0, s // tpb]) // blk_elems, hk, s % tpb].float())
        vs.append(cache[int(offs[src, 1, s // tpb]) // blk_elems, hk, s % tpb].float())
        bias.append(slope * (s - tlength))
    ks.append(qkv[bb, (H + hk) * dh:(H + hk + 1) * dh].float())
    vs.append(qkv[bb, (H + Hkv + hk) * dh:(H + Hkv + hk + 1) * dh].float())
    bias.append(0.0)
    sc = torch.stack([q @ k for k in ks]) / math.sqrt(dh) + torch.tensor(bias)
    p = torch.softmax(sc, 0)
    return (p[:, None] * torch.stack(vs)).sum(0)


def test_beam_indirection_reads_the_named_beam_behind_the_context():
    qkv, seq, pool, offs, kw = _tiny(beam=2, past=(6, 6))
    indir = torch.tensor([[0, 1, 1, 0, 1, 0, 0, 0], [1, 1, 0, 0, 1, 1, 0, 0]], dtype=torch.int32)
    ctx = torch.tensor([3, 3], dtype=torch.int32)
    out = decode_attention_general_reference(qkv, seq, pool.clone(), offs, beam_width=2, cache_indirection=indir,
                                             context_lengths=ctx, max_attention_window=8, **kw)
    for bb in range(2):
        src = [(s, 0 if s < 3 else int(indir[bb, s])) for s in range(6)]
        for h in range(kw["num_heads"]):
            want = _direct(qkv, pool, offs, bb, h, src, 6, kw)
            assert torch.allclose(out[bb].view(-1, 8)[h], want, atol=1e-5)


def test_wrapped_window_attends_to_the_old_slot_then_overwrites_it():
    qkv, seq, pool, offs, kw = _tiny(beam=1, past=(7,), tpb=4)  # table of 2 blocks = 8 slots
    seq[0] = 11 + 1                                             # 11 past tokens in an 8-slot cyclic cache
    before = pool.clone()
    out = decode_attention_general_reference(qkv, seq, pool, offs, cyclic_attention_window_size=8, **kw)
    src = [(s, 0) for s in range(8)]
    want = _direct(qkv, before, offs, 0, 0, src, 11, kw)
    assert torch.allclose(out[0].view(-1, 8)[0], want, atol=1e-5)
    # the new token went to slot 11 % 8 = 3 and nothing else changed
    cache_b, cache_a = before.view(torch.float16).view(-1, 1, 4, 8), pool.view(torch.float16).view(-1, 1, 4, 8)
    changed = (cache_a != cache_b).any(-1).nonzero().tolist()
    kb, vb = int(offs[0, 0, 0]) // 64, int(offs[0, 1, 0]) // 64
    assert sorted(changed) == sorted([[kb, 0, 3], [vb, 0, 3]])
    assert torch.equal(cache_a[kb, 0, 3], qkv[0, 16:24])


def test_alibi_bias_uses_the_distance_to_the_new_token():
    qkv, seq, pool, offs, kw = _tiny(beam=1, past=(6,))
    slopes = torch.tensor([0.5, 0.25])
    out = decode_attention_general_reference(qkv, seq, pool.clone(), offs, alibi_slopes=slopes, **kw)
    for h in range(2):
        want = _direct(qkv, pool, offs, 0, h, [(s, 0) for s in range(6)], 6, kw, slope=float(slopes[h]))
        assert torch.allclose(out[0].view(-1, 8)[h], want, atol=1e-5)


def test_features_off_is_the_plain_oracle():
    qkv, seq, pool, offs, kw = _tiny(beam=1, past=(3, 9, 0), tpb=4)
    pa, pb = pool.clone(), pool.clone()
    a = decode_attention_general_reference(qkv, seq, pa, offs, **kw)
    b = oracle.decode_attention_reference(qkv, seq, pb, offs, **kw)
    assert torch.equal(pa, pb) and (a - b).abs().max().item() < 1e-5


def test_relative_bias_invariances():
    """A bias that is constant along the key axis changes nothing (softmax is shift-invariant); a zero table equals
    no table; the implicit form equals the explicit table built from the same buckets."""
    import oracle.attention_general_ref as G
    B, H, Hkv, Dh, tpb = 3, 4, 2, 64, 16
    g = torch.Generator().manual_seed(2)
    pasts = [5, 40, 77]
    blocks = sum((p + 1 + tpb - 1) // tpb for p in pasts) + 1
    offs = torch.full((B, 2, 6), -1, dtype=torch.int64)
    blk = Hkv * tpb * Dh * 2
    nxt = 0
    for b, p in enumerate(pasts):
        for i in range((p + 1 + tpb - 1) // tpb):
            offs[b, 0, i] = nxt * blk
            offs[b, 1, i] = (nxt + blocks) * blk
            nxt += 1
    pool = oracle.quantize_kv(torch.randn(2 * blocks * Hkv * tpb * Dh, generator=g).to(torch.float16), 1.0,
                              oracle.CACHE_T).reshape(-1).contiguous()
    qkv = torch.randn(B, (H + 2 * Hkv) * Dh, generator=g).to(torch.float16)
    lens = torch.tensor([p + 1 for p in pasts], dtype=torch.int32)
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_size=Dh, tokens_per_block=tpb, cache_mode=oracle.CACHE_T)
    run = lambda **x: G.decode_attention_general_reference(qkv, lens, pool.clone(), offs, **kw, **x)
    plain = run()
    S = 80
    assert torch.equal(run(relative_attention_bias=torch.zeros(H, S, S, dtype=torch.float16)), plain)
    const = torch.randn(H, S, 1, generator=g).expand(H, S, S).to(torch.float16)
    assert (run(relative_attention_bias=const) - plain).abs().max().item() < 1e-5
    table = torch.randn(H, 32, generator=g).to(torch.float16)
    explicit = torch.zeros(H, S, S, dtype=torch.float16)
    for t in range(S):
        for s in range(t + 1):
            explicit[:, t, s] = table[:, G.relative_bucket(s - t, 32, 100)]
    a = run(relative_attention_bias=table, max_distance=100)
    b = run(relative_attention_bias=explicit)
    assert (a - b).abs().max().item() < 1e-6 and (a - plain).abs().max().item() > 1e-2
    # buckets: exact below a quarter of the table, logarithmic and clamped above
    assert [G.relative_bucket(-d, 32, 128) for d in (0, 1, 7, 8, 200)] == [0, 1, 7, 8, 15]
