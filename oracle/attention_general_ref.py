"""TEST INFRASTRUCTURE ONLY - fp32 reference of one generation step with the remaining enqueueGeneration
features: beam search through the cache indirection table, cyclic (sliding-window) cache with sink tokens,
ALiBi.  Position shift is off (the plugin's default).

Restates, from cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h
and cpp/tensorrt_llm/kernels/kvCacheUtils.h:
  tlength = sequence_length - 1 ........................................ Template.h:1480-1482
  kv_loop_length = min(tlength, cyclic_attention_window_size) .......... Template.h:1493
  the kernel walks cache SLOTS 0 .. kv_loop_length-1 (no shift) ........ Template.h:1897-1945
  beams: slot s is read from sequence batch*beam_width + (s < context_length ? 0 : cache_indir[bb][s]);
         a wrapped cache (tlength > window) reads every slot through the table ... Template.h:1497-1498, 2063-2078
  cache_indir row of sequence bb starts at bb * max_attention_window ... Template.h:1875-1879
  ALiBi: score += slope[h] * (s - tlength); nothing for the new token .. Template.h:1797, 1890-1895, 2026
  slot of the new token = tok < sink ? tok : sink + bubble + (tok - sink) % cyclic_len ... kvCacheUtils.h:109-117
  cyclic_len, bubble, "one more block" ................................. kvCacheUtils.h:74-90
The slots are read BEFORE the new token is stored (Template.h:1744, 2207, 2469-2476): a wrapped sequence attends
to the old content of the slot that the new token then overwrites.  The new token itself is read as stored
(quantise, dequantise), like the rest of this oracle.
"""
from __future__ import annotations

import math

import torch

from .quant import CACHE_T, dequantize_kv, quantize_kv


def cyclic_geometry(max_blocks_per_seq: int, tokens_per_block: int, window: int, sink: int):
    """(bubble, one_more_block, cyclic_len) of KVBlockArray's constructor (kvCacheUtils.h:74-90)."""
    in_last = sink % tokens_per_block
    bubble = 0 if in_last == 0 else tokens_per_block - in_last
    one_more = (max_blocks_per_seq - 1) * tokens_per_block >= window + bubble
    cyclic_len = window + tokens_per_block - sink if one_more else window - sink
    return bubble, one_more, cyclic_len


def kv_token_slot(tok: int, sink: int, bubble: int, cyclic_len: int) -> int:
    """KVBlockArray::getKVTokenIdx (kvCacheUtils.h:109-117)."""
    return tok if tok < sink else sink + bubble + (tok - sink) % cyclic_len


def relative_bucket(relative_position: int, table_buckets: int, max_distance: int) -> int:
    """Bucket of a relative position, as the reference computes it on the fly
    (decoderMaskedMultiheadAttentionTemplate.h:1957-1975; float32 arithmetic)."""
    import numpy as np
    num_buckets = table_buckets // 2
    bucket = num_buckets if relative_position > 0 else 0
    rp = abs(relative_position)
    max_exact = num_buckets // 2
    if rp < max_exact:
        return bucket + rp
    f32 = np.float32
    large = max_exact + int(np.log(f32(rp) * f32(1.0) / f32(max_exact)) / np.log(f32(max_distance) / f32(max_exact))
                            * f32(num_buckets - max_exact))
    return bucket + min(large, num_buckets - 1)


def decode_attention_general_reference(qkv, sequence_lengths, pool, offset_table, *, num_heads, num_kv_heads,
                                       head_size, tokens_per_block, cache_mode, q_scaling=1.0,
                                       kv_scale_orig_quant=1.0, kv_scale_quant_orig=1.0, beam_width=1,
                                       cache_indirection=None, context_lengths=None, max_attention_window=None,
                                       cyclic_attention_window_size=None, sink_token_length=0, alibi_slopes=None,
                                       relative_attention_bias=None, max_distance=0, append=True):
    """qkv: T [B, (H + 2 Hkv) Dh] (B counts beams); pool: uint8, mutated when append; offset_table int64
    [B, 2, M] byte offsets.  cache_indirection: int32 [B, max_attention_window]; context_lengths: int32 [B];
    alibi_slopes: [H].  relative_attention_bias: T [H, stride, stride] - slot s of a sequence with `past` earlier
    tokens gets bias[h, past, s] added to its score (decoderMaskedMultiheadAttentionTemplate.h:1773-1797,
    :1981-2026) - or, with max_distance > 0, the bucket table T [H, buckets] of the implicit form
    (relative_bucket below).  Returns fp32 [B, H * Dh]."""
    B = qkv.shape[0]
    H, Hkv, Dh = num_heads, num_kv_heads, head_size
    G = H // Hkv
    M = offset_table.shape[-1]
    tpb = tokens_per_block
    esz = 2 if cache_mode == CACHE_T else 1
    row = Dh * esz
    blk = Hkv * tpb * row
    W = cyclic_attention_window_size if cyclic_attention_window_size is not None else M * tpb
    bubble, one_more, cyclic_len = cyclic_geometry(M, tpb, W, sink_token_length)
    assert bubble == 0, "a partly filled sink block needs position shift"
    inv_sqrt_dh = 1.0 / (math.sqrt(Dh) * q_scaling)
    deq = 1.0 if cache_mode == CACHE_T else kv_scale_quant_orig
    pool_blocks = pool.view(-1, Hkv, tpb, row)
    out = torch.empty(B, H * Dh, dtype=torch.float32)
    writes = []
    for bb in range(B):
        tlength = int(sequence_lengths[bb]) - 1
        kv_len = min(tlength, W)
        assert not (tlength > W and one_more), "walking slots 0..W-1 needs a table without the spare block"
        q = qkv[bb, : H * Dh].view(H, Dh)
        k_new = qkv[bb, H * Dh: (H + Hkv) * Dh].view(Hkv, Dh)
        v_new = qkv[bb, (H + Hkv) * Dh:].view(Hkv, Dh)
        kq = quantize_kv(k_new, kv_scale_orig_quant, cache_mode)  # [Hkv, row]
        vq = quantize_kv(v_new, kv_scale_orig_quant, cache_mode)
        # source sequence of every slot
        if beam_width > 1:
            base = (bb // beam_width) * beam_width
            ctx0 = 0 if tlength > W else int(context_lengths[bb])
            src = [base + (0 if s < ctx0 else int(cache_indirection[bb, s])) for s in range(kv_len)]
        else:
            src = [bb] * kv_len
        kraw = torch.empty(Hkv, kv_len + 1, row, dtype=torch.uint8)
        vraw = torch.empty(Hkv, kv_len + 1, row, dtype=torch.uint8)
        for s in range(kv_len):
            ko, vo = int(offset_table[src[s], 0, s // tpb]), int(offset_table[src[s], 1, s // tpb])
            assert ko >= 0 and vo >= 0 and ko % blk == 0 and vo % blk == 0
            kraw[:, s] = pool_blocks[ko // blk, :, s % tpb]
            vraw[:, s] = pool_blocks[vo // blk, :, s % tpb]
        kraw[:, kv_len] = kq
        vraw[:, kv_len] = vq
        K = dequantize_kv(kraw, cache_mode, qkv.dtype) * deq  # [Hkv, kv_len + 1, Dh]
        V = dequantize_kv(vraw, cache_mode, qkv.dtype) * deq
        qf = q.to(torch.float32).view(Hkv, G, Dh)
        s_ = torch.matmul(qf, K.transpose(1, 2)) * inv_sqrt_dh  # [Hkv, G, kv_len + 1]
        if alibi_slopes is not None:
            dist = torch.arange(kv_len + 1, dtype=torch.float32) - float(tlength)
            dist[kv_len] = 0.0
            s_ = s_ + alibi_slopes.to(torch.float32).view(Hkv, G, 1) * dist.view(1, 1, -1)
        if relative_attention_bias is not None:
            slots = list(range(kv_len)) + [tlength]  # the new token is looked up at its own position
            if max_distance > 0:
                idx = torch.tensor([relative_bucket(s - tlength, relative_attention_bias.shape[1], max_distance)
                                    for s in slots])
                rb = relative_attention_bias.to(torch.float32)[:, idx]  # [H, kv_len + 1]
            else:
                rb = relative_attention_bias.to(torch.float32)[:, tlength, torch.tensor(slots)]
            s_ = s_ + rb.view(Hkv, G, -1)
        p = torch.softmax(s_, dim=-1)
        out[bb] = torch.matmul(p, V).reshape(H * Dh)
        writes.append((bb, kv_token_slot(tlength, sink_token_length, bubble, cyclic_len), kq, vq))
    if append:
        # every sequence reads before any sequence writes (beams read each other's caches)
        for bb, slot, kq, vq in writes:
            ko, vo = int(offset_table[bb, 0, slot // tpb]), int(offset_table[bb, 1, slot // tpb])
            assert ko >= 0 and vo >= 0
            pool_blocks[ko // blk, :, slot % tpb] = kq
            pool_blocks[vo // blk, :, slot % tpb] = vq
    return out
