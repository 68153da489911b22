"""TEST INFRASTRUCTURE ONLY - fp32 reference of one generation step over the paged KV cache.

For every sequence: (1) quantise the new token's K/V and store it at cache index
sequence_length - 1 through the block table, (2) read the whole history back from the cache
(dequantise, multiply by kv_scale_quant_orig), (3) out = softmax(q K^T / (sqrt(Dh) q_scaling)) V
per q head, q head h using kv head h // (H / Hkv).

Restates
  packed QKV split .............. cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:271-283
  softmax scale ................. gptAttentionCommon.cpp:306
  new token position ............ decoderMaskedMultiheadAttentionTemplate.h:1480-1485 (tlength = length - 1)
  head mapping .................. decoderMaskedMultiheadAttentionTemplate.h:1443-1444
  scores / softmax / PV ......... decoderMaskedMultiheadAttentionTemplate.h:1994-2036, 2246-2313, 2377-2422
  append-then-read semantics .... unfusedAttentionKernels_2_template.h:336-387 + decoderXQAImplPrecompiled.cpp:278-290
  quantised-cache attention ..... tensorrt_llm/layers/attention.py:999-1050
The reference's "+1e-6" in the softmax denominator (Template.h:2283) is below fp32 resolution for
these sums and is not reproduced.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .quant import CACHE_T, dequantize_kv, quantize_kv


def decode_attention_reference(qkv: torch.Tensor, sequence_lengths: torch.Tensor, pool: torch.Tensor,
                               offset_table: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_size: int,
                               tokens_per_block: int, cache_mode: int, q_scaling: float = 1.0,
                               kv_scale_orig_quant: float = 1.0, kv_scale_quant_orig: float = 1.0,
                               append: bool = True) -> torch.Tensor:
    """qkv: T [B, (H + 2 Hkv) Dh] on CPU.  pool: uint8 [pool_bytes] on CPU, mutated in place when
    append is True.  offset_table: int64 [B, 2, M] byte offsets from the pool base.
    Returns fp32 [B, H * Dh]."""
    B = qkv.shape[0]
    H, Hkv, Dh = num_heads, num_kv_heads, head_size
    G = H // Hkv
    esz = 2 if cache_mode == CACHE_T else 1
    blk = Hkv * tokens_per_block * Dh * esz
    row = Dh * esz
    inv_sqrt_dh = 1.0 / (math.sqrt(Dh) * q_scaling)
    deq = 1.0 if cache_mode == CACHE_T else kv_scale_quant_orig
    out = torch.empty(B, H * Dh, dtype=torch.float32)
    assert pool.dtype == torch.uint8 and pool.numel() % blk == 0
    pool_blocks = pool.view(-1, Hkv, tokens_per_block, row)  # [2*blocks, Hkv, tpb, Dh*esz]
    for b in range(B):
        total = int(sequence_lengths[b])
        pos = total - 1
        q = qkv[b, : H * Dh].view(H, Dh)
        k_new = qkv[b, H * Dh: (H + Hkv) * Dh].view(Hkv, Dh)
        v_new = qkv[b, (H + Hkv) * Dh:].view(Hkv, Dh)
        if append:
            kq = quantize_kv(k_new, kv_scale_orig_quant, cache_mode)  # [Hkv, row]
            vq = quantize_kv(v_new, kv_scale_orig_quant, cache_mode)
            bi, li = pos // tokens_per_block, pos % tokens_per_block
            ko, vo = int(offset_table[b, 0, bi]), int(offset_table[b, 1, bi])
            assert ko >= 0 and vo >= 0 and ko % blk == 0 and vo % blk == 0
            pool_blocks[ko // blk, :, li, :] = kq
            pool_blocks[vo // blk, :, li, :] = vq
        nb = (total + tokens_per_block - 1) // tokens_per_block
        koffs, voffs = offset_table[b, 0, :nb], offset_table[b, 1, :nb]
        assert bool((koffs >= 0).all()) and bool((voffs >= 0).all())
        kraw = pool_blocks[koffs // blk]  # [nb, Hkv, tpb, row]
        vraw = pool_blocks[voffs // blk]
        kraw = kraw.permute(1, 0, 2, 3).reshape(Hkv, nb * tokens_per_block, row)[:, :total]
        vraw = vraw.permute(1, 0, 2, 3).reshape(Hkv, nb * tokens_per_block, row)[:, :total]
        K = dequantize_kv(kraw, cache_mode, qkv.dtype) * deq  # [Hkv, total, Dh] fp32
        V = dequantize_kv(vraw, cache_mode, qkv.dtype) * deq
        qf = q.to(torch.float32).view(Hkv, G, Dh)
        s = torch.matmul(qf, K.transpose(1, 2)) * inv_sqrt_dh  # [Hkv, G, total]
        p = torch.softmax(s, dim=-1)
        o = torch.matmul(p, V)  # [Hkv, G, Dh]
        out[b] = o.reshape(H * Dh)
    return out


def kv_slot_of_token(t: int, *, tokens_per_block: int, max_blocks_per_seq: int, attention_window_size: int,
                     sink_token_length: int = 0) -> int:
    """KVBlockArray::getKVTokenIdx with the constants its constructor derives
    (cpp/tensorrt_llm/kernels/kvCacheUtils.h:71-90, :109-117): sink tokens keep their index; the others cycle
    behind the sink block(s), skipping the unused rest (bubble) of a partly filled sink block; a table with a
    spare block cycles over attention_window_size + tokens_per_block slots."""
    in_last = sink_token_length % tokens_per_block
    bubble = 0 if in_last == 0 else tokens_per_block - in_last
    one_more = (max_blocks_per_seq - 1) * tokens_per_block >= attention_window_size + bubble
    cyclic_len = attention_window_size + tokens_per_block - sink_token_length if one_more \
        else attention_window_size - sink_token_length
    if t < sink_token_length:
        return t
    return sink_token_length + bubble + (t - sink_token_length) % cyclic_len


def append_context_reference(k: torch.Tensor, v: torch.Tensor, sequence_lengths: torch.Tensor, pool: torch.Tensor,
                             offset_table: torch.Tensor, *, tokens_per_block: int, cache_mode: int,
                             kv_scale_orig_quant: float = 1.0, attention_window_size: Optional[int] = None,
                             sink_token_length: int = 0) -> None:
    """Context-phase KV write, restated from transpose4dBatchMajorKVCache
    (cpp/tensorrt_llm/kernels/unfusedAttentionKernels.cu:1565-1636): for every sequence b, head h and token
    t < sequence_lengths[b], the (quantised) K[b, h, t, :] goes to the block of slot s = getKVTokenIdx(t),
    offset_table[b, 0, s // tpb], at local index (h * tpb + s % tpb) * Dh (kvCacheUtils.h:144-152), V likewise
    through row 1.  Tokens below sequence_lengths[b] - attention_window_size are dropped (:1591-1600).  Tokens are
    written in ascending order, so of two tokens that share a slot the later one stays (the reference leaves that
    to thread timing).
    k, v: T [B, Hkv, seq_len, Dh] on CPU; pool: uint8, mutated in place."""
    B, Hkv, L, Dh = k.shape
    esz = 2 if cache_mode == CACHE_T else 1
    row = Dh * esz
    blk = Hkv * tokens_per_block * row
    M = offset_table.shape[-1]
    window = attention_window_size if attention_window_size is not None else M * tokens_per_block
    pool_blocks = pool.view(-1, Hkv, tokens_per_block, row)
    kq = quantize_kv(k, kv_scale_orig_quant, cache_mode)  # [B, Hkv, L, row]
    vq = quantize_kv(v, kv_scale_orig_quant, cache_mode)
    for b in range(B):
        n_all = int(sequence_lengths[b])
        n = min(n_all, L)
        for t in range(max(n_all - window, 0), n):
            s = kv_slot_of_token(t, tokens_per_block=tokens_per_block, max_blocks_per_seq=M,
                                 attention_window_size=window, sink_token_length=sink_token_length)
            ko, vo = int(offset_table[b, 0, s // tokens_per_block]), int(offset_table[b, 1, s // tokens_per_block])
            assert ko >= 0 and vo >= 0 and ko % blk == 0 and vo % blk == 0
            pool_blocks[ko // blk, :, s % tokens_per_block, :] = kq[b, :, t]
            pool_blocks[vo // blk, :, s % tokens_per_block, :] = vq[b, :, t]
