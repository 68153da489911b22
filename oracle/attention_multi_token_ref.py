"""TEST INFRASTRUCTURE ONLY - fp32 reference of a generation step with several new tokens per sequence
(the reference's Medusa mode: draft tokens verified in one step under a tree mask).

For every sequence b with Q new tokens (sequence_lengths[b] INCLUDES them):
  (1) token t's K/V row is quantised and stored at cache index sequence_lengths[b] - Q + t,
  (2) token t attends to the cache entries before the step and to new token j where bit j of its mask row is
      set; everything is read back from the cache (append-then-read, as the reference's pre-processing kernel
      writes the cache before its attention kernel runs),
  (3) out[b * Q + t] = softmax(q K^T / (sqrt(Dh) q_scaling)) V per q head.

Restates
  row layout / cache index ....... cpp/tensorrt_llm/kernels/unfusedAttentionKernels/unfusedAttentionKernels_2_template.h:244-255
                                   (batch_beam_idx = token / seq_len, token_idx_in_seq = actual_seq_len - seq_len + seq_idx)
  cache write .................... unfusedAttentionKernels_2_template.h:330-387
  rotary position ................ unfusedAttentionKernels_2_template.h:258-262 (offset + actual_seq_len - seq_len)
  packed mask .................... tensorrt_llm/runtime/medusa_utils.py:50-82 (bit j of row t, 32 per int32 word, LSB first);
                                   shapes: cpp/tensorrt_llm/plugins/gptAttentionPlugin/gptAttentionPlugin.cpp:541-556
  launch ......................... cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderXQAImplPrecompiled.cpp:315-338

Parity status of this file: the mask packing and the position offsets are PINNED against vectors produced by
the reference's own medusa_utils.py (tests/golden/medusa_mask_golden.json); the attention under the mask is
UNPINNED - the reference computes it only in pre-compiled XQA kernel images for other GPU architectures, which
cannot run here, and its repository holds no test vectors for it.  What is restated is the contract its call
sites state.
"""
from __future__ import annotations

import math

import torch

from .quant import CACHE_T, dequantize_kv, quantize_kv


def pack_mask(dense: torch.Tensor) -> torch.Tensor:
    """dense: bool [Q, Q] (row t: the new tokens token t attends to) -> int32 [Q, ceil(Q / 32)]."""
    Q = dense.shape[0]
    words = (Q + 31) // 32
    out = torch.zeros(Q, words, dtype=torch.int64)
    for t in range(Q):
        for j in range(Q):
            if bool(dense[t, j]):
                out[t, j // 32] |= 1 << (j % 32)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)  # two's complement into int32
    return out.to(torch.int32)


def unpack_mask(packed: torch.Tensor, q_len: int) -> torch.Tensor:
    """int32 [Q, ceil(Q / 32)] -> bool [Q, Q]."""
    p = packed.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros(q_len, q_len, dtype=torch.bool)
    for t in range(q_len):
        for j in range(q_len):
            out[t, j] = bool((int(p[t, j // 32]) >> (j % 32)) & 1)
    return out


def multi_token_attention_reference(qkv: torch.Tensor, sequence_lengths: torch.Tensor, pool: torch.Tensor,
                                    offset_table: torch.Tensor, packed_mask: torch.Tensor, *, num_heads: int,
                                    num_kv_heads: int, head_size: int, tokens_per_block: int, cache_mode: int,
                                    q_scaling: float = 1.0, kv_scale_orig_quant: float = 1.0,
                                    kv_scale_quant_orig: float = 1.0) -> torch.Tensor:
    """qkv: T [B * Q, (H + 2 Hkv) Dh] on CPU; packed_mask: int32 [B, Q, ceil(Q / 32)]; pool: uint8, mutated in
    place; offset_table: int64 [B, 2, M] byte offsets from the pool base.  Returns fp32 [B * Q, H * Dh]."""
    B, Q = packed_mask.shape[0], packed_mask.shape[1]
    assert qkv.shape[0] == B * Q
    H, Hkv, Dh = num_heads, num_kv_heads, head_size
    G = H // Hkv
    esz = 2 if cache_mode == CACHE_T else 1
    row = Dh * esz
    blk = Hkv * tokens_per_block * row
    inv_sqrt_dh = 1.0 / (math.sqrt(Dh) * q_scaling)
    deq = 1.0 if cache_mode == CACHE_T else kv_scale_quant_orig
    out = torch.empty(B * Q, H * Dh, dtype=torch.float32)
    pool_blocks = pool.view(-1, Hkv, tokens_per_block, row)
    for b in range(B):
        total = int(sequence_lengths[b])
        past = total - Q
        assert past >= 0
        for t in range(Q):
            r = b * Q + t
            pos = past + t
            k_new = qkv[r, H * Dh: (H + Hkv) * Dh].view(Hkv, Dh)
            v_new = qkv[r, (H + Hkv) * Dh:].view(Hkv, Dh)
            bi, li = pos // tokens_per_block, pos % tokens_per_block
            ko, vo = int(offset_table[b, 0, bi]), int(offset_table[b, 1, bi])
            assert ko >= 0 and vo >= 0 and ko % blk == 0 and vo % blk == 0
            pool_blocks[ko // blk, :, li, :] = quantize_kv(k_new, kv_scale_orig_quant, cache_mode)
            pool_blocks[vo // blk, :, li, :] = quantize_kv(v_new, kv_scale_orig_quant, cache_mode)
        nb = (total + tokens_per_block - 1) // tokens_per_block
        koffs, voffs = offset_table[b, 0, :nb], offset_table[b, 1, :nb]
        kraw = pool_blocks[koffs // blk].permute(1, 0, 2, 3).reshape(Hkv, nb * tokens_per_block, row)[:, :total]
        vraw = pool_blocks[voffs // blk].permute(1, 0, 2, 3).reshape(Hkv, nb * tokens_per_block, row)[:, :total]
        K = dequantize_kv(kraw, cache_mode, qkv.dtype) * deq  # [Hkv, total, Dh] fp32
        V = dequantize_kv(vraw, cache_mode, qkv.dtype) * deq
        dense = unpack_mask(packed_mask[b], Q)
        for t in range(Q):
            r = b * Q + t
            allowed = torch.cat([torch.ones(past, dtype=torch.bool), dense[t]])
            qf = qkv[r, : H * Dh].view(Hkv, G, Dh).to(torch.float32)
            s = torch.matmul(qf, K.transpose(1, 2)) * inv_sqrt_dh  # [Hkv, G, total]
            s = s.masked_fill(~allowed.view(1, 1, total), float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[r] = torch.matmul(p, V).reshape(H * Dh)
    return out
