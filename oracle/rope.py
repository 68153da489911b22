"""TEST INFRASTRUCTURE ONLY - QKV bias and rotary position embedding of the decode step, restated.

Follows the reference MMHA kernel:
  bias add in T ................. decoderMaskedMultiheadAttentionTemplate.h:1587-1605 (q, k), :2514 (v)
  GPT-J RoPE (pairs 2p, 2p+1) ... Template.h:1637-1650, Utils.h:2581-2594, 2622-2645
  GPT-NeoX RoPE (p, p+rot/2) .... Template.h:1651-1710 (transpose through shared memory, then the same maths)
  base / scale adjustment ....... Utils.h:2530-2579 (linear: 1/scale; dynamic: base * b^(d/(d-2)), scale 1);
                                  the GPT-J branch uses params.rotary_embedding_base / _scale unadjusted (:1641)
  position ...................... cache index of the new token, sequence_length - 1 (Template.h:1500)
cos / sin / pow are evaluated in fp32 here and by the CUDA math library on the device: the two can differ in
the last bit, so comparisons of the rotated values allow a (stated) small fraction of one-ulp mismatches.
"""
from __future__ import annotations

from typing import Optional

import torch

POS_LEARNED_ABSOLUTE, POS_ROPE_GPTJ, POS_ROPE_GPT_NEOX = 0, 1, 2
ROT_SCALE_NONE, ROT_SCALE_LINEAR, ROT_SCALE_DYNAMIC = 0, 1, 2


def apply_bias_rope(qkv: torch.Tensor, sequence_lengths: torch.Tensor, *, num_heads: int, num_kv_heads: int,
                    head_size: int, position_embedding_type: int = 0, rotary_embedding_dim: int = 0,
                    rotary_embedding_base: float = 10000.0, rotary_embedding_scale_type: int = 0,
                    rotary_embedding_scale: float = 1.0, rotary_embedding_max_positions: int = 1024,
                    qkv_bias: Optional[torch.Tensor] = None, q_len: int = 1,
                    position_offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv: T [B, (H + 2 Hkv) Dh] -> same shape, pre-processed as the decode kernels see it.
    q_len > 1 (several new tokens per sequence, rows b * q_len + t; sequence_lengths has one entry per sequence
    and includes the new tokens): row r is rotated at position_offsets.flatten()[r] + length - q_len
    (unfusedAttentionKernels_2_template.h:258-262)."""
    B = qkv.shape[0]
    H, Hkv, Dh = num_heads, num_kv_heads, head_size
    T = qkv.dtype
    x = qkv.clone().view(B, H + 2 * Hkv, Dh)
    if qkv_bias is not None:
        x = (x + qkv_bias.view(1, H + 2 * Hkv, Dh).to(T)).to(T)  # one rounding to T
    if position_embedding_type == POS_LEARNED_ABSOLUTE:
        return x.view(B, -1)
    rot = rotary_embedding_dim
    f32 = torch.float32
    for b in range(B):
        t_step = int(sequence_lengths[b // q_len]) - 1
        if q_len > 1:
            assert rotary_embedding_scale_type != ROT_SCALE_DYNAMIC
            off = int(position_offsets.flatten()[b]) if position_offsets is not None else b % q_len
            t_step = t_step + 1 - q_len + off
        base = torch.tensor(rotary_embedding_base, dtype=f32)
        scale = torch.tensor(rotary_embedding_scale, dtype=f32)
        if position_embedding_type == POS_ROPE_GPT_NEOX:
            if rotary_embedding_scale_type == ROT_SCALE_DYNAMIC:
                if t_step > rotary_embedding_max_positions:
                    bb = (scale * t_step / rotary_embedding_max_positions) - (scale - 1)
                    pp = torch.tensor(rot / (rot - 2), dtype=f32)
                    base = base * torch.pow(bb, pp)
                scale = torch.tensor(1.0, dtype=f32)
            elif rotary_embedding_scale_type == ROT_SCALE_LINEAR:
                scale = torch.tensor(1.0, dtype=f32) / scale
        p = torch.arange(rot // 2)
        zid = (2 * p).to(f32)
        inv_freq = (torch.tensor(float(t_step), dtype=f32) * scale) / torch.pow(base, zid / torch.tensor(float(rot), dtype=f32))
        c, s = torch.cos(inv_freq), torch.sin(inv_freq)
        if position_embedding_type == POS_ROPE_GPTJ:
            i0, i1 = 2 * p, 2 * p + 1
        else:
            i0, i1 = p, p + rot // 2
        qk = x[b, : H + Hkv]  # q and k heads only
        v0, v1 = qk[:, i0].to(f32), qk[:, i1].to(f32)
        r0 = c * v0 - s * v1
        r1 = c * v1 + s * v0
        qk[:, i0] = r0.to(T)
        qk[:, i1] = r1.to(T)
    return x.view(B, -1)
