// Log-sum-exp merge of split-K partials: one warp per (sequence, q head) row.
//
// Each partition c of a row left an un-normalised numerator o_c[Dh] (fp32), its running maximum
// m_c (log2 units) and its denominator l_c.  The merged output is
//     out = sum_c 2^(m_c - M) o_c / sum_c 2^(m_c - M) l_c,   M = max_c m_c.
// Reference analogue: the last-arriving CTA's merge inside the MMHA kernel
//   cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h:2634-2787
// (which stores partial outputs in T and merges in T; here partials stay fp32).
#pragma once

#include "dx_common.cuh"

namespace dx
{

template <typename T, int DH>
__global__ void __launch_bounds__(128) lse_merge_kernel(const AttnArgs a)
{
    constexpr int VPL = DH / 32; // floats per lane (2 or 4)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp; // b * H + h
    if (row >= a.batch * a.num_heads)
        return;
    const int b = row / a.num_heads;
    const int total = a.seq_len[b];
    griddep_wait(); // launched with programmatic stream serialisation: the partials are complete after this
    const int n = (total + a.chunk_tokens - 1) / a.chunk_tokens; // partitions this sequence used (partition_of)

    const float2* ml = a.part_ml + (size_t) row * a.nsplit;
    float M = -INFINITY;
    for (int c = 0; c < n; ++c)
        M = fmaxf(M, ml[c].x);

    float L = 0.f;
    float o[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
        o[i] = 0.f;
    const float* po = a.part_o + (size_t) row * a.nsplit * DH + lane * VPL;
    for (int c = 0; c < n; ++c)
    {
        const float2 v = ml[c];
        const float f = fast_exp2(v.x - M);
        L = fmaf(v.y, f, L);
        if constexpr (VPL == 4)
        {
            const float4 p = *reinterpret_cast<const float4*>(po + (size_t) c * DH);
            o[0] = fmaf(p.x, f, o[0]);
            o[1] = fmaf(p.y, f, o[1]);
            o[2] = fmaf(p.z, f, o[2]);
            o[3] = fmaf(p.w, f, o[3]);
        }
        else
        {
            const float2 p = *reinterpret_cast<const float2*>(po + (size_t) c * DH);
            o[0] = fmaf(p.x, f, o[0]);
            o[1] = fmaf(p.y, f, o[1]);
        }
    }
    const float inv = 1.f / L;
    T* dst = reinterpret_cast<T*>(a.out) + (size_t) row * DH + lane * VPL;
    if constexpr (VPL == 4)
    {
        uint2 w;
        w.x = TypeOps<T>::pack2(o[0] * inv, o[1] * inv);
        w.y = TypeOps<T>::pack2(o[2] * inv, o[3] * inv);
        *reinterpret_cast<uint2*>(dst) = w;
    }
    else
    {
        *reinterpret_cast<uint32_t*>(dst) = TypeOps<T>::pack2(o[0] * inv, o[1] * inv);
    }
}

} // namespace dx
