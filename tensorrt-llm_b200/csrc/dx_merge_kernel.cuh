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

// VPL (2, 4 or 8) consecutive floats of a partial row.
template <int VPL>
__device__ __forceinline__ void load_partial(const float* p, float (&v)[VPL])
{
    if constexpr (VPL == 2)
    {
        const float2 q = *reinterpret_cast<const float2*>(p);
        v[0] = q.x, v[1] = q.y;
    }
    else
    {
#pragma unroll
        for (int i = 0; i < VPL; i += 4)
        {
            const float4 q = *reinterpret_cast<const float4*>(p + i);
            v[i] = q.x, v[i + 1] = q.y, v[i + 2] = q.z, v[i + 3] = q.w;
        }
    }
}

// Merges the first n partial results of q row `row` (= b * H + h) into the output row.  One warp.
template <typename T, int DH>
__device__ __forceinline__ void merge_row(const AttnArgs& a, int row, int n, int lane)
{
    constexpr int VPL = DH / 32; // floats per lane (2, 4 or 8)
    // (m, l) of up to 32 partitions per pass, one per lane: all loads of a pass are in flight together.
    const float2* ml = a.part_ml + (size_t) row * a.nsplit;
    const float* po = a.part_o + (size_t) row * a.nsplit * DH + lane * VPL;
    // The first 8 partial rows are requested before the maxima are reduced: their latency then overlaps that of
    // the (m, l) loads instead of following it.
    float v0[8][VPL];
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const int c = min(j, n - 1);
        load_partial<VPL>(po + (size_t) c * DH, v0[j]);
    }
    float M = -INFINITY;
    for (int c0 = 0; c0 < n; c0 += 32)
    {
        const float mc = (c0 + lane < n) ? ml[c0 + lane].x : -INFINITY;
        M = fmaxf(M, mc);
    }
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1)
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, x));

    float L = 0.f;
    float o[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
        o[i] = 0.f;
    for (int c0 = 0; c0 < n; c0 += 32)
    {
        // lane j holds the weight of partition c0 + j
        float f = 0.f, lw = 0.f;
        if (c0 + lane < n)
        {
            const float2 v = ml[c0 + lane];
            f = fast_exp2(v.x - M);
            lw = v.y * f;
        }
        L += lw;
        const int cnt = min(32, n - c0);
        for (int j0 = 0; j0 < cnt; j0 += 8)
        {
            // 8 independent row loads, then the weighted sums
            float v[8][VPL];
            if (c0 + j0 == 0)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int i = 0; i < VPL; ++i)
                        v[j][i] = v0[j][i];
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const int c = min(c0 + j0 + j, n - 1); // clamped: weight of a padded slot is 0
                    load_partial<VPL>(po + (size_t) c * DH, v[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                float fj = __shfl_sync(0xffffffffu, f, (j0 + j) & 31);
                if (j0 + j >= cnt)
                    fj = 0.f;
#pragma unroll
                for (int i = 0; i < VPL; ++i)
                    o[i] = fmaf(v[j][i], fj, o[i]);
            }
        }
    }
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1)
        L += __shfl_xor_sync(0xffffffffu, L, x);
    const float inv = 1.f / L;
    T* dst = reinterpret_cast<T*>(a.out) + (size_t) row * DH + lane * VPL;
    if constexpr (VPL == 2)
    {
        *reinterpret_cast<uint32_t*>(dst) = TypeOps<T>::pack2(o[0] * inv, o[1] * inv);
    }
    else
    {
#pragma unroll
        for (int i = 0; i < VPL; i += 4)
        {
            uint2 w;
            w.x = TypeOps<T>::pack2(o[i] * inv, o[i + 1] * inv);
            w.y = TypeOps<T>::pack2(o[i + 2] * inv, o[i + 3] * inv);
            *reinterpret_cast<uint2*>(dst + i) = w;
        }
    }
}

template <typename T, int DH>
__global__ void __launch_bounds__(128) lse_merge_kernel(const AttnArgs a)
{
    griddep_launch_dependents(); // the next step's attention grid may become resident; it waits for this grid
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp; // b * H + h
    if (row >= a.batch * a.num_heads * max(1, a.q_len))
        return;
    const int b = row / (a.num_heads * max(1, a.q_len)); // (q_len > 1: rows are (sequence, new token, head))
    const int total = attended_tokens(a.seq_len[b], a.cyclic_window);
    griddep_wait(); // launched with programmatic stream serialisation: the partials are complete after this
    // partitions this sequence used (partition_of), never more than the launch had and never fewer than one: a
    // device length beyond what the call was planned for was reported by the attention kernel, and the merge
    // must not read another row's partials because of it
    const int n = max(1, min((total + a.chunk_tokens - 1) / a.chunk_tokens, a.nsplit));
    merge_row<T, DH>(a, row, n, lane);
}

// Many partitions per row (long sequences in a small batch): one CTA per q row instead of one warp.  Warp w merges
// partitions w, w + 4, ... into a state of its own (8 row loads in flight per round, a quarter of the rounds of the
// one-warp form), the four states meet in shared memory.  Same arithmetic, same result up to the order of the sums.
template <typename T, int DH>
__global__ void __launch_bounds__(128) lse_merge_many_kernel(const AttnArgs a)
{
    griddep_launch_dependents(); // the next step's attention grid may become resident; it waits for this grid
    constexpr int VPL = DH / 32;
    __shared__ float st_o[4][DH];
    __shared__ float st_ml[4][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x; // b * H + h (x new tokens)
    const int b = row / (a.num_heads * max(1, a.q_len));
    const int total = attended_tokens(a.seq_len[b], a.cyclic_window);
    griddep_wait();
    const int n = max(1, min((total + a.chunk_tokens - 1) / a.chunk_tokens, a.nsplit));
    const float2* ml = a.part_ml + (size_t) row * a.nsplit;
    const float* po = a.part_o + (size_t) row * a.nsplit * DH + lane * VPL;
    const int nw = (n - warp + 3) / 4; // partitions of this warp: warp + 4 j, j < nw (may be 0)
    float M = -INFINITY;
    for (int j0 = 0; j0 < nw; j0 += 32)
        if (j0 + lane < nw)
            M = fmaxf(M, __ldcg(ml + warp + 4 * (j0 + lane)).x);
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1)
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, x));
    float L = 0.f, o[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
        o[i] = 0.f;
    for (int j0 = 0; j0 < nw; j0 += 32)
    {
        float f = 0.f, lw = 0.f; // lane j holds the weight of this warp's partition j0 + j
        if (j0 + lane < nw)
        {
            const float2 v = __ldcg(ml + warp + 4 * (j0 + lane));
            f = (v.x == -INFINITY) ? 0.f : fast_exp2(v.x - M);
            lw = v.y * f;
        }
        L += lw;
        const int cnt = min(32, nw - j0);
        for (int k0 = 0; k0 < cnt; k0 += 8)
        {
            float v[8][VPL];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                load_partial<VPL>(po + (size_t) (warp + 4 * min(j0 + k0 + k, nw - 1)) * DH, v[k]);
#pragma unroll
            for (int k = 0; k < 8; ++k)
            {
                float fk = __shfl_sync(0xffffffffu, f, (k0 + k) & 31);
                if (k0 + k >= cnt)
                    fk = 0.f;
#pragma unroll
                for (int i = 0; i < VPL; ++i)
                    o[i] = fmaf(v[k][i], fk, o[i]);
            }
        }
    }
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1)
        L += __shfl_xor_sync(0xffffffffu, L, x);
#pragma unroll
    for (int i = 0; i < VPL; ++i)
        st_o[warp][lane * VPL + i] = o[i];
    if (lane == 0)
        st_ml[warp][0] = M, st_ml[warp][1] = L;
    __syncthreads();
    for (int d = threadIdx.x; d < DH; d += blockDim.x)
    {
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            Mx = fmaxf(Mx, st_ml[w][0]);
        float Lx = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
        {
            const float f = (st_ml[w][0] == -INFINITY) ? 0.f : fast_exp2(st_ml[w][0] - Mx);
            Lx = fmaf(st_ml[w][1], f, Lx);
            acc = fmaf(st_o[w][d], f, acc);
        }
        reinterpret_cast<T*>(a.out)[(size_t) row * DH + d] = TypeOps<T>::from_float(acc / Lx);
    }
}

// Stream-K launches: a row cut into several pieces has one partial per piece; rows that one CTA covered alone
// were written out by the attention kernel.
template <typename T, int DH>
__global__ void __launch_bounds__(128) lse_merge_sk_kernel(const AttnArgs a, const int hgroups, const __grid_constant__ SkSchedule sk)
{
    griddep_launch_dependents(); // the next step's attention grid may become resident; it waits for this grid
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp; // b * H + h
    if (row >= a.batch * a.num_heads)
        return;
    const int b = row / a.num_heads, h = row % a.num_heads;
    const int G = a.num_heads / a.num_kv_heads;
    const int y = (h / G) * hgroups + (h % G) / 16;
    const int n = min(sk_pieces_of_row(sk, b, y), a.nsplit);
    griddep_wait();
    if (a.tickets != nullptr && blockIdx.x == 0 && threadIdx.x == 0)
        *a.tickets = 0; // the attention grid has finished: its ticket counter starts the next launch at zero
    if (n > 1)
        merge_row<T, DH>(a, row, n, lane);
}

} // namespace dx
