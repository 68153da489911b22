// Feature-complete generation-phase attention: beam search through the cache indirection table, cyclic
// (sliding-window) cache with sink tokens, ALiBi.  One CTA per (sequence, q head); plain 16-byte loads per
// lane, fp32 FMA, online softmax per lane group, merge through shared memory.  Calls that use none of these
// features never come here: they run on the streaming kernels.
//
// What is restated (cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h,
// position shift off):
//   kv_loop_length = min(tlength, cyclic window): the kernel walks cache SLOTS 0 .. kv_loop_length-1        (:1493, :1897-1945)
//   slot of the new token = tok < sink ? tok : sink + (tok - sink) % cyclic_len                  (kvCacheUtils.h:109-117)
//   beams: slot s comes from sequence batch*beam_width + (s < context length ? 0 : cache_indir[bb][s]);
//          a wrapped cache takes every slot through the table                                     (:1497-1498, :2063-2078)
//   ALiBi: score += slope[head] * (s - tlength), nothing for the new token                              (:1797, :2026)
//   relative attention bias: score += bias[head][tlength][s] (new token: s = tlength), or in the implicit form
//          table[head][bucket(s - tlength)] with the T5 bucket function                     (:1773-1797, :1957-1985)
// The new token is read "as stored" (quantised, then dequantised) and written to the cache by
// kv_append_token_kernel, launched behind this kernel: every CTA sees the old content of the slot that is
// about to be overwritten, as the reference's one-CTA-per-head kernel does for its own head.
#pragma once

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh" // dequant_vec, make_cache_vec

namespace dx
{

// Lane mapping of the kernels in this file for any head size whose cache row is a multiple of 16 bytes (the
// reference's MMHA head sizes, decoderMaskedMultiheadAttention.cu:68-85): a row takes CHUNKS 16-byte pieces; LPR, the
// next power of two, lanes form the group that owns a row, of which the first CHUNKS are active (the others hold
// zeros and take part in the shuffles only).  For Dh 64 / 128 every lane is active.
template <int CACHE, int DH>
struct GenTraits
{
    static constexpr int ECB = (CACHE == CACHE_T) ? 2 : 1; // bytes per cache element
    static constexpr int ROW_BYTES = DH * ECB;
    static constexpr int EPL = 16 / ECB;                   // elements per lane
    static constexpr int CHUNKS = ROW_BYTES / 16;
    static constexpr int LPR = CHUNKS <= 1 ? 1 : CHUNKS <= 2 ? 2 : CHUNKS <= 4 ? 4 : CHUNKS <= 8 ? 8 : CHUNKS <= 16 ? 16 : 32;
    static constexpr int TPW = 32 / LPR;                   // rows one warp-wide load covers
    static_assert(ROW_BYTES % 16 == 0 && CHUNKS <= 32, "cache rows are moved in 16-byte pieces");
};

template <typename T, int CACHE, int DH>
__global__ void __launch_bounds__(128) general_decode_kernel(const GeneralArgs a)
{
    using Tr = GenTraits<CACHE, DH>;
    constexpr int LPR = Tr::LPR, TPW = Tr::TPW, EPL = Tr::EPL, ROW_BYTES = Tr::ROW_BYTES;
    constexpr int U = 2;              // token passes in flight per warp
    constexpr int NSTATE = 4 * TPW;   // lane groups of the CTA, each with its own running softmax
    constexpr float LOG2E = 1.4426950408889634f;

    const int h = blockIdx.x, bb = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, sl = lane % LPR;
    const bool active = sl < Tr::CHUNKS; // (always true for Dh 64 / 128)
    const int G = a.num_heads / a.num_kv_heads;
    const int hk = h / G;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    const int tlength = a.seq_len[bb] - 1;
    const int kv_len = min(tlength, a.cyclic_window);
    const bool beams = a.cache_indir != nullptr && a.beam_width > 1;
    const int seq0 = beams ? (bb / a.beam_width) * a.beam_width : bb;
    const int ctx0 = !beams ? kv_len : (tlength > a.cyclic_window ? 0 : (a.context_lengths ? a.context_lengths[bb] : 0));
    const int32_t* indir = beams ? a.cache_indir + (size_t) bb * a.max_attention_window : nullptr;

    const float deq = (CACHE == CACHE_T) ? 1.f : __ldg(a.scale_quant_orig);
    const float sscale = deq * a.softmax_scale_log2;
    float slope = 0.f;
    if (a.alibi_slopes != nullptr)
        slope = TypeOps<T>::to_float(reinterpret_cast<const T*>(a.alibi_slopes)[h]) * LOG2E;
    // Relative attention bias of cache slot s (log2 units), 0 without a table.
    const T* rel = reinterpret_cast<const T*>(a.rel_bias);
    auto rel_bias_of = [&](int s) -> float
    {
        if (rel == nullptr)
            return 0.f;
        if (a.max_distance > 0)
        {
            // the reference's bucket of a relative position (bidirectional layout of the table, the decoder only
            // ever sees positions <= 0)
            int num_buckets = a.rel_stride / 2;
            int relative_position = s - tlength;
            int bucket = relative_position > 0 ? num_buckets : 0;
            relative_position = abs(relative_position);
            const int max_exact = num_buckets / 2;
            const bool is_small = relative_position < max_exact;
            int if_large = max_exact
                + (int) (logf(relative_position * 1.0f / max_exact) / logf((float) a.max_distance / max_exact)
                    * (num_buckets - max_exact));
            if_large = min(if_large, num_buckets - 1);
            bucket += is_small ? relative_position : if_large;
            return TypeOps<T>::to_float(rel[(size_t) h * a.rel_stride + bucket]) * LOG2E;
        }
        return TypeOps<T>::to_float(rel[((size_t) h * a.rel_stride + tlength) * a.rel_stride + s]) * LOG2E;
    };

    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) bb * qkv_stride;
    float q[EPL];
    {
        const T* qp = qkv_b + (size_t) h * DH + sl * EPL;
#pragma unroll
        for (int i = 0; i < EPL; i += 2)
        {
            const float2 v = active ? TypeOps<T>::unpack2(*reinterpret_cast<const uint32_t*>(qp + i)) : make_float2(0.f, 0.f);
            q[i] = v.x;
            q[i + 1] = v.y;
        }
    }

    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i)
        o[i] = 0.f;

    auto accumulate = [&](const uint4& kraw, const uint4& vraw, float bias, bool valid)
    {
        float kf[EPL], vf[EPL];
        dequant_vec<T, CACHE, EPL>(kraw, kf);
        dequant_vec<T, CACHE, EPL>(vraw, vf);
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            d = fmaf(q[i], kf[i], d);
#pragma unroll
        for (int x = LPR / 2; x >= 1; x >>= 1)
            d += __shfl_xor_sync(0xffffffffu, d, x);
        if (valid)
        {
            const float s = fmaf(d, sscale, bias);
            const float mn = fmaxf(m, s);
            const float alpha = fast_exp2(m - mn), p = fast_exp2(s - mn);
            m = mn;
            l = fmaf(l, alpha, p);
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                o[i] = fmaf(o[i], alpha, p * vf[i]);
        }
    };

    const size_t head_off = (size_t) hk * ((size_t) ROW_BYTES << tpb_log2) + sl * 16;
    const int step = 4 * TPW * U;
    for (int base = 0; base < kv_len; base += step)
    {
        uint4 kraw[U], vraw[U];
        int slot[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            slot[u] = base + (warp * U + u) * TPW + sub;
            const int s = min(slot[u], kv_len - 1);
            const int seq = seq0 + ((beams && s >= ctx0) ? __ldg(indir + s) : 0);
            const int64_t* rowp = a.block_ptrs + (int64_t) seq * 2 * a.max_blocks_per_seq;
            const size_t off = head_off + (size_t) (s & tpb_mask) * ROW_BYTES;
            kraw[u] = vraw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (active)
            {
                kraw[u] = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const char*>(table_entry(rowp, s >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off);
                vraw[u] = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const char*>(table_entry(rowp + a.max_blocks_per_seq, s >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            accumulate(kraw[u], vraw[u],
                slope * (float) (slot[u] - tlength) + rel_bias_of(min(slot[u], kv_len - 1)), slot[u] < kv_len);
    }
    // the new token, as it will be stored: one lane group of warp 0 (every lane runs the shuffles)
    {
        const float sc_f = (CACHE == CACHE_T) ? 1.f : __ldg(a.scale_orig_quant);
        const T sc_t = TypeOps<T>::from_float(sc_f);
        const T* kp = qkv_b + (size_t) (a.num_heads + hk) * DH + sl * EPL;
        const T* vp = qkv_b + (size_t) (a.num_heads + a.num_kv_heads + hk) * DH + sl * EPL;
        uint4 kq = make_uint4(0u, 0u, 0u, 0u), vq = kq;
        if (active)
        {
            kq = make_cache_vec<T, CACHE, EPL>(kp, sc_f, sc_t);
            vq = make_cache_vec<T, CACHE, EPL>(vp, sc_f, sc_t);
        }
        if (warp == 0)
            accumulate(kq, vq, rel_bias_of(tlength), sub == 0);
    }

    // ---- merge the NSTATE running states ----
    extern __shared__ __align__(16) unsigned char smem_g[];
    float* st_o = reinterpret_cast<float*>(smem_g); // [NSTATE][DH]
    float* st_m = st_o + NSTATE * DH;                // [NSTATE]
    float* st_l = st_m + NSTATE;                     // [NSTATE]
    const int state = warp * TPW + sub;
    if (active)
    {
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            st_o[state * DH + sl * EPL + i] = o[i];
    }
    if (sl == 0)
    {
        st_m[state] = m;
        st_l[state] = l;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < DH; d += blockDim.x)
    {
        float M = -INFINITY;
        for (int s = 0; s < NSTATE; ++s)
            M = fmaxf(M, st_m[s]);
        float L = 0.f, acc = 0.f;
        for (int s = 0; s < NSTATE; ++s)
        {
            const float f = fast_exp2(st_m[s] - M); // empty states: m = -inf -> 0
            L = fmaf(st_l[s], f, L);
            acc = fmaf(st_o[s * DH + d], f, acc);
        }
        reinterpret_cast<T*>(a.out)[((size_t) bb * a.num_heads + h) * DH + d] = TypeOps<T>::from_float(acc * deq / L);
    }
}

// Writes the new token's K and V rows (quantised as the reference stores them) at its cyclic slot.
// Grid (Hkv, B * q_len), one warp: row bb of QKV is token bb % q_len of sequence bb / q_len and goes to cache index
// sequence length - q_len + token (unfusedAttentionKernels_2_template.h:254-255, :330-387).
template <typename T, int CACHE, int DH>
__global__ void __launch_bounds__(32) kv_append_token_kernel(const GeneralArgs a)
{
    using Tr = GenTraits<CACHE, DH>;
    constexpr int EPL = Tr::EPL, ROW_BYTES = Tr::ROW_BYTES;
    const int hk = blockIdx.x, bb = blockIdx.y, lane = threadIdx.x;
    if (lane >= Tr::CHUNKS)
        return;
    const int seq = bb / a.q_len, tok = bb % a.q_len;
    const int tlength = a.seq_len[seq] - a.q_len + tok;
    const int slot = cyclic_slot(tlength, a.sink, a.cyclic_len);
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) bb * qkv_stride;
    const float sc_f = (CACHE == CACHE_T) ? 1.f : __ldg(a.scale_orig_quant);
    const T sc_t = TypeOps<T>::from_float(sc_f);
    const uint4 kq = make_cache_vec<T, CACHE, EPL>(qkv_b + (size_t) (a.num_heads + hk) * DH + lane * EPL, sc_f, sc_t);
    const uint4 vq = make_cache_vec<T, CACHE, EPL>(
        qkv_b + (size_t) (a.num_heads + a.num_kv_heads + hk) * DH + lane * EPL, sc_f, sc_t);
    const int64_t* rowp = a.block_ptrs + (int64_t) seq * 2 * a.max_blocks_per_seq;
    const size_t off = (size_t) hk * ((size_t) ROW_BYTES << tpb_log2) + (size_t) (slot & tpb_mask) * ROW_BYTES + lane * 16;
    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(table_entry(rowp, slot >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off) = kq;
    *reinterpret_cast<uint4*>(
        reinterpret_cast<char*>(table_entry(rowp + a.max_blocks_per_seq, slot >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off) = vq;
}

// Several new tokens per sequence in one step (the reference's Medusa mode, which it serves with pre-compiled
// multi-query-token XQA kernels: decoderXQAImplPrecompiled.cpp:315-338).  Launched BEHIND kv_append_token_kernel:
// all q_len new tokens are in the cache, and token t of a sequence attends to the cache entries before the step
// and to new token j where bit j of its packed mask row is set.  One CTA per (token row, q head), the lane
// mapping and the merge of general_decode_kernel.  No beams, no cyclic wrap, no ALiBi.
template <typename T, int CACHE, int DH>
__global__ void __launch_bounds__(128) multi_token_decode_kernel(const GeneralArgs a)
{
    using Tr = GenTraits<CACHE, DH>;
    constexpr int LPR = Tr::LPR, TPW = Tr::TPW, EPL = Tr::EPL, ROW_BYTES = Tr::ROW_BYTES;
    constexpr int U = 2;
    constexpr int NSTATE = 4 * TPW;

    const int h = blockIdx.x, bb = blockIdx.y;
    const int seq = bb / a.q_len, tok = bb % a.q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, sl = lane % LPR;
    const bool active = sl < Tr::CHUNKS; // (always true for Dh 64 / 128)
    const int G = a.num_heads / a.num_kv_heads;
    const int hk = h / G;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    const int total = a.seq_len[seq];
    const int past = total - a.q_len;
    const int32_t* mask_row = a.packed_mask + ((size_t) seq * a.q_len + tok) * ((a.q_len + 31) >> 5);

    const float deq = (CACHE == CACHE_T) ? 1.f : __ldg(a.scale_quant_orig);
    const float sscale = deq * a.softmax_scale_log2;
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    float q[EPL];
    {
        const T* qp = reinterpret_cast<const T*>(a.qkv) + (size_t) bb * qkv_stride + (size_t) h * DH + sl * EPL;
#pragma unroll
        for (int i = 0; i < EPL; i += 2)
        {
            const float2 v = active ? TypeOps<T>::unpack2(*reinterpret_cast<const uint32_t*>(qp + i)) : make_float2(0.f, 0.f);
            q[i] = v.x;
            q[i + 1] = v.y;
        }
    }
    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i)
        o[i] = 0.f;

    const int64_t* krow = a.block_ptrs + (int64_t) seq * 2 * a.max_blocks_per_seq;
    const size_t head_off = (size_t) hk * ((size_t) ROW_BYTES << tpb_log2) + sl * 16;
    const int step = 4 * TPW * U;
    for (int base = 0; base < total; base += step)
    {
        uint4 kraw[U], vraw[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const int slot = base + (warp * U + u) * TPW + sub;
            const int s = min(slot, total - 1);
            valid[u] = slot < past;
            if (slot >= past && slot < total)
                valid[u] = (__ldg(mask_row + ((slot - past) >> 5)) >> ((slot - past) & 31)) & 1;
            const size_t off = head_off + (size_t) (s & tpb_mask) * ROW_BYTES;
            kraw[u] = vraw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (active)
            {
                kraw[u] = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const char*>(table_entry(krow, s >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off);
                vraw[u] = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const char*>(table_entry(krow + a.max_blocks_per_seq, s >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            float kf[EPL], vf[EPL];
            dequant_vec<T, CACHE, EPL>(kraw[u], kf);
            dequant_vec<T, CACHE, EPL>(vraw[u], vf);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                d = fmaf(q[i], kf[i], d);
#pragma unroll
            for (int x = LPR / 2; x >= 1; x >>= 1)
                d += __shfl_xor_sync(0xffffffffu, d, x);
            if (valid[u])
            {
                const float s = d * sscale;
                const float mn = fmaxf(m, s);
                const float alpha = fast_exp2(m - mn), p = fast_exp2(s - mn);
                m = mn;
                l = fmaf(l, alpha, p);
#pragma unroll
                for (int i = 0; i < EPL; ++i)
                    o[i] = fmaf(o[i], alpha, p * vf[i]);
            }
        }
    }

    // ---- merge the NSTATE running states ----
    extern __shared__ __align__(16) unsigned char smem_g[];
    float* st_o = reinterpret_cast<float*>(smem_g); // [NSTATE][DH]
    float* st_m = st_o + NSTATE * DH;                // [NSTATE]
    float* st_l = st_m + NSTATE;                     // [NSTATE]
    const int state = warp * TPW + sub;
    if (active)
    {
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            st_o[state * DH + sl * EPL + i] = o[i];
    }
    if (sl == 0)
    {
        st_m[state] = m;
        st_l[state] = l;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < DH; d += blockDim.x)
    {
        float M = -INFINITY;
        for (int s = 0; s < NSTATE; ++s)
            M = fmaxf(M, st_m[s]);
        float L = 0.f, acc = 0.f;
        for (int s = 0; s < NSTATE; ++s)
        {
            const float f = (st_m[s] == -INFINITY) ? 0.f : fast_exp2(st_m[s] - M);
            L = fmaf(st_l[s], f, L);
            acc = fmaf(st_o[s * DH + d], f, acc);
        }
        reinterpret_cast<T*>(a.out)[((size_t) bb * a.num_heads + h) * DH + d] = TypeOps<T>::from_float(acc * deq / L);
    }
}

} // namespace dx
