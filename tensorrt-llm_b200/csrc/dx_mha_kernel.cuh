// Plain multi-head (one q head per kv-head stream) decode attention on CUDA cores.
//
// One CTA per (split-K partition, q head, sequence).  Each of the 4 warps owns every 4th group of
// TG tokens of the partition and runs its own online softmax; the groups arrive in shared memory
// through a warp-private ring of 1-D bulk async copies (cp.async.bulk, one K slab + one V slab per
// stage) completing on mbarriers.  Whole rows of a (block, head) slab are contiguous in the paged
// cache ([heads, tokens_per_block, Dh] per block), so a group is a single contiguous copy.
//
// Replaces, for the G == 1 case and as the generic fallback for any head mapping:
//   masked_multihead_attention_kernel
//     cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h:1303
//   (Q.K loop :1818-2038, softmax :2164-2313, P.V loop :2318-2422, K append :2207-2233, V append :2475-2537).
#pragma once

#include "dx_common.cuh"

namespace dx
{

template <int CACHE, int DH>
struct MhaTraits
{
    static constexpr int ECB = (CACHE == CACHE_T) ? 2 : 1; // bytes per cache element
    static constexpr int ROW_BYTES = DH * ECB;             // 64, 128, 256 or 512 (Dh 256 over a 16-bit cache)
    static constexpr int LPR = ROW_BYTES / 16;             // lanes covering one row with 16 B each
    static constexpr int TPW = 32 / LPR;                   // rows one warp-wide 16 B load covers
    static constexpr int EPL = 16 / ECB;                   // elements per lane
    static constexpr int TG = (ROW_BYTES == 512) ? 4 : (ROW_BYTES == 256) ? 8 : 16; // tokens per stage
    static constexpr int PASSES = TG / TPW;
    static constexpr int STAGES = 4;
    static constexpr int NWARPS = 4;
    static constexpr int SLAB = TG * ROW_BYTES;      // bytes of K (or V) per stage
    static constexpr int STAGE_BYTES = 2 * SLAB;     // K then V
    static constexpr int RING_BYTES = NWARPS * STAGES * STAGE_BYTES;
    static constexpr int MERGE_FLOATS = NWARPS * (DH + 2);
    static constexpr int SMEM_BYTES = RING_BYTES + MERGE_FLOATS * 4 + NWARPS * STAGES * 8 + 16;
};

// 16 cache bytes -> EPL floats (unscaled).
template <typename T, int CACHE, int EPL>
__device__ __forceinline__ void dequant_vec(const uint4& raw, float (&f)[EPL])
{
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    if constexpr (CACHE == CACHE_T)
    {
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            float2 v = TypeOps<T>::unpack2(w[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    else
    {
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            float t[4];
            dequant4<CACHE>(w[i], t);
            f[4 * i] = t[0];
            f[4 * i + 1] = t[1];
            f[4 * i + 2] = t[2];
            f[4 * i + 3] = t[3];
        }
    }
}

// Quantise (or copy) EPL activations of the new token starting at src into the 16 cache bytes
// the reference would store for them.
template <typename T, int CACHE, int EPL>
__device__ __forceinline__ uint4 make_cache_vec(const T* src, float scale_f32, T scale_t)
{
    uint4 r;
    if constexpr (CACHE == CACHE_T)
    {
        r = *reinterpret_cast<const uint4*>(src);
    }
    else
    {
        const uint4 a = reinterpret_cast<const uint4*>(src)[0];
        const uint4 b = reinterpret_cast<const uint4*>(src)[1];
        r.x = quant4<T, CACHE>(a.x, a.y, scale_f32, scale_t);
        r.y = quant4<T, CACHE>(a.z, a.w, scale_f32, scale_t);
        r.z = quant4<T, CACHE>(b.x, b.y, scale_f32, scale_t);
        r.w = quant4<T, CACHE>(b.z, b.w, scale_f32, scale_t);
    }
    return r;
}

template <typename T, int CACHE, int DH>
__global__ void __launch_bounds__(128) mha_decode_kernel(const AttnArgs a)
{
    using Tr = MhaTraits<CACHE, DH>;
    constexpr int LPR = Tr::LPR, TPW = Tr::TPW, EPL = Tr::EPL, TG = Tr::TG, PASSES = Tr::PASSES;
    constexpr int STAGES = Tr::STAGES, NWARPS = Tr::NWARPS, ROW_BYTES = Tr::ROW_BYTES, SLAB = Tr::SLAB;

    // (as a programmatic dependent of the kernel in front of it, the CTA is resident early and waits here)
    griddep_wait();
    const int chunk = blockIdx.x;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int total = a.seq_len[b]; // tokens to attend to, new token included
    int chunk_start, ctoks, nparts;
    partition_of(total, a.chunk_tokens, chunk, chunk_start, ctoks, nparts);
    if (nparts > (int) gridDim.x && chunk == 0 && threadIdx.x == 0)
        report_status(a.status, STATUS_PLAN_EXCEEDED); // the tokens beyond the last partition are not attended to
    if (chunk >= nparts)
        return;                                       // ragged batch: this sequence uses fewer partitions
    const int n_groups = (ctoks + TG - 1) / TG;
    const int new_pos = total - 1;                    // cache index of the new token
    const bool has_new = chunk == nparts - 1;          // the last partition ends with the new token

    griddep_launch_dependents(); // the merge kernel may be scheduled; it waits for this grid to finish
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, sl = lane % LPR;
    const int G = a.num_heads / a.num_kv_heads;
    const int hk = h / G;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem + warp * (STAGES * Tr::STAGE_BYTES);
    float* merge = reinterpret_cast<float*>(smem + Tr::RING_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::RING_BYTES + Tr::MERGE_FLOATS * 4) + warp * STAGES;

    if (lane == 0)
    {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            mbar_init(&bars[s], 1);
        fence_mbar_init();
    }
    __syncwarp();

    const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
    const int64_t* vrow = krow + a.max_blocks_per_seq;
    const size_t head_off = (size_t) hk * ((size_t) ROW_BYTES << tpb_log2);

    // Issues the copies of this warp's i-th group into ring stage i % STAGES (lane 0 only).
    auto issue = [&](int i)
    {
        const int gi = warp + NWARPS * i;
        const int t0 = chunk_start + gi * TG;
        // rows that already live in the cache: everything before the new token
        const int rows = min(TG, new_pos - t0);
        uint64_t* bar = &bars[i % STAGES];
        unsigned char* dst = ring + (i % STAGES) * Tr::STAGE_BYTES;
        const uint32_t bytes = rows > 0 ? (uint32_t) rows * ROW_BYTES : 0u;
        mbar_expect_tx(bar, 2 * bytes);
        if (bytes)
        {
            const size_t off = head_off + (size_t) (t0 & tpb_mask) * ROW_BYTES;
            const char* kb = reinterpret_cast<const char*>(table_entry(krow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            const char* vb = reinterpret_cast<const char*>(table_entry(vrow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            bulk_g2s(dst, kb, bytes, bar);
            bulk_g2s(dst + SLAB, vb, bytes, bar);
        }
    };

    // this lane's q channels are requested before the first ring stages: behind those bulk copies (tens of KB per
    // warp) the same loads would wait for all of their bytes
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
    uint4 q_raw[EPL / 8];
#pragma unroll
    for (int i = 0; i < EPL / 8; ++i)
        q_raw[i] = *reinterpret_cast<const uint4*>(qkv_b + h * DH + sl * EPL + 8 * i);

    const int my_groups = (n_groups > warp) ? (n_groups - warp + NWARPS - 1) / NWARPS : 0;
    if (lane == 0)
    {
        for (int i = 0; i < min(STAGES, my_groups); ++i)
            issue(i);
    }

    // q, pre-multiplied by the softmax scale (log2 units) and the K dequantisation scale.
    const float deq = (CACHE == CACHE_T) ? 1.f : __ldg(a.scale_quant_orig);
    float qf[EPL];
    {
        const float qs = a.softmax_scale_log2 * deq;
#pragma unroll
        for (int i = 0; i < EPL; i += 8)
        {
            const uint4 r = q_raw[i / 8];
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float2 v = TypeOps<T>::unpack2(w[j]);
                qf[i + 2 * j] = v.x * qs;
                qf[i + 2 * j + 1] = v.y * qs;
            }
        }
    }

    float m = -INFINITY, l = 0.f;
    float acc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i)
        acc[i] = 0.f;

    bool timed_out = false;
    int i = 0;
    for (; i < my_groups; ++i)
    {
        const int s = i % STAGES;
        const uint32_t parity = (i / STAGES) & 1;
        unsigned char* kbuf = ring + s * Tr::STAGE_BYTES;
        unsigned char* vbuf = kbuf + SLAB;
        if (!mbar_wait_bounded(&bars[s], parity, a.status))
        {
            timed_out = true;
            break;
        }
        const int gi = warp + NWARPS * i;
        const int t0 = chunk_start + gi * TG;
        int n_valid = min(TG, total - t0);
        if (has_new && new_pos >= t0 && new_pos < t0 + TG)
        {
            // This group ends with the new token: quantise it exactly as it is stored, place it
            // in the staged tile, clear the rows behind it and (first q head of the group only)
            // append it to the paged cache.
            const int r_new = new_pos - t0;
            float sc_f = 1.f;
            T sc_t = TypeOps<T>::from_float(1.f);
            if constexpr (CACHE != CACHE_T)
            {
                sc_f = __ldg(a.scale_orig_quant);
                sc_t = TypeOps<T>::from_float(sc_f);
            }
            if (lane < LPR)
            {
                const T* kp = qkv_b + (a.num_heads + hk) * DH + lane * EPL;
                const T* vp = qkv_b + (a.num_heads + a.num_kv_heads + hk) * DH + lane * EPL;
                const uint4 kq = make_cache_vec<T, CACHE, EPL>(kp, sc_f, sc_t);
                const uint4 vq = make_cache_vec<T, CACHE, EPL>(vp, sc_f, sc_t);
                *reinterpret_cast<uint4*>(kbuf + r_new * ROW_BYTES + lane * 16) = kq;
                *reinterpret_cast<uint4*>(vbuf + r_new * ROW_BYTES + lane * 16) = vq;
                if (h == hk * G)
                {
                    const size_t off = head_off + (size_t) (new_pos & tpb_mask) * ROW_BYTES + lane * 16;
                    char* kb = reinterpret_cast<char*>(table_entry(krow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                    char* vb = reinterpret_cast<char*>(table_entry(vrow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                    *reinterpret_cast<uint4*>(kb) = kq;
                    *reinterpret_cast<uint4*>(vb) = vq;
                }
            }
            // rows behind the new token were never copied: zero them so that 0 * garbage cannot
            // produce NaN in the P.V accumulation.
            for (int idx = lane; idx < (TG - 1 - r_new) * LPR; idx += 32)
            {
                const int off = (r_new + 1) * ROW_BYTES + idx * 16;
                *reinterpret_cast<uint4*>(kbuf + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vbuf + off) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- scores for the TG tokens of this group ----
        float sc[PASSES];
        float gmax = -INFINITY;
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
        {
            const int row = p * TPW + sub;
            const uint4 raw = *reinterpret_cast<const uint4*>(kbuf + row * ROW_BYTES + sl * 16);
            float kf[EPL];
            dequant_vec<T, CACHE, EPL>(raw, kf);
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e)
                d = fmaf(qf[e], kf[e], d);
#pragma unroll
            for (int x = 1; x < LPR; x <<= 1)
                d += __shfl_xor_sync(0xffffffffu, d, x);
            sc[p] = (row < n_valid) ? d : -INFINITY;
            gmax = fmaxf(gmax, sc[p]);
        }
#pragma unroll
        for (int x = LPR; x < 32; x <<= 1)
            gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, x));

        const float m_new = fmaxf(m, gmax);
        const float alpha = fast_exp2(m - m_new); // m == -inf on the first group -> 0
        m = m_new;
        l *= alpha;
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            acc[e] *= alpha;

        // ---- P.V ----
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
        {
            const int row = p * TPW + sub;
            const float pp = fast_exp2(sc[p] - m_new);
            l += pp;
            const uint4 raw = *reinterpret_cast<const uint4*>(vbuf + row * ROW_BYTES + sl * 16);
            float vf[EPL];
            dequant_vec<T, CACHE, EPL>(raw, vf);
#pragma unroll
            for (int e = 0; e < EPL; ++e)
                acc[e] = fmaf(pp, vf[e], acc[e]);
        }

        __syncwarp(); // every lane is done reading this stage
        if (lane == 0 && i + STAGES < my_groups)
            issue(i + STAGES);
    }

    if (timed_out)
    {
        if (lane == 0)
            report_status(a.status, STATUS_TIMEOUT);
        // the copies already requested (groups i .. i + STAGES - 1) must have landed before the CTA exits
        for (int j = i; j < min(i + STAGES, my_groups); ++j)
            mbar_drain(&bars[j % STAGES], (j / STAGES) & 1);
        // fall through: the CTA still meets its barriers below and writes what it has.
    }

    // ---- combine the row sub-groups of the warp ----
#pragma unroll
    for (int x = LPR; x < 32; x <<= 1)
    {
        l += __shfl_xor_sync(0xffffffffu, l, x);
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], x);
    }

    // ---- combine the warps ----
    float* mrow = merge + warp * (DH + 2);
    if (sub == 0)
    {
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            mrow[sl * EPL + e] = acc[e];
        if (sl == 0)
        {
            mrow[DH] = m;
            mrow[DH + 1] = l;
        }
    }
    __syncthreads();

    const float v_deq = deq;
    for (int d = threadIdx.x; d < DH; d += blockDim.x)
    {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w)
            M = fmaxf(M, merge[w * (DH + 2) + DH]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w)
        {
            const float mw = merge[w * (DH + 2) + DH];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L = fmaf(merge[w * (DH + 2) + DH + 1], f, L);
            o = fmaf(merge[w * (DH + 2) + d], f, o);
        }
        const size_t row = (size_t) b * a.num_heads + h;
        if (a.nsplit == 1)
        {
            reinterpret_cast<T*>(a.out)[row * DH + d] = TypeOps<T>::from_float(o * v_deq / L);
        }
        else
        {
            a.part_o[(row * a.nsplit + chunk) * DH + d] = o * v_deq;
            if (d == 0)
                a.part_ml[row * a.nsplit + chunk] = make_float2(M, L);
        }
    }
}

} // namespace dx
