// Plain multi-head decode attention over an INT8 paged KV cache on the CUDA cores, integer math.
//
// Same work split and copy pipeline as mha_decode_kernel (one CTA per (partition, q head,
// sequence); per-warp ring of 1-D bulk async copies completing on mbarriers), but the cache bytes
// are never converted: q is quantised once per CTA into a high and a low int8 part and Q.K^T is
// accumulated with 4-way int8 dot products (dp4a); P is quantised per token group the same way
// and P.V runs as dp4a over 4 tokens after a 4x4 byte transpose of V.  Sums are exact integers
// until they are folded into fp32, and the per-tensor scale is applied once per score / output.
//
// Replaces, for INT8 caches with one q head per kv-head stream:
//   masked_multihead_attention_kernel
//     cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionTemplate.h:1303
//   whose INT8 path converts every element to fp32 (decoderMaskedMultiheadAttentionUtils.h:3456-3503)
//   and multiplies it by the scale (Template.h:755-780, 980-984).
#pragma once

#include "dx_common.cuh"
#include "dx_gqa_kernel.cuh" // split4, transpose4x4, kLoWeight
#include "dx_mha_kernel.cuh" // make_cache_vec

namespace dx
{

template <int DH>
struct MhaInt8Traits
{
    static constexpr int ROW_BYTES = DH;          // 64 or 128
    static constexpr int LPR = ROW_BYTES / 16;    // lanes covering one row with 16 B each
    static constexpr int TPW = 32 / LPR;          // rows one warp-wide 16 B load covers
    static constexpr int PASSES = 4;              // a lane sees 4 tokens per stage (one dp4a word)
    static constexpr int TG = PASSES * TPW;       // tokens per stage: 16 (Dh 128) or 32 (Dh 64)
    static constexpr int STAGES = 4;
    static constexpr int NWARPS = 4;
    static constexpr int SLAB = TG * ROW_BYTES;   // 2 KB
    static constexpr int STAGE_BYTES = 2 * SLAB;
    static constexpr int RING_BYTES = NWARPS * STAGES * STAGE_BYTES;
    static constexpr int MERGE_FLOATS = NWARPS * (DH + 2);
    static constexpr int SMEM_BYTES = RING_BYTES + MERGE_FLOATS * 4 + NWARPS * STAGES * 8 + 16;
};

template <typename T, int DH>
__global__ void __launch_bounds__(128) mha_int8_decode_kernel(const AttnArgs a)
{
    using Tr = MhaInt8Traits<DH>;
    constexpr int LPR = Tr::LPR, TPW = Tr::TPW, TG = Tr::TG, PASSES = Tr::PASSES;
    constexpr int STAGES = Tr::STAGES, NWARPS = Tr::NWARPS, ROW_BYTES = Tr::ROW_BYTES, SLAB = Tr::SLAB;
    constexpr int CACHE = CACHE_INT8;

    // (as a programmatic dependent of the kernel in front of it, the CTA is resident early and waits here)
    griddep_wait();
    const int chunk = blockIdx.x;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int total = a.seq_len[b];
    int chunk_start, ctoks, nparts;
    partition_of(total, a.chunk_tokens, chunk, chunk_start, ctoks, nparts);
    if (nparts > (int) gridDim.x && chunk == 0 && threadIdx.x == 0)
        report_status(a.status, STATUS_PLAN_EXCEEDED); // the tokens beyond the last partition are not attended to
    if (chunk >= nparts)
        return; // ragged batch: this sequence uses fewer partitions
    griddep_launch_dependents(); // the merge kernel may be scheduled; it waits for this grid to finish
    const int n_groups = (ctoks + TG - 1) / TG;
    const int new_pos = total - 1;

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

    auto issue = [&](int i)
    {
        const int gi = warp + NWARPS * i;
        const int t0 = chunk_start + gi * TG;
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
    uint4 q_raw[16 / 8];
#pragma unroll
    for (int i = 0; i < 16 / 8; ++i)
        q_raw[i] = *reinterpret_cast<const uint4*>(qkv_b + h * DH + sl * 16 + 8 * i);

    const int my_groups = (n_groups > warp) ? (n_groups - warp + NWARPS - 1) / NWARPS : 0;
    if (lane == 0)
    {
        for (int i = 0; i < min(STAGES, my_groups); ++i)
            issue(i);
    }

    // ---- q: 16 channels per lane, quantised per head into high + low int8 parts ----
    const float deq = __ldg(a.scale_quant_orig);
    uint32_t qhi[4], qlo[4];
    float sfac;
    {
        float qv[16];
#pragma unroll
        for (int i = 0; i < 16; i += 8)
        {
            const uint4 r = q_raw[i / 8];
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const float2 v = TypeOps<T>::unpack2(w[j]);
                qv[i + 2 * j] = v.x;
                qv[i + 2 * j + 1] = v.y;
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            amax = fmaxf(amax, fabsf(qv[i]));
#pragma unroll
        for (int x = 1; x < LPR; x <<= 1)
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, x));
        const float qs = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
        const float qmul = 1.f / qs;
        sfac = qs * (1.f / kLoWeight) * deq * a.softmax_scale_log2;
#pragma unroll
        for (int w = 0; w < 4; ++w)
            split4<CACHE_INT8>(qv[4 * w] * qmul, qv[4 * w + 1] * qmul, qv[4 * w + 2] * qmul, qv[4 * w + 3] * qmul,
                qhi[w], qlo[w]);
    }

    float m = -INFINITY, l = 0.f;
    float accf[16];
    int ahi[16], alo[16];
#pragma unroll
    for (int e = 0; e < 16; ++e)
        accf[e] = 0.f, ahi[e] = 0, alo[e] = 0;
    auto fold = [&]()
    {
#pragma unroll
        for (int e = 0; e < 16; ++e)
        {
            accf[e] += (float) (ahi[e] * kLoWeight + alo[e]);
            ahi[e] = 0;
            alo[e] = 0;
        }
    };

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
        const int n_valid = min(TG, total - t0);
        if (new_pos < t0 + TG)
        {
            // last group of the sequence: quantise the new token as it is stored, place it in the
            // staged tile, clear the rows behind it, append it to the cache (first q head of the group)
            const int r_new = new_pos - t0;
            const float sc_f = __ldg(a.scale_orig_quant);
            const T sc_t = TypeOps<T>::from_float(sc_f);
            if (lane < LPR)
            {
                const T* kp = qkv_b + (a.num_heads + hk) * DH + lane * 16;
                const T* vp = qkv_b + (a.num_heads + a.num_kv_heads + hk) * DH + lane * 16;
                const uint4 kq = make_cache_vec<T, CACHE, 16>(kp, sc_f, sc_t);
                const uint4 vq = make_cache_vec<T, CACHE, 16>(vp, sc_f, sc_t);
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
            for (int idx = lane; idx < (TG - 1 - r_new) * LPR; idx += 32)
            {
                const int off = (r_new + 1) * ROW_BYTES + idx * 16;
                *reinterpret_cast<uint4*>(kbuf + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vbuf + off) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- scores: 4 tokens per lane sub-group ----
        float sc[PASSES];
        float gmax = -INFINITY;
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
        {
            const int row = p * TPW + sub;
            const uint4 raw = *reinterpret_cast<const uint4*>(kbuf + row * ROW_BYTES + sl * 16);
            int shi = __dp4a((int) raw.x, (int) qhi[0], 0), slo = __dp4a((int) raw.x, (int) qlo[0], 0);
            shi = __dp4a((int) raw.y, (int) qhi[1], shi), slo = __dp4a((int) raw.y, (int) qlo[1], slo);
            shi = __dp4a((int) raw.z, (int) qhi[2], shi), slo = __dp4a((int) raw.z, (int) qlo[2], slo);
            shi = __dp4a((int) raw.w, (int) qhi[3], shi), slo = __dp4a((int) raw.w, (int) qlo[3], slo);
            int tot = shi * kLoWeight + slo;
#pragma unroll
            for (int x = 1; x < LPR; x <<= 1)
                tot += __shfl_xor_sync(0xffffffffu, tot, x);
            sc[p] = (row < n_valid) ? (float) tot * sfac : -INFINITY;
            gmax = fmaxf(gmax, sc[p]);
        }
#pragma unroll
        for (int x = LPR; x < 32; x <<= 1)
            gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, x));

        const float m_new = fmaxf(m, gmax);
        if (m_new != m) // warp-uniform: every lane holds the same m and gmax
        {
            fold();
            const float alpha = fast_exp2(m - m_new);
            l *= alpha;
#pragma unroll
            for (int e = 0; e < 16; ++e)
                accf[e] *= alpha;
            m = m_new;
        }
        else if ((i & 63) == 63)
        {
            fold(); // keeps the pending integer sums far from overflow
        }

        // ---- P (4 tokens of this sub-group) as int8 high / low parts ----
        float pp[PASSES];
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
        {
            pp[p] = fast_exp2(sc[p] - m);
            l += pp[p];
        }
        uint32_t phi, plo;
        split4<CACHE_INT8>(pp[0] * 127.f, pp[1] * 127.f, pp[2] * 127.f, pp[3] * 127.f, phi, plo);

        // ---- P.V: transpose 4 tokens x 4 channels, then one dp4a per channel and part ----
        uint4 rv[PASSES];
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
            rv[p] = *reinterpret_cast<const uint4*>(vbuf + (p * TPW + sub) * ROW_BYTES + sl * 16);
#pragma unroll
        for (int w = 0; w < 4; ++w)
        {
            const uint32_t r0 = w == 0 ? rv[0].x : w == 1 ? rv[0].y : w == 2 ? rv[0].z : rv[0].w;
            const uint32_t r1 = w == 0 ? rv[1].x : w == 1 ? rv[1].y : w == 2 ? rv[1].z : rv[1].w;
            const uint32_t r2 = w == 0 ? rv[2].x : w == 1 ? rv[2].y : w == 2 ? rv[2].z : rv[2].w;
            const uint32_t r3 = w == 0 ? rv[3].x : w == 1 ? rv[3].y : w == 2 ? rv[3].z : rv[3].w;
            uint32_t tr[4];
            transpose4x4(r0, r1, r2, r3, tr);
#pragma unroll
            for (int c = 0; c < 4; ++c)
            {
                ahi[4 * w + c] = __dp4a((int) tr[c], (int) phi, ahi[4 * w + c]);
                alo[4 * w + c] = __dp4a((int) tr[c], (int) plo, alo[4 * w + c]);
            }
        }

        __syncwarp();
        if (lane == 0 && i + STAGES < my_groups)
            issue(i + STAGES);
    }
    fold();

    if (timed_out)
    {
        if (lane == 0)
            report_status(a.status, STATUS_TIMEOUT);
        // the copies already requested (groups i .. i + STAGES - 1) must have landed before the CTA exits
        for (int j = i; j < min(i + STAGES, my_groups); ++j)
            mbar_drain(&bars[j % STAGES], (j / STAGES) & 1);
    }

    // ---- combine the row sub-groups of the warp ----
#pragma unroll
    for (int x = LPR; x < 32; x <<= 1)
    {
        l += __shfl_xor_sync(0xffffffffu, l, x);
#pragma unroll
        for (int e = 0; e < 16; ++e)
            accf[e] += __shfl_xor_sync(0xffffffffu, accf[e], x);
    }

    // ---- combine the warps ----
    float* mrow = merge + warp * (DH + 2);
    if (sub == 0)
    {
#pragma unroll
        for (int e = 0; e < 16; ++e)
            mrow[sl * 16 + e] = accf[e];
        if (sl == 0)
        {
            mrow[DH] = m;
            mrow[DH + 1] = l;
        }
    }
    __syncthreads();

    const float ofac = deq * (1.f / (127.f * kLoWeight));
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
            reinterpret_cast<T*>(a.out)[row * DH + d] = TypeOps<T>::from_float(o * ofac / L);
        }
        else
        {
            a.part_o[(row * a.nsplit + chunk) * DH + d] = o * ofac;
            if (d == 0)
                a.part_ml[row * a.nsplit + chunk] = make_float2(M, L);
        }
    }
}

} // namespace dx
