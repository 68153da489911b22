// Grouped-head (GQA / MQA) decode attention over an 8-bit paged KV cache on the tensor cores.
//
// One CTA per (split-K partition, kv head x 16-head slice of its q group, sequence).  The q heads
// that share the kv head form the M dimension of S = Q K^T (m16n8k32 MMA, fp8 x fp8 -> fp32 or
// s8 x s8 -> s32), so every cache byte is fetched from HBM once for the whole group and is fed to
// the MMA as stored - no per-element dequantisation instruction exists on the read path; the
// per-tensor scale is folded into the score scale and into the final normalisation.  Q and P are
// split into a high and a low 8-bit part (two MMAs) so that they keep ~8 significant bits.
// P V is computed transposed, O^T[Dh x heads] = V^T P^T, which makes the S accumulator fragments
// directly usable as the B operand; V^T fragments are built from 16-byte shared-memory loads
// with a 4x4 byte transpose (PRMT).
//
// Each of the 4 warps owns every 4th 32-token group of the partition and runs its own online
// softmax; groups are staged through a warp-private 3-stage ring filled with 16-byte cp.async
// copies (XOR-swizzled per 128-byte line so that both fragment load patterns are bank-conflict
// free) whose completion is tracked by mbarriers (cp.async.mbarrier.arrive.noinc).
//
// Replaces the XQA kernels (binary-only in the reference, dispatched from
//   cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderXQAImplPrecompiled.cpp:263-374)
// together with their pre-processing launch that appends the new token
//   (cpp/tensorrt_llm/kernels/unfusedAttentionKernels/unfusedAttentionKernels_2_template.h:336-387),
// and the MMHA kernel for grouped heads (decoderMaskedMultiheadAttentionTemplate.h:1303).
#pragma once

#include <type_traits>

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh" // make_cache_vec

namespace dx
{

template <int DH>
struct GqaTraits
{
    static constexpr int TG = 32;           // tokens per stage (per warp)
    static constexpr int KS = DH / 32;      // k-steps of Q K^T
    static constexpr int MT = DH / 16;      // m-tiles of O^T
    static constexpr int NW = DH / 32;      // 32-bit words of V per row per thread
    static constexpr int QV = DH / 4;       // q elements per thread per head row
    static constexpr int SLAB = TG * DH;    // bytes of K (or V) per stage
    static constexpr int STAGE_BYTES = 2 * SLAB;
    static constexpr int STAGES = 3;
    static constexpr int NWARPS = 4;
    static constexpr int RING_BYTES = NWARPS * STAGES * STAGE_BYTES;
    static constexpr int MERGE_BYTES = NWARPS * (16 * DH + 32) * 4;
    static constexpr int SMEM_BYTES = (RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES) + NWARPS * STAGES * 8 + 16;
};

// Token row (within a 32-token group) that S-tile nt, column col refers to.
template <int DH>
__device__ __forceinline__ int sigma_row(int nt, int col)
{
    if constexpr (DH == 128)
        return 8 * nt + col;
    else
        return 4 * col + nt;
}

// Swizzled byte offset inside a K or V slab for a linear (row-major) byte offset.
template <int DH>
__device__ __forceinline__ uint32_t swz(uint32_t off)
{
    const uint32_t line = off >> 7;
    if constexpr (DH == 128)
        return off ^ ((line & 7u) << 4);
    else
    {
        const uint32_t f = ((((line >> 1) ^ (line >> 3)) & 1u) << 2) | (((line >> 2) & 1u) << 1);
        return off ^ (f << 4);
    }
}

__device__ __forceinline__ void cp_async16_zfill(void* dst_smem, const void* src_gmem, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem),
                 "r"(src_bytes)
                 : "memory");
}

__device__ __forceinline__ void mma_e4m3(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 4x4 byte transpose: o[j] byte i = r[i] byte j.
__device__ __forceinline__ void transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&o)[4])
{
    const uint32_t t0 = __byte_perm(r0, r1, 0x5140); // r0.b0 r1.b0 r0.b1 r1.b1
    const uint32_t t1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t t2 = __byte_perm(r0, r1, 0x7362); // r0.b2 r1.b2 r0.b3 r1.b3
    const uint32_t t3 = __byte_perm(r2, r3, 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410);
    o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410);
    o[3] = __byte_perm(t2, t3, 0x7632);
}

// Split x (already scaled into the 8-bit range) into a high and a low 8-bit part.
template <int CACHE>
__device__ __forceinline__ void split_hi_lo(float x, uint32_t& hi, uint32_t& lo)
{
    if constexpr (CACHE == CACHE_FP8)
    {
        const __nv_fp8_storage_t h = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(h, __NV_E4M3);
        const float hf = __half2float(*reinterpret_cast<const __half*>(&hr));
        hi = h;
        lo = __nv_cvt_float_to_fp8(x - hf, __NV_SATFINITE, __NV_E4M3);
    }
    else
    {
        const float h = rintf(x);
        hi = (uint32_t) (__float2int_rn(h) & 0xff);
        lo = (uint32_t) (__float2int_rn((x - h) * 128.f) & 0xff);
    }
}

// HL: weight of the high accumulator relative to the low one for the integer path.
static constexpr int kLoWeight = 128;

template <typename T, int CACHE, int DH, bool H16>
__global__ void __launch_bounds__(128, 2) gqa_decode_kernel(const AttnArgs a, const int hgroups)
{
    static_assert(CACHE == CACHE_INT8 || CACHE == CACHE_FP8, "8-bit caches only");
    using Tr = GqaTraits<DH>;
    constexpr int TG = Tr::TG, KS = Tr::KS, MT = Tr::MT, NW = Tr::NW, QV = Tr::QV;
    constexpr int SLAB = Tr::SLAB, STAGES = Tr::STAGES, NWARPS = Tr::NWARPS;
    constexpr int NR = H16 ? 2 : 1; // head-row halves in use (rows g, and rows g + 8)
    constexpr bool IS_FP8 = CACHE == CACHE_FP8;
    using Acc = typename std::conditional<IS_FP8, float, int>::type;

    const int chunk = blockIdx.x;
    const int hk = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
    const int b = blockIdx.z;
    const int total = a.seq_len[b];
    const int chunk_start = chunk * a.chunk_tokens;
    if (chunk_start >= total)
        return;
    const int ctoks = min(a.chunk_tokens, total - chunk_start);
    const int n_groups = (ctoks + TG - 1) / TG;
    const int new_pos = total - 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = a.num_heads / a.num_kv_heads;
    const int nh = min(16, G - hg * 16);      // q heads handled by this CTA
    const int head0 = hk * G + hg * 16;       // first of them
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* ring = smem + warp * (STAGES * Tr::STAGE_BYTES);
    constexpr int BAR_OFF = (Tr::RING_BYTES > Tr::MERGE_BYTES ? Tr::RING_BYTES : Tr::MERGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFF) + warp * STAGES;

    if (lane == 0)
    {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            mbar_init(&bars[s], 32);
        fence_mbar_init();
    }
    __syncwarp();

    const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
    const int64_t* vrow = krow + a.max_blocks_per_seq;
    const size_t head_off = (size_t) hk * ((size_t) DH << tpb_log2);

    // Every lane copies its share of the i-th group of this warp into ring stage i % STAGES.
    auto issue = [&](int i)
    {
        const int gi = warp + NWARPS * i;
        const int t0 = chunk_start + gi * TG;
        const int rows = min(TG, new_pos - t0); // rows already in the cache
        unsigned char* kdst = ring + (i % STAGES) * Tr::STAGE_BYTES;
        unsigned char* vdst = kdst + SLAB;
        const size_t off = head_off + (size_t) (t0 & tpb_mask) * DH;
        const char* kb = reinterpret_cast<const char*>(__ldg(krow + (t0 >> tpb_log2))) + off;
        const char* vb = reinterpret_cast<const char*>(__ldg(vrow + (t0 >> tpb_log2))) + off;
        const uint32_t valid_bytes = rows > 0 ? (uint32_t) rows * DH : 0u;
#pragma unroll
        for (int j = 0; j < SLAB / 512; ++j)
        {
            const uint32_t lin = (uint32_t) (lane + 32 * j) * 16;
            const bool ok = lin < valid_bytes;
            const uint32_t src_off = ok ? lin : 0u;
            cp_async16_zfill(kdst + swz<DH>(lin), kb + src_off, ok ? 16u : 0u);
            cp_async16_zfill(vdst + swz<DH>(lin), vb + src_off, ok ? 16u : 0u);
        }
        cp_async_mbar_arrive_noinc(&bars[i % STAGES]);
    };

    const int my_groups = (n_groups > warp) ? (n_groups - warp + NWARPS - 1) / NWARPS : 0;
    for (int i = 0; i < min(STAGES, my_groups); ++i)
        issue(i);

    // ---- Q: load the head rows g (and g + 8), scale each row into the 8-bit range, split hi/lo
    // and pack straight into A fragments.  The k index of every MMA is a fixed permutation of Dh
    // chosen so that K fragments are plain 16-byte shared-memory loads. ----
    const float deq = __ldg(a.scale_quant_orig);
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
    uint32_t qa[2][KS][4]; // [hi/lo][k-step][a0..a3]
    float sfac[2];         // accumulator -> score in log2 units, per head-row half
#pragma unroll
    for (int r = 0; r < 2; ++r)
    {
        float qv[QV];
        const int hl = g + 8 * r; // head within this CTA
        const bool valid = (r < NR) && hl < nh;
        if (valid)
        {
            const T* qp = qkv_b + (size_t) (head0 + hl) * DH + t * QV;
#pragma unroll
            for (int i = 0; i < QV; i += 8)
            {
                const uint4 raw = *reinterpret_cast<const uint4*>(qp + i);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const float2 v = TypeOps<T>::unpack2(w[j]);
                    qv[i + 2 * j] = v.x;
                    qv[i + 2 * j + 1] = v.y;
                }
            }
        }
        else
        {
#pragma unroll
            for (int i = 0; i < QV; ++i)
                qv[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < QV; ++i)
            amax = fmaxf(amax, fabsf(qv[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        float qmul, qinv;
        if constexpr (IS_FP8)
        {
            // power-of-two scale that puts amax into [128, 256)
            int e = 0;
            if (amax > 0.f)
                e = 7 - (int) (((__float_as_uint(amax) >> 23) & 0xff) - 127);
            e = max(-100, min(100, e));
            qmul = __uint_as_float((uint32_t) (e + 127) << 23);
            qinv = __uint_as_float((uint32_t) (127 - e) << 23);
        }
        else
        {
            const float qs = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
            qmul = 1.f / qs;
            qinv = qs * (1.f / kLoWeight);
        }
        sfac[r] = qinv * deq * a.softmax_scale_log2;
#pragma unroll
        for (int s = 0; s < KS; ++s)
        {
#pragma unroll
            for (int half = 0; half < 2; ++half)
            {
                // elements of this thread that feed a0/a1 (half 0) or a2/a3 (half 1) of k-step s
                const int base = (DH == 128) ? (16 * half + 4 * s) : (8 * s + 4 * half);
                uint32_t whi = 0, wlo = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                {
                    uint32_t hi, lo;
                    split_hi_lo<CACHE>(qv[base + i] * qmul, hi, lo);
                    whi |= hi << (8 * i);
                    wlo |= lo << (8 * i);
                }
                qa[0][s][2 * half + r] = (r < NR) ? whi : 0u;
                qa[1][s][2 * half + r] = (r < NR) ? wlo : 0u;
            }
        }
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float of[MT][NR][4]; // O^T fragments: [m-tile][head half][c0..c3]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                of[mt][r][c] = 0.f;

    bool timed_out = false;
    for (int i = 0; i < my_groups; ++i)
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
        if (new_pos >= t0 && new_pos < t0 + TG)
        {
            // The group ends with the new token: quantise it exactly as it is stored, put it into
            // the staged tile (rows behind it were zero-filled by the copies) and, from the first
            // head slice only, append it to the paged cache.
            const int r_new = new_pos - t0;
            const float sc_f = __ldg(a.scale_orig_quant);
            const T sc_t = TypeOps<T>::from_float(sc_f);
            if (lane < DH / 16)
            {
                const T* kp = qkv_b + (size_t) (a.num_heads + hk) * DH + lane * 16;
                const T* vp = qkv_b + (size_t) (a.num_heads + a.num_kv_heads + hk) * DH + lane * 16;
                const uint4 kq = make_cache_vec<T, CACHE, 16>(kp, sc_f, sc_t);
                const uint4 vq = make_cache_vec<T, CACHE, 16>(vp, sc_f, sc_t);
                const uint32_t lin = (uint32_t) r_new * DH + lane * 16;
                *reinterpret_cast<uint4*>(kbuf + swz<DH>(lin)) = kq;
                *reinterpret_cast<uint4*>(vbuf + swz<DH>(lin)) = vq;
                if (hg == 0)
                {
                    const size_t off = head_off + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                    char* kb = reinterpret_cast<char*>(__ldg(krow + (new_pos >> tpb_log2))) + off;
                    char* vb = reinterpret_cast<char*>(__ldg(vrow + (new_pos >> tpb_log2))) + off;
                    *reinterpret_cast<uint4*>(kb) = kq;
                    *reinterpret_cast<uint4*>(vb) = vq;
                }
            }
            __syncwarp();
        }

        // ---- S = Q K^T for 16 head rows x 32 tokens ----
        Acc sacc[2][4][4]; // [hi/lo (int8 only)][n-tile][c0..c3]
#pragma unroll
        for (int x = 0; x < 2; ++x)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    sacc[x][nt][c] = 0;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
        {
            const uint32_t off = (uint32_t) sigma_row<DH>(nt, g) * DH + t * (DH / 4);
            uint32_t kw[2 * KS];
            {
                const uint4 v0 = *reinterpret_cast<const uint4*>(kbuf + swz<DH>(off));
                kw[0] = v0.x, kw[1] = v0.y, kw[2] = v0.z, kw[3] = v0.w;
                if constexpr (DH == 128)
                {
                    const uint4 v1 = *reinterpret_cast<const uint4*>(kbuf + swz<DH>(off + 16));
                    kw[4] = v1.x, kw[5] = v1.y, kw[6] = v1.z, kw[7] = v1.w;
                }
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
            {
                const uint32_t b0 = (DH == 128) ? kw[ks] : kw[2 * ks];
                const uint32_t b1 = (DH == 128) ? kw[4 + ks] : kw[2 * ks + 1];
                if constexpr (IS_FP8)
                {
                    mma_e4m3(sacc[0][nt], qa[0][ks], b0, b1);
                    mma_e4m3(sacc[0][nt], qa[1][ks], b0, b1);
                }
                else
                {
                    mma_s8(sacc[0][nt], qa[0][ks], b0, b1);
                    mma_s8(sacc[1][nt], qa[1][ks], b0, b1);
                }
            }
        }

        // ---- online softmax over the 32 tokens (rows g and g + 8) ----
        float p[4][4];
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
        {
#pragma unroll
            for (int c = 0; c < 2 * NR; ++c)
            {
                const int tok = t0 + sigma_row<DH>(nt, 2 * t + (c & 1));
                float sv;
                if constexpr (IS_FP8)
                    sv = sacc[0][nt][c];
                else
                    sv = (float) (sacc[0][nt][c] * kLoWeight + sacc[1][nt][c]);
                sv = (tok < total) ? sv * sfac[c >> 1] : -INFINITY;
                p[nt][c] = sv;
                mx[c >> 1] = fmaxf(mx[c >> 1], sv);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m[r], mx[r]);
            alpha[r] = fast_exp2(m[r] - m_new);
            m[r] = m_new;
            l[r] *= alpha[r];
        }
        constexpr float PSCALE = IS_FP8 ? 256.f : 127.f;
        uint32_t pb[NR][2][2]; // [head half][hi/lo][b0/b1]
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
#pragma unroll
            for (int kh = 0; kh < 2; ++kh)
            {
                uint32_t whi = 0, wlo = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                {
                    const int nt = 2 * kh + (i >> 1);
                    const float pv = fast_exp2(p[nt][2 * r + (i & 1)] - m[r]);
                    l[r] += pv;
                    uint32_t hi, lo;
                    split_hi_lo<CACHE>(pv * PSCALE, hi, lo);
                    whi |= hi << (8 * i);
                    wlo |= lo << (8 * i);
                }
                pb[r][0][kh] = whi;
                pb[r][1][kh] = wlo;
            }
        }

        // ---- rescale the running O^T (its columns are heads 2t, 2t+1 (+8)) ----
        float ac[NR][2];
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
            ac[r][0] = __shfl_sync(0xffffffffu, alpha[r], 8 * t);
            ac[r][1] = __shfl_sync(0xffffffffu, alpha[r], 8 * t + 4);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int r = 0; r < NR; ++r)
            {
                of[mt][r][0] *= ac[r][0];
                of[mt][r][1] *= ac[r][1];
                of[mt][r][2] *= ac[r][0];
                of[mt][r][3] *= ac[r][1];
            }

        // ---- O^T += V^T P^T ----
        uint32_t tr[2][NW][4]; // [k half][word][byte column] -> one A register each
        {
            uint32_t rv[8][NW];
#pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                const int row = sigma_row<DH>(i >> 1, 2 * t + (i & 1));
                if constexpr (DH == 128)
                {
                    const uint4 v = *reinterpret_cast<const uint4*>(vbuf + swz<DH>((uint32_t) row * DH + g * 16));
                    rv[i][0] = v.x, rv[i][1] = v.y, rv[i][2] = v.z, rv[i][3] = v.w;
                }
                else
                {
                    const uint2 v = *reinterpret_cast<const uint2*>(vbuf + swz<DH>((uint32_t) row * DH + g * 8));
                    rv[i][0] = v.x, rv[i][1] = v.y;
                }
            }
#pragma unroll
            for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                for (int w = 0; w < NW; ++w)
                    transpose4x4(rv[4 * kh][w], rv[4 * kh + 1][w], rv[4 * kh + 2][w], rv[4 * kh + 3][w], tr[kh][w]);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
            const int w = mt >> 1, bc = 2 * (mt & 1);
            const uint32_t av[4] = {tr[0][w][bc], tr[0][w][bc + 1], tr[1][w][bc], tr[1][w][bc + 1]};
#pragma unroll
            for (int r = 0; r < NR; ++r)
            {
                if constexpr (IS_FP8)
                {
                    mma_e4m3(of[mt][r], av, pb[r][0][0], pb[r][0][1]);
                    mma_e4m3(of[mt][r], av, pb[r][1][0], pb[r][1][1]);
                }
                else
                {
                    int ohi[4] = {0, 0, 0, 0}, olo[4] = {0, 0, 0, 0};
                    mma_s8(ohi, av, pb[r][0][0], pb[r][0][1]);
                    mma_s8(olo, av, pb[r][1][0], pb[r][1][1]);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        of[mt][r][c] += (float) (ohi[c] * kLoWeight + olo[c]);
                }
            }
        }

        __syncwarp(); // every lane is done reading this stage
        if (i + STAGES < my_groups)
            issue(i + STAGES);
    }

    if (timed_out && lane == 0)
        atomicExch(a.status, STATUS_TIMEOUT);

    // ---- per-warp results -> shared memory, then combine the 4 warps ----
#pragma unroll
    for (int r = 0; r < NR; ++r)
    {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    __syncthreads(); // all warps have drained their rings; the ring memory is reused below
    float* mo = reinterpret_cast<float*>(smem) + warp * (16 * DH + 32);
    float* mm = mo + 16 * DH; // m[16], then l[16]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c)
            {
                const int head = 8 * r + 2 * t + (c & 1);
                const int dh = (DH / 8) * g + 2 * mt + (c >> 1);
                mo[head * DH + dh] = of[mt][r][c];
            }
    if (t == 0)
    {
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
            mm[8 * r + g] = m[r];
            mm[16 + 8 * r + g] = l[r];
        }
    }
    __syncthreads();

    constexpr float ONORM = IS_FP8 ? (1.f / 256.f) : (1.f / (127.f * kLoWeight));
    const float ofac = deq * ONORM;
    const float* base = reinterpret_cast<const float*>(smem);
    for (int idx = threadIdx.x; idx < nh * DH; idx += blockDim.x)
    {
        const int head = idx / DH, dh = idx % DH;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w)
            M = fmaxf(M, base[w * (16 * DH + 32) + 16 * DH + head]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w)
        {
            const float* wb = base + w * (16 * DH + 32);
            const float mw = wb[16 * DH + head];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L = fmaf(wb[16 * DH + 16 + head], f, L);
            o = fmaf(wb[head * DH + dh], f, o);
        }
        const size_t row = (size_t) b * a.num_heads + head0 + head;
        if (a.nsplit == 1)
        {
            reinterpret_cast<T*>(a.out)[row * DH + dh] = TypeOps<T>::from_float(o * ofac / L);
        }
        else
        {
            a.part_o[(row * a.nsplit + chunk) * DH + dh] = o * ofac;
            if (dh == 0)
                a.part_ml[row * a.nsplit + chunk] = make_float2(M, L);
        }
    }
}

} // namespace dx
