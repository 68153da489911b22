// Wide-group (MQA / large GQA) decode attention over an FP8 paged KV cache on the 5th-generation
// tensor cores: tcgen05.mma with shared-memory operand descriptors and TMEM accumulators.
//
// One CTA of 128 threads per (split-K partition, kv head x 128-head slice of its q group, sequence).
// The q heads that share the kv head are the M = 128 rows of both MMAs, so a thread owns one head
// row end to end (TMEM lane = head) and the online softmax needs no cross-thread reduction:
//   S[128 x 64]  = Q[128 x Dh] K^T   tcgen05.mma.kind::f8f6f4, A = Q (smem, K-major), B = K tile (smem, K-major)
//   P            = 2^(S - m) per row, written back to smem as e4m3 high + low parts (K-major A operand)
//   O[128 x Dh]  = P[128 x 64] V     A = P, B = V tile used as stored ([token][Dh], MN-major)
// Cache bytes are consumed by the tensor core exactly as stored: no conversion, no transpose.  Q and P
// are split into a high and a low e4m3 part (two MMAs into the same accumulator).
// K / V tiles of 64 tokens arrive through a ring of 16-byte cp.async copies laid out in the hardware's
// 64-byte / 128-byte swizzle, tracked by mbarriers; MMA completion is tracked with tcgen05.commit on
// mbarriers.  Every wait is bounded; TMEM is freed on every path.
//
// Replaces, for G > 16 with an FP8 cache (Falcon-style 71:1 MQA), what the reference would run as one
// MMHA CTA per q head (decoderMaskedMultiheadAttentionTemplate.h:1303) - XQA has no kernel for it
// (decoderXQARunner.h:87-159 admits only 8 q heads per kv head).
#pragma once

#include "dx_common.cuh"
#include "dx_gqa_kernel.cuh" // split4, cp_async16_*_u32
#include "dx_mha_kernel.cuh" // make_cache_vec

namespace dx
{

template <int DH>
struct WideTraits
{
    static constexpr int TT = 64;                    // tokens per tile
    static constexpr int STAGES = 3;
    static constexpr int KV_TILE = TT * DH;          // bytes of K (or V) per tile
    static constexpr int STAGE_BYTES = 2 * KV_TILE;
    static constexpr int Q_TILE = 128 * DH;          // bytes of the high (or low) part of Q
    static constexpr int P_TILE = 128 * TT;          // bytes of the high (or low) part of P
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;
    static constexpr int OFF_RING = OFF_P + 2 * P_TILE;
    static constexpr int OFF_BAR = OFF_RING + STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 64 + 1024; // + barriers / tmem pointer + alignment slack
    static constexpr int TMEM_COLS = (DH == 64) ? 128 : 256; // S: 64 columns, O: Dh columns (power of two)
    static constexpr uint32_t SWZ_LAYOUT = (DH == 64) ? 4u : 2u; // UMMA layout type: SWIZZLE_64B / SWIZZLE_128B
};

// Hardware swizzle of a row-major tile with `PITCH`-byte rows (64 -> SWIZZLE_64B, 128 -> SWIZZLE_128B).
template <int PITCH>
__device__ __forceinline__ uint32_t hw_swz(uint32_t off)
{
    if constexpr (PITCH == 64)
        return off ^ (((off >> 7) & 3u) << 4);
    else
        return off ^ (((off >> 7) & 7u) << 4);
}

// Shared-memory matrix descriptor (version 1).  lbo / sbo in bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout)
{
    uint64_t d = 0;
    d |= (uint64_t) ((saddr >> 4) & 0x3fffu);
    d |= (uint64_t) ((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t) ((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) (layout & 7u) << 61;
    return d;
}

// D[tmem] (+)= A[smem] * B[smem], e4m3 x e4m3 -> f32, issued by one thread.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t zero = 0;
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 columns of fp32 from TMEM into registers (one row per thread).
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32])
{
    uint32_t r[32];
    __syncwarp(); // .sync.aligned: the warp must be converged (lane 0 may come from the MMA issue branch)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i)
        v[i] = __uint_as_float(r[i]);
}

template <typename T, int DH>
__global__ void __launch_bounds__(128) wide_decode_kernel(const AttnArgs a, const int hgroups)
{
    using Tr = WideTraits<DH>;
    constexpr int TT = Tr::TT, STAGES = Tr::STAGES, KV_TILE = Tr::KV_TILE;
    constexpr uint32_t LAY = Tr::SWZ_LAYOUT;
    constexpr uint32_t SBO_KV = 8 * DH;  // 8 rows of a Dh-byte-pitch tile
    constexpr uint32_t SBO_P = 8 * TT;   // 8 rows of the 64-byte-pitch P tile
    constexpr int CACHE = CACHE_FP8;

    const int chunk = blockIdx.x;
    const int hk = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
    const int b = blockIdx.z;
    const int total = a.seq_len[b];
    int chunk_start, ctoks, nparts;
    partition_of(total, a.chunk_tokens, chunk, chunk_start, ctoks, nparts);
    if (chunk >= nparts)
        return;
    griddep_launch_dependents();
    const int n_tiles = (ctoks + TT - 1) / TT;
    const int new_pos = total - 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.num_heads / a.num_kv_heads;
    const int nh = min(128, G - hg * 128);
    const int head0 = hk * G + hg * 128;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    // descriptors assume tiles aligned to the swizzle period: align the whole layout to 1 KB
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR); // full[STAGES], s_done, o_done
    uint64_t* bar_s = bars + STAGES;
    uint64_t* bar_o = bars + STAGES + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + STAGES + 2);

    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(Tr::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0)
    {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            mbar_init(&bars[s], 128);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        fence_mbar_init();
    }

    const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
    const int64_t* vrow = krow + a.max_blocks_per_seq;
    const size_t head_off = (size_t) hk * ((size_t) DH << tpb_log2);

    // Every thread copies its share of tile i (64 tokens of K and of V) into ring stage i % STAGES.
    auto issue = [&](int i)
    {
        const int t0 = chunk_start + i * TT;
        const int rows = new_pos - t0; // rows already in the cache
        const uint32_t kdst = s_base + Tr::OFF_RING + (i % STAGES) * Tr::STAGE_BYTES;
        const size_t off = head_off + (size_t) (t0 & tpb_mask) * DH;
        const char* kb = reinterpret_cast<const char*>(__ldg(krow + (t0 >> tpb_log2))) + off;
        const char* vb = reinterpret_cast<const char*>(__ldg(vrow + (t0 >> tpb_log2))) + off;
        const int valid_bytes = rows >= TT ? KV_TILE : (rows > 0 ? rows * DH : 0);
#pragma unroll
        for (int j = 0; j < KV_TILE / (128 * 16); ++j)
        {
            const uint32_t lin = (uint32_t) (tid + 128 * j) * 16;
            const bool ok = (int) lin < valid_bytes;
            const uint32_t d = hw_swz<DH>(lin);
            cp_async16_zfill_u32(kdst + d, ok ? kb + lin : kb, ok ? 16u : 0u);
            cp_async16_zfill_u32(kdst + KV_TILE + d, ok ? vb + lin : vb, ok ? 16u : 0u);
        }
        cp_async_mbar_arrive_noinc(&bars[i % STAGES]);
    };
    __syncthreads(); // barriers initialised, TMEM address published
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;      // S: columns [0, 64)
    const uint32_t tmem_o = tmem_base + TT; // O: columns [64, 64 + Dh)
    const uint32_t lane_sel = (uint32_t) (warp * 32) << 16;

    for (int i = 0; i < min(STAGES, n_tiles); ++i)
        issue(i);

    // ---- Q: thread = head row.  Scale the row into the e4m3 range, split high / low, store both
    // parts as K-major rows of the swizzled Q tiles ----
    const float deq = __ldg(a.scale_quant_orig);
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
    float sfac;
    {
        float qv[DH];
        if (tid < nh)
        {
            const T* qp = qkv_b + (size_t) (head0 + tid) * DH;
#pragma unroll
            for (int i = 0; i < DH; i += 8)
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
            for (int i = 0; i < DH; ++i)
                qv[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < DH; ++i)
            amax = fmaxf(amax, fabsf(qv[i]));
        int e = 0;
        if (amax > 0.f)
            e = 7 - (int) (((__float_as_uint(amax) >> 23) & 0xff) - 127);
        e = max(-100, min(100, e));
        const float qmul = __uint_as_float((uint32_t) (e + 127) << 23);
        const float qinv = __uint_as_float((uint32_t) (127 - e) << 23);
        sfac = qinv * deq * a.softmax_scale_log2;
#pragma unroll
        for (int c = 0; c < DH / 16; ++c)
        {
            uint4 hi, lo;
            split4<CACHE>(qv[16 * c] * qmul, qv[16 * c + 1] * qmul, qv[16 * c + 2] * qmul, qv[16 * c + 3] * qmul, hi.x, lo.x);
            split4<CACHE>(qv[16 * c + 4] * qmul, qv[16 * c + 5] * qmul, qv[16 * c + 6] * qmul, qv[16 * c + 7] * qmul, hi.y, lo.y);
            split4<CACHE>(qv[16 * c + 8] * qmul, qv[16 * c + 9] * qmul, qv[16 * c + 10] * qmul, qv[16 * c + 11] * qmul, hi.z, lo.z);
            split4<CACHE>(qv[16 * c + 12] * qmul, qv[16 * c + 13] * qmul, qv[16 * c + 14] * qmul, qv[16 * c + 15] * qmul, hi.w, lo.w);
            const uint32_t d = hw_swz<DH>((uint32_t) tid * DH + c * 16);
            *reinterpret_cast<uint4*>(smem + Tr::OFF_Q + d) = hi;
            *reinterpret_cast<uint4*>(smem + Tr::OFF_Q + Tr::Q_TILE + d) = lo;
        }
    }

    // Warps whose 32 head rows are all padding take part in the barriers only; their P rows stay zero.
    const bool warp_active = warp * 32 < nh;
    if (!warp_active)
    {
#pragma unroll
        for (int c = 0; c < TT / 16; ++c)
        {
            *reinterpret_cast<uint4*>(smem + Tr::OFF_P + tid * TT + c * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(smem + Tr::OFF_P + Tr::P_TILE + tid * TT + c * 16) = make_uint4(0, 0, 0, 0);
        }
    }

    // instruction descriptors: f32 accumulate, e4m3 x e4m3, M = 128
    constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (TT >> 3) << 17) | ((128u >> 4) << 24);            // N = 64, B K-major
    constexpr uint32_t IDESC_O = (1u << 4) | (1u << 16) | ((uint32_t) (DH >> 3) << 17) | ((128u >> 4) << 24); // N = Dh, B MN-major

    float m = -INFINITY, l = 0.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i)
        o[i] = 0.f;

    int fail = 0;
    for (int i = 0; i < n_tiles; ++i)
    {
        const int s = i % STAGES;
        const uint32_t kbuf = s_base + Tr::OFF_RING + s * Tr::STAGE_BYTES;
        const uint32_t vbuf = kbuf + KV_TILE;
        fail |= !mbar_wait_bounded(&bars[s], (i / STAGES) & 1, a.status);
        const int t0 = chunk_start + i * TT;
        const int lim = total - t0; // valid tokens in this tile if < TT
        if (new_pos < t0 + TT && warp == 0)
        {
            // the tile ends with the new token: quantise it as it is stored, place it in the staged tile
            // (rows behind it were zero-filled by the copies) and, from the first head slice, append it
            const int r_new = new_pos - t0;
            const float sc_f = __ldg(a.scale_orig_quant);
            const T sc_t = TypeOps<T>::from_float(sc_f);
            if (lane < DH / 16)
            {
                const T* kp = qkv_b + (size_t) (a.num_heads + hk) * DH + lane * 16;
                const T* vp = qkv_b + (size_t) (a.num_heads + a.num_kv_heads + hk) * DH + lane * 16;
                const uint4 kq = make_cache_vec<T, CACHE, 16>(kp, sc_f, sc_t);
                const uint4 vq = make_cache_vec<T, CACHE, 16>(vp, sc_f, sc_t);
                const uint32_t d = hw_swz<DH>((uint32_t) r_new * DH + lane * 16);
                unsigned char* stage = smem + Tr::OFF_RING + s * Tr::STAGE_BYTES;
                *reinterpret_cast<uint4*>(stage + d) = kq;
                *reinterpret_cast<uint4*>(stage + KV_TILE + d) = vq;
                if (hg == 0)
                {
                    const size_t off = head_off + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                    char* kb = reinterpret_cast<char*>(__ldg(krow + (new_pos >> tpb_log2))) + off;
                    char* vb = reinterpret_cast<char*>(__ldg(vrow + (new_pos >> tpb_log2))) + off;
                    *reinterpret_cast<uint4*>(kb) = kq;
                    *reinterpret_cast<uint4*>(vb) = vq;
                }
            }
        }
        // generic-proxy writes (cp.async, the Q / new-token stores) -> visible to the tensor core
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        fail = __syncthreads_or(fail);
        if (fail)
            break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- S = (Q_hi + Q_lo) K^T ----
        if (tid == 0)
        {
#pragma unroll
            for (int part = 0; part < 2; ++part)
#pragma unroll
                for (int ks = 0; ks < DH / 32; ++ks)
                {
                    const uint64_t da = umma_desc(s_base + Tr::OFF_Q + part * Tr::Q_TILE + ks * 32, 16, SBO_KV, LAY);
                    const uint64_t db = umma_desc(kbuf + ks * 32, 16, SBO_KV, LAY);
                    umma_f8(tmem_s, da, db, IDESC_S, (part | ks) != 0);
                }
            umma_commit(bar_s);
        }
        fail |= !mbar_wait_bounded(bar_s, i & 1, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- online softmax of this thread's head row over the 64 tokens ----
        float alpha = 1.f;
        if (warp_active)
        {
            float sv[TT];
            {
                float h0[32], h1[32];
                tmem_ld32(tmem_s + lane_sel, h0);
                tmem_ld32(tmem_s + lane_sel + 32, h1);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                {
                    sv[j] = h0[j] * sfac;
                    sv[32 + j] = h1[j] * sfac;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < TT; ++j)
            {
                if (j >= lim)
                    sv[j] = -INFINITY;
                mx = fmaxf(mx, sv[j]);
            }
            const float m_new = fmaxf(m, mx);
            alpha = fast_exp2(m - m_new);
            m = m_new;
            l *= alpha;
#pragma unroll
            for (int c = 0; c < TT / 16; ++c)
            {
                float pv[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                {
                    pv[j] = fast_exp2(sv[16 * c + j] - m_new);
                    l += pv[j];
                    pv[j] *= 256.f;
                }
                uint4 hi, lo;
                split4<CACHE>(pv[0], pv[1], pv[2], pv[3], hi.x, lo.x);
                split4<CACHE>(pv[4], pv[5], pv[6], pv[7], hi.y, lo.y);
                split4<CACHE>(pv[8], pv[9], pv[10], pv[11], hi.z, lo.z);
                split4<CACHE>(pv[12], pv[13], pv[14], pv[15], hi.w, lo.w);
                const uint32_t d = hw_swz<TT>((uint32_t) tid * TT + c * 16);
                *reinterpret_cast<uint4*>(smem + Tr::OFF_P + d) = hi;
                *reinterpret_cast<uint4*>(smem + Tr::OFF_P + Tr::P_TILE + d) = lo;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        fail = __syncthreads_or(fail);
        if (fail)
            break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- O_tile = (P_hi + P_lo) V ----
        if (tid == 0)
        {
#pragma unroll
            for (int part = 0; part < 2; ++part)
#pragma unroll
                for (int ks = 0; ks < TT / 32; ++ks)
                {
                    const uint64_t da = umma_desc(s_base + Tr::OFF_P + part * Tr::P_TILE + ks * 32, 16, SBO_P, 4u);
                    const uint64_t db = umma_desc(vbuf + ks * 32 * DH, 16, SBO_KV, LAY);
                    umma_f8(tmem_o, da, db, IDESC_O, (part | ks) != 0);
                }
            umma_commit(bar_o);
        }
        fail |= !mbar_wait_bounded(bar_o, i & 1, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (warp_active)
        {
#pragma unroll
            for (int c = 0; c < DH / 32; ++c)
            {
                float ot[32];
                tmem_ld32(tmem_o + lane_sel + 32 * c, ot);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    o[32 * c + j] = fmaf(o[32 * c + j], alpha, ot[j]);
            }
        }
        // the stage and both accumulators are free again: refill the stage
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        fail = __syncthreads_or(fail);
        if (fail)
            break;
        if (i + STAGES < n_tiles)
            issue(i + STAGES);
    }

    if (fail && tid == 0)
        atomicExch(a.status, STATUS_TIMEOUT);

    // ---- result of this partition: thread = head row ----
    if (!fail && tid < nh)
    {
        const float ofac = deq * (1.f / 256.f);
        const size_t row = (size_t) b * a.num_heads + head0 + tid;
        if (a.nsplit == 1)
        {
            const float inv = ofac / l;
            T* dst = reinterpret_cast<T*>(a.out) + row * DH;
#pragma unroll
            for (int i = 0; i < DH; i += 8)
            {
                uint4 w;
                w.x = TypeOps<T>::pack2(o[i] * inv, o[i + 1] * inv);
                w.y = TypeOps<T>::pack2(o[i + 2] * inv, o[i + 3] * inv);
                w.z = TypeOps<T>::pack2(o[i + 4] * inv, o[i + 5] * inv);
                w.w = TypeOps<T>::pack2(o[i + 6] * inv, o[i + 7] * inv);
                *reinterpret_cast<uint4*>(dst + i) = w;
            }
        }
        else
        {
            float* dst = a.part_o + (row * a.nsplit + chunk) * DH;
#pragma unroll
            for (int i = 0; i < DH; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(o[i] * ofac, o[i + 1] * ofac, o[i + 2] * ofac, o[i + 3] * ofac);
            a.part_ml[row * a.nsplit + chunk] = make_float2(m, l);
        }
    }

    // ---- free TMEM (every path reaches this) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Tr::TMEM_COLS));
}

} // namespace dx
