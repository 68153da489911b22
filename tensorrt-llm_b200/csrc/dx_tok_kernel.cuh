// Grouped-head decode attention over an FP8 paged KV cache on the 5th-generation tensor cores, token-major:
// the 128 tokens of a tile are the M rows of the first MMA, the (few) q heads of the group are its N columns.
//
//   S^T[128 tok x N]  = K_tile[128 tok x Dh] Qx^T      A = K tile as stored (K-major), B = Qx (K-major)
//   O^T[Dh x N]      += V_tile^T[Dh x 128 tok] Px      A = V tile as stored ([token][Dh] = MN-major), B = Px (MN-major)
//
// N = 2 * GP columns: GP (8 or 16) padded heads, high e4m3 parts in columns [0, GP), low parts (times 16) in
// [GP, 2 GP); the two halves are added when the accumulators are read.  Cache bytes reach the tensor core exactly as
// stored.  O^T stays in tensor memory for the whole partition (thread = Dh channel at the end); a thread owns one
// token row of S^T, so the probabilities need no shuffles at all.  The softmax reference m is lazy: it only moves
// when some score exceeds it by more than 2^THR (checked CTA-wide with the barrier that publishes P anyway); then
// the block maximum is taken, O^T is rescaled in tensor memory, and the tile's P is recomputed.  The first tile
// always takes that path (m = -inf).
//
// One CTA of 128 threads per (split-K partition, kv head, sequence); Dh = 128.  Replaces what the reference runs as
// XQA (decoderXQAImplPrecompiled.cpp:223-374) or as one MMHA CTA per q head
// (decoderMaskedMultiheadAttentionTemplate.h:1303) for grouped heads with an FP8 cache.
#pragma once

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh"  // make_cache_vec

#ifndef DX_TOK_STAGES
#define DX_TOK_STAGES 2
#endif
#include "dx_tcgen05.cuh"


namespace dx
{

template <int GP>
struct TokTraits
{
    static constexpr int DH = 128, TT = 128, N = 2 * GP;
    static constexpr int NST = DX_TOK_STAGES; // ring stages for K and for V
    static constexpr int KV_TILE = TT * DH; // bytes of a K (or V) tile
    static constexpr int Q_TILE = N * DH;
    static constexpr int P_TILE = TT * N;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_P = OFF_Q + Q_TILE;     // two buffers
    static constexpr int OFF_K = OFF_P + 2 * P_TILE; // NST stages (multiple of 1 KB: swizzle period)
    static constexpr int OFF_V = OFF_K + NST * KV_TILE;
    static constexpr int OFF_RED = OFF_V + NST * KV_TILE; // float red[4][GP], sfac[GP]
    static constexpr int OFF_BAR = OFF_RED + 5 * GP * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024; // barriers, tmem slot, alignment slack
    static constexpr int TMEM_COLS = 128;                  // S: 2 x 32 columns, O: 32 columns
    static constexpr int MIN_BLOCKS = (227 * 1024) / (SMEM_BYTES + 1024);
    static_assert(OFF_K % 1024 == 0, "tiles must sit on the swizzle period");
};

// Four values (already scaled into the e4m3 range) -> a word of high parts and a word of low parts,
// the low parts being 16 x the residual (so that small residuals stay above the e4m3 subnormal floor).
__device__ __forceinline__ void split4_lo16(float x0, float x1, float x2, float x3, uint32_t& hi, uint32_t& lo)
{
    uint16_t h01, h23, l01, l23;
    uint32_t f01, f23, x01, x23;
    const uint32_t k16 = 0x4C004C00u; // 16.0 in both halves
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h01) : "f"(x1), "f"(x0));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h23) : "f"(x3), "f"(x2));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(f01) : "h"(h01));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(f23) : "h"(h23));
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(x01) : "f"(x1), "f"(x0));
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(x23) : "f"(x3), "f"(x2));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(x01) : "r"(x01), "r"(f01));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(x23) : "r"(x23), "r"(f23));
    asm("mul.f16x2 %0, %1, %2;" : "=r"(x01) : "r"(x01), "r"(k16));
    asm("mul.f16x2 %0, %1, %2;" : "=r"(x23) : "r"(x23), "r"(k16));
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(l01) : "r"(x01));
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(l23) : "r"(x23));
    hi = (uint32_t) h01 | ((uint32_t) h23 << 16);
    lo = (uint32_t) l01 | ((uint32_t) l23 << 16);
}

template <typename T, int GP>
__global__ void __launch_bounds__(128, TokTraits<GP>::MIN_BLOCKS)
    tok_decode_kernel(const AttnArgs a, const int hgroups_unused, const __grid_constant__ SkSchedule sk)
{
    using Tr = TokTraits<GP>;
    constexpr int DH = Tr::DH, TT = Tr::TT, N = Tr::N, KV_TILE = Tr::KV_TILE, P_TILE = Tr::P_TILE, NST = Tr::NST;
    constexpr int CACHE = CACHE_FP8;
    constexpr float LOW = 1.f / 16.f; // weight of the low-part columns
    // The probabilities are kept as p = 2^(s - m) with m = (lazy reference maximum) - 4, so that they go into
    // e4m3 without a further scale: p <= 2^PMAX = 256 while no score exceeds the reference by more than 2^4.
    constexpr float PMAX = 8.f;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.num_heads / a.num_kv_heads;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    // Work of this CTA.  Classic launch: one piece, the (partition, kv head, sequence) of its grid position.
    // Stream-K launch (a.streamk): a contiguous range of 128-token tiles of the whole batch (SkSchedule), i.e. a
    // few pieces of consecutive rows, every CTA the same amount.
    SkCursor cur;
    if (a.streamk)
    {
        if (!sk_begin(sk, (int) blockIdx.x, cur))
            return;
    }
    else
    {
        int cs, ct, np;
        partition_of(a.seq_len[blockIdx.z], a.chunk_tokens, (int) blockIdx.x, cs, ct, np);
        if (np > (int) gridDim.x && blockIdx.x == 0 && threadIdx.x == 0)
            report_status(a.status, STATUS_PLAN_EXCEEDED); // the tokens beyond the last partition are not attended to
        if ((int) blockIdx.x >= np)
            return;
    }
    griddep_launch_dependents();

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    float* red = reinterpret_cast<float*>(smem + Tr::OFF_RED); // [4][GP]
    float* sfac_s = red + 4 * GP;                               // [GP]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    uint64_t* full = bars;              // [NST]: V(j) and K(j+1) have landed
    uint64_t* full_k0 = bars + NST;     // K(0) of a piece has landed
    uint64_t* bar_mma = bars + NST + 1; // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NST + 3);
    uint64_t* bar_drain = bars + NST + 4; // only used after a time-out: the MMAs issued so far have completed

    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(Tr::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0)
    {
#pragma unroll
        for (int s = 0; s < NST; ++s)
            mbar_init(&full[s], 128);
        mbar_init(full_k0, 128);
        mbar_init(&bar_mma[0], 1);
        mbar_init(&bar_mma[1], 1);
        mbar_init(bar_drain, 1);
        fence_mbar_init();
    }
    __syncthreads(); // barriers initialised, TMEM address published
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 64;
    const uint32_t lane_sel = (uint32_t) (warp * 32) << 16;

    constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (N >> 3) << 17) | ((128u >> 4) << 24); // A, B K-major
    constexpr uint32_t IDESC_O = IDESC_S | (1u << 15) | (1u << 16);                             // A, B MN-major
    // Operand descriptors: only the start-address field (16-byte units, low bits of the low word) changes
    // between stages and k-steps, so the bases are built once.
    const uint64_t desc_k = umma_desc(s_base + Tr::OFF_K, 16, 1024, 2u);
    const uint64_t desc_q = umma_desc(s_base + Tr::OFF_Q, 16, 1024, 2u);
    const uint64_t desc_v = umma_desc(s_base + Tr::OFF_V, 16, 1024, 2u);
    const uint64_t desc_p = umma_desc(s_base + Tr::OFF_P, 128, TT * 16, 0u);

    const float deq = __ldg(a.scale_quant_orig);
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const int col = tid & 7, r0 = tid >> 3;
    const uint32_t dst_thread = hw_swz<128>((uint32_t) r0 * 128 + col * 16);

    // Ring / barrier bookkeeping that runs on across the pieces of a stream-K range: tiles (= pairs) and MMA
    // groups put through so far, pieces started.
    int tbase = 0, cbase = 0, npiece = 0;
    int fail = 0;
    for (;;)
    {
        // ---- this piece: row (b, hk), tokens [chunk_start, chunk_start + ctoks), result slot `chunk` ----
        int b, hk, chunk, chunk_start, ctoks;
        bool final_out;
        if (a.streamk)
        {
            int g0, ng;
            sk_piece(sk, cur, b, hk, g0, ng, chunk, final_out);
            chunk_start = g0 * TT;
            ctoks = ng * TT;
        }
        else
        {
            int np;
            chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
            partition_of(a.seq_len[b], a.chunk_tokens, chunk, chunk_start, ctoks, np);
            final_out = a.nsplit == 1;
        }
        const int total = a.seq_len[b];
        if (a.streamk && total > (int) cur.nb * TT && threadIdx.x == 0)
            report_status(a.status, STATUS_PLAN_EXCEEDED); // longer than the host length the ranges were laid out for
        ctoks = max(0, min(ctoks, total - chunk_start)); // the schedule counts host lengths; the device length decides
        const int n_tiles = (ctoks + TT - 1) / TT;
        const int new_pos = total - 1;
        const int head0 = hk * G;
        const int new_tile = (new_pos >= chunk_start && new_pos < chunk_start + ctoks) ? (new_pos - chunk_start) / TT : -1;
        const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
        const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
        const int64_t* vrow = krow + a.max_blocks_per_seq;
        const size_t head_off = (size_t) hk * ((size_t) DH << tpb_log2);
        const size_t src_thread = head_off + (size_t) r0 * DH + col * 16;

        float mref[GP], l[GP]; // mref: the m above
#pragma unroll
        for (int h = 0; h < GP; ++h)
        {
            mref[h] = -INFINITY;
            l[h] = 0.f;
        }

        if (n_tiles > 0)
        {
            // this warp's q rows first (warp w prepares heads w, w + 4, ...): their latency overlaps the rest
            uint2 q_raw[GP / 4];
#pragma unroll
            for (int c = 0; c < GP / 4; ++c)
            {
                const int hh = warp + 4 * c;
                q_raw[c] = (hh < G) ? *reinterpret_cast<const uint2*>(qkv_b + (size_t) (head0 + hh) * DH + lane * 4)
                                    : make_uint2(0u, 0u);
            }

            // Every thread copies 8 of the 1024 16-byte pieces of tile i of K (or V) into stage (tbase + i) % NST, in
            // the 128-byte hardware swizzle: rows r0 + 16 j (j = 0..7) at a fixed 16-byte column, so that the swizzle
            // term and the source offsets are the same for every j.  A tile that lies wholly in the cache (blocks
            // of 64 tokens or more) is copied from two pointers fetched one iteration earlier - rows 0..63 and rows
            // 64..127 - with compile-time offsets; the tile that holds the new token, and 32-token blocks, take the
            // general path, which zero-fills the rows that are not in the cache yet.  The caller arrives on the
            // stage's barrier.
            struct TilePtrs
            {
                const char *lo, *hi; // rows 0..63, rows 64..127 of the tile (this thread's column already added)
            };
            auto tile_ptrs = [&](int i, bool is_v) -> TilePtrs
            {
                TilePtrs r{nullptr, nullptr};
                const int t0 = chunk_start + i * TT;
                if (i < n_tiles && t0 + TT <= new_pos && tpb_log2 >= 6)
                {
                    const int64_t* rowp = is_v ? vrow : krow;
                    const int bi = t0 >> tpb_log2;
                    if (tpb_log2 >= 7)
                    {
                        r.lo = reinterpret_cast<const char*>(table_entry(rowp, bi, a.max_blocks_per_seq, a.status, a.guard)) + src_thread + (size_t) (t0 & tpb_mask) * DH;
                        r.hi = r.lo + 64 * DH;
                    }
                    else
                    {
                        r.lo = reinterpret_cast<const char*>(table_entry(rowp, bi, a.max_blocks_per_seq, a.status, a.guard)) + src_thread;
                        r.hi = reinterpret_cast<const char*>(table_entry(rowp, bi + 1, a.max_blocks_per_seq, a.status, a.guard)) + src_thread;
                    }
                }
                return r;
            };
            auto issue = [&](int i, bool is_v, const TilePtrs& tp)
            {
                const int t0 = chunk_start + i * TT;
                const uint32_t dst = s_base + (is_v ? Tr::OFF_V : Tr::OFF_K) + ((tbase + i) % NST) * KV_TILE + dst_thread;
                if (tp.lo != nullptr)
                {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        cp_async16_u32(dst + j * 2048, tp.lo + j * 2048);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        cp_async16_u32(dst + (4 + j) * 2048, tp.hi + j * 2048);
                }
                else
                {
#pragma unroll 1
                    for (int j = 0; j < 8; ++j)
                    {
                        const int tok = t0 + r0 + 16 * j;
                        const bool ok = tok < new_pos;
                        const int tk = ok ? tok : new_pos; // keeps the table look-up inside the allocated blocks
                        const char* src = reinterpret_cast<const char*>(table_entry(is_v ? vrow : krow, tk >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard))
                            + head_off + (size_t) (tk & tpb_mask) * DH + col * 16;
                        cp_async16_zfill_u32(dst + j * 2048, src, ok ? 16u : 0u);
                    }
                }
            };
            // The tile that ends with the new token: quantise its k (or v) row as it is stored, place it in the
            // staged tile and append it to the cache.  Called by every thread after the tile's copies have landed.
            auto place_new = [&](int i, bool is_v)
            {
                const int t0 = chunk_start + i * TT;
                if (i == new_tile && warp == 0 && lane < DH / 16)
                {
                    const float sc_f = __ldg(a.scale_orig_quant);
                    const T sc_t = TypeOps<T>::from_float(sc_f);
                    const T* src = qkv_b + (size_t) (a.num_heads + (is_v ? a.num_kv_heads : 0) + hk) * DH + lane * 16;
                    const uint4 q = make_cache_vec<T, CACHE, 16>(src, sc_f, sc_t);
                    unsigned char* stage = smem + (is_v ? Tr::OFF_V : Tr::OFF_K) + ((tbase + i) % NST) * KV_TILE;
                    *reinterpret_cast<uint4*>(stage + hw_swz<128>((uint32_t) (new_pos - t0) * 128 + lane * 16)) = q;
                    const int64_t* rowp = is_v ? vrow : krow;
                    char* dst = reinterpret_cast<char*>(table_entry(rowp, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + head_off
                        + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                    *reinterpret_cast<uint4*>(dst) = q;
                }
            };
            auto mma_s = [&](int i) // S^T(i) = K(i) Qx^T
            {
                const uint64_t da = desc_k + (uint64_t) ((((tbase + i) % NST) * KV_TILE) >> 4);
#pragma unroll
                for (int ks = 0; ks < DH / 32; ++ks)
                    umma_f8(tmem_base + (i & 1) * 32, da + (uint64_t) ((ks * 32) >> 4), desc_q + (uint64_t) ((ks * 32) >> 4),
                        IDESC_S, ks != 0);
            };
            auto mma_o = [&](int i) // O^T += V(i)^T Px(i)
            {
                const uint64_t da = desc_v + (uint64_t) ((((tbase + i) % NST) * KV_TILE) >> 4);
                const uint64_t db = desc_p + (uint64_t) (((i & 1) * P_TILE) >> 4);
#pragma unroll
                for (int ks = 0; ks < TT / 32; ++ks)
                    umma_f8(tmem_o, da + (uint64_t) ((ks * 32 * DH) >> 4), db + (uint64_t) ((ks * 32 * 16) >> 4), IDESC_O,
                        (i | ks) != 0);
            };

            // block pointers of everything the prologue and the first iteration copy: one memory latency for all
            const TilePtrs tp_k0 = tile_ptrs(0, false);
            TilePtrs tp_v[NST], tp_k[NST]; // pair j = { V(j), K(j+1) }
#pragma unroll
            for (int j = 0; j < NST; ++j)
            {
                tp_v[j] = tile_ptrs(j, true);
                tp_k[j] = tile_ptrs(j + 1, false);
            }
            // K(0) on its own barrier, then the pairs { V(j), K(j+1) } of the first NST - 1 stages (K(NST) has to
            // wait until S^T(0) has consumed K(0): pair NST - 1 is issued at the top of iteration 0)
            issue(0, false, tp_k0);
            cp_async_mbar_arrive_noinc(full_k0);
#pragma unroll
            for (int j = 0; j < NST - 1; ++j)
            {
                if (j < n_tiles)
                {
                    issue(j, true, tp_v[j]);
                    if (j + 1 < n_tiles)
                        issue(j + 1, false, tp_k[j]);
                    cp_async_mbar_arrive_noinc(&full[(tbase + j) % NST]);
                }
            }
            TilePtrs v_next = tp_v[NST - 1], k_next = tp_k[NST - 1];

            // ---- Qx: row hh = high e4m3 parts of head hh, row GP + hh = 16 x low parts ----
#pragma unroll
            for (int c = 0; c < GP / 4; ++c)
            {
                const int hh = warp + 4 * c;
                const float2 lo2 = TypeOps<T>::unpack2(q_raw[c].x), hi2 = TypeOps<T>::unpack2(q_raw[c].y);
                const float q0 = lo2.x, q1 = lo2.y, q2 = hi2.x, q3 = hi2.y;
                float amax = fmaxf(fmaxf(fabsf(q0), fabsf(q1)), fmaxf(fabsf(q2), fabsf(q3)));
#pragma unroll
                for (int x = 16; x >= 1; x >>= 1)
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, x));
                int e = 0;
                if (amax > 0.f)
                    e = 7 - (int) (((__float_as_uint(amax) >> 23) & 0xff) - 127);
                e = max(-100, min(100, e));
                const float qmul = __uint_as_float((uint32_t) (e + 127) << 23); // row maximum into [128, 256)
                const float qinv = __uint_as_float((uint32_t) (127 - e) << 23);
                uint32_t whi, wlo;
                split4_lo16(q0 * qmul, q1 * qmul, q2 * qmul, q3 * qmul, whi, wlo);
                *reinterpret_cast<uint32_t*>(smem + Tr::OFF_Q + hw_swz<128>((uint32_t) hh * 128 + lane * 4)) = whi;
                *reinterpret_cast<uint32_t*>(smem + Tr::OFF_Q + hw_swz<128>((uint32_t) (GP + hh) * 128 + lane * 4)) = wlo;
                if (lane == 0)
                    sfac_s[hh] = qinv * deq * a.softmax_scale_log2;
            }

            // prologue: S^T(0)
            fail |= !mbar_wait_bounded(full_k0, npiece & 1, a.status);
            place_new(0, false);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            fail = __syncthreads_or(fail);
            float sfac[GP];
#pragma unroll
            for (int h = 0; h < GP; ++h)
                sfac[h] = sfac_s[h];
            if (!fail && tid == 0)
            {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                mma_s(0);
                umma_commit(&bar_mma[cbase & 1]);
            }

            for (int i = 0; i < n_tiles && !fail; ++i)
            {
                // group i = { O^T += tile i-1, S^T(i) } has completed: S^T(i) is readable, the K stage of tile i and
                // the V stage of tile i-1 are free again
                fail |= !mbar_wait_bounded(&bar_mma[(cbase + i) & 1], ((cbase + i) >> 1) & 1, a.status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!fail && i - 1 + NST < n_tiles)
                {
                    const int j = i - 1 + NST; // pair j goes into the stages that tiles i-1 (V) and i (K) have left
                    issue(j, true, v_next);
                    if (j + 1 < n_tiles)
                        issue(j + 1, false, k_next);
                    cp_async_mbar_arrive_noinc(&full[(tbase + j) % NST]);
                    v_next = tile_ptrs(j + 1, true);
                    k_next = tile_ptrs(j + 2, false);
                }

                // ---- this thread's token row of S^T ----
                const int t0 = chunk_start + i * TT;
                float s[GP], p[GP];
                {
                    float r[N];
                    tmem_ld_row<N>(tmem_base + (i & 1) * 32 + lane_sel, r);
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        s[h] = fmaf(r[GP + h], LOW, r[h]) * sfac[h];
                }
                if (t0 + TT > total && t0 + tid >= total) // rows beyond the sequence (last tile only)
                {
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        s[h] = -INFINITY;
                }
                int exceed = 0;
#pragma unroll
                for (int h = 0; h < GP; ++h)
                {
                    const float d = s[h] - mref[h];
                    exceed |= (d > PMAX);
                    p[h] = fast_exp2(d);
                }
                unsigned char* pbuf = smem + Tr::OFF_P + (i & 1) * P_TILE;
                auto store_p = [&]()
                {
                    uint32_t hi[GP / 4], lo[GP / 4];
#pragma unroll
                    for (int c = 0; c < GP / 4; ++c)
                        split4_lo16(p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3], hi[c], lo[c]);
                    if constexpr (GP == 8)
                    {
                        *reinterpret_cast<uint4*>(pbuf + tid * 16) = make_uint4(hi[0], hi[1], lo[0], lo[1]);
                    }
                    else
                    {
                        *reinterpret_cast<uint4*>(pbuf + tid * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(pbuf + TT * 16 + tid * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                };
                if (!exceed)
                    store_p();

                // operands of the MMAs issued behind the barrier: V(i) and K(i+1)
                fail |= !mbar_wait_bounded(&full[(tbase + i) % NST], ((tbase + i) / NST) & 1, a.status);
                if (new_tile >= 0)
                {
                    place_new(i, true);
                    place_new(i + 1, false);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                const int slow = __syncthreads_or(exceed | fail);
                if (slow)
                {
                    // Rare path: a time-out somewhere, or some score left the range the current reference covers.
                    fail = __syncthreads_or(fail);
                    if (fail)
                        break;
                    float mx[GP];
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                    {
                        mx[h] = s[h];
#pragma unroll
                        for (int x = 16; x >= 1; x >>= 1)
                            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], x));
                    }
                    if (lane == 0)
                    {
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                            red[warp * GP + h] = mx[h];
                    }
                    __syncthreads();
                    float f[GP];
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                    {
                        const float mt = fmaxf(fmaxf(red[h], red[GP + h]), fmaxf(red[2 * GP + h], red[3 * GP + h]));
                        const float mnew = fmaxf(mref[h], mt - 4.f);
                        f[h] = fast_exp2(mref[h] - mnew);
                        mref[h] = mnew;
                        l[h] *= f[h];
                        p[h] = fast_exp2(s[h] - mnew);
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (i > 0)
                    {
                        // O^T row of this thread's Dh channel: every column is one head (high or low part)
                        float o[N];
                        tmem_ld_row<N>(tmem_o + lane_sel, o);
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            o[h] *= f[h];
                            o[GP + h] *= f[h];
                        }
                        tmem_st_row<N>(tmem_o + lane_sel, o);
                    }
                    store_p();
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncthreads(); // also protects red[] against the next use
                }
#pragma unroll
                for (int h = 0; h < GP; ++h)
                    l[h] += p[h];
                if (tid == 0)
                {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    mma_o(i);
                    if (i + 1 < n_tiles)
                        mma_s(i + 1);
                    umma_commit(&bar_mma[(cbase + i + 1) & 1]);
                }
            }

            // ---- the last group: O^T complete ----
            if (!fail)
                fail |= !mbar_wait_bounded(&bar_mma[(cbase + n_tiles) & 1], ((cbase + n_tiles) >> 1) & 1, a.status);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tbase += n_tiles;
            cbase += n_tiles + 1;
            ++npiece;
        }
        fail = __syncthreads_or(fail);
        if (fail)
            break;

        // ---- result of the piece: thread = Dh channel ----
        {
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
#pragma unroll
                for (int x = 16; x >= 1; x >>= 1)
                    l[h] += __shfl_xor_sync(0xffffffffu, l[h], x);
            }
            if (lane == 0)
            {
#pragma unroll
                for (int h = 0; h < GP; ++h)
                    red[warp * GP + h] = l[h];
            }
            __syncthreads();
            float o[N];
            if (n_tiles > 0)
            {
                tmem_ld_row<N>(tmem_o + lane_sel, o);
            }
            else
            {
#pragma unroll
                for (int c = 0; c < N; ++c)
                    o[c] = 0.f;
            }
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
                if (h < G)
                {
                    const float lt = red[h] + red[GP + h] + red[2 * GP + h] + red[3 * GP + h];
                    const float ov = fmaf(o[GP + h], LOW, o[h]) * deq;
                    const size_t row = (size_t) b * a.num_heads + head0 + h;
                    if (final_out)
                    {
                        reinterpret_cast<T*>(a.out)[row * DH + tid] = TypeOps<T>::from_float(ov / lt);
                    }
                    else
                    {
                        a.part_o[(row * a.nsplit + chunk) * DH + tid] = ov;
                        if (tid == 0)
                            a.part_ml[row * a.nsplit + chunk] = make_float2(mref[h], lt);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads(); // red[] and the accumulators are free for the next piece
        }
        if (!a.streamk || !sk_next(sk, cur))
            break;
    }

    if (fail)
    {
        if (tid == 0)
        {
            report_status(a.status, STATUS_TIMEOUT);
            umma_commit(bar_drain); // no MMA may still be writing tensor memory when it is freed below
            mbar_drain(bar_drain, 0);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
    // ---- free tensor memory (every path reaches this) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Tr::TMEM_COLS));
}

} // namespace dx
