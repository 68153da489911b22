// Wide-group (MQA / large GQA) decode attention over an FP8 paged KV cache on the 5th-generation
// tensor cores: tcgen05.mma with shared-memory operand descriptors and TMEM accumulators.
//
// One CTA of 128 threads per (split-K partition, kv head x 128-head slice of its q group, sequence).
// The q heads that share the kv head are the M = 128 rows of both MMAs, so a thread owns one head
// row end to end (TMEM lane = head) and the online softmax needs no cross-thread reduction:
//   S[128 x 64]   = Q[128 x Dh] K^T   tcgen05.mma.kind::f8f6f4, A = Q (smem, K-major), B = K tile (smem, K-major)
//   P             = 2^(S - m) per row, written to smem as e4m3 high + low parts (K-major A operand)
//   O[128 x Dh]  += P[128 x 64] V     A = P, B = V tile used as stored ([token][Dh], MN-major)
// Cache bytes are consumed by the tensor core exactly as stored: no conversion, no transpose.  Q and P
// are split into a high and a low e4m3 part (two MMAs into the same accumulator).  O stays in tensor
// memory for the whole partition; a row's reference m moves only when a score exceeds it by more than 2^4,
// and then the warp rescales its 32 rows of O in place (tcgen05.ld / st) before the next MMA is issued.
// Per 64-token tile the CTA issues { O += P(i) V(i), S(i+1) = Q K(i+1)^T } as one group behind the barrier
// that publishes P(i); the group's completion (tcgen05.commit on an mbarrier) frees the K and V stages, the
// P tile and S.  K / V tiles arrive through rings of 16-byte cp.async copies laid out in the hardware's
// 64-byte / 128-byte swizzle.  Every wait is bounded; TMEM is freed on every path.
//
// Replaces, for G > 16 with an FP8 cache (Falcon-style 71:1 MQA), what the reference would run as one
// MMHA CTA per q head (decoderMaskedMultiheadAttentionTemplate.h:1303) - XQA has no kernel for it
// (decoderXQARunner.h:87-159 admits only 8 q heads per kv head).
#pragma once

#include "dx_common.cuh"
#include "dx_gqa_kernel.cuh" // split4, cp_async16_*_u32
#include "dx_mha_kernel.cuh" // make_cache_vec
#include "dx_tcgen05.cuh"

namespace dx
{

template <int DH>
struct WideTraits
{
    static constexpr int TT = 64;           // tokens per tile
    static constexpr int NST = 2;           // ring stages for K and for V
    static constexpr int KV_TILE = TT * DH; // bytes of a K (or V) tile
    static constexpr int Q_TILE = 128 * DH; // bytes of the high (or low) part of Q
    static constexpr int P_TILE = 128 * TT; // bytes of the high (or low) part of P
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;
    static constexpr int OFF_K = OFF_P + 2 * P_TILE;
    static constexpr int OFF_V = OFF_K + NST * KV_TILE;
    static constexpr int OFF_BAR = OFF_V + NST * KV_TILE;
    static constexpr int SMEM_BYTES = OFF_BAR + 64 + 1024;   // barriers, tmem slot, alignment slack
    static constexpr int TMEM_COLS = (DH == 64) ? 128 : 256; // S: 64 columns, O: Dh columns (power of two)
    static constexpr uint32_t LAYOUT = (DH == 64) ? 4u : 2u; // UMMA layout type: SWIZZLE_64B / SWIZZLE_128B
    static constexpr int COPIES = KV_TILE / 2048;            // 16-byte copies per thread and tile (2 or 4)
    static constexpr int MIN_BLOCKS = (DH == 64) ? 3 : 2;    // CTAs per SM the kernel is built for (4 would cost spills)
    static_assert(OFF_K % 1024 == 0, "tiles must sit on the swizzle period");
};

template <typename T, int DH>
__global__ void __launch_bounds__(128, WideTraits<DH>::MIN_BLOCKS) wide_decode_kernel(const AttnArgs a, const int hgroups)
{
    using Tr = WideTraits<DH>;
    constexpr int TT = Tr::TT, NST = Tr::NST, KV_TILE = Tr::KV_TILE, COPIES = Tr::COPIES;
    constexpr uint32_t LAY = Tr::LAYOUT;
    constexpr uint32_t SBO_KV = 8 * DH; // 8 rows of a Dh-byte-pitch tile
    constexpr uint32_t SBO_P = 8 * TT;  // 8 rows of the 64-byte-pitch P tile
    constexpr int CACHE = CACHE_FP8;
    // p = 2^(s - m) with m = (lazy row reference) - 4: p <= 2^PMAX = 256 goes into e4m3 without a further scale
    constexpr float PMAX = 8.f;

    // (as a programmatic dependent of the kernel in front of it, the CTA is resident early and waits here)
    griddep_wait();
    const int chunk = blockIdx.x;
    const int hk = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
    const int b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.num_heads / a.num_kv_heads;
    const int nh = min(128, G - hg * 128);
    const int head0 = hk * G + hg * 128;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    // Loads that depend on nothing but the launch go first: this thread's q row and the scales.
    const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
    const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
    uint4 q_raw[DH / 8];
    if (tid < nh)
    {
        const uint4* qp = reinterpret_cast<const uint4*>(qkv_b + (size_t) (head0 + tid) * DH);
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
            q_raw[i] = qp[i];
    }
    else
    {
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
            q_raw[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    const float deq = __ldg(a.scale_quant_orig);

    const int total = a.seq_len[b];
    int chunk_start, ctoks, nparts;
    partition_of(total, a.chunk_tokens, chunk, chunk_start, ctoks, nparts);
    if (nparts > (int) gridDim.x && chunk == 0 && threadIdx.x == 0)
        report_status(a.status, STATUS_PLAN_EXCEEDED); // the tokens beyond the last partition are not attended to
    if (chunk >= nparts)
        return;
    griddep_launch_dependents();
    const int n_tiles = (ctoks + TT - 1) / TT;
    const int new_pos = total - 1;
    const int new_tile = (new_pos >= chunk_start && new_pos < chunk_start + ctoks) ? (new_pos - chunk_start) / TT : -1;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    // descriptors assume tiles aligned to the swizzle period: align the whole layout to 1 KB
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    uint64_t* full = bars;              // [NST]: V(j) and K(j+1) have landed, stage j % NST
    uint64_t* full_k0 = bars + NST;     // K(0) has landed
    uint64_t* bar_mma = bars + NST + 1; // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NST + 3);
    uint64_t* bar_drain = bars + NST + 4; // only used after a time-out: the MMAs issued so far have completed

    const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
    const int64_t* vrow = krow + a.max_blocks_per_seq;
    const size_t head_off = (size_t) hk * ((size_t) DH << tpb_log2);

    // Every thread copies COPIES of the 16-byte pieces of tile i of K (or V) into stage i % NST, in the hardware
    // swizzle: rows r0 + (2048 / Dh) j at a fixed 16-byte column, so that the swizzle term is the same for every j
    // and source and destination both advance by 2 KB.  A tile lies in one block (blocks hold 64 tokens or
    // more); its pointer is fetched one iteration ahead.  The tile that holds the new token takes the general
    // path, which zero-fills the rows that are not in the cache yet.  The caller arrives on the stage's barrier.
    constexpr int CPR = DH / 16; // 16-byte pieces per row
    const int col = tid % CPR, r0 = tid / CPR;
    const uint32_t dst_thread = hw_swz<DH>((uint32_t) r0 * DH + col * 16);
    const size_t src_thread = head_off + (size_t) r0 * DH + col * 16;
    auto tile_ptr = [&](int i, bool is_v) -> const char*
    {
        const int t0 = chunk_start + i * TT;
        if (i >= n_tiles || t0 + TT > new_pos)
            return nullptr;
        return reinterpret_cast<const char*>(table_entry(is_v ? vrow : krow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + src_thread
            + (size_t) (t0 & tpb_mask) * DH;
    };
    auto issue = [&](int i, bool is_v, const char* tp)
    {
        const int t0 = chunk_start + i * TT;
        const uint32_t dst = s_base + (is_v ? Tr::OFF_V : Tr::OFF_K) + (i % NST) * KV_TILE + dst_thread;
        if (tp != nullptr)
        {
#pragma unroll
            for (int j = 0; j < COPIES; ++j)
                cp_async16_u32(dst + j * 2048, tp + j * 2048);
        }
        else
        {
            const char* base = reinterpret_cast<const char*>(table_entry(is_v ? vrow : krow, min(t0, new_pos) >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard))
                + src_thread + (size_t) (t0 & tpb_mask) * DH;
#pragma unroll
            for (int j = 0; j < COPIES; ++j)
            {
                const bool ok = t0 + r0 + (2048 / DH) * j < new_pos;
                cp_async16_zfill_u32(dst + j * 2048, ok ? base + j * 2048 : base, ok ? 16u : 0u);
            }
        }
    };
    // The tile that ends with the new token: quantise its k (or v) row as it is stored, place it in the staged
    // tile and (first head slice only) append it to the cache.  Called after the tile's copies have landed.
    auto place_new = [&](int i, bool is_v)
    {
        if (i == new_tile && warp == 0 && lane < CPR)
        {
            const int t0 = chunk_start + i * TT;
            const float sc_f = __ldg(a.scale_orig_quant);
            const T sc_t = TypeOps<T>::from_float(sc_f);
            const T* src = qkv_b + (size_t) (a.num_heads + (is_v ? a.num_kv_heads : 0) + hk) * DH + lane * 16;
            const uint4 q = make_cache_vec<T, CACHE, 16>(src, sc_f, sc_t);
            unsigned char* stage = smem + (is_v ? Tr::OFF_V : Tr::OFF_K) + (i % NST) * KV_TILE;
            *reinterpret_cast<uint4*>(stage + hw_swz<DH>((uint32_t) (new_pos - t0) * DH + lane * 16)) = q;
            if (hg == 0)
            {
                const int64_t* rowp = is_v ? vrow : krow;
                char* dst = reinterpret_cast<char*>(table_entry(rowp, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + head_off
                    + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                *reinterpret_cast<uint4*>(dst) = q;
            }
        }
    };

    // block pointers of everything the prologue and the first iteration copy: one memory latency for all
    const char* tp_k0 = tile_ptr(0, false);
    const char *tp_v[NST], *tp_k[NST]; // pair j = { V(j), K(j+1) }
#pragma unroll
    for (int j = 0; j < NST; ++j)
    {
        tp_v[j] = tile_ptr(j, true);
        tp_k[j] = tile_ptr(j + 1, false);
    }

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
    const uint32_t tmem_s = tmem_base;      // S: columns [0, 64)
    const uint32_t tmem_o = tmem_base + TT; // O: columns [64, 64 + Dh)
    const uint32_t lane_sel = (uint32_t) (warp * 32) << 16;

    // K(0) on its own barrier, then the pairs { V(j), K(j+1) } of the first NST - 1 stages (K(NST) has to
    // wait until S(0) has consumed K(0): pair NST - 1 is issued at the top of iteration 0)
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
            cp_async_mbar_arrive_noinc(&full[j]);
        }
    }
    const char *v_next = tp_v[NST - 1], *k_next = tp_k[NST - 1];

    // ---- Q: thread = head row.  Scale the row into the e4m3 range, split high / low, store both
    // parts as K-major rows of the swizzled Q tiles ----
    float sfac;
    {
        float qv[DH];
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
        {
            const uint32_t w[4] = {q_raw[i].x, q_raw[i].y, q_raw[i].z, q_raw[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const float2 v = TypeOps<T>::unpack2(w[j]);
                qv[8 * i + 2 * j] = v.x;
                qv[8 * i + 2 * j + 1] = v.y;
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < DH; ++i)
            amax = fmaxf(amax, fabsf(qv[i]));
        int e = 0;
        if (amax > 0.f)
            e = 7 - (int) (((__float_as_uint(amax) >> 23) & 0xff) - 127);
        e = max(-100, min(100, e));
        const float qmul = __uint_as_float((uint32_t) (e + 127) << 23); // row maximum into [128, 256)
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

    // instruction descriptors (f32 accumulate, e4m3 x e4m3, M = 128) and operand descriptor bases: only the
    // start-address field (16-byte units, low bits of the low word) changes between stages and k-steps
    constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (TT >> 3) << 17) | ((128u >> 4) << 24);              // N = 64, B K-major
    constexpr uint32_t IDESC_O = (1u << 4) | (1u << 16) | ((uint32_t) (DH >> 3) << 17) | ((128u >> 4) << 24); // N = Dh, B MN-major
    const uint64_t desc_q = umma_desc(s_base + Tr::OFF_Q, 16, SBO_KV, LAY);
    const uint64_t desc_k = umma_desc(s_base + Tr::OFF_K, 16, SBO_KV, LAY);
    const uint64_t desc_p = umma_desc(s_base + Tr::OFF_P, 16, SBO_P, 4u);
    const uint64_t desc_v = umma_desc(s_base + Tr::OFF_V, 16, SBO_KV, LAY);
    auto mma_s = [&](int i) // S(i) = (Q_hi + Q_lo) K(i)^T
    {
        const uint64_t db = desc_k + (uint64_t) (((i % NST) * KV_TILE) >> 4);
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
            for (int ks = 0; ks < DH / 32; ++ks)
                umma_f8(tmem_s, desc_q + (uint64_t) ((part * Tr::Q_TILE + ks * 32) >> 4), db + (uint64_t) ((ks * 32) >> 4),
                    IDESC_S, (part | ks) != 0);
    };
    auto mma_o = [&](int i) // O += (P_hi + P_lo) V(i)
    {
        const uint64_t db = desc_v + (uint64_t) (((i % NST) * KV_TILE) >> 4);
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
            for (int ks = 0; ks < TT / 32; ++ks)
                umma_f8(tmem_o, desc_p + (uint64_t) ((part * Tr::P_TILE + ks * 32) >> 4),
                    db + (uint64_t) ((ks * 32 * DH) >> 4), IDESC_O, (i | part | ks) != 0);
    };

    int fail = 0;
    // prologue: S(0)
    fail |= !mbar_wait_bounded(full_k0, 0, a.status);
    place_new(0, false);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    fail = __syncthreads_or(fail);
    if (!fail && tid == 0)
    {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        mma_s(0);
        umma_commit(&bar_mma[0]);
    }

    float mref = -INFINITY, l = 0.f; // mref: the m above
    for (int i = 0; i < n_tiles && !fail; ++i)
    {
        // group i = { O += tile i-1, S(i) } has completed: S(i) is readable, the K stage of tile i, the V stage
        // of tile i-1 and the P tile are free again
        fail |= !mbar_wait_bounded(&bar_mma[i & 1], (i >> 1) & 1, a.status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!fail && i - 1 + NST < n_tiles)
        {
            const int j = i - 1 + NST; // pair j goes into the stages that tiles i-1 (V) and i (K) have left
            issue(j, true, v_next);
            if (j + 1 < n_tiles)
                issue(j + 1, false, k_next);
            cp_async_mbar_arrive_noinc(&full[j % NST]);
            v_next = tile_ptr(j + 1, true);
            k_next = tile_ptr(j + 2, false);
        }

        // ---- this thread's head row of S(i): scores -> probabilities -> P tile ----
        if (warp_active)
        {
            const int lim = total - (chunk_start + i * TT); // valid tokens in this tile if < TT
            float sv[TT];
            {
                float h0[32], h1[32];
                tmem_ld32(tmem_s + lane_sel, h0);
                tmem_ld32(tmem_s + lane_sel + 32, h1);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                {
                    sv[j] = h0[j];
                    sv[32 + j] = h1[j];
                }
            }
            if (lim < TT)
            {
#pragma unroll
                for (int j = 0; j < TT; ++j)
                    if (j >= lim)
                        sv[j] = -INFINITY;
            }
            float mx = sv[0];
#pragma unroll
            for (int j = 1; j < TT; ++j)
                mx = fmaxf(mx, sv[j]);
            mx *= sfac; // sfac > 0
            // the reference of a row moves only when a score leaves the range it covers; O is then rescaled
            // in tensor memory by the whole warp (rows that did not move scale by 1)
            const bool move = mx - mref > PMAX;
            if (__any_sync(0xffffffffu, move))
            {
                const float mnew = move ? mx - 4.f : mref;
                const float alpha = fast_exp2(mref - mnew); // first tile: 2^-inf = 0, l = 0
                mref = mnew;
                l *= alpha;
                if (i > 0)
                {
#pragma unroll
                    for (int c = 0; c < DH / 32; ++c)
                    {
                        float ot[32];
                        tmem_ld_row<32>(tmem_o + lane_sel + 32 * c, ot);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            ot[j] *= alpha;
                        tmem_st_row<32>(tmem_o + lane_sel + 32 * c, ot);
                    }
                }
            }
            // all 64 exponentials first (independent), four partial sums, then the e4m3 split
            const float moff = -mref;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < TT; ++j)
            {
                sv[j] = fast_exp2(fmaf(sv[j], sfac, moff));
                l4[j & 3] += sv[j];
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
#pragma unroll
            for (int c = 0; c < TT / 16; ++c)
            {
                uint4 hi, lo;
                split4<CACHE>(sv[16 * c], sv[16 * c + 1], sv[16 * c + 2], sv[16 * c + 3], hi.x, lo.x);
                split4<CACHE>(sv[16 * c + 4], sv[16 * c + 5], sv[16 * c + 6], sv[16 * c + 7], hi.y, lo.y);
                split4<CACHE>(sv[16 * c + 8], sv[16 * c + 9], sv[16 * c + 10], sv[16 * c + 11], hi.z, lo.z);
                split4<CACHE>(sv[16 * c + 12], sv[16 * c + 13], sv[16 * c + 14], sv[16 * c + 15], hi.w, lo.w);
                const uint32_t d = hw_swz<TT>((uint32_t) tid * TT + c * 16);
                *reinterpret_cast<uint4*>(smem + Tr::OFF_P + d) = hi;
                *reinterpret_cast<uint4*>(smem + Tr::OFF_P + Tr::P_TILE + d) = lo;
            }
        }

        // operands of the MMAs issued behind the barrier: V(i) and K(i+1)
        fail |= !mbar_wait_bounded(&full[i % NST], (i / NST) & 1, a.status);
        if (new_tile >= 0)
        {
            place_new(i, true);
            place_new(i + 1, false);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        fail = __syncthreads_or(fail);
        if (fail)
            break;
        if (tid == 0)
        {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            mma_o(i);
            if (i + 1 < n_tiles)
                mma_s(i + 1);
            umma_commit(&bar_mma[(i + 1) & 1]);
        }
    }

    // ---- the last group: O complete ----
    if (!fail)
        fail |= !mbar_wait_bounded(&bar_mma[n_tiles & 1], (n_tiles >> 1) & 1, a.status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    fail = __syncthreads_or(fail);
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
    else if (warp_active)
    {
        // thread = head row (every lane of the warp takes part in the loads)
        const size_t row = (size_t) b * a.num_heads + head0 + min(tid, nh - 1);
        const float inv = (a.nsplit == 1) ? deq / l : deq;
#pragma unroll
        for (int c = 0; c < DH / 32; ++c)
        {
            float ot[32];
            tmem_ld_row<32>(tmem_o + lane_sel + 32 * c, ot);
            if (tid < nh)
            {
                if (a.nsplit == 1)
                {
                    T* dst = reinterpret_cast<T*>(a.out) + row * DH + 32 * c;
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                    {
                        uint4 w;
                        w.x = TypeOps<T>::pack2(ot[j] * inv, ot[j + 1] * inv);
                        w.y = TypeOps<T>::pack2(ot[j + 2] * inv, ot[j + 3] * inv);
                        w.z = TypeOps<T>::pack2(ot[j + 4] * inv, ot[j + 5] * inv);
                        w.w = TypeOps<T>::pack2(ot[j + 6] * inv, ot[j + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + j) = w;
                    }
                }
                else
                {
                    float* dst = a.part_o + (row * a.nsplit + chunk) * DH + 32 * c;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(dst + j)
                            = make_float4(ot[j] * inv, ot[j + 1] * inv, ot[j + 2] * inv, ot[j + 3] * inv);
                }
            }
        }
        if (tid < nh && a.nsplit > 1)
            a.part_ml[row * a.nsplit + chunk] = make_float2(mref, l);
    }

    // ---- free TMEM (every path reaches this) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Tr::TMEM_COLS));
}

} // namespace dx
