// Grouped-head decode attention over an FP8 paged KV cache on the 5th-generation tensor cores: the persistent,
// warp-specialised form of the token-major kernel (dx_tok_kernel.cuh).  Opt-in (DX_ATTN_TOKWS=1).  A CTA walks a range of
// the batch's 128-token tiles (SkSchedule: one static range per CTA and, optionally, short ranges taken from a device
// counter afterwards) and its copy stream never stops at a row or range boundary:
//
//   warp 4  producer : walks the tiles, copies K and V tiles (16-byte cp.async into the 128-byte hardware swizzle)
//                      into a ring of NST stages as soon as the stage's K (or V) half is free; quantises and appends
//                      the new token
//   warp 5  MMA      : one thread issues  S^T(g) = K(g) Qx^T  and, one tile behind,  O^T += V(g-1)^T Px(g-1)
//                      (tcgen05.mma kind::f8f6f4, cache bytes as stored, accumulators in tensor memory);
//                      tcgen05.commit on mbarriers frees the K half behind S^T, the V half behind O^T, and
//                      publishes S^T / O^T
//   warp 6  aux      : prepares Qx (high / low e4m3 parts of the q rows) of the next piece into the other Q buffer,
//                      and draws the ticket of the next dynamic range when the range before it is used up
//   warps 0-3 softmax: thread = token row of S^T (tensor-memory lane); lazy reference maximum, probabilities as
//                      high / low e4m3 parts into the P buffer; at the end of a piece thread = Dh channel of O^T
//
// S^T, P and O^T are double-buffered (tile parity, piece parity), so the tensor core computes S^T(g+1) while the
// softmax warps work on tile g, and the epilogue of a piece overlaps the first tiles of the next one.  Groups of up
// to 8 heads run two such CTAs per SM (three ring stages each), so that one CTA's piece boundaries and
// synchronisation latencies run beside the other's tiles; 16 padded heads run one CTA with six stages.
// Operand layouts, descriptors and the high / low split are those of the token-major kernel.
// Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, records STATUS_TIMEOUT, and every role
// leaves its loop; copies and MMAs in flight are drained and tensor memory is freed on every path.
//
// What was measured on B200 while building it (Llama-2-70B-shaped batch, 793 MB of FP8 KV, 148 SMs):
//   * one thread issues a tcgen05.mma (M 128, K 32, any N up to 128) every ~60 cycles at best, ~107 cycles in
//     groups of four: the eight MMAs of a tile cost the issuing thread 0.3-0.5 us, as much as the softmax of a tile;
//   * one warp issues a 16-byte cp.async every ~35-40 cycles: 64 of them per tile and lane keep a producer warp busy
//     for ~1.1 us per tile, so one producer warp feeds at most ~28 GB/s;
//   * a piece boundary costs a softmax group 4-6 us (accumulator read-out behind the last MMAs, row-sum reduction,
//     strided result stores behind the copy traffic, first-tile maximum of the next piece), which is why short
//     dynamic ranges make this kernel slower, not faster;
//   * this form: 150 us per step against 140 us for the mma.sync kernel in the same run; variants with one CTA per
//     SM, two softmax groups sharing the tiles of a piece, four MMA-issuing threads and separate K / V producer
//     warps reached 155 us; with tiled bulk-tensor copies through a tensor map of the KV pool 267 us (each copy
//     instruction then held its issuing thread for ~0.25 us).  It therefore stays opt-in.
//
// Replaces what the reference runs as XQA (decoderXQAImplPrecompiled.cpp:223-374) or as one MMHA CTA per q head
// (decoderMaskedMultiheadAttentionTemplate.h:1303) for grouped heads with an FP8 cache.
#pragma once

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh" // make_cache_vec
#include "dx_tcgen05.cuh"
#include "dx_tok_kernel.cuh" // split4_lo16

namespace dx
{

template <int GP, int STAGES>
struct TokWsTraits
{
    static constexpr int DH = 128, TT = 128, N = 2 * GP;
    static constexpr int NST = STAGES;       // ring stages (a K tile and a V tile each)
    static constexpr int KV_TILE = TT * DH;  // bytes of a K (or V) tile
    static constexpr int Q_TILE = N * DH;
    static constexpr int P_TILE = TT * N;
    static constexpr int OFF_Q = 0;                      // two buffers (piece parity)
    static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;     // two buffers (tile parity)
    static constexpr int OFF_KV = OFF_P + 2 * P_TILE;    // NST x { K tile, V tile }
    static constexpr int OFF_SFAC = OFF_KV + NST * 2 * KV_TILE; // float sfac[2][GP]
    static constexpr int OFF_RED = OFF_SFAC + 2 * GP * 4;       // float red_l[2][4][GP], red_m[4][GP]
    static constexpr int OFF_MISC = OFF_RED + 12 * GP * 4;      // int tickets[4], abort, tmem slot
    static constexpr int OFF_BAR = OFF_MISC + 32;
    static constexpr int NBAR = 4 * NST + 16 + 8 + 1;
    static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 1024; // + alignment slack
    static constexpr int TMEM_COLS = 128; // S^T: columns 0 / 32, O^T: columns 64 / 96
    static constexpr int THREADS = 224;
    static_assert(OFF_KV % 1024 == 0 && KV_TILE % 1024 == 0, "tiles must sit on the swizzle period");
    static_assert(OFF_BAR % 8 == 0, "barrier alignment");
};

// One piece of a row as every role sees it.
struct WsPiece
{
    int b, hk, slot, chunk_start, n_tiles, total;
    bool final_out;
};

// Position of a role in this CTA's sequence of ranges and pieces.
struct WsWalker
{
    SkCursor cur;
    uint32_t range_idx;
    int k;      // ranges started so far (0: the static one comes next)
    bool open;  // cur is inside a range
    bool done;
};

struct WsShared
{
    volatile int* tickets; // [4]
    volatile int* abort;
    uint64_t *tk_full, *tk_empty;
    int32_t* status;
};

// Bounded wait of this kernel: also ends when another role raised the abort flag.
__device__ __forceinline__ bool ws_wait(uint64_t* bar, uint32_t parity, const WsShared& sh)
{
#pragma unroll 1
    for (int it = 0; it < (1 << 22); ++it)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((it & 63) == 63)
        {
            if (*sh.abort)
                return false;
            if ((it & 1023) == 1023 && *reinterpret_cast<const volatile int32_t*>(sh.status) != 0)
                break;
        }
    }
    *sh.abort = 1;
    report_status(sh.status, STATUS_TIMEOUT);
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Next piece of this CTA, the same sequence for every role: the pieces of the static range, then those of every
// dynamic range a ticket was drawn for.  Readers of a ticket (every role but the one that draws them) release its
// slot once read.  False: no more work (or the kernel is aborting).
struct WsNoDraw
{
    __device__ __forceinline__ void operator()() const {}
};

template <int TT, typename Draw = WsNoDraw>
__device__ __forceinline__ bool ws_next_piece(const SkSchedule& sk, const AttnArgs& a, const WsShared& sh, WsWalker& w,
    WsPiece& p, const bool is_aux, const bool warp_wide, const int lane, Draw draw = Draw())
{
    // warp_wide: all 32 lanes of the warp walk together (their decisions are made uniform); otherwise one thread
    // walks alone and no warp-level synchronisation may be executed
    for (;;)
    {
        if (w.done)
            return false;
        if (w.open)
        {
            if (w.cur.u < w.cur.u1)
            {
                const SkCursor& c = w.cur;
                const uint32_t ng = min(c.nb - c.g0, c.u1 - c.u);
                const uint32_t row_start = sk.rows_per_seq * sk.prefix[c.b] + c.y * c.nb;
                p.b = (int) c.b;
                p.hk = (int) c.y;
                p.slot = (int) (w.range_idx - sk_range_of_unit(sk, row_start));
                p.final_out = c.g0 == 0 && ng == c.nb;
                p.chunk_start = (int) c.g0 * TT;
                p.total = a.seq_len[p.b];
                const int ctoks = max(0, min((int) ng * TT, p.total - p.chunk_start)); // the device length decides
                p.n_tiles = (ctoks + TT - 1) / TT;
                if (p.total > (int) c.nb * TT && lane == 0 && is_aux)
                    report_status(sh.status, STATUS_PLAN_EXCEEDED); // longer than the host length the line was laid out for
                sk_next(sk, w.cur);
                return true;
            }
            w.open = false;
        }
        uint32_t ridx;
        if (w.k == 0)
        {
            ridx = blockIdx.x;
        }
        else
        {
            if (sk.n2 == 0)
            {
                w.done = true;
                return false;
            }
            const int j = w.k - 1, s = j & 3;
            if (is_aux)
                draw(); // the ticket of the next range is drawn now, when the one before is used up: as late as possible
            bool got = is_aux || ws_wait(&sh.tk_full[s], (j >> 2) & 1, sh);
            if (warp_wide)
                got = __all_sync(0xffffffffu, got);
            if (!got)
            {
                w.done = true;
                return false;
            }
            const int t = sh.tickets[s];
            if (warp_wide)
                __syncwarp();
            if (!is_aux && lane == 0)
                mbar_arrive(&sh.tk_empty[s]);
            if (t < 0 || (uint32_t) t >= sk.n2)
            {
                w.done = true;
                return false;
            }
            ridx = sk.n1 + (uint32_t) t;
        }
        ++w.k;
        uint32_t u0, u1;
        sk_range_units(sk, ridx, u0, u1);
        if (u0 >= u1)
            continue;
        sk_seek(sk, u0, u1, w.cur);
        w.range_idx = ridx;
        w.open = true;
    }
}

// Warp-uniform form of ws_wait: every lane of the warp gets the same answer.
__device__ __forceinline__ bool ws_wait_warp(uint64_t* bar, uint32_t parity, const WsShared& sh)
{
    return __all_sync(0xffffffffu, ws_wait(bar, parity, sh));
}

// OR over the 128 threads of the softmax warps (named barrier 1).
__device__ __forceinline__ int softmax_warps_or(int flag)
{
    int r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.b32 p, %1, 0;\nbar.red.or.pred q, 1, 128, p;\nselp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(r)
        : "r"(flag)
        : "memory");
    return r;
}

__device__ __forceinline__ void softmax_warps_sync()
{
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <typename T, int GP, int STAGES, int MINB>
__global__ void __launch_bounds__(TokWsTraits<GP, STAGES>::THREADS, MINB)
    tokws_decode_kernel(const AttnArgs a, const int hgroups_unused, const __grid_constant__ SkSchedule sk)
{
    using Tr = TokWsTraits<GP, STAGES>;
    constexpr int DH = Tr::DH, TT = Tr::TT, N = Tr::N, KV_TILE = Tr::KV_TILE, P_TILE = Tr::P_TILE, NST = Tr::NST;
    constexpr int Q_TILE = Tr::Q_TILE;
    constexpr int CACHE = CACHE_FP8;
    constexpr float LOW = 1.f / 16.f; // weight of the low-part columns
    constexpr float PMAX = 8.f;       // p = 2^(s - m) <= 2^PMAX goes into e4m3 without a further scale

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.num_heads / a.num_kv_heads;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    float* sfac_s = reinterpret_cast<float*>(smem + Tr::OFF_SFAC); // [2][GP]
    float* red_l = reinterpret_cast<float*>(smem + Tr::OFF_RED);   // [2][4][GP]
    float* red_m = red_l + 8 * GP;                                 // [4][GP]
    int* misc = reinterpret_cast<int*>(smem + Tr::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 5);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    uint64_t* full_k = bars;             // [NST] K tile of the stage has landed
    uint64_t* full_v = bars + NST;       // [NST] V tile of the stage has landed
    uint64_t* empty_k = bars + 2 * NST;  // [NST] S^T of the stage's tile has completed: the K half is free
    uint64_t* empty_v = bars + 3 * NST;  // [NST] O^T += of the stage's tile has completed: the V half is free
    uint64_t* s_full = bars + 4 * NST;   // [2] S^T(g) is in tensor memory
    uint64_t* s_empty = s_full + 2;      // [2] the softmax warps have read S^T(g)
    uint64_t* p_full = s_full + 4;       // [2] Px(g) is in shared memory
    uint64_t* p_empty = s_full + 6;      // [2] O^T += V(g)^T Px(g) has completed
    uint64_t* o_full = s_full + 8;       // [2] O^T of the piece is complete
    uint64_t* o_empty = s_full + 10;     // [2] the softmax warps have read O^T of the piece
    uint64_t* q_full = s_full + 12;      // [2] Qx and the score factors of the piece are in shared memory
    uint64_t* q_empty = s_full + 14;     // [2] the MMAs of the piece have completed
    uint64_t* tk_full = s_full + 16;     // [4]
    uint64_t* tk_empty = s_full + 20;    // [4]
    uint64_t* bar_drain = s_full + 24;

    WsShared sh;
    sh.tickets = misc;
    sh.abort = misc + 4;
    sh.tk_full = tk_full;
    sh.tk_empty = tk_empty;
    sh.status = a.status;

    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(Tr::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 32)
    {
#pragma unroll
        for (int s = 0; s < NST; ++s)
        {
            mbar_init(&full_k[s], 64); // per lane: its copies have landed + it is past its own shared-memory stores
            mbar_init(&full_v[s], 64);
            mbar_init(&empty_k[s], 1);
            mbar_init(&empty_v[s], 1);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
        {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 128);
            mbar_init(&p_full[i], 128);
            mbar_init(&p_empty[i], 1);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_empty[i], 128);
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], 1);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            mbar_init(&tk_full[i], 1);
            mbar_init(&tk_empty[i], 6); // producer, MMA and the four softmax warps read every ticket
        }
        mbar_init(bar_drain, 1);
        misc[4] = 0; // abort
        fence_mbar_init();
    }
    griddep_launch_dependents(); // the merge kernel may be scheduled; it waits for this grid to finish
    __syncthreads();             // barriers initialised, tensor-memory address published
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    WsWalker w;
    w.k = 0;
    w.open = false;
    w.done = false;
    w.range_idx = 0;
    WsPiece pc;

    if (warp == 4)
    {
        // =========================== producer ===========================
        // Lane l copies, for each 32-row quarter of a tile, the 16-byte pieces l, l + 32, ..., l + 224 of the
        // quarter's contiguous 4 KB: piece l + 32 j = row 4 j + (l >> 3), column l & 7, which the 128-byte swizzle
        // puts at column (l & 7) ^ (4 (j & 1) + (l >> 3)).
        const uint32_t rl = lane >> 3, cl = lane & 7;
        const uint32_t d_even = rl * 128 + ((cl ^ rl) << 4), d_odd = rl * 128 + ((cl ^ (4 + rl)) << 4);
        int g = 0; // tiles put through the ring so far
        while (ws_next_piece<TT>(sk, a, sh, w, pc, false, true, lane))
        {
            if (pc.n_tiles == 0)
                continue;
            const int new_pos = pc.total - 1;
            const bool has_new = new_pos >= pc.chunk_start && new_pos < pc.chunk_start + pc.n_tiles * TT;
            const int64_t* krow = a.block_ptrs + (int64_t) pc.b * 2 * a.max_blocks_per_seq;
            const int64_t* vrow = krow + a.max_blocks_per_seq;
            const size_t head_off = (size_t) pc.hk * ((size_t) DH << tpb_log2);
            uint4 kq = make_uint4(0u, 0u, 0u, 0u), vq = kq;
            if (has_new && lane < DH / 16)
            {
                // the new token's k / v, quantised exactly as stored; appended to the paged cache right away (no
                // copy of this step reads that row: the tiles take it from these registers)
                const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
                const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) pc.b * qkv_stride;
                const float sc_f = __ldg(a.scale_orig_quant);
                const T sc_t = TypeOps<T>::from_float(sc_f);
                kq = make_cache_vec<T, CACHE, 16>(qkv_b + (size_t) (a.num_heads + pc.hk) * DH + lane * 16, sc_f, sc_t);
                vq = make_cache_vec<T, CACHE, 16>(
                    qkv_b + (size_t) (a.num_heads + a.num_kv_heads + pc.hk) * DH + lane * 16, sc_f, sc_t);
                const size_t off = head_off + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(table_entry(krow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off) = kq;
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(table_entry(vrow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off) = vq;
            }
            bool ok = true;
            for (int i = 0; i < pc.n_tiles && ok; ++i, ++g)
            {
                const int s = g % NST;
                const int t0 = pc.chunk_start + i * TT;
                const uint32_t kdst = s_base + Tr::OFF_KV + s * (2 * KV_TILE), vdst = kdst + KV_TILE;
                // block pointers of the tile's four quarters, requested before the wait for the stage
                const char *kp[4], *vp[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                {
                    const int t = min(t0 + 32 * q, new_pos); // keeps the look-up inside the allocated blocks
                    const size_t off = head_off + (size_t) (t & tpb_mask) * DH + lane * 16;
                    kp[q] = reinterpret_cast<const char*>(table_entry(krow, t >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                    vp[q] = reinterpret_cast<const char*>(table_entry(vrow, t >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                }
                const bool whole = t0 + TT <= new_pos; // every row of the tile is in the cache
#pragma unroll
                for (int kv = 0; kv < 2; ++kv)
                {
                    ok = ws_wait_warp(kv ? &empty_v[s] : &empty_k[s], ((g / NST) & 1) ^ 1, sh);
                    if (!ok)
                        break;
                    const uint32_t dst = kv ? vdst : kdst;
                    if (whole)
                    {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                        {
                            const char* src = kv ? vp[q] : kp[q];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                cp_async16_u32(dst + (32 * q + 4 * j) * 128 + ((j & 1) ? d_odd : d_even), src + j * 512);
                        }
                    }
                    else
                    {
                        // the tile that ends the sequence: rows at and behind the new token are not read from the
                        // cache (zero-filled); the new token's row is written from registers below
#pragma unroll 1
                        for (int q = 0; q < 4; ++q)
                        {
                            const char* src = kv ? vp[q] : kp[q];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                            {
                                const int row = 32 * q + 4 * j + (int) rl;
                                const uint32_t d = dst + (32 * q + 4 * j) * 128 + ((j & 1) ? d_odd : d_even);
                                if (t0 + row < new_pos)
                                    cp_async16_u32(d, src + j * 512);
                                else if (t0 + row > new_pos)
                                    *reinterpret_cast<uint4*>(smem + (d - s_base)) = make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
                        if (lane < DH / 16)
                        {
                            const uint32_t r = (uint32_t) (new_pos - t0);
                            *reinterpret_cast<uint4*>(smem + Tr::OFF_KV + s * (2 * KV_TILE) + kv * KV_TILE
                                + hw_swz<128>(r * 128 + lane * 16))
                                = kv ? vq : kq;
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    uint64_t* fb = kv ? &full_v[s] : &full_k[s];
                    cp_async_mbar_arrive_noinc(fb); // arrives when this lane's copies have landed
                    mbar_arrive(fb);                // this lane's own stores are done
                }
            }
            if (!ok)
                break;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
    else if (warp == 5)
    {
        // =========================== MMA issue ===========================
        if (lane == 0)
        {
            constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (N >> 3) << 17) | ((128u >> 4) << 24); // A, B K-major
            constexpr uint32_t IDESC_O = IDESC_S | (1u << 15) | (1u << 16);                             // A, B MN-major
            const uint64_t desc_kv = umma_desc(s_base + Tr::OFF_KV, 16, 1024, 2u);
            const uint64_t desc_q = umma_desc(s_base + Tr::OFF_Q, 16, 1024, 2u);
            const uint64_t desc_p = umma_desc(s_base + Tr::OFF_P, 128, TT * 16, 0u);
            int g = 0, np = 0; // tiles, non-empty pieces so far
            // the O^T MMAs of a tile are issued one tile late, behind S^T of the next tile
            bool pend = false, pend_first = false, pend_last = false;
            int pend_g = 0, pend_ob = 0;
            bool ok = true;
            auto issue_o = [&]() -> bool
            {
                const int s = pend_g % NST, pb = pend_g & 1;
                if (!ws_wait(&p_full[pb], (pend_g >> 1) & 1, sh) || !ws_wait(&full_v[s], (pend_g / NST) & 1, sh))
                    return false;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = desc_kv + (uint64_t) ((s * (2 * KV_TILE) + KV_TILE) >> 4);
                const uint64_t db = desc_p + (uint64_t) ((pb * P_TILE) >> 4);
#pragma unroll
                for (int ks = 0; ks < TT / 32; ++ks)
                    umma_f8(tmem_base + 64 + pend_ob * 32, da + (uint64_t) ((ks * 32 * DH) >> 4),
                        db + (uint64_t) ((ks * 32 * 16) >> 4), IDESC_O, (!pend_first || ks != 0) ? 1u : 0u);
                umma_commit(&empty_v[s]);
                umma_commit(&p_empty[pb]);
                if (pend_last)
                {
                    umma_commit(&o_full[pend_ob]);
                    umma_commit(&q_empty[pend_ob]);
                }
                pend = false;
                return true;
            };
            while (ok && ws_next_piece<TT>(sk, a, sh, w, pc, false, false, 0))
            {
                if (pc.n_tiles == 0)
                    continue;
                const int ob = np & 1; // Q buffer, O^T buffer of this piece
                ok = ws_wait(&q_full[ob], (np >> 1) & 1, sh) && ws_wait(&o_empty[ob], ((np >> 1) & 1) ^ 1, sh);
                for (int i = 0; i < pc.n_tiles && ok; ++i, ++g)
                {
                    const int s = g % NST;
                    ok = ws_wait(&full_k[s], (g / NST) & 1, sh) && ws_wait(&s_empty[g & 1], ((g >> 1) & 1) ^ 1, sh);
                    if (!ok)
                        break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = desc_kv + (uint64_t) ((s * (2 * KV_TILE)) >> 4);
                    const uint64_t db = desc_q + (uint64_t) ((ob * Q_TILE) >> 4);
#pragma unroll
                    for (int ks = 0; ks < DH / 32; ++ks)
                        umma_f8(tmem_base + (g & 1) * 32, da + (uint64_t) ((ks * 32) >> 4), db + (uint64_t) ((ks * 32) >> 4),
                            IDESC_S, ks != 0);
                    umma_commit(&s_full[g & 1]);
                    umma_commit(&empty_k[s]);
                    if (pend)
                        ok = issue_o();
                    pend = true;
                    pend_g = g;
                    pend_ob = ob;
                    pend_first = i == 0;
                    pend_last = i == pc.n_tiles - 1;
                }
                ++np;
            }
            if (ok && pend)
                ok = issue_o();
            // every MMA issued has completed before tensor memory is freed
            umma_commit(bar_drain);
            mbar_drain(bar_drain, 0);
        }
        __syncwarp();
    }
    else if (warp == 6)
    {
        // =========================== aux: tickets and Qx ===========================
        int pub = 0;           // tickets published so far
        bool pub_done = sk.n2 == 0;
        auto publish = [&]()
        {
            if (pub_done)
                return;
            const int s = pub & 3;
            if (!ws_wait_warp(&tk_empty[s], ((pub >> 2) & 1) ^ 1, sh))
            {
                pub_done = true;
                return;
            }
            int t = 0;
            if (lane == 0)
                t = atomicAdd(a.tickets, 1);
            t = __shfl_sync(0xffffffffu, t, 0);
            if (lane == 0)
            {
                sh.tickets[s] = t;
                mbar_arrive(&tk_full[s]);
            }
            __syncwarp();
            if ((uint32_t) t >= sk.n2)
                pub_done = true;
            ++pub;
        };
        int np = 0;
        const float deq = __ldg(a.scale_quant_orig);
        const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
        while (ws_next_piece<TT>(sk, a, sh, w, pc, true, true, lane, publish))
        {
            if (pc.n_tiles == 0)
                continue;
            const int qb = np & 1;
            const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) pc.b * qkv_stride;
            uint2 q_raw[GP];
#pragma unroll
            for (int hh = 0; hh < GP; ++hh)
                q_raw[hh] = (hh < G) ? *reinterpret_cast<const uint2*>(qkv_b + (size_t) (pc.hk * G + hh) * DH + lane * 4)
                                     : make_uint2(0u, 0u);
            if (!ws_wait_warp(&q_empty[qb], ((np >> 1) & 1) ^ 1, sh))
                break;
            unsigned char* qbuf = smem + Tr::OFF_Q + qb * Q_TILE;
#pragma unroll
            for (int hh = 0; hh < GP; ++hh)
            {
                const float2 lo2 = TypeOps<T>::unpack2(q_raw[hh].x), hi2 = TypeOps<T>::unpack2(q_raw[hh].y);
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
                *reinterpret_cast<uint32_t*>(qbuf + hw_swz<128>((uint32_t) hh * 128 + lane * 4)) = whi;
                *reinterpret_cast<uint32_t*>(qbuf + hw_swz<128>((uint32_t) (GP + hh) * 128 + lane * 4)) = wlo;
                if (lane == 0)
                    sfac_s[qb * GP + hh] = qinv * deq * a.softmax_scale_log2;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&q_full[qb]);
            ++np;
        }
    }
    else
    {
        // =========================== softmax warps (threads 0 .. 127) ===========================
        // The four warps meet at named barrier 1.  A thread only leaves this role right behind one of those
        // barriers, on a decision all 128 threads share (no more work, or the abort flag): nobody is ever left
        // waiting at a barrier for a thread that has gone.  A wait that gave up makes the thread skip its work
        // (`ok`, made warp-uniform because the tensor-memory loads are warp-wide) until the next barrier.
        const uint32_t lane_sel = (uint32_t) (warp * 32) << 16;
        const float deq = __ldg(a.scale_quant_orig);
        int g = 0, np = 0, pi = 0; // tiles, non-empty pieces, pieces so far
        for (;;)
        {
            const bool got = ws_next_piece<TT>(sk, a, sh, w, pc, false, true, lane);
            if (softmax_warps_or(got ? 0 : 1))
                break; // out of work (every thread sees the same tickets) or aborting
            const int head0 = pc.hk * G;
            float mref[GP], l[GP];
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
                mref[h] = -INFINITY;
                l[h] = 0.f;
            }
            float o[N];
#pragma unroll
            for (int c = 0; c < N; ++c)
                o[c] = 0.f;
            const int ob = np & 1;
            bool ok = true, leave = false;
            if (pc.n_tiles > 0)
            {
                ok = ws_wait_warp(&q_full[ob], (np >> 1) & 1, sh);
                float sfac[GP];
#pragma unroll
                for (int h = 0; h < GP; ++h)
                    sfac[h] = sfac_s[ob * GP + h];
                for (int i = 0; i < pc.n_tiles; ++i, ++g)
                {
                    const int sb = g & 1;
                    ok = ok && ws_wait_warp(&s_full[sb], (g >> 1) & 1, sh);
                    float s[GP], p[GP];
                    int exceed = 0;
                    if (ok)
                    {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        float r[N];
                        tmem_ld_row<N>(tmem_base + sb * 32 + lane_sel, r);
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                            s[h] = fmaf(r[GP + h], LOW, r[h]) * sfac[h];
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(&s_empty[sb]); // S^T(g) is in registers: the buffer may take S^T(g + 2)
                        const int t0 = pc.chunk_start + i * TT;
                        if (t0 + tid >= pc.total) // rows beyond the sequence (last tile only)
                        {
#pragma unroll
                            for (int h = 0; h < GP; ++h)
                                s[h] = -INFINITY;
                        }
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            const float d = s[h] - mref[h];
                            exceed |= (d > PMAX);
                            p[h] = fast_exp2(d);
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                            s[h] = 0.f, p[h] = 0.f;
                    }
                    const int slow = softmax_warps_or(exceed | (ok ? 0 : 1));
                    if (slow)
                    {
                        if (softmax_warps_or(*sh.abort)) // (a reduction again: other roles raise the flag at any time)
                        {
                            leave = true;
                            break;
                        }
                        // Some score left the range the current reference covers (always on the first tile of a
                        // piece): take the tile's maximum, rescale O^T in tensor memory, recompute the tile's P.
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
                                red_m[warp * GP + h] = mx[h];
                        }
                        softmax_warps_sync();
                        float f[GP];
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            const float mt = fmaxf(fmaxf(red_m[h], red_m[GP + h]), fmaxf(red_m[2 * GP + h], red_m[3 * GP + h]));
                            const float mnew = fmaxf(mref[h], mt - 4.f);
                            f[h] = fast_exp2(mref[h] - mnew);
                            mref[h] = mnew;
                            l[h] *= f[h];
                            p[h] = fast_exp2(s[h] - mnew);
                        }
                        softmax_warps_sync(); // red_m is free for the next use
                        if (i > 0)
                        {
                            // O^T holds tiles 0 .. i-1 of the piece once the MMAs of tile i-1 have completed
                            ok = ws_wait_warp(&p_empty[(g - 1) & 1], ((g - 1) >> 1) & 1, sh);
                            if (ok)
                            {
                                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                                float oo[N];
                                tmem_ld_row<N>(tmem_base + 64 + ob * 32 + lane_sel, oo);
#pragma unroll
                                for (int h = 0; h < GP; ++h)
                                {
                                    oo[h] *= f[h];
                                    oo[GP + h] *= f[h];
                                }
                                tmem_st_row<N>(tmem_base + 64 + ob * 32 + lane_sel, oo);
                                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            }
                        }
                    }
                    // the P buffer of this parity is free once the O^T MMAs of tile g - 2 have completed
                    ok = ok && ws_wait_warp(&p_empty[sb], ((g >> 1) & 1) ^ 1, sh);
                    if (ok)
                    {
                        unsigned char* pbuf = smem + Tr::OFF_P + sb * P_TILE;
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
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        mbar_arrive(&p_full[sb]);
                    }
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        l[h] += p[h];
                }
                if (leave)
                    break;
                // ---- O^T of the piece ----
                ok = ok && ws_wait_warp(&o_full[ob], (np >> 1) & 1, sh);
                if (ok)
                {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    tmem_ld_row<N>(tmem_base + 64 + ob * 32 + lane_sel, o);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&o_empty[ob]);
                }
                ++np;
            }
            // ---- result of the piece: thread = Dh channel ----
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
#pragma unroll
                for (int x = 16; x >= 1; x >>= 1)
                    l[h] += __shfl_xor_sync(0xffffffffu, l[h], x);
            }
            float* rl = red_l + (pi & 1) * 4 * GP; // two buffers in turn: one barrier per piece is enough
            ++pi;
            if (lane == 0)
            {
#pragma unroll
                for (int h = 0; h < GP; ++h)
                    rl[warp * GP + h] = l[h];
            }
            if (softmax_warps_or((*sh.abort || !ok) ? 1 : 0))
                break;
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
                if (h < G)
                {
                    const float lt = rl[h] + rl[GP + h] + rl[2 * GP + h] + rl[3 * GP + h];
                    const float ov = fmaf(o[GP + h], LOW, o[h]) * deq;
                    const size_t row = (size_t) pc.b * a.num_heads + head0 + h;
                    if (pc.final_out)
                    {
                        reinterpret_cast<T*>(a.out)[row * DH + tid] = TypeOps<T>::from_float(ov / lt);
                    }
                    else
                    {
                        a.part_o[(row * a.nsplit + pc.slot) * DH + tid] = ov;
                        if (tid == 0)
                            a.part_ml[row * a.nsplit + pc.slot] = make_float2(mref[h], lt);
                    }
                }
            }
        }
    }

    // ---- every role ends here: free tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Tr::TMEM_COLS));
}

} // namespace dx
