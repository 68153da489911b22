// Grouped-head decode attention over an FP8 paged KV cache on the 5th-generation tensor cores: the persistent,
// warp-specialised form of the token-major kernel (dx_tok_kernel.cuh).  One CTA per SM walks ranges of the batch's
// 128-token tiles (SkSchedule: a long static range first, then short ranges taken from a device counter, so that
// the SMs that stream faster take more of the tail) and the copy stream never stops at a row or range boundary:
//
//   warps 0-3, 4-7  two softmax groups; the tiles of a piece go to them in turn (even tiles to group 0, odd ones to
//                   group 1), each group keeping its own online-softmax state and its own O^T accumulator, merged
//                   at the end of the piece.  Thread = token row of S^T (tensor-memory lane); lazy reference
//                   maximum; probabilities as high / low e4m3 parts into the group's P buffer.
//   warp 8, 9       producers: walk the tiles and copy the K (warp 8) and V (warp 9) tiles with 16-byte cp.async
//                   into the 128-byte hardware swizzle of a ring of 16 KB units, as soon as a unit is free; the
//                   block pointers are fetched one tile ahead; they also quantise and append the new token.
//   warps 10, 13    MMA issue, one thread each, for softmax group 0 / 1:  S^T(g) = K(g) Qx^T  as soon as K(g) has landed
//   warps 12, 14    and  O^T += V(g)^T Px(g)  as the group's Px arrive  (tcgen05.mma kind::f8f6f4, cache bytes as
//                   stored, accumulators in tensor memory); tcgen05.commit on mbarriers frees each unit right behind
//                   the MMA that read it and publishes S^T / O^T.
//   warp 11         aux: prepares Qx (high / low e4m3 parts of the q rows) of the next piece into the other Q
//                   buffer and draws the tickets of the dynamic ranges.
//
// S^T and P are double-buffered per group, O^T per group and piece parity, so the tensor core runs ahead of the
// softmax groups and the end of a piece overlaps the first tiles of the next one; every role knows the next piece
// (and has requested its length) one piece ahead.  Operand layouts, descriptors and the high / low split are those
// of the token-major kernel.
// Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, records STATUS_TIMEOUT, and every role
// leaves its loop; copies and MMAs in flight are drained and tensor memory is freed on every path.
//
// Replaces what the reference runs as XQA (decoderXQAImplPrecompiled.cpp:223-374) or as one MMHA CTA per q head
// (decoderMaskedMultiheadAttentionTemplate.h:1303) for grouped heads with an FP8 cache.
#pragma once

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh" // make_cache_vec
#include "dx_tcgen05.cuh"
#include "dx_tok_kernel.cuh" // split4_lo16

// Optional cycle accounting of the roles (development builds only, -DDX_TOKWS_TRACE): every wait category adds the
// cycles it spent to a counter behind the handle's status word.
#ifdef DX_TOKWS_TRACE
#define WS_TIMED(cat, expr) [&]() { const long long t0_ = clock64(); const bool r_ = (expr); ws_acc[cat] += clock64() - t0_; return r_; }()
#define WS_STAMP(var) const long long var = clock64()
#define WS_SINCE(cat, var) ws_acc[cat] += clock64() - var
#else
#define WS_TIMED(cat, expr) (expr)
#define WS_STAMP(var)
#define WS_SINCE(cat, var)
#endif

namespace dx
{

template <int GP, int UNITS>
struct TokWsTraits
{
    static constexpr int DH = 128, TT = 128, N = 2 * GP;
    static constexpr int NU = UNITS;         // ring units of one K or V tile each; K(g) -> unit 2g, V(g) -> 2g + 1
    static constexpr int KV_TILE = TT * DH;  // bytes of a K (or V) tile
    static constexpr int Q_TILE = N * DH;
    static constexpr int P_TILE = TT * N;
    static constexpr int X_TILE = GP * TT * 4;           // float [GP][128]: O^T of softmax group 1 for the merge
    static constexpr int OFF_Q = 0;                      // two buffers (piece parity)
    static constexpr int OFF_P = OFF_Q + 2 * Q_TILE;     // four buffers: [group][tile parity of the group]
    static constexpr int OFF_KV = OFF_P + 4 * P_TILE;    // NU units
    static constexpr int OFF_X = OFF_KV + NU * KV_TILE;  // two buffers (piece parity)
    static constexpr int OFF_SFAC = OFF_X + 2 * X_TILE;  // float sfac[8][GP]: score factors of the last eight pieces
    static constexpr int OFF_RED = OFF_SFAC + 8 * GP * 4; // float red_l[2][2][4][GP], red_m[2][4][GP], mref_x[2][GP], lsum_x[2][GP]
    static constexpr int OFF_MISC = OFF_RED + 28 * GP * 4; // int tickets[16], abort, tmem slot
    static constexpr int OFF_BAR = OFF_MISC + 80;
    static constexpr int NBAR = 2 * NU + 24 + 4 + 32 + 4 + 4;
    static constexpr int SMEM_BYTES = OFF_BAR + NBAR * 8 + 1024; // + alignment slack
    static constexpr int TMEM_COLS = 256; // S^T[group][parity]: columns 0 / 32 / 64 / 96, O^T[group][parity]: 128 ...
    static constexpr int THREADS = 480;
    static constexpr int TICKET_READERS = 14; // two producers, four MMA threads, eight softmax warps
    static_assert(NU % 2 == 0, "K units are the even ones");
    static_assert(OFF_KV % 1024 == 0 && KV_TILE % 1024 == 0, "tiles must sit on the swizzle period");
    static_assert(OFF_BAR % 8 == 0, "barrier alignment");
};

// Geometry of one piece of a row (what the schedule alone decides), and the piece as every role sees it once the
// device length of its sequence is known.
struct WsGeo
{
    int b, hk, slot, chunk_start, ntoks, row_toks;
    bool final_out;
};

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
    volatile int* tickets; // [16]: the roles are up to several ranges apart
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

// Warp-uniform form of ws_wait: every lane of the warp gets the same answer.
__device__ __forceinline__ bool ws_wait_warp(uint64_t* bar, uint32_t parity, const WsShared& sh)
{
    return __all_sync(0xffffffffu, ws_wait(bar, parity, sh));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Geometry of the next piece of this CTA, the same sequence for every role: the pieces of the static range, then
// those of every dynamic range a ticket was drawn for.  Readers of a ticket (every role but the one that draws
// them) release its slot once read.  False: no more work (or the kernel is aborting).
// warp_wide: all 32 lanes of the warp walk together (their decisions are made uniform); otherwise one thread walks
// alone and no warp-level synchronisation may be executed.
template <int TT>
__device__ __forceinline__ bool ws_advance(
    const SkSchedule& sk, const WsShared& sh, WsWalker& w, WsGeo& p, const bool is_aux, const bool warp_wide, const int lane)
{
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
                p.ntoks = (int) ng * TT;
                p.row_toks = (int) c.nb * TT;
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
            const int j = w.k - 1, s = j & 15;
            bool got = is_aux || ws_wait(&sh.tk_full[s], (j >> 4) & 1, sh);
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

template <int TT>
__device__ __forceinline__ WsPiece ws_piece(const WsGeo& g, const int total)
{
    WsPiece p;
    p.b = g.b, p.hk = g.hk, p.slot = g.slot, p.chunk_start = g.chunk_start, p.final_out = g.final_out;
    p.total = total;
    const int ctoks = max(0, min(g.ntoks, total - g.chunk_start)); // the schedule counts host lengths; the device length decides
    p.n_tiles = (ctoks + TT - 1) / TT;
    return p;
}

// OR over the threads that meet at a named barrier.
template <int ID, int COUNT>
__device__ __forceinline__ int named_or(int flag)
{
    int r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.b32 p, %1, 0;\nbar.red.or.pred q, %2, %3, p;\nselp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(r)
        : "r"(flag), "n"(ID), "n"(COUNT)
        : "memory");
    return r;
}

__device__ __forceinline__ int group_or(int wg, int flag)
{
    return wg == 0 ? named_or<1, 128>(flag) : named_or<2, 128>(flag);
}

__device__ __forceinline__ void group_sync(int wg)
{
    if (wg == 0)
        asm volatile("bar.sync 1, 128;" ::: "memory");
    else
        asm volatile("bar.sync 2, 128;" ::: "memory");
}

template <typename T, int GP, int UNITS>
__global__ void __launch_bounds__(TokWsTraits<GP, UNITS>::THREADS, 1)
    tokws_decode_kernel(const AttnArgs a, const int hgroups_unused, const __grid_constant__ SkSchedule sk)
{
    using Tr = TokWsTraits<GP, UNITS>;
    constexpr int DH = Tr::DH, TT = Tr::TT, N = Tr::N, KV_TILE = Tr::KV_TILE, P_TILE = Tr::P_TILE, NU = Tr::NU;
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
    float* xbuf = reinterpret_cast<float*>(smem + Tr::OFF_X);      // [2][GP][128]
    // [8][GP]: the softmax groups may be up to four or five pieces behind the warp that writes these (two Q buffers
    // ahead of the MMA thread, which is up to two tiles per group ahead of the groups)
    float* sfac_s = reinterpret_cast<float*>(smem + Tr::OFF_SFAC);
    float* red_l = reinterpret_cast<float*>(smem + Tr::OFF_RED);   // [2][2][4][GP]
    float* red_m = red_l + 16 * GP;                                // [2][4][GP]
    float* mref_x = red_m + 8 * GP;                                // [2][GP]
    float* lsum_x = mref_x + 2 * GP;                               // [2][GP]
    int* misc = reinterpret_cast<int*>(smem + Tr::OFF_MISC);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 17);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    uint64_t* full = bars;               // [NU] the unit's tile has landed
    uint64_t* empty = bars + NU;         // [NU] the MMAs that read the unit have completed
    uint64_t* s_full = bars + 2 * NU;    // [4] S^T of the group's tile is in tensor memory      (index group * 2 + parity)
    uint64_t* s_empty = s_full + 4;      // [4] the group has read it
    uint64_t* p_full = s_full + 8;       // [4] Px of the group's tile is in shared memory
    uint64_t* p_empty = s_full + 12;     // [4] O^T += V^T Px of that tile has completed
    uint64_t* o_full = s_full + 16;      // [4] the group's O^T of the piece is complete          (group * 2 + piece parity)
    uint64_t* o_empty = s_full + 20;     // [4] the group has read it
    uint64_t* q_full = s_full + 24;      // [2] Qx and the score factors of the piece are in shared memory
    uint64_t* q_empty = s_full + 26;     // [2] the S^T MMAs of the piece have completed
    uint64_t* tk_full = s_full + 28;     // [16]
    uint64_t* tk_empty = s_full + 44;    // [16]
    uint64_t* bar_drain = s_full + 60;   // [4]
    uint64_t* x_full = s_full + 64;      // [2] the other group's share of a piece is in the exchange buffer
    uint64_t* x_empty = s_full + 66;     // [2] it has been read

    WsShared sh;
    sh.tickets = misc;
    sh.abort = misc + 16;
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
#pragma unroll 1
        for (int u = 0; u < NU; ++u)
        {
            mbar_init(&full[u], 64); // per lane: its copies have landed + it is past its own shared-memory stores
            mbar_init(&empty[u], 1);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 128);
            mbar_init(&p_full[i], 128);
            mbar_init(&p_empty[i], 1);
            mbar_init(&o_full[i], 1);
            mbar_init(&o_empty[i], 128);
        }
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
        {
            mbar_init(&tk_full[i], 1);
            mbar_init(&tk_empty[i], Tr::TICKET_READERS);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
        {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], 2); // both S^T issuers are done with the piece
        }
        for (int i = 0; i < 4; ++i)
            mbar_init(&bar_drain[i], 1);
        for (int i = 0; i < 2; ++i)
        {
            mbar_init(&x_full[i], 128);
            mbar_init(&x_empty[i], 128);
        }
        misc[16] = 0; // abort
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
#ifdef DX_TOKWS_TRACE
    long long ws_acc[24];
#pragma unroll
    for (int i = 0; i < 24; ++i)
        ws_acc[i] = 0;
    const long long ws_start = clock64();
#endif

    if (warp == 8 || warp == 9)
    {
        // =========================== producers: warp 8 copies the K tiles, warp 9 the V tiles ===========================
        // Lane l copies, for each 32-row quarter of a tile, the 16-byte pieces l, l + 32, ..., l + 224 of the
        // quarter's contiguous 4 KB: piece l + 32 j = row 4 j + (l >> 3), column l & 7, which the 128-byte swizzle
        // puts at column (l & 7) ^ (4 (j & 1) + (l >> 3)).
        const int kv = warp - 8;
        const uint32_t rl = lane >> 3, cl = lane & 7;
        const uint32_t d_even = rl * 128 + ((cl ^ rl) << 4), d_odd = rl * 128 + ((cl ^ (4 + rl)) << 4);
        const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
        // source of this lane's share of the four quarters of tile i of a piece; look-ups are kept inside the
        // allocated blocks (tokens up to the new one)
        auto tile_ptrs = [&](const WsPiece& pc, int i, const char*(&out)[4])
        {
            const int64_t* row = a.block_ptrs + ((int64_t) pc.b * 2 + kv) * a.max_blocks_per_seq;
            const size_t head_off = (size_t) pc.hk * ((size_t) DH << tpb_log2);
            const int t0 = pc.chunk_start + i * TT;
#pragma unroll
            for (int q = 0; q < 4; ++q)
            {
                const int t = min(t0 + 32 * q, pc.total - 1);
                out[q] = reinterpret_cast<const char*>(__ldg(row + (t >> tpb_log2))) + head_off + (size_t) (t & tpb_mask) * DH
                    + lane * 16;
            }
        };
        int g = 0; // tiles put through the ring so far
        const float sc_f = (a.scale_orig_quant != nullptr) ? __ldg(a.scale_orig_quant) : 1.f;
        const T sc_t = TypeOps<T>::from_float(sc_f);
        // the k (or v) row of the next piece's sequence is requested together with its length, one piece ahead
        auto new_row = [&](const WsGeo& ge, uint4(&raw)[2])
        {
            if (lane < DH / 16)
            {
                const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.qkv) + (size_t) ge.b * qkv_stride
                    + (size_t) (a.num_heads + kv * a.num_kv_heads + ge.hk) * DH + lane * 16);
                raw[0] = src[0];
                raw[1] = src[1];
            }
        };
        WsGeo ngeo;
        bool have = WS_TIMED(15, ws_advance<TT>(sk, sh, w, ngeo, false, true, lane));
        int ntotal = have ? a.seq_len[ngeo.b] : 0;
        uint4 nraw[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
        if (have)
            new_row(ngeo, nraw);
        const char* pre[4] = {nullptr, nullptr, nullptr, nullptr};
        bool pre_valid = false;
        bool ok = true;
        while (have && ok)
        {
            const WsPiece pc = ws_piece<TT>(ngeo, ntotal);
            const uint4 raw0 = nraw[0], raw1 = nraw[1];
            have = WS_TIMED(15, ws_advance<TT>(sk, sh, w, ngeo, false, true, lane));
            if (have)
            {
                ntotal = a.seq_len[ngeo.b]; // requested now, needed when this piece is done
                new_row(ngeo, nraw);
            }
            if (pc.n_tiles == 0)
                continue;
            const int new_pos = pc.total - 1;
            const bool has_new = new_pos >= pc.chunk_start && new_pos < pc.chunk_start + pc.n_tiles * TT;
            uint4 nq = make_uint4(0u, 0u, 0u, 0u);
            if (has_new && lane < DH / 16)
            {
                // the new token's k (or v), quantised exactly as stored; appended to the paged cache right away (no
                // copy of this step reads that row: the tiles take it from this register)
                nq.x = quant4<T, CACHE>(raw0.x, raw0.y, sc_f, sc_t);
                nq.y = quant4<T, CACHE>(raw0.z, raw0.w, sc_f, sc_t);
                nq.z = quant4<T, CACHE>(raw1.x, raw1.y, sc_f, sc_t);
                nq.w = quant4<T, CACHE>(raw1.z, raw1.w, sc_f, sc_t);
                const int64_t* row = a.block_ptrs + ((int64_t) pc.b * 2 + kv) * a.max_blocks_per_seq;
                const size_t off
                    = (size_t) pc.hk * ((size_t) DH << tpb_log2) + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(__ldg(row + (new_pos >> tpb_log2))) + off) = nq;
            }
            for (int i = 0; i < pc.n_tiles; ++i, ++g)
            {
                const int u = (2 * g + kv) % NU;
                const int t0 = pc.chunk_start + i * TT;
                const uint32_t dst = s_base + Tr::OFF_KV + u * KV_TILE;
                const char* src[4];
                if (pre_valid)
                {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        src[q] = pre[q];
                }
                else
                {
                    tile_ptrs(pc, i, src);
                }
                // block pointers of the next tile (of this piece, or the first of the next one): in flight while
                // this tile is copied
                pre_valid = false;
                if (i + 1 < pc.n_tiles)
                {
                    tile_ptrs(pc, i + 1, pre);
                    pre_valid = true;
                }
                else if (have)
                {
                    const WsPiece nx = ws_piece<TT>(ngeo, ntotal);
                    if (nx.n_tiles > 0)
                    {
                        tile_ptrs(nx, 0, pre);
                        pre_valid = true;
                    }
                }
                ok = WS_TIMED(0, ws_wait_warp(&empty[u], (((2 * g + kv) / NU) & 1) ^ 1, sh));
                if (!ok)
                    break;
                if (t0 + TT <= new_pos) // every row of the tile is in the cache
                {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                    {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            cp_async16_u32(dst + (32 * q + 4 * j) * 128 + ((j & 1) ? d_odd : d_even), src[q] + j * 512);
                    }
                }
                else
                {
                    // the tile that ends the sequence: rows at and behind the new token are not read from the cache;
                    // the new token's row is written from the register, the rows behind it are zeroed
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                    {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                        {
                            const int row = 32 * q + 4 * j + (int) rl;
                            const uint32_t d = dst + (32 * q + 4 * j) * 128 + ((j & 1) ? d_odd : d_even);
                            if (t0 + row < new_pos)
                                cp_async16_u32(d, src[q] + j * 512);
                            else if (t0 + row > new_pos)
                                *reinterpret_cast<uint4*>(smem + (d - s_base)) = make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                    if (lane < DH / 16)
                        *reinterpret_cast<uint4*>(
                            smem + Tr::OFF_KV + u * KV_TILE + hw_swz<128>((uint32_t) (new_pos - t0) * 128 + lane * 16))
                            = nq;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                cp_async_mbar_arrive_noinc(&full[u]); // arrives when this lane's copies have landed
                mbar_arrive(&full[u]);                // this lane's own stores are done
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }
    else if (warp == 10 || warp == 13)
    {
        // =========================== issue of S^T = K Qx^T for one softmax group ===========================
        // (One thread issues a tcgen05.mma every ~60 cycles at best, whatever its N, and a tile is eight of them
        // plus the commits: the issue is split over four threads, S^T and O^T for each softmax group.)
        if (lane == 0)
        {
            const int mg = warp == 13 ? 1 : 0;
            constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (N >> 3) << 17) | ((128u >> 4) << 24); // A, B K-major
            const uint64_t desc_kv = umma_desc(s_base + Tr::OFF_KV, 16, 1024, 2u);
            const uint64_t desc_q = umma_desc(s_base + Tr::OFF_Q, 16, 1024, 2u);
            int g = 0, np = 0, c = 0; // tiles, non-empty pieces, tiles of this group so far
            bool ok = true;
            WsGeo ngeo;
            bool have = WS_TIMED(7, ws_advance<TT>(sk, sh, w, ngeo, false, false, 0));
            int ntotal = have ? a.seq_len[ngeo.b] : 0;
            while (have && ok)
            {
                const WsPiece pc = ws_piece<TT>(ngeo, ntotal);
                have = WS_TIMED(7, ws_advance<TT>(sk, sh, w, ngeo, false, false, 0));
                if (have)
                    ntotal = a.seq_len[ngeo.b];
                if (pc.n_tiles == 0)
                    continue;
                const int qb = np & 1;
                // (waited for even without a tile of this group in the piece: the arrival on q_empty below must not
                // run ahead of the piece it belongs to)
                ok = WS_TIMED(6, ws_wait(&q_full[qb], (np >> 1) & 1, sh));
                if (!ok)
                    break;
                if (pc.n_tiles > mg)
                {
                    for (int i = mg; i < pc.n_tiles && ok; i += 2, ++c)
                    {
                        const int si = mg * 2 + (c & 1);
                        const int gg = g + i, uk = (2 * gg) % NU;
                        ok = WS_TIMED(2, ws_wait(&full[uk], ((2 * gg) / NU) & 1, sh))
                            && WS_TIMED(3, ws_wait(&s_empty[si], ((c >> 1) & 1) ^ 1, sh));
                        if (!ok)
                            break;
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t da = desc_kv + (uint64_t) ((uk * KV_TILE) >> 4);
                        const uint64_t db = desc_q + (uint64_t) ((qb * Q_TILE) >> 4);
#pragma unroll
                        for (int ks = 0; ks < DH / 32; ++ks)
                            umma_f8(tmem_base + si * 32, da + (uint64_t) ((ks * 32) >> 4), db + (uint64_t) ((ks * 32) >> 4),
                                IDESC_S, ks != 0);
                        umma_commit(&s_full[si]);
                        umma_commit(&empty[uk]);
                    }
                    umma_commit(&q_empty[qb]); // this group's S^T MMAs of the piece
                }
                else
                {
                    mbar_arrive(&q_empty[qb]); // (no tile of this group in the piece)
                }
                g += pc.n_tiles;
                ++np;
            }
            // every MMA issued has completed before tensor memory is freed
            umma_commit(&bar_drain[mg]);
            mbar_drain(&bar_drain[mg], 0);
        }
        __syncwarp();
    }
    else if (warp == 12 || warp == 14)
    {
        // =========================== issue of O^T += V^T Px for one softmax group ===========================
        if (lane == 0)
        {
            const int mg = warp == 14 ? 1 : 0;
            constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (N >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t IDESC_O = IDESC_S | (1u << 15) | (1u << 16); // A, B MN-major
            const uint64_t desc_kv = umma_desc(s_base + Tr::OFF_KV, 16, 1024, 2u);
            const uint64_t desc_p = umma_desc(s_base + Tr::OFF_P, 128, TT * 16, 0u);
            int g = 0, c = 0, npw = 0; // tiles, tiles of this group, pieces in which it had tiles
            bool ok = true;
            WsGeo ngeo;
            bool have = WS_TIMED(14, ws_advance<TT>(sk, sh, w, ngeo, false, false, 0));
            int ntotal = have ? a.seq_len[ngeo.b] : 0;
            while (have && ok)
            {
                const WsPiece pc = ws_piece<TT>(ngeo, ntotal);
                have = WS_TIMED(14, ws_advance<TT>(sk, sh, w, ngeo, false, false, 0));
                if (have)
                    ntotal = a.seq_len[ngeo.b];
                if (pc.n_tiles <= mg)
                {
                    g += pc.n_tiles;
                    continue;
                }
                const int oi = mg * 2 + (npw & 1);
                // the group's first tile of the piece overwrites the accumulator: the group must have read what it
                // held two pieces ago
                ok = WS_TIMED(6, ws_wait(&o_empty[oi], ((npw >> 1) & 1) ^ 1, sh));
                for (int i = mg; i < pc.n_tiles && ok; i += 2, ++c)
                {
                    const int pi = mg * 2 + (c & 1);
                    const int gg = g + i, uv = (2 * gg + 1) % NU;
                    ok = WS_TIMED(4, ws_wait(&p_full[pi], (c >> 1) & 1, sh))
                        && WS_TIMED(5, ws_wait(&full[uv], ((2 * gg + 1) / NU) & 1, sh));
                    if (!ok)
                        break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = desc_kv + (uint64_t) ((uv * KV_TILE) >> 4);
                    const uint64_t db = desc_p + (uint64_t) ((pi * P_TILE) >> 4);
#pragma unroll
                    for (int ks = 0; ks < TT / 32; ++ks)
                        umma_f8(tmem_base + 128 + oi * 32, da + (uint64_t) ((ks * 32 * DH) >> 4),
                            db + (uint64_t) ((ks * 32 * 16) >> 4), IDESC_O, (i >= 2 || ks != 0) ? 1u : 0u);
                    umma_commit(&empty[uv]);
                    umma_commit(&p_empty[pi]);
                }
                if (ok)
                    umma_commit(&o_full[oi]);
                g += pc.n_tiles;
                ++npw;
            }
            umma_commit(&bar_drain[2 + mg]);
            mbar_drain(&bar_drain[2 + mg], 0);
        }
        __syncwarp();
    }
    else if (warp == 11)
    {
        // =========================== aux: tickets and Qx ===========================
        int pub = 0; // tickets published so far
        bool pub_done = sk.n2 == 0;
        auto publish = [&]()
        {
            const int s = pub & 15;
            if (!ws_wait_warp(&tk_empty[s], ((pub >> 4) & 1) ^ 1, sh))
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
        // two tickets ahead of the range this warp is in: the ticket of a range is there long before any role gets
        // to it
        auto keep_ahead = [&]()
        {
            while (!pub_done && pub < max(2, w.k + 1))
                publish();
        };
        keep_ahead();
        int np = 0;
        const float deq = __ldg(a.scale_quant_orig);
        const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
        WsGeo ngeo;
        bool have = ws_advance<TT>(sk, sh, w, ngeo, true, true, lane);
        keep_ahead();
        int ntotal = have ? a.seq_len[ngeo.b] : 0;
        while (have)
        {
            const WsPiece pc = ws_piece<TT>(ngeo, ntotal);
            if (pc.total > ngeo.row_toks && lane == 0)
                report_status(a.status, STATUS_PLAN_EXCEEDED); // longer than the host length the line was laid out for
            have = ws_advance<TT>(sk, sh, w, ngeo, true, true, lane);
            keep_ahead();
            if (have)
                ntotal = a.seq_len[ngeo.b];
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
                    sfac_s[(np & 7) * GP + hh] = qinv * deq * a.softmax_scale_log2;
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
        // =========================== softmax groups (threads 0 .. 255) ===========================
        // A group meets at its own named barrier (1 or 2); the two groups only meet through mbarriers (the exchange
        // buffer of a piece), with bounded waits.  A thread only leaves this role right behind a barrier of its
        // group, on a decision all 128 threads share (no more work, or the abort flag): nobody is ever left waiting at
        // a barrier for a thread that has gone.  A wait that gave up makes the thread skip its work (`ok`, made
        // warp-uniform because the tensor-memory loads are warp-wide) until then.
        const int wg = warp >> 2, wl = warp & 3, row = tid & 127;
        const uint32_t lane_sel = (uint32_t) (wl * 32) << 16;
        const float deq = __ldg(a.scale_quant_orig);
        int c = 0, npw = 0, np = 0, pl = 0, hx = 0; // the group's tiles and pieces, non-empty pieces, pieces, hand-overs so far
        WsGeo ngeo;
        bool have = WS_TIMED(12, ws_advance<TT>(sk, sh, w, ngeo, false, true, lane));
        int ntotal = have ? a.seq_len[ngeo.b] : 0;
        for (;;)
        {
            if (group_or(wg, (have ? 0 : 1) | *sh.abort))
                break; // out of work (every thread sees the same tickets) or aborting
            const WsPiece pc = ws_piece<TT>(ngeo, ntotal);
            have = WS_TIMED(12, ws_advance<TT>(sk, sh, w, ngeo, false, true, lane));
            if (have)
                ntotal = a.seq_len[ngeo.b];
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
            for (int cc = 0; cc < N; ++cc)
                o[cc] = 0.f;
            const int ob = npw & 1, oi = wg * 2 + ob;
            const bool mine = pc.n_tiles > wg; // this group has tiles in the piece
            bool ok = true;
            if (mine)
            {
                // (No wait for q_full here: this group may be several pieces behind the warp that writes Qx, more
                // than the one phase a parity wait can tell apart.  The score factors are read behind the first
                // s_full of the piece instead - the MMA thread waited for q_full before it issued that tile - and
                // they sit in a ring of eight.)
                const float* sfac = sfac_s + (np & 7) * GP;
                for (int i = wg; i < pc.n_tiles; i += 2, ++c)
                {
                    const int si = wg * 2 + (c & 1);
                    ok = ok && WS_TIMED(8, ws_wait_warp(&s_full[si], (c >> 1) & 1, sh));
                    float s[GP], p[GP];
                    int exceed = 0;
                    if (ok)
                    {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        float r[N];
                        tmem_ld_row<N>(tmem_base + si * 32 + lane_sel, r);
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                            s[h] = fmaf(r[GP + h], LOW, r[h]) * sfac[h];
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive(&s_empty[si]); // S^T is in registers: the buffer may take the group's tile after next
                        const int t0 = pc.chunk_start + i * TT;
                        if (t0 + row >= pc.total) // rows beyond the sequence (last tile only)
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
                    const int slow = WS_TIMED(11, group_or(wg, exceed | (ok ? 0 : 1)));
                    if (slow)
                    {
                        WS_STAMP(t_slow);
                        // Some score left the range the current reference covers (always on the group's first tile of
                        // a piece): take the tile's maximum, rescale O^T in tensor memory, recompute the tile's P.
                        float mx[GP];
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            mx[h] = s[h];
#pragma unroll
                            for (int x = 16; x >= 1; x >>= 1)
                                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], x));
                        }
                        float* rm = red_m + wg * 4 * GP;
                        if (lane == 0)
                        {
#pragma unroll
                            for (int h = 0; h < GP; ++h)
                                rm[wl * GP + h] = mx[h];
                        }
                        group_sync(wg);
                        float f[GP];
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            const float mt = fmaxf(fmaxf(rm[h], rm[GP + h]), fmaxf(rm[2 * GP + h], rm[3 * GP + h]));
                            const float mnew = fmaxf(mref[h], mt - 4.f);
                            f[h] = fast_exp2(mref[h] - mnew);
                            mref[h] = mnew;
                            l[h] *= f[h];
                            p[h] = fast_exp2(s[h] - mnew);
                        }
                        group_sync(wg); // red_m is free for the next use
                        if (i >= 2)
                        {
                            // O^T holds the group's earlier tiles of the piece once the MMAs of its previous tile
                            // have completed
                            ok = ok && WS_TIMED(9, ws_wait_warp(&p_empty[wg * 2 + ((c - 1) & 1)], ((c - 1) >> 1) & 1, sh));
                            if (ok)
                            {
                                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                                float oo[N];
                                tmem_ld_row<N>(tmem_base + 128 + oi * 32 + lane_sel, oo);
#pragma unroll
                                for (int h = 0; h < GP; ++h)
                                {
                                    oo[h] *= f[h];
                                    oo[GP + h] *= f[h];
                                }
                                tmem_st_row<N>(tmem_base + 128 + oi * 32 + lane_sel, oo);
                                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            }
                        }
                        WS_SINCE(23, t_slow);
                    }
                    // the P buffer of this parity is free once the O^T MMAs of the group's tile before last have completed
                    ok = ok && WS_TIMED(9, ws_wait_warp(&p_empty[si], ((c >> 1) & 1) ^ 1, sh));
                    if (ok)
                    {
                        unsigned char* pbuf = smem + Tr::OFF_P + si * P_TILE;
                        uint32_t hi[GP / 4], lo[GP / 4];
#pragma unroll
                        for (int q = 0; q < GP / 4; ++q)
                            split4_lo16(p[4 * q], p[4 * q + 1], p[4 * q + 2], p[4 * q + 3], hi[q], lo[q]);
                        if constexpr (GP == 8)
                        {
                            *reinterpret_cast<uint4*>(pbuf + row * 16) = make_uint4(hi[0], hi[1], lo[0], lo[1]);
                        }
                        else
                        {
                            *reinterpret_cast<uint4*>(pbuf + row * 16) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                            *reinterpret_cast<uint4*>(pbuf + TT * 16 + row * 16) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        mbar_arrive(&p_full[si]);
                    }
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        l[h] += p[h];
                }
                // ---- the group's O^T of the piece ----
                ok = ok && WS_TIMED(10, ws_wait_warp(&o_full[oi], (npw >> 1) & 1, sh));
                if (ok)
                {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    tmem_ld_row<N>(tmem_base + 128 + oi * 32 + lane_sel, o);
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&o_empty[oi]);
                }
                ++npw;
            }
            if (pc.n_tiles > 0)
                ++np;
            // ---- result of the piece: thread = Dh channel.  With tiles in both groups the group that does not hold
            // the last tile (it is done first) takes the other one's share from the exchange buffer and writes;
            // the other group hands its share over and goes on with the next piece. ----
            WS_STAMP(t_epi);
            const bool two = pc.n_tiles > 1;
            const int merger = two ? (pc.n_tiles & 1) : 0;
            if (!mine && wg != merger)
                continue; // (no tile here and nothing to write)
#pragma unroll
            for (int h = 0; h < GP; ++h)
            {
#pragma unroll
                for (int x = 16; x >= 1; x >>= 1)
                    l[h] += __shfl_xor_sync(0xffffffffu, l[h], x);
            }
            float* rl = red_l + (wg * 2 + (pl & 1)) * 4 * GP; // two buffers in turn: one barrier per piece is enough
            ++pl;
            if (lane == 0)
            {
#pragma unroll
                for (int h = 0; h < GP; ++h)
                    rl[wl * GP + h] = l[h];
            }
            group_sync(wg);
            WS_SINCE(1, t_epi); // (l reduction and group barrier)
            const int par = hx & 1;
            if (wg != merger)
            {
                ok = ok && WS_TIMED(13, ws_wait_warp(&x_empty[par], ((hx >> 1) & 1) ^ 1, sh));
                if (ok)
                {
                    float* xb = xbuf + par * GP * TT;
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        xb[h * TT + row] = fmaf(o[GP + h], LOW, o[h]);
                    if (row == 0)
                    {
#pragma unroll
                        for (int h = 0; h < GP; ++h)
                        {
                            mref_x[par * GP + h] = mref[h];
                            lsum_x[par * GP + h] = rl[h] + rl[GP + h] + rl[2 * GP + h] + rl[3 * GP + h];
                        }
                    }
                    mbar_arrive(&x_full[par]);
                }
                ++hx;
                continue;
            }
            if (two)
            {
                ok = ok && WS_TIMED(13, ws_wait_warp(&x_full[par], (hx >> 1) & 1, sh));
                ++hx;
            }
            if (!ok)
                continue; // (aborting: the next barrier of the group ends the role)
            {
                const float* xb = xbuf + par * GP * TT;
#pragma unroll
                for (int h = 0; h < GP; ++h)
                {
                    if (h < G)
                    {
                        const float la = rl[h] + rl[GP + h] + rl[2 * GP + h] + rl[3 * GP + h];
                        const float oa = fmaf(o[GP + h], LOW, o[h]);
                        float m = mref[h], lt = la, ov = oa;
                        if (two)
                        {
                            const float mb = mref_x[par * GP + h];
                            m = fmaxf(mref[h], mb);
                            const float fa = fast_exp2(mref[h] - m), fb = fast_exp2(mb - m);
                            lt = la * fa + lsum_x[par * GP + h] * fb;
                            ov = oa * fa + xb[h * TT + row] * fb;
                        }
                        ov *= deq;
                        const size_t orow = (size_t) pc.b * a.num_heads + head0 + h;
                        if (pc.final_out)
                        {
                            reinterpret_cast<T*>(a.out)[orow * DH + row] = TypeOps<T>::from_float(ov / lt);
                        }
                        else
                        {
                            a.part_o[(orow * a.nsplit + pc.slot) * DH + row] = ov;
                            if (row == 0)
                                a.part_ml[orow * a.nsplit + pc.slot] = make_float2(m, lt);
                        }
                    }
                }
                if (two)
                    mbar_arrive(&x_empty[par]);
            }
            WS_SINCE(22, t_epi);
        }
    }

#ifdef DX_TOKWS_TRACE
    if (lane == 0 && (warp == 0 || (warp >= 8 && warp <= 12)))
    {
        ws_acc[16 + (warp >= 8 ? (warp < 13 ? warp - 7 : 7) : 0)] = clock64() - ws_start; // role life: 16 softmax, 17 K, 18 V, 19 S MMA, 20 aux, 21 O MMA
        unsigned long long* ctr = reinterpret_cast<unsigned long long*>(a.status + 32);
        for (int i = 0; i < 24; ++i)
            if (ws_acc[i])
                atomicAdd(ctr + i, (unsigned long long) ws_acc[i]);
    }
#endif
    // ---- every role ends here: free tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Tr::TMEM_COLS));
}

} // namespace dx
