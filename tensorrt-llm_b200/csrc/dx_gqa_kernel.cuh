// Grouped-head (GQA / MQA) decode attention over an 8-bit paged KV cache on the tensor cores.
//
// One CTA per (split-K partition, kv head x 16-head slice of its q group, sequence).  The q heads
// that share the kv head form the M dimension of S = Q K^T, so every cache byte is fetched from
// HBM once for the whole group.  The per-tensor dequantisation scale is never applied per element:
// it is folded into the score scale and into the final normalisation.
//   FP8 cache : legacy fp8 mma.sync is emulated on sm_100a (conversions + f16 MMA + extra adds), so
//               the bytes are converted in registers with packed cvt.f16x2.e4m3x2 (exact, one
//               instruction per two bytes) and fed to m16n8k16 f16 MMAs with fp32 accumulation;
//               Q and P stay 16-bit.
//   INT8 cache: bytes go into m16n8k32 s8 MMAs as stored; Q and P are split into a high and a low
//               8-bit part so that they keep ~15 / ~14 significant bits.
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

// CTAs per SM the kernel is built for: 3 (with a 2-stage ring) where the register budget allows
// it - more resident warps hide the fixed instruction latencies better than a deeper ring - else 2
// (3-stage ring).  WARPS = 6: the stream-K form of the FP8 / Dh 128 kernel, two CTAs of six warps with 2-stage
// rings - the same twelve warps and 192 KB of rings per SM as three CTAs of four, but when a CTA has finished its
// range the other one still keeps 96 KB in flight instead of 64 KB (c4: 140.5 us against 142.2 us in the same run;
// one CTA of twelve warps: 152 us, every piece boundary then stalls the whole SM).
template <int CACHE, int DH, bool H16, int WARPS = 4>
constexpr int gqa_min_blocks()
{
    return WARPS == 6 ? 2 : (CACHE == CACHE_FP8 && DH == 128 && !H16) ? 3 : 2;
}

template <int DH, int MINB, int WARPS = 4>
struct GqaTraits
{
    static constexpr int TG = 32;           // tokens per stage (per warp)
    static constexpr int KS = DH / 32;      // k-steps of Q K^T
    static constexpr int MT = DH / 16;      // m-tiles of O^T
    static constexpr int NW = DH / 32;      // 32-bit words of V per row per thread
    static constexpr int QV = DH / 4;       // q elements per thread per head row
    static constexpr int SLAB = TG * DH;    // bytes of K (or V) per stage
    static constexpr int STAGE_BYTES = 2 * SLAB;
    static constexpr int STAGES = ((MINB >= 3 || WARPS == 6) && DH == 128) ? 2 : 3;
    static constexpr int NWARPS = WARPS;
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

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two e4m3 bytes (one 16-bit half of a word) -> f16x2, exact.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_lo(uint32_t w)
{
    uint32_t r;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(r) : "r"(w));
    return r;
}

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_hi(uint32_t w)
{
    uint32_t r;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(r) : "r"(w));
    return r;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
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

// Weight of the high 8-bit part relative to the low one on the integer path.
static constexpr int kLoWeight = 128;

// Four values (already scaled into the 8-bit range) -> one word of high parts, one of low parts.
// FP8: packed conversions, residual taken in f16x2 (exact: hi has 4 significant bits).
// INT8: round-to-nearest through the 1.5 * 2^23 magic constant; the low byte of the biased float is
// the two's-complement integer.
template <int CACHE>
__device__ __forceinline__ void split4(float x0, float x1, float x2, float x3, uint32_t& hi, uint32_t& lo)
{
    if constexpr (CACHE == CACHE_FP8)
    {
        uint16_t h01, h23, l01, l23;
        uint32_t f01, f23, x01, x23;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h01) : "f"(x1), "f"(x0));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h23) : "f"(x3), "f"(x2));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(f01) : "h"(h01));
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(f23) : "h"(h23));
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(x01) : "f"(x1), "f"(x0));
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(x23) : "f"(x3), "f"(x2));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(x01) : "r"(x01), "r"(f01));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(x23) : "r"(x23), "r"(f23));
        asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(l01) : "r"(x01));
        asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(l23) : "r"(x23));
        hi = (uint32_t) h01 | ((uint32_t) h23 << 16);
        lo = (uint32_t) l01 | ((uint32_t) l23 << 16);
    }
    else
    {
        constexpr float M = 12582912.f;
        const float y0 = x0 + M, y1 = x1 + M, y2 = x2 + M, y3 = x3 + M;
        const float z0 = fmaf(x0 - (y0 - M), (float) kLoWeight, M), z1 = fmaf(x1 - (y1 - M), (float) kLoWeight, M);
        const float z2 = fmaf(x2 - (y2 - M), (float) kLoWeight, M), z3 = fmaf(x3 - (y3 - M), (float) kLoWeight, M);
        hi = __byte_perm(__byte_perm(__float_as_uint(y0), __float_as_uint(y1), 0x0040),
            __byte_perm(__float_as_uint(y2), __float_as_uint(y3), 0x0040), 0x5410);
        lo = __byte_perm(__byte_perm(__float_as_uint(z0), __float_as_uint(z1), 0x0040),
            __byte_perm(__float_as_uint(z2), __float_as_uint(z3), 0x0040), 0x5410);
    }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// FEAT = 1: the feature form (classic launches only).  Beam search: cache slot s of sequence b is read from sequence
// request * beam_width + (s < context_lengths[b] ? 0 : cache_indir[b][s]), so every token row of a group has its own
// source block (decoderMaskedMultiheadAttentionTemplate.h:1497-1498, :2063-2078).  Cyclic cache: the kernel walks
// slots 0 .. min(past, window) - 1 as they are (:1493).  The new token is taken from the QKV row as it will be stored and
// appended by kv_append_token_kernel behind this kernel (its slot may be one that is read in this step).  ALiBi: score += slope[head] * (s - past), nothing for the new token (:1797, :2026).
// FEAT = 2: several new tokens per sequence (the reference's Medusa mode; classic launches only).  The new tokens are in
// the cache already (kv_append_token_kernel runs first); the rows of a kv head are its q_len x G (token, head) pairs,
// token-major, cut into 16-row slices (hg), so one pass over the cache serves 16 of them; row (t, h) attends to
// the cache entries before the step and to new token j where bit j of its packed mask row is set.
template <typename T, int CACHE, int DH, bool H16, int WARPS = 4, int FEAT = 0>
__global__ void __launch_bounds__(WARPS * 32, gqa_min_blocks<CACHE, DH, H16, WARPS>())
    gqa_decode_kernel(const AttnArgs a, const int hgroups, const __grid_constant__ SkSchedule sk)
{
    static_assert(CACHE == CACHE_INT8 || CACHE == CACHE_FP8, "8-bit caches only");
    using Tr = GqaTraits<DH, gqa_min_blocks<CACHE, DH, H16, WARPS>(), WARPS>;
    constexpr int TG = Tr::TG, KS = Tr::KS, MT = Tr::MT, NW = Tr::NW, QV = Tr::QV;
    constexpr int SLAB = Tr::SLAB, STAGES = Tr::STAGES, NWARPS = Tr::NWARPS;
    constexpr int NR = H16 ? 2 : 1;  // head-row halves in use (rows g, and rows g + 8)
    constexpr bool IS_FP8 = CACHE == CACHE_FP8;
    // Score accumulator sets: only 16 heads on the integer path need the low part separately
    // (with <= 8 heads the low parts of Q sit in rows 8..15 of the same MMA).
    constexpr int NSA = (H16 && !IS_FP8) ? 2 : 1;
    constexpr int NCP = (DH == 128) ? 2 : 4; // distinct per-lane destination offsets of the copies
    using Acc = typename std::conditional<IS_FP8, float, int>::type;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = a.num_heads / a.num_kv_heads;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    // Launched as a programmatic dependent of the kernel in front of it (the previous step's merge), the CTAs become
    // resident while that kernel drains; nothing in global memory is touched before it has completed.  (Without
    // that launch attribute the wait returns at once.)
    griddep_wait();

    // Work of this CTA.  Classic launch: one piece, the (partition, kv-head slice, sequence) of its grid
    // position.  Stream-K launch (a.streamk): a contiguous range of 32-token groups of the whole batch
    // (SkSchedule), i.e. a few pieces of consecutive rows, every CTA the same amount.
    SkCursor cur;
    if (a.streamk)
    {
        if (!sk_begin(sk, (int) blockIdx.x, cur))
            return;
    }
    else
    {
        int cs, ct, np;
        partition_of(FEAT == 1 ? attended_tokens(a.seq_len[blockIdx.z], a.cyclic_window) : a.seq_len[blockIdx.z], a.chunk_tokens,
            (int) blockIdx.x, cs, ct, np);
        if (np > (int) gridDim.x && blockIdx.x == 0 && threadIdx.x == 0)
            report_status(a.status, STATUS_PLAN_EXCEEDED); // the tokens beyond the last partition are not attended to
        if ((int) blockIdx.x >= np)
            return; // ragged batch: this sequence uses fewer partitions
    }
    griddep_launch_dependents(); // the merge kernel may be scheduled; it waits for this grid to finish

    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int BAR_OFF = (Tr::RING_BYTES > Tr::MERGE_BYTES ? Tr::RING_BYTES : Tr::MERGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFF) + warp * STAGES;
    const uint32_t ring_u32 = smem_u32(smem) + warp * (STAGES * Tr::STAGE_BYTES);

    if (lane == 0)
    {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            mbar_init(&bars[s], 32);
        fence_mbar_init();
    }
    __syncwarp();

    int ring_base = 0; // groups this warp has put through its ring so far (stage / phase bookkeeping across pieces)
    for (;;)
    {
        // ---- this piece: row (b, hk, hg), tokens [chunk_start, chunk_start + ctoks), result slot `chunk` ----
        int b, hk, hg, chunk, chunk_start, ctoks;
        bool final_out;
        if (a.streamk)
        {
            int y, g0, ng;
            sk_piece(sk, cur, b, y, g0, ng, chunk, final_out);
            hk = y / hgroups, hg = y % hgroups;
            chunk_start = g0 * TG;
            ctoks = ng * TG;
        }
        else
        {
            int np;
            chunk = blockIdx.x, hk = blockIdx.y / hgroups, hg = blockIdx.y % hgroups, b = blockIdx.z;
            partition_of(FEAT == 1 ? attended_tokens(a.seq_len[b], a.cyclic_window) : a.seq_len[b], a.chunk_tokens, chunk,
                chunk_start, ctoks, np);
            final_out = a.nsplit == 1;
        }
        const int nh = min(16, (FEAT == 2 ? G * a.q_len : G) - hg * 16); // q rows handled in this piece
        const int head0 = hk * G + hg * 16;  // first of them (FEAT = 2: see row_token / row_head)
        // FEAT = 2: row hl of the slice is new token (hg * 16 + hl) / G, head (hg * 16 + hl) % G of the kv head
        auto q_row_of = [&](int hl) -> size_t
        {
            if constexpr (FEAT == 2)
            {
                const int R = hg * 16 + hl, tk = R / G;
                return ((size_t) b * a.q_len + tk) * (size_t) ((a.num_heads + 2 * a.num_kv_heads) * DH) + (size_t) (hk * G + R - tk * G) * DH;
            }
            else
                return (size_t) b * (size_t) ((a.num_heads + 2 * a.num_kv_heads) * DH) + (size_t) (head0 + hl) * DH;
        };
        auto out_row_of = [&](int hl) -> size_t
        {
            if constexpr (FEAT == 2)
            {
                const int R = hg * 16 + hl, tk = R / G;
                return ((size_t) b * a.q_len + tk) * a.num_heads + (size_t) (hk * G + R - tk * G);
            }
            else
                return (size_t) b * a.num_heads + head0 + hl;
        };
        // The q rows of this thread are requested before anything else of the piece: behind the first ring
        // stages of K / V (tens of KB per warp) the same loads would wait for all of those bytes.
        const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
        const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
        uint4 q_raw[NR][QV / 8];
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
            const int hl = g + 8 * r; // head within this CTA
            const T* qp = reinterpret_cast<const T*>(a.qkv) + q_row_of(min(hl, nh - 1)) + t * QV;
#pragma unroll
            for (int i = 0; i < QV / 8; ++i)
                q_raw[r][i] = *reinterpret_cast<const uint4*>(qp + 8 * i);
        }
        const float deq = __ldg(a.scale_quant_orig);
        // (feature form: `total` counts the cache slots walked plus the new token; past_true is the real history)
        const int past_true = a.seq_len[b] - 1;
        const int total = FEAT == 1 ? attended_tokens(past_true + 1, a.cyclic_window) : past_true + 1;
        if (a.streamk && total > (int) cur.nb * TG && threadIdx.x == 0)
            report_status(a.status, STATUS_PLAN_EXCEEDED); // longer than the host length the ranges were laid out for
        ctoks = max(0, min(ctoks, total - chunk_start)); // the schedule counts host lengths; the device length decides
        const int n_groups = (ctoks + TG - 1) / TG;
        // (FEAT = 2: nothing is staged, every token up to `total` is read from the cache)
        const int new_pos = FEAT == 2 ? total : total - 1;
        // FEAT = 2: packed mask words of this thread's rows (q_len <= 64) and the first new token
        uint32_t mw[NR][2];
        int first_new = 0;
        if constexpr (FEAT == 2)
        {
            first_new = total - a.q_len;
            const int words = (a.q_len + 31) >> 5;
#pragma unroll
            for (int r = 0; r < NR; ++r)
            {
                const int tk = (hg * 16 + min(g + 8 * r, nh - 1)) / G;
                const int32_t* mrow = a.packed_mask + ((size_t) b * a.q_len + tk) * words;
                mw[r][0] = (uint32_t) __ldg(mrow);
                mw[r][1] = words > 1 ? (uint32_t) __ldg(mrow + 1) : 0u;
            }
        }

        const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
        const int64_t* vrow = krow + a.max_blocks_per_seq;
        const size_t head_off = (size_t) hk * ((size_t) DH << tpb_log2);
        // feature form: source of a slot (beam search) and ALiBi slopes of this thread's head rows (log2 units)
        int seq0 = b, ctx0 = 0;
        const int32_t* indir = nullptr;
        float slope[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r)
            slope[r] = 0.f;
        if constexpr (FEAT == 1)
        {
            if (a.cache_indir != nullptr && a.beam_width > 1)
            {
                seq0 = (b / a.beam_width) * a.beam_width;
                ctx0 = (a.cyclic_window > 0 && past_true > a.cyclic_window) ? 0 : a.context_lengths[b]; // wrapped: all via the table
                indir = a.cache_indir + (size_t) b * a.max_attention_window;
            }
            if (a.alibi_slopes != nullptr)
            {
#pragma unroll
                for (int r = 0; r < NR; ++r)
                    slope[r] = TypeOps<T>::to_float(reinterpret_cast<const T*>(a.alibi_slopes)[head0 + min(g + 8 * r, nh - 1)])
                        * 1.4426950408889634f;
            }
        }

        // Per-lane constant destination offsets of the 16-byte copies (copy j of a slab moves linear
        // bytes [(lane + 32 j) * 16, +16)).
        uint32_t cdst[NCP];
#pragma unroll
        for (int j = 0; j < NCP; ++j)
            cdst[j] = swz<DH>((uint32_t) (lane + 32 * j) * 16);

        // Every lane copies its share of the i-th group of this warp into ring stage (ring_base + i) % STAGES.
        auto issue = [&](int i)
        {
            const int gi = warp + NWARPS * i;
            const int t0 = chunk_start + gi * TG;
            const int rows = new_pos - t0; // rows already in the cache (>= TG for all but the last group)
            const uint32_t kdst = ring_u32 + ((ring_base + i) % STAGES) * Tr::STAGE_BYTES;
            if constexpr (FEAT == 1)
            {
                // every 16-byte piece looks up the block of its own token row
#pragma unroll
                for (int j = 0; j < SLAB / 512; ++j)
                {
                    const uint32_t d = (DH == 128) ? cdst[j & 1] + (j >> 1) * 1024 : cdst[j];
                    const int lin = (lane + 32 * j) * 16;
                    const int s = t0 + lin / DH;
                    const bool ok = s < new_pos;
                    const int sc = ok ? s : 0;
                    const int seq = (indir != nullptr && sc >= ctx0) ? seq0 + __ldg(indir + sc) : seq0;
                    const int64_t* srow = a.block_ptrs + (int64_t) seq * 2 * a.max_blocks_per_seq;
                    const size_t o = head_off + (size_t) (sc & tpb_mask) * DH + lin % DH;
                    const char* ks = reinterpret_cast<const char*>(
                        table_entry(srow, sc >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + o;
                    const char* vs = reinterpret_cast<const char*>(
                        table_entry(srow + a.max_blocks_per_seq, sc >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + o;
                    cp_async16_zfill_u32(kdst + d, ks, ok ? 16u : 0u);
                    cp_async16_zfill_u32(kdst + SLAB + d, vs, ok ? 16u : 0u);
                }
                cp_async_mbar_arrive_noinc(&bars[(ring_base + i) % STAGES]);
                return;
            }
            const size_t off = head_off + (size_t) (t0 & tpb_mask) * DH + lane * 16;
            const char* kb = reinterpret_cast<const char*>(table_entry(krow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            const char* vb = reinterpret_cast<const char*>(table_entry(vrow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            if (rows >= TG)
            {
#pragma unroll
                for (int j = 0; j < SLAB / 512; ++j)
                {
                    const uint32_t d = (DH == 128) ? cdst[j & 1] + (j >> 1) * 1024 : cdst[j];
                    cp_async16_u32(kdst + d, kb + j * 512);
                    cp_async16_u32(kdst + SLAB + d, vb + j * 512);
                }
            }
            else
            {
                // last group of the sequence: rows at and behind the new token are zero-filled
                const int valid_bytes = rows > 0 ? rows * DH : 0;
#pragma unroll
                for (int j = 0; j < SLAB / 512; ++j)
                {
                    const uint32_t d = (DH == 128) ? cdst[j & 1] + (j >> 1) * 1024 : cdst[j];
                    const bool ok = (lane + 32 * j) * 16 < valid_bytes;
                    cp_async16_zfill_u32(kdst + d, ok ? kb + j * 512 : kb, ok ? 16u : 0u);
                    cp_async16_zfill_u32(kdst + SLAB + d, ok ? vb + j * 512 : vb, ok ? 16u : 0u);
                }
            }
            cp_async_mbar_arrive_noinc(&bars[(ring_base + i) % STAGES]);
        };

        const int my_groups = (n_groups > warp) ? (n_groups - warp + NWARPS - 1) / NWARPS : 0;
        for (int i = 0; i < min(STAGES, my_groups); ++i)
            issue(i);

        // ---- Q: load the head rows, scale each row into the 8-bit range, split into high and low
        // parts and pack straight into A fragments.  The k index of every MMA is a fixed permutation
        // of Dh chosen so that a K fragment is one (Dh 64) or two (Dh 128) 16-byte shared loads.
        //   <= 8 heads : one fragment set, rows 0..7 = high parts, rows 8..15 = low parts of head g
        //   16 heads   : two fragment sets (high, low), rows = heads g and g + 8 ----
        // FP8 cache: Q stays 16-bit (f16 A fragments, one k16 step per 4 channels of a thread);
        // INT8 cache: 8-bit high/low fragments as described above.
        constexpr int KS16 = DH / 16;
        uint32_t qa[IS_FP8 ? 1 : NR][IS_FP8 ? KS16 : KS][4];
        float sfac[NR]; // accumulator -> score in log2 units, per head-row half
#pragma unroll
        for (int r = 0; r < NR; ++r)
        {
            float qv[QV];
            const int hl = g + 8 * r; // head within this CTA
            if (hl < nh)
            {
#pragma unroll
                for (int i = 0; i < QV; i += 8)
                {
                    const uint4 raw = q_raw[r][i / 8];
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
            if constexpr (IS_FP8)
            {
                // k16 step j of this thread covers channels 4j .. 4j+3 of its QV-channel slice:
                // (4j, 4j+1) -> k slots (2t, 2t+1), (4j+2, 4j+3) -> k slots (2t+8, 2t+9).
#pragma unroll
                for (int j = 0; j < KS16; ++j)
                {
                    qa[0][j][r] = pack_f16x2(qv[4 * j] * qmul, qv[4 * j + 1] * qmul);
                    qa[0][j][2 + r] = pack_f16x2(qv[4 * j + 2] * qmul, qv[4 * j + 3] * qmul);
                    if constexpr (!H16)
                    {
                        qa[0][j][1] = 0u;
                        qa[0][j][3] = 0u;
                    }
                }
            }
            else
            {
#pragma unroll
                for (int s = 0; s < KS; ++s)
                {
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                    {
                        // elements of this thread that feed the low-k (half 0) or high-k (half 1) registers of k-step s
                        const int base = (DH == 128) ? (16 * half + 4 * s) : (8 * s + 4 * half);
                        uint32_t whi, wlo;
                        split4<CACHE>(qv[base] * qmul, qv[base + 1] * qmul, qv[base + 2] * qmul, qv[base + 3] * qmul, whi, wlo);
                        if constexpr (H16)
                        {
                            qa[0][s][2 * half + r] = whi; // set 0 = high parts, register = row half r
                            qa[1][s][2 * half + r] = wlo; // set 1 = low parts
                        }
                        else
                        {
                            qa[0][s][2 * half] = whi;     // rows 0..7
                            qa[0][s][2 * half + 1] = wlo; // rows 8..15
                        }
                    }
                }
            }
        }

        // Per-thread shared-memory offsets of the fragment loads (inside a K / V slab).
        uint32_t koff[4], voff[8];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
            koff[nt] = swz<DH>((uint32_t) sigma_row<DH>(nt, g) * DH + t * (DH / 4));
#pragma unroll
        for (int i = 0; i < 8; ++i)
            voff[i] = swz<DH>((uint32_t) sigma_row<DH>(i >> 1, 2 * t + (i & 1)) * DH + g * (DH / 8));

        float m[NR], l[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r)
            m[r] = -INFINITY, l[r] = 0.f;
        float of[MT][NR][4]; // O^T fragments: [m-tile][head half][c0..c3]
        int oi[IS_FP8 ? 1 : 2][IS_FP8 ? 1 : MT][NR][4]; // integer path: pending high / low sums
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                {
                    of[mt][r][c] = 0.f;
                    if constexpr (!IS_FP8)
                        oi[0][mt][r][c] = 0, oi[1][mt][r][c] = 0;
                }
        // integer path: move the pending integer sums into the fp32 running sums
        auto fold = [&]()
        {
            if constexpr (!IS_FP8)
            {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int r = 0; r < NR; ++r)
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                        {
                            of[mt][r][c] += (float) (oi[0][mt][r][c] * kLoWeight + oi[1][mt][r][c]);
                            oi[0][mt][r][c] = 0;
                            oi[1][mt][r][c] = 0;
                        }
            }
        };

        bool timed_out = false;
        for (int i = 0; i < my_groups; ++i)
        {
            const int s = (ring_base + i) % STAGES;
            const uint32_t parity = ((ring_base + i) / STAGES) & 1;
            const uint32_t kbuf = ring_u32 + s * Tr::STAGE_BYTES;
            const uint32_t vbuf = kbuf + SLAB;
            if (!mbar_wait_bounded(&bars[s], parity, a.status))
            {
                timed_out = true;
                break;
            }
            const int gi = warp + NWARPS * i;
            const int t0 = chunk_start + gi * TG;
            const int lim = total - t0; // valid tokens in this group if < TG
            if (FEAT != 2 && new_pos < t0 + TG)
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
                    const uint32_t lin = swz<DH>((uint32_t) r_new * DH + lane * 16);
                    unsigned char* stage = smem + warp * (STAGES * Tr::STAGE_BYTES) + s * Tr::STAGE_BYTES;
                    *reinterpret_cast<uint4*>(stage + lin) = kq;
                    *reinterpret_cast<uint4*>(stage + SLAB + lin) = vq;
                    if (FEAT == 0 && hg == 0) // (feature form: kv_append_token_kernel stores the token behind this kernel)
                    {
                        const size_t off = head_off + (size_t) (new_pos & tpb_mask) * DH + lane * 16;
                        char* kb = reinterpret_cast<char*>(table_entry(krow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                        char* vb = reinterpret_cast<char*>(table_entry(vrow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                        *reinterpret_cast<uint4*>(kb) = kq;
                        *reinterpret_cast<uint4*>(vb) = vq;
                    }
                }
                __syncwarp();
            }

            // ---- S = Q K^T for the head rows x 32 tokens ----
            Acc sacc[NSA][4][4];
#pragma unroll
            for (int x = 0; x < NSA; ++x)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        sacc[x][nt][c] = 0;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
            {
                uint32_t kw[2 * KS];
                {
                    const uint4 v0 = lds128(kbuf + koff[nt]);
                    kw[0] = v0.x, kw[1] = v0.y, kw[2] = v0.z, kw[3] = v0.w;
                    if constexpr (DH == 128)
                    {
                        const uint4 v1 = lds128(kbuf + (koff[nt] ^ 16u));
                        kw[4] = v1.x, kw[5] = v1.y, kw[6] = v1.z, kw[7] = v1.w;
                    }
                }
                if constexpr (IS_FP8)
                {
                    // word j of this thread's K bytes = channels 4j..4j+3 = one k16 step
#pragma unroll
                    for (int j = 0; j < KS16; ++j)
                        mma_f16(sacc[0][nt], qa[0][j], e4m3x2_to_f16x2_lo(kw[j]), e4m3x2_to_f16x2_hi(kw[j]));
                }
                else
                {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks)
                    {
                        const uint32_t b0 = (DH == 128) ? kw[ks] : kw[2 * ks];
                        const uint32_t b1 = (DH == 128) ? kw[4 + ks] : kw[2 * ks + 1];
                        mma_s8(sacc[0][nt], qa[0][ks], b0, b1);
                        if constexpr (H16)
                            mma_s8(sacc[1][nt], qa[1][ks], b0, b1);
                    }
                }
            }

            // ---- online softmax over the 32 tokens ----
            float p[4][2 * NR];
            float mx[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r)
                mx[r] = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
            {
#pragma unroll
                for (int c = 0; c < 2 * NR; ++c)
                {
                    float sv;
                    if constexpr (IS_FP8)
                        sv = sacc[0][nt][c]; // rows g (c = 0, 1) and g + 8 (c = 2, 3)
                    else if constexpr (H16)
                        sv = (float) (sacc[0][nt][c] * kLoWeight + sacc[NSA - 1][nt][c]);
                    else
                        sv = (float) (sacc[0][nt][c] * kLoWeight + sacc[0][nt][c + 2]);
                    p[nt][c] = sv * sfac[c >> 1];
                    if constexpr (FEAT == 1)
                    {
                        const int tok = t0 + sigma_row<DH>(nt, 2 * t + (c & 1));
                        p[nt][c] = fmaf(slope[c >> 1], tok == new_pos ? 0.f : (float) (tok - past_true), p[nt][c]);
                    }
                }
            }
            if constexpr (FEAT == 2)
            {
                if (t0 + TG > first_new) // the group holds new tokens: each row sees those its mask row names
                {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int c = 0; c < 2 * NR; ++c)
                        {
                            const int j = t0 + sigma_row<DH>(nt, 2 * t + (c & 1)) - first_new;
                            if (j >= 0 && j < 64 && (((j < 32 ? mw[c >> 1][0] : mw[c >> 1][1]) >> (j & 31)) & 1u) == 0u)
                                p[nt][c] = -INFINITY;
                        }
                }
            }
            if (lim < TG)
            {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int c = 0; c < 2 * NR; ++c)
                        if (sigma_row<DH>(nt, 2 * t + (c & 1)) >= lim)
                            p[nt][c] = -INFINITY;
            }
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int c = 0; c < 2 * NR; ++c)
                    mx[c >> 1] = fmaxf(mx[c >> 1], p[nt][c]);
            float alpha[NR], msub[NR];
            bool changed = false;
#pragma unroll
            for (int r = 0; r < NR; ++r)
            {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r]);
                // (FEAT = 2: under its mask a row may have seen nothing yet; -inf minus -inf must not reach exp2)
                msub[r] = (FEAT == 2 && m_new == -INFINITY) ? 0.f : m_new;
                alpha[r] = fast_exp2(m[r] - msub[r]);
                changed |= m_new != m[r];
                m[r] = m_new;
                l[r] *= alpha[r];
            }
            // FP8 cache: P as f16 (scaled by 1024 to stay clear of f16 subnormals), pb[r][k16 step][b0/b1];
            // INT8 cache: P split into high / low 8-bit parts, pb[r][hi/lo][b0/b1].
            constexpr float PSCALE = IS_FP8 ? 1024.f : 127.f;
            uint32_t pb[NR][2][2];
#pragma unroll
            for (int r = 0; r < NR; ++r)
            {
#pragma unroll
                for (int kh = 0; kh < 2; ++kh)
                {
                    float pv[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                    {
                        pv[q4] = fast_exp2(p[2 * kh + (q4 >> 1)][2 * r + (q4 & 1)] - msub[r]);
                        l[r] += pv[q4];
                    }
                    if constexpr (IS_FP8)
                    {
                        pb[r][kh][0] = pack_f16x2(pv[0] * PSCALE, pv[1] * PSCALE);
                        pb[r][kh][1] = pack_f16x2(pv[2] * PSCALE, pv[3] * PSCALE);
                    }
                    else
                    {
                        split4<CACHE>(pv[0] * PSCALE, pv[1] * PSCALE, pv[2] * PSCALE, pv[3] * PSCALE, pb[r][0][kh], pb[r][1][kh]);
                    }
                }
            }

            // ---- rescale the running O^T when a row maximum moved (its columns are heads 2t, 2t+1 (+8)) ----
            if (__any_sync(0xffffffffu, changed))
            {
                fold();
#pragma unroll
                for (int r = 0; r < NR; ++r)
                {
                    const float a0 = __shfl_sync(0xffffffffu, alpha[r], 8 * t);
                    const float a1 = __shfl_sync(0xffffffffu, alpha[r], 8 * t + 4);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                    {
                        of[mt][r][0] *= a0;
                        of[mt][r][1] *= a1;
                        of[mt][r][2] *= a0;
                        of[mt][r][3] *= a1;
                    }
                }
            }
            else if ((i & 255) == 255)
            {
                fold(); // keeps the pending integer sums far from overflow on very long partitions
            }

            // ---- O^T += V^T P^T ----
            uint32_t tr[2][NW][4]; // [k half][word][byte column] -> one A register each
#pragma unroll
            for (int kh = 0; kh < 2; ++kh)
            {
                uint32_t rv[4][NW];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                {
                    if constexpr (DH == 128)
                    {
                        const uint4 v = lds128(vbuf + voff[4 * kh + q4]);
                        rv[q4][0] = v.x, rv[q4][1] = v.y, rv[q4][2] = v.z, rv[q4][3] = v.w;
                    }
                    else
                    {
                        const uint2 v = lds64(vbuf + voff[4 * kh + q4]);
                        rv[q4][0] = v.x, rv[q4][1] = v.y;
                    }
                }
#pragma unroll
                for (int w = 0; w < NW; ++w)
                    transpose4x4(rv[0][w], rv[1][w], rv[2][w], rv[3][w], tr[kh][w]);
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
                        // two k16 steps: tokens of k half 0 (av[0], av[1]) and of k half 1 (av[2], av[3])
                        const uint32_t a0[4] = {e4m3x2_to_f16x2_lo(av[0]), e4m3x2_to_f16x2_lo(av[1]),
                            e4m3x2_to_f16x2_hi(av[0]), e4m3x2_to_f16x2_hi(av[1])};
                        const uint32_t a1[4] = {e4m3x2_to_f16x2_lo(av[2]), e4m3x2_to_f16x2_lo(av[3]),
                            e4m3x2_to_f16x2_hi(av[2]), e4m3x2_to_f16x2_hi(av[3])};
                        mma_f16(of[mt][r], a0, pb[r][0][0], pb[r][0][1]);
                        mma_f16(of[mt][r], a1, pb[r][1][0], pb[r][1][1]);
                    }
                    else
                    {
                        mma_s8(oi[0][mt][r], av, pb[r][0][0], pb[r][0][1]);
                        mma_s8(oi[1][mt][r], av, pb[r][1][0], pb[r][1][1]);
                    }
                }
            }

            __syncwarp(); // every lane is done reading this stage
            if (i + STAGES < my_groups)
                issue(i + STAGES);
        }
        fold();

        if (timed_out)
        {
            if (lane == 0)
                report_status(a.status, STATUS_TIMEOUT);
            asm volatile("cp.async.wait_all;" ::: "memory"); // the ring is reused below and the CTA then exits
        }

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

        constexpr float ONORM = IS_FP8 ? (1.f / 1024.f) : (1.f / (127.f * kLoWeight));
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
            const size_t row = out_row_of(head);
            if (final_out)
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
        // ---- next piece (the merge scratch above aliases the rings: everybody must be done reading it) ----
        ring_base += my_groups;
        const int stop = __syncthreads_or(timed_out ? 1 : 0);
        if (!a.streamk || stop || !sk_next(sk, cur))
            break;
    }
}

} // namespace dx
