// Grouped-head (GQA / MQA) decode attention over a 16-bit (fp16 / bf16) paged KV cache on the tensor cores.
//
// One CTA per (split-K partition, kv head x 16-head slice of its q group, sequence).  The q heads that share
// the kv head are the M rows of S = Q K^T and of O = P V (mma.sync.m16n8k16, fp32 accumulation), so every cache
// byte is fetched from HBM once for the whole group instead of once per q head.  Cache rows are used as stored:
// K rows are the "col" B operand of Q K^T (ldmatrix), V rows the B operand of P V (ldmatrix.trans); the S
// accumulators of two 8-token tiles are exactly the A fragment of P for a 16-token k-step.
//
// Each of the 4 warps owns every 4th 16-token group of the partition and runs its own online softmax; groups are
// staged through a warp-private 3-stage ring filled with 16-byte cp.async copies (16-byte chunks XOR-swizzled
// with the row number so that both ldmatrix patterns are bank-conflict free) whose completion is tracked by
// mbarriers (cp.async.mbarrier.arrive.noinc).  Every wait is bounded.
//
// Replaces, for an unquantised cache, the XQA kernels (binary-only in the reference, dispatched from
//   cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderXQAImplPrecompiled.cpp:263-374)
// and the MMHA kernel for grouped heads (decoderMaskedMultiheadAttentionTemplate.h:1303).
#pragma once

#include <type_traits>

#include "dx_common.cuh"

namespace dx
{

template <int DH>
struct Gqa16Traits
{
    static constexpr int TG = 16;                 // tokens per stage (per warp)
    static constexpr int ROW = DH * 2;            // bytes of a token row
    static constexpr int CPR = ROW / 16;          // 16-byte chunks per row
    static constexpr int SLAB = TG * ROW;         // bytes of K (or V) per stage
    static constexpr int STAGE_BYTES = 2 * SLAB;
    static constexpr int STAGES = DH == 256 ? 2 : 3; // (Dh 256: 16 KB per stage and warp, one CTA per SM)
    static constexpr int NWARPS = 4;
    static constexpr int NCP = SLAB / 512;        // 16-byte copies per lane and slab
    static constexpr int RING_BYTES = NWARPS * STAGES * STAGE_BYTES;
    static constexpr int MERGE_BYTES = NWARPS * (16 * DH + 32) * 4;
    static constexpr int SMEM_BYTES = (RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES) + NWARPS * STAGES * 8 + 16;
    static constexpr int MIN_BLOCKS = DH == 256 ? 1 : 2;
};

// Byte offset of 16-byte chunk `chunk` of row `row` inside a slab (chunks swizzled with the row number).
template <int DH>
__device__ __forceinline__ uint32_t sw16(uint32_t row, uint32_t chunk)
{
    return row * (uint32_t) (DH * 2) + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_16bit(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    if constexpr (std::is_same<T, __half>::value)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    else
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// FEAT = 1 / 2: the feature forms, as in gqa_decode_kernel (dx_gqa_kernel.cuh): beam search / cyclic window / ALiBi with
// a per-row source block and the new token appended by kv_append_token_kernel; several new tokens per sequence as
// (token, head) rows under the packed mask.  Classic launches only.
template <typename T, int DH, int FEAT = 0>
__global__ void __launch_bounds__(128, Gqa16Traits<DH>::MIN_BLOCKS) gqa16_decode_kernel(const AttnArgs a, const int hgroups, const __grid_constant__ SkSchedule sk)
{
    using Tr = Gqa16Traits<DH>;
    constexpr int TG = Tr::TG, ROW = Tr::ROW, CPR = Tr::CPR, SLAB = Tr::SLAB, STAGES = Tr::STAGES;
    constexpr int NWARPS = Tr::NWARPS, NCP = Tr::NCP;
    constexpr int KSTEPS = DH / 16; // k-steps of Q K^T
    constexpr int NT = DH / 8;      // n-tiles (8 channels) of O

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = a.num_heads / a.num_kv_heads;
    const int tpb_log2 = a.tpb_log2, tpb_mask = (1 << tpb_log2) - 1;

    // (as a programmatic dependent of the kernel in front of it, the CTA is resident early and waits here)
    griddep_wait();
    // Work of this CTA.  Classic launch: one piece, the (partition, kv-head slice, sequence) of its grid
    // position.  Stream-K launch (a.streamk): a contiguous range of 16-token groups of the whole batch
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
        const int past_true = a.seq_len[b] - 1;
        const int total = FEAT == 1 ? attended_tokens(past_true + 1, a.cyclic_window) : past_true + 1;
        if (a.streamk && total > (int) cur.nb * TG && threadIdx.x == 0)
            report_status(a.status, STATUS_PLAN_EXCEEDED); // longer than the host length the ranges were laid out for
        ctoks = max(0, min(ctoks, total - chunk_start)); // the schedule counts host lengths; the device length decides
        const int n_groups = (ctoks + TG - 1) / TG;
        const int new_pos = FEAT == 2 ? total : total - 1; // (FEAT = 2: nothing is staged, everything comes from the cache)
        const int nh = min(16, (FEAT == 2 ? G * a.q_len : G) - hg * 16); // q rows handled in this piece
        const int head0 = hk * G + hg * 16;  // first of them
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
        // feature forms: source of a slot (beam search), ALiBi slopes of rows g and g + 8 (log2 units), mask words
        int seq0 = b, ctx0 = 0, first_new = 0;
        const int32_t* indir = nullptr;
        float slope[2] = {0.f, 0.f};
        uint32_t mw[2][2] = {{0u, 0u}, {0u, 0u}};
        if constexpr (FEAT == 1)
        {
            if (a.cache_indir != nullptr && a.beam_width > 1)
            {
                seq0 = (b / a.beam_width) * a.beam_width;
                ctx0 = (a.cyclic_window > 0 && past_true > a.cyclic_window) ? 0 : a.context_lengths[b];
                indir = a.cache_indir + (size_t) b * a.max_attention_window;
            }
            if (a.alibi_slopes != nullptr)
            {
#pragma unroll
                for (int r = 0; r < 2; ++r)
                    slope[r] = TypeOps<T>::to_float(reinterpret_cast<const T*>(a.alibi_slopes)[head0 + min(g + 8 * r, nh - 1)])
                        * 1.4426950408889634f;
            }
        }
        if constexpr (FEAT == 2)
        {
            first_new = total - a.q_len;
            const int words = (a.q_len + 31) >> 5;
#pragma unroll
            for (int r = 0; r < 2; ++r)
            {
                const int tk = (hg * 16 + min(g + 8 * r, nh - 1)) / G;
                const int32_t* mrow = a.packed_mask + ((size_t) b * a.q_len + tk) * words;
                mw[r][0] = (uint32_t) __ldg(mrow);
                mw[r][1] = words > 1 ? (uint32_t) __ldg(mrow + 1) : 0u;
            }
        }

        const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
        const int64_t* vrow = krow + a.max_blocks_per_seq;
        const size_t head_off = (size_t) hk * ((size_t) ROW << tpb_log2);

        // Copy j of a slab moves linear bytes [(lane + 32 j) * 16, +16) = chunk (lane + 32 j) % CPR of row (lane + 32 j) / CPR.
        uint32_t cdst[NCP];
#pragma unroll
        for (int j = 0; j < NCP; ++j)
            cdst[j] = sw16<DH>((uint32_t) (lane + 32 * j) / CPR, (uint32_t) (lane + 32 * j) % CPR);

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
                for (int j = 0; j < NCP; ++j)
                {
                    const int piece = lane + 32 * j;
                    const int s = t0 + piece / CPR;
                    const bool ok = s < new_pos;
                    const int sc = ok ? s : 0;
                    const int seq = (indir != nullptr && sc >= ctx0) ? seq0 + __ldg(indir + sc) : seq0;
                    const int64_t* srow = a.block_ptrs + (int64_t) seq * 2 * a.max_blocks_per_seq;
                    const size_t o = head_off + (size_t) (sc & tpb_mask) * ROW + (piece % CPR) * 16;
                    const char* ks = reinterpret_cast<const char*>(
                        table_entry(srow, sc >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + o;
                    const char* vs = reinterpret_cast<const char*>(
                        table_entry(srow + a.max_blocks_per_seq, sc >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + o;
                    cp_async16_zfill_u32(kdst + cdst[j], ks, ok ? 16u : 0u);
                    cp_async16_zfill_u32(kdst + SLAB + cdst[j], vs, ok ? 16u : 0u);
                }
                cp_async_mbar_arrive_noinc(&bars[(ring_base + i) % STAGES]);
                return;
            }
            const size_t off = head_off + (size_t) (t0 & tpb_mask) * ROW + lane * 16;
            const char* kb = reinterpret_cast<const char*>(table_entry(krow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            const char* vb = reinterpret_cast<const char*>(table_entry(vrow, t0 >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
            if (rows >= TG)
            {
#pragma unroll
                for (int j = 0; j < NCP; ++j)
                {
                    cp_async16_u32(kdst + cdst[j], kb + j * 512);
                    cp_async16_u32(kdst + SLAB + cdst[j], vb + j * 512);
                }
            }
            else
            {
                // last group of the sequence: rows at and behind the new token are zero-filled
                const int valid_bytes = rows > 0 ? rows * ROW : 0;
#pragma unroll
                for (int j = 0; j < NCP; ++j)
                {
                    const bool ok = (lane + 32 * j) * 16 < valid_bytes;
                    cp_async16_zfill_u32(kdst + cdst[j], ok ? kb + j * 512 : kb, ok ? 16u : 0u);
                    cp_async16_zfill_u32(kdst + SLAB + cdst[j], ok ? vb + j * 512 : vb, ok ? 16u : 0u);
                }
            }
            cp_async_mbar_arrive_noinc(&bars[(ring_base + i) % STAGES]);
        };

        // ---- Q as A fragments: rows = heads g and g + 8, k-step j covers channels 16 j .. 16 j + 15.  Requested
        // before the first ring stages: behind those tens of KB per warp the same loads would wait for all of them ----
        const int qkv_stride = (a.num_heads + 2 * a.num_kv_heads) * DH;
        const T* qkv_b = reinterpret_cast<const T*>(a.qkv) + (size_t) b * qkv_stride;
        uint32_t qa[KSTEPS][4];
        {
            const uint32_t* q0 = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(a.qkv) + q_row_of(min(g, nh - 1)));
            const uint32_t* q1 = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(a.qkv) + q_row_of(min(g + 8, nh - 1)));
            const bool v0 = g < nh, v1 = g + 8 < nh;
#pragma unroll
            for (int j = 0; j < KSTEPS; ++j)
            {
                qa[j][0] = v0 ? q0[8 * j + t] : 0u;     // (row g, channels 16 j + 2 t, + 1)
                qa[j][1] = v1 ? q1[8 * j + t] : 0u;     // (row g + 8, same channels)
                qa[j][2] = v0 ? q0[8 * j + 4 + t] : 0u; // (row g, channels 16 j + 8 + 2 t, + 1)
                qa[j][3] = v1 ? q1[8 * j + 4 + t] : 0u;
            }
        }
        const int my_groups = (n_groups > warp) ? (n_groups - warp + NWARPS - 1) / NWARPS : 0;
        for (int i = 0; i < min(STAGES, my_groups); ++i)
            issue(i);

        const float sscale = a.softmax_scale_log2;

        // Per-lane ldmatrix row addresses inside a slab.
        //   K, 8-token tile nt, k-steps 2 jj and 2 jj + 1: matrix q = lane >> 3 is chunk 4 jj + q of rows 8 nt + (lane & 7)
        //   V, channel tiles 2 a and 2 a + 1: matrices (tokens 0-7 | 8-15) x (chunk 2 a | 2 a + 1), transposed on load
        const uint32_t k_row = lane & 7, k_q = lane >> 3;
        const uint32_t v_row = (lane & 7) + 8 * ((lane >> 3) & 1), v_q = lane >> 4;

        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float of[NT][4]; // O fragments: [channel tile][c0, c1: head g | c2, c3: head g + 8]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                of[nt][c] = 0.f;

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
                // The group ends with the new token: put its k / v rows into the staged tile (rows behind it were
                // zero-filled by the copies) and, from the first head slice only, append them to the paged cache.
                const int r_new = new_pos - t0;
                if (lane < CPR)
                {
                    const T* kp = qkv_b + (size_t) (a.num_heads + hk) * DH + lane * 8;
                    const T* vp = qkv_b + (size_t) (a.num_heads + a.num_kv_heads + hk) * DH + lane * 8;
                    const uint4 kq = *reinterpret_cast<const uint4*>(kp);
                    const uint4 vq = *reinterpret_cast<const uint4*>(vp);
                    unsigned char* stage = smem + warp * (STAGES * Tr::STAGE_BYTES) + s * Tr::STAGE_BYTES;
                    const uint32_t lin = sw16<DH>((uint32_t) r_new, (uint32_t) lane);
                    *reinterpret_cast<uint4*>(stage + lin) = kq;
                    *reinterpret_cast<uint4*>(stage + SLAB + lin) = vq;
                    if (FEAT == 0 && hg == 0) // (feature form: kv_append_token_kernel stores the token behind this kernel)
                    {
                        const size_t off = head_off + (size_t) (new_pos & tpb_mask) * ROW + lane * 16;
                        char* kb = reinterpret_cast<char*>(table_entry(krow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                        char* vb = reinterpret_cast<char*>(table_entry(vrow, new_pos >> tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
                        *reinterpret_cast<uint4*>(kb) = kq;
                        *reinterpret_cast<uint4*>(vb) = vq;
                    }
                }
                __syncwarp();
            }

            // ---- S = Q K^T: 16 head rows x 16 tokens (two 8-token tiles) ----
            float sacc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    sacc[nt][c] = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
            {
#pragma unroll
                for (int jj = 0; jj < KSTEPS / 2; ++jj)
                {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, kbuf + sw16<DH>(8 * nt + k_row, 4 * jj + k_q));
                    mma_16bit<T>(sacc[nt], qa[2 * jj], kf[0], kf[1]);
                    mma_16bit<T>(sacc[nt], qa[2 * jj + 1], kf[2], kf[3]);
                }
            }

            // ---- online softmax over the 16 tokens: thread holds tokens 8 nt + 2 t, + 1 of head rows g and g + 8 ----
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                {
                    p[nt][c] = sacc[nt][c] * sscale;
                    const int tok = t0 + 8 * nt + 2 * t + (c & 1);
                    if constexpr (FEAT == 1)
                        p[nt][c] = fmaf(slope[c >> 1], tok == new_pos ? 0.f : (float) (tok - past_true), p[nt][c]);
                    if constexpr (FEAT == 2)
                    {
                        const int j = tok - first_new;
                        if (j >= 0 && j < 64 && (((j < 32 ? mw[c >> 1][0] : mw[c >> 1][1]) >> (j & 31)) & 1u) == 0u)
                            p[nt][c] = -INFINITY;
                    }
                }
            if (lim < TG)
            {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (8 * nt + 2 * t + (c & 1) >= lim)
                            p[nt][c] = -INFINITY;
            }
            float alpha[2], msub[2];
            bool changed = false;
#pragma unroll
            for (int r = 0; r < 2; ++r)
            {
                float mx = fmaxf(fmaxf(p[0][2 * r], p[0][2 * r + 1]), fmaxf(p[1][2 * r], p[1][2 * r + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[r], mx);
                // (FEAT = 2: under its mask a row may have seen nothing yet; -inf minus -inf must not reach exp2)
                msub[r] = (FEAT == 2 && m_new == -INFINITY) ? 0.f : m_new;
                alpha[r] = fast_exp2(m[r] - msub[r]);
                changed |= m_new != m[r];
                m[r] = m_new;
                l[r] *= alpha[r];
            }
            // P as the A fragment of the 16-token k-step: a0 / a1 from tile 0 (rows g / g + 8), a2 / a3 from tile 1
            uint32_t pa[4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int r = 0; r < 2; ++r)
                {
                    const float p0 = fast_exp2(p[nt][2 * r] - msub[r]), p1 = fast_exp2(p[nt][2 * r + 1] - msub[r]);
                    l[r] += p0 + p1;
                    pa[2 * nt + r] = TypeOps<T>::pack2(p0, p1);
                }
            // ---- rescale the running O when a row maximum moved ----
            if (__any_sync(0xffffffffu, changed))
            {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                {
                    of[nt][0] *= alpha[0];
                    of[nt][1] *= alpha[0];
                    of[nt][2] *= alpha[1];
                    of[nt][3] *= alpha[1];
                }
            }
            // ---- O += P V ----
#pragma unroll
            for (int av = 0; av < NT / 2; ++av)
            {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vbuf + sw16<DH>(v_row, 2 * av + v_q));
                mma_16bit<T>(of[2 * av], pa, vf[0], vf[1]);
                mma_16bit<T>(of[2 * av + 1], pa, vf[2], vf[3]);
            }

            __syncwarp(); // every lane is done reading this stage
            if (i + STAGES < my_groups)
                issue(i + STAGES);
        }

        if (timed_out)
        {
            if (lane == 0)
                report_status(a.status, STATUS_TIMEOUT);
            asm volatile("cp.async.wait_all;" ::: "memory"); // the ring is reused below and the CTA then exits
        }

        // ---- per-warp results -> shared memory, then combine the 4 warps ----
#pragma unroll
        for (int r = 0; r < 2; ++r)
        {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads(); // all warps have drained their rings; the ring memory is reused below
        float* mo = reinterpret_cast<float*>(smem) + warp * (16 * DH + 32);
        float* mm = mo + 16 * DH; // m[16], then l[16]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                mo[(g + 8 * (c >> 1)) * DH + 8 * nt + 2 * t + (c & 1)] = of[nt][c];
        if (t == 0)
        {
            mm[g] = m[0];
            mm[8 + g] = m[1];
            mm[16 + g] = l[0];
            mm[16 + 8 + g] = l[1];
        }
        __syncthreads();

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
                reinterpret_cast<T*>(a.out)[row * DH + dh] = TypeOps<T>::from_float(o / L);
            }
            else
            {
                a.part_o[(row * a.nsplit + chunk) * DH + dh] = o;
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
