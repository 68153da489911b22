// Shared device helpers for the decode-attention kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dx
{

// Cache element kinds.
enum CacheKind : int
{
    CACHE_T = 0,    // same 16-bit type as the activations, no quantisation
    CACHE_INT8 = 1, // int8, per-tensor scale
    CACHE_FP8 = 2   // e4m3, per-tensor scale
};

// What the bounds-checked build (-DDECODE_ATTN_BOUNDS_CHECK) needs to validate a block pointer and to redirect a bad
// access; all zero in the regular build, where table_entry() is a plain load.
struct TableGuard
{
    int64_t safe_block; // device block of the handle (one cache block, zeros): target of redirected accesses
    int64_t pool_lo;    // registered range of valid block start addresses [pool_lo, pool_hi); 0, 0: not registered
    int64_t pool_hi;
};

// Arguments shared by every attention kernel.  Passed by value (fits the 4 KB parameter space).
struct AttnArgs
{
    const void* qkv;              // T [B, (H + 2 Hkv) Dh]
    void* out;                    // T [B, H Dh]
    const int32_t* seq_len;       // int32 [B], includes the new token
    const int64_t* block_ptrs;    // int64 [B, 2, M]
    const float* scale_orig_quant; // device float[1] or nullptr
    const float* scale_quant_orig; // device float[1] or nullptr
    float* part_o;                // fp32 [B*H, nsplit, Dh]  (split-K partial numerators)
    float2* part_ml;              // (m, l) [B*H, nsplit]     (running max in log2 units, denominator)
    int32_t* status;              // device status word (0 ok)
    int32_t batch;
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t max_blocks_per_seq;
    int32_t tpb_log2;
    int32_t chunk_tokens; // upper bound of tokens per split-K partition (multiple of 128), see partition_of()
    int32_t nsplit;       // grid.x; 1 => kernels write the final output themselves.  Stream-K: result slots per row
    float softmax_scale_log2; // log2(e) / (sqrt(Dh) * q_scaling)
    int32_t streamk;          // 1: the CTAs walk equal ranges of the batch's token groups (SkSchedule), see below
    int32_t* tickets;         // device counter of the dynamic ranges of a two-level schedule (the merge kernel clears it)
    TableGuard guard;
    // Feature form of the grouped-head 8-bit kernel (beam search, ALiBi); null / 0 on the plain path
    const int32_t* cache_indir;     // int32 [B, max_attention_window]: beam a slot of sequence b comes from
    const int32_t* context_lengths; // int32 [B]: slots below it come from beam 0 of the request
    const void* alibi_slopes;       // T [H]
    int32_t beam_width;
    int32_t max_attention_window;
    // Several new tokens per sequence on the grouped-head kernel (q_len > 1): the rows of a kv head are (token, head)
    // pairs, token-major; every new token is in the cache already; packed_mask as in GeneralArgs
    int32_t q_len;
    const int32_t* packed_mask;
    int32_t cyclic_window; // > 0: the cache is cyclic; the kernels walk slots 0 .. min(past, cyclic_window) - 1 and the
                           // new token is appended behind them by kv_append_token_kernel (0 on the plain path)
};

// Arguments of the feature-complete path (beam search, cyclic window, sink tokens, ALiBi).
struct GeneralArgs
{
    const void* qkv;   // T [B, (H + 2 Hkv) Dh]
    void* out;         // T [B, H Dh]
    const int32_t* seq_len;      // [B] including the new token
    const int64_t* block_ptrs;   // [B, 2, M]
    const float* scale_orig_quant;
    const float* scale_quant_orig;
    const int32_t* cache_indir;     // [B, max_attention_window] or null (B counts beams)
    const int32_t* context_lengths; // [B] or null
    const void* alibi_slopes;       // T [H] or null
    int32_t num_heads;
    int32_t num_kv_heads;
    int32_t max_blocks_per_seq;
    int32_t tpb_log2;
    int32_t beam_width;
    int32_t max_attention_window;
    int32_t cyclic_window; // slots the kernel may walk
    int32_t cyclic_len;    // period of the non-sink part of the cache
    int32_t sink;
    float softmax_scale_log2;
    // several new tokens per sequence (the reference's Medusa mode): qkv / out row r is token r % q_len of sequence
    // r / q_len; seq_len includes all q_len new tokens
    int32_t q_len;               // 1: the usual single token
    const int32_t* packed_mask;  // [B, q_len, (q_len + 31) / 32]: bit j of row t = token t attends new token j
    // relative attention bias: T [H, stride, stride] (max_distance 0) or the bucket table T [H, stride]
    const void* rel_bias;
    int32_t rel_stride;
    int32_t max_distance;
    int32_t* status; // device status word (0 ok)
    TableGuard guard;
};

// Tokens a step attends to (cache slots walked + the new token) for a sequence of `total` tokens including the new
// one: all of them, or with a cyclic cache min(past, window) + 1 (decoderMaskedMultiheadAttentionTemplate.h:1493).
__host__ __device__ __forceinline__ int attended_tokens(int total, int cyclic_window)
{
    const int past = total - 1;
    return cyclic_window > 0 && past > cyclic_window ? cyclic_window + 1 : total;
}

__host__ __device__ __forceinline__ int cyclic_slot(int tok, int sink, int cyclic_len)
{
    return tok < sink ? tok : sink + (tok - sink) % cyclic_len;
}

// Values of the device status word (0 = ok).  The first report of a step stays (atomicCAS from 0): later ones do
// not overwrite it.
static constexpr int32_t STATUS_TIMEOUT = 5;       // a bounded wait ran out
static constexpr int32_t STATUS_NO_BLOCKS = 6;     // dx_kv_cache_step: free list or table row exhausted
static constexpr int32_t STATUS_PLAN_EXCEEDED = 7; // a device length needs more partitions than the launch has
static constexpr int32_t STATUS_BAD_TABLE = 8;     // bounds-checked build: block index or block pointer out of bounds

__device__ __forceinline__ void report_status(int32_t* status, int32_t what)
{
    atomicCAS(status, 0, what);
}

// Entry idx of a block-table row (K or V row of one sequence, max_blocks entries): the address of a cache block.
// Regular build: a load.  Bounds-checked build: an index outside the row, a null or misaligned pointer, or one
// outside the registered pool is recorded in the status word (STATUS_BAD_TABLE, first violation wins) and the
// access goes to the handle's spare block instead, so that nothing outside the caller's memory is touched.
__device__ __forceinline__ int64_t table_entry(
    const int64_t* row, int idx, int max_blocks, int32_t* status, const TableGuard& g)
{
#ifdef DECODE_ATTN_BOUNDS_CHECK
    if ((unsigned) idx >= (unsigned) max_blocks)
    {
        report_status(status, STATUS_BAD_TABLE);
        return g.safe_block;
    }
    const int64_t p = __ldg(row + idx);
    if (p == 0 || (p & 15) != 0 || (g.pool_hi != 0 && (p < g.pool_lo || p >= g.pool_hi)))
    {
        report_status(status, STATUS_BAD_TABLE);
        return g.safe_block;
    }
    return p;
#else
    (void) max_blocks, (void) status, (void) g;
    return __ldg(row + idx);
#endif
}

// ----------------------------------------------------------------------------------------------
// Stream-K schedule of the grouped-head kernels.  The rows of the batch - (sequence b, kv-head slice y), y fastest -
// are laid end to end in units of token groups (32 tokens for the 8-bit kernels, 16 for the 16-bit one); row (b, y)
// has n_b = prefix[b+1] - prefix[b] groups and starts at unit rows_per_seq * prefix[b] + y * n_b.  CTA c owns units
// [c * units_per_cta, (c+1) * units_per_cta): a few pieces of consecutive rows, every CTA the same amount of
// streaming, whatever the mix of lengths.  A row cut into several pieces leaves one partial result per piece in
// slot (c - first CTA of the row); a row inside one CTA is written out directly.  The lengths are the HOST lengths
// the call was planned with; the kernels clamp every piece to the device length.
// ----------------------------------------------------------------------------------------------
static constexpr int DX_SK_MAX_SEQ = 1024;

struct SkSchedule
{
    uint32_t units_per_cta;
    uint32_t total_units;
    uint32_t rows_per_seq;
    uint32_t nseq;
    // Two-level form (the persistent tcgen05 kernel): ranges 0 .. n1-1 are the static ones above, one per CTA,
    // units [r * units_per_cta, (r+1) * units_per_cta); what they leave, units [n1 * units_per_cta, total_units), is
    // cut into n2 short ranges of u2 units, numbered n1, n1+1, ..., that the CTAs take from a device counter as
    // they finish.  Single-level schedules have n1 = number of CTAs, n2 = u2 = 0.
    uint32_t n1, n2, u2;
    uint32_t prefix[DX_SK_MAX_SEQ + 1];
};

// Range that holds unit u.
__host__ __device__ __forceinline__ uint32_t sk_range_of_unit(const SkSchedule& sk, uint32_t u)
{
    const uint32_t static_units = sk.n1 * sk.units_per_cta;
    return u < static_units ? u / sk.units_per_cta : sk.n1 + (u - static_units) / sk.u2;
}

// Units [u0, u1) of range r.
__host__ __device__ __forceinline__ void sk_range_units(const SkSchedule& sk, uint32_t r, uint32_t& u0, uint32_t& u1)
{
    if (r < sk.n1)
    {
        u0 = r * sk.units_per_cta;
        u1 = u0 + sk.units_per_cta;
    }
    else
    {
        u0 = sk.n1 * sk.units_per_cta + (r - sk.n1) * sk.u2;
        u1 = u0 + sk.u2;
    }
    u0 = u0 < sk.total_units ? u0 : sk.total_units;
    u1 = u1 < sk.total_units ? u1 : sk.total_units;
}

struct SkCursor
{
    uint32_t u, u1;  // next unit, end of this CTA's range
    uint32_t b, y;   // row the cursor is in
    uint32_t g0, nb; // group inside the row, groups of the row
};

__device__ __forceinline__ bool sk_begin(const SkSchedule& sk, int cta, SkCursor& c)
{
    c.u = (uint32_t) cta * sk.units_per_cta;
    if (c.u >= sk.total_units)
        return false;
    c.u1 = min(c.u + sk.units_per_cta, sk.total_units);
    uint32_t lo = 0, hi = sk.nseq - 1;
    while (lo < hi) // largest b whose first unit is <= u
    {
        const uint32_t mid = (lo + hi + 1) >> 1;
        if (sk.rows_per_seq * sk.prefix[mid] <= c.u)
            lo = mid;
        else
            hi = mid - 1;
    }
    c.b = lo;
    c.nb = sk.prefix[lo + 1] - sk.prefix[lo];
    const uint32_t rem = c.u - sk.rows_per_seq * sk.prefix[lo];
    c.y = rem / c.nb;
    c.g0 = rem - c.y * c.nb;
    return true;
}

// The piece under the cursor: row (b, y), groups [g0, g0 + ng), result slot, and whether it is the whole row.
__device__ __forceinline__ void sk_piece(
    const SkSchedule& sk, const SkCursor& c, int& b, int& y, int& g0, int& ng, int& slot, bool& whole)
{
    b = (int) c.b, y = (int) c.y, g0 = (int) c.g0;
    ng = (int) min(c.nb - c.g0, c.u1 - c.u);
    const uint32_t row_start = sk.rows_per_seq * sk.prefix[c.b] + c.y * c.nb;
    slot = (int) (blockIdx.x - row_start / sk.units_per_cta);
    whole = c.g0 == 0 && (uint32_t) ng == c.nb;
}

// Moves the cursor behind the current piece; false when the CTA's range is used up.
__device__ __forceinline__ bool sk_next(const SkSchedule& sk, SkCursor& c)
{
    const uint32_t ng = min(c.nb - c.g0, c.u1 - c.u);
    c.u += ng;
    c.g0 += ng;
    if (c.g0 == c.nb)
    {
        c.g0 = 0;
        if (++c.y == sk.rows_per_seq)
        {
            c.y = 0;
            ++c.b;
            if (c.u < c.u1)
                c.nb = sk.prefix[c.b + 1] - sk.prefix[c.b];
        }
    }
    return c.u < c.u1;
}

// Pieces row (b, y) was cut into (1: the kernel wrote the final output itself).
__device__ __forceinline__ int sk_pieces_of_row(const SkSchedule& sk, int b, int y)
{
    const uint32_t nb = sk.prefix[b + 1] - sk.prefix[b];
    const uint32_t row_start = sk.rows_per_seq * sk.prefix[b] + (uint32_t) y * nb;
    return (int) (sk_range_of_unit(sk, row_start + nb - 1) - sk_range_of_unit(sk, row_start)) + 1;
}

// Cursor on unit u0 of the line, range end u1 (u0 < u1 <= total_units).
__device__ __forceinline__ void sk_seek(const SkSchedule& sk, uint32_t u0, uint32_t u1, SkCursor& c)
{
    c.u = u0;
    c.u1 = u1;
    uint32_t lo = 0, hi = sk.nseq - 1;
    while (lo < hi) // largest b whose first unit is <= u
    {
        const uint32_t mid = (lo + hi + 1) >> 1;
        if (sk.rows_per_seq * sk.prefix[mid] <= u0)
            lo = mid;
        else
            hi = mid - 1;
    }
    c.b = lo;
    c.nb = sk.prefix[lo + 1] - sk.prefix[lo];
    const uint32_t rem = u0 - sk.rows_per_seq * sk.prefix[lo];
    c.y = rem / c.nb;
    c.g0 = rem - c.y * c.nb;
}

// Split-K partitioning of one sequence: `total` tokens are cut into the fewest partitions of at
// most `target` tokens, and those partitions are made equal (rounded up to 128 tokens) so that no
// CTA is left with a sliver.  Attention kernels and the merge kernel derive the same numbers.
__host__ __device__ __forceinline__ void partition_of(
    int total, int target, int part, int& start, int& len, int& nparts)
{
    nparts = (total + target - 1) / target;
    const int size = (((total + nparts - 1) / nparts) + 127) & ~127;
    start = part * size;
    len = part < nparts ? (total - start < size ? total - start : size) : 0;
}

// ----------------------------------------------------------------------------------------------
// PTX wrappers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: every spin in this library has an iteration limit.  Returns false when it gave up,
// either because the limit ran out or (CHECK_STATUS) because the status word already holds a report
// (so that one stuck copy cannot add up to many serial time-outs).
template <bool CHECK_STATUS = true>
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, const int32_t* status, int limit)
{
#pragma unroll 1
    for (int it = 0; it < limit; ++it)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if (CHECK_STATUS && (it & 255) == 255 && *reinterpret_cast<const volatile int32_t*>(status) != 0)
            return false;
    }
    return false;
}

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, const int32_t* status)
{
    return mbar_wait_limit<true>(bar, parity, status, 1 << 20);
}

// After a wait gave up: waits once more, with a limit of its own and without looking at the status word, for a
// copy that was already requested, so that nothing is in flight into this CTA's shared memory when it exits.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity)
{
    (void) mbar_wait_limit<false>(bar, parity, nullptr, 1 << 22);
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// 1-D bulk async copy global -> this CTA's shared memory, completion counted in bytes on an
// mbarrier.  dst, src 16-byte aligned, bytes a multiple of 16.  Never multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// 16-byte Ampere-style async copy (used where the destination layout is swizzled per 16 B).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}

// Makes the executing thread's prior cp.async operations arrive on the mbarrier when they land.
// 16-byte asynchronous copy global -> shared (shared address as a 32-bit window offset); the zfill form
// copies src_bytes (0 or 16) and zero-fills the rest.
__device__ __forceinline__ void cp_async16_u32(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async16_zfill_u32(uint32_t dst, const void* src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void griddep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void griddep_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ----------------------------------------------------------------------------------------------
// 16-bit activation type helpers
// ----------------------------------------------------------------------------------------------
template <typename T>
struct TypeOps;

template <>
struct TypeOps<__half>
{
    using T2 = __half2;
    static __device__ __forceinline__ float to_float(__half x)
    {
        return __half2float(x);
    }
    static __device__ __forceinline__ __half from_float(float x)
    {
        return __float2half_rn(x);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t w)
    {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b)
    {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    // scale_T * x_T with one rounding to T, then RN-even saturating-finite e4m3: the byte the
    // reference stores (decoderMaskedMultiheadAttentionUtils.h:3753-3763 with T_scale = half).
    static __device__ __forceinline__ uint8_t quant_fp8(__half x, __half scale)
    {
        __half p = __hmul(scale, x);
        return (uint8_t) __nv_cvt_halfraw_to_fp8(static_cast<__half_raw>(p), __NV_SATFINITE, __NV_E4M3);
    }
};

template <>
struct TypeOps<__nv_bfloat16>
{
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x)
    {
        return __bfloat162float(x);
    }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x)
    {
        return __float2bfloat16_rn(x);
    }
    static __device__ __forceinline__ float2 unpack2(uint32_t w)
    {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b)
    {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint8_t quant_fp8(__nv_bfloat16 x, __nv_bfloat16 scale)
    {
        __nv_bfloat16 p = __hmul(scale, x);
        return (uint8_t) __nv_cvt_bfloat16raw_to_fp8(static_cast<__nv_bfloat16_raw>(p), __NV_SATFINITE, __NV_E4M3);
    }
};

// round-to-nearest-even, saturating float -> int8: the instruction the reference issues
// (decoderMaskedMultiheadAttentionUtils.h:3629-3639).
__device__ __forceinline__ int8_t quant_int8(float x)
{
    short r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=h"(r) : "f"(x));
    return (int8_t) r;
}

// Quantise 4 consecutive activations (two packed 32-bit words of T) into 4 cache bytes.
template <typename T, int CACHE>
__device__ __forceinline__ uint32_t quant4(uint32_t w0, uint32_t w1, float scale_f32, T scale_t)
{
    const T* a = reinterpret_cast<const T*>(&w0);
    const T* b = reinterpret_cast<const T*>(&w1);
    uint32_t r;
    if constexpr (CACHE == CACHE_INT8)
    {
        uint32_t b0 = (uint8_t) quant_int8(TypeOps<T>::to_float(a[0]) * scale_f32);
        uint32_t b1 = (uint8_t) quant_int8(TypeOps<T>::to_float(a[1]) * scale_f32);
        uint32_t b2 = (uint8_t) quant_int8(TypeOps<T>::to_float(b[0]) * scale_f32);
        uint32_t b3 = (uint8_t) quant_int8(TypeOps<T>::to_float(b[1]) * scale_f32);
        r = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
    else
    {
        uint32_t b0 = TypeOps<T>::quant_fp8(a[0], scale_t);
        uint32_t b1 = TypeOps<T>::quant_fp8(a[1], scale_t);
        uint32_t b2 = TypeOps<T>::quant_fp8(b[0], scale_t);
        uint32_t b3 = TypeOps<T>::quant_fp8(b[1], scale_t);
        r = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
    return r;
}

// ----------------------------------------------------------------------------------------------
// Dequantise-in-register: 4 packed cache bytes -> 4 floats (without the per-tensor scale, which
// the callers fold into q and into the final normalisation).
// ----------------------------------------------------------------------------------------------
template <int CACHE>
__device__ __forceinline__ void dequant4(uint32_t w, float (&f)[4])
{
    if constexpr (CACHE == CACHE_INT8)
    {
        // byte -> 2^23 + (byte ^ 0x80) by byte permute, then subtract 2^23 + 128: exact.
        const uint32_t u = w ^ 0x80808080u;
        f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.f;
        f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.f;
        f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.f;
        f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.f;
    }
    else
    {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t) (w & 0xffffu), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t) (w >> 16), __NV_E4M3);
        float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
        float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
        f[0] = a.x;
        f[1] = a.y;
        f[2] = b.x;
        f[3] = b.y;
    }
}

} // namespace dx
