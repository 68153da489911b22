// Context-phase KV append: writes the K and V of a whole prompt into the paged (optionally quantised)
// cache, with the same quantise-on-write chain as the decode step.
//
// Source layout [B, Hkv, seq_len, Dh] (batch-major, what the context attention leaves behind);
// destination: block table rows, block = [Hkv, tokens_per_block, Dh] cache elements.  One thread
// moves 16 bytes of cache (16 elements of an 8-bit cache, 8 of a 16-bit one) for K and for V:
// loads and stores are 16-byte, consecutive threads touch consecutive addresses on both sides.
// HBM-bound: 2 * (2 + e_c) bytes per element.
//
// Replaces transpose4dBatchMajorKVCache / invokeTranspose4dBatchMajor
//   cpp/tensorrt_llm/kernels/unfusedAttentionKernels.cu:1565-1666
// (same argument meaning; tokens beyond sequence_lengths[b] are skipped; with a window shorter than the prompt
// the cache is cyclic and only the last `window` tokens are kept, :1591-1600).
#pragma once

#include "dx_common.cuh"
#include "dx_mha_kernel.cuh" // make_cache_vec

namespace dx
{

struct AppendArgs
{
    const void* k_src;            // T [B, Hkv, seq_len, Dh]
    const void* v_src;
    const int32_t* seq_len;       // int32 [B]: tokens to store per sequence
    const int64_t* block_ptrs;    // int64 [B, 2, M]
    const float* scale_orig_quant; // device float[1] or nullptr
    int32_t batch;
    int32_t num_kv_heads;
    int32_t src_seq_len;          // row stride of the source, tokens
    int32_t max_blocks_per_seq;
    int32_t tpb_log2;
    // cyclic cache (KVBlockArray::getKVTokenIdx, kvCacheUtils.h:109-117): token t >= sink lives in slot
    // sink + bubble + (t - sink) % cyclic_len; only the last `window` tokens of a sequence are stored
    int32_t window;
    int32_t sink;
    int32_t bubble;
    int32_t cyclic_len;
    int32_t* status; // device status word (0 ok)
    TableGuard guard;
};

template <typename T, int CACHE, int DH>
__global__ void __launch_bounds__(256) kv_append_context_kernel(const AppendArgs a)
{
    constexpr int ECB = (CACHE == CACHE_T) ? 2 : 1;
    constexpr int EPL = 16 / ECB;    // elements per thread
    constexpr int LPR = DH / EPL;    // threads per token row
    const int b = blockIdx.y, h = blockIdx.z;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int tok = idx / LPR, part = idx % LPR;
    const int len = a.seq_len[b];
    // tokens that left the window are dropped, as in the reference (the sink tokens too when the prompt is longer
    // than the window: unfusedAttentionKernels.cu:1591-1600 tests the lower bound for every token)
    if (tok >= min(len, a.src_seq_len) || tok < len - a.window)
        return;
    // With sink tokens and no spare block the window holds more tokens than slots cycle: of the tokens that share a
    // slot the latest stays (in the reference whichever thread stores last wins; this is the outcome that keeps
    // the newest tokens, and it is deterministic).
    if (tok >= a.sink && tok + a.cyclic_len < len)
        return;
    const int slot = tok < a.sink ? tok : a.sink + a.bubble + (tok - a.sink) % a.cyclic_len;
    float sc_f = 1.f;
    T sc_t = TypeOps<T>::from_float(1.f);
    if constexpr (CACHE != CACHE_T)
    {
        sc_f = __ldg(a.scale_orig_quant);
        sc_t = TypeOps<T>::from_float(sc_f);
    }
    const size_t src = (((size_t) b * a.num_kv_heads + h) * a.src_seq_len + tok) * DH + part * EPL;
    const uint4 kq = make_cache_vec<T, CACHE, EPL>(reinterpret_cast<const T*>(a.k_src) + src, sc_f, sc_t);
    const uint4 vq = make_cache_vec<T, CACHE, EPL>(reinterpret_cast<const T*>(a.v_src) + src, sc_f, sc_t);
    const int64_t* krow = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
    const int64_t* vrow = krow + a.max_blocks_per_seq;
    const int tpb_mask = (1 << a.tpb_log2) - 1;
    const size_t off = ((size_t) h * ((size_t) 1 << a.tpb_log2) + (slot & tpb_mask)) * (DH * ECB) + part * 16;
    char* kb = reinterpret_cast<char*>(table_entry(krow, slot >> a.tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
    char* vb = reinterpret_cast<char*>(table_entry(vrow, slot >> a.tpb_log2, a.max_blocks_per_seq, a.status, a.guard)) + off;
    *reinterpret_cast<uint4*>(kb) = kq;
    *reinterpret_cast<uint4*>(vb) = vq;
}

} // namespace dx
