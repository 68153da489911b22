/*
 * TEST INFRASTRUCTURE ONLY - never linked into, imported by or called from the product library.
 *
 * Thin driver around the reference's own masked-multihead-attention (MMHA) CUDA source, compiled
 * for sm_100a straight from the reference tree (nothing is copied: the reference headers are
 * #included from where they lie, see oracle/Makefile).  It instantiates only the paged-KV,
 * self-attention launcher for one (T, Dh) pair per translation unit (REF_T / REF_DH) and exposes
 * a C entry point that fills Masked_multihead_attention_params the way
 * cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:243-349
 * (fusedQKV_masked_attention_dispatch) and :1159-1364 (enqueueGeneration) do.
 *
 * Used by the GPU parity tests to pin the oracle (KV bytes written, paging, attention output)
 * against the reference kernel itself, and by bench.py as the "reference kernel recompiled for
 * B200" timing line.
 */
#include "tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionLaunch.h"

#include <cstdint>
#include <cstring>

#ifndef REF_DH
#error "REF_DH must be defined"
#endif

#if REF_T_IS_BF16
using RefT = __nv_bfloat16;
#define REF_FN(name) name##_bf16
#else
using RefT = uint16_t; // the reference spells fp16 as uint16_t in MMHA
#define REF_FN(name) name##_fp16
#endif

#define REF_CAT2(a, b) a##_##b
#define REF_CAT(a, b) REF_CAT2(a, b)

namespace tensorrt_llm
{
namespace kernels
{
namespace mmha
{
template void mmha_launch_kernel<RefT, KVBlockArray, Masked_multihead_attention_params<RefT>, REF_DH, false>(
    const Masked_multihead_attention_params<RefT>& params, const KVBlockArray& kv_cache_buffer,
    const KVLinearBuffer& shift_k_cache, const cudaStream_t& stream);
// the variant that computes the relative-position bucket on the fly (chosen like decoderMaskedMultiheadAttention.cu:62;
// the reference instantiates it for head sizes 32, 64 and 128 only)
#if REF_DH == 32 || REF_DH == 64 || REF_DH == 128
#define REF_HAS_IMPLICIT_REL_BIAS 1
template void mmha_launch_kernel<RefT, KVBlockArray, Masked_multihead_attention_params<RefT>, REF_DH, true>(
    const Masked_multihead_attention_params<RefT>& params, const KVBlockArray& kv_cache_buffer,
    const KVLinearBuffer& shift_k_cache, const cudaStream_t& stream);
#else
#define REF_HAS_IMPLICIT_REL_BIAS 0
#endif
} // namespace mmha
} // namespace kernels
} // namespace tensorrt_llm

using namespace tensorrt_llm::kernels;

/* Returns 0 on success, a cudaError_t value otherwise.
 * workspace layout (caller allocates, 128-byte aligned sub-buffers, same order as the plugin):
 *   partial_out [tiles,B,H,Dh] T | partial_sum [B*H*tiles] f32 | partial_max [B*H*tiles] f32 | block_counter [B*H] i32
 * tiles == 0 disables multi-block mode. */
struct RefExtras
{
    int32_t beam_width = 1;
    const int32_t* cache_indir = nullptr;   // [batch, max_attention_window]
    const int32_t* input_lengths = nullptr; // [batch]
    int32_t cyclic_attention_window_size = 0; // 0: same as max_attention_window
    int32_t sink_token_length = 0;
    const void* linear_bias_slopes = nullptr; // T [num_heads]
    const void* relative_attention_bias = nullptr; // T [num_heads, stride, stride], or [num_heads, stride] (implicit)
    int32_t relative_attention_bias_stride = 0;
    int32_t max_distance = 0;                      // > 0: implicit form, stride = number of buckets
};

static int ref_mmha_impl(const void* qkv, void* out, const int32_t* sequence_length_dev,
    int64_t* block_pointers_dev, int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t max_blocks_per_seq,
    int32_t tokens_per_block, int32_t max_attention_window, int32_t past_kv_length, float q_scaling,
    const float* kv_scale_orig_quant_dev, const float* kv_scale_quant_orig_dev, int32_t int8_kv, int32_t fp8_kv,
    int32_t tiles, void* workspace, int32_t sm_count, cudaStream_t stream, const void* qkv_bias,
    int32_t position_embedding_type, int32_t rotary_embedding_dim, float rotary_embedding_base,
    int32_t rotary_embedding_scale_type, float rotary_embedding_scale, int32_t rotary_embedding_max_positions,
    const RefExtras& x)
{
    const int Dh = REF_DH;
    const size_t elem = (int8_kv || fp8_kv) ? 1 : sizeof(RefT);
    const int32_t cyclic = x.cyclic_attention_window_size > 0 ? x.cyclic_attention_window_size : max_attention_window;
    KVBlockArray kv(batch, max_blocks_per_seq, tokens_per_block, (int32_t) (num_kv_heads * Dh * elem), cyclic,
        x.sink_token_length, false);
    kv.data = block_pointers_dev;
    KVLinearBuffer shift_k;

    Masked_multihead_attention_params<RefT> p;
    memset(&p, 0, sizeof(p));
    const int hq = num_heads * Dh, hkv = num_kv_heads * Dh;
    p.out = reinterpret_cast<RefT*>(out);
    p.q = reinterpret_cast<const RefT*>(qkv);
    p.k = p.q + hq;
    p.v = p.q + hq + hkv;
    p.int8_kv_cache = int8_kv != 0;
    p.fp8_kv_cache = fp8_kv != 0;
    if (int8_kv || fp8_kv)
    {
        p.kv_scale_orig_quant = kv_scale_orig_quant_dev;
        p.kv_scale_quant_orig = kv_scale_quant_orig_dev;
    }
    p.stride = hq + 2 * hkv;
    p.batch_size = batch;
    p.beam_width = x.beam_width;
    p.cache_indir = x.beam_width > 1 ? x.cache_indir : nullptr;
    p.input_lengths = x.input_lengths;
    p.linear_bias_slopes = reinterpret_cast<const RefT*>(x.linear_bias_slopes);
    p.relative_attention_bias = reinterpret_cast<const RefT*>(x.relative_attention_bias);
    p.relative_attention_bias_stride = x.relative_attention_bias_stride;
    p.max_distance = x.max_distance;
    p.max_attention_window_size = max_attention_window;
    p.cyclic_attention_window_size = cyclic;
    p.sink_token_length = x.sink_token_length;
    p.length_per_sample = sequence_length_dev;
    p.timestep = past_kv_length;
    p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads;
    p.hidden_size_per_head = Dh;
    p.position_embedding_type = static_cast<PositionEmbeddingType>(position_embedding_type);
    p.rotary_embedding_dim = rotary_embedding_dim;
    p.rotary_embedding_base = rotary_embedding_base;
    p.rotary_embedding_scale_type = static_cast<RotaryScalingType>(rotary_embedding_scale_type);
    p.rotary_embedding_scale = rotary_embedding_scale;
    p.rotary_embedding_max_positions = rotary_embedding_max_positions;
    if (qkv_bias)
    {
        p.q_bias = reinterpret_cast<const RefT*>(qkv_bias);
        p.k_bias = p.q_bias + hq;
        p.v_bias = p.q_bias + hq + hkv;
    }
    p.inv_sqrt_dh = 1.F / (sqrtf((float) Dh) * q_scaling);
    p.multi_processor_count = sm_count;
    p.multi_block_mode = tiles > 1;
    if (tiles > 1)
    {
        auto up = [](size_t x) { return (x + 127) / 128 * 128; };
        char* w = reinterpret_cast<char*>(workspace);
        size_t off = 0;
        p.partial_out = reinterpret_cast<RefT*>(w + off);
        off += up(sizeof(RefT) * (size_t) batch * num_heads * Dh * tiles);
        p.partial_sum = reinterpret_cast<float*>(w + off);
        off += up(sizeof(float) * (size_t) batch * num_heads * tiles);
        p.partial_max = reinterpret_cast<float*>(w + off);
        off += up(sizeof(float) * (size_t) batch * num_heads * tiles);
        p.block_counter = reinterpret_cast<int*>(w + off);
        p.min_seq_len_tile = 1;
        p.max_seq_len_tile = tiles;
        cudaError_t e = cudaMemsetAsync(p.block_counter, 0, sizeof(int) * (size_t) batch * num_heads, stream);
        if (e != cudaSuccess)
            return (int) e;
    }
    try
    {
        if (p.max_distance > 0 && p.relative_attention_bias != nullptr)
        {
#if REF_HAS_IMPLICIT_REL_BIAS
            mmha::mmha_launch_kernel<RefT, KVBlockArray, Masked_multihead_attention_params<RefT>, REF_DH, true>(
                p, kv, shift_k, stream);
#else
            return -2; // not instantiated by the reference for this head size
#endif
        }
        else
            mmha::mmha_launch_kernel<RefT, KVBlockArray, Masked_multihead_attention_params<RefT>, REF_DH, false>(
                p, kv, shift_k, stream);
    }
    catch (...)
    {
        return -1;
    }
    return (int) cudaGetLastError();
}

extern "C" int REF_CAT(REF_FN(ref_mmha), REF_DH)(const void* qkv, void* out, const int32_t* sequence_length_dev,
    int64_t* block_pointers_dev, int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t max_blocks_per_seq,
    int32_t tokens_per_block, int32_t max_attention_window, int32_t past_kv_length, float q_scaling,
    const float* kv_scale_orig_quant_dev, const float* kv_scale_quant_orig_dev, int32_t int8_kv, int32_t fp8_kv,
    int32_t tiles, void* workspace, int32_t sm_count, cudaStream_t stream, const void* qkv_bias,
    int32_t position_embedding_type, int32_t rotary_embedding_dim, float rotary_embedding_base,
    int32_t rotary_embedding_scale_type, float rotary_embedding_scale, int32_t rotary_embedding_max_positions)
{
    return ref_mmha_impl(qkv, out, sequence_length_dev, block_pointers_dev, batch, num_heads, num_kv_heads,
        max_blocks_per_seq, tokens_per_block, max_attention_window, past_kv_length, q_scaling, kv_scale_orig_quant_dev,
        kv_scale_quant_orig_dev, int8_kv, fp8_kv, tiles, workspace, sm_count, stream, qkv_bias, position_embedding_type,
        rotary_embedding_dim, rotary_embedding_base, rotary_embedding_scale_type, rotary_embedding_scale,
        rotary_embedding_max_positions, RefExtras{});
}

/* Relative attention bias (T5-style): explicit table [num_heads, stride, stride] or, with max_distance > 0, the
 * implicit form with a bucket table [num_heads, stride]. */
extern "C" int REF_CAT(REF_FN(ref_mmha_relbias), REF_DH)(const void* qkv, void* out, const int32_t* sequence_length_dev,
    int64_t* block_pointers_dev, int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t max_blocks_per_seq,
    int32_t tokens_per_block, int32_t max_attention_window, int32_t past_kv_length, float q_scaling,
    const float* kv_scale_orig_quant_dev, const float* kv_scale_quant_orig_dev, int32_t int8_kv, int32_t fp8_kv,
    int32_t sm_count, cudaStream_t stream, const void* relative_attention_bias, int32_t relative_attention_bias_stride,
    int32_t max_distance)
{
    RefExtras x;
    x.relative_attention_bias = relative_attention_bias;
    x.relative_attention_bias_stride = relative_attention_bias_stride;
    x.max_distance = max_distance;
    return ref_mmha_impl(qkv, out, sequence_length_dev, block_pointers_dev, batch, num_heads, num_kv_heads,
        max_blocks_per_seq, tokens_per_block, max_attention_window, past_kv_length, q_scaling, kv_scale_orig_quant_dev,
        kv_scale_quant_orig_dev, int8_kv, fp8_kv, 0, nullptr, sm_count, stream, nullptr, 5, 0, 10000.f, 0, 1.f, 0, x);
}

/* Same call with the remaining enqueueGeneration features: beam search (batch counts beams; cache_indir
 * [batch, max_attention_window], input_lengths [batch]), cyclic window, sink tokens, ALiBi slopes (T [num_heads]).
 * Single-block mode only; position shift off. */
extern "C" int REF_CAT(REF_FN(ref_mmha_ext), REF_DH)(const void* qkv, void* out, const int32_t* sequence_length_dev,
    int64_t* block_pointers_dev, int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t max_blocks_per_seq,
    int32_t tokens_per_block, int32_t max_attention_window, int32_t past_kv_length, float q_scaling,
    const float* kv_scale_orig_quant_dev, const float* kv_scale_quant_orig_dev, int32_t int8_kv, int32_t fp8_kv,
    int32_t sm_count, cudaStream_t stream, int32_t beam_width, const int32_t* cache_indir,
    const int32_t* input_lengths, int32_t cyclic_attention_window_size, int32_t sink_token_length,
    const void* linear_bias_slopes)
{
    RefExtras x;
    x.beam_width = beam_width;
    x.cache_indir = cache_indir;
    x.input_lengths = input_lengths;
    x.cyclic_attention_window_size = cyclic_attention_window_size;
    x.sink_token_length = sink_token_length;
    x.linear_bias_slopes = linear_bias_slopes;
    return ref_mmha_impl(qkv, out, sequence_length_dev, block_pointers_dev, batch, num_heads, num_kv_heads,
        max_blocks_per_seq, tokens_per_block, max_attention_window, past_kv_length, q_scaling, kv_scale_orig_quant_dev,
        kv_scale_quant_orig_dev, int8_kv, fp8_kv, 0, nullptr, sm_count, stream, nullptr,
        linear_bias_slopes ? 3 : 0, 0, 10000.f, 0, 1.f, 0, x);
}
