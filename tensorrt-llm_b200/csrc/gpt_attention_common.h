// Host-side C++ mirror of the reference plugin's generation interface, layered over the C ABI.
//
// A maintainer replacing the decode branch of the reference plugin keeps calling
//   enqueueGeneration(EnqueueGenerationParams<T>, stream)
// with the same field names as
//   GPTAttentionPluginCommon::EnqueueGenerationParams
//     (cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.h:127-166)
// and the same static attributes as the plugin constructor
//     (cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:375-443).
// Header-only, no CUDA headers needed: the stream is passed through as an opaque pointer.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/decode_attn.h"

namespace dx
{

struct half_tag
{
};
struct bf16_tag
{
};

template <typename T>
struct EnqueueGenerationParams
{
    T const* attention_input = nullptr;
    T const* qkv_bias = nullptr; // needs setQkvBiasEnabled(true) before initialize()
    int32_t input_seq_length = 1;
    int32_t const* sequence_lengths = nullptr;
    int32_t past_kv_length = 0;
    int32_t beam_width = 1;
    int32_t const* context_lengths = nullptr;
    float const* kv_scale_orig_quant = nullptr;
    float const* kv_scale_quant_orig = nullptr;
    T const* alibi_slopes = nullptr; // needs an ALiBi position embedding type (setPositionEmbedding)
    // Medusa mode (gptAttentionCommon.h:162-165): input_seq_length > 1 new tokens per sequence under a packed mask
    int32_t const* medusa_packed_mask = nullptr;
    int32_t const* medusa_position_offsets = nullptr;
    // relative position (gptAttentionCommon.h:156-158); max_distance is the plugin attribute of that name
    T const* relative_attention_bias = nullptr;
    int relative_attention_bias_stride = 0;
    int max_distance = 0;
    T* context_buf = nullptr;
    void* key_value_cache = nullptr; // contiguous cache: not supported, must be nullptr
    void* block_pointers = nullptr;
    int32_t max_attention_window = 0;
    int32_t cyclic_attention_window_size = 0;
    int32_t sink_token_length = 0;
    int32_t num_requests = 0;
    int32_t max_blocks_per_sequence = 0;
    int32_t const* cache_indir = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0; // addition: the reference trusts getWorkspaceSize(); this library checks
    int32_t const* host_past_key_value_lengths = nullptr;
};

class GPTAttentionCommon
{
public:
    GPTAttentionCommon(int layer_idx, int num_heads, int num_kv_heads, int head_size, float q_scaling, int tp_size,
        int tp_rank, bool multi_block_mode, bool enable_xqa, int kv_cache_quant_mode, bool paged_kv_cache,
        int tokens_per_block, int type_id /* DX_DTYPE_FP16 | DX_DTYPE_BF16 */, int device)
    {
        mConfig.struct_size = sizeof(dx_attn_config);
        mConfig.layer_idx = layer_idx;
        mConfig.num_heads = num_heads;
        mConfig.num_kv_heads = num_kv_heads;
        mConfig.head_size = head_size;
        mConfig.q_scaling = q_scaling;
        mConfig.tp_size = tp_size;
        mConfig.tp_rank = tp_rank;
        mConfig.multi_block_mode = multi_block_mode;
        mConfig.enable_xqa = enable_xqa;
        mConfig.kv_cache_quant_mode = kv_cache_quant_mode;
        mConfig.paged_kv_cache = paged_kv_cache;
        mConfig.tokens_per_block = tokens_per_block;
        mConfig.type_id = type_id;
        mConfig.device = device;
    }

    // Rotary position embedding / bias applied inside the step (call before initialize()); values are the
    // reference's PositionEmbeddingType / RotaryScalingType (cpp/tensorrt_llm/kernels/gptKernels.h:41-58).
    void setPositionEmbedding(int position_embedding_type, int rotary_embedding_dim, float rotary_embedding_base,
        int rotary_embedding_scale_type, float rotary_embedding_scale, int rotary_embedding_max_positions)
    {
        mConfig.position_embedding_type = position_embedding_type;
        mConfig.rotary_embedding_dim = rotary_embedding_dim;
        mConfig.rotary_embedding_base = rotary_embedding_base;
        mConfig.rotary_embedding_scale_type = rotary_embedding_scale_type;
        mConfig.rotary_embedding_scale = rotary_embedding_scale;
        mConfig.rotary_embedding_max_positions = rotary_embedding_max_positions;
    }

    void setQkvBiasEnabled(bool enabled)
    {
        mConfig.qkv_bias_enabled = enabled;
    }

    GPTAttentionCommon(GPTAttentionCommon const&) = delete;
    GPTAttentionCommon& operator=(GPTAttentionCommon const&) = delete;

    ~GPTAttentionCommon()
    {
        terminate();
    }

    // reference: GPTAttentionPluginCommon::initialize (gptAttentionCommon.cpp:1423-1490)
    int initialize()
    {
        if (mHandle)
            return DX_OK;
        return dx_attn_create(&mConfig, &mHandle);
    }

    void terminate()
    {
        if (mHandle)
            dx_attn_destroy(mHandle);
        mHandle = nullptr;
    }

    // reference: getWorkspaceSizeForGeneration (gptAttentionCommon.cpp:585-626)
    size_t getWorkspaceSizeForGeneration(int32_t total_num_seq, int32_t max_attention_window) const
    {
        return mHandle ? dx_attn_workspace_size(mHandle, total_num_seq, max_attention_window) : 0;
    }

    // reference: enqueueGeneration (gptAttentionCommon.cpp:1159-1364).  Returns a DX_* status.
    template <typename T>
    int enqueueGeneration(EnqueueGenerationParams<T> const& params, void* stream)
    {
        if (!mHandle)
            return DX_ERR_BAD_ARG;
        if (params.key_value_cache)
            return DX_ERR_UNSUPPORTED; // contiguous cache
        dx_attn_generation_params p{};
        p.struct_size = sizeof(p);
        p.attention_input = params.attention_input;
        p.sequence_lengths = params.sequence_lengths;
        p.host_past_key_value_lengths = params.host_past_key_value_lengths;
        p.past_kv_length = params.past_kv_length;
        p.beam_width = params.beam_width;
        p.num_requests = params.num_requests;
        p.max_blocks_per_sequence = params.max_blocks_per_sequence;
        p.max_attention_window = params.max_attention_window;
        p.cyclic_attention_window_size = params.cyclic_attention_window_size;
        p.sink_token_length = params.sink_token_length;
        p.block_pointers = static_cast<const int64_t*>(params.block_pointers);
        p.kv_scale_orig_quant = params.kv_scale_orig_quant;
        p.kv_scale_quant_orig = params.kv_scale_quant_orig;
        p.context_buf = params.context_buf;
        p.workspace = params.workspace;
        p.workspace_bytes = params.workspace_bytes;
        p.cache_indir = params.cache_indir;
        p.qkv_bias = params.qkv_bias;
        p.context_lengths = params.context_lengths;
        p.alibi_slopes = params.alibi_slopes;
        p.input_seq_length = params.input_seq_length;
        p.medusa_packed_mask = params.medusa_packed_mask;
        p.medusa_position_offsets = params.medusa_position_offsets;
        p.relative_attention_bias = params.relative_attention_bias;
        p.relative_attention_bias_stride = params.relative_attention_bias_stride;
        p.max_distance = params.max_distance;
        return dx_attn_enqueue_generation(mHandle, &p, stream);
    }

    dx_attn_t* handle() const
    {
        return mHandle;
    }

    // Reference behaviour on errors is to throw (TLLM_CHECK); callers that want that can use this.
    static void throwOnError(int status, char const* what)
    {
        if (status != DX_OK)
            throw std::runtime_error(std::string(what) + ": " + dx_strerror(status));
    }

private:
    dx_attn_config mConfig{};
    dx_attn_t* mHandle = nullptr;
};

} // namespace dx
