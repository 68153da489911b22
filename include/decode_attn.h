/*
 * decode_attn.h - C ABI of the B200 (sm_100a) generation-phase attention over a paged KV cache.
 *
 * Drop-in boundary for the generation branch of the reference's GPT attention plugin:
 *   GPTAttentionPluginCommon::enqueueGeneration
 *       cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:1159-1364
 * i.e. everything that branch does today through masked_multihead_attention()
 *   (cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention.h:230-243) or DecoderXQARunner::dispatch
 *   (cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderXQARunner.h:172-181):
 * for every sequence, append the new token's K/V to its cache block (quantising on write),
 * then compute softmax(q K^T / (sqrt(Dh) q_scaling)) V over past + new token, reading the paged,
 * optionally INT8 / FP8-E4M3 cache through the per-sequence block-pointer table.
 *
 * Plain C: pointers and sizes only, no C++/torch types.  All entry points return an int status
 * (DX_OK == 0); nothing throws across the boundary, nothing calls exit().
 *
 * Ownership: the caller owns every buffer (packed QKV, KV pool, pointer table, scales, output,
 * workspace).  dx_attn_enqueue_generation() is asynchronous on the given stream, allocates no device
 * memory and never synchronises.  The KV pool is mutated in place (new token appended), as in the
 * reference.
 */
#ifndef DECODE_ATTN_H_
#define DECODE_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DX_ABI_VERSION 1

/* Status codes. */
enum
{
    DX_OK = 0,
    DX_ERR_BAD_ARG = 1,     /* null / misaligned pointer, negative size, inconsistent lengths           */
    DX_ERR_UNSUPPORTED = 2, /* head size / dtype / feature outside what this library implements         */
    DX_ERR_WORKSPACE = 3,   /* workspace smaller than dx_attn_workspace_size() asks for                 */
    DX_ERR_CUDA = 4,        /* a CUDA runtime call failed; dx_attn_last_cuda_error() has the code       */
    DX_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (reported by dx_attn_device_status)    */
    DX_ERR_BOUNDS = 6       /* dx_attn_validate(): a block pointer or length is outside the given pool  */
};

/* Activation dtype (reference: plugin field "type_id", nvinfer1::DataType kHALF / kBF16). */
enum
{
    DX_DTYPE_FP16 = 0,
    DX_DTYPE_BF16 = 1
};

/* KV-cache quantisation bits, same values as tensorrt_llm::common::QuantMode
 * (cpp/tensorrt_llm/common/quantization.h:79-87, tensorrt_llm/quantization/mode.py:47-49). */
#define DX_QUANT_INT8_KV_CACHE (1 << 6)
#define DX_QUANT_FP8_KV_CACHE (1 << 7)

/* Static attributes.  Field names follow the plugin's creator fields
 * (cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:1558-1596). */
typedef struct dx_attn_config
{
    uint32_t struct_size; /* = sizeof(dx_attn_config); lets the struct grow compatibly */
    int32_t layer_idx;
    int32_t num_heads;    /* q heads on THIS rank (already divided by tp_size, as the plugin is built) */
    int32_t num_kv_heads; /* kv heads on this rank; num_heads % num_kv_heads == 0                     */
    int32_t head_size;    /* 64 or 128: streaming kernels; 256: the streaming per-head kernel, or the 16-bit grouped-head
                           * kernel for grouped heads over an unquantised cache.  32, 48, 80, 96, 104, 112, 144, 160, 192, 224
                           * (the other sizes of the reference's MMHA switch,
                           * decoderMaskedMultiheadAttention.cu:68-85): one CTA per sequence and q head, no
                           * split-K; a cache row must be a multiple of 16 bytes, so 104 needs a 16-bit cache */
    float q_scaling;      /* softmax scale = 1 / (sqrt(head_size) * q_scaling)                        */
    int32_t tp_size;      /* recorded only: heads are sharded by the caller, no communication here    */
    int32_t tp_rank;
    int32_t multi_block_mode;    /* 0: one CTA walks a whole sequence; 1: split-K + LSE merge allowed  */
    int32_t enable_xqa;          /* accepted for compatibility, ignored                                */
    int32_t kv_cache_quant_mode; /* 0, DX_QUANT_INT8_KV_CACHE or DX_QUANT_FP8_KV_CACHE                */
    int32_t paged_kv_cache;      /* must be 1                                                          */
    int32_t tokens_per_block;    /* power of two, 16..256                                              */
    int32_t type_id;             /* DX_DTYPE_FP16 / DX_DTYPE_BF16                                      */
    int32_t device;              /* CUDA device ordinal this handle launches on                        */
    /* --- optional tail (struct_size tells whether it is present; absent = all zero) ---
     * In-step pre-processing of the packed QKV row, as the reference kernels do it
     * (decoderMaskedMultiheadAttentionTemplate.h:1587-1712): bias add, then rotary embedding on q and k.
     * Values of position_embedding_type / rotary_embedding_scale_type are the reference's
     * (cpp/tensorrt_llm/kernels/gptKernels.h:41-58): 0 learned-absolute (nothing to do), 1 RoPE GPT-J,
     * 2 RoPE GPT-NeoX, 3 ALiBi, 4 ALiBi with scale (both: slopes per call, dx_attn_generation_params.alibi_slopes),
     * 5 relative (bias table per call, dx_attn_generation_params.relative_attention_bias);
     * scale type 0 none, 1 linear, 2 dynamic. */
    int32_t position_embedding_type;
    int32_t rotary_embedding_dim;
    float rotary_embedding_base;
    int32_t rotary_embedding_scale_type;
    float rotary_embedding_scale;
    int32_t rotary_embedding_max_positions;
    int32_t qkv_bias_enabled;    /* 1: calls may pass dx_attn_generation_params.qkv_bias (sizes the workspace) */
} dx_attn_config;
/* size of dx_attn_config without the optional tail (accepted by dx_attn_create) */
#define DX_ATTN_CONFIG_SIZE_V1 60u

/* Per-call arguments.  Field names and meaning follow
 * GPTAttentionPluginCommon::EnqueueGenerationParams
 *   (cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.h:127-166)
 * and the plugin's input list (cpp/tensorrt_llm/plugins/gptAttentionPlugin/gptAttentionPlugin.h:43-68). */
typedef struct dx_attn_generation_params
{
    uint32_t struct_size; /* = sizeof(dx_attn_generation_params) */
    /* device, T [num_requests, (num_heads + 2*num_kv_heads) * head_size]: Q | K | V of the new token
     * (bias / rotary embedding already applied). */
    const void* attention_input;
    /* device, int32 [num_requests]: sequence length INCLUDING the new token; the new token is
     * written at cache index sequence_lengths[b] - 1. */
    const int32_t* sequence_lengths;
    /* host, int32 [num_requests]: past length of every sequence (== sequence_lengths[b] - 1).
     * Used on the host to size the launch; may be NULL if past_kv_length is given. */
    const int32_t* host_past_key_value_lengths;
    /* max over the batch of the past length (the plugin computes it from the host array,
     * gptAttentionPlugin.cpp:558-563).  Ignored when host_past_key_value_lengths != NULL. */
    int32_t past_kv_length;
    int32_t beam_width;                   /* > 1: every per-sequence array has num_requests * beam_width rows
                                           * (the reference's batch_beam, gptAttentionCommon.cpp:1186);
                                           * cache_indir and context_lengths must be given          */
    int32_t num_requests;                 /* batch                                                  */
    int32_t max_blocks_per_sequence;      /* M: row length of the pointer table                     */
    int32_t max_attention_window;         /* cache capacity in tokens (row length of cache_indir)   */
    int32_t cyclic_attention_window_size; /* sliding window W: a sequence with more than W past tokens attends to
                                           * the W cache slots (and the new token), which then overwrites the
                                           * oldest non-sink slot (kvCacheUtils.h:109-117); needs a table without
                                           * the spare block, (M-1)*tokens_per_block < W                       */
    int32_t sink_token_length;            /* tokens that are never overwritten; a multiple of tokens_per_block
                                           * (other values need the reference's position shift: unsupported)   */
    /* device, int64 [num_requests, 2, M]: KVBlockArray::data for this layer - K row then V row of
     * device pointers per sequence (cpp/tensorrt_llm/kernels/kvCacheUtils.h:36-153). */
    const int64_t* block_pointers;
    /* optional host mirror of block_pointers (plugin input host_kv_cache_block_pointers); only
     * used by dx_attn_validate(). */
    const int64_t* host_block_pointers;
    const float* kv_scale_orig_quant; /* device float[1]: multiply to quantise                     */
    const float* kv_scale_quant_orig; /* device float[1]: multiply to dequantise                   */
    void* context_buf;                /* device, T [num_requests, num_heads * head_size]: output   */
    void* workspace;                  /* device, >= dx_attn_workspace_size(); 128-byte aligned      */
    size_t workspace_bytes;
    /* device, int32 [num_requests * beam_width, max_attention_window] or NULL: for beam search, the beam whose cache holds
     * slot t of this sequence (decoderMaskedMultiheadAttentionTemplate.h:2063-2078) */
    const int32_t* cache_indir;
    /* optional tail 1: device, T [(num_heads + 2*num_kv_heads) * head_size] or NULL (plugin input qkv_bias) */
    const void* qkv_bias;
    /* optional tail 2 */
    /* device, int32 [num_requests * beam_width]: prompt length of every sequence; with beams, slots below it are read
     * from beam 0 of the request (decoderMaskedMultiheadAttentionTemplate.h:1497-1498) */
    const int32_t* context_lengths;
    /* device, T [num_heads] or NULL: ALiBi slopes of this rank's heads; score += slope * (slot - past length)
     * (decoderMaskedMultiheadAttentionTemplate.h:1890-1895, :2026).  Needs position_embedding_type 3 or 4. */
    const void* alibi_slopes;
    /* optional tail 3: several new tokens per sequence in one step - the reference's Medusa mode
     * (is_medusa_enabled; gptAttentionPlugin.cpp:541-556, :622-627, :646-650; gptAttentionCommon.cpp:195-239).
     * input_seq_length = Q = number of draft tokens + 1 (0 and 1 both mean the usual single token).  With Q > 1:
     *   attention_input / context_buf have num_requests * Q rows, row b * Q + t is token t of sequence b;
     *   sequence_lengths[b] INCLUDES the Q new tokens, token t is stored at cache index sequence_lengths[b] - Q + t
     *     (unfusedAttentionKernels_2_template.h:254-255);
     *   host_past_key_value_lengths[b] = sequence_lengths[b] - Q;
     *   token t attends to every earlier cache entry and to new token j where bit j of its mask row is set
     *     (bit j of row t = bit j % 32 of word j / 32; tensorrt_llm/runtime/medusa_utils.py:50-82; its own bit t is set);
     *   with a rotary embedding configured, token t is rotated at position
     *     medusa_position_offsets[b * Q + t] + sequence_lengths[b] - Q (unfusedAttentionKernels_2_template.h:258-262).
     * beam_width must be 1; no cyclic window shorter than the sequences, no sink tokens, no ALiBi, no dynamic
     * rotary scaling (DX_ERR_UNSUPPORTED).  Unlike the reference (whose multi-token kernels take 16-bit caches only,
     * decoderXQAImplPrecompiled.cpp:322-323) every cache type is served. */
    int32_t input_seq_length;
    int32_t reserved0; /* 0 */
    /* device, int32 [num_requests, Q, (Q + 31) / 32] (plugin input medusa_packed_mask) */
    const int32_t* medusa_packed_mask;
    /* device, int32 [num_requests, Q] or NULL = offset t for token t (plugin input medusa_position_offsets) */
    const int32_t* medusa_position_offsets;
    /* optional tail 4: relative attention bias (T5-style; EnqueueGenerationParams::relative_attention_bias,
     * gptAttentionCommon.h:156-158).  Needs position_embedding_type 5 (relative).
     *   max_distance == 0: device, T [num_heads, stride, stride]; the score of cache slot s gets
     *     bias[head][past length][s] added (decoderMaskedMultiheadAttentionTemplate.h:1773-1797, :1981-2026);
     *   max_distance > 0 (the plugin attribute of that name): the implicit form, device T [num_heads, stride] with
     *     stride = number of buckets; the bias is table[head][bucket(s - past length)] with the reference's bucket
     *     function (decoderMaskedMultiheadAttentionTemplate.h:1957-1978). */
    const void* relative_attention_bias;
    int32_t relative_attention_bias_stride;
    int32_t max_distance;
} dx_attn_generation_params;
/* sizes of dx_attn_generation_params without the optional tails (all are accepted by the enqueue calls) */
#define DX_ATTN_GENERATION_PARAMS_SIZE_V1 offsetof(dx_attn_generation_params, qkv_bias)
#define DX_ATTN_GENERATION_PARAMS_SIZE_V2 offsetof(dx_attn_generation_params, context_lengths)
#define DX_ATTN_GENERATION_PARAMS_SIZE_V3 offsetof(dx_attn_generation_params, input_seq_length)
#define DX_ATTN_GENERATION_PARAMS_SIZE_V4 offsetof(dx_attn_generation_params, relative_attention_bias)

typedef struct dx_attn dx_attn_t;

/* Replaces GPTAttentionPluginCommon's constructor checks + initialize()
 * (gptAttentionCommon.cpp:445-464, :1423-1490).  Queries the device (SM count, shared memory),
 * sets kernel attributes and allocates one 256-byte device status word. */
int dx_attn_create(const dx_attn_config* config, dx_attn_t** out);
void dx_attn_destroy(dx_attn_t* handle);

/* Replaces GPTAttentionPluginCommon::getWorkspaceSizeForGeneration (gptAttentionCommon.cpp:585-626).
 * Upper bound for any call with num_requests <= batch; 0 when multi_block_mode is off and no in-step
 * pre-processing (bias / rotary embedding) is configured.  `batch` counts rows of attention_input: sequences x beams,
 * and x input_seq_length for calls with several new tokens per sequence (the reference sizes by total_num_seq too). */
size_t dx_attn_workspace_size(const dx_attn_t* handle, int32_t batch, int32_t max_past_len);

/* Replaces GPTAttentionPluginCommon::enqueueGeneration (gptAttentionCommon.cpp:1159-1364). */
int dx_attn_enqueue_generation(dx_attn_t* handle, const dx_attn_generation_params* params, void* cuda_stream);

/* Same call for callers whose step inputs live in HOST memory (pinned or pageable): copies
 * attention_input, sequence_lengths and block_pointers to device staging owned by the handle
 * (grown on demand, the only allocation this library ever makes after create), runs the step and
 * copies context_buf back to the host pointer.  All of params' attention_input, sequence_lengths,
 * block_pointers and context_buf are HOST pointers here; the scales, the KV pool and the workspace
 * stay on the device.  Mirrors what the reference runtime does every step before enqueueV3
 * (tensorrt_llm/runtime/generation.py:2219-2221).
 * The copies run on two streams owned by the handle, the kernels on cuda_stream, with four staging slots:
 * with sync == 0 the call returns at once and the copies of later calls overlap these kernels; the
 * output is in host memory after dx_attn_host_sync() (or when the fourth call after this one returns: it
 * waits for the slot).  With sync != 0 the output is in host memory on return.  The host buffers of a
 * call must stay untouched until then. */
int dx_attn_enqueue_generation_host(
    dx_attn_t* handle, const dx_attn_generation_params* params, void* cuda_stream, int32_t sync);

/* No counterpart in the reference.  Same step as dx_attn_enqueue_generation for callers that cannot
 * hand over a workspace: hosts whose scratch request was fixed before the live batch was known, code
 * running while the device allocator is frozen or simply absent (cudaMalloc is off limits there).
 * The split-K partial results go to a fixed DX_STATIC_SCRATCH_BYTES array inside the library's device
 * image instead of params->workspace (which is ignored); every GPU that loads the library holds that
 * array until the process exits.  The call allocates nothing and calls no allocating routine.
 *  - A batch whose partials need more than DX_STATIC_SCRATCH_BYTES is refused with DX_ERR_WORKSPACE
 *    before anything is launched (dx_attn_workspace_size() gives an upper bound of the need).  Calls that need
 *    no partials - a wrapped sliding window, sink tokens, relative attention bias, several new tokens per
 *    sequence, head sizes other than 64 / 128 - are never refused for their length.
 *  - The first call on a device looks the array's device address up (cudaGetSymbolAddress), which may make the
 *    driver load the library's device code (a driver-side allocation): make that first call before any stream
 *    capture and before the allocator is frozen.  From the second call on a device nothing is allocated.
 *  - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in
 *    it has to start at zero, but two calls that overlap on the GPU (different streams, no ordering)
 *    race on it: serialise them. */
#define DX_STATIC_SCRATCH_BYTES (8u << 20)
int dx_attn_enqueue_generation_static_scratch(
    dx_attn_t* handle, const dx_attn_generation_params* params, void* cuda_stream);
size_t dx_attn_static_scratch_bytes(void);

/* Context-phase KV append: stores the K and V of whole prompts, k_src / v_src = device T
 * [batch, num_kv_heads, seq_len, head_size], into the paged cache with the same quantise-on-write as the
 * decode step; tokens at or beyond sequence_lengths[b] are skipped.  Replaces invokeTranspose4dBatchMajor
 * (cpp/tensorrt_llm/kernels/unfusedAttentionKernels.cu:1638-1666), same argument meaning.
 * attention_window_size < sequence_lengths[b]: the cache is cyclic, only the last attention_window_size tokens
 * of the sequence are stored (:1591-1600), token t in slot t % attention_window_size - or, in a table with a spare
 * block ((max_blocks_per_sequence - 1) * tokens_per_block >= attention_window_size), in slot
 * t % (attention_window_size + tokens_per_block), as KVBlockArray::getKVTokenIdx lays it out
 * (cpp/tensorrt_llm/kernels/kvCacheUtils.h:71-117). */
int dx_attn_append_context(dx_attn_t* handle, const void* k_src, const void* v_src,
    const int32_t* sequence_lengths, int32_t batch, int32_t seq_len, int32_t attention_window_size,
    const int64_t* block_pointers, int32_t max_blocks_per_sequence, const float* kv_scale_orig_quant,
    void* cuda_stream);

/* The same with sink tokens (the KVBlockArray the reference builds for the context phase carries
 * params.sink_token_length, cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:659-660):
 * tokens below sink_token_length keep their slots, the others cycle behind them; sink tokens that end inside
 * a block leave the rest of that block unused.  0 <= sink_token_length < attention_window_size. */
int dx_attn_append_context_cyclic(dx_attn_t* handle, const void* k_src, const void* v_src,
    const int32_t* sequence_lengths, int32_t batch, int32_t seq_len, int32_t attention_window_size,
    int32_t sink_token_length, const int64_t* block_pointers, int32_t max_blocks_per_sequence,
    const float* kv_scale_orig_quant, void* cuda_stream);

/* Waits until the outputs of all dx_attn_enqueue_generation_host calls made so far are in host memory.
 * No reference counterpart (the reference runtime synchronises the whole stream every step). */
int dx_attn_host_sync(dx_attn_t* handle);

/* Device-resident form of the runtime's per-step cache bookkeeping (KVCacheManager.step + get_block_pointers for
 * unfinished sequences, tensorrt_llm/runtime/kv_cache_manager.py:305-345, :380-387, which the reference runs on
 * the host and uploads every step, tensorrt_llm/runtime/generation.py:2219-2221).  On the stream: every
 * sequence_lengths[b] grows by one (it then counts the token the next decode step writes); a sequence whose new
 * token starts a block takes the next entry of free_blocks (device, int64 [n_free, 2]: K block pointer, V block
 * pointer) in batch order, written into block_pointers (device, int64 [num_requests, 2, M]); *free_cursor
 * (device) is the first unused entry, read and advanced.  The table is the one the host manager builds for the
 * same free list.  An exhausted list or table row is reported by dx_attn_device_status as DX_ERR_BOUNDS (the
 * pointer is then not written).  Launches one kernel; allocates nothing; may be captured in a CUDA graph
 * together with dx_attn_enqueue_generation. */
int dx_kv_cache_step(dx_attn_t* handle, int32_t* sequence_lengths, int64_t* block_pointers, int32_t num_requests,
    int32_t max_blocks_per_sequence, const int64_t* free_blocks, int32_t n_free, int32_t* free_cursor,
    void* cuda_stream);

/* Host-side check of a block-pointer table against the pool it must point into; launches nothing.
 * Stands in for the bounds checking the reference does not have (its kernels trust the table). */
int dx_attn_validate(const dx_attn_t* handle, const int64_t* host_block_pointers,
    const int32_t* host_past_key_value_lengths, int32_t num_requests, int32_t max_blocks_per_sequence,
    const void* pool_base, size_t pool_bytes);

/* Number of split-K partitions and tokens per partition the next enqueue would use for this batch /
 * max past length (reference analogue: multi_block_grid_setup,
 * cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionLaunch.h:94-143). */
int dx_attn_plan(const dx_attn_t* handle, int32_t batch, int32_t max_past_len, int32_t* num_partitions,
    int32_t* tokens_per_partition, int32_t* kernel_kind);
/* The same for a given vector of host past lengths: exactly what dx_attn_enqueue_generation plans when it is
 * passed host_past_key_value_lengths and enough workspace (dx_attn_plan assumes every sequence has max_past_len
 * tokens).  A stream-K launch (equal ranges of the batch's tokens per CTA instead of per-sequence partitions) is
 * reported as *num_partitions = -(number of CTAs), *tokens_per_partition = tokens per CTA. */
int dx_attn_plan_lengths(const dx_attn_t* handle, const int32_t* host_past_key_value_lengths, int32_t batch,
    int32_t* num_partitions, int32_t* tokens_per_partition, int32_t* kernel_kind);

/* Reads (synchronously) and clears the device status word.  DX_OK; DX_ERR_TIMEOUT: a bounded device-side wait ran
 * out; DX_ERR_BOUNDS: dx_kv_cache_step ran out of blocks, or a device sequence length needed more split-K
 * partitions than the call was planned with (host_past_key_value_lengths smaller than the device lengths).
 * The word is sticky: while it holds a report every later wait on the device gives up after a few hundred polls, so
 * the steps enqueued after the failing one return quickly with undefined results.  After any report the caller
 * must read it with this call (which clears it) before results are trusted again.  No reference counterpart (the
 * reference's kernels wait without a limit). */
int dx_attn_device_status(dx_attn_t* handle);
/* Self-test of that reporting path, no reference counterpart: launches one warp that waits, for at most poll_limit
 * polls (1 .. 2^20), on a barrier nothing ever arrives on, and then records a time-out exactly as the attention
 * kernels would.  dx_attn_device_status() returns DX_ERR_TIMEOUT afterwards.  Nothing hangs or faults. */
int dx_attn_selftest_wait_timeout(dx_attn_t* handle, int32_t poll_limit, void* cuda_stream);

/* Bounds-checked build (compiled with -DDECODE_ATTN_BOUNDS_CHECK, libdecode_attn_checked.so; a debugging aid with no
 * reference counterpart - the reference relies on compute-sanitizer runs): every block-table look-up of the kernels
 * checks that the block index lies inside the table row and that the pointer is non-null, 16-byte aligned and, once
 * a pool range is registered, inside that pool; the first violation is recorded (dx_attn_device_status() returns
 * DX_ERR_BOUNDS) and the access goes to a spare block the handle owns, so nothing outside the caller's memory is
 * read or written.  dx_build_has_bounds_check() tells which build is loaded; dx_attn_set_pool_range() registers
 * [pool, pool + pool_bytes) as the only memory cache blocks may lie in (NULL, 0: no range; the regular build
 * stores it and ignores it). */
int dx_build_has_bounds_check(void);
int dx_attn_set_pool_range(dx_attn_t* handle, const void* pool, size_t pool_bytes);
/* Last cudaError_t seen by this handle (0 if none). */
int dx_attn_last_cuda_error(const dx_attn_t* handle);
/* Kernels launched by this handle since creation (for launch accounting in benchmarks). */
int64_t dx_attn_launch_count(const dx_attn_t* handle);

const char* dx_strerror(int status);
int dx_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DECODE_ATTN_H_ */
