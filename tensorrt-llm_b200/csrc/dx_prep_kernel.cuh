// Decode-step pre-processing of the packed QKV row: + bias, rotary position embedding on q and k.
//
// The result goes to a scratch copy of QKV that the attention kernels then read (the reference's
// XQA route also runs bias / RoPE as its own launch before the attention kernel,
//   cpp/tensorrt_llm/kernels/unfusedAttentionKernels/unfusedAttentionKernels_2_template.h:161-390;
// its MMHA kernel does the same arithmetic inline,
//   decoderMaskedMultiheadAttentionTemplate.h:1587-1712 with the helpers of
//   decoderMaskedMultiheadAttentionUtils.h:2530-2760).
// Arithmetic as in the reference: bias is added in T (one rounding); a rotary pair is converted to
// fp32, rotated with cosf / sinf of  t * scale / powf(base, 2p / rot_dim), and rounded back to T.
// GPT-J pairs adjacent channels (2p, 2p+1) and uses base / scale as given; GPT-NeoX pairs
// (p, p + rot_dim/2) and uses the scale-type-adjusted base / scale.  The position is the cache
// index of the new token (sequence_length - 1).  QKV is tiny (a few MB): one thread per pair.
#pragma once

#include "dx_common.cuh"

namespace dx
{

enum : int
{
    POS_LEARNED_ABSOLUTE = 0,
    POS_ROPE_GPTJ = 1,
    POS_ROPE_GPT_NEOX = 2,
    POS_ALIBI = 3,           // no change of q / k; slopes are added to the scores
    POS_ALIBI_WITH_SCALE = 4,
    POS_RELATIVE = 5         // no change of q / k; a bias table is added to the scores
};

enum : int
{
    ROT_SCALE_NONE = 0,
    ROT_SCALE_LINEAR = 1,
    ROT_SCALE_DYNAMIC = 2
};

struct PrepArgs
{
    const void* qkv;   // T [B, (H + 2 Hkv) Dh]
    const void* bias;  // T [(H + 2 Hkv) Dh] or nullptr
    void* out;         // T [B, (H + 2 Hkv) Dh]
    const int32_t* seq_len;
    // several new tokens per sequence: row r is token r % q_len of sequence r / q_len, rotated at position
    // pos_offsets[r] (or r % q_len) + sequence length - q_len (unfusedAttentionKernels_2_template.h:254-262)
    const int32_t* pos_offsets;
    int32_t q_len; // 1: the usual single token at position sequence length - 1
    int32_t batch, num_heads, num_kv_heads, head_size; // batch: rows
    int32_t pos_type, rot_dim, rot_scale_type, rot_max_positions;
    float rot_base, rot_scale;
};

template <typename T>
__global__ void __launch_bounds__(256) qkv_bias_rope_kernel(const PrepArgs a)
{
    const int half_dh = a.head_size / 2;
    const int heads = a.num_heads + 2 * a.num_kv_heads;
    const long idx = (long) blockIdx.x * blockDim.x + threadIdx.x;
    const long per_seq = (long) heads * half_dh;
    if (idx >= per_seq * a.batch)
        return;
    const int b = (int) (idx / per_seq);
    const int rem = (int) (idx % per_seq);
    const int head = rem / half_dh, p = rem % half_dh;
    const bool is_v = head >= a.num_heads + a.num_kv_heads;
    int t_step = a.seq_len[b / a.q_len] - 1;
    if (a.q_len > 1)
        t_step += 1 - a.q_len + (a.pos_offsets ? a.pos_offsets[b] : b % a.q_len);

    // which two channels this thread owns
    const bool rope = !is_v && a.pos_type != POS_LEARNED_ABSOLUTE && 2 * p < a.rot_dim;
    int c0, c1;
    if (a.pos_type == POS_ROPE_GPT_NEOX && 2 * p < a.rot_dim)
    {
        c0 = p;
        c1 = p + a.rot_dim / 2;
    }
    else
    {
        c0 = 2 * p;
        c1 = 2 * p + 1;
    }
    const size_t row = ((size_t) b * heads + head) * a.head_size;
    const T* src = reinterpret_cast<const T*>(a.qkv) + row;
    T x0 = src[c0], x1 = src[c1];
    if (a.bias)
    {
        const T* bias = reinterpret_cast<const T*>(a.bias) + (size_t) head * a.head_size;
        x0 = __hadd(x0, bias[c0]);
        x1 = __hadd(x1, bias[c1]);
    }
    if (rope)
    {
        float base = a.rot_base, scale = a.rot_scale;
        if (a.pos_type == POS_ROPE_GPT_NEOX)
        {
            if (a.rot_scale_type == ROT_SCALE_DYNAMIC)
            {
                if (t_step > a.rot_max_positions)
                {
                    const float bb = (scale * t_step / a.rot_max_positions) - (scale - 1);
                    const float pp = static_cast<float>(a.rot_dim) / (a.rot_dim - 2);
                    base = base * __powf(bb, pp);
                }
                scale = 1.0f;
            }
            else if (a.rot_scale_type == ROT_SCALE_LINEAR)
            {
                scale = 1.0f / scale;
            }
        }
        const int zid = 2 * p;
        const float inv_freq = float(t_step * scale) / powf(base, zid / (float) a.rot_dim);
        const float2 coef = make_float2(cosf(inv_freq), sinf(inv_freq));
        const float2 v = make_float2(TypeOps<T>::to_float(x0), TypeOps<T>::to_float(x1));
        float2 rot_v;
        rot_v.x = coef.x * v.x - coef.y * v.y;
        rot_v.y = coef.x * v.y + coef.y * v.x;
        x0 = TypeOps<T>::from_float(rot_v.x);
        x1 = TypeOps<T>::from_float(rot_v.y);
    }
    T* dst = reinterpret_cast<T*>(a.out) + row;
    dst[c0] = x0;
    dst[c1] = x1;
}

} // namespace dx
