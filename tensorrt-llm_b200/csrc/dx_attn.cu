// C-ABI implementation: argument checking, launch planning (split-K), workspace carving and the
// kernel launches for the generation-phase attention.  Host logic mirrors
//   GPTAttentionPluginCommon::enqueueGeneration
//     cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:1159-1364
// and the launcher side of the reference kernels
//     cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention/decoderMaskedMultiheadAttentionLaunch.h:94-295.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/decode_attn.h"
#include "dx_append_kernel.cuh"
#include "dx_kvstep_kernel.cuh"
#include "dx_launch.h"
#include "dx_merge_kernel.cuh"
#include "dx_prep_kernel.cuh"
#include "dx_selftest_kernel.cuh"

using namespace dx;

namespace
{

enum KernelKind : int
{
    KIND_MHA = 0, // CUDA-core kernel, one CTA per q head
    KIND_GQA = 1, // tensor-core kernel, one CTA per kv head (x 16-head slice)
    KIND_TOK = 3, // tcgen05 kernel, token-major, one CTA per kv head, FP8 cache, Dh 128, up to 16 heads per kv head
    KIND_WIDE = 2, // tcgen05 kernel, one CTA per kv head (x 128-head slice), FP8 cache, more than 16 heads per kv head
    KIND_TOKWS = 4, // persistent warp-specialised tcgen05 kernel, token-major, one CTA per SM, two-level stream-K ranges
    KIND_GENERAL = 5 // feature-complete kernels (reported by the plan queries for head sizes other than 64 / 128)
};

struct Plan
{
    int kind = KIND_MHA;
    int hgroups = 1;    // 16-head slices per kv head (GQA kernel)
    bool heads16 = false;
    int rows = 0;       // grid.y * grid.z
    int resident = 2;   // CTAs per SM of the chosen kernel
    bool six = false;   // stream-K launch on the six-warp form of the grouped-head kernel
    int nsplit = 1;     // grid.x
    int chunk_tokens = 0;
    size_t part_o_bytes = 0, part_ml_bytes = 0;
    size_t workspace() const
    {
        return part_o_bytes + part_ml_bytes;
    }
};

size_t align_up(size_t x, size_t a)
{
    return (x + a - 1) / a * a;
}

} // namespace

struct dx_attn
{
    dx_attn_config cfg{};
    int sm_count = 0;
    int max_smem_optin = 0;
    int cache_kind = CACHE_T;
    int tpb_log2 = 0;
    int group = 1; // q heads per kv head
    int waves = 8;               // bound on the partitions a call may need: waves * SMs * 3 CTAs (workspace sizing)
    int min_chunk = 256;         // smallest partition bound, tokens
    int fixed_cost_tokens = 400; // per-CTA fixed cost (prologue, pipeline fill, epilogue) in tokens of streaming time
    KernelInfo k_mha{}, k_gqa[2]{}, k_wide{}, k_tok{}, k_merge{}, k_append{}; // k_gqa[16 heads per CTA?]
    KernelInfo k_gqa_feat[2]{}; // feature form of k_gqa (beam search, cyclic window, ALiBi)
    KernelInfo k_gqa_multi[2]{}; // several-new-tokens form of k_gqa (rows = (token, head) pairs of a kv head)
    bool no_dependent_launch = false; // set while the host-buffer entry point enqueues its step
    int pdl_other = 1;           // the same for the wide-group and per-head kernels (DX_ATTN_PDL_OTHER; c1 10.2 -> 9.6, c2 135.2 -> 134.4, c3 34.5 -> 33.4 us)
    int pdl_attention = -1;      // the 8-bit grouped-head kernel as a programmatic dependent of its predecessor:
                                 // 1 always, 0 never, -1 for stream-K launches with ranges of 4096 tokens or more
                                 // (measured: c4 / its TP2 shard / c5 gain ~1 %, the short ranges of small shards lose)
    bool feature_gqa = true;    // beams / ALiBi on grouped heads run on it (0: on the per-head feature kernel)
    KernelInfo k_gqa_six{}; // stream-K form of k_gqa[0] with two six-warp CTAs per SM (where built)
    bool wide = false;       // wide-group kernel usable for this configuration
    bool tok = false;        // token-major tcgen05 kernel usable for this configuration
    KernelInfo k_tokws{};    // its persistent warp-specialised form
    bool tokws = false;
    int ws_tail_pct = 0;     // share of the tiles (per cent) handed out as short dynamic ranges (0: static ranges only)
    int ws_tail_div = 8;     // a dynamic range is 1/ws_tail_div of a static one ...
    int ws_min_u2 = 2;       // ... but at least this many 128-token tiles
    int ws_min_u1 = 8;       // below this many tiles per static range the schedule stays single-level
    GeneralKernels k_general{}; // beams / cyclic window / sinks / ALiBi
    const void* k_merge_sk = nullptr;
    const void* k_merge_many = nullptr; // classic merge with one CTA per q row, for launches with many partitions
    int merge_many_from = 32;           // partitions from which it is used (DX_ATTN_MERGE_MANY_FROM; 0: never): c5 TP8 shard, 50
                                        // partitions: 22.2 -> 20.8 us; no difference at 25 partitions
    bool streamk = true;        // grouped-head kernels: equal ranges of token groups per CTA instead of per-row partitions
    int sk_min_units = 48;      // stream-K only when a CTA's range is at least this many token groups: below, the
                                // second prologue / epilogue of a CTA that straddles a row boundary costs more
                                // than the even split wins (measured on the TP8 shards)
    int six_min_tokens = 4096;  // stream-K launches use the six-warp CTAs when a range is at least this long
    bool streamk16 = false;     // the 16-bit kernel measured slower with it on its benchmark shape (131 -> 137 us): opt-in
    int sk_row_factor = 6;      // ... and only when the average row is at most this many ranges long
    SkSchedule sk_zero{};       // third argument of classic launches of the grouped-head kernels
    int force_chunk = 0;     // > 0: partition bound forced (tuning)
    double wave_slack_from = 2.0; // waves beyond which 5 % of a wave of extra CTAs is not counted as a further wave
    bool prep = false; // bias / rotary embedding configured: QKV is pre-processed into the workspace
    int32_t* status_dev = nullptr;
    TableGuard guard{}; // bounds-checked build: spare block and registered pool range (all zero otherwise)
    bool general_only = false; // head size without streaming kernels: every step runs on the feature-complete kernels
    int last_cuda_error = 0;
    std::atomic<int64_t> launches{0};
    // staging for the host-buffer entry point
    static constexpr int HOST_SLOTS = 4; // host-path steps that may be in flight
    void* stage_dev = nullptr;           // HOST_SLOTS slots of stage_bytes each
    size_t stage_bytes = 0;
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr; // copy streams of the host path (created on first use)
    cudaEvent_t ev_in[HOST_SLOTS] = {};   // inputs of the slot are on the device
    cudaEvent_t ev_done[HOST_SLOTS] = {}; // kernels of the slot have finished
    cudaEvent_t ev_out[HOST_SLOTS] = {};  // output of the slot is in host memory
    bool out_pending[HOST_SLOTS] = {};
    unsigned host_calls = 0;
};

namespace
{

// Accepts both layouts of dx_attn_generation_params (with and without the optional tail).
bool read_params(const dx_attn_generation_params* in, dx_attn_generation_params& out)
{
    if (!in)
        return false;
    if (in->struct_size != sizeof(dx_attn_generation_params) && in->struct_size != DX_ATTN_GENERATION_PARAMS_SIZE_V1
        && in->struct_size != DX_ATTN_GENERATION_PARAMS_SIZE_V2 && in->struct_size != DX_ATTN_GENERATION_PARAMS_SIZE_V3
        && in->struct_size != DX_ATTN_GENERATION_PARAMS_SIZE_V4)
        return false;
    memset(&out, 0, sizeof(out));
    memcpy(&out, in, in->struct_size);
    out.struct_size = sizeof(dx_attn_generation_params);
    return true;
}

// Partitions of one sequence of `total` tokens for a partition bound of `target` tokens.
inline long parts_of(long total, long target)
{
    return (total + target - 1) / target;
}

// Launch plan.  With multi_block_mode the partition bound T is chosen from the (host) lengths so
// that the CTAs fill k whole waves of resident CTAs, for the k in 1..4 (or no split at all) that
// minimises  waves * (fixed cost + tokens per CTA);  the kernels then cut every sequence into equal
// partitions of at most T tokens (partition_of).  host_past may be null: all sequences are then
// taken to have max_past_len tokens.
// First half: which kernel, how many CTA rows per sequence, resident CTAs per SM.  No partitioning yet.
Plan plan_shape(const dx_attn* h, int batch, int& rows_per_seq_out)
{
    Plan p;
    const dx_attn_config& c = h->cfg;
    const bool grouped = h->group > 1 && c.tokens_per_block >= (h->cache_kind == CACHE_T ? 16 : 32) && h->k_gqa[0].fn;
    p.kind = grouped ? KIND_GQA : KIND_MHA;
    int resident = 2, rows_per_seq = c.num_heads;
    if (grouped && h->wide)
    {
        p.kind = KIND_WIDE;
        p.hgroups = (h->group + 127) / 128;
        rows_per_seq = c.num_kv_heads * p.hgroups;
        resident = h->k_wide.resident;
    }
    else if (grouped && h->tok)
    {
        p.kind = KIND_TOK;
        p.hgroups = 1;
        rows_per_seq = c.num_kv_heads;
        resident = h->k_tok.resident;
    }
    else if (grouped)
    {
        p.hgroups = (h->group + 15) / 16;
        p.heads16 = h->group > 8;
        rows_per_seq = c.num_kv_heads * p.hgroups;
        resident = (h->cache_kind == CACHE_FP8 && c.head_size == 128 && !p.heads16) ? 3 : 2;
        if (h->k_gqa[p.heads16 ? 1 : 0].resident > 0)
            resident = h->k_gqa[p.heads16 ? 1 : 0].resident; // (the 16-bit kernel states it: 1 at head size 256)
    }
    else
    {
        resident = 3;
    }
    p.rows = batch * rows_per_seq;
    p.resident = resident;
    rows_per_seq_out = rows_per_seq;
    return p;
}

// Second half: the partition bound.  This runs on the host in front of every enqueue, so the search is kept
// cheap: the bounds tried are multiples of 128 tokens, for which ceil(len / T) only depends on ceil(len / 128) -
// the lengths are counted into 128-token buckets once and every candidate costs one division per occupied bucket.
void plan_partitions(const dx_attn* h, Plan& p, int batch, int rows_per_seq, int max_past_len, const int32_t* host_past)
{
    const dx_attn_config& c = h->cfg;
    const int resident = p.resident;
    const long max_total = (long) max_past_len + 1;
    long target = (long) align_up((size_t) max_total, 128);
    if (c.multi_block_mode)
    {
        const long t_min = std::max<long>(128, h->min_chunk);
        // Cost model, in tokens of one CTA's streaming time (fitted to measurements on B200):
        //     cost(T) = waves(T) * fixed + T / 2
        // waves(T) = CTAs / resident CTA slots, rounded up: every wave pays the per-CTA fixed cost
        // (prologue, pipeline fill, epilogue) once; T / 2 is the expected idle tail while the last
        // CTAs finish.  The streaming term (total tokens / slots) does not depend on T.
        const long slots = (long) h->sm_count * resident;
        const double fixed = (double) h->fixed_cost_tokens;
        const long t_max = (long) align_up((size_t) max_total, 128);
        double best = 1e300;
        // occupied buckets: (ceil(len / 128), sequences)
        constexpr int MAX_BUCKETS = 512;
        const uint32_t nb128 = (uint32_t) (t_max / 128);
        uint32_t bucket_len[MAX_BUCKETS], bucket_cnt[MAX_BUCKETS];
        int nbuckets = 0;
        const bool bucketed = host_past != nullptr && nb128 < MAX_BUCKETS;
        if (bucketed)
        {
            uint32_t hist[MAX_BUCKETS];
            for (uint32_t i = 0; i <= nb128; ++i)
                hist[i] = 0;
            for (int i = 0; i < batch; ++i)
                ++hist[std::min<uint32_t>(((uint32_t) host_past[i] + 128) >> 7, nb128)]; // ceil((past + 1) / 128)
            for (uint32_t i = 0; i <= nb128; ++i)
            {
                if (hist[i])
                {
                    bucket_len[nbuckets] = i;
                    bucket_cnt[nbuckets++] = hist[i];
                }
            }
        }
        for (long t = std::min(t_min, t_max); t <= t_max;)
        {
            long cnt = 0;
            if (!host_past)
            {
                cnt = (long) batch * parts_of(max_total, t);
            }
            else if (bucketed && (t & 127) == 0)
            {
                const uint32_t t128 = (uint32_t) (t >> 7);
                uint32_t acc = 0;
                for (int i = 0; i < nbuckets; ++i)
                    acc += bucket_cnt[i] * ((bucket_len[i] + t128 - 1) / t128);
                cnt = (long) acc;
            }
            else
            {
                for (int i = 0; i < batch; ++i)
                    cnt += parts_of((long) host_past[i] + 1, t);
            }
            cnt *= rows_per_seq;
            // a few CTAs over a whole number of waves ride along with the ragged finish of many waves, but cost a
            // whole extra round when there are only one or two
            const double fill = (double) cnt / (double) slots;
            const double waves = std::max(1.0, std::ceil(fill - (fill > h->wave_slack_from ? 0.05 : 0.0)));
            const double cost = waves * fixed + 0.5 * (double) std::min(t, max_total);
            const bool allowed = t == t_max || cnt <= (long) h->waves * slots; // keeps workspace_bound() valid
            if (allowed && cost < best)
            {
                best = cost;
                target = t;
            }
            if (t == t_max)
                break;
            // candidate bounds: every 128 tokens up to 2K, then coarser (about 6 % steps)
            const long step = t < 2048 ? 128 : align_up((size_t) (t / 16), 128);
            t = std::min(t + step, t_max);
        }
        if (h->force_chunk > 0)
            target = std::min<long>((long) align_up((size_t) h->force_chunk, 128), (long) align_up((size_t) max_total, 128));
    }
    p.chunk_tokens = (int) target;
    p.nsplit = (int) parts_of(max_total, target);
    if (p.nsplit > 1)
    {
        const size_t qrows = (size_t) batch * c.num_heads;
        p.part_o_bytes = align_up(qrows * p.nsplit * c.head_size * sizeof(float), 128);
        p.part_ml_bytes = align_up(qrows * p.nsplit * sizeof(float2), 128);
    }
}

Plan make_plan(const dx_attn* h, int batch, int max_past_len, const int32_t* host_past = nullptr)
{
    int rows_per_seq = 1;
    Plan p = plan_shape(h, batch, rows_per_seq);
    plan_partitions(h, p, batch, rows_per_seq, max_past_len, host_past);
    return p;
}

// Stream-K schedule (SkSchedule in dx_common.cuh) for a call planned on a grouped-head mma.sync kernel.  On
// success the plan's slot count and partial sizes are those of the schedule.  False: keep the classic plan.
bool build_streamk(const dx_attn* h, Plan& plan, const int32_t* host_past, int batch, SkSchedule& sk, int& ctas)
{
    const dx_attn_config& c = h->cfg;
    if (!h->streamk || !c.multi_block_mode || (plan.kind != KIND_GQA && plan.kind != KIND_TOK) || !host_past
        || batch > DX_SK_MAX_SEQ || !h->k_merge_sk || (h->cache_kind == CACHE_T && !h->streamk16))
        return false;
    // tokens per schedule unit: a token group of the mma.sync kernels, a tile of the token-major tcgen05 kernel
    const uint32_t unit = plan.kind == KIND_TOK ? 128 : h->cache_kind == CACHE_T ? 16 : 32;
    const uint32_t unit_log2 = unit == 128 ? 7 : unit == 32 ? 5 : 4;
    const uint32_t Y = (uint32_t) (c.num_kv_heads * plan.hgroups);
    uint64_t acc = 0;
    uint32_t nmax = 1;
    sk.prefix[0] = 0;
    for (int i = 0; i < batch; ++i)
    {
        const uint32_t n = ((uint32_t) host_past[i] + unit) >> unit_log2; // ceil((past + 1) / unit)
        nmax = std::max(nmax, n);
        acc += n;
        sk.prefix[i + 1] = (uint32_t) acc;
    }
    const uint64_t total = acc * Y;
    if (total >= (1ull << 31))
        return false;
    const uint64_t slots = (uint64_t) h->sm_count * plan.resident;
    const uint64_t U = (total + slots - 1) / slots;
    // Worth it when the ranges are long (see sk_min_units) and the rows are not many times longer than a range:
    // few very long rows are cut evenly by the classic partitions already.
    if (U * unit < (uint64_t) h->sk_min_units * 32 || acc > (uint64_t) h->sk_row_factor * U * (uint64_t) batch)
        return false;
    const uint64_t pmax = (nmax - 1) / U + 2; // pieces of the longest row, at most
    const size_t qrows = (size_t) batch * c.num_heads;
    sk.units_per_cta = (uint32_t) U;
    sk.total_units = (uint32_t) total;
    sk.rows_per_seq = Y;
    sk.nseq = (uint32_t) batch;
    ctas = (int) ((total + U - 1) / U);
    sk.n1 = (uint32_t) ctas;
    sk.n2 = 0;
    sk.u2 = 0;
    plan.nsplit = (int) pmax;
    plan.chunk_tokens = (int) (U * unit);
    plan.part_o_bytes = align_up(qrows * pmax * c.head_size * sizeof(float), 128);
    plan.part_ml_bytes = align_up(qrows * pmax * sizeof(float2), 128);
    return true;
}

// Two-level schedule of the persistent tcgen05 kernel: one CTA per SM; the first (100 - tail) per cent of the tiles in
// equal static ranges, the rest in short ranges the CTAs draw from a device counter as they finish.  On success
// the plan is that of the persistent kernel.  False: the call stays with the other kernels.
bool build_streamk_ws(const dx_attn* h, Plan& plan, const int32_t* host_past, int batch, SkSchedule& sk, int& ctas)
{
    const dx_attn_config& c = h->cfg;
    if (!h->tokws || !c.multi_block_mode || !host_past || batch > DX_SK_MAX_SEQ || !h->k_merge_sk)
        return false;
    const uint32_t Y = (uint32_t) c.num_kv_heads;
    uint64_t acc = 0;
    uint32_t nmax = 1;
    sk.prefix[0] = 0;
    for (int i = 0; i < batch; ++i)
    {
        const uint32_t n = ((uint32_t) host_past[i] + 128) >> 7; // ceil((past + 1) / 128)
        nmax = std::max(nmax, n);
        acc += n;
        sk.prefix[i + 1] = (uint32_t) acc;
    }
    const uint64_t total = acc * Y;
    if (total >= (1ull << 31))
        return false;
    const uint64_t n1 = std::min<uint64_t>((uint64_t) h->sm_count * (uint64_t) std::max(1, h->k_tokws.resident), total);
    uint64_t u1 = total * (uint64_t) (100 - h->ws_tail_pct) / 100 / n1, u2 = 0, n2 = 0;
    if (h->ws_tail_pct <= 0 || u1 < (uint64_t) h->ws_min_u1)
    {
        u1 = (total + n1 - 1) / n1; // single level
    }
    else
    {
        u2 = std::max<uint64_t>((uint64_t) h->ws_min_u2, u1 / (uint64_t) std::max(1, h->ws_tail_div));
        n2 = (total - n1 * u1 + u2 - 1) / u2;
    }
    const uint64_t umin = n2 ? std::min(u1, u2) : u1;
    const uint64_t pmax = (nmax - 1) / umin + 2; // pieces of the longest row, at most
    const size_t qrows = (size_t) batch * c.num_heads;
    sk.units_per_cta = (uint32_t) u1;
    sk.total_units = (uint32_t) total;
    sk.rows_per_seq = Y;
    sk.nseq = (uint32_t) batch;
    sk.n1 = (uint32_t) n1;
    sk.n2 = (uint32_t) n2;
    sk.u2 = (uint32_t) u2;
    ctas = (int) n1;
    plan.kind = KIND_TOKWS;
    plan.hgroups = 1;
    plan.heads16 = false;
    plan.six = false;
    plan.resident = std::max(1, h->k_tokws.resident);
    plan.rows = batch * c.num_kv_heads;
    plan.nsplit = (int) pmax;
    plan.chunk_tokens = (int) (u1 * 128);
    plan.part_o_bytes = align_up(qrows * pmax * c.head_size * sizeof(float), 128);
    plan.part_ml_bytes = align_up(qrows * pmax * sizeof(float2), 128);
    return true;
}

// build_streamk for the kernel form stream-K launches use: the six-warp CTAs where they exist (two per SM, which
// changes the number of ranges), else the kernel of the plan.
bool plan_streamk(const dx_attn* h, Plan& plan, const int32_t* host_past, int batch, SkSchedule& sk, int& ctas)
{
    const Plan shape = plan;
    plan.six = plan.kind == KIND_GQA && !plan.heads16 && h->k_gqa_six.fn != nullptr;
    if (plan.six)
    {
        // pays when the ranges are long (c4: 10.6 K tokens per CTA, 140.5 against 142.2 us; its TP2 shard 78.2 / 78.7);
        // the TP4 shard (2.7 K tokens) is 1 % slower with it
        plan.resident = h->k_gqa_six.resident;
        if (build_streamk(h, plan, host_past, batch, sk, ctas) && plan.chunk_tokens >= h->six_min_tokens)
            return true;
        plan = shape;
    }
    return build_streamk(h, plan, host_past, batch, sk, ctas);
}

// Upper bound of Plan::workspace() over every length vector with lengths <= max_past_len.
size_t workspace_bound(const dx_attn* h, int batch, int max_past_len)
{
    const dx_attn_config& c = h->cfg;
    if (!c.multi_block_mode)
        return 0;
    const Plan shape = make_plan(h, batch, max_past_len); // for kind / rows only
    const long rows_per_seq = std::max(1, shape.rows / std::max(1, batch));
    const long resident = 3;
    const long max_total = (long) max_past_len + 1;
    const long t_min = std::max<long>(128, h->min_chunk);
    long nsplit = std::min(parts_of(max_total, t_min), std::max<long>(1, h->waves * h->sm_count * resident / rows_per_seq));
    nsplit = std::max<long>(nsplit, shape.nsplit);
    const bool sk_kind = shape.kind == KIND_GQA || shape.kind == KIND_TOK;
    if (nsplit <= 1 && !sk_kind)
        return 0;
    if (sk_kind)
        nsplit += 2; // stream-K launches: a row of n groups cut by ranges of U groups has at most n / U + 2 pieces
    const size_t qrows = (size_t) batch * c.num_heads;
    return align_up(qrows * nsplit * c.head_size * sizeof(float), 128) + align_up(qrows * nsplit * sizeof(float2), 128);
}

// Bytes of the pre-processed QKV copy at the start of the workspace (0 when nothing is configured).
size_t prep_bytes(const dx_attn* h, int batch)
{
    if (!h->prep)
        return 0;
    const dx_attn_config& c = h->cfg;
    return align_up((size_t) batch * (c.num_heads + 2 * c.num_kv_heads) * c.head_size * 2, 128);
}

int check_cuda(dx_attn* h, cudaError_t e)
{
    if (e == cudaSuccess)
        return DX_OK;
    h->last_cuda_error = (int) e;
    return DX_ERR_CUDA;
}

int set_smem(dx_attn* h, const KernelInfo& k)
{
    if (!k.fn)
        return DX_OK;
    if (k.smem > h->max_smem_optin)
        return DX_ERR_UNSUPPORTED;
    return check_cuda(h, cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem));
}

template <typename T, int DH>
const void* merge_fn()
{
    return reinterpret_cast<const void*>(&lse_merge_kernel<T, DH>);
}

template <typename T, int DH>
const void* merge_many_fn()
{
    return reinterpret_cast<const void*>(&lse_merge_many_kernel<T, DH>);
}

const void* merge_many_kernel(int dtype, int dh)
{
    if (dh == 64)
        return dtype == 0 ? merge_many_fn<__half, 64>() : merge_many_fn<__nv_bfloat16, 64>();
    if (dh == 128)
        return dtype == 0 ? merge_many_fn<__half, 128>() : merge_many_fn<__nv_bfloat16, 128>();
    if (dh == 256)
        return dtype == 0 ? merge_many_fn<__half, 256>() : merge_many_fn<__nv_bfloat16, 256>();
    return nullptr;
}

template <typename T, int DH>
const void* merge_sk_fn()
{
    return reinterpret_cast<const void*>(&lse_merge_sk_kernel<T, DH>);
}

const void* merge_sk_kernel(int dtype, int dh)
{
    if (dh == 64)
        return dtype == 0 ? merge_sk_fn<__half, 64>() : merge_sk_fn<__nv_bfloat16, 64>();
    if (dh == 128)
        return dtype == 0 ? merge_sk_fn<__half, 128>() : merge_sk_fn<__nv_bfloat16, 128>();
    return nullptr;
}

} // namespace

namespace dx
{
KernelInfo merge_kernel_info(int dtype, int dh)
{
    KernelInfo k;
    if (dh == 64)
        k.fn = dtype == 0 ? merge_fn<__half, 64>() : merge_fn<__nv_bfloat16, 64>();
    else if (dh == 128)
        k.fn = dtype == 0 ? merge_fn<__half, 128>() : merge_fn<__nv_bfloat16, 128>();
    else if (dh == 256)
        k.fn = dtype == 0 ? merge_fn<__half, 256>() : merge_fn<__nv_bfloat16, 256>();
    return k;
}
} // namespace dx

// ---------------------------------------------------------------------------------------------
// Fixed split-K scratch for dx_attn_enqueue_generation_static_scratch: lives in the library's
// device image, so every GPU that loads the library holds DX_STATIC_SCRATCH_BYTES of it until the
// process exits.  In host code the name below is only a stand-in for the symbol, not an address a
// kernel could use; the device address is asked for once per device with cudaGetSymbolAddress.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[DX_STATIC_SCRATCH_BYTES];

namespace
{
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of g_static_scratch on `device`, which must be the current device.
int static_scratch_address(dx_attn* h, int device, void** out)
{
    if (device < 0 || device >= kMaxDevices)
        return DX_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[device])
    {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
        {
            h->last_cuda_error = (int) e;
            return DX_ERR_CUDA;
        }
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return DX_OK;
}
} // namespace

namespace
{

// Launches the optional bias / rotary pre-processing of the new token into the start of the workspace.
int launch_prep(dx_attn* h, const dx_attn_generation_params& p, int nseq, cudaStream_t stream)
{
    const dx_attn_config& c = h->cfg;
    PrepArgs pa{};
    pa.qkv = p.attention_input;
    pa.bias = p.qkv_bias;
    pa.out = p.workspace;
    pa.seq_len = p.sequence_lengths;
    pa.q_len = std::max(1, p.input_seq_length);
    pa.pos_offsets = pa.q_len > 1 ? p.medusa_position_offsets : nullptr;
    pa.batch = nseq;
    pa.num_heads = c.num_heads;
    pa.num_kv_heads = c.num_kv_heads;
    pa.head_size = c.head_size;
    pa.pos_type = c.position_embedding_type <= POS_ROPE_GPT_NEOX ? c.position_embedding_type : POS_LEARNED_ABSOLUTE;
    pa.rot_dim = c.rotary_embedding_dim;
    pa.rot_scale_type = c.rotary_embedding_scale_type;
    pa.rot_max_positions = c.rotary_embedding_max_positions;
    pa.rot_base = c.rotary_embedding_base;
    pa.rot_scale = c.rotary_embedding_scale;
    const long pairs = (long) nseq * (c.num_heads + 2 * c.num_kv_heads) * (c.head_size / 2);
    void* pargs[] = {&pa};
    const void* fn = c.type_id == DX_DTYPE_FP16 ? reinterpret_cast<const void*>(&qkv_bias_rope_kernel<__half>)
                                                : reinterpret_cast<const void*>(&qkv_bias_rope_kernel<__nv_bfloat16>);
    const int st = check_cuda(h, cudaLaunchKernel(fn, dim3((unsigned) ((pairs + 255) / 256)), dim3(256), pargs, 0, stream));
    if (st == DX_OK)
        h->launches.fetch_add(1);
    return st;
}

// Cyclic-cache geometry of a generation step (KVBlockArray, kvCacheUtils.h:74-90) and the checks both feature paths
// share.  A table with a spare block keeps W + tokens_per_block slots cycling.  Returns DX_OK and the period of the
// non-sink part of the cache, or the status to refuse the call with.
int window_geometry(const dx_attn* h, const dx_attn_generation_params& p, int max_past, int& cyclic_len)
{
    const int tpb = h->cfg.tokens_per_block;
    const int W = p.cyclic_attention_window_size, sink = p.sink_token_length;
    if (p.max_attention_window < W || sink >= W)
        return DX_ERR_BAD_ARG;
    if (sink % tpb != 0)
        return DX_ERR_UNSUPPORTED; // a partly filled sink block needs the reference's position shift
    const bool one_more_block = (int64_t) (p.max_blocks_per_sequence - 1) * tpb >= W;
    cyclic_len = one_more_block ? W + tpb - sink : W - sink;
    if (max_past > W && one_more_block)
        return DX_ERR_UNSUPPORTED; // the walked slots 0..W-1 are the live window only without the spare block
    const int64_t slots_used = std::min<int64_t>((int64_t) max_past + 1, (int64_t) sink + cyclic_len);
    if (slots_used > (int64_t) p.max_blocks_per_sequence * tpb)
        return DX_ERR_BAD_ARG; // the table cannot hold that many tokens
    return DX_OK;
}

// Launches an attention kernel, optionally as a programmatic dependent of the kernel in front of it on the stream
// (in a decode loop the previous step's merge or attention kernel): its CTAs become resident while that kernel
// drains and wait at their top (griddepcontrol.wait) before they touch global memory.
int launch_attention(dx_attn* h, const void* fn, dim3 grid, dim3 block, size_t smem, void** args, bool dependent,
    cudaStream_t stream)
{
    if (!dependent || h->no_dependent_launch)
        return check_cuda(h, cudaLaunchKernel(fn, grid, block, args, smem, stream));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(h, cudaLaunchKernelExC(&cfg, fn, args));
}

// The split-K merge behind an attention launch, as a programmatic dependent: the merge grid is scheduled while the
// attention grid drains and blocks in griddepcontrol.wait until that grid has completed (hides the launch gap).
// rows: output rows (sequences x new tokens x q heads).  Stream-K launches pass their schedule.
int launch_merge(dx_attn* h, AttnArgs& a, size_t rows, int hgroups, const SkSchedule* sk, cudaStream_t stream)
{
    void* args[] = {&a, &hgroups, const_cast<SkSchedule*>(sk)}; // (the classic merge kernel takes the first)
    // many partitions per row: a CTA per row (its four warps share the partitions) instead of a warp per row
    const bool many = !sk && h->k_merge_many && h->merge_many_from > 0 && a.nsplit >= h->merge_many_from;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = many ? dim3((unsigned) rows) : dim3((unsigned) ((rows + 3) / 4));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int st = check_cuda(h, cudaLaunchKernelExC(&cfg, many ? h->k_merge_many : (sk ? h->k_merge_sk : h->k_merge.fn), args));
    if (st == DX_OK)
        h->launches.fetch_add(1);
    return st;
}

// Beam search / cyclic window / sink tokens / ALiBi: one CTA per (sequence, q head) reads the cache as it is,
// then a second kernel appends the new token at its (cyclic) slot.
int enqueue_general(dx_attn* h, const dx_attn_generation_params& p, int max_past, void* cuda_stream)
{
    const dx_attn_config& c = h->cfg;
    const int W = p.cyclic_attention_window_size, sink = p.sink_token_length;
    const int nseq = p.num_requests * p.beam_width; // the reference's batch_beam (gptAttentionCommon.cpp:1186)
    if (!h->k_general.attn)
        return DX_ERR_UNSUPPORTED;
    int cyclic_len = 0;
    if (const int gs = window_geometry(h, p, max_past, cyclic_len); gs != DX_OK)
        return gs;
    if (p.beam_width > 1)
    {
        if (!p.cache_indir || !p.context_lengths)
            return DX_ERR_BAD_ARG;
        if (((uintptr_t) p.cache_indir | (uintptr_t) p.context_lengths) & 3)
            return DX_ERR_BAD_ARG;
    }
    const size_t prep = prep_bytes(h, nseq);
    if (prep)
    {
        if (!p.workspace || ((uintptr_t) p.workspace & 127))
            return p.workspace ? DX_ERR_BAD_ARG : DX_ERR_WORKSPACE;
        if (p.workspace_bytes < prep)
            return DX_ERR_WORKSPACE;
    }
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st == DX_OK && prep)
        st = launch_prep(h, p, nseq, stream);
    if (st != DX_OK)
        return st;

    GeneralArgs g{};
    g.qkv = prep ? p.workspace : p.attention_input;
    g.out = p.context_buf;
    g.seq_len = p.sequence_lengths;
    g.block_ptrs = p.block_pointers;
    g.scale_orig_quant = p.kv_scale_orig_quant;
    g.scale_quant_orig = p.kv_scale_quant_orig;
    g.cache_indir = p.beam_width > 1 ? p.cache_indir : nullptr;
    g.context_lengths = p.context_lengths;
    const bool alibi_type = c.position_embedding_type == POS_ALIBI || c.position_embedding_type == POS_ALIBI_WITH_SCALE;
    g.alibi_slopes = alibi_type ? p.alibi_slopes : nullptr;
    if (c.position_embedding_type == POS_RELATIVE && p.relative_attention_bias)
    {
        g.rel_bias = p.relative_attention_bias;
        g.rel_stride = p.relative_attention_bias_stride;
        g.max_distance = p.max_distance;
    }
    g.num_heads = c.num_heads;
    g.num_kv_heads = c.num_kv_heads;
    g.max_blocks_per_seq = p.max_blocks_per_sequence;
    g.tpb_log2 = h->tpb_log2;
    g.beam_width = p.beam_width;
    g.max_attention_window = p.max_attention_window;
    g.cyclic_window = W;
    g.cyclic_len = cyclic_len;
    g.sink = sink;
    g.softmax_scale_log2 = 1.4426950408889634f / (sqrtf((float) c.head_size) * c.q_scaling);
    g.status = h->status_dev;
    g.guard = h->guard;
    g.q_len = 1;
    void* args[] = {&g};
    st = check_cuda(h, cudaLaunchKernel(h->k_general.attn, dim3(c.num_heads, nseq), dim3(128), args,
                           (size_t) h->k_general.smem, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    st = check_cuda(h, cudaLaunchKernel(h->k_general.append, dim3(c.num_kv_heads, nseq), dim3(32), args, 0, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    return DX_OK;
}

// Beam search, cyclic window / sink tokens and ALiBi on grouped heads with an 8-bit cache: the feature form of the
// tensor-core grouped-head kernel (the q heads of a kv head share every cache read; beams of a request are
// sequences of their own whose shared context comes out of L2), classic split-K partitions, the usual merge.
int enqueue_feature_gqa(dx_attn* h, const dx_attn_generation_params& p, int max_past, void* cuda_stream)
{
    const dx_attn_config& c = h->cfg;
    const int nseq = p.num_requests * p.beam_width;
    if (p.beam_width > 1)
    {
        if (!p.cache_indir || !p.context_lengths)
            return DX_ERR_BAD_ARG;
        if (((uintptr_t) p.cache_indir | (uintptr_t) p.context_lengths) & 3)
            return DX_ERR_BAD_ARG;
    }
    const int W = p.cyclic_attention_window_size, sink = p.sink_token_length;
    int cyclic_len = 0;
    if (const int gs = window_geometry(h, p, max_past, cyclic_len); gs != DX_OK)
        return gs;
    const bool wrapped = max_past > W; // some sequence walks W slots instead of its whole history
    Plan plan;
    plan.kind = KIND_GQA;
    plan.hgroups = (h->group + 15) / 16;
    plan.heads16 = h->group > 8;
    const int rows_per_seq = c.num_kv_heads * plan.hgroups;
    plan.rows = nseq * rows_per_seq;
    plan.resident = std::max(1, h->k_gqa_feat[plan.heads16 ? 1 : 0].resident);
    // (with a wrapped window the partitions are planned for W walked slots per sequence, an upper bound)
    plan_partitions(h, plan, nseq, rows_per_seq, wrapped ? W : max_past, wrapped ? nullptr : p.host_past_key_value_lengths);
    const size_t prep = prep_bytes(h, nseq);
    if (plan.nsplit > 1 || prep)
    {
        if (!p.workspace || ((uintptr_t) p.workspace & 127))
            return p.workspace ? DX_ERR_BAD_ARG : DX_ERR_WORKSPACE;
        if (p.workspace_bytes < prep + plan.workspace())
            return DX_ERR_WORKSPACE;
    }
    char* const ws_partials = reinterpret_cast<char*>(p.workspace) + prep;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st == DX_OK && prep)
        st = launch_prep(h, p, nseq, stream);
    if (st != DX_OK)
        return st;

    AttnArgs a{};
    a.qkv = prep ? p.workspace : p.attention_input;
    a.out = p.context_buf;
    a.seq_len = p.sequence_lengths;
    a.block_ptrs = p.block_pointers;
    a.scale_orig_quant = p.kv_scale_orig_quant;
    a.scale_quant_orig = p.kv_scale_quant_orig;
    a.part_o = plan.nsplit > 1 ? reinterpret_cast<float*>(ws_partials) : nullptr;
    a.part_ml = plan.nsplit > 1 ? reinterpret_cast<float2*>(ws_partials + plan.part_o_bytes) : nullptr;
    a.status = h->status_dev;
    a.batch = nseq;
    a.num_heads = c.num_heads;
    a.num_kv_heads = c.num_kv_heads;
    a.max_blocks_per_seq = p.max_blocks_per_sequence;
    a.tpb_log2 = h->tpb_log2;
    a.chunk_tokens = plan.chunk_tokens;
    a.nsplit = plan.nsplit;
    a.softmax_scale_log2 = 1.4426950408889634f / (sqrtf((float) c.head_size) * c.q_scaling);
    a.guard = h->guard;
    a.cache_indir = p.beam_width > 1 ? p.cache_indir : nullptr;
    a.context_lengths = p.context_lengths;
    const bool alibi_type = c.position_embedding_type == POS_ALIBI || c.position_embedding_type == POS_ALIBI_WITH_SCALE;
    a.alibi_slopes = alibi_type ? p.alibi_slopes : nullptr;
    a.beam_width = p.beam_width;
    a.max_attention_window = p.max_attention_window;
    a.cyclic_window = W;

    const KernelInfo& k = h->k_gqa_feat[plan.heads16 ? 1 : 0];
    int hgroups = plan.hgroups;
    void* args[] = {&a, &hgroups, &h->sk_zero};
    st = check_cuda(h, cudaLaunchKernel(k.fn, dim3(plan.nsplit, c.num_kv_heads * plan.hgroups, nseq), dim3(k.threads), args,
                           (size_t) k.smem, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    if (plan.nsplit > 1)
    {
        st = launch_merge(h, a, (size_t) nseq * c.num_heads, hgroups, nullptr, stream);
        if (st != DX_OK)
            return st;
    }
    // the new token into its (cyclic) slot, behind every read of the old content of that slot
    GeneralArgs g{};
    g.qkv = a.qkv;
    g.seq_len = p.sequence_lengths;
    g.block_ptrs = p.block_pointers;
    g.scale_orig_quant = p.kv_scale_orig_quant;
    g.num_heads = c.num_heads;
    g.num_kv_heads = c.num_kv_heads;
    g.max_blocks_per_seq = p.max_blocks_per_sequence;
    g.tpb_log2 = h->tpb_log2;
    g.cyclic_len = cyclic_len;
    g.sink = sink;
    g.q_len = 1;
    g.status = h->status_dev;
    g.guard = h->guard;
    void* gargs[] = {&g};
    st = check_cuda(h, cudaLaunchKernel(h->k_general.append, dim3(c.num_kv_heads, nseq), dim3(32), gargs, 0, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    return DX_OK;
}

// Several new tokens per sequence (the reference's Medusa mode): append all of them, then one CTA per
// (token, q head) reads the cache under the token's mask row.
int enqueue_multi_token(dx_attn* h, const dx_attn_generation_params& p, int max_past, void* cuda_stream)
{
    const dx_attn_config& c = h->cfg;
    const int Q = p.input_seq_length;
    if (!h->k_general.multi)
        return DX_ERR_UNSUPPORTED;
    if (Q > 4096 || !p.medusa_packed_mask || ((uintptr_t) p.medusa_packed_mask & 3)
        || ((uintptr_t) p.medusa_position_offsets & 3))
        return DX_ERR_BAD_ARG;
    // the reference runs this mode on its XQA kernels only: beam width 1, no sliding window, no sink tokens
    // (decoderXQARunner.h:87-159), and asserts when they do not apply (gptAttentionCommon.cpp:1225-1228)
    const int64_t need = (int64_t) max_past + Q;
    if (p.beam_width != 1 || p.sink_token_length > 0 || c.position_embedding_type >= POS_ALIBI // (ALiBi, relative)
        || p.cyclic_attention_window_size < need || p.max_attention_window < need)
        return DX_ERR_UNSUPPORTED;
    if (c.position_embedding_type != POS_LEARNED_ABSOLUTE && c.rotary_embedding_scale_type == ROT_SCALE_DYNAMIC)
        return DX_ERR_UNSUPPORTED; // (the reference's multi-token pre-processing rescales the base at every length)
    if (need > (int64_t) p.max_blocks_per_sequence * c.tokens_per_block)
        return DX_ERR_BAD_ARG; // the table cannot hold that many tokens
    const int64_t rows64 = (int64_t) p.num_requests * Q;
    if (rows64 > 65535)
        return DX_ERR_UNSUPPORTED; // grid.y
    const int rows = (int) rows64;
    const size_t prep = prep_bytes(h, rows);
    if (prep)
    {
        if (!p.workspace || ((uintptr_t) p.workspace & 127))
            return p.workspace ? DX_ERR_BAD_ARG : DX_ERR_WORKSPACE;
        if (p.workspace_bytes < prep)
            return DX_ERR_WORKSPACE;
    }
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st == DX_OK && prep)
        st = launch_prep(h, p, rows, stream);
    if (st != DX_OK)
        return st;

    GeneralArgs g{};
    g.qkv = prep ? p.workspace : p.attention_input;
    g.out = p.context_buf;
    g.seq_len = p.sequence_lengths;
    g.block_ptrs = p.block_pointers;
    g.scale_orig_quant = p.kv_scale_orig_quant;
    g.scale_quant_orig = p.kv_scale_quant_orig;
    g.num_heads = c.num_heads;
    g.num_kv_heads = c.num_kv_heads;
    g.max_blocks_per_seq = p.max_blocks_per_sequence;
    g.tpb_log2 = h->tpb_log2;
    g.beam_width = 1;
    g.max_attention_window = p.max_attention_window;
    g.cyclic_window = p.cyclic_attention_window_size;
    g.cyclic_len = p.max_blocks_per_sequence * c.tokens_per_block; // no wrap: slot = token index
    g.sink = 0;
    g.softmax_scale_log2 = 1.4426950408889634f / (sqrtf((float) c.head_size) * c.q_scaling);
    g.status = h->status_dev;
    g.guard = h->guard;
    g.q_len = Q;
    g.packed_mask = p.medusa_packed_mask;
    void* args[] = {&g};
    st = check_cuda(h, cudaLaunchKernel(h->k_general.append, dim3(c.num_kv_heads, rows), dim3(32), args, 0, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    // Grouped heads over an 8-bit cache, up to 64 new tokens: the (token, head) rows of a kv head share one pass
    // over the cache on the tensor-core grouped-head kernel, 16 rows per CTA, split-K and merge as on the plain
    // path.  Needs room for the partials behind the bias / rotary copy; without it the per-row kernel below runs.
    const int QG = Q * h->group;
    const KernelInfo& km = h->k_gqa_multi[QG > 8 ? 1 : 0];
    if (h->feature_gqa && !h->general_only && h->group > 1 && Q <= 64
        && c.tokens_per_block >= (h->cache_kind == CACHE_T ? 16 : 32) && km.fn)
    {
        Plan plan;
        plan.kind = KIND_GQA;
        plan.hgroups = (QG + 15) / 16;
        plan.heads16 = QG > 8;
        const int rows_per_seq = c.num_kv_heads * plan.hgroups;
        plan.rows = p.num_requests * rows_per_seq;
        plan.resident = std::max(1, km.resident);
        plan_partitions(h, plan, p.num_requests, rows_per_seq, (int) need - 1, nullptr);
        const size_t qrows = (size_t) rows * c.num_heads;
        plan.part_o_bytes = plan.nsplit > 1 ? align_up(qrows * plan.nsplit * c.head_size * sizeof(float), 128) : 0;
        plan.part_ml_bytes = plan.nsplit > 1 ? align_up(qrows * plan.nsplit * sizeof(float2), 128) : 0;
        const bool room = plan.nsplit == 1
            || (p.workspace && !((uintptr_t) p.workspace & 127) && p.workspace_bytes >= prep + plan.workspace());
        if (room && (int64_t) c.num_kv_heads * plan.hgroups <= 65535)
        {
            char* const ws_partials = reinterpret_cast<char*>(p.workspace) + prep;
            AttnArgs a{};
            a.qkv = g.qkv;
            a.out = p.context_buf;
            a.seq_len = p.sequence_lengths;
            a.block_ptrs = p.block_pointers;
            a.scale_orig_quant = p.kv_scale_orig_quant;
            a.scale_quant_orig = p.kv_scale_quant_orig;
            a.part_o = plan.nsplit > 1 ? reinterpret_cast<float*>(ws_partials) : nullptr;
            a.part_ml = plan.nsplit > 1 ? reinterpret_cast<float2*>(ws_partials + plan.part_o_bytes) : nullptr;
            a.status = h->status_dev;
            a.batch = p.num_requests;
            a.num_heads = c.num_heads;
            a.num_kv_heads = c.num_kv_heads;
            a.max_blocks_per_seq = p.max_blocks_per_sequence;
            a.tpb_log2 = h->tpb_log2;
            a.chunk_tokens = plan.chunk_tokens;
            a.nsplit = plan.nsplit;
            a.softmax_scale_log2 = g.softmax_scale_log2;
            a.guard = h->guard;
            a.q_len = Q;
            a.packed_mask = p.medusa_packed_mask;
            int hgroups = plan.hgroups;
            void* kargs[] = {&a, &hgroups, &h->sk_zero};
            st = check_cuda(h, cudaLaunchKernel(km.fn, dim3(plan.nsplit, c.num_kv_heads * plan.hgroups, p.num_requests),
                                   dim3(km.threads), kargs, (size_t) km.smem, stream));
            if (st != DX_OK)
                return st;
            h->launches.fetch_add(1);
            if (plan.nsplit > 1)
            {
                st = launch_merge(h, a, qrows, hgroups, nullptr, stream);
                if (st != DX_OK)
                    return st;
            }
            return DX_OK;
        }
    }
    st = check_cuda(h, cudaLaunchKernel(h->k_general.multi, dim3(c.num_heads, rows), dim3(128), args,
                           (size_t) h->k_general.smem, stream));
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);
    return DX_OK;
}

} // namespace

extern "C" {

int dx_abi_version(void)
{
    return DX_ABI_VERSION;
}

const char* dx_strerror(int status)
{
    switch (status)
    {
    case DX_OK: return "ok";
    case DX_ERR_BAD_ARG: return "bad argument";
    case DX_ERR_UNSUPPORTED: return "unsupported configuration";
    case DX_ERR_WORKSPACE: return "workspace too small";
    case DX_ERR_CUDA: return "CUDA runtime error";
    case DX_ERR_TIMEOUT: return "device-side wait timed out";
    case DX_ERR_BOUNDS: return "block pointer or length out of bounds";
    default: return "unknown status";
    }
}

int dx_attn_create(const dx_attn_config* config, dx_attn_t** out)
{
    if (!config || !out)
        return DX_ERR_BAD_ARG;
    *out = nullptr;
    if (config->struct_size != sizeof(dx_attn_config) && config->struct_size != DX_ATTN_CONFIG_SIZE_V1)
        return DX_ERR_BAD_ARG;
    dx_attn_config full;
    memset(&full, 0, sizeof(full));
    memcpy(&full, config, config->struct_size);
    full.struct_size = sizeof(dx_attn_config);
    const dx_attn_config& c = full;
    if (c.position_embedding_type < 0 || c.position_embedding_type > POS_RELATIVE)
        return DX_ERR_UNSUPPORTED; // relative position bias is not implemented
    if (c.position_embedding_type == POS_ROPE_GPTJ || c.position_embedding_type == POS_ROPE_GPT_NEOX)
    {
        if (c.rotary_embedding_dim <= 0 || (c.rotary_embedding_dim & 3) || c.rotary_embedding_dim > c.head_size
            || !(c.rotary_embedding_base > 0.f) || c.rotary_embedding_scale_type < ROT_SCALE_NONE
            || c.rotary_embedding_scale_type > ROT_SCALE_DYNAMIC)
            return DX_ERR_BAD_ARG;
        if (c.rotary_embedding_scale_type != ROT_SCALE_NONE && !(c.rotary_embedding_scale > 0.f))
            return DX_ERR_BAD_ARG;
        if (c.rotary_embedding_scale_type == ROT_SCALE_DYNAMIC && c.rotary_embedding_max_positions <= 0)
            return DX_ERR_BAD_ARG;
    }
    if (c.num_heads <= 0 || c.num_kv_heads <= 0 || c.num_heads % c.num_kv_heads != 0)
        return DX_ERR_BAD_ARG;
    if (!(c.q_scaling > 0.f) || c.tokens_per_block <= 0 || (c.tokens_per_block & (c.tokens_per_block - 1)))
        return DX_ERR_BAD_ARG;
    // Head sizes of the reference's MMHA switch (decoderMaskedMultiheadAttention.cu:68-85).  64 and 128 run on the
    // streaming kernels; the others on the feature-complete kernels (one CTA per sequence and q head).
    // (256: the per-head streaming kernel only; grouped heads then run one CTA per q head)
    const bool streaming_dh = c.head_size == 64 || c.head_size == 128 || c.head_size == 256;
    {
        static const int sizes[] = {32, 48, 64, 80, 96, 104, 112, 128, 144, 160, 192, 224, 256};
        bool known = false;
        for (int v : sizes)
            known |= v == c.head_size;
        if (!known)
            return DX_ERR_UNSUPPORTED;
    }
    if (c.type_id != DX_DTYPE_FP16 && c.type_id != DX_DTYPE_BF16)
        return DX_ERR_UNSUPPORTED;
    if (!c.paged_kv_cache || c.tokens_per_block < 16 || c.tokens_per_block > 256)
        return DX_ERR_UNSUPPORTED;
    const int q = c.kv_cache_quant_mode & (DX_QUANT_INT8_KV_CACHE | DX_QUANT_FP8_KV_CACHE);
    if (q == (DX_QUANT_INT8_KV_CACHE | DX_QUANT_FP8_KV_CACHE))
        return DX_ERR_BAD_ARG;
    if ((c.head_size * (q ? 1 : 2)) % 16 != 0)
        return DX_ERR_UNSUPPORTED; // cache rows are moved in 16-byte pieces (head size 104 needs a 16-bit cache)

    dx_attn* h = new (std::nothrow) dx_attn;
    if (!h)
        return DX_ERR_BAD_ARG;
    h->cfg = c;
    h->prep = c.position_embedding_type == POS_ROPE_GPTJ || c.position_embedding_type == POS_ROPE_GPT_NEOX
        || c.qkv_bias_enabled != 0;
    h->cache_kind = q == DX_QUANT_INT8_KV_CACHE ? CACHE_INT8 : (q == DX_QUANT_FP8_KV_CACHE ? CACHE_FP8 : CACHE_T);
    h->group = c.num_heads / c.num_kv_heads;
    while ((1 << h->tpb_log2) < c.tokens_per_block)
        ++h->tpb_log2;
    if (const char* w = getenv("DX_ATTN_PDL_OTHER"))
        h->pdl_other = atoi(w) != 0 ? 1 : 0;
    if (const char* w = getenv("DX_ATTN_PDL_ATTENTION"))
        h->pdl_attention = atoi(w) != 0 ? 1 : 0;
    if (const char* w = getenv("DX_ATTN_WAVES"))
        h->waves = std::max(1, atoi(w));
    if (const char* w = getenv("DX_ATTN_MIN_CHUNK"))
        h->min_chunk = std::max(128, atoi(w));
    if (const char* w = getenv("DX_ATTN_FIXED_COST"))
        h->fixed_cost_tokens = std::max(0, atoi(w));
    if (const char* w = getenv("DX_ATTN_FORCE_CHUNK"))
        h->force_chunk = atoi(w);
    if (const char* w = getenv("DX_ATTN_WAVE_SLACK_FROM"))
        h->wave_slack_from = atof(w);
    if (const char* w = getenv("DX_ATTN_STREAMK"))
        h->streamk = atoi(w) != 0;
    if (const char* w = getenv("DX_ATTN_SK_MIN_UNITS"))
        h->sk_min_units = std::max(1, atoi(w));
    if (const char* w = getenv("DX_ATTN_STREAMK_16BIT"))
        h->streamk16 = atoi(w) != 0;
    if (const char* w = getenv("DX_ATTN_SK_ROW_FACTOR"))
        h->sk_row_factor = std::max(1, atoi(w));

    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st == DX_OK)
        st = check_cuda(h, cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, c.device));
    if (st == DX_OK)
        st = check_cuda(
            h, cudaDeviceGetAttribute(&h->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, c.device));
    if (st == DX_OK)
    {
        h->k_mha = mha_kernel_info(c.type_id, h->cache_kind, c.head_size, c.tokens_per_block);
        h->k_merge = merge_kernel_info(c.type_id, c.head_size);
        h->k_merge_sk = merge_sk_kernel(c.type_id, c.head_size);
        h->k_merge_many = merge_many_kernel(c.type_id, c.head_size);
        if (const char* w = getenv("DX_ATTN_MERGE_MANY_FROM"))
            h->merge_many_from = std::max(0, atoi(w));
        h->k_append = append_kernel_info(c.type_id, h->cache_kind, c.head_size);
        h->k_general = general_kernel_info(c.type_id, h->cache_kind, c.head_size);
        const char* g16 = getenv("DX_ATTN_GQA16"); // "0": grouped heads over a 16-bit cache stay on the per-head kernel
        if (h->cache_kind != CACHE_T || !g16 || atoi(g16) != 0)
        {
            for (int h16 = 0; h16 < 2; ++h16)
                h->k_gqa[h16] = gqa_kernel_info(c.type_id, h->cache_kind, c.head_size, h16 != 0);
        }
        if (!streaming_dh)
        {
            // (a cache row that is not a multiple of 16 bytes - head size 104 in an 8-bit cache - has no kernel)
            if (!h->k_general.attn)
                st = DX_ERR_UNSUPPORTED;
            h->k_append.fn = h->k_general.context_append;
            h->general_only = true;
        }
        else if (!h->k_mha.fn || !h->k_merge.fn)
            st = DX_ERR_UNSUPPORTED;
        if (!h->k_append.fn)
            h->k_append.fn = h->k_general.context_append; // (head size 256)
    }
    if (st == DX_OK)
        st = set_smem(h, h->k_mha);
    for (int i = 0; i < 2 && st == DX_OK; ++i)
        st = set_smem(h, h->k_gqa[i]);
    if (st == DX_OK && h->k_gqa[0].fn)
    {
        if (const char* w = getenv("DX_ATTN_FEATURE_GQA"))
            h->feature_gqa = atoi(w) != 0;
        for (int i = 0; i < 2 && h->feature_gqa; ++i)
        {
            h->k_gqa_feat[i] = gqa_feature_kernel_info(c.type_id, h->cache_kind, c.head_size, i != 0);
            if (!h->k_gqa_feat[i].fn || set_smem(h, h->k_gqa_feat[i]) != DX_OK)
                h->feature_gqa = false;
            h->k_gqa_multi[i] = gqa_multi_token_kernel_info(c.type_id, h->cache_kind, c.head_size, i != 0);
            if (h->k_gqa_multi[i].fn && set_smem(h, h->k_gqa_multi[i]) != DX_OK)
                h->k_gqa_multi[i] = KernelInfo{};
        }
    }
    else
        h->feature_gqa = false;
    if (st == DX_OK && h->k_gqa[0].fn)
    {
        const char* w = getenv("DX_ATTN_SK_SIX_WARPS"); // "0": stream-K launches stay on the four-warp CTAs
        if (const char* m = getenv("DX_ATTN_SK_SIX_MIN_TOKENS"))
            h->six_min_tokens = std::max(1, atoi(m));
        if (!w || atoi(w) != 0)
        {
            h->k_gqa_six = gqa_streamk_kernel_info(c.type_id, h->cache_kind, c.head_size, false);
            if (h->k_gqa_six.fn && set_smem(h, h->k_gqa_six) != DX_OK)
                h->k_gqa_six = KernelInfo{};
        }
    }
    if (st == DX_OK && h->cache_kind == CACHE_FP8 && h->group > 16 && c.tokens_per_block >= 64)
    {
        const char* w = getenv("DX_ATTN_WIDE"); // "0": keep such groups on the 16-head-slice kernel
        if (!w || atoi(w) != 0)
        {
            h->k_wide = wide_kernel_info(c.type_id, c.head_size);
            h->wide = h->k_wide.fn != nullptr && set_smem(h, h->k_wide) == DX_OK;
        }
    }
    if (st == DX_OK && h->cache_kind == CACHE_FP8 && h->group > 1 && h->group <= 16 && c.head_size == 128
        && c.tokens_per_block >= 32)
    {
        const char* w = getenv("DX_ATTN_TOK");
        if (w && atoi(w) != 0)
        {
            h->k_tok = tok_kernel_info(c.type_id, c.head_size, h->group);
            h->tok = h->k_tok.fn != nullptr && set_smem(h, h->k_tok) == DX_OK;
        }
    }
    if (st == DX_OK && h->cache_kind == CACHE_FP8 && h->group > 1 && h->group <= 16 && c.head_size == 128
        && c.tokens_per_block >= 32)
    {
        const char* w = getenv("DX_ATTN_TOKWS");
        if (w && atoi(w) != 0)
        {
            h->k_tokws = tokws_kernel_info(c.type_id, c.head_size, h->group);
            h->tokws = h->k_tokws.fn != nullptr && set_smem(h, h->k_tokws) == DX_OK;
        }
        if (const char* m = getenv("DX_ATTN_WS_TAIL_PCT"))
            h->ws_tail_pct = std::max(0, std::min(90, atoi(m)));
        if (const char* m = getenv("DX_ATTN_WS_TAIL_DIV"))
            h->ws_tail_div = std::max(1, atoi(m));
        if (const char* m = getenv("DX_ATTN_WS_MIN_U2"))
            h->ws_min_u2 = std::max(1, atoi(m));
        if (const char* m = getenv("DX_ATTN_WS_MIN_U1"))
            h->ws_min_u1 = std::max(1, atoi(m));
    }
    if (st == DX_OK)
        st = check_cuda(h, cudaMalloc(reinterpret_cast<void**>(&h->status_dev), 512));
    if (st == DX_OK)
        st = check_cuda(h, cudaMemset(h->status_dev, 0, 512));
#ifdef DECODE_ATTN_BOUNDS_CHECK
    if (st == DX_OK)
    {
        // the spare block that out-of-bounds accesses are redirected to: one cache block of zeros
        const size_t block_bytes = (size_t) c.num_kv_heads * c.tokens_per_block * c.head_size * (h->cache_kind == CACHE_T ? 2 : 1);
        void* spare = nullptr;
        st = check_cuda(h, cudaMalloc(&spare, block_bytes));
        if (st == DX_OK)
            st = check_cuda(h, cudaMemset(spare, 0, block_bytes));
        h->guard.safe_block = reinterpret_cast<int64_t>(spare);
    }
#endif
    if (st != DX_OK)
    {
        if (h->status_dev)
            cudaFree(h->status_dev);
        delete h;
        return st;
    }
    *out = h;
    return DX_OK;
}

void dx_attn_destroy(dx_attn_t* h)
{
    if (!h)
        return;
    cudaSetDevice(h->cfg.device);
    if (h->status_dev)
        cudaFree(h->status_dev);
    if (h->guard.safe_block)
        cudaFree(reinterpret_cast<void*>(h->guard.safe_block));
    if (h->stage_dev)
        cudaFree(h->stage_dev);
    for (int i = 0; i < dx_attn::HOST_SLOTS; ++i)
    {
        if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
        if (h->ev_done[i]) cudaEventDestroy(h->ev_done[i]);
        if (h->ev_out[i]) cudaEventDestroy(h->ev_out[i]);
    }
    if (h->h2d_stream) cudaStreamDestroy(h->h2d_stream);
    if (h->d2h_stream) cudaStreamDestroy(h->d2h_stream);
    delete h;
}

size_t dx_attn_workspace_size(const dx_attn_t* h, int32_t batch, int32_t max_past_len)
{
    if (!h || batch <= 0 || max_past_len < 0)
        return 0;
    return prep_bytes(h, batch) + (h->general_only ? 0 : workspace_bound(h, batch, max_past_len));
}

int dx_attn_plan(const dx_attn_t* h, int32_t batch, int32_t max_past_len, int32_t* num_partitions,
    int32_t* tokens_per_partition, int32_t* kernel_kind)
{
    if (!h || batch <= 0 || max_past_len < 0)
        return DX_ERR_BAD_ARG;
    if (h->general_only)
    {
        if (num_partitions)
            *num_partitions = 1;
        if (tokens_per_partition)
            *tokens_per_partition = max_past_len + 1;
        if (kernel_kind)
            *kernel_kind = KIND_GENERAL;
        return DX_OK;
    }
    const Plan p = make_plan(h, batch, max_past_len);
    if (num_partitions)
        *num_partitions = p.nsplit;
    if (tokens_per_partition)
        *tokens_per_partition = p.chunk_tokens;
    if (kernel_kind)
        *kernel_kind = p.kind;
    return DX_OK;
}

int dx_attn_plan_lengths(const dx_attn_t* h, const int32_t* host_past_key_value_lengths, int32_t batch,
    int32_t* num_partitions, int32_t* tokens_per_partition, int32_t* kernel_kind)
{
    if (!h || batch <= 0 || !host_past_key_value_lengths)
        return DX_ERR_BAD_ARG;
    int max_past = 0;
    for (int i = 0; i < batch; ++i)
    {
        if (host_past_key_value_lengths[i] < 0)
            return DX_ERR_BAD_ARG;
        max_past = std::max(max_past, host_past_key_value_lengths[i]);
    }
    if (h->general_only)
        return dx_attn_plan(h, batch, max_past, num_partitions, tokens_per_partition, kernel_kind);
    int rows_per_seq = 1;
    Plan p = plan_shape(h, batch, rows_per_seq);
    SkSchedule sk;
    int ctas = 0;
    bool streamk = build_streamk_ws(h, p, host_past_key_value_lengths, batch, sk, ctas);
    if (!streamk)
        streamk = plan_streamk(h, p, host_past_key_value_lengths, batch, sk, ctas);
    if (!streamk)
        plan_partitions(h, p, batch, rows_per_seq, max_past, host_past_key_value_lengths);
    if (num_partitions)
        *num_partitions = streamk ? -ctas : p.nsplit; // stream-K: minus the number of CTAs, each tokens_per_partition tokens
    if (tokens_per_partition)
        *tokens_per_partition = p.chunk_tokens;
    if (kernel_kind)
        *kernel_kind = p.kind;
    return DX_OK;
}

int dx_attn_enqueue_generation(dx_attn_t* h, const dx_attn_generation_params* params, void* cuda_stream)
{
    dx_attn_generation_params p;
    if (!h || !read_params(params, p))
        return DX_ERR_BAD_ARG;
    const dx_attn_config& c = h->cfg;
    if (p.num_requests < 0 || p.max_blocks_per_sequence <= 0)
        return DX_ERR_BAD_ARG;
    if (p.num_requests == 0)
        return DX_OK; // empty batch: nothing to do, nothing launched
    if (p.qkv_bias && (!c.qkv_bias_enabled || ((uintptr_t) p.qkv_bias & 1)))
        return DX_ERR_BAD_ARG; // a bias needs qkv_bias_enabled at create time (it sizes the workspace)
    if (!p.attention_input || !p.sequence_lengths || !p.block_pointers || !p.context_buf)
        return DX_ERR_BAD_ARG;
    if (((uintptr_t) p.attention_input | (uintptr_t) p.context_buf) & 15)
        return DX_ERR_BAD_ARG;
    if (((uintptr_t) p.block_pointers & 7) || ((uintptr_t) p.sequence_lengths & 3))
        return DX_ERR_BAD_ARG;
    if (h->cache_kind != CACHE_T && (!p.kv_scale_orig_quant || !p.kv_scale_quant_orig))
        return DX_ERR_BAD_ARG;
    if (p.beam_width < 1 || p.sink_token_length < 0 || p.cyclic_attention_window_size < 1)
        return DX_ERR_BAD_ARG;
    const bool alibi_type = c.position_embedding_type == POS_ALIBI || c.position_embedding_type == POS_ALIBI_WITH_SCALE;
    const bool alibi = alibi_type && p.alibi_slopes != nullptr;
    if (p.alibi_slopes != nullptr && !alibi_type)
        return DX_ERR_BAD_ARG; // slopes need an ALiBi position embedding type at create time
    const bool relative = c.position_embedding_type == POS_RELATIVE && p.relative_attention_bias != nullptr;
    if (p.relative_attention_bias != nullptr)
    {
        // a bias table needs the relative position embedding type at create time; the implicit form needs at
        // least four buckets (the bucket function divides by a quarter of their number)
        if (c.position_embedding_type != POS_RELATIVE || ((uintptr_t) p.relative_attention_bias & 1)
            || p.relative_attention_bias_stride <= 0 || p.max_distance < 0
            || (p.max_distance > 0 && (p.relative_attention_bias_stride < 4 || p.max_distance <= p.relative_attention_bias_stride / 4)))
            return DX_ERR_BAD_ARG;
    }

    int max_past = p.past_kv_length;
    if (p.host_past_key_value_lengths)
    {
        max_past = 0;
        for (int i = 0; i < p.num_requests * p.beam_width; ++i) // one entry per sequence (request x beam)
        {
            const int v = p.host_past_key_value_lengths[i];
            if (v < 0)
                return DX_ERR_BAD_ARG;
            max_past = std::max(max_past, v);
        }
    }
    if (max_past < 0)
        return DX_ERR_BAD_ARG;
    if (relative && p.max_distance == 0 && p.relative_attention_bias_stride < max_past + 1)
        return DX_ERR_BAD_ARG; // the explicit table must cover every position
    if (p.input_seq_length < 0 || p.reserved0 != 0)
        return DX_ERR_BAD_ARG;
    if (p.input_seq_length > 1)
        return enqueue_multi_token(h, p, max_past, cuda_stream);
    // Beam search, a window shorter than some sequence, sink tokens and ALiBi go to the feature-complete kernel.
    const bool general = h->general_only || p.beam_width > 1 || p.sink_token_length > 0 || alibi || relative
        || p.cyclic_attention_window_size < max_past + 1 || p.max_attention_window < max_past + 1;
    // beams / windows / sinks / ALiBi over grouped heads with an 8-bit cache share the cache reads of a kv head
    if (general && h->feature_gqa && !h->general_only && h->group > 1
        && c.tokens_per_block >= (h->cache_kind == CACHE_T ? 16 : 32) && !relative && h->k_general.append)
        return enqueue_feature_gqa(h, p, max_past, cuda_stream);
    if (general)
        return enqueue_general(h, p, max_past, cuda_stream);
    if ((int64_t) max_past + 1 > (int64_t) p.max_blocks_per_sequence * c.tokens_per_block)
        return DX_ERR_BAD_ARG; // the table cannot hold that many tokens

    int rows_per_seq = 1;
    Plan plan = plan_shape(h, p.num_requests, rows_per_seq);
    if (plan.kind == KIND_MHA && c.tokens_per_block < 16)
        return DX_ERR_UNSUPPORTED;
    const size_t prep = prep_bytes(h, p.num_requests);

    // Stream-K schedule for the 8-bit grouped-head kernel: equal ranges of 32-token groups per CTA, computed from
    // the host lengths.  Used when the workspace given can hold one partial result per piece of a cut row.
    SkSchedule sk;
    int sk_ctas = 0;
    const auto fits = [&](const Plan& pl)
    { return p.workspace && !((uintptr_t) p.workspace & 127) && p.workspace_bytes >= prep + pl.workspace(); };
    // first choice where it applies: the persistent tcgen05 kernel on a two-level schedule
    bool use_sk = plan.kind == KIND_GQA && build_streamk_ws(h, plan, p.host_past_key_value_lengths, p.num_requests, sk, sk_ctas);
    if (use_sk && !fits(plan))
    {
        use_sk = false;
        plan = plan_shape(h, p.num_requests, rows_per_seq);
    }
    if (!use_sk)
        use_sk = plan_streamk(h, plan, p.host_past_key_value_lengths, p.num_requests, sk, sk_ctas);
    if (use_sk && !fits(plan))
    {
        use_sk = false;
        plan = plan_shape(h, p.num_requests, rows_per_seq);
    }
    if (!use_sk)
        plan_partitions(h, plan, p.num_requests, rows_per_seq, max_past, p.host_past_key_value_lengths);
    if (plan.nsplit > 1 || prep)
    {
        if (!p.workspace || ((uintptr_t) p.workspace & 127))
            return p.workspace ? DX_ERR_BAD_ARG : DX_ERR_WORKSPACE;
        if (p.workspace_bytes < prep + plan.workspace())
            return DX_ERR_WORKSPACE;
    }
    char* const ws_partials = reinterpret_cast<char*>(p.workspace) + prep;

    AttnArgs a{};
    a.qkv = prep ? p.workspace : p.attention_input;
    a.out = p.context_buf;
    a.seq_len = p.sequence_lengths;
    a.block_ptrs = p.block_pointers;
    a.scale_orig_quant = p.kv_scale_orig_quant;
    a.scale_quant_orig = p.kv_scale_quant_orig;
    a.part_o = plan.nsplit > 1 ? reinterpret_cast<float*>(ws_partials) : nullptr;
    a.part_ml = plan.nsplit > 1 ? reinterpret_cast<float2*>(ws_partials + plan.part_o_bytes) : nullptr;
    a.status = h->status_dev;
    a.batch = p.num_requests;
    a.num_heads = c.num_heads;
    a.num_kv_heads = c.num_kv_heads;
    a.max_blocks_per_seq = p.max_blocks_per_sequence;
    a.tpb_log2 = h->tpb_log2;
    a.chunk_tokens = plan.chunk_tokens;
    a.nsplit = plan.nsplit;
    a.softmax_scale_log2 = 1.4426950408889634f / (sqrtf((float) c.head_size) * c.q_scaling);
    a.streamk = use_sk ? 1 : 0;
    a.tickets = (use_sk && plan.kind == KIND_TOKWS && sk.n2 > 0) ? h->status_dev + 16 : nullptr;
    a.guard = h->guard;

    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st != DX_OK)
        return st;

    if (prep)
    {
        // bias + rotary embedding of the new token's q / k (bias only for v) into the workspace copy
        st = launch_prep(h, p, p.num_requests, stream);
        if (st != DX_OK)
            return st;
    }

    if (plan.kind == KIND_WIDE)
    {
        int hgroups = plan.hgroups;
        void* args[] = {&a, &hgroups};
        dim3 grid(plan.nsplit, c.num_kv_heads * plan.hgroups, p.num_requests);
        st = launch_attention(h, h->k_wide.fn, grid, dim3(128), (size_t) h->k_wide.smem, args, h->pdl_other == 1, stream);
    }
    else if (plan.kind == KIND_TOK)
    {
        int hgroups = 1;
        void* args[] = {&a, &hgroups, use_sk ? &sk : &h->sk_zero};
        const dim3 grid = use_sk ? dim3(sk_ctas) : dim3(plan.nsplit, c.num_kv_heads, p.num_requests);
        st = check_cuda(h, cudaLaunchKernel(h->k_tok.fn, grid, dim3(128), args, (size_t) h->k_tok.smem, stream));
    }
    else if (plan.kind == KIND_TOKWS)
    {
        int hgroups = 1;
        void* args[] = {&a, &hgroups, &sk};
        st = check_cuda(h, cudaLaunchKernel(h->k_tokws.fn, dim3(sk_ctas), dim3(h->k_tokws.threads), args,
                               (size_t) h->k_tokws.smem, stream));
    }
    else if (plan.kind == KIND_GQA)
    {
        const KernelInfo& k = plan.six ? h->k_gqa_six : h->k_gqa[plan.heads16 ? 1 : 0];
        if (!k.fn)
            return DX_ERR_UNSUPPORTED;
        int hgroups = plan.hgroups;
        void* args[] = {&a, &hgroups, use_sk ? &sk : &h->sk_zero};
        const dim3 grid = use_sk ? dim3(sk_ctas) : dim3(plan.nsplit, c.num_kv_heads * plan.hgroups, p.num_requests);
        const bool dependent = h->pdl_attention == 1 || (h->pdl_attention < 0 && use_sk && plan.chunk_tokens >= 4096);
        st = launch_attention(h, k.fn, grid, dim3(k.threads), (size_t) k.smem, args, dependent, stream);
    }
    else
    {
        void* args[] = {&a};
        dim3 grid(plan.nsplit, c.num_heads, p.num_requests);
        st = launch_attention(h, h->k_mha.fn, grid, dim3(128), (size_t) h->k_mha.smem, args, h->pdl_other == 1, stream);
    }
    if (st != DX_OK)
        return st;
    h->launches.fetch_add(1);

    if (plan.nsplit > 1)
        return launch_merge(h, a, (size_t) p.num_requests * c.num_heads, plan.hgroups, use_sk ? &sk : nullptr, stream);
    return DX_OK;
}

int dx_attn_enqueue_generation_host(
    dx_attn_t* h, const dx_attn_generation_params* params, void* cuda_stream, int32_t sync)
{
    dx_attn_generation_params p;
    if (!h || !read_params(params, p))
        return DX_ERR_BAD_ARG;
    const dx_attn_config& c = h->cfg;
    if (p.num_requests < 0 || p.max_blocks_per_sequence <= 0)
        return DX_ERR_BAD_ARG;
    if (p.num_requests == 0)
        return DX_OK;
    if (!p.attention_input || !p.sequence_lengths || !p.block_pointers || !p.context_buf)
        return DX_ERR_BAD_ARG;
    if (p.input_seq_length > 1)
        return DX_ERR_UNSUPPORTED; // several tokens per sequence: device buffers only
    const size_t B = (size_t) p.num_requests * (size_t) std::max(1, p.beam_width); // sequences
    const size_t qkv_bytes = B * (size_t) (c.num_heads + 2 * c.num_kv_heads) * c.head_size * 2;
    const size_t out_bytes = B * (size_t) c.num_heads * c.head_size * 2;
    const size_t tbl_bytes = B * 2 * (size_t) p.max_blocks_per_sequence * sizeof(int64_t);
    const size_t len_bytes = B * sizeof(int32_t);
    const size_t o_qkv = 0, o_out = align_up(qkv_bytes, 256), o_tbl = o_out + align_up(out_bytes, 256),
                 o_len = o_tbl + align_up(tbl_bytes, 256), total = o_len + align_up(len_bytes, 256);

    cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st != DX_OK)
        return st;
    if (!h->h2d_stream)
    {
        st = check_cuda(h, cudaStreamCreateWithFlags(&h->h2d_stream, cudaStreamNonBlocking));
        if (st == DX_OK)
            st = check_cuda(h, cudaStreamCreateWithFlags(&h->d2h_stream, cudaStreamNonBlocking));
        for (int i = 0; i < dx_attn::HOST_SLOTS && st == DX_OK; ++i)
        {
            st = check_cuda(h, cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
            if (st == DX_OK)
                st = check_cuda(h, cudaEventCreateWithFlags(&h->ev_done[i], cudaEventDisableTiming));
            if (st == DX_OK)
                st = check_cuda(h, cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming));
        }
        if (st != DX_OK)
            return st;
    }
    if (h->stage_bytes < total)
    {
        // Growing the staging area is the one allocation made after create(); it synchronises.
        st = check_cuda(h, cudaDeviceSynchronize());
        if (st != DX_OK)
            return st;
        for (bool& pending : h->out_pending)
            pending = false;
        if (h->stage_dev)
            cudaFree(h->stage_dev);
        h->stage_dev = nullptr;
        h->stage_bytes = 0;
        st = check_cuda(h, cudaMalloc(&h->stage_dev, dx_attn::HOST_SLOTS * total));
        if (st != DX_OK)
            return st;
        h->stage_bytes = total;
    }
    // Staging slots: the copies of this step run on their own streams beside the kernels of the steps before
    // it.  A slot is reused only after the output of the step that used it last is in host memory.
    const int slot = (int) (h->host_calls % dx_attn::HOST_SLOTS);
    if (h->out_pending[slot])
    {
        st = check_cuda(h, cudaEventSynchronize(h->ev_out[slot]));
        if (st != DX_OK)
            return st;
        h->out_pending[slot] = false;
    }
    char* base = reinterpret_cast<char*>(h->stage_dev) + (size_t) slot * h->stage_bytes;
    st = check_cuda(h, cudaMemcpyAsync(base + o_qkv, p.attention_input, qkv_bytes, cudaMemcpyHostToDevice, h->h2d_stream));
    if (st == DX_OK)
        st = check_cuda(
            h, cudaMemcpyAsync(base + o_tbl, p.block_pointers, tbl_bytes, cudaMemcpyHostToDevice, h->h2d_stream));
    if (st == DX_OK)
        st = check_cuda(
            h, cudaMemcpyAsync(base + o_len, p.sequence_lengths, len_bytes, cudaMemcpyHostToDevice, h->h2d_stream));
    if (st == DX_OK)
        st = check_cuda(h, cudaEventRecord(h->ev_in[slot], h->h2d_stream));
    if (st == DX_OK)
        st = check_cuda(h, cudaStreamWaitEvent(stream, h->ev_in[slot], 0));
    if (st != DX_OK)
        return st;
    void* host_out = p.context_buf;
    p.attention_input = base + o_qkv;
    p.block_pointers = reinterpret_cast<const int64_t*>(base + o_tbl);
    p.sequence_lengths = reinterpret_cast<const int32_t*>(base + o_len);
    p.context_buf = base + o_out;
    // (between the kernels of consecutive steps this stream waits for copies: nothing to overlap a dependent launch with,
    // and the attribute costs the pipelined figure 3 %)
    h->no_dependent_launch = true;
    st = dx_attn_enqueue_generation(h, &p, cuda_stream);
    h->no_dependent_launch = false;
    if (st != DX_OK)
        return st;
    st = check_cuda(h, cudaEventRecord(h->ev_done[slot], stream));
    if (st == DX_OK)
        st = check_cuda(h, cudaStreamWaitEvent(h->d2h_stream, h->ev_done[slot], 0));
    if (st == DX_OK)
        st = check_cuda(h, cudaMemcpyAsync(host_out, base + o_out, out_bytes, cudaMemcpyDeviceToHost, h->d2h_stream));
    if (st == DX_OK)
        st = check_cuda(h, cudaEventRecord(h->ev_out[slot], h->d2h_stream));
    if (st != DX_OK)
        return st;
    h->out_pending[slot] = true;
    ++h->host_calls;
    if (sync)
    {
        st = check_cuda(h, cudaEventSynchronize(h->ev_out[slot]));
        h->out_pending[slot] = false;
    }
    return st;
}

int dx_attn_host_sync(dx_attn_t* h)
{
    if (!h)
        return DX_ERR_BAD_ARG;
    int st = DX_OK;
    for (int i = 0; i < dx_attn::HOST_SLOTS; ++i)
    {
        if (h->out_pending[i])
        {
            const int e = check_cuda(h, cudaEventSynchronize(h->ev_out[i]));
            if (e != DX_OK)
                st = e;
            h->out_pending[i] = false;
        }
    }
    return st;
}

int dx_attn_validate(const dx_attn_t* h, const int64_t* host_block_pointers,
    const int32_t* host_past_key_value_lengths, int32_t num_requests, int32_t max_blocks_per_sequence,
    const void* pool_base, size_t pool_bytes)
{
    if (!h || !host_block_pointers || !host_past_key_value_lengths || num_requests < 0
        || max_blocks_per_sequence <= 0 || !pool_base)
        return DX_ERR_BAD_ARG;
    const dx_attn_config& c = h->cfg;
    const size_t esz = h->cache_kind == CACHE_T ? 2 : 1;
    const size_t block_bytes = (size_t) c.num_kv_heads * c.tokens_per_block * c.head_size * esz;
    const uintptr_t lo = (uintptr_t) pool_base, hi = lo + pool_bytes;
    for (int b = 0; b < num_requests; ++b)
    {
        const int past = host_past_key_value_lengths[b];
        if (past < 0)
            return DX_ERR_BAD_ARG;
        const int64_t need = ((int64_t) past + 1 + c.tokens_per_block - 1) / c.tokens_per_block;
        if (need > max_blocks_per_sequence)
            return DX_ERR_BOUNDS;
        for (int kv = 0; kv < 2; ++kv)
        {
            const int64_t* row = host_block_pointers + ((size_t) b * 2 + kv) * max_blocks_per_sequence;
            for (int64_t i = 0; i < need; ++i)
            {
                const uintptr_t ptr = (uintptr_t) row[i];
                if (ptr & 15)
                    return DX_ERR_BAD_ARG;
                if (ptr < lo || ptr + block_bytes > hi)
                    return DX_ERR_BOUNDS;
            }
        }
    }
    return DX_OK;
}

int dx_attn_device_status(dx_attn_t* h)
{
    if (!h)
        return DX_ERR_BAD_ARG;
    int32_t v = 0;
    int st = check_cuda(h, cudaSetDevice(h->cfg.device));
    if (st == DX_OK)
        st = check_cuda(h, cudaMemcpy(&v, h->status_dev, sizeof(v), cudaMemcpyDeviceToHost));
    if (st != DX_OK)
        return st;
    if (v != 0)
    {
        st = check_cuda(h, cudaMemset(h->status_dev, 0, sizeof(v)));
        if (st != DX_OK)
            return st;
    }
    if (v == 0)
        return DX_OK;
    if (v == STATUS_TIMEOUT)
        return DX_ERR_TIMEOUT;
    return (v == STATUS_NO_BLOCKS || v == STATUS_PLAN_EXCEEDED || v == STATUS_BAD_TABLE) ? DX_ERR_BOUNDS : DX_ERR_CUDA;
}

int dx_kv_cache_step(dx_attn_t* h, int32_t* sequence_lengths, int64_t* block_pointers, int32_t num_requests,
    int32_t max_blocks_per_sequence, const int64_t* free_blocks, int32_t n_free, int32_t* free_cursor, void* cuda_stream)
{
    if (!h || num_requests < 0 || max_blocks_per_sequence <= 0 || n_free < 0)
        return DX_ERR_BAD_ARG;
    if (num_requests == 0)
        return DX_OK;
    if (!sequence_lengths || !block_pointers || !free_cursor || (n_free > 0 && !free_blocks))
        return DX_ERR_BAD_ARG;
    if (((uintptr_t) sequence_lengths | (uintptr_t) free_cursor) & 3)
        return DX_ERR_BAD_ARG;
    if (((uintptr_t) block_pointers | (uintptr_t) free_blocks) & 7)
        return DX_ERR_BAD_ARG;
    int st = check_cuda(h, cudaSetDevice(h->cfg.device));
    if (st != DX_OK)
        return st;
    KvStepArgs a{};
    a.seq_len = sequence_lengths;
    a.block_ptrs = block_pointers;
    a.free_list = free_blocks;
    a.free_cursor = free_cursor;
    a.status = h->status_dev;
    a.batch = num_requests;
    a.max_blocks_per_seq = max_blocks_per_sequence;
    a.tpb_log2 = h->tpb_log2;
    a.n_free = n_free;
    void* args[] = {&a};
    st = check_cuda(h, cudaLaunchKernel(reinterpret_cast<const void*>(&kv_cache_step_kernel), dim3(1), dim3(1024), args, 0,
                           reinterpret_cast<cudaStream_t>(cuda_stream)));
    if (st == DX_OK)
        h->launches.fetch_add(1);
    return st;
}

size_t dx_attn_static_scratch_bytes(void)
{
    return DX_STATIC_SCRATCH_BYTES;
}

int dx_attn_enqueue_generation_static_scratch(
    dx_attn_t* h, const dx_attn_generation_params* params, void* cuda_stream)
{
    dx_attn_generation_params full;
    if (!h || !read_params(params, full))
        return DX_ERR_BAD_ARG;
    params = &full;
    if (params->num_requests <= 0)
        return params->num_requests == 0 ? DX_OK : DX_ERR_BAD_ARG;
    // No size check of its own: the forwarded call plans the step (stream-K, classic partitions, the feature paths
    // that need no partials at all) and returns DX_ERR_WORKSPACE before it launches anything when the fixed array
    // is too small for that plan.
    int st = check_cuda(h, cudaSetDevice(h->cfg.device));
    if (st != DX_OK)
        return st;
    void* scratch = nullptr;
    st = static_scratch_address(h, h->cfg.device, &scratch); // first call on a device: symbol look-up
    if (st != DX_OK)
        return st;
    // Nothing in the array has to start at zero: every partition the merge reads is written by
    // this call's attention kernel first.
    dx_attn_generation_params p = *params;
    p.workspace = scratch;
    p.workspace_bytes = DX_STATIC_SCRATCH_BYTES;
    return dx_attn_enqueue_generation(h, &p, cuda_stream);
}

int dx_attn_append_context(dx_attn_t* h, const void* k_src, const void* v_src, const int32_t* sequence_lengths,
    int32_t batch, int32_t seq_len, int32_t attention_window_size, const int64_t* block_pointers,
    int32_t max_blocks_per_sequence, const float* kv_scale_orig_quant, void* cuda_stream)
{
    return dx_attn_append_context_cyclic(h, k_src, v_src, sequence_lengths, batch, seq_len, attention_window_size, 0,
        block_pointers, max_blocks_per_sequence, kv_scale_orig_quant, cuda_stream);
}

int dx_attn_append_context_cyclic(dx_attn_t* h, const void* k_src, const void* v_src, const int32_t* sequence_lengths,
    int32_t batch, int32_t seq_len, int32_t attention_window_size, int32_t sink_token_length,
    const int64_t* block_pointers, int32_t max_blocks_per_sequence, const float* kv_scale_orig_quant, void* cuda_stream)
{
    if (!h || batch < 0 || seq_len < 0 || max_blocks_per_sequence <= 0 || attention_window_size < 1
        || sink_token_length < 0 || sink_token_length >= attention_window_size)
        return DX_ERR_BAD_ARG;
    if (batch == 0 || seq_len == 0)
        return DX_OK;
    if (!k_src || !v_src || !sequence_lengths || !block_pointers)
        return DX_ERR_BAD_ARG;
    if ((((uintptr_t) k_src | (uintptr_t) v_src) & 15) || ((uintptr_t) block_pointers & 7))
        return DX_ERR_BAD_ARG;
    const dx_attn_config& c = h->cfg;
    if (h->cache_kind != CACHE_T && !kv_scale_orig_quant)
        return DX_ERR_BAD_ARG;
    // Slot arithmetic of KVBlockArray (kvCacheUtils.h:71-90): sink tokens that end inside a block leave the rest of
    // that block unused (the bubble); a table with a spare block keeps window + tokens_per_block slots cycling.
    const int tpb = c.tokens_per_block;
    const int in_last = sink_token_length % tpb;
    const int bubble = in_last == 0 ? 0 : tpb - in_last;
    const bool one_more_block = (int64_t) (max_blocks_per_sequence - 1) * tpb >= (int64_t) attention_window_size + bubble;
    const int64_t cyclic_len = one_more_block ? (int64_t) attention_window_size + tpb - sink_token_length
                                              : (int64_t) attention_window_size - sink_token_length;
    // the highest slot a prompt of seq_len tokens can touch has to be inside the table
    const int64_t top_slot = seq_len <= sink_token_length
        ? (int64_t) seq_len - 1
        : (int64_t) sink_token_length + bubble + std::min<int64_t>((int64_t) seq_len - sink_token_length, cyclic_len) - 1;
    if (top_slot >= (int64_t) max_blocks_per_sequence * tpb)
        return DX_ERR_BAD_ARG;
    if (!h->k_append.fn)
        return DX_ERR_UNSUPPORTED;
    AppendArgs a{};
    a.k_src = k_src;
    a.v_src = v_src;
    a.seq_len = sequence_lengths;
    a.block_ptrs = block_pointers;
    a.scale_orig_quant = kv_scale_orig_quant;
    a.batch = batch;
    a.num_kv_heads = c.num_kv_heads;
    a.src_seq_len = seq_len;
    a.max_blocks_per_seq = max_blocks_per_sequence;
    a.tpb_log2 = h->tpb_log2;
    a.status = h->status_dev;
    a.guard = h->guard;
    a.window = attention_window_size;
    a.sink = sink_token_length;
    a.bubble = bubble;
    a.cyclic_len = (int32_t) cyclic_len;
    int st = check_cuda(h, cudaSetDevice(c.device));
    if (st != DX_OK)
        return st;
    const int esz = h->cache_kind == CACHE_T ? 2 : 1;
    const long threads = (long) seq_len * (c.head_size * esz / 16);
    void* args[] = {&a};
    dim3 grid((unsigned) ((threads + 255) / 256), batch, c.num_kv_heads);
    st = check_cuda(h, cudaLaunchKernel(h->k_append.fn, grid, dim3(256), args, 0, reinterpret_cast<cudaStream_t>(cuda_stream)));
    if (st == DX_OK)
        h->launches.fetch_add(1);
    return st;
}

int dx_build_has_bounds_check(void)
{
#ifdef DECODE_ATTN_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}

int dx_attn_set_pool_range(dx_attn_t* h, const void* pool, size_t pool_bytes)
{
    if (!h || (pool == nullptr) != (pool_bytes == 0))
        return DX_ERR_BAD_ARG;
    const dx_attn_config& c = h->cfg;
    const size_t block_bytes = (size_t) c.num_kv_heads * c.tokens_per_block * c.head_size * (h->cache_kind == CACHE_T ? 2 : 1);
    if (pool && pool_bytes < block_bytes)
        return DX_ERR_BAD_ARG;
    h->guard.pool_lo = pool ? reinterpret_cast<int64_t>(pool) : 0;
    h->guard.pool_hi = pool ? reinterpret_cast<int64_t>(pool) + (int64_t) (pool_bytes - block_bytes) + 1 : 0;
    return DX_OK;
}

int dx_attn_selftest_wait_timeout(dx_attn_t* h, int32_t poll_limit, void* cuda_stream)
{
    if (!h || poll_limit < 1 || poll_limit > (1 << 20))
        return DX_ERR_BAD_ARG;
    int st = check_cuda(h, cudaSetDevice(h->cfg.device));
    if (st != DX_OK)
        return st;
    int32_t* status = h->status_dev;
    int limit = poll_limit;
    void* args[] = {&status, &limit};
    st = check_cuda(h, cudaLaunchKernel(reinterpret_cast<const void*>(&wait_timeout_selftest_kernel), dim3(1), dim3(32),
                           args, 0, reinterpret_cast<cudaStream_t>(cuda_stream)));
    if (st == DX_OK)
        h->launches.fetch_add(1);
    return st;
}

int dx_attn_last_cuda_error(const dx_attn_t* h)
{
    return h ? h->last_cuda_error : 0;
}

int64_t dx_attn_launch_count(const dx_attn_t* h)
{
    return h ? h->launches.load() : 0;
}

} // extern "C"
