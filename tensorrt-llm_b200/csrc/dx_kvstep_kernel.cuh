// Device-resident form of the runtime's per-step cache bookkeeping: every sequence grows by one token, and a
// sequence whose new token starts a block takes the next block of a device-resident free list, in batch order.
// Restates KVCacheManager.step + get_block_pointers for unfinished sequences
// (tensorrt_llm/runtime/kv_cache_manager.py:305-345, :380-387), which the reference runs on the host and uploads
// every step (tensorrt_llm/runtime/generation.py:2219-2221); here lengths and table never leave the device, so a
// captured graph can replay generation steps without host work.
//
// One CTA; blocks are handed out in batch order (block-wide exclusive scan of the "needs a block" flags), so the
// table is identical to the host manager's for the same free list.
#pragma once

#include "dx_common.cuh"

namespace dx
{

struct KvStepArgs
{
    int32_t* seq_len;          // [B] in: tokens so far; out: + 1 (the token the next decode step writes)
    int64_t* block_ptrs;       // [B, 2, M] in/out
    const int64_t* free_list;  // [n_free, 2]: K block pointer, V block pointer
    int32_t* free_cursor;      // [1] in/out: first unused entry of free_list
    int32_t* status;           // set to STATUS_NO_BLOCKS when the list or a table row is exhausted
    int32_t batch;
    int32_t max_blocks_per_seq;
    int32_t tpb_log2;
    int32_t n_free;
};


__global__ void __launch_bounds__(1024) kv_cache_step_kernel(const KvStepArgs a)
{
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0)
        carry = *a.free_cursor;
    __syncthreads();
    const int tpb_mask = (1 << a.tpb_log2) - 1;
    for (int base = 0; base < a.batch; base += blockDim.x)
    {
        const int b = base + tid;
        const int len = b < a.batch ? a.seq_len[b] : 1;
        const int need = (b < a.batch && (len & tpb_mask) == 0) ? 1 : 0;
        // exclusive scan of `need` over the CTA
        int incl = need;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1)
        {
            const int v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d)
                incl += v;
        }
        if (lane == 31)
            warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0)
        {
            int w = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1)
            {
                const int v = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d)
                    w += v;
            }
            warp_sums[lane] = w; // inclusive over warps
        }
        __syncthreads();
        const int before = carry + (warp ? warp_sums[warp - 1] : 0) + incl - need;
        const int total = warp_sums[31];
        if (need)
        {
            const int blk = len >> a.tpb_log2;
            if (before < a.n_free && blk < a.max_blocks_per_seq)
            {
                int64_t* row = a.block_ptrs + (int64_t) b * 2 * a.max_blocks_per_seq;
                row[blk] = a.free_list[2 * before];
                row[a.max_blocks_per_seq + blk] = a.free_list[2 * before + 1];
            }
            else
            {
                report_status(a.status, STATUS_NO_BLOCKS);
            }
        }
        if (b < a.batch)
            a.seq_len[b] = len + 1;
        __syncthreads();
        if (tid == 0)
            carry += total;
        __syncthreads();
    }
    if (tid == 0)
        *a.free_cursor = min(carry, a.n_free);
}

} // namespace dx
