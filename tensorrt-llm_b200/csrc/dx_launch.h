// Internal: kernel lookup shared by the C-ABI translation unit and the instantiation units.
#pragma once
#include "dx_common.cuh"

namespace dx
{
struct KernelInfo
{
    const void* fn = nullptr; // __global__ function address for cudaLaunchKernel
    int smem = 0;             // dynamic shared memory per CTA, bytes
    int resident = 0;         // CTAs per SM the kernel was built for (0: not stated)
    int threads = 128;        // threads per CTA
};

// dtype: 0 fp16, 1 bf16.  cache: CacheKind.  dh: 64 or 128.
KernelInfo mha_kernel_info(int dtype, int cache, int dh, int tokens_per_block);
KernelInfo gqa_kernel_info(int dtype, int cache, int dh, bool heads16);
KernelInfo gqa_streamk_kernel_info(int dtype, int cache, int dh, bool heads16); // 6-warp CTAs; empty where not built
KernelInfo gqa_feature_kernel_info(int dtype, int cache, int dh, bool heads16); // beam search / ALiBi form, 8-bit caches
KernelInfo gqa_multi_token_kernel_info(int dtype, int cache, int dh, bool heads16); // several new tokens per sequence
KernelInfo wide_kernel_info(int dtype, int dh); // FP8 cache only
KernelInfo tok_kernel_info(int dtype, int dh, int group); // FP8 cache, Dh 128, group <= 16
KernelInfo tokws_kernel_info(int dtype, int dh, int group); // the persistent warp-specialised form of it
struct GeneralKernels
{
    const void* attn = nullptr;   // general_decode_kernel: grid (H, B), 128 threads, `smem` dynamic bytes
    const void* append = nullptr; // kv_append_token_kernel: grid (Hkv, B * q_len), 32 threads
    const void* multi = nullptr;  // multi_token_decode_kernel: grid (H, B * q_len), 128 threads, `smem` dynamic bytes
    const void* context_append = nullptr; // kv_append_context_kernel (set for the head sizes other than 64 / 128)
    int smem = 0;
};
GeneralKernels general_kernel_info(int dtype, int cache, int dh);
// head sizes 32, 48, 80, 96, 104, 112, 144, 160, 192, 224, 256; empty where a cache row is not a multiple of 16 bytes
GeneralKernels general_kernel_info_other_head_sizes(int dtype, int cache, int dh);
KernelInfo merge_kernel_info(int dtype, int dh);
KernelInfo append_kernel_info(int dtype, int cache, int dh);
} // namespace dx
