// Instantiations of the CUDA-core multi-head decode kernel.
#include "dx_launch.h"
#include "dx_append_kernel.cuh"
#include "dx_mha_int8_kernel.cuh"
#include "dx_mha_kernel.cuh"

namespace dx
{
template <typename T, int CACHE, int DH>
static KernelInfo mk()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&mha_decode_kernel<T, CACHE, DH>);
    k.smem = MhaTraits<CACHE, DH>::SMEM_BYTES;
    return k;
}

template <typename T>
static KernelInfo by_cache_dh(int cache, int dh)
{
    if (dh == 64)
    {
        if (cache == CACHE_T) return mk<T, CACHE_T, 64>();
        if (cache == CACHE_INT8) return mk<T, CACHE_INT8, 64>();
        if (cache == CACHE_FP8) return mk<T, CACHE_FP8, 64>();
    }
    else if (dh == 128)
    {
        if (cache == CACHE_T) return mk<T, CACHE_T, 128>();
        if (cache == CACHE_INT8) return mk<T, CACHE_INT8, 128>();
        if (cache == CACHE_FP8) return mk<T, CACHE_FP8, 128>();
    }
    else if (dh == 256) // (GPT-J- / Gemma-shaped heads: the streaming per-head kernel, split-K and merge included)
    {
        if (cache == CACHE_T) return mk<T, CACHE_T, 256>();
        if (cache == CACHE_INT8) return mk<T, CACHE_INT8, 256>();
        if (cache == CACHE_FP8) return mk<T, CACHE_FP8, 256>();
    }
    return KernelInfo{};
}

template <typename T, int DH>
static KernelInfo mk_int8()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&mha_int8_decode_kernel<T, DH>);
    k.smem = MhaInt8Traits<DH>::SMEM_BYTES;
    return k;
}

KernelInfo mha_kernel_info(int dtype, int cache, int dh, int tokens_per_block)
{
    // INT8 caches take the integer (dp4a) kernel when a token group fits a cache block.
    if (cache == CACHE_INT8 && dh == 128 && tokens_per_block >= MhaInt8Traits<128>::TG)
        return dtype == 0 ? mk_int8<__half, 128>() : mk_int8<__nv_bfloat16, 128>();
    if (cache == CACHE_INT8 && dh == 64 && tokens_per_block >= MhaInt8Traits<64>::TG)
        return dtype == 0 ? mk_int8<__half, 64>() : mk_int8<__nv_bfloat16, 64>();
    return dtype == 0 ? by_cache_dh<__half>(cache, dh) : by_cache_dh<__nv_bfloat16>(cache, dh);
}
template <typename T>
static KernelInfo append_by(int cache, int dh)
{
    KernelInfo k;
#define DX_APPEND_CASE(C, D)                                                                       \
    if (cache == C && dh == D)                                                                     \
        k.fn = reinterpret_cast<const void*>(&kv_append_context_kernel<T, C, D>);
    DX_APPEND_CASE(CACHE_T, 64)
    DX_APPEND_CASE(CACHE_T, 128)
    DX_APPEND_CASE(CACHE_INT8, 64)
    DX_APPEND_CASE(CACHE_INT8, 128)
    DX_APPEND_CASE(CACHE_FP8, 64)
    DX_APPEND_CASE(CACHE_FP8, 128)
#undef DX_APPEND_CASE
    return k;
}

KernelInfo append_kernel_info(int dtype, int cache, int dh)
{
    return dtype == 0 ? append_by<__half>(cache, dh) : append_by<__nv_bfloat16>(cache, dh);
}
} // namespace dx
