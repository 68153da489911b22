// Instantiations of the feature-complete decode kernels and of the context-phase writer for the head sizes of the
// reference's MMHA switch other than 64 and 128
// (cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttention.cu:68-85: 32, 48, 80, 96, 104, 112, 144, 160, 192, 224, 256).
// A cache row has to be a multiple of 16 bytes: head size 104 exists for 16-bit caches only.
#include "dx_append_kernel.cuh"
#include "dx_general_kernel.cuh"
#include "dx_launch.h"

namespace dx
{
template <typename T, int CACHE, int DH>
static GeneralKernels mk()
{
    GeneralKernels k;
    if constexpr ((DH * (CACHE == CACHE_T ? 2 : 1)) % 16 == 0)
    {
        k.attn = reinterpret_cast<const void*>(&general_decode_kernel<T, CACHE, DH>);
        k.append = reinterpret_cast<const void*>(&kv_append_token_kernel<T, CACHE, DH>);
        k.multi = reinterpret_cast<const void*>(&multi_token_decode_kernel<T, CACHE, DH>);
        k.context_append = reinterpret_cast<const void*>(&kv_append_context_kernel<T, CACHE, DH>);
        k.smem = (4 * GenTraits<CACHE, DH>::TPW * (DH + 2)) * (int) sizeof(float);
    }
    return k;
}

template <typename T, int DH>
static GeneralKernels by_cache(int cache)
{
    if (cache == CACHE_T) return mk<T, CACHE_T, DH>();
    if (cache == CACHE_INT8) return mk<T, CACHE_INT8, DH>();
    if (cache == CACHE_FP8) return mk<T, CACHE_FP8, DH>();
    return GeneralKernels{};
}

template <typename T>
static GeneralKernels by_dh(int cache, int dh)
{
    switch (dh)
    {
    case 32: return by_cache<T, 32>(cache);
    case 48: return by_cache<T, 48>(cache);
    case 80: return by_cache<T, 80>(cache);
    case 96: return by_cache<T, 96>(cache);
    case 104: return by_cache<T, 104>(cache);
    case 112: return by_cache<T, 112>(cache);
    case 144: return by_cache<T, 144>(cache);
    case 160: return by_cache<T, 160>(cache);
    case 192: return by_cache<T, 192>(cache);
    case 224: return by_cache<T, 224>(cache);
    case 256: return by_cache<T, 256>(cache);
    default: return GeneralKernels{};
    }
}

GeneralKernels general_kernel_info_other_head_sizes(int dtype, int cache, int dh)
{
    return dtype == 0 ? by_dh<__half>(cache, dh) : by_dh<__nv_bfloat16>(cache, dh);
}
} // namespace dx
