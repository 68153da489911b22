// Instantiations of the feature-complete decode kernel (beams, cyclic window, sinks, ALiBi) and of the
// kernel that appends the new token behind it.
#include "dx_general_kernel.cuh"
#include "dx_launch.h"

namespace dx
{
template <typename T, int CACHE, int DH>
static GeneralKernels mk()
{
    GeneralKernels k;
    k.attn = reinterpret_cast<const void*>(&general_decode_kernel<T, CACHE, DH>);
    k.append = reinterpret_cast<const void*>(&kv_append_token_kernel<T, CACHE, DH>);
    k.multi = reinterpret_cast<const void*>(&multi_token_decode_kernel<T, CACHE, DH>);
    k.smem = (4 * GenTraits<CACHE, DH>::TPW * (DH + 2)) * (int) sizeof(float);
    return k;
}

template <typename T>
static GeneralKernels by_cache_dh(int cache, int dh)
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
    return GeneralKernels{};
}

GeneralKernels general_kernel_info(int dtype, int cache, int dh)
{
    if (dh != 64 && dh != 128)
        return general_kernel_info_other_head_sizes(dtype, cache, dh);
    return dtype == 0 ? by_cache_dh<__half>(cache, dh) : by_cache_dh<__nv_bfloat16>(cache, dh);
}
} // namespace dx
