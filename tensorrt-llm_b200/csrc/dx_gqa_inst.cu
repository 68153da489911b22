// Instantiations of the tensor-core grouped-head decode kernel.
#include <type_traits>

#include "dx_gqa16_kernel.cuh"
#include "dx_gqa_kernel.cuh"
#include "dx_launch.h"

namespace dx
{
template <typename T, int CACHE, int DH, bool H16>
static KernelInfo mk()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&gqa_decode_kernel<T, CACHE, DH, H16>);
    k.smem = GqaTraits<DH, gqa_min_blocks<CACHE, DH, H16>()>::SMEM_BYTES;
    return k;
}

// 16-bit cache: one kernel for any group size up to 16 heads per CTA
template <typename T, int DH>
static KernelInfo mk16()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&gqa16_decode_kernel<T, DH>);
    k.smem = Gqa16Traits<DH>::SMEM_BYTES;
    k.resident = Gqa16Traits<DH>::MIN_BLOCKS;
    return k;
}

template <typename T, bool H16>
static KernelInfo by_cache_dh(int cache, int dh)
{
    if (cache == CACHE_T)
        return dh == 64 ? mk16<T, 64>() : (dh == 128 ? mk16<T, 128>() : KernelInfo{});
    if (dh == 64)
    {
        if (cache == CACHE_INT8) return mk<T, CACHE_INT8, 64, H16>();
        if (cache == CACHE_FP8) return mk<T, CACHE_FP8, 64, H16>();
    }
    else if (dh == 128)
    {
        if (cache == CACHE_INT8) return mk<T, CACHE_INT8, 128, H16>();
        if (cache == CACHE_FP8) return mk<T, CACHE_FP8, 128, H16>();
    }
    return KernelInfo{};
}

KernelInfo gqa_kernel_info(int dtype, int cache, int dh, bool heads16)
{
    if (dtype == 0)
        return heads16 ? by_cache_dh<__half, true>(cache, dh) : by_cache_dh<__half, false>(cache, dh);
    return heads16 ? by_cache_dh<__nv_bfloat16, true>(cache, dh) : by_cache_dh<__nv_bfloat16, false>(cache, dh);
}
} // namespace dx
