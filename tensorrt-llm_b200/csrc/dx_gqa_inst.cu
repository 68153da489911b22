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

// The feature forms of the same kernel (FEAT 1: beam search, cyclic window, ALiBi; FEAT 2: several new tokens per
// sequence): classic launches only.
template <typename T, int CACHE, int DH, bool H16, int FEAT>
static KernelInfo mk_feature()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&gqa_decode_kernel<T, CACHE, DH, H16, 4, FEAT>);
    k.smem = GqaTraits<DH, gqa_min_blocks<CACHE, DH, H16>()>::SMEM_BYTES;
    k.resident = gqa_min_blocks<CACHE, DH, H16>();
    return k;
}

template <typename T, int DH, int FEAT>
static KernelInfo mk16_feature()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&gqa16_decode_kernel<T, DH, FEAT>);
    k.smem = Gqa16Traits<DH>::SMEM_BYTES;
    k.resident = Gqa16Traits<DH>::MIN_BLOCKS;
    return k;
}

template <typename T, bool H16, int FEAT>
static KernelInfo feature_by_cache_dh(int cache, int dh)
{
    if (cache == CACHE_T)
        return dh == 64 ? mk16_feature<T, 64, FEAT>()
                        : (dh == 128 ? mk16_feature<T, 128, FEAT>() : (dh == 256 ? mk16_feature<T, 256, FEAT>() : KernelInfo{}));
    if (dh == 64)
    {
        if (cache == CACHE_INT8) return mk_feature<T, CACHE_INT8, 64, H16, FEAT>();
        if (cache == CACHE_FP8) return mk_feature<T, CACHE_FP8, 64, H16, FEAT>();
    }
    else if (dh == 128)
    {
        if (cache == CACHE_INT8) return mk_feature<T, CACHE_INT8, 128, H16, FEAT>();
        if (cache == CACHE_FP8) return mk_feature<T, CACHE_FP8, 128, H16, FEAT>();
    }
    return KernelInfo{};
}

KernelInfo gqa_feature_kernel_info(int dtype, int cache, int dh, bool heads16)
{
    if (dtype == 0)
        return heads16 ? feature_by_cache_dh<__half, true, 1>(cache, dh) : feature_by_cache_dh<__half, false, 1>(cache, dh);
    return heads16 ? feature_by_cache_dh<__nv_bfloat16, true, 1>(cache, dh) : feature_by_cache_dh<__nv_bfloat16, false, 1>(cache, dh);
}

KernelInfo gqa_multi_token_kernel_info(int dtype, int cache, int dh, bool heads16)
{
    if (dtype == 0)
        return heads16 ? feature_by_cache_dh<__half, true, 2>(cache, dh) : feature_by_cache_dh<__half, false, 2>(cache, dh);
    return heads16 ? feature_by_cache_dh<__nv_bfloat16, true, 2>(cache, dh) : feature_by_cache_dh<__nv_bfloat16, false, 2>(cache, dh);
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
        return dh == 64 ? mk16<T, 64>() : (dh == 128 ? mk16<T, 128>() : (dh == 256 ? mk16<T, 256>() : KernelInfo{}));
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

// The stream-K form with two CTAs of six warps per SM (FP8 cache, Dh 128, groups of up to 8 heads).
template <typename T>
static KernelInfo mk_six()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&gqa_decode_kernel<T, CACHE_FP8, 128, false, 6>);
    k.smem = GqaTraits<128, gqa_min_blocks<CACHE_FP8, 128, false, 6>(), 6>::SMEM_BYTES;
    k.resident = 2;
    k.threads = 192;
    return k;
}

KernelInfo gqa_streamk_kernel_info(int dtype, int cache, int dh, bool heads16)
{
    if (cache != CACHE_FP8 || dh != 128 || heads16)
        return KernelInfo{};
    return dtype == 0 ? mk_six<__half>() : mk_six<__nv_bfloat16>();
}

KernelInfo gqa_kernel_info(int dtype, int cache, int dh, bool heads16)
{
    if (dtype == 0)
        return heads16 ? by_cache_dh<__half, true>(cache, dh) : by_cache_dh<__half, false>(cache, dh);
    return heads16 ? by_cache_dh<__nv_bfloat16, true>(cache, dh) : by_cache_dh<__nv_bfloat16, false>(cache, dh);
}
} // namespace dx
