// Instantiations of the persistent warp-specialised tcgen05 grouped-head decode kernel (FP8 cache, Dh 128, up to 16
// q heads per kv head).
#include "dx_launch.h"
#include "dx_tokws_kernel.cuh"

namespace dx
{
// Ring units (16 KB each) per CTA: what fits beside the Q / P / merge buffers.
template <int GP>
struct TokWsBuild
{
    static constexpr int UNITS = GP == 8 ? 12 : 10;
};

// One CTA per SM by shared memory, so the 256 tensor-memory columns it allocates are always there: tcgen05.alloc,
// which has no bounded form, cannot block.
template <int GP>
constexpr bool tokws_fits()
{
    using Tr = TokWsTraits<GP, TokWsBuild<GP>::UNITS>;
    return Tr::SMEM_BYTES <= 227 * 1024 && 2 * Tr::SMEM_BYTES > 227 * 1024;
}
static_assert(tokws_fits<8>() && tokws_fits<16>(), "shared memory budget: exactly one CTA per SM");

template <typename T, int GP>
static KernelInfo mk()
{
    constexpr int U = TokWsBuild<GP>::UNITS;
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&tokws_decode_kernel<T, GP, U>);
    k.smem = TokWsTraits<GP, U>::SMEM_BYTES;
    k.resident = 1;
    k.threads = TokWsTraits<GP, U>::THREADS;
    return k;
}

KernelInfo tokws_kernel_info(int dtype, int dh, int group)
{
    if (dh != 128 || group < 1 || group > 16)
        return KernelInfo{};
    if (group <= 8)
        return dtype == 0 ? mk<__half, 8>() : mk<__nv_bfloat16, 8>();
    return dtype == 0 ? mk<__half, 16>() : mk<__nv_bfloat16, 16>();
}
} // namespace dx
