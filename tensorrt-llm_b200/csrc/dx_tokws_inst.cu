// Instantiations of the persistent warp-specialised tcgen05 grouped-head decode kernel (FP8 cache, Dh 128, up to 16
// q heads per kv head).
#include "dx_launch.h"
#include "dx_tokws_kernel.cuh"

namespace dx
{
// One CTA per SM by shared memory, so the 128 tensor-memory columns it allocates are always there: tcgen05.alloc,
// which has no bounded form, cannot block.
static_assert(2 * TokWsTraits<8>::SMEM_BYTES > 227 * 1024 && 2 * TokWsTraits<16>::SMEM_BYTES > 227 * 1024,
    "more than one CTA per SM would fit");
static_assert(TokWsTraits<16>::SMEM_BYTES <= 227 * 1024, "shared memory");

template <typename T, int GP>
static KernelInfo mk()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&tokws_decode_kernel<T, GP>);
    k.smem = TokWsTraits<GP>::SMEM_BYTES;
    k.resident = 1;
    k.threads = TokWsTraits<GP>::THREADS;
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
