// Instantiations of the tcgen05 wide-group decode kernel (FP8 cache, more than 16 q heads per kv head).
#include "dx_launch.h"
#include "dx_wide_kernel.cuh"

namespace dx
{
// The kernel allocates tensor memory without a bounded wait, so the CTAs that fit on one SM by
// shared memory must never ask for more than its 512 columns.
template <int DH>
constexpr bool tmem_fits()
{
    return (227 * 1024 / WideTraits<DH>::SMEM_BYTES) * WideTraits<DH>::TMEM_COLS <= 512;
}
static_assert(tmem_fits<64>() && tmem_fits<128>(), "tensor memory over-subscribed");

template <typename T, int DH>
static KernelInfo mk()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&wide_decode_kernel<T, DH>);
    k.smem = WideTraits<DH>::SMEM_BYTES;
    k.resident = WideTraits<DH>::MIN_BLOCKS;
    return k;
}

KernelInfo wide_kernel_info(int dtype, int dh)
{
    if (dh == 64)
        return dtype == 0 ? mk<__half, 64>() : mk<__nv_bfloat16, 64>();
    if (dh == 128)
        return dtype == 0 ? mk<__half, 128>() : mk<__nv_bfloat16, 128>();
    return KernelInfo{};
}
} // namespace dx
