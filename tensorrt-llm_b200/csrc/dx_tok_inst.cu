// Instantiations of the token-major tcgen05 grouped-head decode kernel (FP8 cache, Dh 128, up to 16 q heads per kv head).
#include "dx_launch.h"
#include "dx_tok_kernel.cuh"

namespace dx
{
// tcgen05.alloc has no bounded form: the CTAs that fit on one SM by shared memory must fit in its 512 columns.
template <int GP>
constexpr bool tok_tmem_fits()
{
    return (227 * 1024 / TokTraits<GP>::SMEM_BYTES) * TokTraits<GP>::TMEM_COLS <= 512;
}
static_assert(tok_tmem_fits<8>() && tok_tmem_fits<16>(), "tensor memory over-subscribed");

template <typename T, int GP>
static KernelInfo mk()
{
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&tok_decode_kernel<T, GP>);
    k.smem = TokTraits<GP>::SMEM_BYTES;
    k.resident = TokTraits<GP>::MIN_BLOCKS;
    return k;
}

KernelInfo tok_kernel_info(int dtype, int dh, int group)
{
    if (dh != 128 || group < 1 || group > 16)
        return KernelInfo{};
    if (group <= 8)
        return dtype == 0 ? mk<__half, 8>() : mk<__nv_bfloat16, 8>();
    return dtype == 0 ? mk<__half, 16>() : mk<__nv_bfloat16, 16>();
}
} // namespace dx
