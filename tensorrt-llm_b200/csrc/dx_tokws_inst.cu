// Instantiations of the persistent warp-specialised tcgen05 grouped-head decode kernel (FP8 cache, Dh 128, up to 16
// q heads per kv head).
#include "dx_launch.h"
#include "dx_tokws_kernel.cuh"

namespace dx
{
// CTAs per SM and ring stages per CTA.  Two CTAs with three stages each: two independent softmax / MMA pipelines per
// SM hide each other's piece boundaries and synchronisation latencies; the ring memory per SM is the same.
template <int GP>
struct TokWsBuild
{
    static constexpr int MINB = 2, NST = 3;
};
template <> // 16 padded heads: the Q and P buffers are twice as large and two CTAs no longer fit
struct TokWsBuild<16>
{
    static constexpr int MINB = 1, NST = 6;
};

// tcgen05.alloc has no bounded form: the CTAs that fit on one SM by shared memory must fit in its 512 columns.
template <int GP>
constexpr bool tokws_fits()
{
    using Tr = TokWsTraits<GP, TokWsBuild<GP>::NST>;
    const int by_smem = 227 * 1024 / Tr::SMEM_BYTES;
    return by_smem >= TokWsBuild<GP>::MINB && by_smem * Tr::TMEM_COLS <= 512;
}
static_assert(tokws_fits<8>() && tokws_fits<16>(), "shared memory / tensor memory budget");

template <typename T, int GP>
static KernelInfo mk()
{
    using B = TokWsBuild<GP>;
    KernelInfo k;
    k.fn = reinterpret_cast<const void*>(&tokws_decode_kernel<T, GP, B::NST, B::MINB>);
    k.smem = TokWsTraits<GP, B::NST>::SMEM_BYTES;
    k.resident = B::MINB;
    k.threads = TokWsTraits<GP, B::NST>::THREADS;
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
