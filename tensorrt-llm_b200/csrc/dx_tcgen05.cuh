// tcgen05 / tensor-memory building blocks shared by the kernels that run on the 5th-generation tensor cores:
// hardware swizzle of shared-memory tiles, shared-memory matrix descriptors, the e4m3 MMA, commit on an
// mbarrier, and loads / stores of accumulator rows (one row of 32 lanes x N columns per warp instruction).
#pragma once

#include "dx_common.cuh"

namespace dx
{

// Hardware swizzle of a row-major tile with `PITCH`-byte rows (64 -> SWIZZLE_64B, 128 -> SWIZZLE_128B).
template <int PITCH>
__device__ __forceinline__ uint32_t hw_swz(uint32_t off)
{
    if constexpr (PITCH == 64)
        return off ^ (((off >> 7) & 3u) << 4);
    else
        return off ^ (((off >> 7) & 7u) << 4);
}

// Shared-memory matrix descriptor (version 1).  lbo / sbo in bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout)
{
    uint64_t d = 0;
    d |= (uint64_t) ((saddr >> 4) & 0x3fffu);
    d |= (uint64_t) ((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t) ((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) (layout & 7u) << 61;
    return d;
}

// D[tmem] (+)= A[smem] * B[smem], e4m3 x e4m3 -> f32, issued by one thread.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t zero = 0;
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 columns of fp32 from TMEM into registers (one row per thread).
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32])
{
    uint32_t r[32];
    __syncwarp(); // .sync.aligned: the warp must be converged (lane 0 may come from the MMA issue branch)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i)
        v[i] = __uint_as_float(r[i]);
}

// One row (32 lanes x NC columns) of fp32 accumulators: tensor memory -> registers and back.
template <int NC>
__device__ __forceinline__ void tmem_ld_row(uint32_t addr, float (&v)[NC])
{
    static_assert(NC == 16 || NC == 32, "16 or 32 columns");
    if constexpr (NC == 32)
    {
        tmem_ld32(addr, v);
    }
    else
    {
        uint32_t r[16];
        __syncwarp();
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(addr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 16; ++i)
            v[i] = __uint_as_float(r[i]);
    }
}

template <int NC>
__device__ __forceinline__ void tmem_st_row(uint32_t addr, const float (&v)[NC])
{
    static_assert(NC == 16 || NC == 32, "16 or 32 columns");
    __syncwarp();
#pragma unroll
    for (int c = 0; c < NC; c += 16)
    {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
                addr + c),
            "r"(__float_as_uint(v[c])), "r"(__float_as_uint(v[c + 1])), "r"(__float_as_uint(v[c + 2])),
            "r"(__float_as_uint(v[c + 3])), "r"(__float_as_uint(v[c + 4])), "r"(__float_as_uint(v[c + 5])),
            "r"(__float_as_uint(v[c + 6])), "r"(__float_as_uint(v[c + 7])), "r"(__float_as_uint(v[c + 8])),
            "r"(__float_as_uint(v[c + 9])), "r"(__float_as_uint(v[c + 10])), "r"(__float_as_uint(v[c + 11])),
            "r"(__float_as_uint(v[c + 12])), "r"(__float_as_uint(v[c + 13])), "r"(__float_as_uint(v[c + 14])),
            "r"(__float_as_uint(v[c + 15]))
            : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

} // namespace dx
