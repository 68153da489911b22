/* TEST INFRASTRUCTURE ONLY.
 * Second, independent statement of the quantise-on-write bytes in C++, using the CUDA toolkit's
 * host-callable fp8/half/bfloat16 conversions - the same cuda_fp8.h the reference kernels include
 * (cpp/tensorrt_llm/kernels/decoderMaskedMultiheadAttentionUtils.h:3510-3624, :3753-3763) - and the
 * expected-value functions of the reference's known-answer test
 * (cpp/tests/runtime/transposeKVKernelTest.cpp:76-88: int8 = round(clip(x*scale)), fp8 = e4m3(x*scale)).
 * Host code only; nothing here runs on a GPU. */
#include <cmath>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

extern "C" {

/* kernel chain, fp16 activations: scale -> half, half*half (one rounding), half -> e4m3 satfinite */
void qc_fp8_from_fp16(const uint16_t* x, int n, float scale, uint8_t* out)
{
    const __half s = __float2half_rn(scale);
    for (int i = 0; i < n; ++i)
    {
        __half_raw r;
        r.x = x[i];
        const __half p = __float2half_rn(__half2float(s) * __half2float(__half(r)));
        out[i] = (uint8_t) __nv_cvt_halfraw_to_fp8(static_cast<__half_raw>(p), __NV_SATFINITE, __NV_E4M3);
    }
}

/* kernel chain, bf16 activations */
void qc_fp8_from_bf16(const uint16_t* x, int n, float scale, uint8_t* out)
{
    const __nv_bfloat16 s = __float2bfloat16_rn(scale);
    for (int i = 0; i < n; ++i)
    {
        __nv_bfloat16_raw r;
        r.x = x[i];
        const __nv_bfloat16 p = __float2bfloat16_rn(__bfloat162float(s) * __bfloat162float(__nv_bfloat16(r)));
        out[i] = (uint8_t) __nv_cvt_bfloat16raw_to_fp8(static_cast<__nv_bfloat16_raw>(p), __NV_SATFINITE, __NV_E4M3);
    }
}

/* kernel chain, int8: rint (half to even) of the fp32 product, saturated */
void qc_int8_from_f32(const float* x, int n, float scale, int8_t* out)
{
    for (int i = 0; i < n; ++i)
    {
        float v = nearbyintf(x[i] * scale);
        v = fminf(127.f, fmaxf(-128.f, v));
        out[i] = (int8_t) v;
    }
}

/* the reference known-answer test's expectation for int8: clip, then std::round (half away) */
void qc_kat_int8(const float* x, int n, float scale, int8_t* out)
{
    for (int i = 0; i < n; ++i)
    {
        const float clipped = fminf(127.f, fmaxf(x[i] * scale, -128.f));
        out[i] = (int8_t) roundf(clipped);
    }
}

/* the reference known-answer test's expectation for fp8: __nv_fp8_e4m3(float) */
void qc_kat_fp8(const float* x, int n, float scale, uint8_t* out)
{
    for (int i = 0; i < n; ++i)
    {
        const __nv_fp8_e4m3 v(x[i] * scale);
        out[i] = (uint8_t) v.__x;
    }
}

/* e4m3 byte -> float, for the dequantise side */
void qc_fp8_to_f32(const uint8_t* x, int n, float* out)
{
    for (int i = 0; i < n; ++i)
    {
        __nv_fp8_e4m3 v;
        v.__x = x[i];
        out[i] = float(v);
    }
}
}
