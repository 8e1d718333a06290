// Device-side helpers shared by the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>

#include "../../include/darknet_b200.h"

namespace dnb {

// Darknet's activation functions (src/activations.h:19-53), evaluated in fp32
// as the reference's device code does (src/activation_kernels.cu:13-77).  The
// CPU reference evaluates the constants in double; the difference is at most
// one fp32 ulp and far inside the layer tolerances.
__device__ __forceinline__ float activate(float x, int a)
{
    switch (a) {
    case DNB_LINEAR:   return x;
    case DNB_LEAKY:    return x > 0.f ? x : 0.1f * x;
    case DNB_LOGISTIC: return 1.f / (1.f + expf(-x));
    case DNB_RELU:     return x > 0.f ? x : 0.f;
    case DNB_RELIE:    return x > 0.f ? x : 0.01f * x;
    case DNB_RAMP:     return (x > 0.f ? x : 0.f) + 0.1f * x;
    case DNB_TANH:     return (expf(2.f * x) - 1.f) / (expf(2.f * x) + 1.f);
    case DNB_LOGGY:    return 2.f / (1.f + expf(-x)) - 1.f;
    case DNB_ELU:      return x >= 0.f ? x : expf(x) - 1.f;
    case DNB_SELU:     return x >= 0.f ? 1.0507f * x : 1.0507f * 1.6732f * (expf(x) - 1.f);
    case DNB_PLSE:
        if (x < -4.f) return 0.01f * (x + 4.f);
        if (x > 4.f) return 0.01f * (x - 4.f) + 1.f;
        return 0.125f * x + 0.5f;
    case DNB_STAIR: {
        int n = (int)floorf(x);
        if (n % 2 == 0) return floorf(x / 2.f);
        return (x - n) + floorf(x / 2.f);
    }
    case DNB_HARDTAN:  return x < -1.f ? -1.f : (x > 1.f ? 1.f : x);
    case DNB_LHTAN:
        if (x < 0.f) return 0.001f * x;
        if (x > 1.f) return 0.001f * (x - 1.f) + 1.f;
        return x;
    }
    return 0.f;
}

// Same function for hot loops: the two common activations inline, the 14-way switch out of line (inlined
// into an unrolled epilogue it multiplies the code size).
static __device__ __noinline__ float activate_call(float x, int a) { return activate(x, a); }
__device__ __forceinline__ float activate_fast(float x, int a)
{
    if (a == DNB_LEAKY) return fmaxf(x, 0.1f * x);   // x > 0 ? x : 0.1x
    if (a == DNB_LINEAR) return x;
    return activate_call(x, a);
}

// Round an fp32 value to the nearest TF32 (10-bit mantissa) value, ties away from zero, low 13 mantissa
// bits clear: what cvt.rna.tf32.f32 computes for finite values, written as an integer add and a mask
// because the conversion instruction issues at a fraction of the rate and the epilogues run it per element.
// (Infinity stays infinity; a NaN may become infinity.)
__device__ __forceinline__ float round_tf32(float x)
{
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace dnb
