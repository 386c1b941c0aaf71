// H128 and the input/output stage arithmetic of the staged float32 contract
// (reference python/strix_trellis/linear.py:82-163, src/hadamard.hpp:17-37,
// src/transforms.hpp:8-52).  Every operation that the contract rounds separately
// is written with a non-contractable intrinsic (__fmul_rn/__fadd_rn/__fsub_rn), so
// the result does not depend on -fmad.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "backend.h"

namespace st {

// One warp transforms one 128-block.  Lane l holds elements l, l+32, l+64, l+96.
// Strides 1..16 cross lanes (butterfly partner = lane ^ stride), strides 32 and 64
// stay in registers; order and operand sides match the ascending-stride reference:
// lower index gets lo+hi, upper index gets lo-hi.  Across lanes both cases are ONE fused
// multiply-add, peer + sign*v with sign = +1 (lower) or -1 (upper): the product is exact, so
// the single rounding is that of the add or subtract.
__device__ __forceinline__ void hadamard128_warp(float (&v)[4], int lane) {
#pragma unroll
    for (int stride = 1; stride < 32; stride <<= 1) {
        const float sign = (lane & stride) ? -1.0f : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float peer = __shfl_xor_sync(0xFFFFFFFFu, v[j], stride);
            v[j] = __fmaf_rn(v[j], sign, peer);
        }
    }
    {   // stride 32: pairs (0,1) and (2,3)
        float a = v[0], b = v[1]; v[0] = __fadd_rn(a, b); v[1] = __fsub_rn(a, b);
        a = v[2]; b = v[3];       v[2] = __fadd_rn(a, b); v[3] = __fsub_rn(a, b);
    }
    {   // stride 64: pairs (0,2) and (1,3)
        float a = v[0], b = v[2]; v[0] = __fadd_rn(a, b); v[2] = __fsub_rn(a, b);
        a = v[1]; b = v[3];       v[1] = __fadd_rn(a, b); v[3] = __fsub_rn(a, b);
    }
    const float scale = 0x1.6a09e6p-4f;  // RN32(1/sqrt(128))
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(v[j], scale);
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// RN16(RN32(x * f32(suh))) as a float holding the binary16 value.  The product is
// rounded to float32 first; converting the exact product straight to binary16 would
// round differently on ties (reference tests/test_numerics.py:46-54).
__device__ __forceinline__ __half scale_input(float x, uint16_t suh) {
    return __float2half_rn(__fmul_rn(x, half_bits_to_float(suh)));
}

// Element `index` of a tensor of `dtype` as float32 (exact widening), and the store of a
// float32 result into one (round to nearest even).
__device__ __forceinline__ float load_element(const void* base, int dtype, long long index) {
    if (dtype == DT_F32) return static_cast<const float*>(base)[index];
    const uint16_t bits = static_cast<const uint16_t*>(base)[index];
    return dtype == DT_F16 ? __half2float(__ushort_as_half(bits)) : __uint_as_float((uint32_t)bits << 16);
}
__device__ __forceinline__ void store_element(void* base, int dtype, long long index, float value) {
    if (dtype == DT_F32) static_cast<float*>(base)[index] = value;
    else if (dtype == DT_F16) static_cast<__half*>(base)[index] = __float2half_rn(value);
    else static_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(value);
}
// The tail of the output stages on a finished value: + bias was done by the caller; alpha, beta
// over the old element (never read when beta is zero of either sign), store.
__device__ __forceinline__ void scale_and_store(void* y, int dtype, long long index, float value, float alpha, float beta) {
    value = __fmul_rn(value, alpha);
    if (beta != 0.0f) value = __fadd_rn(value, __fmul_rn(beta, load_element(y, dtype, index)));
    store_element(y, dtype, index, value);
}

// alpha * (had * svh + bias) + beta * old, each step rounded on its own; beta == 0
// (either sign) never touches `old` (src/transforms.hpp:44-50).
__device__ __forceinline__ float finish_output(float had, uint16_t svh, const float* bias, int col,
                                               float alpha, float beta, const float* old_ptr) {
    float value = __fmul_rn(had, half_bits_to_float(svh));
    if (bias) value = __fadd_rn(value, bias[col]);
    value = __fmul_rn(value, alpha);
    if (beta != 0.0f) value = __fadd_rn(value, __fmul_rn(beta, *old_ptr));
    return value;
}

}  // namespace st
