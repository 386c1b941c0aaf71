// H128 and the input/output stage arithmetic of the staged float32 contract
// (reference python/strix_trellis/linear.py:82-163, src/hadamard.hpp:17-37,
// src/transforms.hpp:8-52).  Every operation that the contract rounds separately
// is written with a non-contractable intrinsic (__fmul_rn/__fadd_rn/__fsub_rn), so
// the result does not depend on -fmad.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

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
