// 128-point Walsh-Hadamard transform (Sylvester order) held by one warp: lane l owns elements
// 4l .. 4l+3.  Two butterfly stages run in registers, five across lanes with shuffles.
// The 1/sqrt(128) normalisation is left to the caller.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace exl3 {

constexpr float kHadScale = 0.08838834764831845f;  // 1/sqrt(128)

__device__ __forceinline__ void fwht128_warp(float (&v)[4], int lane) {
    {
        const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
        v[0] = a0 + a2;
        v[1] = a1 + a3;
        v[2] = a0 - a2;
        v[3] = a1 - a3;
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool upper = lane & m;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float other = __shfl_xor_sync(0xffffffffu, v[k], m);
            v[k] = upper ? other - v[k] : v[k] + other;
        }
    }
}

// The same butterflies for kernels that do little else: the lane's sign of every shuffle stage is computed once
// (sgn[i] = -1 when bit i of the lane is set), which makes a stage one shuffle and one fused multiply-add per value.
// Bitwise the same results: a product with +-1 is exact.
__device__ __forceinline__ void fwht128_signs(int lane, float (&sgn)[5]) {
#pragma unroll
    for (int i = 0; i < 5; ++i) sgn[i] = ((lane >> i) & 1) ? -1.f : 1.f;
}
__device__ __forceinline__ void fwht128_warp_signed(float (&v)[4], const float (&sgn)[5]) {
    {
        const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
        v[0] = a0 + a2;
        v[1] = a1 + a3;
        v[2] = a0 - a2;
        v[3] = a1 - a3;
    }
#pragma unroll
    for (int i = 0; i < 5; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float other = __shfl_xor_sync(0xffffffffu, v[k], 1 << i);
            v[k] = fmaf(v[k], sgn[i], other);
        }
}

}  // namespace exl3
