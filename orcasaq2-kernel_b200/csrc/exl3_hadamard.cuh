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

}  // namespace exl3
