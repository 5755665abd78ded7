// Standalone blockwise 128-Hadamard with optional elementwise pre-/post-scale vectors.
// One warp per four consecutive (row, 128-block)s; fp16 in, fp32 butterflies, one rounding to fp16 on the way out.
#include "exl3_common.cuh"
#include "exl3_hadamard.cuh"

namespace exl3 {

constexpr int kHadWarps = 8;
constexpr int kHadUnroll = 4;      // 128-blocks per warp, all loads issued before the first butterfly

__device__ __forceinline__ void unpack4(const uint2 &r, float (&v)[4]) {
    const __half2 a = *reinterpret_cast<const __half2 *>(&r.x), b = *reinterpret_cast<const __half2 *>(&r.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

__global__ void __launch_bounds__(kHadWarps * 32)
had_r_128_kernel(const __half *__restrict__ in, __half *__restrict__ out, const __half *__restrict__ pre,
                 const __half *__restrict__ post, float scale, long long nblocks, int blocks_per_row) {
    const int lane = threadIdx.x & 31;
    const long long wid0 = ((long long)blockIdx.x * kHadWarps + (threadIdx.x >> 5)) * kHadUnroll;
    if (wid0 >= nblocks) return;
    // The kernel moves 4 bytes per element and does almost nothing else: what matters is how many loads a warp has
    // in flight.  (One block per warp: 2.8 TB/s on B200; four: see the profile notes.)  In place is fine: a warp
    // reads all of its blocks before it writes any of them.
    uint2 raw[kHadUnroll], pr[kHadUnroll], po[kHadUnroll];
    const uint2 ones = make_uint2(0x3C003C00u, 0x3C003C00u);
#pragma unroll
    for (int u = 0; u < kHadUnroll; ++u) {
        const long long wid = wid0 + u;
        const bool live = wid < nblocks;
        const int col = (int)((live ? wid : wid0) % blocks_per_row) * 128 + 4 * lane;
        raw[u] = live ? *reinterpret_cast<const uint2 *>(in + (size_t)wid * 128 + 4 * lane) : make_uint2(0u, 0u);
        pr[u] = pre ? *reinterpret_cast<const uint2 *>(pre + col) : ones;
        po[u] = post ? *reinterpret_cast<const uint2 *>(post + col) : ones;
    }
    const float s = kHadScale * scale;
#pragma unroll
    for (int u = 0; u < kHadUnroll; ++u) {
        if (wid0 + u >= nblocks) break;
        float v[4], p[4], q[4];
        unpack4(raw[u], v);
        unpack4(pr[u], p);
        unpack4(po[u], q);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] *= p[k];
        fwht128_warp(v, lane);
        const __half2 o01 = __floats2half2_rn(v[0] * s * q[0], v[1] * s * q[1]);
        const __half2 o23 = __floats2half2_rn(v[2] * s * q[2], v[3] * s * q[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t *>(&o01);
        o.y = *reinterpret_cast<const uint32_t *>(&o23);
        *reinterpret_cast<uint2 *>(out + (size_t)(wid0 + u) * 128 + 4 * lane) = o;
    }
}

}  // namespace exl3

extern "C" int exl3_had_r_128(const void *in, void *out, const void *pre, const void *post, float scale,
                              int rows, int n, void *stream) {
    using namespace exl3;
    if (!in || !out) return EXL3_E_NULL;
    if (rows < 0 || n <= 0 || (n & 127)) return EXL3_E_SHAPE;
    if (!aligned(in, 8) || !aligned(out, 8) || (pre && !aligned(pre, 8)) || (post && !aligned(post, 8)))
        return EXL3_E_ALIGN;
    if (rows == 0) return EXL3_OK;
    const int bpr = n / 128;
    const long long nblocks = (long long)rows * bpr;
    const long long grid = (nblocks + kHadWarps * kHadUnroll - 1) / (kHadWarps * kHadUnroll);
    if (grid > 0x7fffffffLL) return EXL3_E_SHAPE;
    had_r_128_kernel<<<(unsigned)grid, kHadWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half *>(in), static_cast<__half *>(out), static_cast<const __half *>(pre),
        static_cast<const __half *>(post), scale, nblocks, bpr);
    return launch_status();
}
