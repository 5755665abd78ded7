// Standalone blockwise 128-Hadamard with optional elementwise pre-/post-scale vectors.
// One warp per (row, 128-block); fp16 in, fp32 butterflies, one rounding to fp16 on the way out.
#include "exl3_common.cuh"
#include "exl3_hadamard.cuh"

namespace exl3 {

constexpr int kHadWarps = 8;

__global__ void __launch_bounds__(kHadWarps * 32)
had_r_128_kernel(const __half *__restrict__ in, __half *__restrict__ out, const __half *__restrict__ pre,
                 const __half *__restrict__ post, float scale, long long nblocks, int blocks_per_row) {
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * kHadWarps + (threadIdx.x >> 5);
    if (wid >= nblocks) return;
    const int blk = (int)(wid % blocks_per_row);
    const size_t off = (size_t)wid * 128 + 4 * lane;  // rows are contiguous: row*n + blk*128
    const int col = blk * 128 + 4 * lane;

    const uint2 raw = *reinterpret_cast<const uint2 *>(in + off);
    const __half2 h01 = *reinterpret_cast<const __half2 *>(&raw.x);
    const __half2 h23 = *reinterpret_cast<const __half2 *>(&raw.y);
    float v[4] = {__low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23)};
    if (pre) {
        const uint2 p = *reinterpret_cast<const uint2 *>(pre + col);
        const __half2 p01 = *reinterpret_cast<const __half2 *>(&p.x);
        const __half2 p23 = *reinterpret_cast<const __half2 *>(&p.y);
        v[0] *= __low2float(p01);
        v[1] *= __high2float(p01);
        v[2] *= __low2float(p23);
        v[3] *= __high2float(p23);
    }
    fwht128_warp(v, lane);
    const float s = kHadScale * scale;
    float q[4] = {1.f, 1.f, 1.f, 1.f};
    if (post) {
        const uint2 p = *reinterpret_cast<const uint2 *>(post + col);
        const __half2 p01 = *reinterpret_cast<const __half2 *>(&p.x);
        const __half2 p23 = *reinterpret_cast<const __half2 *>(&p.y);
        q[0] = __low2float(p01);
        q[1] = __high2float(p01);
        q[2] = __low2float(p23);
        q[3] = __high2float(p23);
    }
    const __half2 o01 = __floats2half2_rn(v[0] * s * q[0], v[1] * s * q[1]);
    const __half2 o23 = __floats2half2_rn(v[2] * s * q[2], v[3] * s * q[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&o01);
    o.y = *reinterpret_cast<const uint32_t *>(&o23);
    *reinterpret_cast<uint2 *>(out + off) = o;
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
    const long long grid = (nblocks + kHadWarps - 1) / kHadWarps;
    if (grid > 0x7fffffffLL) return EXL3_E_SHAPE;
    had_r_128_kernel<<<(unsigned)grid, kHadWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half *>(in), static_cast<__half *>(out), static_cast<const __half *>(pre),
        static_cast<const __half *>(post), scale, nblocks, bpr);
    return launch_status();
}
