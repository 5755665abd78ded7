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

// PRE / POST: whether the scale vectors exist (a missing one costs no loads, conversions or multiplies)
template <bool PRE, bool POST>
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
    // one division per warp (32-bit when the block count allows): 64-bit remainders per block were a visible share
    // of this kernel's instructions
    const unsigned bpr = (unsigned)blocks_per_row;
    const unsigned blk0 = nblocks <= 0x7fffffffLL ? (unsigned)wid0 % bpr : (unsigned)(wid0 % blocks_per_row);
    float sgn[5];
    fwht128_signs(lane, sgn);
#pragma unroll
    for (int u = 0; u < kHadUnroll; ++u) {
        const long long wid = wid0 + u;
        const bool live = wid < nblocks;
        unsigned b = blk0 + u;
        while (b >= bpr) b -= bpr;
        const int col = (int)b * 128 + 4 * lane;
        raw[u] = live ? *reinterpret_cast<const uint2 *>(in + (size_t)wid * 128 + 4 * lane) : make_uint2(0u, 0u);
        if (PRE) pr[u] = *reinterpret_cast<const uint2 *>(pre + col);
        if (POST) po[u] = *reinterpret_cast<const uint2 *>(post + col);
    }
    const float s = kHadScale * scale;
#pragma unroll
    for (int u = 0; u < kHadUnroll; ++u) {
        if (wid0 + u >= nblocks) break;
        float v[4];
        unpack4(raw[u], v);
        if (PRE) {
            float p[4];
            unpack4(pr[u], p);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] *= p[k];
        }
        fwht128_warp_signed(v, sgn);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] *= s;
        if (POST) {
            float q[4];
            unpack4(po[u], q);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] *= q[k];
        }
        const __half2 o01 = __floats2half2_rn(v[0], v[1]);
        const __half2 o23 = __floats2half2_rn(v[2], v[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t *>(&o01);
        o.y = *reinterpret_cast<const uint32_t *>(&o23);
        *reinterpret_cast<uint2 *>(out + (size_t)(wid0 + u) * 128 + 4 * lane) = o;
    }
}

// The same transform with sixteen values per lane (eight lanes per 128-block, four blocks per warp as above): four
// butterfly stages stay in registers and only three cross lanes, 12 shuffles per block instead of 20 -- the shuffles
// share the load/store pipe with the memory traffic and were what bound the kernel above -- and a lane moves 32
// contiguous bytes.  Same stage order, hence the same bits.  Needs 16-byte aligned pointers.
__device__ __forceinline__ void unpack8(const uint4 &r, float *v) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __low2float(h[i]);
        v[2 * i + 1] = __high2float(h[i]);
    }
}
template <bool PRE, bool POST>
__global__ void __launch_bounds__(kHadWarps * 32)
had_r_128_wide_kernel(const __half *__restrict__ in, __half *__restrict__ out, const __half *__restrict__ pre,
                      const __half *__restrict__ post, float scale, long long nblocks, int blocks_per_row) {
    const int lane = threadIdx.x & 31, sub = lane & 7;
    const long long wid0 = ((long long)blockIdx.x * kHadWarps + (threadIdx.x >> 5)) * kHadUnroll;
    if (wid0 >= nblocks) return;
    const long long wid = wid0 + (lane >> 3);                       // this lane's block; in place is fine as above
    const bool live = wid < nblocks;
    unsigned blk = 0;
    if (live) blk = nblocks <= 0x7fffffffLL ? (unsigned)wid % (unsigned)blocks_per_row : (unsigned)(wid % blocks_per_row);
    uint4 r0 = make_uint4(0u, 0u, 0u, 0u), r1 = r0, p0 = r0, p1 = r0, q0 = r0, q1 = r0;
    if (live) {
        const uint4 *src = reinterpret_cast<const uint4 *>(in + (size_t)wid * 128 + 16 * sub);
        r0 = src[0];
        r1 = src[1];
        if (PRE) {
            const uint4 *ps = reinterpret_cast<const uint4 *>(pre + (size_t)blk * 128 + 16 * sub);
            p0 = ps[0];
            p1 = ps[1];
        }
        if (POST) {
            const uint4 *qs = reinterpret_cast<const uint4 *>(post + (size_t)blk * 128 + 16 * sub);
            q0 = qs[0];
            q1 = qs[1];
        }
    }
    float v[16];
    unpack8(r0, v);
    unpack8(r1, v + 8);
    if (PRE) {
        float p[16];
        unpack8(p0, p);
        unpack8(p1, p + 8);
#pragma unroll
        for (int k = 0; k < 16; ++k) v[k] *= p[k];
    }
#pragma unroll
    for (int h = 1; h < 16; h <<= 1)
#pragma unroll
        for (int e = 0; e < 16; ++e)
            if ((e & h) == 0) {
                const float a = v[e], b = v[e + h];
                v[e] = a + b;
                v[e + h] = a - b;
            }
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const float sg = ((lane >> i) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float other = __shfl_xor_sync(0xffffffffu, v[k], 1 << i);
            v[k] = fmaf(v[k], sg, other);
        }
    }
    const float s = kHadScale * scale;
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] *= s;
    if (POST) {
        float q[16];
        unpack8(q0, q);
        unpack8(q1, q + 8);
#pragma unroll
        for (int k = 0; k < 16; ++k) v[k] *= q[k];
    }
    if (live) {
        uint4 o[2];
        uint32_t *ow = reinterpret_cast<uint32_t *>(o);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const __half2 hv = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
            ow[k] = *reinterpret_cast<const uint32_t *>(&hv);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)wid * 128 + 16 * sub);
        dst[0] = o[0];
        dst[1] = o[1];
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
    const __half *i16 = static_cast<const __half *>(in), *pre16 = static_cast<const __half *>(pre), *post16 = static_cast<const __half *>(post);
    __half *o16 = static_cast<__half *>(out);
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = (unsigned)grid, t = kHadWarps * 32;
    const bool wide = aligned(in, 16) && aligned(out, 16) && (!pre || aligned(pre, 16)) && (!post || aligned(post, 16));
    if (wide) {
        if (pre && post) had_r_128_wide_kernel<true, true><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
        else if (pre) had_r_128_wide_kernel<true, false><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
        else if (post) had_r_128_wide_kernel<false, true><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
        else had_r_128_wide_kernel<false, false><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
        return launch_status();
    }
    if (pre && post) had_r_128_kernel<true, true><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
    else if (pre) had_r_128_kernel<true, false><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
    else if (post) had_r_128_kernel<false, true><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
    else had_r_128_kernel<false, false><<<g, t, 0, st>>>(i16, o16, pre16, post16, scale, nblocks, bpr);
    return launch_status();
}
