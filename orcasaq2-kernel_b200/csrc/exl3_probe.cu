// Measurement probe, not part of the layer's path: how fast can one GPU decode the 3INST codebook at all?
//
// exl3_probe_decode_rate runs the SAME decode routines the kernels use (exl3_decode_fast.cuh) on words that never
// leave registers and feeds the codewords to mma.sync exactly as the fused GEMV does, on every SM with sixteen
// warps each, and reports the time.  No global or shared memory traffic is involved (mode 0), so the result is
// the ceiling that the integer decode and the legacy tensor-core path set for any kernel of this design, whatever
// its memory system does.  Mode 1 adds what a streaming loop cannot avoid: the packed words come from a
// shared-memory ring that 1-D bulk async copies refill (from a small L2-resident buffer), with the mbarrier wait,
// the neighbour shuffle and the activation-fragment load of the real loop.  kernel_bench.py prints both as
// weights per second; bench.py quotes mode 0 per bitrate beside the GEMV's achieved rate.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "exl3_codec.cuh"
#include "exl3_common.cuh"
#include "exl3_decode_fast.cuh"

namespace exl3 {
namespace probe {

constexpr int kWarps = 16, kDepth = 4;

__device__ __forceinline__ uint32_t s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mma(float (&d)[4], const uint32_t *a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
template <int K>
__device__ __forceinline__ void consume(const uint32_t (&w)[K + 1], float (&acc)[4][4], uint4 xa, const DecodeConsts &dc) {
    uint32_t z[32];
    decode_chunk_fast<K>(w, z, dc);
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int a = 0; a < 4; ++a) mma(acc[a], &z[8 * a + 4 * b], b ? xa.z : xa.x, b ? xa.w : xa.y);
}

template <int K, int MODE>
__global__ void __launch_bounds__(kWarps * 32, 1) rate_kernel(int iters, float *sink, uint32_t one, const unsigned char *src_base,
                                                              unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kSlot = (256 * K + 127) & ~127;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    unsigned char *ring = smem + 1024 + warp * kDepth * kSlot;
    uint32_t *xf = reinterpret_cast<uint32_t *>(smem + 1024 + kWarps * kDepth * kSlot);
    const uint32_t bar0 = s32(bars + warp * kDepth), ring0 = s32(ring);
    float acc[2][4][4] = {};
    const DecodeConsts dc(one);
    uint32_t wa[K + 1], wb[K + 1];
#pragma unroll
    for (int k = 0; k <= K; ++k) { wa[k] = threadIdx.x * 2654435761u + k * 40503u + blockIdx.x; wb[k] = wa[k] * 3u + 1u; }
    uint4 xa = make_uint4(0x3c003c00u * one, 0x3c003c00u * one, 0x3c003c00u * one, 0x3c003c00u * one);
    const unsigned char *src = src_base + (size_t)((blockIdx.x * kWarps + warp) & 255) * 4096;
    if (MODE == 1) {
        for (int i = threadIdx.x; i < (kWarps * kDepth * kSlot + 4096) / 4; i += kWarps * 32)
            reinterpret_cast<uint32_t *>(smem + 1024)[i] = i * 2654435761u;
        if (lane == 0) {
            for (int s = 0; s < kDepth; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8 * s), "r"(1));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
        if (lane == 0)
            for (int s = 0; s < kDepth; ++s) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar0 + 8 * s), "r"(256 * K) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(ring0 + s * kSlot), "l"(src), "r"(256 * K), "r"(bar0 + 8 * s) : "memory");
            }
    }
    const int nxt = (lane & 24) | ((lane + 1) & 7);
    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
        if (MODE == 1) {
            bool d = false;
            for (int p = 0; p < (1 << 20) && !d; ++p) d = try_wait(bar0 + 8 * slot, phase);
            ok = __all_sync(0xffffffffu, d);
            if (!ok) { if (lane == 0) atomicOr(status, 1u); break; }
            const uint32_t *stage = reinterpret_cast<const uint32_t *>(ring + slot * kSlot);
            load_words<K>(stage + lane * K, wa);
            load_words<K>(stage + 32 * K + lane * K, wb);
            xa = *reinterpret_cast<const uint4 *>(xf + ((it & 63) * 16) + (lane & 3) * 4);
            wa[K] = __shfl_sync(0xffffffffu, wa[0], nxt);
            wb[K] = __shfl_sync(0xffffffffu, wb[0], nxt);
        } else {
#pragma unroll
            for (int k = 0; k <= K; ++k) { wa[k] += 0x9e3779b9u * one; wb[k] += 0x7f4a7c15u * one; }
        }
        consume<K>(wa, acc[0], xa, dc);
        if (MODE == 1) {
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar0 + 8 * slot), "r"(256 * K) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(ring0 + slot * kSlot), "l"(src + (it & 3) * 1024), "r"(256 * K), "r"(bar0 + 8 * slot) : "memory");
            }
        }
        consume<K>(wb, acc[1], xa, dc);
        if (++slot == kDepth) { slot = 0; phase ^= 1u; }
    }
    if (MODE == 1) {     // the copies still in flight land before the CTA goes away (bounded)
        for (int s = 0; s < kDepth; ++s) {
            bool d = false;
            for (int p = 0; p < (1 << 20) && !d; ++p) d = try_wait(bar0 + 8 * s, s < slot ? phase ^ 1u : phase);
        }
    }
    float s = 0.f;
    for (int h = 0; h < 2; ++h)
        for (int a = 0; a < 4; ++a)
            for (int e = 0; e < 4; ++e) s += acc[h][a][e];
    if (s == 1.2345f) sink[0] = s;      // keeps the arithmetic alive
}

template <int K>
static int run(int mode, int iters, int sms, float *sink, const unsigned char *src, unsigned *status, cudaStream_t st) {
    constexpr int kSlot = (256 * K + 127) & ~127;
    const size_t smem = 1024 + (size_t)kWarps * kDepth * kSlot + 4096;
    if (mode == 0) {
        rate_kernel<K, 0><<<sms, kWarps * 32, 0, st>>>(iters, sink, 1u, src, status);
    } else {
        if (cudaFuncSetAttribute(rate_kernel<K, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return EXL3_E_LAUNCH;
        }
        rate_kernel<K, 1><<<sms, kWarps * 32, smem, st>>>(iters, sink, 1u, src, status);
    }
    return launch_status();
}

}  // namespace probe
}  // namespace exl3

extern "C" int exl3_probe_decode_rate(int k, int mode, int iters, void *scratch, size_t scratch_bytes, double *weights_out,
                                      void *stream) {
    using namespace exl3::probe;
    if (k < 1 || k > 8 || mode < 0 || mode > 1 || iters < 1 || iters > (1 << 20)) return EXL3_E_SHAPE;
    if (!scratch || !weights_out) return EXL3_E_NULL;
    if (scratch_bytes < (size_t)(1 << 20) + 8192 + 256 || !exl3::aligned(scratch, 256)) return EXL3_E_WORKSPACE;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    unsigned char *base = static_cast<unsigned char *>(scratch);
    unsigned *status = reinterpret_cast<unsigned *>(base);
    float *sink = reinterpret_cast<float *>(base + 64);
    const unsigned char *src = base + 256;                   // 1 MiB + 8 KiB of anything: the copies' source
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    *weights_out = (double)sms * kWarps * 32 * 64.0 * iters;
    switch (k) {
        case 1: return run<1>(mode, iters, sms, sink, src, status, st);
        case 2: return run<2>(mode, iters, sms, sink, src, status, st);
        case 3: return run<3>(mode, iters, sms, sink, src, status, st);
        case 4: return run<4>(mode, iters, sms, sink, src, status, st);
        case 5: return run<5>(mode, iters, sms, sink, src, status, st);
        case 6: return run<6>(mode, iters, sms, sink, src, status, st);
        case 7: return run<7>(mode, iters, sms, sink, src, status, st);
        default: return run<8>(mode, iters, sms, sink, src, status, st);
    }
}
