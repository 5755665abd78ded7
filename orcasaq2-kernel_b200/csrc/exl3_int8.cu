// int8-packed embedding table and tied head: rows of int8 with one scale per row.
//
//   exl3_int8_embed   out[t][:] = dt(q[id_t][:]) * s[id_t]       (gather, scale on the gathered rows)
//   exl3_int8_head    logits[r][v] = s[v] * sum_h x[r][h] * q[v][h]
//
// The head never materialises the dequantised table: it streams the int8 rows once (HBM-bound,
// one byte per weight), turns bytes into fp16 with a byte permute and one exact subtraction, and
// contracts on the tensor cores with the vocabulary on the M side (16 rows per warp) and the
// batch rows on the N side.  Activations sit in shared memory for the whole (persistent) CTA.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "exl3_common.cuh"

namespace exl3 {

// ------------------------------------------------------------------------------------ gather
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, typename I>
__global__ void __launch_bounds__(256)
int8_embed_kernel(const int8_t *__restrict__ q, const T *__restrict__ s, const I *__restrict__ ids,
                  T *__restrict__ out, int vocab, int hidden, unsigned *__restrict__ bad) {
    const int t = blockIdx.x;
    long long id = (long long)ids[t];
    if (id < 0 || id >= vocab) {
        // out-of-range id: report through the optional flag and emit zeros, never read outside
        if (bad && threadIdx.x == 0) atomicOr(bad, 1u);
        for (int h = threadIdx.x * 16; h < hidden; h += blockDim.x * 16) {
            uint4 z = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(out + (size_t)t * hidden + h) = z;
            *reinterpret_cast<uint4 *>(out + (size_t)t * hidden + h + 8) = z;
        }
        return;
    }
    const float sc = to_float<T>(s[id]);
    const int8_t *row = q + (size_t)id * hidden;
    for (int h = threadIdx.x * 16; h < hidden; h += blockDim.x * 16) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(row + h));
        const int8_t *b = reinterpret_cast<const int8_t *>(&raw);
        __align__(16) T o[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) o[k] = from_float<T>((float)b[k] * sc);   // exact product, one rounding
        *reinterpret_cast<uint4 *>(out + (size_t)t * hidden + h) = *reinterpret_cast<uint4 *>(&o[0]);
        *reinterpret_cast<uint4 *>(out + (size_t)t * hidden + h + 8) = *reinterpret_cast<uint4 *>(&o[8]);
    }
}

// ------------------------------------------------------------------------------------ head
constexpr int kHeadWarps = 16;
constexpr int kHeadThreads = kHeadWarps * 32;
constexpr int kHeadPad = 8;          // halves of padding per staged activation row

__device__ __forceinline__ void mma16816h(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// four int8 (two's complement, packed in one word) -> two half2 holding the exact values
__device__ __forceinline__ void int8x4_to_half2x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;                       // bytes now hold q + 128
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(u), "r"(0x64646464u));   // 1024 + u0 | 1024 + u1
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(u), "r"(0x64646464u));   // 1024 + u2 | 1024 + u3
    const __half2 off = __half2half2(__ushort_as_half((unsigned short)0x6480));   // 1152
    const __half2 ra = __hsub2(*reinterpret_cast<__half2 *>(&a), off);
    const __half2 rb = __hsub2(*reinterpret_cast<__half2 *>(&b), off);
    lo = *reinterpret_cast<const uint32_t *>(&ra);
    hi = *reinterpret_cast<const uint32_t *>(&rb);
}

template <typename T, int NT>
__global__ void __launch_bounds__(kHeadThreads, 1)
int8_head_kernel(const int8_t *__restrict__ q, const T *__restrict__ s, const T *__restrict__ x,
                 T *__restrict__ out, int rows, int vocab, int hidden, long long ldo) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int pitch = hidden + kHeadPad;                        // halves
    __half *xs = reinterpret_cast<__half *>(smem_raw);          // [NT*8][pitch]
    float *rscale = reinterpret_cast<float *>(xs + (size_t)NT * 8 * pitch);   // [NT*8] undo factors

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;

    // ---- stage activations as fp16; bf16 rows are scaled by a power of two so their largest
    //      magnitude fits fp16 (exact for every value within 2^24 of the row maximum)
    for (int r = warp; r < NT * 8; r += kHeadWarps) {
        float inv = 1.f, undo = 1.f;
        if (r < rows && sizeof(T) == 2 && !std::is_same<T, __half>::value) {
            float m = 0.f;
            for (int h = lane; h < hidden; h += 32) m = fmaxf(m, fabsf(to_float<T>(x[(size_t)r * hidden + h])));
#pragma unroll
            for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            int e = 0;
            if (m > 16384.f && m < 3.0e38f) { frexpf(m, &e); e -= 14; }
            inv = ldexpf(1.f, -e);
            undo = ldexpf(1.f, e);
        }
        if (lane == 0) rscale[r] = undo;
        for (int h = lane; h < hidden; h += 32) {
            const float v = r < rows ? to_float<T>(x[(size_t)r * hidden + h]) * inv : 0.f;
            xs[(size_t)r * pitch + h] = __float2half_rn(v);
        }
    }
    __syncthreads();

    const int groups = (vocab + 15) >> 4;
    const int gstride = gridDim.x * kHeadWarps;
    for (int grp = blockIdx.x * kHeadWarps + warp; grp < groups; grp += gstride) {
        const int v0 = grp * 16;
        const int va = min(v0 + g, vocab - 1), vb = min(v0 + g + 8, vocab - 1);
        const int8_t *ra = q + (size_t)va * hidden + 16 * tig;
        const int8_t *rb = q + (size_t)vb * hidden + 16 * tig;
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

#pragma unroll 4
        for (int h0 = 0; h0 < hidden; h0 += 64) {
            const uint4 wa = __ldg(reinterpret_cast<const uint4 *>(ra + h0));
            const uint4 wb = __ldg(reinterpret_cast<const uint4 *>(rb + h0));
            const uint32_t aw[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t bw[4] = {wb.x, wb.y, wb.z, wb.w};
            uint4 xa[NT][2];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const __half *xr = xs + (size_t)(8 * t + g) * pitch + h0 + 16 * tig;
                xa[t][0] = *reinterpret_cast<const uint4 *>(xr);
                xa[t][1] = *reinterpret_cast<const uint4 *>(xr + 8);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a0, a2, a1, a3;
                int8x4_to_half2x2(aw[j], a0, a2);
                int8x4_to_half2x2(bw[j], a1, a3);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const uint32_t *xw = reinterpret_cast<const uint32_t *>(&xa[t][j >> 1]);
                    mma16816h(acc[t], a0, a1, a2, a3, xw[2 * (j & 1)], xw[2 * (j & 1) + 1]);
                }
            }
        }
        const float sa = to_float<T>(s[va]), sb = to_float<T>(s[vb]);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int n0 = 8 * t + 2 * tig;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = n0 + e;
                if (n < rows) {
                    const float un = rscale[n];
                    if (v0 + g < vocab) out[(size_t)n * ldo + v0 + g] = from_float<T>(acc[t][e] * sa * un);
                    if (v0 + g + 8 < vocab) out[(size_t)n * ldo + v0 + g + 8] = from_float<T>(acc[t][2 + e] * sb * un);
                }
            }
        }
    }
}

template <typename T>
static int launch_head(const void *q, const void *s, const void *x, void *out, int rows, int vocab, int hidden,
                       long long ldo, cudaStream_t st) {
    const int nt = rows > 8 ? 2 : 1;
    const size_t smem = (size_t)nt * 8 * (hidden + kHeadPad) * 2 + (size_t)nt * 8 * 4;
    if (smem > 220 * 1024) return EXL3_E_SHAPE;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int groups = (vocab + 15) / 16;
    int grid = (groups + kHeadWarps - 1) / kHeadWarps;
    if (grid > sms) grid = sms;
    cudaError_t e;
    if (nt == 1) {
        e = cudaFuncSetAttribute(int8_head_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
        int8_head_kernel<T, 1><<<grid, kHeadThreads, smem, st>>>(
            static_cast<const int8_t *>(q), static_cast<const T *>(s), static_cast<const T *>(x),
            static_cast<T *>(out), rows, vocab, hidden, ldo);
    } else {
        e = cudaFuncSetAttribute(int8_head_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
        int8_head_kernel<T, 2><<<grid, kHeadThreads, smem, st>>>(
            static_cast<const int8_t *>(q), static_cast<const T *>(s), static_cast<const T *>(x),
            static_cast<T *>(out), rows, vocab, hidden, ldo);
    }
    return launch_status();
}

// ------------------------------------------------------------------------------------ head, 17..64 rows
// More rows than the kernel above keeps resident: the table is still streamed ONCE per call.  A CTA takes 256
// vocabulary rows at a time (16 per warp, accumulators for all batch rows in registers) and walks the hidden
// dimension in chunks of 256; the activations of a chunk -- [rows][256] fp16, converted once -- are staged in
// shared memory for all sixteen warps (double-buffered: the next chunk is fetched from L2 into registers while
// this one is multiplied).  Per call the table crosses HBM once and the activations cross L2 -> SM once per 256
// vocabulary rows, i.e. about as many bytes as the table itself.
constexpr int kRowsChunk = 256;            // hidden channels per staged chunk
constexpr int kRowsPitch = kRowsChunk + 8; // halves per staged activation row (bank-conflict padding)

template <typename T, int NT>
__global__ void __launch_bounds__(kHeadThreads, 1)
int8_head_rows_kernel(const int8_t *__restrict__ q, const T *__restrict__ s, const T *__restrict__ x,
                      T *__restrict__ out, int rows, int vocab, int hidden, long long ldo) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kRowsPad = NT * 8;
    __half *xs = reinterpret_cast<__half *>(smem_raw);                            // [2][kRowsPad][kRowsPitch]
    float *rscale = reinterpret_cast<float *>(xs + 2 * kRowsPad * kRowsPitch);    // [kRowsPad] undo factors
    float *rinv = rscale + kRowsPad;                                              // [kRowsPad] scale factors
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;

    // power-of-two scale per bf16 row so that its largest magnitude fits fp16 (as in the resident kernel)
    for (int r = warp; r < kRowsPad; r += kHeadWarps) {
        float inv = 1.f, undo = 1.f;
        if (r < rows && sizeof(T) == 2 && !std::is_same<T, __half>::value) {
            float m = 0.f;
            for (int h = lane; h < hidden; h += 32) m = fmaxf(m, fabsf(to_float<T>(x[(size_t)r * hidden + h])));
#pragma unroll
            for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            int e = 0;
            if (m > 16384.f && m < 3.0e38f) { frexpf(m, &e); e -= 14; }
            inv = ldexpf(1.f, -e);
            undo = ldexpf(1.f, e);
        }
        if (lane == 0) { rscale[r] = undo; rinv[r] = inv; }
    }
    __syncthreads();

    // staging: a thread moves kPer pieces of eight values per chunk; piece p covers row p / 32, columns 8 * (p % 32)
    constexpr int kPieces = kRowsPad * (kRowsChunk / 8);
    constexpr int kPer = kPieces / kHeadThreads;
    static_assert(kPieces % kHeadThreads == 0, "chunk pieces divide among the threads");
    uint4 stage[kPer];
    auto fetch = [&](int h0) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int p = threadIdx.x + i * kHeadThreads;
            const int r = p >> 5, c = (p & 31) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(x + (size_t)r * hidden + h0 + c);
                if (std::is_same<T, __half>::value) v = raw;
                else {
                    const T *t8 = reinterpret_cast<const T *>(&raw);
                    const float inv = rinv[r];
                    __half2 *o = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = __floats2half2_rn(to_float<T>(t8[2 * k]) * inv, to_float<T>(t8[2 * k + 1]) * inv);
                }
            }
            stage[i] = v;
        }
    };
    auto put = [&](int buf) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int p = threadIdx.x + i * kHeadThreads;
            const int r = p >> 5, c = (p & 31) * 8;
            *reinterpret_cast<uint4 *>(xs + ((size_t)buf * kRowsPad + r) * kRowsPitch + c) = stage[i];
        }
    };

    const int nchunks = hidden / kRowsChunk;
    const int batches = (vocab + 16 * kHeadWarps - 1) / (16 * kHeadWarps);
    int buf = 0;
    for (int b = blockIdx.x; b < batches; b += gridDim.x) {
        const int v0 = (b * kHeadWarps + warp) * 16;
        const int va = min(v0 + g, vocab - 1), vb = min(v0 + g + 8, vocab - 1);
        const int8_t *ra = q + (size_t)va * hidden + 16 * tig;
        const int8_t *rb = q + (size_t)vb * hidden + 16 * tig;
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
        fetch(0);
        __syncthreads();                               // the previous batch's last chunk has been read
        put(buf);
        __syncthreads();
        for (int c = 0; c < nchunks; ++c) {
            const int h0 = c * kRowsChunk;
            // this chunk's table bytes (four 64-channel steps), all loads in flight at once
            uint4 wa[4], wb[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                wa[k] = __ldg(reinterpret_cast<const uint4 *>(ra + h0 + 64 * k));
                wb[k] = __ldg(reinterpret_cast<const uint4 *>(rb + h0 + 64 * k));
            }
            if (c + 1 < nchunks) fetch(h0 + kRowsChunk);
            const __half *xc = xs + (size_t)buf * kRowsPad * kRowsPitch;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t aw[4] = {wa[k].x, wa[k].y, wa[k].z, wa[k].w};
                const uint32_t bw[4] = {wb[k].x, wb[k].y, wb[k].z, wb[k].w};
                uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int8x4_to_half2x2(aw[j], a0[j], a2[j]);
                    int8x4_to_half2x2(bw[j], a1[j], a3[j]);
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const __half *xr = xc + (size_t)(8 * t + g) * kRowsPitch + 64 * k + 16 * tig;
                    const uint4 x0 = *reinterpret_cast<const uint4 *>(xr);
                    const uint4 x1 = *reinterpret_cast<const uint4 *>(xr + 8);
                    mma16816h(acc[t], a0[0], a1[0], a2[0], a3[0], x0.x, x0.y);
                    mma16816h(acc[t], a0[1], a1[1], a2[1], a3[1], x0.z, x0.w);
                    mma16816h(acc[t], a0[2], a1[2], a2[2], a3[2], x1.x, x1.y);
                    mma16816h(acc[t], a0[3], a1[3], a2[3], a3[3], x1.z, x1.w);
                }
            }
            if (c + 1 < nchunks) {
                put(buf ^ 1);                          // nobody reads that buffer: its last readers passed the barrier below
                __syncthreads();
                buf ^= 1;
            }
        }
        if (v0 < vocab) {
            const float sa = to_float<T>(s[va]), sb = to_float<T>(s[vb]);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int n0 = 8 * t + 2 * tig;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + e;
                    if (n < rows) {
                        const float un = rscale[n];
                        if (v0 + g < vocab) out[(size_t)n * ldo + v0 + g] = from_float<T>(acc[t][e] * sa * un);
                        if (v0 + g + 8 < vocab) out[(size_t)n * ldo + v0 + g + 8] = from_float<T>(acc[t][2 + e] * sb * un);
                    }
                }
            }
        }
    }
}

template <typename T, int NT>
static int launch_head_rows_nt(const void *q, const void *s, const void *x, void *out, int rows, int vocab, int hidden,
                               long long ldo, int sms, cudaStream_t st) {
    const size_t smem = (size_t)2 * NT * 8 * kRowsPitch * 2 + (size_t)2 * NT * 8 * 4;
    if (cudaFuncSetAttribute(int8_head_rows_kernel<T, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    const int batches = (vocab + 16 * kHeadWarps - 1) / (16 * kHeadWarps);
    const int grid = batches < sms ? batches : sms;
    int8_head_rows_kernel<T, NT><<<grid, kHeadThreads, smem, st>>>(
        static_cast<const int8_t *>(q), static_cast<const T *>(s), static_cast<const T *>(x), static_cast<T *>(out),
        rows, vocab, hidden, ldo);
    return launch_status();
}
template <typename T>
static int launch_head_rows(const void *q, const void *s, const void *x, void *out, int rows, int vocab, int hidden,
                            long long ldo, cudaStream_t st) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return rows <= 32 ? launch_head_rows_nt<T, 4>(q, s, x, out, rows, vocab, hidden, ldo, sms, st)
                      : launch_head_rows_nt<T, 8>(q, s, x, out, rows, vocab, hidden, ldo, sms, st);
}

}  // namespace exl3

extern "C" int exl3_int8_embed(const void *qweight, const void *scales, const void *ids, void *out, int tokens,
                               int vocab, int hidden, int is_bf16, int ids_are_i32, void *bad_id_flag,
                               void *stream) {
    using namespace exl3;
    if (!qweight || !scales || !ids || !out) return EXL3_E_NULL;
    if (tokens < 0 || vocab <= 0 || hidden <= 0 || (hidden & 15)) return EXL3_E_SHAPE;
    if (!aligned(qweight, 16) || !aligned(out, 16)) return EXL3_E_ALIGN;
    if (tokens == 0) return EXL3_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned *bad = static_cast<unsigned *>(bad_id_flag);
    const int8_t *q = static_cast<const int8_t *>(qweight);
#define EXL3_EMBED(T, I)                                                                            \
    int8_embed_kernel<T, I><<<tokens, 256, 0, st>>>(q, static_cast<const T *>(scales),              \
                                                    static_cast<const I *>(ids), static_cast<T *>(out), \
                                                    vocab, hidden, bad)
    if (is_bf16) {
        if (ids_are_i32) EXL3_EMBED(__nv_bfloat16, int); else EXL3_EMBED(__nv_bfloat16, long long);
    } else {
        if (ids_are_i32) EXL3_EMBED(__half, int); else EXL3_EMBED(__half, long long);
    }
#undef EXL3_EMBED
    return launch_status();
}

extern "C" int exl3_int8_head(const void *qweight, const void *scales, const void *x, void *logits, int rows,
                              int vocab, int hidden, long long ld_logits, int is_bf16, void *stream) {
    using namespace exl3;
    if (!qweight || !scales || !x || !logits) return EXL3_E_NULL;
    if (rows < 1 || rows > EXL3_INT8_HEAD_MAX_ROWS || vocab <= 0 || hidden <= 0 || (hidden & 63) || ld_logits < vocab)
        return EXL3_E_SHAPE;
    if (!aligned(qweight, 16)) return EXL3_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows > 16) {
        // the staged form: hidden in chunks of 256, activation rows read 16 bytes at a time
        if ((hidden & 255) || !aligned(x, 16)) return EXL3_E_SHAPE;
        return is_bf16 ? launch_head_rows<__nv_bfloat16>(qweight, scales, x, logits, rows, vocab, hidden, ld_logits, st)
                       : launch_head_rows<__half>(qweight, scales, x, logits, rows, vocab, hidden, ld_logits, st);
    }
    return is_bf16 ? launch_head<__nv_bfloat16>(qweight, scales, x, logits, rows, vocab, hidden, ld_logits, st)
                   : launch_head<__half>(qweight, scales, x, logits, rows, vocab, hidden, ld_logits, st);
}
