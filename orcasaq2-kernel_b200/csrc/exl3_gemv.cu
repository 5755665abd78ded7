// Fused trellis-decode GEMV for 1..16 rows, grouped over the shards of a fused layer:
//     y[:, out_col : out_col+oc] = H128( H128(x * suh) . W(trellis) ) * svh
// in two launches (activation pre-pass, GEMV), with no intermediate tensor in global memory except the rotated
// activations.
//
// Work unit: one 128-wide block of output channels (the width of the output Hadamard) times one
// slice of the input channels.  A CTA of eight warps owns one unit:
//   prologue  H128(x*suh) for its input slice is computed with warp shuffles and left in
//             shared memory in mma B-fragment order; meanwhile the first trellis stages are
//             already in flight.
//   main loop each warp streams [4 tiles x 32K bytes] pieces of the packed trellis with 1-D bulk
//             async copies (TMA) into its private shared-memory ring (mbarrier completion, no
//             block-wide synchronisation), decodes 32 weights per lane in registers and feeds
//             the raw codewords to mma.m16n8k16: a codeword's two fp16 halves occupy two
//             consecutive K slots that see the same activation, so their sum -- the weight --
//             is formed inside the fp32 accumulator and never rounded to fp16.
//   epilogue  warps are reduced through shared memory; the slices of a unit are the CTAs of one thread-block
//             cluster and are reduced through distributed shared memory into the cluster's first CTA, which adds
//             them in slice order (bitwise reproducible), applies H128 and svh and writes fp16.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "exl3_codec.cuh"
#include "exl3_common.cuh"
#include "exl3_decode_fast.cuh"
#include "exl3_hadamard.cuh"

namespace exl3 {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
// Ring slots per warp.  About 48-64 KB of trellis in flight per SM keeps HBM busy; measured on
// B200, deeper rings LOSE bandwidth again (1 KB pieces: 7.2 TB/s at depth 4, 3.0 TB/s at depth 8).
__host__ __device__ constexpr int ring_depth(int K) { return K <= 4 ? 4 : 3; }
constexpr int kTargetCtas = 296;       // two resident CTAs on each of 148 SMs
constexpr int kMaxSplitK = 8;          // slices of a unit = CTAs of one cluster (portable cluster size)
constexpr int kCtaSmemBytes = 112 * 1024;   // dynamic shared memory of one CTA (two CTAs per SM)
constexpr int kBarBytes = 1024;
constexpr int kSpinLimit = 1 << 22;
constexpr unsigned kStatusTimeout = 1u;

// Workspace layout: [status word, 256 B][rotated activations of every shard].
constexpr int kWsStatusBytes = 256;
constexpr int kWsMaxUnits = 8192;                 // 128-column blocks per launch (oc total <= 1M)
constexpr size_t kWsHeadBytes = kWsStatusBytes;

struct GemvShardDev {
    const uint32_t *trellis;
    const __half *suh;
    const __half *svh;
    long long xf_off;       // in 32-bit words, into the fragment scratch
    int tiles_j;            // oc / 16
    int K;
    int out_col;
    int cta_begin;
    int splitk;
    int unit_begin;
};

struct GemvParams {
    const __half *x;
    __half *y;
    const __half *residual;   // optional [rows][ld_res], added to the result before the final rounding
    const __half *norm_w;     // RMSNorm weight [ic] (in_mode 1), may be null for all ones
    float eps;
    int in_mode;              // 0 plain, 1 RMSNorm of x, 2 silu(x[:, :ic]) * x[:, ic:]
    int ldx, ld_res;
    uint32_t *xfg;          // rotated activations in B-fragment order, per shard
    unsigned *status;
    int rows, ic, ldy, kblocks;
    int nb;         // rows held per group of eight (1, 2, 4 or 8)
    int xf_bytes;   // bytes reserved for activation fragments
    int xf_blocks;  // 128-blocks of fragments those bytes hold
    uint32_t one;   // the value 1, opaque to the compiler (keeps multiplies on the multiply pipe)
    int nshards;
    GemvShardDev sh[EXL3_MAX_SHARDS];
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait, the same answer in every lane of the warp: gives up after `limit` polls and reports through
// the status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned *status, int limit = kSpinLimit) {
    bool done = false;
    for (int it = 0; it < limit && !done; ++it) done = mbar_try_wait(bar, parity);
    done = __all_sync(0xffffffffu, done);
    if (!done && (threadIdx.x & 31) == 0) atomicOr(status, kStatusTimeout);
    return done;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t *a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// all threads of all CTAs of the cluster
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// The 32 codewords of one chunk (four tiles' worth of one lane) times the activations: acc[t][h][a] += ...
template <int K, int NT>
__device__ __forceinline__ void consume_chunk(const uint32_t (&w)[K + 1], float (&acc)[NT][2][4][4], const int h,
                                              const uint4 (&xa)[NT], const DecodeConsts &dc) {
    uint32_t z[32];
    if constexpr (K == 1) {
        decode_chunk_fast<K>(w, z, dc);
#pragma unroll
        for (int bsel = 0; bsel < 2; ++bsel)
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    mma16816(acc[t][h][a], &z[8 * a + 4 * bsel], bsel ? xa[t].z : xa[t].x, bsel ? xa[t].w : xa[t].y);
    } else {
        uint32_t v[K];
        shifted_words<K>(w, v);
        decode_range_fast<K, 0, 16>(w, v, z, dc);
#pragma unroll
        for (int bsel = 0; bsel < 2; ++bsel)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    mma16816(acc[t][h][a], &z[8 * a + 4 * bsel], bsel ? xa[t].z : xa[t].x, bsel ? xa[t].w : xa[t].y);
        decode_range_fast<K, 16, 32>(w, v, z, dc);
#pragma unroll
        for (int bsel = 0; bsel < 2; ++bsel)
#pragma unroll
            for (int a = 2; a < 4; ++a)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    mma16816(acc[t][h][a], &z[8 * a + 4 * bsel], bsel ? xa[t].z : xa[t].x, bsel ? xa[t].w : xa[t].y);
    }
}

// ---------------------------------------------------------------------------------------------
template <int K, int NT>
__device__ __forceinline__ void gemv_cta(const GemvParams &P, const GemvShardDev &S, int local,
                                         unsigned char *smem) {
    constexpr int kDepth = ring_depth(K);
    constexpr int kHalfWords = 4 * 8 * K;            // four tiles
    constexpr int kStageWords = 2 * kHalfWords;      // one tile row of the 128-column block
    constexpr uint32_t kStageBytes = kStageWords * 4;
    // More than eight rows: the activation fragments of a step (1 KB per warp) no longer fit in shared memory for a
    // whole slice, so they ride in the warp's own ring behind the packed words of the same step (a second bulk copy
    // on the same barrier) instead of being fetched for the whole CTA in batches that every warp has to wait for.
    constexpr bool kStreamX = NT == 2;
    constexpr int kFragWords = kStreamX ? NT * 8 * 16 : 0;
    constexpr uint32_t kFragBytes = kFragWords * 4;
    constexpr int kSlotWords = kStageWords + kFragWords;
    constexpr uint32_t kSlotBytes = kSlotWords * 4;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int NB = P.nb;
    const DecodeConsts dc(P.one);

    const int ob = local / S.splitk, ks = local - ob * S.splitk;
    const int kb0 = (int)((long long)ks * P.kblocks / S.splitk);
    const int kb1 = (int)((long long)(ks + 1) * P.kblocks / S.splitk);
    const int nblk = kb1 - kb0;                      // = steps per warp (one tile of each block)

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    uint32_t *xf = reinterpret_cast<uint32_t *>(smem + kBarBytes);
    unsigned char *region = smem + kBarBytes + P.xf_bytes;
    uint32_t *ring = reinterpret_cast<uint32_t *>(region) + warp * (kDepth * kSlotWords);
    const uint32_t bar0 = smem_u32(bars + warp * 8);
    const uint32_t ring0 = smem_u32(ring);

    const uint32_t xbar = smem_u32(bars + kWarps * 8);      // CTA-wide: activation fragments landed
    uint32_t xphase = 0;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kDepth; ++s) mbar_init(bar0 + 8 * s, 1);
        if (warp == 0) mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // warp w owns tile rows kb0*8 + w + 8*s of the 128-column block ob
    const uint32_t *src0 = S.trellis + ((size_t)(kb0 * 8 + warp) * S.tiles_j + (size_t)ob * 8) * (size_t)(8 * K);
    const size_t src_step = (size_t)8 * S.tiles_j * (8 * K);
    if (lane == 0) {
        const int pre = nblk < kDepth ? nblk : kDepth;
        for (int s = 0; s < pre; ++s) {
            mbar_expect_tx(bar0 + 8 * s, kStageBytes + kFragBytes);   // the fragments follow after the dependency wait
            bulk_g2s(ring0 + s * kSlotBytes, src0 + s * src_step, kStageBytes, bar0 + 8 * s);
        }
    }

    float acc[NT][2][4][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[t][h][a][e] = 0.f;

    const int nrow = NT * NB;
    const int xf_tile_words = nrow * 16;             // words of fragments per tile
    const uint32_t *xf_lane = xf + ((g & (NB - 1)) * 4 + q) * 4 + warp * xf_tile_words;
    const int nxt_lane = (lane & 24) | ((lane + 1) & 7);
    const int sub_max = kStreamX ? nblk : P.xf_blocks;   // blocks of fragments that fit at once
    // streamed fragments: this warp's tile of block kb0 + s
    const uint32_t *xsrc0 = P.xfg + S.xf_off + ((size_t)kb0 * 8 + warp) * xf_tile_words;
    const size_t xsrc_step = (size_t)8 * xf_tile_words;
    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;

    // Programmatic dependent launch: everything above touched only constants (the trellis stream
    // and its barriers).  From here on the kernel reads the activations, which the previous grid
    // on the stream may still be writing, and later the shared scratch: wait for that grid to
    // finish, and let the grid after this one begin its own weight prefetch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    if (kStreamX && lane == 0) {
        const int pre = nblk < kDepth ? nblk : kDepth;
        for (int s = 0; s < pre; ++s)
            bulk_g2s(ring0 + s * kSlotBytes + kStageBytes, xsrc0 + s * xsrc_step, kFragBytes, bar0 + 8 * s);
    }

    for (int b0 = 0; b0 < nblk; b0 += sub_max) {
        const int nb_sub = min(sub_max, nblk - b0);
        if constexpr (!kStreamX) {
            if (b0) __syncthreads();                 // the previous fragments are no longer read
            // ---- rotated activations of these blocks: one bulk copy from the fragment scratch
            if (tid == 0) {
                const uint32_t bytes = (uint32_t)nb_sub * 8u * (uint32_t)xf_tile_words * 4u;
                mbar_expect_tx(xbar, bytes);
                bulk_g2s(smem_u32(xf), P.xfg + S.xf_off + (size_t)(kb0 + b0) * 8 * xf_tile_words, bytes, xbar);
            }
            ok = mbar_wait(xbar, xphase, P.status) && ok;
            xphase ^= 1u;
        }

        // ---- stream, decode, multiply
        const uint32_t *xfp = xf_lane;
        for (int s = b0; s < b0 + nb_sub && ok; ++s) {
            ok = mbar_wait(bar0 + 8 * slot, phase, P.status);
            const uint32_t *stage = ring + slot * kSlotWords + lane * K;
            uint32_t wa[K + 1], wb[K + 1];
            load_words<K>(stage, wa);
            load_words<K>(stage + kHalfWords, wb);
            uint4 xa[NT];
            if constexpr (kStreamX) {
                const uint32_t *xs = ring + slot * kSlotWords + kStageWords + (g * 4 + q) * 4;
#pragma unroll
                for (int t = 0; t < NT; ++t) xa[t] = *reinterpret_cast<const uint4 *>(xs + t * 8 * 16);
            } else {
#pragma unroll
                for (int t = 0; t < NT; ++t) xa[t] = *reinterpret_cast<const uint4 *>(xfp + t * NB * 16);
                xfp += 8 * xf_tile_words;
            }
            wa[K] = __shfl_sync(0xffffffffu, wa[0], nxt_lane);
            wb[K] = __shfl_sync(0xffffffffu, wb[0], nxt_lane);

            consume_chunk<K, NT>(wa, acc, 0, xa, dc);
            // every lane has consumed the slot (its words are in registers): refill it
            __syncwarp();
            if (lane == 0 && s + kDepth < nblk) {
                mbar_expect_tx(bar0 + 8 * slot, kStageBytes + kFragBytes);
                bulk_g2s(ring0 + slot * kSlotBytes, src0 + (size_t)(s + kDepth) * src_step, kStageBytes,
                         bar0 + 8 * slot);
                if constexpr (kStreamX)
                    bulk_g2s(ring0 + slot * kSlotBytes + kStageBytes, xsrc0 + (size_t)(s + kDepth) * xsrc_step,
                             kFragBytes, bar0 + 8 * slot);
            }
            consume_chunk<K, NT>(wb, acc, 1, xa, dc);
            if (++slot == kDepth) { slot = 0; phase ^= 1u; }
        }
    }
    // a wait that ran out leaves copies that may still be in flight into this warp's ring: give them one more
    // bounded chance to land before the region is reused and the CTA goes away
    if (!ok) {
#pragma unroll
        for (int s = 0; s < kDepth; ++s) mbar_wait(bar0 + 8 * s, s < slot ? phase ^ 1u : phase, P.status, 1 << 16);
    }
    __syncthreads();   // every warp is done with its ring: the region is reused below

    // ---- reduce the eight warps, eight rows (one accumulator tile) per pass: the staging buffer stays
    // small enough for two CTAs per SM also with sixteen rows
    float *red = reinterpret_cast<float *>(region);                  // [8 warps][8 rows][128]
    float *fin = red + kWarps * 8 * 128;                             // [NT*8][128]
    const int ocl = tid & 127;
    // Split units: the slices of a unit are the CTAs of one thread-block cluster (cluster rank = slice).  Every
    // CTA writes its sums into the FIRST CTA's shared memory (distributed shared memory, plain remote stores),
    // the cluster synchronises, and the first CTA adds the slices in slice order: no global scratch, no ticket,
    // bitwise reproducible.  The first cluster barrier makes sure that the first CTA's warps have left their
    // rings, which the slices' sums overwrite.
    const bool split = S.splitk > 1;
    float *slices = fin + NT * 8 * 128;                              // [splitk][rows][128], used in the first CTA only
    uint32_t slices_remote = 0;
    if (split) {
        cluster_sync();
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(slices_remote) : "r"(smem_u32(slices)));
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (t) __syncthreads();                                      // the previous pass has been summed
        {
            const int u = g >> 1, p = g & 1;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const int oc_lo = 64 * h + 16 * u + 4 * a + p;
                    const int n0 = 8 * t + 2 * q;
                    float *r0 = red + ((size_t)(warp * 8 + 2 * q)) * 128 + oc_lo;
                    if (n0 < P.rows) { r0[0] = acc[t][h][a][0]; r0[2] = acc[t][h][a][2]; }
                    if (n0 + 1 < P.rows) { r0[128] = acc[t][h][a][1]; r0[130] = acc[t][h][a][3]; }
                }
        }
        __syncthreads();
        for (int nl = tid >> 7; nl < 8 && 8 * t + nl < P.rows; nl += 2) {
            const int n = 8 * t + nl;
            float v = 0.f;
#pragma unroll
            for (int r = 0; r < kWarps; ++r) v += red[((size_t)(r * 8 + nl)) * 128 + ocl];
            if (!split) fin[n * 128 + ocl] = v;
            else st_cluster_f32(slices_remote + (uint32_t)(((ks * P.rows + n) * 128 + ocl) * 4), v);
        }
    }
    if (split) {
        cluster_sync();                                              // every slice's sums have landed in the first CTA
        if (ks != 0) return;
        for (int n = tid >> 7; n < P.rows; n += 2) {
            float v = 0.f;
            for (int k2 = 0; k2 < S.splitk; ++k2) v += slices[(k2 * P.rows + n) * 128 + ocl];
            fin[n * 128 + ocl] = v;
        }
    }
    __syncthreads();

    // ---- output Hadamard, svh, fp16
    const int ocol = S.out_col + ob * 128 + 4 * lane;
    const uint2 sv = __ldg(reinterpret_cast<const uint2 *>(S.svh + ob * 128 + 4 * lane));
    const __half2 sv01 = *reinterpret_cast<const __half2 *>(&sv.x);
    const __half2 sv23 = *reinterpret_cast<const __half2 *>(&sv.y);
    for (int n = warp; n < P.rows; n += kWarps) {
        const float4 f = *reinterpret_cast<const float4 *>(fin + n * 128 + 4 * lane);
        float v[4] = {f.x, f.y, f.z, f.w};
        fwht128_warp(v, lane);
        float r[4] = {0.f, 0.f, 0.f, 0.f};
        if (P.residual) {
            const uint2 rr = *reinterpret_cast<const uint2 *>(P.residual + (size_t)n * P.ld_res + ocol);
            const __half2 r01 = *reinterpret_cast<const __half2 *>(&rr.x), r23 = *reinterpret_cast<const __half2 *>(&rr.y);
            r[0] = __low2float(r01); r[1] = __high2float(r01); r[2] = __low2float(r23); r[3] = __high2float(r23);
        }
        const __half2 o01 = __floats2half2_rn(v[0] * kHadScale * __low2float(sv01) + r[0],
                                              v[1] * kHadScale * __high2float(sv01) + r[1]);
        const __half2 o23 = __floats2half2_rn(v[2] * kHadScale * __low2float(sv23) + r[2],
                                              v[3] * kHadScale * __high2float(sv23) + r[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t *>(&o01);
        o.y = *reinterpret_cast<const uint32_t *>(&o23);
        *reinterpret_cast<uint2 *>(P.y + (size_t)n * P.ldy + ocol) = o;
    }
}

// Pre-pass: H128(x * suh) of every shard, rounded to fp16 once, written in the order the GEMV's
// mma B fragments read it (per 16-channel tile: [row group][row][q][4 slots], both halves of a
// word equal).  One warp per (shard, row, 128-block).
__global__ void __launch_bounds__(256) xfrag_kernel(const __grid_constant__ GemvParams P, int nt) {
    asm volatile("griddepcontrol.wait;" ::: "memory");          // x may come from the previous kernel
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const int nrow = nt * P.nb;
    const int per_shard = nrow * P.kblocks;
    const int task = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (task >= per_shard * P.nshards) return;
    const int sh = task / per_shard, r = task - sh * per_shard;
    const int blk = r / nrow, n = r - blk * nrow;
    const GemvShardDev &S = P.sh[sh];
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (n < P.rows) {
        const int col = blk * 128 + 4 * lane;
        const __half *xrow = P.x + (size_t)n * P.ldx;
        const uint2 xr = *reinterpret_cast<const uint2 *>(xrow + col);
        const uint2 sr = __ldg(reinterpret_cast<const uint2 *>(S.suh + col));
        const __half2 x01 = *reinterpret_cast<const __half2 *>(&xr.x), x23 = *reinterpret_cast<const __half2 *>(&xr.y);
        const __half2 s01 = *reinterpret_cast<const __half2 *>(&sr.x), s23 = *reinterpret_cast<const __half2 *>(&sr.y);
        v[0] = __low2float(x01); v[1] = __high2float(x01); v[2] = __low2float(x23); v[3] = __high2float(x23);
        if (P.in_mode == 1) {
            // RMSNorm folded in: every warp reduces the whole row (it is short and sits in L2)
            float ss = 0.f;
            for (int c = 8 * lane; c < P.ic; c += 256) {
                const uint4 q4 = *reinterpret_cast<const uint4 *>(xrow + c);
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&q4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h2[j]);
                    ss += f.x * f.x + f.y * f.y;
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rn = rsqrtf(ss / (float)P.ic + P.eps);
            float g[4] = {1.f, 1.f, 1.f, 1.f};
            if (P.norm_w) {
                const uint2 gr = __ldg(reinterpret_cast<const uint2 *>(P.norm_w + col));
                const __half2 g01 = *reinterpret_cast<const __half2 *>(&gr.x), g23 = *reinterpret_cast<const __half2 *>(&gr.y);
                g[0] = __low2float(g01); g[1] = __high2float(g01); g[2] = __low2float(g23); g[3] = __high2float(g23);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __half2float(__float2half_rn(v[j] * rn * g[j]));   // the norm's own fp16 output
        } else if (P.in_mode == 2) {
            const uint2 ur = *reinterpret_cast<const uint2 *>(xrow + P.ic + col);
            const __half2 u01 = *reinterpret_cast<const __half2 *>(&ur.x), u23 = *reinterpret_cast<const __half2 *>(&ur.y);
            const float u[4] = {__low2float(u01), __high2float(u01), __low2float(u23), __high2float(u23)};
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __half2float(__float2half_rn(v[j] / (1.f + __expf(-v[j])) * u[j]));
        }
        v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
        fwht128_warp(v, lane);
    }
    const int xf_tile_words = nrow * 16;
    const int tile = blk * 8 + (lane >> 2);
    const int t = (nt == 2) ? (n >> 3) : 0;
    const int nn = (nt == 2) ? (n & 7) : n;
    uint32_t *dst = P.xfg + S.xf_off + (size_t)tile * xf_tile_words + ((t * P.nb + nn) * 4) * 4 + (lane & 3);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __half2 d = __float2half2_rn(v[k] * kHadScale);
        dst[k * 4] = *reinterpret_cast<const uint32_t *>(&d);
    }
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    int s = 0;
    while (s + 1 < P.nshards && (int)blockIdx.x >= P.sh[s + 1].cta_begin) ++s;
    const GemvShardDev &S = P.sh[s];
    const int local = blockIdx.x - S.cta_begin;
    switch (S.K) {
        case 1: gemv_cta<1, NT>(P, S, local, smem); break;
        case 2: gemv_cta<2, NT>(P, S, local, smem); break;
        case 3: gemv_cta<3, NT>(P, S, local, smem); break;
        case 4: gemv_cta<4, NT>(P, S, local, smem); break;
        case 5: gemv_cta<5, NT>(P, S, local, smem); break;
        case 6: gemv_cta<6, NT>(P, S, local, smem); break;
        case 7: gemv_cta<7, NT>(P, S, local, smem); break;
        case 8: gemv_cta<8, NT>(P, S, local, smem); break;
    }
}

// ---------------------------------------------------------------------------------------------
// host-side plan: how the shards are cut into CTAs and how the scratch is laid out
struct GemvPlan {
    int nt, nb, xf_bytes, xf_blocks, region_bytes, total_ctas, total_units, kblocks, splitk;
    long long xf_words;
    long long xf_off[EXL3_MAX_SHARDS];
    int cta_begin[EXL3_MAX_SHARDS], unit_begin[EXL3_MAX_SHARDS], K[EXL3_MAX_SHARDS];
};

static int make_plan(const exl3_shard *sh, int n, int rows, int ic, GemvPlan &pl, int max_splitk = kMaxSplitK) {
    if (!sh) return EXL3_E_NULL;
    if (n < 1 || n > EXL3_MAX_SHARDS || rows < 1 || rows > EXL3_GEMV_MAX_ROWS || ic <= 0 || (ic & 127))
        return EXL3_E_SHAPE;
    pl.kblocks = ic / 128;
    pl.nt = rows > 8 ? 2 : 1;
    pl.nb = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8;
    const int frag_bytes_per_block = 8 * pl.nt * pl.nb * 64;
    const bool stream_x = pl.nt == 2;                 // fragments ride in the warps' rings (1 KB per warp and step)
    int units = 0, ring = 0;
    for (int i = 0; i < n; ++i) {
        if (sh[i].oc <= 0 || (sh[i].oc & 127) || sh[i].out_col < 0 || (sh[i].out_col & 3)) return EXL3_E_SHAPE;
        if (sh[i].mcg || sh[i].mul1) return EXL3_E_UNSUPPORTED;
        const int K = integer_k(sh[i].k_times_2);
        if (!K) return EXL3_E_UNSUPPORTED;
        if (!sh[i].trellis || !sh[i].suh || !sh[i].svh) return EXL3_E_NULL;
        if (!aligned(sh[i].trellis, 16) || !aligned(sh[i].suh, 8) || !aligned(sh[i].svh, 8)) return EXL3_E_ALIGN;
        pl.K[i] = K;
        pl.unit_begin[i] = units;
        units += sh[i].oc / 128;
        const int r = kWarps * ring_depth(K) * (8 * 8 * K * 4 + (stream_x ? frag_bytes_per_block / 8 : 0));
        ring = r > ring ? r : ring;
    }
    if (units > kWsMaxUnits) return EXL3_E_SHAPE;
    // Every unit (128 output channels) is cut into the same number of input slices: as many as fit two CTAs on
    // every SM, at most one cluster's worth and at most one slice per 128 inputs.
    // (The kernel is bound by the decode, not by bytes, so units of every bitrate weigh the same.)
    int sk = kTargetCtas / units;                                    // never more than one wave of CTAs
    if (sk < 1) sk = 1;
    if (sk > pl.kblocks) sk = pl.kblocks;
    if (sk > kMaxSplitK) sk = kMaxSplitK;
    if (sk > max_splitk) sk = max_splitk < 1 ? 1 : max_splitk;
    int max_nblk, max_slice;
    for (;; --sk) {
        max_nblk = (pl.kblocks + sk - 1) / sk;
        // staging of one reduction pass, the summed rows, and (first CTA of a cluster) the slices' sums
        const int red = (kWarps * 8 + pl.nt * 8) * 128 * 4 + (sk > 1 ? sk * rows * 128 * 4 : 0);
        pl.region_bytes = ring > red ? ring : red;
        // the activation fragments of as many 128-blocks at once as the rest of the CTA's shared memory holds
        if (stream_x) {
            max_slice = kBarBytes + pl.region_bytes <= kCtaSmemBytes ? max_nblk : 0;
            if (max_slice || sk == 1) break;
            continue;
        }
        max_slice = (kCtaSmemBytes - kBarBytes - pl.region_bytes) / frag_bytes_per_block;
        if (max_slice >= (max_nblk < 2 ? max_nblk : 2) || sk == 1) break;     // fewer slices leave more room
    }
    if (max_slice < 1) return EXL3_E_SHAPE;
    pl.splitk = sk;
    pl.total_units = units;
    pl.total_ctas = units * sk;
    pl.xf_words = 0;
    for (int i = 0; i < n; ++i) {
        pl.cta_begin[i] = pl.unit_begin[i] * sk;
        pl.xf_off[i] = pl.xf_words;
        pl.xf_words += (long long)pl.kblocks * frag_bytes_per_block / 4;
    }
    pl.xf_blocks = max_nblk < max_slice ? max_nblk : max_slice;
    pl.xf_bytes = stream_x ? 0 : pl.xf_blocks * frag_bytes_per_block;
    return EXL3_OK;
}

// How many clusters of `c` CTAs of this kernel the current device can hold at once (cached; 0 on error).
static int clusters_that_fit(void (*kernel)(GemvParams), int nt, int c, size_t smem) {
    static std::mutex mu;
    struct Entry { int dev, nt, c; size_t smem; int n; };
    static Entry cache[64];
    static int used = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    const size_t key = (smem + 4095) & ~(size_t)4095;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
        if (cache[i].dev == dev && cache[i].nt == nt && cache[i].c == c && cache[i].smem == key) return cache[i].n;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)key) != cudaSuccess) { cudaGetLastError(); return 0; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(c * 64));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = key;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    if (used < 64) cache[used++] = Entry{dev, nt, c, key, n};
    return n;
}

static size_t plan_workspace_bytes(const GemvPlan &pl) {
    return kWsHeadBytes + (size_t)pl.xf_words * 4;
}

// Shrink the plan's clusters until all of them can be resident on the current device at once.
static int fit_clusters(const exl3_shard *shards, int nshards, int rows, int ic, GemvPlan &pl) {
    void (*kernel)(GemvParams) = pl.nt == 1 ? gemv_kernel<1> : gemv_kernel<2>;
    for (;;) {
        const size_t need = (size_t)kBarBytes + pl.xf_bytes + pl.region_bytes;
        if (pl.splitk == 1 || clusters_that_fit(kernel, pl.nt, pl.splitk, need) >= pl.total_units) return EXL3_OK;
        const int rc = make_plan(shards, nshards, rows, ic, pl, pl.splitk - 1);
        if (rc != EXL3_OK) return rc;
    }
}

}  // namespace exl3

extern "C" int exl3_gemv_plan(const exl3_shard *shards, int nshards, int rows, int ic, int *ctas_out, int *slices_out) {
    exl3::GemvPlan pl;
    int rc = exl3::make_plan(shards, nshards, rows, ic, pl);
    if (rc == EXL3_OK) rc = exl3::fit_clusters(shards, nshards, rows, ic, pl);
    if (rc != EXL3_OK) return rc;
    if (ctas_out) *ctas_out = pl.total_ctas;
    if (slices_out) *slices_out = pl.splitk;
    return EXL3_OK;
}

extern "C" size_t exl3_gemv_workspace_bytes(const exl3_shard *shards, int nshards, int rows, int ic) {
    exl3::GemvPlan pl;
    if (exl3::make_plan(shards, nshards, rows, ic, pl) != EXL3_OK) return 0;
    return exl3::plan_workspace_bytes(pl);
}

extern "C" int exl3_gemv_grouped_ex(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                                    int ic, int ldy, void *workspace, size_t workspace_bytes,
                                    const exl3_gemv_fusion *fusion, void *stream) {
    using namespace exl3;
    GemvPlan pl;
    const int rc = make_plan(shards, nshards, rows, ic, pl);
    if (rc != EXL3_OK) return rc;
    if (!x || !y) return EXL3_E_NULL;
    if (!aligned(x, 8) || !aligned(y, 8) || (ldy & 3)) return EXL3_E_ALIGN;
    for (int i = 0; i < nshards; ++i)
        if (shards[i].out_col + shards[i].oc > ldy) return EXL3_E_SHAPE;
    if (!workspace || workspace_bytes < plan_workspace_bytes(pl)) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;

    GemvParams P;
    P.x = static_cast<const __half *>(x);
    P.y = static_cast<__half *>(y);
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    P.status = reinterpret_cast<unsigned *>(ws);
    P.xfg = reinterpret_cast<uint32_t *>(ws + kWsHeadBytes);
    P.rows = rows;
    P.ic = ic;
    P.ldy = ldy;
    P.residual = nullptr; P.norm_w = nullptr; P.eps = 0.f; P.in_mode = 0; P.ldx = ic; P.ld_res = ldy;
    if (fusion) {
        if (fusion->in_mode < 0 || fusion->in_mode > 2) return EXL3_E_UNSUPPORTED;
        P.in_mode = fusion->in_mode;
        P.norm_w = static_cast<const __half *>(fusion->norm_weight);
        P.eps = fusion->eps;
        P.ldx = fusion->ldx > 0 ? fusion->ldx : (fusion->in_mode == 2 ? 2 * ic : ic);
        P.residual = static_cast<const __half *>(fusion->residual);
        P.ld_res = fusion->ld_residual > 0 ? fusion->ld_residual : ldy;
        if ((P.ldx & 7) || (P.ld_res & 3) || (P.norm_w && !aligned(P.norm_w, 8)) || (P.residual && !aligned(P.residual, 8)) || !aligned(x, 16))
            return EXL3_E_ALIGN;
        if (P.ldx < (P.in_mode == 2 ? 2 * ic : ic)) return EXL3_E_SHAPE;
    }
    P.kblocks = pl.kblocks;
    P.nb = pl.nb;
    P.xf_bytes = pl.xf_bytes;
    P.xf_blocks = pl.xf_blocks;
    P.one = 1u;
    P.nshards = nshards;
    for (int i = 0; i < nshards; ++i) {
        GemvShardDev &d = P.sh[i];
        d.trellis = static_cast<const uint32_t *>(shards[i].trellis);
        d.suh = static_cast<const __half *>(shards[i].suh);
        d.svh = static_cast<const __half *>(shards[i].svh);
        d.xf_off = pl.xf_off[i];
        d.tiles_j = shards[i].oc / 16;
        d.K = pl.K[i];
        d.out_col = shards[i].out_col;
        d.cta_begin = pl.cta_begin[i];
        d.splitk = pl.splitk;
        d.unit_begin = pl.unit_begin[i];
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The slices of a unit form one thread-block cluster.  Clusters are placed whole inside one GPC, so not every
    // cluster size lets all clusters of the grid run at once: take the largest size that does (the answer of the
    // occupancy query is cached per kernel, size and shared-memory need).
    void (*kernel)(GemvParams) = pl.nt == 1 ? gemv_kernel<1> : gemv_kernel<2>;
    const int rc2 = fit_clusters(shards, nshards, rows, ic, pl);
    if (rc2 != EXL3_OK) return rc2;
    for (int i = 0; i < nshards; ++i) {
        P.sh[i].cta_begin = pl.cta_begin[i];
        P.sh[i].splitk = pl.splitk;
    }
    P.xf_bytes = pl.xf_bytes;
    P.xf_blocks = pl.xf_blocks;
    const size_t smem = (size_t)kBarBytes + pl.xf_bytes + pl.region_bytes;
    // launched with programmatic stream serialization: this grid may start (and prefetch weights)
    // while the previous kernel on the stream drains; it synchronises inside (griddepcontrol.wait)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.total_ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;                 // the slices of a unit form one cluster
    attr[1].val.clusterDim.x = (unsigned)pl.splitk;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pl.splitk > 1 ? 2 : 1;
    cudaError_t e;
    {
        const int tasks = pl.nt * pl.nb * pl.kblocks * nshards;
        cudaLaunchConfig_t pc = cfg;
        pc.numAttrs = 1;
        pc.gridDim = dim3((unsigned)((tasks + 7) / 8));
        pc.blockDim = dim3(256);
        pc.dynamicSmemBytes = 0;
        e = cudaLaunchKernelEx(&pc, xfrag_kernel, P, pl.nt);
        if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    }
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    e = cudaLaunchKernelEx(&cfg, kernel, P);
    if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return launch_status();
}

extern "C" int exl3_gemv_grouped(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                                 int ic, int ldy, void *workspace, size_t workspace_bytes, void *stream) {
    return exl3_gemv_grouped_ex(shards, nshards, x, y, rows, ic, ldy, workspace, workspace_bytes, nullptr, stream);
}

extern "C" int exl3_gemv(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
                         int rows, int ic, int oc, int k_times_2, int mcg, int mul1, void *workspace,
                         size_t workspace_bytes, void *stream) {
    exl3_shard s;
    s.trellis = trellis;
    s.suh = suh;
    s.svh = svh;
    s.oc = oc;
    s.k_times_2 = k_times_2;
    s.mcg = mcg;
    s.mul1 = mul1;
    s.out_col = 0;
    return exl3_gemv_grouped(&s, 1, x, y, rows, ic, oc, workspace, workspace_bytes, stream);
}

// Self-test of the bounded wait: one warp waits `polls` polls, through the helper the GEMV uses, on a barrier that
// nothing will ever complete.  The wait runs out, the status word of `workspace` is set, the kernel returns.
namespace exl3 {
__global__ void gemv_wait_selftest_kernel(unsigned *status, int polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    mbar_wait(smem_u32(&bar), 0, status, polls);
}
}  // namespace exl3
extern "C" int exl3_gemv_selftest_wait(void *workspace, int polls, void *stream) {
    if (!workspace) return EXL3_E_NULL;
    if (polls < 1 || polls > (1 << 20)) return EXL3_E_SHAPE;
    exl3::gemv_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned *>(workspace), polls);
    return exl3::launch_status();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch of exl3_gemv_grouped lives in this library's own device
// memory instead of a caller buffer.
//
// The array below is reserved on every GPU that loads the library and stays reserved until the
// process exits; the loader zero-fills it, which is the state its status word needs (every launch overwrites
// the rest before reading it).  In HOST code its name is only a handle,
// not a device address, so the address is looked up once per device with cudaGetSymbolAddress
// (with that device current) and cached.
#define EXL3_STATIC_WS_BYTES_IMPL (2u << 20)
static __device__ __align__(256) unsigned char g_exl3_static_ws[EXL3_STATIC_WS_BYTES_IMPL];

namespace exl3 {
constexpr int kMaxDevices = 64;
static void *g_static_ws_ptr[kMaxDevices];       // device address of g_exl3_static_ws, per device
static std::mutex g_static_ws_mutex;

// Device address of the built-in scratch on the CURRENT device; resolved under a lock on first use, so
// two host threads making the first call on one device get the same answer and nothing is queued.
static int static_ws_for_current_device(void **out, int *dev_out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    void *p = __atomic_load_n(&g_static_ws_ptr[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        std::lock_guard<std::mutex> lock(g_static_ws_mutex);
        p = g_static_ws_ptr[dev];
        if (!p) {
            if (cudaGetSymbolAddress(&p, g_exl3_static_ws) != cudaSuccess || !p) { cudaGetLastError(); return EXL3_E_LAUNCH; }
            __atomic_store_n(&g_static_ws_ptr[dev], p, __ATOMIC_RELEASE);
        }
    }
    *out = p;
    if (dev_out) *dev_out = dev;
    return EXL3_OK;
}

// The device a pointer belongs to, or -1 when the runtime does not know it as device memory.
static int device_of(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged) return -1;
    return a.device;
}
}  // namespace exl3

extern "C" size_t exl3_gemv_static_capacity(void) { return EXL3_STATIC_WS_BYTES_IMPL; }

extern "C" int exl3_gemv_grouped_static(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                                        int ic, int ldy, void *stream) {
    using namespace exl3;
    GemvPlan pl;
    const int rc = make_plan(shards, nshards, rows, ic, pl);
    if (rc != EXL3_OK) return rc;
    if (plan_workspace_bytes(pl) > (size_t)EXL3_STATIC_WS_BYTES_IMPL) return EXL3_E_WORKSPACE;   // beyond the built-in scratch
    if (!x || !y) return EXL3_E_NULL;
    void *ws = nullptr;
    int dev = -1;
    const int rs = static_ws_for_current_device(&ws, &dev);
    if (rs != EXL3_OK) return rs;
    // the scratch is the CURRENT device's copy of the array: refuse tensors that live elsewhere
    if (device_of(x) != dev || device_of(y) != dev) return EXL3_E_DEVICE;
    return exl3_gemv_grouped(shards, nshards, x, y, rows, ic, ldy, ws, EXL3_STATIC_WS_BYTES_IMPL, stream);
}

extern "C" int exl3_gemv_static_status(unsigned *status_out) {
    using namespace exl3;
    if (!status_out) return EXL3_E_NULL;
    void *ws = nullptr;
    const int rs = static_ws_for_current_device(&ws, nullptr);
    if (rs != EXL3_OK) return rs;
    unsigned v = 0;
    if (cudaMemcpy(&v, static_cast<unsigned char *>(ws) + EXL3_WS_STATUS_OFFSET, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    *status_out = v;
    return EXL3_OK;
}
