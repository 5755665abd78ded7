// EXL3 GEMM for many rows (mid-batch and prefill): trellis decode into shared-memory fp16 tiles
// that feed tcgen05.mma, accumulators in tensor memory.
//
//     Yt[tokens][oc] = Xh[tokens][ic] . W(trellis)[ic][oc]          (fp16 in, fp32 accumulate, fp16 out)
//
// where Xh = H128(x * suh) is produced by a small pre-pass and the output Hadamard / svh by a
// post-pass (exl3_gemm_tc below chains the three).  The weights are the M side of the MMA (128
// output channels per CTA = the 128 TMEM lanes), tokens the N side (up to 512 per CTA = all 512
// TMEM columns), so every decoded weight tile is used for up to 512 tokens.
//
// CTA = 19 warps, one CTA per SM (up to 256 rows: 11 warps, one decode group, two CTAs per SM, so
// that one CTA's pipeline bubbles are filled by the other):
//   warp 0      producer of the packed trellis: 1-D bulk copies into a deep ring (mbarrier completion)
//   warp 18     producer of the activation tiles: 2-D tiled TMA loads with 128-byte swizzle
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..17 decode (two groups of eight, alternating stages): packed words -> 3INST codewords -> fp16 (the same rounding as
//               reconstruct) -> swizzled K-major A tile in shared memory; afterwards the epilogue
//               (tcgen05.ld of their TMEM lane quadrant, fp16 stores)
// The K order inside each 16-channel tile is permuted (k' = 4*(ic&3) + (ic>>2)) so that the four
// input channels a lane decodes for one output channel are adjacent in shared memory; the
// pre-pass writes Xh in the same order, which leaves the contraction unchanged.
// Every wait is bounded; a wait that runs out sets a status word and the kernel still frees its
// tensor memory and exits.
//
// Further down: the decode-once route for many rows (reconstruct_t_kernel + gemm_dense_pair_kernel, a persistent
// dense GEMM on CTA pairs with tcgen05.mma.cta_group::2 whose epilogue applies the output rotation), and the host code that picks between the two routes and
// the tensor-memory-operand kernel of exl3_gemm_ts.cuh.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "exl3_codec.cuh"
#include "exl3_common.cuh"
#include "exl3_decode_fast.cuh"
#include "exl3_hadamard.cuh"

#ifndef EXL3_TC_WAIT_OP
#define EXL3_TC_WAIT_OP "try_wait"
#endif

namespace exl3 {
namespace tc {

// warps: 0 trellis producer, 1 MMA issue, 2 .. 2+8G-1 decode (G groups of eight), last = activation producer
__host__ __device__ constexpr int threads_for(int groups) { return 32 * (3 + 8 * groups); }
constexpr int kDecodeWarps = 8;          // per group; two groups take alternate stages
constexpr int kBM = 128;                 // output channels per CTA
constexpr int kBK = 64;                  // input channels per stage (one 128-byte swizzle row)
constexpr int kBN = 256;                 // tokens per accumulator / per TMA box
constexpr int kMaxHalves = 2;            // accumulators per CTA (512 tokens)
constexpr int kSmallRows = 64;           // up to here: one decode group per CTA, two CTAs per SM
constexpr int kStagesA = 4;
constexpr int kMaxSlotsB = 16;            // ring of token-half tiles: 4 x 32 KB, more when the tiles are small
constexpr int kABytes = kBM * kBK * 2;               // 16 KB
constexpr int kBHalfBytes = kBN * kBK * 2;           // 32 KB
constexpr int kSpin = 1 << 26;
constexpr unsigned long long kWaitNs = 1000000000ull;   // one second

static __device__ unsigned g_tc_status;  // sticky: non-zero after a bounded wait ran out

__device__ __forceinline__ uint32_t s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: polls the barrier; after kWaitNs without success it records the failure in the
// status word and returns false (the caller stops its loop, the kernel still exits cleanly).
// `sleep_ns` > 0 backs off between polls: a spinning warp competes with the decode warps for issue
// slots (measured: more than half of the kernel's instructions were polls before this).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned sleep_ns = 0,
                                          unsigned long long limit_ns = kWaitNs) {
    unsigned long long t0 = 0;
    for (int it = 0; it < kSpin; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier." EXL3_TC_WAIT_OP ".parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((it & 255) == 255) {
            const unsigned long long t = now_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > limit_ns) break;
        }
    }
    atomicOr(&g_tc_status, 1u);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// K-major, 128-byte-swizzled operand whose rows are exactly 128 bytes: 8-row groups are 1024 bytes
// apart (SBO), the leading-dimension field is unused, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, fp16 A and B (both K-major), fp32 accumulate, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Position in a ring of `n` slots: slot index, phase bit of the current round, and whether the
// first round is over (only then does a producer have to wait for the slot to be released).
struct Cursor {
    int idx, n;
    uint32_t phase;
    bool wrapped;
    __device__ __forceinline__ Cursor(int start, int slots) : idx(start), n(slots), phase(0), wrapped(false) {}
    __device__ __forceinline__ void advance(int by) {
        idx += by;
        if (idx >= n) { idx -= n; phase ^= 1u; wrapped = true; }
    }
};

struct Params {
    const uint32_t *trellis;
    __half *y;             // [tokens][ldy]
    int tokens, ic, oc, ldy;
    int tiles_j;           // oc / 16
    int box_rows;          // token rows of one TMA box (<= 256)
    int b_slot_bytes;      // box_rows * 128, rounded up to 1024
    int raw_stages;        // depth of the packed-trellis ring
    int b_slots;           // depth of the activation-tile ring
    int tmem_cols;         // tensor-memory columns to allocate (power of two, 32..512)
    int a_stages;          // decoded-tile stages in use (<= kStagesA)
    int splitk;            // slices of the input dimension (grid.z)
    float *partial;        // [splitk][tokens][oc] fp32 when splitk > 1
    uint32_t one;
};

constexpr int kMaxRawStages = 32;
struct Barriers {
    uint64_t raw_full[kMaxRawStages], raw_empty[kMaxRawStages];
    uint64_t a_full[kStagesA], a_empty[kStagesA];
    uint64_t b_full[kMaxSlotsB], b_empty[kMaxSlotsB];
    uint64_t acc_full;
    uint32_t tmem_base;
};
// shared-memory plan: [A stages][B slots][barriers][raw trellis ring]
struct SmemView {
    unsigned char *a, *b;
    Barriers *bar;
    uint32_t *raw;
};

// Per-warp cycle counts of the decode loop's phases, compiled in only for the timing study.
#define TC_CLK(v) do { } while (0)
#define TC_ACC(i, a, b) do { } while (0)

template <int K, int G>
__global__ void __launch_bounds__(threads_for(G), G == 1 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const Params P) {
    extern __shared__ unsigned char smem_dyn[];
    // swizzled tiles need 1024-byte alignment; the launch reserves the slack
    unsigned char *smem_raw = smem_dyn + ((1024u - (s32(smem_dyn) & 1023u)) & 1023u);
    constexpr int kRawWords = 4 * 8 * 8 * K;                      // four tile rows of eight tiles
    constexpr uint32_t kRawRowBytes = 8 * 8 * K * 4;
    unsigned char *const smA = smem_raw;
    const int nStagesA = P.a_stages;
    unsigned char *const smB = smem_raw + nStagesA * kABytes;
    Barriers &S = *reinterpret_cast<Barriers *>(smB + (size_t)P.b_slots * P.b_slot_bytes);
    uint32_t *raw = reinterpret_cast<uint32_t *>(reinterpret_cast<unsigned char *>(&S) + 1024);
    const int kStagesRaw = P.raw_stages;
    const int kSlotsB = P.b_slots;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ob = blockIdx.x;                                    // 128-column block of outputs
    const int tok0 = blockIdx.y * (kBN * kMaxHalves);
    const int tok_here = min(P.tokens - tok0, kBN * kMaxHalves);
    const int halves = tok_here > kBN ? 2 : 1;
    const int total_steps = P.ic / kBK;
    const int step0 = (int)((long long)blockIdx.z * total_steps / P.splitk);
    const int nsteps = (int)((long long)(blockIdx.z + 1) * total_steps / P.splitk) - step0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesRaw; ++s) { mbar_init(s32(&S.raw_full[s]), 1); mbar_init(s32(&S.raw_empty[s]), kDecodeWarps); }
        for (int s = 0; s < kStagesA; ++s) { mbar_init(s32(&S.a_full[s]), kDecodeWarps); mbar_init(s32(&S.a_empty[s]), 1); }
        for (int s = 0; s < kSlotsB; ++s) { mbar_init(s32(&S.b_full[s]), 1); mbar_init(s32(&S.b_empty[s]), 1); }
        mbar_init(s32(&S.acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory: all 512 columns (one CTA per SM by construction)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&S.tmem_base)), "r"(P.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;

    if (warp == 0) {
        // ---------------- producer of the packed trellis (runs ahead by the whole ring).  Lanes 0..3
        // each issue one of the four row copies of a stage: issuing them from one thread was the
        // bottleneck of the whole kernel (about a quarter microsecond per bulk copy).
        {
            const uint32_t *src_row0 = P.trellis + (size_t)ob * 8 * (8 * K);
            const size_t row_words = (size_t)P.tiles_j * (8 * K);
            bool ok = true;
            Cursor rc(0, kStagesRaw);
            for (int s = 0; s < nsteps; ++s, rc.advance(1)) {
                const int rs = rc.idx;
                if (lane == 0) {
                    if (rc.wrapped) ok = mbar_wait(s32(&S.raw_empty[rs]), rc.phase ^ 1u, 200);
                    if (ok) mbar_expect_tx(s32(&S.raw_full[rs]), 4 * kRawRowBytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < 4)
                    bulk_g2s(s32(raw + rs * kRawWords + lane * (kRawWords / 4)),
                             src_row0 + (size_t)(4 * (step0 + s) + lane) * row_words, kRawRowBytes, s32(&S.raw_full[rs]));
            }
        }
    } else if (warp == threads_for(G) / 32 - 1) {
        // ---------------- producer of the activation tiles
        if (lane == 0) {
            const uint32_t box_bytes = (uint32_t)P.box_rows * (kBK * 2);
            Cursor bc(0, kSlotsB);                               // ring of token-half tiles
            bool ok = true;
            for (int s = 0; s < nsteps && ok; ++s) {
                for (int h = 0; h < halves && ok; ++h, bc.advance(1)) {
                    const int bs = bc.idx;
                    if (bc.wrapped) ok = mbar_wait(s32(&S.b_empty[bs]), bc.phase ^ 1u, 200);
                    if (!ok) break;
                    mbar_expect_tx(s32(&S.b_full[bs]), box_bytes);
                    tma_2d(s32(smB + (size_t)bs * P.b_slot_bytes), &xmap, (step0 + s) * kBK, tok0 + h * kBN, s32(&S.b_full[bs]));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue
        if (lane == 0) {
            const int n_last = ((tok_here - (halves - 1) * kBN) + 15) & ~15;      // tokens in the last half, padded to 16
            bool ok = true;
            Cursor ac(0, nStagesA), bc(0, kSlotsB);
            for (int s = 0; s < nsteps && ok; ++s, ac.advance(1)) {
                const int as = ac.idx;
                ok = mbar_wait(s32(&S.a_full[as]), ac.phase, G == 1 ? 40 : 0);
                const uint32_t a0 = s32(smA + as * kABytes);
                for (int h = 0; h < halves && ok; ++h, bc.advance(1)) {
                    const int bs = bc.idx;
                    ok = mbar_wait(s32(&S.b_full[bs]), bc.phase, G == 1 ? 40 : 0);
                    if (!ok) break;
                    if (G == 1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // decoded tile: generic writes -> tensor-core reads
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t b0 = s32(smB + (size_t)bs * P.b_slot_bytes);
                    const uint32_t idesc = umma_idesc(h == halves - 1 ? n_last : kBN);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma(tmem + h * kBN, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), idesc, (s | k) ? 1u : 0u);
                    umma_commit(s32(&S.b_empty[bs]));   // arrives when the MMAs above have read smem
                }
                umma_commit(s32(&S.a_empty[as]));
            }
            umma_commit(s32(&S.acc_full));
        }
    } else {
        // ---------------- decode warps
        const int grp = (warp - 2) >> 3;           // stages s = grp, grp + 2, ...
        const int dw = (warp - 2) & 7;             // 0..7 inside the group
        // A warp takes ONE output tile (dw) and all four 16-channel input tiles of the stage: lane
        // group u = lane >> 3 works on input tile u.  (Four output tiles at one input tile would send
        // the four groups to the same shared-memory banks: the swizzle only depends on row & 7.)
        const int u = lane >> 3, c = lane & 7, p = c >> 2, q = c & 3;
        const DecodeConsts dc(P.one);
        const int nxt_lane = (lane & 24) | ((lane + 1) & 7);
        bool ok = true;
        Cursor rc(grp, kStagesRaw), ac(grp, nStagesA);
        for (int s = grp; s < nsteps && ok; s += G, rc.advance(G), ac.advance(G)) {
            const int rs = rc.idx, as = ac.idx;
            TC_CLK(c0);
            ok = mbar_wait(s32(&S.raw_full[rs]), rc.phase, 60);
            TC_CLK(c1);
            TC_ACC(0, c0, c1);
            uint32_t wd[K + 1];
            {
                const uint32_t *src = raw + rs * kRawWords + u * (kRawWords / 4) + dw * (8 * K) + c * K;
                load_words<K>(src, wd);
            }
            wd[K] = __shfl_sync(0xffffffffu, wd[0], nxt_lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(s32(&S.raw_empty[rs]));
            uint32_t z[32];
            decode_chunk_fast<K>(wd, z, dc);
            TC_CLK(c2);
            TC_ACC(1, c1, c2);
            if (ac.wrapped) ok = ok && mbar_wait(s32(&S.a_empty[as]), ac.phase ^ 1u, 60);
            TC_CLK(c3);
            TC_ACC(2, c2, c3);
            // weights of output channel (a, hm): input channels j = 2b + hk, adjacent in k'
            unsigned char *abase = smA + as * kABytes;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int hm = 0; hm < 2; ++hm) {
                    const uint32_t z0 = z[8 * a + hm], z1 = z[8 * a + 2 + hm], z2 = z[8 * a + 4 + hm], z3 = z[8 * a + 6 + hm];
                    uint32_t lo01, hi01, lo23, hi23;
                    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(lo01) : "r"(z0), "r"(z1));
                    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(hi01) : "r"(z0), "r"(z1));
                    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(lo23) : "r"(z2), "r"(z3));
                    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(hi23) : "r"(z2), "r"(z3));
                    const __half2 w01 = __hadd2(*reinterpret_cast<__half2 *>(&lo01), *reinterpret_cast<__half2 *>(&hi01));
                    const __half2 w23 = __hadd2(*reinterpret_cast<__half2 *>(&lo23), *reinterpret_cast<__half2 *>(&hi23));
                    const int r = 16 * dw + 4 * a + 2 * hm + p;                         // row of the A tile
                    const int chunk = (2 * u + (q >> 1)) ^ (r & 7);                     // 128-byte swizzle
                    uint2 v;
                    v.x = *reinterpret_cast<const uint32_t *>(&w01);
                    v.y = *reinterpret_cast<const uint32_t *>(&w23);
                    *reinterpret_cast<uint2 *>(abase + r * 128 + chunk * 16 + (q & 1) * 8) = v;
                }
            // release the tile.  Few rows (G == 1): decode is the critical path, so the MMA-issuing
            // thread, which acquires the tile through the barrier, makes the generic-proxy writes
            // visible to the tensor core with one proxy fence on its side.  Many rows (G == 2): the
            // MMA issue is the critical path, so the writers fence instead.
            if (G == 2) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // many rows: the writers have slack
            __syncwarp();
            if (lane == 0) mbar_arrive(s32(&S.a_full[as]));
            TC_CLK(c4);
            TC_ACC(3, c3, c4);
        }

        // ---------------- epilogue: TMEM -> fp16 -> y[token][oc]
        ok = mbar_wait(s32(&S.acc_full), 0, 200) && ok;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quad = warp & 3;                                  // TMEM lanes 32*quad .. +31
        const int oc_row = ob * kBM + 32 * quad + lane;
        // the two warps of a quadrant split the columns of every half
        const int col_part = (warp - 2) >> 2;     // four warps share a lane quadrant
        for (int h = 0; h < halves; ++h) {
            const int ncols = min(kBN, tok_here - h * kBN);
            for (int c0 = col_part * 32; c0 < ncols; c0 += 64 * G) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(h * kBN + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = tok0 + h * kBN + c0 + j;
                        if (c0 + j < ncols) {
                            if (P.splitk > 1)
                                P.partial[((size_t)blockIdx.z * P.tokens + tok) * P.oc + oc_row] = __uint_as_float(v[j]);
                            else
                                P.y[(size_t)tok * P.ldy + oc_row] = __float2half_rn(__uint_as_float(v[j]));
                        }
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P.tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Many rows (>= kDenseMinRows): decode ONCE, then a dense tcgen05 GEMM on CTA pairs.
//
// With thousands of rows the in-kernel decode above repeats the integer decode of every weight once per 512 rows
// and its sixteen decode warps cannot keep the tensor pipe fed (measured: the MMA-issuing thread waits for a
// decoded tile in every step).  So from kDenseMinRows rows the weight is rebuilt once, transposed (Wt[oc][ic], the
// K-major form tcgen05 wants), and this kernel multiplies it with the rotated activations:
//     Yt[oc][tokens] += Wt[oc][ic] . Xh[tokens][ic]^T        (fp16 in, fp32 in tensor memory, fp16 out)
// One MMA spans two SMs (tcgen05.mma.cta_group::2, M = 256 output channels, N = 256 tokens): each CTA of the pair
// loads its own 128 rows of Wt and HALF of the token tile (128 of the 256 rows), so the token tile crosses
// L2 -> shared memory once per 256 output channels and each SM reads 8 KB of operands per MMA instead of 12.
// All loads are per-CTA 2-D TMA loads of this GPU's own memory (no multicast); both CTAs' loads are counted on the
// first CTA's barrier (the cta_group::2 form of the load), the first CTA's commits arrive on the barriers of both.
// Warps: 0 and 10 = producers (one lane each: weight rows / token rows), 1 = MMA issue (first CTA of the pair only),
// 2..9 = epilogue (tcgen05.ld of their lane quadrant, fp16 stores).  Four stages of 48 KB.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled TMA load into THIS CTA's shared memory whose bytes are counted on a barrier of the pair's first CTA
// (`bar_cluster`: a shared::cluster address).  Not a multicast load: one CTA's own tile of this GPU's memory.
__device__ __forceinline__ void tma_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void umma2(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// kind::f16, fp16 A and B (both K-major), fp32 accumulate, M = 256 (128 per CTA), N = n
__device__ __forceinline__ uint32_t umma2_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

constexpr int kDenseMinRows = 1024;                                    // from here always (given an even number of output blocks)
constexpr int kDenseStages = 7;
constexpr int kDenseBand = 8;                                          // channel pairs (of 256 channels) per L2 band
constexpr int kDenseHalfBytes = (kBN / 2) * kBK * 2;                   // this CTA's 128 token rows of a 256-token tile: 16 KB
constexpr int kDenseStageBytes = kABytes + kDenseHalfBytes;            // 32 KB
constexpr int kDenseEpiWarps = 8;
constexpr int kDenseBWarp = 2 + kDenseEpiWarps;                        // the token-tile producer (after the epilogue warps)
constexpr int kDenseThreads = 32 * (3 + kDenseEpiWarps);
constexpr size_t kDenseSmem = (size_t)kDenseStages * kDenseStageBytes + 1024 /*barriers*/ + 1024 /*alignment*/;

struct DenseParams {
    __half *y;             // [tokens][ldy]
    int tokens, ic, oc, ldy;
    int npx, nty;          // tiles: pairs of 128-channel blocks x 256-token tiles
    int npairs;            // CTA pairs launched (each walks work items pair, pair + npairs, ...)
    // The tiles beyond the last full round of `npairs` are cut into `tail_f` (1, 2 or 4) narrower items of
    // 256 / tail_f tokens each, so that the last round is shorter instead of mostly idle.
    int full_items;        // items that are whole tiles
    int items;             // full_items + (tiles - full_items) * tail_f
    int tail_f;
    int wide_st;           // epilogue rotation: output rows are 32-byte aligned (256-bit stores: whole sectors per lane)
};
struct DenseBarriers {
    uint64_t full[kDenseStages], empty[kDenseStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
};

// tile number (in launch order) -> (channel pair, token tile): bands of kDenseBand channel pairs are walked token
// tile by token tile, so that the pairs running at the same time share a band's weight rows in L2
__device__ __forceinline__ void dense_tile(const DenseParams &P, int L, int &px, int &ty) {
    const int full_bands = P.npx / kDenseBand;
    const int in_full = full_bands * kDenseBand * P.nty;
    if (L < in_full) {
        const int band = L / (kDenseBand * P.nty), r = L - band * (kDenseBand * P.nty);
        px = band * kDenseBand + r % kDenseBand;
        ty = r / kDenseBand;
    } else {                                                      // the last, narrower band
        const int w = P.npx - full_bands * kDenseBand, r = L - in_full;
        px = full_bands * kDenseBand + r % w;
        ty = r / w;
    }
}

// work item (in launch order) -> tile, first token and width of its slice of the tile
__device__ __forceinline__ void dense_item(const DenseParams &P, int L, int &px, int &tok0, int &ntok) {
    int ty;
    if (L < P.full_items) {
        dense_tile(P, L, px, ty);
        tok0 = ty * kBN;
        ntok = kBN;
    } else {
        const int t = L - P.full_items;
        dense_tile(P, P.full_items + t / P.tail_f, px, ty);
        ntok = kBN / P.tail_f;
        tok0 = ty * kBN + (t % P.tail_f) * ntok;
    }
}

// The same for the kernel that keeps tokens in the accumulator's lanes: a leftover tile is cut along its CHANNELS
// (halves of 128: one rotation block), `n0` is the first channel and `n` the width of the item.
__device__ __forceinline__ void dense_item_rot(const DenseParams &P, int L, int &tok0, int &n0, int &n) {
    int px, ty;
    if (L < P.full_items) {
        dense_tile(P, L, px, ty);
        n0 = px * kBN;
        n = kBN;
    } else {
        const int t = L - P.full_items;
        dense_tile(P, P.full_items + t / P.tail_f, px, ty);
        n = kBN / P.tail_f;
        n0 = px * kBN + (t % P.tail_f) * n;
    }
    tok0 = ty * kBN;
}

// two fp32 values per instruction (sm_100 packed arithmetic on register pairs)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// 32 consecutive accumulator columns of this warp's 32 lanes (no wait: several loads may be in flight)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

// Persistent: every CTA pair walks its share of the 256-channel x 256-token tiles.  Tensor memory holds two
// accumulators (2 x 256 columns): while the epilogue warps drain one tile, the MMAs of the next tile fill the other.
// ROT = false: the weight rows are the M operand (accumulator lanes = output channels, columns = tokens), the weight
// comes with the output rotation folded in or a rotation pass follows.  ROT = true: the TOKENS are the M operand
// (lanes = tokens, columns = output channels), so one thread holds a token's 128 consecutive channels: the epilogue
// applies the output rotation in registers (7 x 64 butterflies in fp32) and the signs and scale, and writes the
// final result; the weight is the plain transposed decode and `tail` is a map of the weight with narrower boxes.
template <bool ROT>
__global__ void __launch_bounds__(kDenseThreads, 1)
gemm_dense_pair_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                       const __grid_constant__ CUtensorMap xmap_tail, const DenseParams P, const __half *__restrict__ svh) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *smem_raw = smem_dyn + ((1024u - (s32(smem_dyn) & 1023u)) & 1023u);   // swizzled tiles: 1024-byte alignment
    DenseBarriers &S = *reinterpret_cast<DenseBarriers *>(smem_raw + (size_t)kDenseStages * kDenseStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();                     // 0 issues the MMAs of the pair
    const int pair = blockIdx.x >> 1;
    const int nitems = P.items;
    const int nsteps = P.ic / kBK;
    constexpr uint32_t kTmemCols = 2 * kBN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDenseStages; ++s) {
            mbar_init(s32(&S.full[s]), 1);
            mbar_init(s32(&S.empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s32(&S.acc_full[b]), 1);
            mbar_init(s32(&S.acc_empty[b]), 2 * kDenseEpiWarps);   // the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory of the pair: one warp of each CTA, together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&S.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                  // the other CTA's barriers exist before anything is signalled across
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = S.tmem_base;

    if (warp == 0 || warp == kDenseBWarp) {
        // ---------------- producers: warp 0 loads this CTA's 128 weight rows, warp kDenseBWarp its half of the token
        // tile, every step of every work item of the pair (two warps: issuing a TMA load costs its thread a few
        // dozen cycles, and one thread issuing everything was measured to hold the ring back; L2 prefetches issued
        // from here cost more than they gained).  The bytes of BOTH CTAs are counted on the first CTA's `full`
        // barrier (which that CTA's weight producer arms with the sum), so the MMA-issuing lane learns of the
        // second CTA's tiles without a relay.
        if (lane == 0) {
            const bool is_a = warp == 0;
            bool ok = true;
            uint32_t full0;                                          // full[0] of the pair's first CTA
            asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(full0) : "r"(s32(&S.full[0])));
            Cursor c(0, kDenseStages);
            for (int L = pair; L < nitems && ok; L += P.npairs) {
                // M operand: 128 rows per CTA; N operand: this CTA's half of the item's n rows
                const CUtensorMap *ma, *mb;
                int row_a, row_b, n;
                if constexpr (ROT) {
                    int tok0, n0;
                    dense_item_rot(P, L, tok0, n0, n);
                    ma = &xmap;                                      // token rows out of range arrive as zeros
                    mb = n == kBN ? &wmap : &xmap_tail;              // box of n / 2 weight rows
                    row_a = tok0 + (int)crank * kBM;
                    row_b = n0 + (int)crank * (n / 2);
                } else {
                    int px, tok0;
                    dense_item(P, L, px, tok0, n);
                    ma = &wmap;
                    mb = n == kBN ? &xmap : &xmap_tail;              // box of n / 2 token rows
                    row_a = (2 * px + (int)crank) * kBM;
                    row_b = tok0 + (int)crank * (n / 2);
                }
                const uint32_t bytes = 2 * (kABytes + (n / 2) * kBK * 2);
                for (int s = 0; s < nsteps && ok; ++s, c.advance(1)) {
                    if (c.wrapped) ok = mbar_wait(s32(&S.empty[c.idx]), c.phase ^ 1u, 20);
                    if (!ok) break;
                    const uint32_t bar = full0 + 8 * c.idx;
                    const uint32_t st = s32(smem_raw + (size_t)c.idx * kDenseStageBytes);
                    if (is_a) {
                        if (crank == 0) mbar_expect_tx(s32(&S.full[c.idx]), bytes);
                        tma_2d_pair(st, ma, s * kBK, row_a, bar);
                    } else {
                        tma_2d_pair(st + kABytes, mb, s * kBK, row_b, bar);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && crank == 0) {
            // ---------------- first CTA: MMA issue for the pair
            bool ok = true;
            Cursor c(0, kDenseStages);
            int i = 0;                                               // items of this pair so far
            for (int L = pair; L < nitems && ok; L += P.npairs, ++i) {
                const int b = i & 1, use = i >> 1;
                const uint32_t idesc = umma2_idesc(L < P.full_items ? kBN : kBN / P.tail_f);
                // the epilogue warps of both CTAs have drained this accumulator's previous tile
                if (use > 0) ok = mbar_wait(s32(&S.acc_empty[b]), (uint32_t)(use - 1) & 1u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int s = 0; s < nsteps && ok; ++s, c.advance(1)) {
                    ok = mbar_wait(s32(&S.full[c.idx]), c.phase);    // both CTAs' tiles of this stage have landed
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a0 = s32(smem_raw + (size_t)c.idx * kDenseStageBytes), b0 = a0 + kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma2(tmem + b * kBN, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), idesc, (s | k) ? 1u : 0u);
                    umma2_commit(s32(&S.empty[c.idx]));  // both CTAs' stage is free once these MMAs have read it
                }
                umma2_commit(s32(&S.acc_full[b]));       // both CTAs' epilogue warps may read the accumulator
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> fp16 -> y[token][oc], tile after tile, one accumulator behind the MMAs
        const int quad = warp & 3;                                  // TMEM lanes 32*quad .. +31
        const int col_part = (warp - 2) >> 2;                       // the two warps of a quadrant split the columns
        uint32_t acc_empty0;                                        // acc_empty[0] of the pair's first CTA
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(acc_empty0) : "r"(s32(&S.acc_empty[0])));
        bool ok = true;
        int i = 0;
        for (int L = pair; L < nitems && ok; L += P.npairs, ++i) {
            const int b = i & 1, use = i >> 1;
            if constexpr (ROT) {
                int tok0, n0, n;
                dense_item_rot(P, L, tok0, n0, n);
                const int tok = tok0 + (int)crank * kBM + 32 * quad + lane;
                ok = mbar_wait(s32(&S.acc_full[b]), (uint32_t)use & 1u, 100);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (col_part * 128 < n) {                           // a 128-channel item: the quadrant's first warp alone
                    float f[128];
                    const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(b * kBN + col_part * 128);
#pragma unroll
                    for (int g = 0; g < 4; ++g) tmem_ld32(taddr + 32 * g, reinterpret_cast<uint32_t *>(f) + 32 * g);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // 128-point Walsh-Hadamard transform of the thread's own values: the first stage pairs neighbours,
                    // the other six run on packed pairs (two fp32 per instruction).  Measured: the MMAs of the next
                    // tile wait while the epilogue warps issue this burst, so its instruction count is what it costs
                    // (896 scalar additions: +5 % on the whole kernel; packed: +2 %; pauses between the stages do not help).
                    uint64_t p2[64];
#pragma unroll
                    for (int e = 0; e < 64; ++e) p2[e] = pack2(f[2 * e] + f[2 * e + 1], f[2 * e] - f[2 * e + 1]);
#pragma unroll
                    for (int h = 1; h < 64; h <<= 1)
#pragma unroll
                        for (int e = 0; e < 64; ++e)
                            if ((e & h) == 0) {
                                const uint64_t u0 = p2[e], u1 = p2[e + h];
                                p2[e] = add2(u0, u1);
                                p2[e + h] = sub2(u0, u1);
                            }
                    if (ok && tok < P.tokens) {
                        const int ch0 = n0 + col_part * 128;
                        const uint4 *sv = reinterpret_cast<const uint4 *>(svh + ch0);
                        uint4 *dst = reinterpret_cast<uint4 *>(P.y + (size_t)tok * P.ldy + ch0);
                        const uint64_t hs2 = pack2(kHadScale, kHadScale);
                        // a lane writes 16 bytes of its own row per plain store: half a sector, which travels to L2 as
                        // a masked whole one (measured: twice the write traffic); 256-bit stores fill the sectors
#pragma unroll
                        for (int g = 0; g < 16; g += 2) {
                            uint32_t ow[8];
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                const uint4 s8 = __ldg(sv + g + t);
                                const __half2 *sh = reinterpret_cast<const __half2 *>(&s8);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 sf = __half22float2(sh[e]);
                                    float lo, hi;
                                    unpack2(mul2(p2[4 * (g + t) + e], mul2(pack2(sf.x, sf.y), hs2)), lo, hi);
                                    const __half2 hv = __floats2half2_rn(lo, hi);
                                    ow[4 * t + e] = *reinterpret_cast<const uint32_t *>(&hv);
                                }
                            }
                            if (P.wide_st) {
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + g), "r"(ow[0]), "r"(ow[1]),
                                             "r"(ow[2]), "r"(ow[3]), "r"(ow[4]), "r"(ow[5]), "r"(ow[6]), "r"(ow[7]) : "memory");
                            } else {
                                dst[g] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                                dst[g + 1] = make_uint4(ow[4], ow[5], ow[6], ow[7]);
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(acc_empty0 + 8 * b) : "memory");
                continue;
            }
            int px, tok0, ntok;
            dense_item(P, L, px, tok0, ntok);
            const int oc_row = (2 * px + (int)crank) * kBM + 32 * quad + lane;
            const int ncols = min(ntok, P.tokens - tok0);
            ok = mbar_wait(s32(&S.acc_full[b]), (uint32_t)use & 1u, 100);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int c0 = col_part * 32; c0 < ntok; c0 += 64) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(b * kBN + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < ncols)
                            P.y[(size_t)(tok0 + c0 + j) * P.ldy + oc_row] = __float2half_rn(__uint_as_float(v[j]));
                }
            }
            // this warp's reads of the accumulator are complete: hand it back to the MMAs (first CTA's barrier)
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(acc_empty0 + 8 * b) : "memory");
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                  // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Wt[oc][ic'] = svh[oc] * (H128 over each block of 128 output channels of the decoded weight) / sqrt(128), transposed
// (ic' = the permuted order of the rotated activations).  Rebuilding the weight once per call leaves room to fold
// the layer's OUTPUT rotation and signs into it:  H (W^T xh) = (H W^T) xh,  so the GEMM's epilogue writes the final
// result and no pass over the [tokens][oc] output follows.  One CTA = 128 output channels x 64 input channels: warp w
// decodes the four tiles (lane = 8*tile + chunk) of output tile w that follow each other along the input
// dimension and stages them transposed in shared memory; then the CTA multiplies the block by the 128 x 128 sign
// matrix on the tensor cores (mma.sync, fp32 accumulation: exact), scales, rounds to fp16 ONCE, and writes 128 rows of 64 contiguous input channels (128 bytes) with 16-byte stores.
constexpr int kRecTPitch = 72;
template <int K, bool FOLD>
__global__ void __launch_bounds__(256)
reconstruct_t_kernel(const uint32_t *__restrict__ trellis, const __half *__restrict__ svh, __half *__restrict__ wt,
                     int tiles_j, int ic) {
    __shared__ __align__(16) __half stage[8][16][kRecTPitch];       // [output tile][output channel][input channel]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // A fragments of the sign matrix for this warp's 16 output rows: H[r][c] = (-1)^popcount(r & c), generated once
    uint32_t afr[8][4];
#pragma unroll
    for (int kt = 0; kt < 8; ++kt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = 16 * warp + (lane >> 2) + (e & 1) * 8, c = 16 * kt + 2 * (lane & 3) + (e >> 1) * 8;
            const uint32_t lo = (__popc(r & c) & 1) ? 0xBC00u : 0x3C00u;
            const uint32_t hi = (__popc(r & (c + 1)) & 1) ? 0xBC00u : 0x3C00u;
            afr[kt][e] = lo | (hi << 16);
        }
    for (int cy = blockIdx.y; cy < ic / 64; cy += gridDim.y) {      // 64 input channels per pass
    {
        const int u = lane >> 3, c = lane & 7;
        const int tj = blockIdx.x * 8 + warp;                       // oc is a multiple of 128: always in range
        const int ti = cy * 4 + u;
        uint32_t wd[K + 1];
        const uint32_t *src = trellis + ((size_t)ti * tiles_j + tj) * (size_t)(8 * K) + c * K;
#pragma unroll
        for (int k = 0; k < K; ++k) wd[k] = __ldg(src + k);
        wd[K] = __shfl_sync(0xffffffffu, wd[0], (lane & 24) | ((c + 1) & 7));
        uint32_t z[32];
        decode_chunk<K>(wd, z);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            // the K order inside a 16-channel tile is the one xh_permute_kernel writes: channel 8b + 4h + q at 4q + 2b + h
            const int r = tile_row(c, i);
            stage[warp][tile_col(c, i)][16 * u + 4 * (r & 3) + 2 * (r >> 3) + ((r >> 2) & 1)] = codeword_to_half(z[i]);
        }
    }
    __syncthreads();
    if constexpr (FOLD) {
        // H (128 x 128, entries +-1) times the staged block (128 output channels x 64 input channels) on the tensor
        // cores: warp w produces output rows 16w .. 16w+15; the staged block is the B operand through transposing
        // ldmatrix loads.
        const int g = lane >> 2, q = lane & 3;
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
        const int lj = lane >> 3, lr = lane & 7;
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
            const uint32_t (&a)[4] = afr[kt];
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int k = 16 * kt + (lj & 1) * 8 + lr, n0 = 16 * np + (lj >> 1) * 8;
                uint32_t b[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(s32(&stage[k >> 4][k & 15][n0])));
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    asm volatile(
                        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                        : "+f"(acc[2 * np + h][0]), "+f"(acc[2 * np + h][1]), "+f"(acc[2 * np + h][2]), "+f"(acc[2 * np + h][3])
                        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[2 * h]), "r"(b[2 * h + 1]));
            }
        }
        __syncthreads();                                            // every warp has read the whole block
        const float s0 = kHadScale * __half2float(__ldg(svh + (size_t)blockIdx.x * 128 + 16 * warp + g));
        const float s1 = kHadScale * __half2float(__ldg(svh + (size_t)blockIdx.x * 128 + 16 * warp + g + 8));
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<__half2 *>(&stage[warp][g][8 * nt + 2 * q]) = __floats2half2_rn(acc[nt][0] * s0, acc[nt][1] * s0);
            *reinterpret_cast<__half2 *>(&stage[warp][g + 8][8 * nt + 2 * q]) = __floats2half2_rn(acc[nt][2] * s1, acc[nt][3] * s1);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 32 + lane;
        const int r = idx >> 3, seg = idx & 7;
        const uint4 val = *reinterpret_cast<const uint4 *>(&stage[warp][r][seg * 8]);
        *reinterpret_cast<uint4 *>(wt + (size_t)(128 * blockIdx.x + 16 * warp + r) * ic + 64 * cy + seg * 8) = val;
    }
    __syncthreads();                                                // the block is re-staged by the next pass
    }
}

// The same fold (Wt = svh * H128 Wt / sqrt(128) per 128-channel block), with the sign-matrix product on tcgen05:
//     D[oc' (128 TMEM lanes)][ic (256 columns)] = H[oc'][oc] (A, generated once per CTA) x W[ic][oc]^T (B, K-major: the
//     decoded weights staged in shared memory as rows of input channels, 128-byte swizzle, two K halves of 64)
// Eight MMAs (M = 128, N = 256, K = 128) per 128 x 256 block: the product disappears behind the decode, and the
// epilogue reads every output row's 256 consecutive input channels straight out of tensor memory.  CTA = 8 warps:
// all decode and all read the accumulator back; one lane of warp 0 issues the MMAs.  Two CTAs share an SM (96 KB of
// shared memory and 256 tensor-memory columns each).
constexpr int kFoldN = 256;                          // input channels per pass
constexpr int kFoldABytes = 2 * 128 * 128;           // H: two K halves of [128 rows][64]
constexpr int kFoldBBytes = 2 * kFoldN * 128;        // W: two K halves of [256 rows][64]
constexpr size_t kFoldSmem = kFoldABytes + kFoldBBytes + 1024 /*barrier, tmem base*/ + 1024 /*alignment*/;
template <int K>
__global__ void __launch_bounds__(256, 2)
reconstruct_fold_kernel(const uint32_t *__restrict__ trellis, const __half *__restrict__ svh, __half *__restrict__ wt,
                        int tiles_j, int ic) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *smem_raw = smem_dyn + ((1024u - (s32(smem_dyn) & 1023u)) & 1023u);
    unsigned char *smA = smem_raw, *smB = smem_raw + kFoldABytes;
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem_raw + kFoldABytes + kFoldBBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // A[r][p] = H[r][oc(p)] = (-1)^popcount(r & oc(p)) as fp16, K-major rows of 128 bytes per K half, 128-byte
    // swizzle.  The K order p is free (A and B share it): it is chosen so that the eight output channels a lane
    // decodes for one input channel are adjacent (one 16-byte store): p = 16 tile + 8 c2 + 4 i4 + 2 i3 + i0 holds
    // channel 16 tile + 8 i4 + 4 i3 + 2 i0 + c2.
    for (int i = tid; i < 128 * 128 / 2; i += 256) {
        const int r = i >> 6, p = 2 * (i & 63);
        const int o0 = (p & ~15) + 8 * ((p >> 2) & 1) + 4 * ((p >> 1) & 1) + ((p >> 3) & 1), o1 = o0 + 2;
        const uint32_t lo = (__popc(r & o0) & 1) ? 0xBC00u : 0x3C00u, hi = (__popc(r & o1) & 1) ? 0xBC00u : 0x3C00u;
        const int h = p >> 6, c = p & 63;
        *reinterpret_cast<uint32_t *>(smA + h * 16384 + r * 128 + ((((c >> 3) ^ (r & 7))) << 4) + (c & 7) * 2) = lo | (hi << 16);
    }
    if (tid == 0) {
        mbar_init(s32(bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(kFoldN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const float sc = kHadScale * __half2float(__ldg(svh + (size_t)blockIdx.x * 128 + 32 * (warp & 3) + lane));
    uint32_t phase = 0;
    bool ok = true;

    // the packed words of a whole 256-channel chunk (four passes of four input tiles) are fetched ahead: the ones of
    // the next chunk fly while this chunk's product and epilogue run (only 16 warps share an SM here, too few to hide
    // the memory latency by themselves)
    uint32_t wn[kFoldN / 64][K];
    auto fetch = [&](int cy) {
        const int u = lane >> 3, c = lane & 7;
#pragma unroll
        for (int pass = 0; pass < kFoldN / 64; ++pass) {
            const int ti = cy * (kFoldN / 16) + pass * 4 + u;
            const uint32_t *src = trellis + ((size_t)ti * tiles_j + blockIdx.x * 8 + warp) * (size_t)(8 * K) + c * K;
#pragma unroll
            for (int k = 0; k < K; ++k) wn[pass][k] = __ldg(src + k);
        }
    };
    if ((int)blockIdx.y < ic / kFoldN) fetch(blockIdx.y);
    for (int cy = blockIdx.y; cy < ic / kFoldN && ok; cy += gridDim.y) {
        // ---- decode 128 output channels x 256 input channels: a warp takes output tile `warp` and, per pass, four
        // input tiles; weight (input channel i, output channel o) goes to row p(i) of the B tile, where p is the K
        // order of the rotated activations inside a 16-channel tile (channel 8b + 4h + q at 4q + 2b + h)
        {
            const int u = lane >> 3, c = lane & 7;
#pragma unroll
            for (int pass = 0; pass < kFoldN / 64; ++pass) {
                uint32_t wd[K + 1];
#pragma unroll
                for (int k = 0; k < K; ++k) wd[k] = wn[pass][k];
                wd[K] = __shfl_sync(0xffffffffu, wd[0], (lane & 24) | ((c + 1) & 7));
                uint32_t z[32];
                decode_chunk<K>(wd, z);
                // weight i of chunk c: input channel 8 i2 + 4 i1 + (c & 3), output channel 4 (i >> 3) + 2 i0 + (c >> 2)
#pragma unroll
                for (int rb = 0; rb < 4; ++rb) {                     // rb = 2 i2 + i1
                    const int row = pass * 64 + 16 * u + 4 * (c & 3) + rb;                                // B row (input channel)
                    uint4 o;
                    uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {                    // e = 2 i4 + i3
                        const __half2 hv = __halves2half2(codeword_to_half(z[8 * e + 2 * rb]), codeword_to_half(z[8 * e + 2 * rb + 1]));
                        ow[e] = *reinterpret_cast<const uint32_t *>(&hv);
                    }
                    const int chunk = 2 * (warp & 3) + (c >> 2);
                    *reinterpret_cast<uint4 *>(smB + (warp >> 2) * (kFoldN * 128) + row * 128 + ((chunk ^ (row & 7)) << 4)) = o;
                }
            }
        }
        if (cy + (int)gridDim.y < ic / kFoldN) fetch(cy + gridDim.y);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t idesc = umma_idesc(kFoldN);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                umma(tmem, umma_desc(s32(smA) + (k >> 2) * 16384 + (k & 3) * 32),
                     umma_desc(s32(smB) + (k >> 2) * (kFoldN * 128) + (k & 3) * 32), idesc, k ? 1u : 0u);
            umma_commit(s32(bar));
        }
        ok = mbar_wait(s32(bar), phase, 20);
        phase ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // ---- output rows: lane quadrant = 32 output channels, the two warps of a quadrant split the 256 columns.
        // The rounded rows pass through the (now free) B tile, 512 bytes per row with the 16-byte pieces XOR-ed by
        // the row number, so that both the per-row writes here and the per-row reads below are conflict-free and
        // global memory sees whole 512-byte rows.
        {
            const int quad = warp & 3, half_cols = (warp >> 2) * (kFoldN / 2), R = 32 * quad + lane;
#pragma unroll 1
            for (int c0 = half_cols; c0 < half_cols + kFoldN / 2; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 o;
                    uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 hv = __floats2half2_rn(__uint_as_float(v[j + 2 * e]) * sc, __uint_as_float(v[j + 2 * e + 1]) * sc);
                        ow[e] = *reinterpret_cast<const uint32_t *>(&hv);
                    }
                    *reinterpret_cast<uint4 *>(smB + R * 512 + ((((c0 + j) >> 3) ^ lane) << 4)) = o;
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (ok) {
#pragma unroll 4
            for (int rr = 0; rr < 16; ++rr) {
                const int r = 16 * warp + rr;
                const uint4 val = *reinterpret_cast<const uint4 *>(smB + r * 512 + ((lane ^ (r & 31)) << 4));
                *reinterpret_cast<uint4 *>(wt + (size_t)(blockIdx.x * 128 + r) * ic + (size_t)cy * kFoldN + 8 * lane) = val;
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();                                             // tensor memory and the B tile are free again
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kFoldN) : "memory");
    }
}

// The elementwise neighbours of the layer that the pre-pass can absorb (see exl3_gemv_fusion).
struct XhFusion {
    int in_mode;            // 0 plain, 1 RMSNorm, 2 silu(x[:, :ic]) * x[:, ic:]
    const __half *norm_w;   // RMSNorm weight or null
    float eps;
    int ldx;                // row pitch of x in elements
    int ic;
};
// four consecutive activations as floats; bf16 is narrowed to fp16 first (the reference casts
// activations to fp16: config.py:233)
template <bool BF16>
__device__ __forceinline__ void load4(const void *x, size_t off, float (&v)[4]) {
    if (BF16) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const unsigned short *>(x) + off);
        v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k]));
    } else {
        const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const __half *>(x) + off);
        const __half2 h01 = *reinterpret_cast<const __half2 *>(&raw.x), h23 = *reinterpret_cast<const __half2 *>(&raw.y);
        v[0] = __low2float(h01); v[1] = __high2float(h01); v[2] = __low2float(h23); v[3] = __high2float(h23);
    }
}

// The plain case (no fused norm / activation) of the pre-pass below for many rows: the kernel moves 4 bytes per element
// and little else, so each warp takes four consecutive 128-blocks and issues all of their loads before the first
// butterfly (one block per warp: 2.6 TB/s on B200).  Same arithmetic, same output order.
template <bool BF16>
__global__ void __launch_bounds__(256)
xh_permute4_kernel(const void *__restrict__ x, const __half *__restrict__ suh, __half *__restrict__ xh,
                   long long nblocks, int blocks_per_row, int ldx) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const long long wid0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * 4;
    if (wid0 >= nblocks) return;
    uint2 raw[4], sg[4];
    // one division per warp (32-bit when the block count allows) instead of a 64-bit one per block
    const unsigned bpr = (unsigned)blocks_per_row;
    long long row0;
    unsigned blk0;
    if (nblocks <= 0x7fffffffLL) {
        const unsigned r = (unsigned)wid0 / bpr;
        row0 = r;
        blk0 = (unsigned)wid0 - r * bpr;
    } else {
        row0 = wid0 / blocks_per_row;
        blk0 = (unsigned)(wid0 - row0 * blocks_per_row);
    }
    float sgn[5];
    fwht128_signs(lane, sgn);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        unsigned blk = blk0;
        long long row = row0;
        if (wid0 + u < nblocks) {
            blk += u;
            while (blk >= bpr) { blk -= bpr; ++row; }
        }
        raw[u] = *reinterpret_cast<const uint2 *>(static_cast<const unsigned short *>(x) + (size_t)row * ldx + (size_t)blk * 128 + 4 * lane);
        sg[u] = *reinterpret_cast<const uint2 *>(suh + blk * 128 + 4 * lane);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        if (wid0 + u >= nblocks) break;
        float v[4];
        if (BF16) {
            v[0] = __uint_as_float(raw[u].x << 16); v[1] = __uint_as_float(raw[u].x & 0xFFFF0000u);
            v[2] = __uint_as_float(raw[u].y << 16); v[3] = __uint_as_float(raw[u].y & 0xFFFF0000u);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k]));
        } else {
            const __half2 h01 = *reinterpret_cast<const __half2 *>(&raw[u].x), h23 = *reinterpret_cast<const __half2 *>(&raw[u].y);
            v[0] = __low2float(h01); v[1] = __high2float(h01); v[2] = __low2float(h23); v[3] = __high2float(h23);
        }
        const __half2 s01 = *reinterpret_cast<const __half2 *>(&sg[u].x), s23 = *reinterpret_cast<const __half2 *>(&sg[u].y);
        v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
        fwht128_warp_signed(v, sgn);
        __half *dst = xh + (size_t)(wid0 + u) * 128 + 16 * (lane >> 2) + (lane & 3);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[4 * j] = __float2half_rn(v[j] * kHadScale);
    }
}

// The plain pre-pass with sixteen values per lane (eight lanes per 128-block, four blocks per warp): four butterfly
// stages in registers, three across lanes (12 shuffles per block instead of 20), and a lane's sixteen channels are
// exactly one 16-channel tile, so the permuted K order is a reordering of its own registers and the lane stores 32
// contiguous bytes.  Same stage order and rounding as xh_permute4_kernel.  Needs 16-byte aligned rows.
template <bool BF16>
__global__ void __launch_bounds__(256)
xh_permute16_kernel(const void *__restrict__ x, const __half *__restrict__ suh, __half *__restrict__ xh,
                    long long nblocks, int blocks_per_row, int ldx) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31, sub = lane & 7;
    const long long wid0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * 4;
    if (wid0 >= nblocks) return;
    const long long wid = wid0 + (lane >> 3);
    const bool live = wid < nblocks;
    long long row = 0;
    unsigned blk = 0;
    if (live) {
        if (nblocks <= 0x7fffffffLL) {
            const unsigned r = (unsigned)wid / (unsigned)blocks_per_row;
            row = r;
            blk = (unsigned)wid - r * (unsigned)blocks_per_row;
        } else {
            row = wid / blocks_per_row;
            blk = (unsigned)(wid - row * blocks_per_row);
        }
    }
    uint4 r[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)}, sg[2] = {r[0], r[0]};
    if (live) {
        const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(x) + (size_t)row * ldx + (size_t)blk * 128 + 16 * sub);
        const uint4 *ss = reinterpret_cast<const uint4 *>(suh + (size_t)blk * 128 + 16 * sub);
        r[0] = src[0]; r[1] = src[1];
        sg[0] = ss[0]; sg[1] = ss[1];
    }
    float v[16];
    {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(r);
        const __half2 *sh = reinterpret_cast<const __half2 *>(sg);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float lo, hi;
            if (BF16) {
                lo = __half2float(__float2half_rn(__uint_as_float(w[i] << 16)));
                hi = __half2float(__float2half_rn(__uint_as_float(w[i] & 0xFFFF0000u)));
            } else {
                const __half2 hv = *reinterpret_cast<const __half2 *>(&w[i]);
                lo = __low2float(hv);
                hi = __high2float(hv);
            }
            v[2 * i] = lo * __low2float(sh[i]);
            v[2 * i + 1] = hi * __high2float(sh[i]);
        }
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
        const float sgn = ((lane >> i) & 1) ? -1.f : 1.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float other = __shfl_xor_sync(0xffffffffu, v[k], 1 << i);
            v[k] = fmaf(v[k], sgn, other);
        }
    }
    if (live) {
        // position p = 4q + 2b + h of the tile holds channel 8b + 4h + q
        uint4 o[2];
        uint32_t *ow = reinterpret_cast<uint32_t *>(o);
#pragma unroll
        for (int p = 0; p < 16; p += 2) {
            const int c0 = 8 * ((p >> 1) & 1) + (p >> 2), c1 = c0 + 4;      // p even: h = 0; p + 1: h = 1
            const __half2 hv = __halves2half2(__float2half_rn(v[c0] * kHadScale), __float2half_rn(v[c1] * kHadScale));
            ow[p >> 1] = *reinterpret_cast<const uint32_t *>(&hv);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(xh + (size_t)wid * 128 + 16 * sub);
        dst[0] = o[0];
        dst[1] = o[1];
    }
}

// Pre-pass: Xh = H128(x * suh) as fp16, with the K order permuted inside every 16-channel tile
// (channel 8b + 4h + q is stored at 4q + 2b + h) to match the A tiles written by the decode warps.
// x may be fp16 or bf16 (the reference casts activations to fp16 first: config.py:233).
template <bool BF16>
__global__ void __launch_bounds__(256)
xh_permute_kernel(const void *__restrict__ x, const __half *__restrict__ suh, __half *__restrict__ xh,
                  long long nblocks, int blocks_per_row, XhFusion F) {
    // no-ops unless launched with programmatic stream serialization: x and the scratch may still be
    // in use by the kernels before this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wid >= nblocks) return;
    const int blk = (int)(wid % blocks_per_row);
    const long long row = wid / blocks_per_row;
    const size_t off = (size_t)row * F.ldx + (size_t)blk * 128 + 4 * lane;
    float v[4];
    load4<BF16>(x, off, v);
    if (F.in_mode == 1) {
        // RMSNorm folded in: the row is short and sits in L2, every warp reduces it itself
        float ss = 0.f;
        for (int c = 4 * lane; c < F.ic; c += 128) {
            float t[4];
            load4<BF16>(x, (size_t)row * F.ldx + c, t);
            ss += t[0] * t[0] + t[1] * t[1] + t[2] * t[2] + t[3] * t[3];
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rn = rsqrtf(ss / (float)F.ic + F.eps);
        float g[4] = {1.f, 1.f, 1.f, 1.f};
        if (F.norm_w) load4<false>(F.norm_w, (size_t)blk * 128 + 4 * lane, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k] * rn * g[k]));     // the norm's own fp16 output
    } else if (F.in_mode == 2) {
        float u[4];
        load4<BF16>(x, off + F.ic, u);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k] / (1.f + __expf(-v[k])) * u[k]));
    }
    const uint2 sr = *reinterpret_cast<const uint2 *>(suh + blk * 128 + 4 * lane);
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sr.x), s23 = *reinterpret_cast<const __half2 *>(&sr.y);
    v[0] *= __low2float(s01); v[1] *= __high2float(s01); v[2] *= __low2float(s23); v[3] *= __high2float(s23);
    fwht128_warp(v, lane);
    // lane holds channels 16T + 4*(lane&3) + j (j = 0..3) of tile T = lane >> 2: b = (lane&3)>>1,
    // h = lane&1, q = j  ->  position 4j + (lane&3)
    __half *dst = xh + (size_t)wid * 128 + 16 * (lane >> 2) + (lane & 3);
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[4 * j] = __float2half_rn(v[j] * kHadScale);
}

// Post-pass for split-K: sum the fp32 slices in order, H128, svh, fp16.
__global__ void __launch_bounds__(256)
reduce_had_kernel(const float *__restrict__ partial, int splitk, const __half *__restrict__ svh,
                  __half *y, long long nblocks, int blocks_per_row, size_t slice_elems, int ldy,
                  const __half *residual, int ld_res) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wid >= nblocks) return;
    const int blk = (int)(wid % blocks_per_row);
    const size_t off = (size_t)wid * 128 + 4 * lane;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < splitk; ++k) {
        const float4 p = *reinterpret_cast<const float4 *>(partial + k * slice_elems + off);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __half2float(__float2half_rn(v[j]));   // same rounding point as the unsplit path
    fwht128_warp(v, lane);
    const uint2 sr = *reinterpret_cast<const uint2 *>(svh + blk * 128 + 4 * lane);
    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sr.x), s23 = *reinterpret_cast<const __half2 *>(&sr.y);
    const long long row = wid / blocks_per_row;
    float r[4] = {0.f, 0.f, 0.f, 0.f};
    if (residual) load4<false>(residual, (size_t)row * ld_res + (size_t)blk * 128 + 4 * lane, r);   // may alias y
    const __half2 o01 = __floats2half2_rn(v[0] * kHadScale * __low2float(s01) + r[0], v[1] * kHadScale * __high2float(s01) + r[1]);
    const __half2 o23 = __floats2half2_rn(v[2] * kHadScale * __low2float(s23) + r[2], v[3] * kHadScale * __high2float(s23) + r[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&o01);
    o.y = *reinterpret_cast<const uint32_t *>(&o23);
    *reinterpret_cast<uint2 *>(y + (size_t)row * ldy + (size_t)blk * 128 + 4 * lane) = o;
}

// ---- grouped forms of the two passes: every shard of a fused layer in one launch -------------
struct XhGroup {
    int nshards;
    const __half *suh[EXL3_MAX_SHARDS];
    __half *xh[EXL3_MAX_SHARDS];
};
template <bool BF16>
__global__ void __launch_bounds__(256)
xh_permute_grouped_kernel(const void *__restrict__ x, const __grid_constant__ XhGroup G, long long nblocks,
                          int blocks_per_row, XhFusion F) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const long long wall = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wall >= nblocks * G.nshards) return;
    const int sh = (int)(wall / nblocks);
    const long long wid = wall - (long long)sh * nblocks;
    const int blk = (int)(wid % blocks_per_row);
    const long long row = wid / blocks_per_row;
    const size_t off = (size_t)row * F.ldx + (size_t)blk * 128 + 4 * lane;
    float v[4];
    load4<BF16>(x, off, v);
    if (F.in_mode == 1) {
        float ss = 0.f;
        for (int c = 4 * lane; c < F.ic; c += 128) {
            float t[4];
            load4<BF16>(x, (size_t)row * F.ldx + c, t);
            ss += t[0] * t[0] + t[1] * t[1] + t[2] * t[2] + t[3] * t[3];
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rn = rsqrtf(ss / (float)F.ic + F.eps);
        float g[4] = {1.f, 1.f, 1.f, 1.f};
        if (F.norm_w) load4<false>(F.norm_w, (size_t)blk * 128 + 4 * lane, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k] * rn * g[k]));
    } else if (F.in_mode == 2) {
        float u[4];
        load4<BF16>(x, off + F.ic, u);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = __half2float(__float2half_rn(v[k] / (1.f + __expf(-v[k])) * u[k]));
    }
    float sg[4];
    load4<false>(G.suh[sh], (size_t)blk * 128 + 4 * lane, sg);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] *= sg[k];
    fwht128_warp(v, lane);
    __half *dst = G.xh[sh] + (size_t)wid * 128 + 16 * (lane >> 2) + (lane & 3);     // same K order as xh_permute_kernel
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[4 * j] = __float2half_rn(v[j] * kHadScale);
}

struct ReduceGroup {
    int nshards;
    long long blk_begin[EXL3_MAX_SHARDS + 1];   // 128-blocks (row-major over [rows][oc / 128]) before each shard
    const float *partial[EXL3_MAX_SHARDS];
    const __half *svh[EXL3_MAX_SHARDS];
    int splitk[EXL3_MAX_SHARDS], blocks_per_row[EXL3_MAX_SHARDS], out_col[EXL3_MAX_SHARDS];
    long long slice_elems[EXL3_MAX_SHARDS];
};
__global__ void __launch_bounds__(256)
reduce_had_grouped_kernel(const __grid_constant__ ReduceGroup G, __half *y, int ldy, const __half *residual, int ld_res) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const long long wall = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wall >= G.blk_begin[G.nshards]) return;
    int sh = 0;
    while (sh + 1 < G.nshards && wall >= G.blk_begin[sh + 1]) ++sh;
    const long long wid = wall - G.blk_begin[sh];
    const int bpr = G.blocks_per_row[sh];
    const int blk = (int)(wid % bpr);
    const long long row = wid / bpr;
    const size_t off = (size_t)wid * 128 + 4 * lane;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < G.splitk[sh]; ++k) {
        const float4 p = *reinterpret_cast<const float4 *>(G.partial[sh] + (size_t)k * G.slice_elems[sh] + off);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __half2float(__float2half_rn(v[j]));   // same rounding point as the single-shard path
    fwht128_warp(v, lane);
    float sv[4];
    load4<false>(G.svh[sh], (size_t)blk * 128 + 4 * lane, sv);
    const size_t col = (size_t)G.out_col[sh] + (size_t)blk * 128 + 4 * lane;
    float r[4] = {0.f, 0.f, 0.f, 0.f};
    if (residual) load4<false>(residual, (size_t)row * ld_res + col, r);         // may alias y
    const __half2 o01 = __floats2half2_rn(v[0] * kHadScale * sv[0] + r[0], v[1] * kHadScale * sv[1] + r[1]);
    const __half2 o23 = __floats2half2_rn(v[2] * kHadScale * sv[2] + r[2], v[3] * kHadScale * sv[3] + r[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t *>(&o01);
    o.y = *reinterpret_cast<const uint32_t *>(&o23);
    *reinterpret_cast<uint2 *>(y + (size_t)row * ldy + col) = o;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

template <int K, int G>
static int launch_g(const CUtensorMap &map, Params P, cudaStream_t st) {
    const size_t raw_stage = (size_t)(4 * 8 * 8 * K) * 4;
    P.b_slots = 4;
    P.a_stages = G == 1 ? 3 : kStagesA;
    const size_t fixed = (size_t)P.a_stages * kABytes + (size_t)P.b_slots * P.b_slot_bytes + 1024 /*barriers*/ + 1024 /*alignment*/;
    // G == 1: two CTAs share an SM (about 110 KB each); G == 2: one CTA owns it
    const size_t budget = (G == 1 ? 112 : 226) * 1024;
    if (fixed + 2 * raw_stage > budget) return EXL3_E_SHAPE;
    size_t stages = (budget - fixed) / raw_stage;
    const size_t want = ((G == 1 ? 32 : 64) * 1024 + raw_stage - 1) / raw_stage;   // packed trellis in flight per CTA
    if (stages > want) stages = want;
    if (stages > (size_t)kMaxRawStages) stages = kMaxRawStages;
    P.raw_stages = (int)stages;
    const size_t smem = fixed + stages * raw_stage;
    if (cudaFuncSetAttribute(gemm_tc_kernel<K, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    dim3 grid(P.oc / kBM, (P.tokens + kBN * kMaxHalves - 1) / (kBN * kMaxHalves), P.splitk);
    gemm_tc_kernel<K, G><<<grid, threads_for(G), smem, st>>>(map, P);
    return launch_status();
}

template <int K>
static int launch(const CUtensorMap &map, const Params &P, cudaStream_t st) {
    return P.tokens <= kSmallRows ? launch_g<K, 1>(map, P, st) : launch_g<K, 2>(map, P, st);
}

}  // namespace tc
}  // namespace exl3

#include "exl3_gemm_ts.cuh"

extern "C" int exl3_had_r_128(const void *in, void *out, const void *pre, const void *post, float scale, int rows,
                              int n, void *stream);

extern "C" unsigned exl3_gemm_tc_status(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, exl3::tc::g_tc_status, sizeof(v)) != cudaSuccess) { cudaGetLastError(); return ~0u; }
    return v;
}
extern "C" int exl3_gemm_tc_status_reset(void) {
    const unsigned v = 0;
    if (cudaMemcpyToSymbol(exl3::tc::g_tc_status, &v, sizeof(v)) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return EXL3_OK;
}

// Self-test of the bounded waits: one warp waits, with a limit of `limit_us` microseconds, on a barrier that
// nothing will ever complete, through the very helper the kernels use (which 0: the shared-memory-operand
// kernel's, 1: the tensor-memory kernel's).  The wait runs out, the sticky status word is set, the kernel returns.
namespace exl3 { namespace tc {
__global__ void wait_selftest_kernel(int which, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(s32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (which == 0) mbar_wait(s32(&bar), 0, 32, limit_ns);
    else t5::mbar_wait(s32(&bar), 0, &g_tc_status, 32, limit_ns);
}
}}  // namespace exl3::tc
extern "C" int exl3_gemm_tc_selftest_wait(int which, unsigned limit_us, void *stream) {
    if (which < 0 || which > 1 || limit_us == 0 || limit_us > 1000000u) return EXL3_E_SHAPE;
    exl3::tc::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(which, (unsigned long long)limit_us * 1000ull);
    return exl3::launch_status();
}

namespace exl3 { namespace tc {
// slices of the input dimension: fill the 148 SMs when the output grid alone cannot
static int choose_splitk(int rows, int ic, int oc) {
    const int ctas = (oc / kBM) * ((rows + kBN * kMaxHalves - 1) / (kBN * kMaxHalves));
    const int steps = ic / kBK;
    int sk = 1;
    const int slots = rows <= kSmallRows ? 296 : 148;   // small batches: two CTAs share an SM
    if (ctas < slots * 4 / 5) sk = (slots + ctas / 2) / ctas;
    if (sk > steps / 8) sk = steps / 8;
    return sk < 1 ? 1 : sk;
}
static size_t xh_bytes(int rows, int ic) { return (((size_t)rows * ic * 2) + 255) & ~(size_t)255; }
// The decode-once route: output blocks that pair up, and enough rows to amortise rebuilding the weight.  Crossover
// with the in-kernel-decode kernel, measured on B200 (us per call, decode-once against in-kernel decode):
//   5120 -> 17408 @3: 141 / 122 at 512 rows, 178 / 195 at 768;   17408 -> 5120 @4: 154 / 131 at 256, 161 / 181 at 384,
//   166 / 193 at 512;   5120 -> 6144 @4: 74 / 63 at 512, 80 / 99 at 768;   5120 -> 1024 @5: 60 / 47 at 1000 (too few tiles).
static bool use_dense(int rows, int ic, int oc) {
    if ((oc / kBM) & 1) return false;
    if (rows >= kDenseMinRows) return true;
    if (oc < 2048) return false;
    return rows >= 640 || (rows >= 384 && ic >= 2 * oc);
}

template <int K>
static int launch_reconstruct_t(const void *trellis, const void *svh, void *wt, int ic, int oc, bool fold, cudaStream_t st) {
    const int tiles_j = oc / 16;
    dim3 grid(oc / 128, (ic / 64 + 3) / 4);                          // four passes per CTA: the sign fragments are reused
    if (fold && ic % kFoldN == 0) {
        if (cudaFuncSetAttribute(reconstruct_fold_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFoldSmem) != cudaSuccess) {
            cudaGetLastError();
            return EXL3_E_LAUNCH;
        }
        // CTAs loop over 256-channel chunks with stride gridDim.y: take the split with the fewest (waves x passes),
        // counting a CTA's set-up (sign matrix, tensor-memory allocation) as a quarter of a pass
        const int chunks = ic / kFoldN, bx = oc / 128, slots = 2 * 148;
        int best_y = 1;
        float best = 1e30f;
        for (int y = 1; y <= chunks; ++y) {
            const float cost = (float)((bx * y + slots - 1) / slots) * ((float)((chunks + y - 1) / y) + 0.25f);
            if (cost < best) { best = cost; best_y = y; }
        }
        dim3 fgrid(bx, best_y);
        reconstruct_fold_kernel<K><<<fgrid, 256, kFoldSmem, st>>>(static_cast<const uint32_t *>(trellis), static_cast<const __half *>(svh),
                                                                   static_cast<__half *>(wt), tiles_j, ic);
    } else if (fold)
        reconstruct_t_kernel<K, true><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(trellis), static_cast<const __half *>(svh),
                                                            static_cast<__half *>(wt), tiles_j, ic);
    else
        reconstruct_t_kernel<K, false><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(trellis), static_cast<const __half *>(svh),
                                                             static_cast<__half *>(wt), tiles_j, ic);
    return launch_status();
}

typedef int (*DenseTailMapFn)(void *ctx, int box_rows, CUtensorMap *out);
template <bool ROT>
static int launch_dense(const CUtensorMap &wmap, const CUtensorMap &xmap, DenseTailMapFn tail_map, void *tail_ctx,
                        DenseParams P, const __half *svh, cudaStream_t st) {
    if (cudaFuncSetAttribute(gemm_dense_pair_kernel<ROT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDenseSmem) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kDenseThreads);
    cfg.dynamicSmemBytes = kDenseSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;                 // the two CTAs of a pair
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // as many pairs as the device holds at once (cached per device), each walking its share of the tiles
    static int pairs_on[64] = {};                                     // (one table per instantiation)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    int fit = dev >= 0 && dev < 64 ? pairs_on[dev] : 0;
    if (fit == 0) {
        cfg.gridDim = dim3(2 * 1024);
        if (cudaOccupancyMaxActiveClusters(&fit, gemm_dense_pair_kernel<ROT>, &cfg) != cudaSuccess || fit < 1) {
            cudaGetLastError();
            return EXL3_E_LAUNCH;
        }
        if (dev >= 0 && dev < 64) pairs_on[dev] = fit;
    }
    const int ntiles = P.npx * P.nty;
    P.npairs = ntiles < fit ? ntiles : fit;
    // the tiles left over after the last full round: cut them in 2 or 4 when the pieces still fit one round
    const int tail = ntiles % P.npairs;
    P.tail_f = tail == 0 ? 1 : (!ROT && 4 * tail <= P.npairs) ? 4 : 2 * tail <= P.npairs ? 2 : 1;   // ROT: whole rotation blocks
    P.full_items = ntiles - (P.tail_f > 1 ? tail : 0);
    P.items = P.full_items + (ntiles - P.full_items) * P.tail_f;
    CUtensorMap xtail = xmap;
    if (P.tail_f > 1) {
        const int rc = tail_map(tail_ctx, kBN / 2 / P.tail_f, &xtail);
        if (rc != EXL3_OK) return rc;
    }
    cfg.gridDim = dim3((unsigned)(2 * P.npairs));
    if (cudaLaunchKernelEx(&cfg, gemm_dense_pair_kernel<ROT>, wmap, xmap, xtail, P, svh) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return launch_status();
}
} }

extern "C" size_t exl3_gemm_tc_scratch_bytes(int rows, int ic, int oc) {
    if (rows < 1 || ic <= 0 || oc <= 0) return 0;
    if (exl3::ts::eligible(rows, ic, oc)) return exl3::ts::scratch_bytes(rows, ic, oc);
    if (exl3::tc::use_dense(rows, ic, oc)) return exl3::tc::xh_bytes(rows, ic) + (size_t)ic * oc * 2;   // + the rebuilt weight
    const int sk = exl3::tc::choose_splitk(rows, ic, oc);
    return exl3::tc::xh_bytes(rows, ic) + (sk > 1 ? (size_t)sk * rows * oc * 4 : 0);
}

extern "C" int exl3_gemm_tc(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
                            void *scratch, size_t scratch_bytes, int rows, int ic, int oc, int k_times_2, int mcg,
                            int mul1, int x_is_bf16, void *stream) {
    return exl3_gemm_tc_ex(x, trellis, y, suh, svh, scratch, scratch_bytes, rows, ic, oc, k_times_2, mcg, mul1,
                           x_is_bf16, oc, nullptr, stream);
}

extern "C" int exl3_gemm_tc_ex(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
                               void *scratch, size_t scratch_bytes, int rows, int ic, int oc, int k_times_2, int mcg,
                               int mul1, int x_is_bf16, int ldy, const exl3_gemv_fusion *fusion, void *stream) {
    using namespace exl3;
    using namespace exl3::tc;
    if (!x || !trellis || !y || !suh || !svh || !scratch) return EXL3_E_NULL;
    void *xh_scratch = scratch;
    if (rows < 1 || ic <= 0 || oc <= 0 || (ic & 127) || (oc & 127) || oc / kBM > 65535 || ldy < oc) return EXL3_E_SHAPE;
    if (mcg || mul1) return EXL3_E_UNSUPPORTED;
    const int K = integer_k(k_times_2);
    if (!K) return EXL3_E_UNSUPPORTED;
    if (!aligned(x, 8) || !aligned(y, 8) || !aligned(trellis, 16) || !aligned(scratch, 256) || !aligned(suh, 8) ||
        !aligned(svh, 8) || (ldy & 3))
        return EXL3_E_ALIGN;
    if (scratch_bytes < exl3_gemm_tc_scratch_bytes(rows, ic, oc)) return EXL3_E_WORKSPACE;
    XhFusion F;
    F.in_mode = 0; F.norm_w = nullptr; F.eps = 0.f; F.ldx = ic; F.ic = ic;
    const __half *residual = nullptr;
    int ld_res = ldy;
    if (fusion) {
        if (fusion->in_mode < 0 || fusion->in_mode > 2) return EXL3_E_UNSUPPORTED;
        F.in_mode = fusion->in_mode;
        F.norm_w = static_cast<const __half *>(fusion->norm_weight);
        F.eps = fusion->eps;
        F.ldx = fusion->ldx > 0 ? fusion->ldx : (fusion->in_mode == 2 ? 2 * ic : ic);
        residual = static_cast<const __half *>(fusion->residual);
        ld_res = fusion->ld_residual > 0 ? fusion->ld_residual : ldy;
        if ((F.ldx & 3) || (ld_res & 3) || (F.norm_w && !aligned(F.norm_w, 8)) || (residual && !aligned(residual, 8)))
            return EXL3_E_ALIGN;
        if (F.ldx < (F.in_mode == 2 ? 2 * ic : ic) || ld_res < oc) return EXL3_E_SHAPE;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    EncodeTiledFn enc = encode_fn();
    if (!enc) return EXL3_E_LAUNCH;

    if (ts::eligible(rows, ic, oc)) {
        // ---- up to 128 rows: codewords go from registers to tensor memory (exl3_gemm_ts.cuh)
        const int sk = ts::choose_splitk(ic, oc);
        const long long nblocks = (long long)rows * (ic / 128);
        const unsigned g1 = (unsigned)((nblocks + 7) / 8);
        const cudaError_t e1 =
            x_is_bf16 ? launch_pdl(xh_permute_kernel<true>, dim3(g1), dim3(256), 0, st, x, static_cast<const __half *>(suh),
                                   static_cast<__half *>(scratch), nblocks, ic / 128, F)
                      : launch_pdl(xh_permute_kernel<false>, dim3(g1), dim3(256), 0, st, x, static_cast<const __half *>(suh),
                                   static_cast<__half *>(scratch), nblocks, ic / 128, F);
        if (e1 != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
        ts::Params P;
        P.trellis = static_cast<const uint32_t *>(trellis);
        P.tokens = rows; P.npad = (rows + 15) & ~15;
        P.ic = ic; P.oc = oc; P.tiles_j = oc / 16; P.splitk = sk; P.one = 1u;
        P.b_slot_bytes = (P.npad * 128 + 1023) & ~1023;
        P.bufs = (ts::kTmemCols - 2 * P.npad) / 64;
        if (P.bufs > ts::kMaxBufs) P.bufs = ts::kMaxBufs;
        // always through fp32 partial sums (one slice at least): the post-pass then carries the output
        // pitch and the residual
        P.partial = reinterpret_cast<float *>(static_cast<unsigned char *>(scratch) + ts::xh_bytes(rows, ic));
        CUtensorMap map;
        const cuuint64_t gdim[2] = {(cuuint64_t)ic, (cuuint64_t)rows};
        const cuuint64_t gstr[1] = {(cuuint64_t)ic * 2};
        const cuuint32_t box[2] = {64u, (cuuint32_t)P.npad};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scratch, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return EXL3_E_LAUNCH;
        int rc;
        switch (K) {
            case 1: rc = ts::launch<1>(map, P, st); break;
            case 2: rc = ts::launch<2>(map, P, st); break;
            case 3: rc = ts::launch<3>(map, P, st); break;
            case 4: rc = ts::launch<4>(map, P, st); break;
            case 5: rc = ts::launch<5>(map, P, st); break;
            case 6: rc = ts::launch<6>(map, P, st); break;
            case 7: rc = ts::launch<7>(map, P, st); break;
            default: rc = ts::launch<8>(map, P, st); break;
        }
        if (rc != EXL3_OK) return rc;
        const long long nb = (long long)rows * (oc / 128);
        if (launch_pdl(reduce_had_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, st, (const float *)P.partial, sk,
                       static_cast<const __half *>(svh), static_cast<__half *>(y), nb, oc / 128, (size_t)rows * oc, ldy,
                       residual, ld_res) != cudaSuccess) {
            cudaGetLastError();
            return EXL3_E_LAUNCH;
        }
        return EXL3_OK;
    }
    if (use_dense(rows, ic, oc)) {
        // ---- many rows: rotate the activations, rebuild the weight once (transposed), dense tcgen05 GEMM on CTA pairs.
        // The output rotation and signs: in the GEMM's epilogue (tokens in the accumulator's lanes, a thread rotates
        // its token's 128-channel blocks in registers: no extra pass and no extra work on the weight), which needs
        // 16-byte aligned output rows and signs.  Otherwise either folded into the rebuilt weight (0.29 us per 2^20
        // weights on tcgen05, 0.89 on the legacy tensor path when the input dimension is not a multiple of 256) or
        // as a pass over the output (0.49 us per 2^20 outputs while it stays in L2, 1.22 beyond), whichever is
        // cheaper; a pitched output cannot be rotated in place afterwards and is always folded.
        const bool rot = (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(svh) & 15) == 0 && ldy % 8 == 0;
        const double had_per = (double)rows * oc * 2 > 96.0 * 1048576.0 ? 1.22 : 0.49;
        const bool fold = !rot && (had_per * rows > (ic % kFoldN == 0 ? 0.29 : 0.89) * ic || ldy != oc);
        if (residual) return EXL3_E_UNSUPPORTED;
        if (oc / 128 > 65535 || ic / 64 > 65535) return EXL3_E_SHAPE;
        __half *xh = static_cast<__half *>(scratch);
        __half *wt = reinterpret_cast<__half *>(static_cast<unsigned char *>(scratch) + xh_bytes(rows, ic));
        const long long nblocks = (long long)rows * (ic / 128);
        const unsigned g1 = (unsigned)((nblocks + 7) / 8);
        if (F.in_mode == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(suh) & 15) == 0 && F.ldx % 8 == 0) {
            const unsigned g4 = (unsigned)((nblocks + 31) / 32);
            if (x_is_bf16)
                xh_permute16_kernel<true><<<g4, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F.ldx);
            else
                xh_permute16_kernel<false><<<g4, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F.ldx);
        } else if (F.in_mode == 0) {
            const unsigned g4 = (unsigned)((nblocks + 31) / 32);
            if (x_is_bf16)
                xh_permute4_kernel<true><<<g4, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F.ldx);
            else
                xh_permute4_kernel<false><<<g4, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F.ldx);
        } else if (x_is_bf16) {
            xh_permute_kernel<true><<<g1, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F);
        } else {
            xh_permute_kernel<false><<<g1, 256, 0, st>>>(x, static_cast<const __half *>(suh), xh, nblocks, ic / 128, F);
        }
        if (cudaGetLastError() != cudaSuccess) return EXL3_E_LAUNCH;
        int rc;
        switch (K) {
            case 1: rc = launch_reconstruct_t<1>(trellis, svh, wt, ic, oc, fold, st); break;
            case 2: rc = launch_reconstruct_t<2>(trellis, svh, wt, ic, oc, fold, st); break;
            case 3: rc = launch_reconstruct_t<3>(trellis, svh, wt, ic, oc, fold, st); break;
            case 4: rc = launch_reconstruct_t<4>(trellis, svh, wt, ic, oc, fold, st); break;
            case 5: rc = launch_reconstruct_t<5>(trellis, svh, wt, ic, oc, fold, st); break;
            case 6: rc = launch_reconstruct_t<6>(trellis, svh, wt, ic, oc, fold, st); break;
            case 7: rc = launch_reconstruct_t<7>(trellis, svh, wt, ic, oc, fold, st); break;
            default: rc = launch_reconstruct_t<8>(trellis, svh, wt, ic, oc, fold, st); break;
        }
        if (rc != EXL3_OK) return rc;
        CUtensorMap wmap, xmap;
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)(kBN / 2)};
        const cuuint32_t estr[2] = {1, 1};
        const cuuint64_t gstr[1] = {(cuuint64_t)ic * 2};
        const cuuint64_t wdim[2] = {(cuuint64_t)ic, (cuuint64_t)oc};
        const cuuint64_t xdim[2] = {(cuuint64_t)ic, (cuuint64_t)rows};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, wt, wdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, xdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return EXL3_E_LAUNCH;
        DenseParams D;
        D.y = static_cast<__half *>(y);
        D.tokens = rows; D.ic = ic; D.oc = oc; D.ldy = ldy;
        D.npx = oc / kBM / 2;
        D.nty = (rows + kBN - 1) / kBN;
        D.npairs = 0;
        D.wide_st = (reinterpret_cast<uintptr_t>(y) & 31) == 0 && ldy % 16 == 0;
        if ((long long)D.npx * D.nty > 0x3fffffffLL) return EXL3_E_SHAPE;
        // the narrower boxes of a cut tile: of the token rows, or (epilogue rotation) of the weight rows
        struct TailCtx { EncodeTiledFn enc; void *xh; cuuint64_t xdim[2]; cuuint64_t gstr[1]; } tctx = {enc, xh, {xdim[0], xdim[1]}, {gstr[0]}};
        if (rot) { tctx.xh = wt; tctx.xdim[1] = wdim[1]; }
        auto tail_map = [](void *c, int box_rows, CUtensorMap *out) -> int {
            TailCtx *t = static_cast<TailCtx *>(c);
            const cuuint32_t tbox[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
            const cuuint32_t one[2] = {1, 1};
            return t->enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, t->xh, t->xdim, t->gstr, tbox, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
                       ? EXL3_OK : EXL3_E_LAUNCH;
        };
        if (rot) return launch_dense<true>(wmap, xmap, tail_map, &tctx, D, static_cast<const __half *>(svh), st);
        rc = launch_dense<false>(wmap, xmap, tail_map, &tctx, D, nullptr, st);
        if (rc != EXL3_OK || fold) return rc;
        return exl3_had_r_128(y, y, nullptr, svh, 1.0f, rows, oc, stream);
    }
    const int splitk = choose_splitk(rows, ic, oc);
    // the unsplit shared-memory kernel writes y itself and rotates it in place: no pitch, no residual
    if (splitk == 1 && (ldy != oc || residual)) return EXL3_E_UNSUPPORTED;

    // 1. rotate and permute the activations
    const long long nblocks = (long long)rows * (ic / 128);
    const unsigned g1 = (unsigned)((nblocks + 7) / 8);
    if (x_is_bf16)
        xh_permute_kernel<true><<<g1, 256, 0, st>>>(x, static_cast<const __half *>(suh), static_cast<__half *>(xh_scratch), nblocks, ic / 128, F);
    else
        xh_permute_kernel<false><<<g1, 256, 0, st>>>(x, static_cast<const __half *>(suh), static_cast<__half *>(xh_scratch), nblocks, ic / 128, F);
    if (cudaGetLastError() != cudaSuccess) return EXL3_E_LAUNCH;

    // 2. decode + tcgen05 contraction
    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)ic, (cuuint64_t)rows};
    const cuuint64_t gstr[1] = {(cuuint64_t)ic * 2};
    const int box_rows = rows >= kBN ? kBN : ((rows + 15) & ~15);
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh_scratch, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return EXL3_E_LAUNCH;
    Params P;
    P.trellis = static_cast<const uint32_t *>(trellis);
    P.y = static_cast<__half *>(y);
    P.tokens = rows; P.ic = ic; P.oc = oc; P.ldy = oc; P.tiles_j = oc / 16; P.one = 1u;
    P.splitk = splitk;
    P.box_rows = box_rows;
    {
        int cols = 32;
        const int need = rows > kBN ? kBN * kMaxHalves : box_rows;
        while (cols < need) cols <<= 1;
        P.tmem_cols = cols;
    }
    P.b_slot_bytes = (box_rows * kBK * 2 + 1023) & ~1023;
    P.partial = splitk > 1 ? reinterpret_cast<float *>(static_cast<unsigned char *>(scratch) + xh_bytes(rows, ic)) : nullptr;
    int rc;
    switch (K) {
        case 1: rc = launch<1>(map, P, st); break;
        case 2: rc = launch<2>(map, P, st); break;
        case 3: rc = launch<3>(map, P, st); break;
        case 4: rc = launch<4>(map, P, st); break;
        case 5: rc = launch<5>(map, P, st); break;
        case 6: rc = launch<6>(map, P, st); break;
        case 7: rc = launch<7>(map, P, st); break;
        default: rc = launch<8>(map, P, st); break;
    }
    if (rc != EXL3_OK) return rc;

    // 3. output rotation and signs (in place), or the split-K reduction fused with them
    if (splitk == 1) return exl3_had_r_128(y, y, nullptr, svh, 1.0f, rows, oc, stream);
    const long long nb = (long long)rows * (oc / 128);
    reduce_had_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, st>>>(P.partial, splitk, static_cast<const __half *>(svh),
                                                               static_cast<__half *>(y), nb, oc / 128, (size_t)rows * oc, ldy,
                                                               residual, ld_res);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// All shards of a fused layer (qkv_proj, gate_up_proj) at 17..128 rows: three launches in total.
namespace exl3 { namespace ts {
struct GroupPlan {
    int splitk, units;
    size_t xh_off[EXL3_MAX_SHARDS], partial_off[EXL3_MAX_SHARDS], total;
};
static int plan_group(const exl3_shard *sh, int n, int rows, int ic, GroupPlan &pl) {
    if (!sh) return EXL3_E_NULL;
    if (n < 1 || n > EXL3_MAX_SHARDS || rows < 1 || ic <= 0 || (ic & 127)) return EXL3_E_SHAPE;
    if (rows > kMaxTokens) return EXL3_E_UNSUPPORTED;
    int units = 0;
    for (int i = 0; i < n; ++i) {
        if (sh[i].oc <= 0 || (sh[i].oc & 127) || sh[i].out_col < 0 || (sh[i].out_col & 3)) return EXL3_E_SHAPE;
        if (sh[i].mcg || sh[i].mul1 || !integer_k(sh[i].k_times_2)) return EXL3_E_UNSUPPORTED;
        if (!sh[i].trellis || !sh[i].suh || !sh[i].svh) return EXL3_E_NULL;
        if (!aligned(sh[i].trellis, 16) || !aligned(sh[i].suh, 8) || !aligned(sh[i].svh, 8)) return EXL3_E_ALIGN;
        units += (sh[i].oc + kOcCta - 1) / kOcCta;
    }
    // every shard has the same input size, hence the same work per output block: one slice count for all
    int sk = 148 / units;
    if (sk > ic / 64 / 4) sk = ic / 64 / 4;
    if (sk < 1) sk = 1;
    pl.splitk = sk;
    pl.units = units;
    size_t off = 0;
    for (int i = 0; i < n; ++i) { pl.xh_off[i] = off; off += xh_bytes(rows, ic); }
    for (int i = 0; i < n; ++i) { pl.partial_off[i] = off; off += (((size_t)sk * rows * sh[i].oc * 4) + 255) & ~(size_t)255; }
    pl.total = off;
    return EXL3_OK;
}
} }

extern "C" size_t exl3_gemm_tc_grouped_scratch_bytes(const exl3_shard *shards, int nshards, int rows, int ic) {
    exl3::ts::GroupPlan pl;
    if (exl3::ts::plan_group(shards, nshards, rows, ic, pl) != EXL3_OK) return 0;
    return pl.total;
}

extern "C" int exl3_gemm_tc_grouped(const exl3_shard *shards, int nshards, const void *x, void *y, int rows, int ic,
                                    int ldy, void *scratch, size_t scratch_bytes, int x_is_bf16,
                                    const exl3_gemv_fusion *fusion, void *stream) {
    using namespace exl3;
    using namespace exl3::tc;
    ts::GroupPlan pl;
    const int rcp = ts::plan_group(shards, nshards, rows, ic, pl);
    if (rcp != EXL3_OK) return rcp;
    if (!x || !y || !scratch) return EXL3_E_NULL;
    if (!aligned(x, 8) || !aligned(y, 8) || !aligned(scratch, 256) || (ldy & 3)) return EXL3_E_ALIGN;
    for (int i = 0; i < nshards; ++i)
        if (shards[i].out_col + shards[i].oc > ldy) return EXL3_E_SHAPE;
    if (scratch_bytes < pl.total) return EXL3_E_WORKSPACE;
    XhFusion F;
    F.in_mode = 0; F.norm_w = nullptr; F.eps = 0.f; F.ldx = ic; F.ic = ic;
    const __half *residual = nullptr;
    int ld_res = ldy;
    if (fusion) {
        if (fusion->in_mode < 0 || fusion->in_mode > 2) return EXL3_E_UNSUPPORTED;
        F.in_mode = fusion->in_mode;
        F.norm_w = static_cast<const __half *>(fusion->norm_weight);
        F.eps = fusion->eps;
        F.ldx = fusion->ldx > 0 ? fusion->ldx : (fusion->in_mode == 2 ? 2 * ic : ic);
        residual = static_cast<const __half *>(fusion->residual);
        ld_res = fusion->ld_residual > 0 ? fusion->ld_residual : ldy;
        if ((F.ldx & 3) || (ld_res & 3) || (F.norm_w && !aligned(F.norm_w, 8)) || (residual && !aligned(residual, 8)))
            return EXL3_E_ALIGN;
        if (F.ldx < (F.in_mode == 2 ? 2 * ic : ic)) return EXL3_E_SHAPE;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    EncodeTiledFn enc = encode_fn();
    if (!enc) return EXL3_E_LAUNCH;
    unsigned char *base = static_cast<unsigned char *>(scratch);

    // 1. rotated activations of every shard
    XhGroup XG;
    XG.nshards = nshards;
    for (int i = 0; i < nshards; ++i) {
        XG.suh[i] = static_cast<const __half *>(shards[i].suh);
        XG.xh[i] = reinterpret_cast<__half *>(base + pl.xh_off[i]);
    }
    const long long nblocks = (long long)rows * (ic / 128);
    const unsigned g1 = (unsigned)((nblocks * nshards + 7) / 8);
    const cudaError_t e1 = x_is_bf16 ? launch_pdl(xh_permute_grouped_kernel<true>, dim3(g1), dim3(256), 0, st, x, XG, nblocks, ic / 128, F)
                                     : launch_pdl(xh_permute_grouped_kernel<false>, dim3(g1), dim3(256), 0, st, x, XG, nblocks, ic / 128, F);
    if (e1 != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }

    // 2. decode + contraction
    ts::MapPack maps;
    ts::GroupArgs G;
    G.nshards = nshards;
    const int npad = (rows + 15) & ~15;
    int bufs = (ts::kTmemCols - 2 * npad) / 64;
    if (bufs > ts::kMaxBufs) bufs = ts::kMaxBufs;
    const int b_slot_bytes = (npad * 128 + 1023) & ~1023;
    size_t smem = 0;
    int ctas = 0;
    for (int i = 0; i < nshards; ++i) {
        ts::Params &P = G.p[i];
        P.trellis = static_cast<const uint32_t *>(shards[i].trellis);
        P.partial = reinterpret_cast<float *>(base + pl.partial_off[i]);
        P.tokens = rows; P.npad = npad; P.ic = ic; P.oc = shards[i].oc; P.tiles_j = shards[i].oc / 16;
        P.splitk = pl.splitk; P.b_slot_bytes = b_slot_bytes; P.bufs = bufs; P.one = 1u;
        G.K[i] = integer_k(shards[i].k_times_2);
        G.cta_begin[i] = ctas;
        ctas += ((shards[i].oc + ts::kOcCta - 1) / ts::kOcCta) * pl.splitk;
        const size_t sm = ts::smem_bytes(G.K[i], bufs, b_slot_bytes);
        smem = sm > smem ? sm : smem;
        const cuuint64_t gdim[2] = {(cuuint64_t)ic, (cuuint64_t)rows};
        const cuuint64_t gstr[1] = {(cuuint64_t)ic * 2};
        const cuuint32_t box[2] = {64u, (cuuint32_t)npad};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base + pl.xh_off[i], gdim, gstr, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return EXL3_E_LAUNCH;
    }
    G.cta_begin[nshards] = ctas;
    for (int i = nshards; i < EXL3_MAX_SHARDS; ++i) maps.m[i] = maps.m[0];
    if (smem > 226 * 1024) return EXL3_E_SHAPE;
    if (cudaFuncSetAttribute(ts::gemm_ts_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    if (launch_pdl(ts::gemm_ts_grouped_kernel, dim3((unsigned)ctas), dim3(ts::kThreads), smem, st, maps, G) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }

    // 3. slices summed, output rotation, signs, residual, fp16 into the shards' column blocks
    ReduceGroup RG;
    RG.nshards = nshards;
    long long nb = 0;
    for (int i = 0; i < nshards; ++i) {
        RG.blk_begin[i] = nb;
        nb += (long long)rows * (shards[i].oc / 128);
        RG.partial[i] = reinterpret_cast<const float *>(base + pl.partial_off[i]);
        RG.svh[i] = static_cast<const __half *>(shards[i].svh);
        RG.splitk[i] = pl.splitk;
        RG.blocks_per_row[i] = shards[i].oc / 128;
        RG.out_col[i] = shards[i].out_col;
        RG.slice_elems[i] = (long long)rows * shards[i].oc;
    }
    RG.blk_begin[nshards] = nb;
    if (launch_pdl(reduce_had_grouped_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, st, RG, static_cast<__half *>(y), ldy,
                   residual, ld_res) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    return EXL3_OK;
}

