// EXL3 GEMM for a few dozen rows (17 .. 128): the decoded weights never touch shared memory.
//
//     Yt[tokens][oc] = Xh[tokens][ic] . W(trellis)[ic][oc]          (fp16 in, fp32 accumulate)
//
// Decode warps turn the packed trellis into fp16 weights in registers exactly as the decode GEMV
// reads it (one 32-weight chunk per lane, four tiles side by side per warp; weight = sum of the
// codeword's two halves, the same rounding as reconstruct) and store them with tcgen05.st straight
// into TENSOR MEMORY, where tcgen05.mma reads them as its A operand; the activations (B operand)
// come from shared memory, loaded by TMA.  The registers of an mma.sync A fragment are what
// tcgen05.st.16x256b writes as a 16-row x 8-column block, so the chunk layout of the packed format
// maps onto tensor memory without any shuffle: per chunk two stores of eight registers.
//
// Issuing a tcgen05 instruction costs the issuing thread about 55 cycles (measured), so the loop
// is organised to need few of them: a ROUND is four tile rows (64 input channels, one tile row per
// decode group), and costs each of the two issuing threads one wait, one fence, four MMAs and one commit.
//
// CTA = 256 output channels (128 in the last block of an odd width) x a slice of the input channels x up
// to 128 tokens, one CTA per SM:
//   warp 0        lanes 0..3: packed trellis of the four decode groups (1-D bulk copies into
//                 per-group rings)
//   warp 19       activation tiles (2-D tiled TMA, 128-byte swizzle), one per round
//   warps 1, 18   issue tcgen05.mma (one lane each: accumulator X and accumulator Y) and commit to
//                 mbarriers; warp 1 also allocates and frees the tensor memory
//   warps 2..17   four decode groups of four warps (one warp per TMEM lane quarter = 64 output
//                 channels); group g takes the tile rows g, g+4, ... of the slice; afterwards the
//                 epilogue (tcgen05.ld, fp32 partial sums)
// Tensor memory: accumulators X and Y (rows a = 0,1 and a = 2,3 of every four-tile span) in columns
// [0, 2 npad), then 4 .. 7 A buffers of 64 columns (16 per group: 8 for X, 8 for Y).
// The K order inside a tile row is k = 4 (ic & 3) + 2 (ic >> 3) + ((ic >> 2) & 1), the order in which
// a lane's registers hold it; the activation pre-pass writes the same order.
// Every wait is bounded; a wait that runs out sets the status word and the kernel still frees its
// tensor memory and exits.
#pragma once
#include "exl3_tcgen05.cuh"

namespace exl3 {
namespace ts {
using namespace t5;

constexpr int kOcCta = 256;
constexpr int kGroups = 4;
constexpr int kDecodeWarps = 4 * kGroups;
constexpr int kThreads = 32 * (4 + kDecodeWarps);   // + trellis producer, activation producer, two MMA issuers
constexpr int kWarpMmaY = 2 + kDecodeWarps;         // warp 1 issues for accumulator X, this one for Y
constexpr int kWarpActs = 3 + kDecodeWarps;         // activation tiles
constexpr int kMaxBufs = 7;             // rounds in flight (A buffers in tensor memory = activation tiles in shared
                                        // memory): as many as the 512 columns allow, (512 - 2 npad) / 64
// Packed tile rows in flight per group: about 12 KB per group (48 KB per SM) keeps the stream ahead of
// the decode warps; a tile row of the CTA's sixteen tiles is 512 K bytes.
__host__ __device__ constexpr int raw_depth(int K) { return K <= 2 ? 12 : K == 3 ? 8 : K == 4 ? 6 : K == 5 ? 5 : 4; }
constexpr int kMaxRawDepth = 12;
constexpr int kMaxTokens = 128;
constexpr int kTmemCols = 512;

struct Params {
    const uint32_t *trellis;
    float *partial;        // [splitk][tokens][oc] fp32: the post-pass sums the slices, rotates and writes y
    int tokens, npad;      // npad: tokens rounded up to 16 (MMA N, TMA box rows)
    int ic, oc, tiles_j, splitk;
    int b_slot_bytes;      // npad * 128, rounded up to 1024
    int bufs;              // rounds in flight, 4 .. kMaxBufs
    uint32_t one;
};

struct Barriers {
    uint64_t raw_full[kGroups][kMaxRawDepth], raw_empty[kGroups][kMaxRawDepth];
    uint64_t full[kMaxBufs];        // all sixteen decode warps have stored their chunk of the round AND its
                                    // activation tile has landed (sixteen arrivals + the producer's, with the bytes)
    uint64_t empty[kMaxBufs];       // both issuers' MMAs of the round are done: A buffer and activation tile are free
    uint64_t acc_full;
    uint32_t tmem_base;
};

// One chunk: packed words -> 3INST codewords -> fp16 weights, two per register, in the order of the two
// tensor-memory stores.  Fragment (a, b) = codewords z[8a + 4b ..+3]: output rows r and r+8 (codewords
// 0/2 and 1/3) at input channels 8b + q (0, 1) and 8b + 4 + q (2, 3).  Register (a, b, row half) holds
// the two input channels of one row; the store puts b = 0, 1 side by side, so column 2q + b of the row
// carries K elements 4q + 2b and 4q + 2b + 1.
template <int K>
__device__ __forceinline__ void decode_pack(const uint32_t (&wd)[K + 1], uint32_t (&wreg)[16], const DecodeConsts &dc) {
    uint32_t z[32];
    decode_chunk_fast<K>(wd, z, dc);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int hr = 0; hr < 2; ++hr)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint32_t z0 = z[8 * a + 4 * b + hr], z1 = z[8 * a + 4 * b + 2 + hr];
                const __half2 w0 = __hadd2(__low2half2(*reinterpret_cast<const __half2 *>(&z0)),
                                           __high2half2(*reinterpret_cast<const __half2 *>(&z0)));
                const __half2 w1 = __hadd2(__low2half2(*reinterpret_cast<const __half2 *>(&z1)),
                                           __high2half2(*reinterpret_cast<const __half2 *>(&z1)));
                const __half2 pk = __lows2half2(w0, w1);
                // [a & 1 selects the store][a >> 1: accumulator X then Y][row half][b]
                wreg[8 * (a & 1) + 4 * (a >> 1) + 2 * hr + b] = *reinterpret_cast<const uint32_t *>(&pk);
            }
}

// The work of one CTA: output block `bx` (256 channels) and input slice `by` of one shard.
template <int K>
__device__ __forceinline__ void ts_body(const CUtensorMap *xmap, const Params &P, const int bx, const int by,
                                        unsigned char *smem_dyn) {
    unsigned char *smem = smem_dyn + ((1024u - (s32(smem_dyn) & 1023u)) & 1023u);
    constexpr int kRawWords = 16 * 8 * K;                  // one tile row of the CTA's sixteen tiles
    constexpr uint32_t kRawBytes = kRawWords * 4;
    constexpr int kRawDepth = raw_depth(K);
    unsigned char *const smB = smem;
    Barriers &S = *reinterpret_cast<Barriers *>(smB + (size_t)P.bufs * P.b_slot_bytes);
    uint32_t *const raw = reinterpret_cast<uint32_t *>(reinterpret_cast<unsigned char *>(&S) + 1024);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned *const status = &tc::g_tc_status;
    // slice of the input dimension, in units of four tile rows (one per decode group)
    const int units = P.ic / 64;
    const int u0 = (int)((long long)by * units / P.splitk);
    const int u1 = (int)((long long)(by + 1) * units / P.splitk);
    const int r0 = 4 * u0;                 // first tile row
    const int nper = u1 - u0;              // rounds = tile rows per group

    if (threadIdx.x == 0) {
        for (int g = 0; g < kGroups; ++g) {
            for (int s = 0; s < kRawDepth; ++s) { mbar_init(s32(&S.raw_full[g][s]), 1); mbar_init(s32(&S.raw_empty[g][s]), 4); }
        }
        for (int s = 0; s < P.bufs; ++s) { mbar_init(s32(&S.full[s]), kDecodeWarps + 1); mbar_init(s32(&S.empty[s]), 2); }
        mbar_init(s32(&S.acc_full), 2);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(s32(&S.tmem_base), kTmemCols);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = S.tmem_base;
    const uint32_t d_x = tmem, d_y = tmem + (uint32_t)P.npad;
    // Everything above touched only this CTA's own state; the packed trellis is constant.  Whoever
    // reads the rotated activations or writes results waits for the kernels before this one first.
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t a_cols = tmem + 2u * (uint32_t)P.npad;       // A buffer b, group g: X at a_cols + 64 b + 16 g, Y 8 columns further

    if (warp == 0) {
        // ---------------- packed trellis: lane g feeds decode group g (tile rows r0 + g, r0 + g + 4, ...).
        // The four lanes stay in ONE loop and issue their copies with one instruction: issuing a bulk
        // copy holds the warp for about a quarter of a microsecond, and four diverged lanes would pay it
        // four times per round (measured: that alone bounded the kernel at ~1500 cycles per round).
        const int g = lane & 3;
        const uint32_t *src = P.trellis + ((size_t)(r0 + g) * P.tiles_j + (size_t)bx * 16) * (size_t)(8 * K);
        const size_t src_step = (size_t)4 * P.tiles_j * (8 * K);
        // the last block of a shard whose width is an odd multiple of 128 has eight tiles: the upper two
        // lane quarters then decode whatever the ring holds, into accumulator rows that are never read
        const int ntiles = min(16, P.tiles_j - bx * 16);
        const uint32_t row_bytes = (uint32_t)ntiles * (8 * K) * 4;
        bool ok = true;
        Cursor rc(0, kRawDepth);
        for (int s = 0; s < nper; ++s, rc.advance(1)) {
            if (lane < kGroups && rc.wrapped) ok = mbar_wait(s32(&S.raw_empty[g][rc.idx]), rc.phase ^ 1u, status, 40);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane < kGroups) {
                const uint32_t bar = s32(&S.raw_full[g][rc.idx]);
                mbar_expect_tx(bar, row_bytes);
                bulk_g2s(s32(raw + (size_t)(g * kRawDepth + rc.idx) * kRawWords), src + (size_t)s * src_step, row_bytes, bar);
            }
        }
    } else if (warp == kWarpActs) {
        // ---------------- activation tiles: one per round (64 input channels), a warp of its own so that
        // its waits do not hold back the trellis stream
        if (lane == 0) {
            const uint32_t box_bytes = (uint32_t)P.npad * 128u;
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            Cursor bc(0, P.bufs);
            for (int j = 0; j < nper && ok; ++j, bc.advance(1)) {
                if (bc.wrapped) ok = mbar_wait(s32(&S.empty[bc.idx]), bc.phase ^ 1u, status, 100);
                if (!ok) break;
                const uint32_t bar = s32(&S.full[bc.idx]);
                mbar_expect_tx(bar, box_bytes);
                tma_2d(s32(smB + (size_t)bc.idx * P.b_slot_bytes), xmap, 64 * (u0 + j), 0, bar);
            }
        }
    } else if (warp == 1 || warp == kWarpMmaY) {
        // ---------------- MMA issue: per round four MMAs (four tile rows) into this issuer's accumulator, one commit
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(128, P.npad);
            const uint64_t bdesc0 = umma_desc_sw128(s32(smB));      // activation tile 0; the others follow at b_slot_bytes
            const uint32_t d_acc = warp == 1 ? d_x : d_y;
            const uint32_t a_off = warp == 1 ? 0u : 8u;
            bool ok = true;
            Cursor bc(0, P.bufs);
            for (int s = 0; s < nper && ok; ++s, bc.advance(1)) {
                TC_CLK(m0);
                ok = mbar_wait(s32(&S.full[bc.idx]), bc.phase, status, 0);
                TC_CLK(m1);
                TC_ACC(0, m0, m1);
                if (!ok) break;
                fence_after_sync();
                const uint32_t a = a_cols + 64u * (uint32_t)bc.idx + a_off;
                // descriptor start addresses are in 16-byte units: tile row g of the round is 32 bytes further
                const uint64_t bk = bdesc0 + (uint64_t)((uint32_t)bc.idx * (uint32_t)P.b_slot_bytes >> 4);
                umma_f16_ts(d_acc, a, bk, idesc, s ? 1u : 0u);
                umma_f16_ts(d_acc, a + 16u, bk + 2u, idesc, 1u);
                umma_f16_ts(d_acc, a + 32u, bk + 4u, idesc, 1u);
                umma_f16_ts(d_acc, a + 48u, bk + 6u, idesc, 1u);
                umma_commit(s32(&S.empty[bc.idx]));
                TC_CLK(m3);
                TC_ACC(2, m1, m3);
            }
            umma_commit(s32(&S.acc_full));
        }
    } else {
        // ---------------- decode warps
        const int dw = warp - 2;
        const int g = dw >> 2;
        const int quad = warp & 3;                 // TMEM lanes 32 quad .. +31 <-> tiles 4 quad .. +3 of the CTA's sixteen
        const DecodeConsts dc(P.one);
        const int nxt_lane = (lane & 24) | ((lane + 1) & 7);
        const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
        bool ok = true;
        Cursor rc(0, kRawDepth), ac(0, P.bufs);
        // Two rounds per iteration: the sixteen decode warps move in lock step (a round's MMAs need all of
        // them), so within one warp the barrier polls, shared-memory loads, shuffles and tensor-memory
        // stores of a single chunk are a chain of exposed latencies.  Two independent chunks halve them.
        // The completion of a pair's stores is awaited, and announced, after the next pair is decoded.
        int pending[2] = {-1, -1};
        auto announce = [&]() {
            if (pending[0] >= 0) {
                tmem_wait_st();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(s32(&S.full[pending[0]]));
                    if (pending[1] >= 0) mbar_arrive(s32(&S.full[pending[1]]));
                }
                pending[0] = pending[1] = -1;
            }
        };
        for (int s = 0; s < nper && ok; s += 2) {
            const bool two = s + 1 < nper;
            TC_CLK(c0);
            const int ri0 = rc.idx;
            const uint32_t rp0 = rc.phase;
            rc.advance(1);
            const int ri1 = rc.idx;
            const uint32_t rp1 = rc.phase;
            if (two) rc.advance(1);
            ok = mbar_wait(s32(&S.raw_full[g][ri0]), rp0, status, 40);
            if (ok && two) ok = mbar_wait(s32(&S.raw_full[g][ri1]), rp1, status, 40);
            TC_CLK(c1);
            TC_ACC(0, c0, c1);
            if (!ok) break;
            uint32_t wd0[K + 1], wd1[K + 1];
            const uint32_t *wsrc = raw + (size_t)(g * kRawDepth) * kRawWords + quad * (32 * K) + lane * K;
            load_words<K>(wsrc + (size_t)ri0 * kRawWords, wd0);
            if (two) load_words<K>(wsrc + (size_t)ri1 * kRawWords, wd1);
            else {
#pragma unroll
                for (int k = 0; k < K; ++k) wd1[k] = 0u;
            }
            wd0[K] = __shfl_sync(0xffffffffu, wd0[0], nxt_lane);
            wd1[K] = __shfl_sync(0xffffffffu, wd1[0], nxt_lane);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(s32(&S.raw_empty[g][ri0]));
                if (two) mbar_arrive(s32(&S.raw_empty[g][ri1]));
            }
            uint32_t wreg0[16], wreg1[16];
            decode_pack<K>(wd0, wreg0, dc);
            if (two) decode_pack<K>(wd1, wreg1, dc);
            TC_CLK(c2);
            TC_ACC(1, c1, c2);
            announce();                            // the previous pair's stores have had two decodes to land
            const int ai0 = ac.idx;
            if (ac.wrapped) ok = mbar_wait(s32(&S.empty[ai0]), ac.phase ^ 1u, status, 40);
            ac.advance(1);
            const int ai1 = ac.idx;
            if (two) {
                if (ok && ac.wrapped) ok = mbar_wait(s32(&S.empty[ai1]), ac.phase ^ 1u, status, 40);
                ac.advance(1);
            }
            TC_CLK(c3);
            TC_ACC(2, c2, c3);
            if (!ok) break;
            fence_after_sync();
            const uint32_t tg = a_cols + lane_base + 16u * (uint32_t)g;
            tmem_st_16x256b_x2(tg + 64u * (uint32_t)ai0, wreg0[0], wreg0[1], wreg0[2], wreg0[3], wreg0[4], wreg0[5], wreg0[6], wreg0[7]);
            tmem_st_16x256b_x2(tg + 64u * (uint32_t)ai0 + (16u << 16), wreg0[8], wreg0[9], wreg0[10], wreg0[11], wreg0[12], wreg0[13], wreg0[14], wreg0[15]);
            pending[0] = ai0;
            if (two) {
                tmem_st_16x256b_x2(tg + 64u * (uint32_t)ai1, wreg1[0], wreg1[1], wreg1[2], wreg1[3], wreg1[4], wreg1[5], wreg1[6], wreg1[7]);
                tmem_st_16x256b_x2(tg + 64u * (uint32_t)ai1 + (16u << 16), wreg1[8], wreg1[9], wreg1[10], wreg1[11], wreg1[12], wreg1[13], wreg1[14], wreg1[15]);
                pending[1] = ai1;
            }
            TC_CLK(c4);
            TC_ACC(3, c3, c4);
        }
        announce();

        // ---------------- epilogue: accumulators -> fp32 partial sums
        ok = mbar_wait(s32(&S.acc_full), 0, status, 200) && ok;
        fence_after_sync();
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int n16 = P.npad / 16;
        const int i16 = lane & 15, gg = i16 & 7, hi8 = i16 >> 3;
        for (int o = g; o < 2 * n16; o += kGroups) {
            const int R = o / n16, c0 = (o - R * n16) * 16;
            uint32_t v[16];
            tmem_ld_32x32b_x16(tmem + lane_base + (uint32_t)(R * P.npad + c0), v);
            const int a = 2 * R + (lane >> 4);
            const int oc_idx = bx * kOcCta + 64 * quad + 16 * (gg >> 1) + 4 * a + 2 * hi8 + (gg & 1);
            if (ok) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = c0 + j;
                    if (tok < P.tokens && oc_idx < P.oc) {
                        P.partial[((size_t)by * P.tokens + tok) * P.oc + oc_idx] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }

    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem, kTmemCols);
    }
}


template <int K>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ts_kernel(const __grid_constant__ CUtensorMap xmap, const Params P) {
    extern __shared__ unsigned char smem_dyn[];
    ts_body<K>(&xmap, P, blockIdx.x, blockIdx.y, smem_dyn);
}

// All shards of a fused layer in one launch: CTAs are numbered shard by shard (output block fastest),
// every shard brings its own bitrate, tensor map (its own rotated activations) and partial sums.
struct GroupArgs {
    int nshards;
    int cta_begin[EXL3_MAX_SHARDS + 1];
    int K[EXL3_MAX_SHARDS];
    Params p[EXL3_MAX_SHARDS];
};
struct MapPack {
    CUtensorMap m[EXL3_MAX_SHARDS];
};
__global__ void __launch_bounds__(kThreads, 1)
gemm_ts_grouped_kernel(const __grid_constant__ MapPack maps, const __grid_constant__ GroupArgs G) {
    extern __shared__ unsigned char smem_dyn[];
    int s = 0;
    while (s + 1 < G.nshards && (int)blockIdx.x >= G.cta_begin[s + 1]) ++s;
    const Params &P = G.p[s];
    const int local = blockIdx.x - G.cta_begin[s];
    const int ux = (P.oc + kOcCta - 1) / kOcCta;
    const int bx = local % ux, by = local / ux;
    switch (G.K[s]) {
        case 1: ts_body<1>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 2: ts_body<2>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 3: ts_body<3>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 4: ts_body<4>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 5: ts_body<5>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 6: ts_body<6>(&maps.m[s], P, bx, by, smem_dyn); break;
        case 7: ts_body<7>(&maps.m[s], P, bx, by, smem_dyn); break;
        default: ts_body<8>(&maps.m[s], P, bx, by, smem_dyn); break;
    }
}

__host__ __device__ constexpr size_t smem_bytes(int K, int bufs, int b_slot_bytes) {
    return (size_t)bufs * b_slot_bytes + 1024 /*barriers*/ + (size_t)kGroups * raw_depth(K) * (16 * 8 * K) * 4 + 1024 /*alignment*/;
}

template <int K>
static int launch(const CUtensorMap &map, const Params &P, cudaStream_t st) {
    const size_t smem = smem_bytes(K, P.bufs, P.b_slot_bytes);
    if (smem > 226 * 1024) return EXL3_E_SHAPE;
    if (cudaFuncSetAttribute(gemm_ts_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    dim3 grid((P.oc + kOcCta - 1) / kOcCta, P.splitk);
    if (launch_pdl(gemm_ts_kernel<K>, grid, dim3(kThreads), smem, st, map, P) != cudaSuccess) {
        cudaGetLastError();
        return EXL3_E_LAUNCH;
    }
    return EXL3_OK;
}

// the shapes this path takes; everything else stays on the shared-memory kernel
static bool eligible(int rows, int ic, int oc) { return rows <= kMaxTokens && (oc % 128) == 0 && (ic % 128) == 0; }

static int choose_splitk(int ic, int oc) {
    const int ctas = (oc + kOcCta - 1) / kOcCta, units = ic / 64;
    int sk = (148 + ctas / 2) / ctas;
    if (sk > units / 4) sk = units / 4;
    return sk < 1 ? 1 : sk;
}
static size_t xh_bytes(int rows, int ic) { return (((size_t)rows * ic * 2) + 255) & ~(size_t)255; }
static size_t scratch_bytes(int rows, int ic, int oc) {
    return xh_bytes(rows, ic) + (size_t)choose_splitk(ic, oc) * rows * oc * 4;     // always at least one slice of partial sums
}

}  // namespace ts
}  // namespace exl3
