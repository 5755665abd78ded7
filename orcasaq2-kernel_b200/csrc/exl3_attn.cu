// Decode attention (one query token per sequence) over a contiguous fp16 KV cache, head size 256,
// grouped-query layout with up to eight query heads per KV head:
//     out[b, h] = softmax(q[b, h] . K[b, h / G]^T * scale) . V[b, h / G]
// The step is bound by the HBM read of K and V, so the kernel is built around keeping that stream
// busy at any batch size: the sequence is cut into splits (grid.x) so that even one sequence fills
// the GPU, every warp runs a private ring of 16-token stages filled with 16-byte asynchronous
// copies (no block-wide synchronisation in the main loop), and each K / V byte is read from shared
// memory exactly once by an ldmatrix that feeds mma.m16n8k16:
//     S[head][token]  = Q (A operand, heads on the M side) x K^T (B operand, plain ldmatrix)
//     O^T[dim][head]  = V^T (A operand, ldmatrix.trans)    x P^T (B operand)
// In this orientation the accumulator fragment of S is, register for register, the B fragment of
// the second product, so the probabilities never leave registers.  Shared-memory rows are 512
// bytes; 16-byte chunks are XOR-swizzled with the row number so that ldmatrix has no bank
// conflicts.  Splits are merged by a second small kernel (log-sum-exp weights, fixed order).
//
// fp8 caches (e4m3, one scale per tensor for K and one for V, the form `--kv-cache-dtype fp8` keeps): the same
// kernel with rows of 256 bytes, so a ring stage is half as large and two CTAs share an SM.  ldmatrix moves pairs
// of fp8 values as its 16-bit units; the pairs are widened to fp16 in registers (cvt.rn.f16x2.e4m3x2) and fed to
// the same mma.m16n8k16.  The order in which head dimensions meet inside a 16-wide k step is then a permutation of
// the fp16 one, which the query fragments (first product) and the accumulator-to-output mapping (second product)
// follow; the scales fold into the softmax scale and the final normalisation.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "exl3_common.cuh"

namespace exl3 {

constexpr int kHD = 256;                 // head size (elements)
constexpr int kRowBytes = kHD * 2;       // one token of K or V for one head
constexpr int kTile = 16;                // tokens per stage
constexpr int kAttnWarps = 4;
constexpr int kAttnStages = 3;
constexpr int kTileBytes = kTile * kRowBytes;              // 8 KB
constexpr int kStageBytes = 2 * kTileBytes;                // K then V
constexpr int kAttnSmem = kAttnWarps * kAttnStages * kStageBytes;   // 192 KB
constexpr int kRowBytes8 = kHD;                            // fp8 cache: one byte per element
constexpr int kTileBytes8 = kTile * kRowBytes8;            // 4 KB
constexpr int kStageBytes8 = 2 * kTileBytes8;
constexpr int kAttnSmem8 = kAttnWarps * kAttnStages * kStageBytes8; // 96 KB: two CTAs per SM

struct AttnParams {
    const __half *q;      // [B][qh][256]
    const void *k;        // [B][kvh][cap][256], fp16 or e4m3
    const void *v;
    __half *out;          // [B][qh][256]
    float *part_o;        // [B][kvh][nsplit][G][256]   (unnormalised)
    float *part_ml;       // [B][kvh][nsplit][G][2]     (running maximum in log2 units, sum)
    long long q_bstride, o_bstride;          // elements between batches of q / out
    long long kv_bstride, kv_hstride;        // elements between batches / heads of the cache
    int B, qh, kvh, G, seq_len, nsplit, split_tokens;
    float scale_log2;     // scale * log2(e) (* the K scale of an fp8 cache)
    float out_scale;      // 1, or the V scale of an fp8 cache
    // paged form: k / v are page pools, a page holds page_size tokens of every KV head
    const int *block_table;   // [B][bt_stride]: page number of every page_size tokens of a sequence
    const int *seq_lens;      // [B] tokens to read per sequence (seq_len is then their upper bound)
    long long page_stride, tok_stride;       // elements between pages / between tokens of a head
    int bt_stride, page_size;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;       // 0 bytes read: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// One warp copies a 16-token tile of K and of V (16 x 512 bytes each): one instruction moves one
// token row, 32 lanes x 16 bytes, into its swizzled place.  krow / vrow point at the tile's first
// token; rows at or beyond `nvalid` are zero-filled.
__device__ __forceinline__ void load_tile(uint32_t stage, const __half *krow, const __half *vrow, long long tok_stride,
                                          int nvalid, int lane) {
#pragma unroll
    for (int r = 0; r < kTile; ++r) {
        const bool ok = r < nvalid;
        const size_t off = (size_t)(ok ? r : 0) * tok_stride + lane * 8;
        const uint32_t dst = stage + r * kRowBytes + ((lane ^ (r & 7)) << 4);
        cp_async16(dst, krow + off, ok);
        cp_async16(dst + kTileBytes, vrow + off, ok);
    }
}

// Where the tile that starts at token tok0 of (sequence b, KV head hk) lies.  Contiguous cache: rows 256
// elements apart behind the head's base.  Paged cache: a tile never straddles a page (page sizes are
// multiples of 16 and tiles start at multiples of 16), so one block-table entry locates it.
// The same for an fp8 cache: rows of 256 bytes, one instruction moves two token rows (16 lanes x 16 bytes each).
__device__ __forceinline__ void load_tile8(uint32_t stage, const unsigned char *krow, const unsigned char *vrow,
                                           long long tok_stride, int nvalid, int lane) {
#pragma unroll
    for (int r2 = 0; r2 < kTile / 2; ++r2) {
        const int r = 2 * r2 + (lane >> 4), c = lane & 15;
        const bool ok = r < nvalid;
        const size_t off = (size_t)(ok ? r : 0) * tok_stride + c * 16;
        const uint32_t dst = stage + r * kRowBytes8 + ((c ^ (r & 7)) << 4);
        cp_async16(dst, krow + off, ok);
        cp_async16(dst + kTileBytes8, vrow + off, ok);
    }
}

template <bool PAGED, bool FP8>
__device__ __forceinline__ void issue_tile(const AttnParams &P, uint32_t stage, int b, int hk, int tok0, int t_end,
                                           int lane) {
    size_t off;
    long long tok_stride;
    if constexpr (PAGED) {
        const int page = __ldg(P.block_table + (size_t)b * P.bt_stride + tok0 / P.page_size);
        off = (size_t)page * P.page_stride + (size_t)hk * P.kv_hstride + (size_t)(tok0 % P.page_size) * P.tok_stride;
        tok_stride = P.tok_stride;
    } else {
        off = (size_t)b * P.kv_bstride + (size_t)hk * P.kv_hstride + (size_t)tok0 * kHD;
        tok_stride = kHD;
    }
    if constexpr (FP8)
        load_tile8(stage, static_cast<const unsigned char *>(P.k) + off, static_cast<const unsigned char *>(P.v) + off,
                   tok_stride, t_end - tok0, lane);
    else
        load_tile(stage, static_cast<const __half *>(P.k) + off, static_cast<const __half *>(P.v) + off, tok_stride,
                  t_end - tok0, lane);
}

// Four e4m3 values of one register -> two fp16 pairs (bytes 0,1 and bytes 2,3).
__device__ __forceinline__ void widen_e4m3x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(w));
}
// The same after gathering bytes (0, 2) and (1, 3): `even` pairs the first value of each 16-bit unit, `odd` the second.
__device__ __forceinline__ void widen_e4m3x4_interleaved(uint32_t w, uint32_t &even, uint32_t &odd) {
    uint32_t t;
    asm("prmt.b32 %0, %1, %1, 0x3120;" : "=r"(t) : "r"(w));
    widen_e4m3x4(t, even, odd);
}

template <bool PAGED, bool FP8>
__global__ void __launch_bounds__(kAttnWarps * 32, FP8 ? 2 : 1) decode_attn_kernel(const __grid_constant__ AttnParams P) {
    constexpr int kStage = FP8 ? kStageBytes8 : kStageBytes;
    constexpr int kTileB = FP8 ? kTileBytes8 : kTileBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q4 = lane & 3;
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int G = P.G;

    const int seq_len = PAGED && P.seq_lens ? min(P.seq_len, __ldg(P.seq_lens + b)) : P.seq_len;
    const int t_begin = split * P.split_tokens;
    const int t_end = min(seq_len, t_begin + P.split_tokens);
    const int ntiles = t_end > t_begin ? (t_end - t_begin + kTile - 1) / kTile : 0;
    const int my_tiles = ntiles > warp ? (ntiles - warp + kAttnWarps - 1) / kAttnWarps : 0;

    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kAttnStages * kStage);

    // Both the query and the newest cache row may come from kernels just before this one on the
    // stream: wait for them, then let the next kernel get ready behind this one.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");

#pragma unroll
    for (int s = 0; s < kAttnStages - 1; ++s) {
        if (s < my_tiles)
            issue_tile<PAGED, FP8>(P, ring + s * kStage, b, hk, t_begin + (warp + s * kAttnWarps) * kTile, t_end, lane);
        cp_async_commit();
    }

    // Query heads of this KV head as A fragments (rows 8..15 of the M side are padding).  With an fp8 cache a
    // lane's K fragment of a 16-wide k step holds dimensions 4*q4 .. 4*q4+3 (four bytes of one ldmatrix unit pair).
    uint32_t qa[16][2];
    {
        const __half *qrow = P.q + (size_t)b * P.q_bstride + (size_t)(hk * G + (g < G ? g : 0)) * kHD;
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
            const uint32_t lo = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + (FP8 ? 4 * q4 : 2 * q4));
            const uint32_t hi = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + (FP8 ? 4 * q4 + 2 : 8 + 2 * q4));
            qa[ks][0] = g < G ? lo : 0u;
            qa[ks][1] = g < G ? hi : 0u;
        }
    }

    float o[16][4];
#pragma unroll
    for (int mt = 0; mt < 16; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[mt][e] = 0.f;
    float m_run = -INFINITY;     // running maximum of head g (log2 units), equal in the four lanes of a group
    float l_run = 0.f;           // this lane's share of the running sum of head g

    // ldmatrix lane addressing inside a stage (before the swizzle): matrix j = lane / 8, row r = lane % 8
    const int lj = lane >> 3, lr = lane & 7;

    for (int i = 0; i < my_tiles; ++i) {
        // keep the ring full: the stage consumed last iteration is free again
        {
            const int nxt = i + kAttnStages - 1;
            if (nxt < my_tiles)
                issue_tile<PAGED, FP8>(P, ring + (nxt % kAttnStages) * kStage, b, hk,
                                       t_begin + (warp + nxt * kAttnWarps) * kTile, t_end, lane);
            cp_async_commit();
        }
        cp_async_wait<kAttnStages - 1>();
        __syncwarp();
        const uint32_t ks_base = ring + (i % kAttnStages) * kStage;
        const uint32_t vs_base = ks_base + kTileB;
        const int tok0 = t_begin + (warp + i * kAttnWarps) * kTile;

        // ---- S = Q K^T for 16 tokens (two 8-token column tiles)
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        if constexpr (FP8) {
#pragma unroll
            for (int kp = 0; kp < 8; ++kp) {         // 32 head dimensions per iteration: matrices (tokens 0-7 | 8-15) x 2 chunks
                const int row = (lj & 1) * 8 + lr;
                const int chunk = kp * 2 + (lj >> 1);
                uint32_t kb[4];
                ldsm4(kb, ks_base + row * kRowBytes8 + ((chunk ^ (row & 7)) << 4));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t b0, b1;
                    widen_e4m3x4(kb[j], b0, b1);
                    mma_f16(s[j & 1], qa[2 * kp + (j >> 1)][0], 0u, qa[2 * kp + (j >> 1)][1], 0u, b0, b1);
                }
            }
        } else {
#pragma unroll
        for (int kp = 0; kp < 8; ++kp) {             // 32 head dimensions per iteration
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int row = nt * 8 + lr;
                const int chunk = kp * 4 + lj;
                uint32_t kb[4];
                ldsm4(kb, ks_base + row * kRowBytes + ((chunk ^ (row & 7)) << 4));
                mma_f16(s[nt], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, kb[0], kb[1]);
                mma_f16(s[nt], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, kb[2], kb[3]);
            }
        }
        }
        // ---- online softmax for head g over tokens tok0 + nt*8 + 2*q4 (+1)
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = tok0 + nt * 8 + 2 * q4 + e;
                s[nt][e] = tok < t_end ? s[nt][e] * P.scale_log2 : -INFINITY;
                mx = fmaxf(mx, s[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);        // finite: every tile holds at least one valid token
        const float corr = exp2f(m_run - m_new);     // 0 on the first tile
        m_run = m_new;
        float p[2][2], psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[nt][e] = exp2f(s[nt][e] - m_new);
                psum += p[nt][e];
            }
        l_run = l_run * corr + psum;
        // the accumulators hold heads 2*q4 and 2*q4+1: fetch their correction factors
        const float c0 = __shfl_sync(0xffffffffu, corr, (2 * q4) * 4);
        const float c1 = __shfl_sync(0xffffffffu, corr, (2 * q4 + 1) * 4);
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
            for (int mt = 0; mt < 16; ++mt) {
                o[mt][0] *= c0; o[mt][1] *= c1; o[mt][2] *= c0; o[mt][3] *= c1;
            }
        }
        // ---- O^T += V^T P^T
        const uint32_t pb0 = pack_h2(p[0][0], p[0][1]);
        const uint32_t pb1 = pack_h2(p[1][0], p[1][1]);
        if constexpr (FP8) {
            // one transposed load = 32 dimensions x 16 tokens; the first value of every 16-bit unit goes to
            // accumulator 2*mt (dimensions 32*mt + 2*g and + 16), the second to 2*mt + 1 (one dimension further)
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int row = (lj >> 1) * 8 + lr;  // token inside the tile
                const int chunk = mt * 2 + (lj & 1); // sixteen head dimensions
                uint32_t va[4], ev[4], od[4];
                ldsm4_t(va, vs_base + row * kRowBytes8 + ((chunk ^ (row & 7)) << 4));
#pragma unroll
                for (int j = 0; j < 4; ++j) widen_e4m3x4_interleaved(va[j], ev[j], od[j]);
                mma_f16(o[2 * mt], ev[0], ev[1], ev[2], ev[3], pb0, pb1);
                mma_f16(o[2 * mt + 1], od[0], od[1], od[2], od[3], pb0, pb1);
            }
        } else {
#pragma unroll
        for (int mt = 0; mt < 16; ++mt) {
            const int row = (lj >> 1) * 8 + lr;      // token inside the tile
            const int chunk = mt * 2 + (lj & 1);     // eight head dimensions
            uint32_t va[4];
            ldsm4_t(va, vs_base + row * kRowBytes + ((chunk ^ (row & 7)) << 4));
            mma_f16(o[mt], va[0], va[1], va[2], va[3], pb0, pb1);
        }
        }
        __syncwarp();                                // every lane is done reading this stage
    }
    cp_async_wait<0>();
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();                                 // all rings are idle: the memory is reused

    // ---- merge the four warps: [warp][head][256] partial outputs + (m, l) per head
    float *wo = reinterpret_cast<float *>(smem);                       // 4 x 8 x 256 floats = 32 KB
    float *wml = wo + kAttnWarps * 8 * kHD;                            // [warp][head][2]
#pragma unroll
    for (int mt = 0; mt < 16; ++mt) {
        // dimension of accumulator rows g / g + 8: fp16 cache 16*mt + g / + 8; fp8 cache 32*(mt/2) + 2*g + (mt&1) / + 16
        const int d0 = FP8 ? 32 * (mt >> 1) + 2 * g + (mt & 1) : mt * 16 + g;
        constexpr int dstep = FP8 ? 16 : 8;
        float *dst = wo + ((size_t)warp * 8 + 2 * q4) * kHD + d0;
        dst[0] = o[mt][0]; dst[kHD] = o[mt][1]; dst[dstep] = o[mt][2]; dst[kHD + dstep] = o[mt][3];
    }
    if (q4 == 0) { wml[(warp * 8 + g) * 2] = m_run; wml[(warp * 8 + g) * 2 + 1] = l_run; }
    __syncthreads();

    for (int h = 0; h < G; ++h) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, wml[(w * 8 + h) * 2]);
        float L = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = wml[(w * 8 + h) * 2];
            const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += wml[(w * 8 + h) * 2 + 1] * wgt;
            const float2 ov = *reinterpret_cast<const float2 *>(wo + ((size_t)w * 8 + h) * kHD + 2 * tid);
            a0 += ov.x * wgt; a1 += ov.y * wgt;
        }
        if (P.nsplit == 1) {
            const float inv = L > 0.f ? P.out_scale / L : 0.f;
            __half2 r = __floats2half2_rn(a0 * inv, a1 * inv);
            *reinterpret_cast<__half2 *>(P.out + (size_t)b * P.o_bstride + (size_t)(hk * G + h) * kHD + 2 * tid) = r;
        } else {
            const size_t idx = (((size_t)b * P.kvh + hk) * P.nsplit + split) * G + h;
            *reinterpret_cast<float2 *>(P.part_o + idx * kHD + 2 * tid) = make_float2(a0, a1);
            if (tid == 0) { P.part_ml[idx * 2] = M; P.part_ml[idx * 2 + 1] = L; }
        }
    }
}

// Merge of the splits: one CTA of 128 threads per (batch, query head), two dimensions per thread.
__global__ void __launch_bounds__(128) decode_attn_merge_kernel(const __grid_constant__ AttnParams P) {
    __shared__ float w_s[256];       // weight of every split (nsplit <= 256)
    __shared__ float red[8];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = h / P.G, hg = h - hk * P.G;
    const size_t base = ((size_t)b * P.kvh + hk) * P.nsplit;
    // (maximum, sum) of the splits, one or two splits per thread: all loads are in flight at once
    float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
    if (tid < P.nsplit) {
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(P.part_ml + ((base + tid) * P.G + hg) * 2));
        m0 = ml.x; l0 = ml.y;
    }
    if (tid + 128 < P.nsplit) {
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(P.part_ml + ((base + tid + 128) * P.G + hg) * 2));
        m1 = ml.x; l1 = ml.y;
    }
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) red[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - M);
    const float w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - M);
    w_s[tid] = w0;
    w_s[tid + 128] = w1;
    float L = l0 * w0 + l1 * w1;
#pragma unroll
    for (int o = 16; o; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0) red[4 + warp] = L;
    __syncthreads();
    L = (red[4] + red[5]) + (red[6] + red[7]);
    // weighted sum of the partial outputs in split order, eight loads in flight per thread
    const float *po = P.part_o + (base * P.G + hg) * kHD + 2 * tid;
    const size_t step = (size_t)P.G * kHD;
    float a0 = 0.f, a1 = 0.f;
    int s = 0;
    for (; s + 8 <= P.nsplit; s += 8) {
        float2 ov[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) ov[u] = __ldcg(reinterpret_cast<const float2 *>(po + (s + u) * step));
#pragma unroll
        for (int u = 0; u < 8; ++u) { a0 += ov[u].x * w_s[s + u]; a1 += ov[u].y * w_s[s + u]; }
    }
    for (; s < P.nsplit; ++s) {
        const float2 ov = __ldcg(reinterpret_cast<const float2 *>(po + s * step));
        a0 += ov.x * w_s[s]; a1 += ov.y * w_s[s];
    }
    const float inv = L > 0.f ? P.out_scale / L : 0.f;
    *reinterpret_cast<__half2 *>(P.out + (size_t)b * P.o_bstride + (size_t)h * kHD + 2 * tid) =
        __floats2half2_rn(a0 * inv, a1 * inv);
}

// Rotary embedding of the query and key heads of one decoded token per sequence and the append of
// the rotated key and the value to the cache, in one launch (the step before decode_attn_kernel).
// Rotate-half form: out[i] = t[i] cos[i] - t[i+128] sin[i],  out[i+128] = t[i+128] cos[i] + t[i] sin[i],
// computed in fp32 and rounded once.  grid = (q_heads + 2 kv_heads, batch), 128 threads.
struct RopeParams {
    __half *qkv;             // [B][ld]: q heads, then k heads, then v heads, 256 each
    const __half *cos, *sin; // [B or 1][128]
    void *k, *v;             // caches [B][kvh][cap][256], fp16 or e4m3
    long long kv_bstride, kv_hstride;
    int ld, qh, kvh, pos, cs_stride;
    float k_inv_scale, v_inv_scale;   // fp8 caches store value / scale
};

__device__ __forceinline__ unsigned char to_e4m3(float x) {
    return static_cast<unsigned char>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// With an fp8 cache the rotated key is rounded to fp16 first (the value the fp16 cache would hold), then divided
// by the scale and rounded to e4m3 with saturation; the query stays fp16.
template <bool FP8>
__global__ void __launch_bounds__(128) rope_append_kernel(const __grid_constant__ RopeParams P) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int h = blockIdx.x, b = blockIdx.y, i = threadIdx.x;
    __half *t = P.qkv + (size_t)b * P.ld + (size_t)h * kHD;
    if (h >= P.qh + P.kvh) {                                   // value head: copy
        const size_t off = (size_t)b * P.kv_bstride + (size_t)(h - P.qh - P.kvh) * P.kv_hstride + (size_t)P.pos * kHD;
        if constexpr (FP8) {
            const __half2 v2 = reinterpret_cast<const __half2 *>(t)[i];
            unsigned char *dst = static_cast<unsigned char *>(P.v) + off;
            const unsigned short pair = (unsigned short)to_e4m3(__low2float(v2) * P.v_inv_scale) |
                                        (unsigned short)to_e4m3(__high2float(v2) * P.v_inv_scale) << 8;
            reinterpret_cast<unsigned short *>(dst)[i] = pair;
        } else {
            __half *dst = static_cast<__half *>(P.v) + off;
            reinterpret_cast<uint32_t *>(dst)[i] = reinterpret_cast<const uint32_t *>(t)[i];
        }
        return;
    }
    const float c = __half2float(P.cos[(size_t)b * P.cs_stride + i]);
    const float sn = __half2float(P.sin[(size_t)b * P.cs_stride + i]);
    const float lo = __half2float(t[i]), hi = __half2float(t[i + 128]);
    const __half olo = __float2half_rn(lo * c - hi * sn), ohi = __float2half_rn(hi * c + lo * sn);
    if (h < P.qh) {
        t[i] = olo;
        t[i + 128] = ohi;
        return;
    }
    const size_t off = (size_t)b * P.kv_bstride + (size_t)(h - P.qh) * P.kv_hstride + (size_t)P.pos * kHD;
    if constexpr (FP8) {
        unsigned char *dst = static_cast<unsigned char *>(P.k) + off;
        dst[i] = to_e4m3(__half2float(olo) * P.k_inv_scale);
        dst[i + 128] = to_e4m3(__half2float(ohi) * P.k_inv_scale);
    } else {
        __half *dst = static_cast<__half *>(P.k) + off;
        dst[i] = olo;
        dst[i + 128] = ohi;
    }
}

static int pick_splits(int B, int kvh, int seq_len, int slots = 148) {
    // A CTA takes a whole SM (192 KB of rings) and costs a few microseconds whatever its length, so a
    // second wave of short CTAs is dear (measured on B200, one sequence of 4096 tokens: 9.5-9.9 us with
    // 72-148 CTAs, 13.8 us with 260).  Few (sequence, KV head) pairs: as many splits as fit in one wave
    // of 148 CTAs.  Many pairs: about two CTAs per SM, which evens out the tail.  A split is never
    // shorter than 64 tokens.  `slots`: CTAs resident at once (148, or 296 with the half-size rings of an fp8 cache).
    const int pairs = B * kvh;
    int want = 2 * pairs <= slots ? slots / pairs : (2 * slots) / pairs;
    const int max_by_len = (seq_len + 63) / 64;
    if (want > max_by_len) want = max_by_len;
    if (want < 1) want = 1;
    if (want > 256) want = 256;
    return want;
}

// Split choice, workspace carving and the one or two launches, shared by the contiguous and the paged form.
static int launch_attn(AttnParams &P, bool paged, bool fp8, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    P.nsplit = pick_splits(P.B, P.kvh, P.seq_len, fp8 ? 296 : 148);
    const int tiles = (P.seq_len + kTile - 1) / kTile;
    const int per = (tiles + P.nsplit - 1) / P.nsplit;
    P.split_tokens = per * kTile;
    P.nsplit = (tiles + per - 1) / per;              // no split beyond the longest sequence
    if (P.nsplit > 1) {
        const size_t rows = (size_t)P.B * P.qh * P.nsplit;
        if (!workspace || workspace_bytes < rows * kHD * 4 + rows * 8) return EXL3_E_WORKSPACE;
        if (!aligned(workspace, 16)) return EXL3_E_ALIGN;
        P.part_o = (float *)workspace;
        P.part_ml = P.part_o + rows * kHD;
    }
    auto kernel = fp8 ? (paged ? decode_attn_kernel<true, true> : decode_attn_kernel<false, true>)
                      : (paged ? decode_attn_kernel<true, false> : decode_attn_kernel<false, false>);
    const int smem = fp8 ? kAttnSmem8 : kAttnSmem;
    static bool attr_done[4][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[2 * fp8 + paged][dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return EXL3_E_LAUNCH;
        attr_done[2 * fp8 + paged][dev] = true;
    }
    if (launch_pdl(kernel, dim3(P.nsplit, P.kvh, P.B), dim3(kAttnWarps * 32), smem, st, P) != cudaSuccess)
        return EXL3_E_LAUNCH;
    if (P.nsplit > 1 &&
        launch_pdl(decode_attn_merge_kernel, dim3(P.qh, P.B), dim3(128), 0, st, P) != cudaSuccess)
        return EXL3_E_LAUNCH;
    return launch_status();
}

// ---- argument checks and parameter blocks shared by the fp16 and the fp8 entry points
static int attn_contiguous(bool fp8, const void *q, const void *k_cache, const void *v_cache, void *out, void *workspace,
                           size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim, int seq_len,
                           long long q_batch_stride, long long out_batch_stride, long long kv_batch_stride,
                           long long kv_head_stride, float scale, float k_scale, float v_scale, void *stream) {
    if (!q || !k_cache || !v_cache || !out) return EXL3_E_NULL;
    if (head_dim != kHD) return EXL3_E_UNSUPPORTED;
    if (batch <= 0 || batch > 65535 || kv_heads <= 0 || kv_heads > 65535 || q_heads <= 0 || q_heads % kv_heads ||
        seq_len <= 0 || !(k_scale > 0.f) || !(v_scale > 0.f))
        return EXL3_E_SHAPE;
    const int G = q_heads / kv_heads;
    if (G > 8) return EXL3_E_UNSUPPORTED;
    const long long amask = fp8 ? 15 : 7;            // 16-byte copies
    if (kv_head_stride < (long long)seq_len * kHD || (kv_head_stride & amask) || (kv_batch_stride & amask) ||
        (q_batch_stride & 1) || (out_batch_stride & 1))
        return EXL3_E_SHAPE;
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(q, 4) || !aligned(out, 4)) return EXL3_E_ALIGN;
    AttnParams P = {};
    P.q = (const __half *)q; P.k = k_cache; P.v = v_cache; P.out = (__half *)out;
    P.q_bstride = q_batch_stride; P.o_bstride = out_batch_stride;
    P.kv_bstride = kv_batch_stride; P.kv_hstride = kv_head_stride;
    P.B = batch; P.qh = q_heads; P.kvh = kv_heads; P.G = G; P.seq_len = seq_len;
    P.scale_log2 = scale * k_scale * 1.4426950408889634f;
    P.out_scale = v_scale;
    return launch_attn(P, false, fp8, workspace, workspace_bytes, (cudaStream_t)stream);
}

static int attn_paged(bool fp8, const void *q, const void *k_pages, const void *v_pages, const void *block_table,
                      const void *seq_lens, void *out, void *workspace, size_t workspace_bytes, int batch, int q_heads,
                      int kv_heads, int head_dim, int max_seq_len, int page_size, int block_table_stride,
                      long long q_batch_stride, long long out_batch_stride, long long page_stride, long long head_stride,
                      long long token_stride, float scale, float k_scale, float v_scale, void *stream) {
    if (!q || !k_pages || !v_pages || !block_table || !out) return EXL3_E_NULL;
    if (head_dim != kHD) return EXL3_E_UNSUPPORTED;
    if (batch <= 0 || batch > 65535 || kv_heads <= 0 || kv_heads > 65535 || q_heads <= 0 || q_heads % kv_heads ||
        max_seq_len <= 0 || page_size <= 0 || (page_size % kTile) || !(k_scale > 0.f) || !(v_scale > 0.f))
        return EXL3_E_SHAPE;
    const int G = q_heads / kv_heads;
    if (G > 8) return EXL3_E_UNSUPPORTED;
    const long long amask = fp8 ? 15 : 7;
    if (block_table_stride < (max_seq_len + page_size - 1) / page_size || token_stride < kHD || (token_stride & amask) ||
        (head_stride & amask) || (page_stride & amask) || head_stride <= 0 || page_stride <= 0 || (q_batch_stride & 1) ||
        (out_batch_stride & 1))
        return EXL3_E_SHAPE;
    if (!aligned(k_pages, 16) || !aligned(v_pages, 16) || !aligned(q, 4) || !aligned(out, 4) || !aligned(block_table, 4) ||
        !aligned(seq_lens, 4))
        return EXL3_E_ALIGN;
    AttnParams P = {};
    P.q = (const __half *)q; P.k = k_pages; P.v = v_pages; P.out = (__half *)out;
    P.q_bstride = q_batch_stride; P.o_bstride = out_batch_stride;
    P.kv_hstride = head_stride; P.page_stride = page_stride; P.tok_stride = token_stride;
    P.block_table = (const int *)block_table; P.seq_lens = (const int *)seq_lens;
    P.bt_stride = block_table_stride; P.page_size = page_size;
    P.B = batch; P.qh = q_heads; P.kvh = kv_heads; P.G = G; P.seq_len = max_seq_len;
    P.scale_log2 = scale * k_scale * 1.4426950408889634f;
    P.out_scale = v_scale;
    return launch_attn(P, true, fp8, workspace, workspace_bytes, (cudaStream_t)stream);
}

static int rope_append(bool fp8, void *qkv, int ld_qkv, const void *cos, const void *sin, int cos_sin_batch_stride,
                       void *k_cache, void *v_cache, int batch, int q_heads, int kv_heads, int head_dim, int pos,
                       long long kv_batch_stride, long long kv_head_stride, float k_scale, float v_scale, void *stream) {
    if (!qkv || !cos || !sin || !k_cache || !v_cache) return EXL3_E_NULL;
    if (head_dim != kHD) return EXL3_E_UNSUPPORTED;
    if (batch <= 0 || batch > 65535 || q_heads <= 0 || kv_heads <= 0 || pos < 0 ||
        ld_qkv < (q_heads + 2 * kv_heads) * kHD || (ld_qkv & 1) || cos_sin_batch_stride < 0 ||
        kv_head_stride < (long long)(pos + 1) * kHD || (kv_head_stride & 1) || (kv_batch_stride & 1) ||
        !(k_scale > 0.f) || !(v_scale > 0.f))
        return EXL3_E_SHAPE;
    if (!aligned(qkv, 4) || !aligned(k_cache, 4) || !aligned(v_cache, 4)) return EXL3_E_ALIGN;
    RopeParams P = {};
    P.qkv = (__half *)qkv; P.cos = (const __half *)cos; P.sin = (const __half *)sin;
    P.k = k_cache; P.v = v_cache;
    P.kv_bstride = kv_batch_stride; P.kv_hstride = kv_head_stride;
    P.ld = ld_qkv; P.qh = q_heads; P.kvh = kv_heads; P.pos = pos; P.cs_stride = cos_sin_batch_stride;
    P.k_inv_scale = 1.f / k_scale; P.v_inv_scale = 1.f / v_scale;
    auto kernel = fp8 ? rope_append_kernel<true> : rope_append_kernel<false>;
    if (launch_pdl(kernel, dim3(q_heads + 2 * kv_heads, batch), dim3(128), 0, (cudaStream_t)stream, P) != cudaSuccess)
        return EXL3_E_LAUNCH;
    return launch_status();
}

static size_t attn_workspace_bytes(bool fp8, int batch, int q_heads, int kv_heads, int seq_len) {
    if (batch <= 0 || kv_heads <= 0 || q_heads <= 0 || q_heads % kv_heads || seq_len <= 0) return 0;
    const int ns = pick_splits(batch, kv_heads, seq_len, fp8 ? 296 : 148);
    if (ns == 1) return 0;
    const size_t rows = (size_t)batch * q_heads * ns;
    return rows * kHD * 4 + rows * 2 * 4;
}

}  // namespace exl3

extern "C" size_t exl3_decode_attn_workspace_bytes(int batch, int q_heads, int kv_heads, int seq_len) {
    return exl3::attn_workspace_bytes(false, batch, q_heads, kv_heads, seq_len);
}
extern "C" size_t exl3_decode_attn_fp8_workspace_bytes(int batch, int q_heads, int kv_heads, int seq_len) {
    return exl3::attn_workspace_bytes(true, batch, q_heads, kv_heads, seq_len);
}

extern "C" int exl3_decode_attn(const void *q, const void *k_cache, const void *v_cache, void *out,
                                void *workspace, size_t workspace_bytes, int batch, int q_heads, int kv_heads,
                                int head_dim, int seq_len, long long q_batch_stride, long long out_batch_stride,
                                long long kv_batch_stride, long long kv_head_stride, float scale, void *stream) {
    return exl3::attn_contiguous(false, q, k_cache, v_cache, out, workspace, workspace_bytes, batch, q_heads, kv_heads,
                                 head_dim, seq_len, q_batch_stride, out_batch_stride, kv_batch_stride, kv_head_stride,
                                 scale, 1.f, 1.f, stream);
}
extern "C" int exl3_decode_attn_fp8(const void *q, const void *k_cache, const void *v_cache, void *out,
                                    void *workspace, size_t workspace_bytes, int batch, int q_heads, int kv_heads,
                                    int head_dim, int seq_len, long long q_batch_stride, long long out_batch_stride,
                                    long long kv_batch_stride, long long kv_head_stride, float scale, float k_scale,
                                    float v_scale, void *stream) {
    return exl3::attn_contiguous(true, q, k_cache, v_cache, out, workspace, workspace_bytes, batch, q_heads, kv_heads,
                                 head_dim, seq_len, q_batch_stride, out_batch_stride, kv_batch_stride, kv_head_stride,
                                 scale, k_scale, v_scale, stream);
}

extern "C" int exl3_decode_attn_paged(const void *q, const void *k_pages, const void *v_pages, const void *block_table,
                                      const void *seq_lens, void *out, void *workspace, size_t workspace_bytes,
                                      int batch, int q_heads, int kv_heads, int head_dim, int max_seq_len,
                                      int page_size, int block_table_stride, long long q_batch_stride,
                                      long long out_batch_stride, long long page_stride, long long head_stride,
                                      long long token_stride, float scale, void *stream) {
    return exl3::attn_paged(false, q, k_pages, v_pages, block_table, seq_lens, out, workspace, workspace_bytes, batch,
                            q_heads, kv_heads, head_dim, max_seq_len, page_size, block_table_stride, q_batch_stride,
                            out_batch_stride, page_stride, head_stride, token_stride, scale, 1.f, 1.f, stream);
}
extern "C" int exl3_decode_attn_paged_fp8(const void *q, const void *k_pages, const void *v_pages,
                                          const void *block_table, const void *seq_lens, void *out, void *workspace,
                                          size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim,
                                          int max_seq_len, int page_size, int block_table_stride,
                                          long long q_batch_stride, long long out_batch_stride, long long page_stride,
                                          long long head_stride, long long token_stride, float scale, float k_scale,
                                          float v_scale, void *stream) {
    return exl3::attn_paged(true, q, k_pages, v_pages, block_table, seq_lens, out, workspace, workspace_bytes, batch,
                            q_heads, kv_heads, head_dim, max_seq_len, page_size, block_table_stride, q_batch_stride,
                            out_batch_stride, page_stride, head_stride, token_stride, scale, k_scale, v_scale, stream);
}

extern "C" int exl3_rope_append(void *qkv, int ld_qkv, const void *cos, const void *sin, int cos_sin_batch_stride,
                                void *k_cache, void *v_cache, int batch, int q_heads, int kv_heads, int head_dim,
                                int pos, long long kv_batch_stride, long long kv_head_stride, void *stream) {
    return exl3::rope_append(false, qkv, ld_qkv, cos, sin, cos_sin_batch_stride, k_cache, v_cache, batch, q_heads,
                             kv_heads, head_dim, pos, kv_batch_stride, kv_head_stride, 1.f, 1.f, stream);
}
extern "C" int exl3_rope_append_fp8(void *qkv, int ld_qkv, const void *cos, const void *sin, int cos_sin_batch_stride,
                                    void *k_cache, void *v_cache, int batch, int q_heads, int kv_heads, int head_dim,
                                    int pos, long long kv_batch_stride, long long kv_head_stride, float k_scale,
                                    float v_scale, void *stream) {
    return exl3::rope_append(true, qkv, ld_qkv, cos, sin, cos_sin_batch_stride, k_cache, v_cache, batch, q_heads,
                             kv_heads, head_dim, pos, kv_batch_stride, kv_head_stride, k_scale, v_scale, stream);
}
