// Standalone reconstruct: packed trellis -> dense fp16 inner weight w[ic][oc].
// HBM-bound: reads K/8 bytes and writes 2 bytes per weight.
//
// One warp decodes four neighbouring tiles of one tile-row (lane = 8*tile + chunk, 32 weights
// per lane), transposes them through shared memory and writes 16 rows of 64 contiguous columns
// with 16-byte stores.  A block of eight warps covers 512 contiguous output columns.
#include "exl3_codec.cuh"
#include "exl3_common.cuh"

namespace exl3 {

constexpr int kRecWarps = 8;
constexpr int kRecPitch = 72;  // halves per staged row: 64 + 8 keeps rows 16-byte aligned

template <int K>
__global__ void __launch_bounds__(kRecWarps * 32)
reconstruct_kernel(const uint32_t *__restrict__ trellis, __half *__restrict__ w, int tiles_j, int oc) {
    __shared__ __align__(16) __half stage[kRecWarps][16][kRecPitch];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int u = lane >> 3;        // tile within the warp's group of four
    const int c = lane & 7;         // chunk within the tile
    const int ti = blockIdx.y;
    const int j0 = (blockIdx.x * kRecWarps + warp) * 4;
    const int tj = j0 + u;
    const bool live = tj < tiles_j;

    uint32_t wd[K + 1];
    if (live) {
        const uint32_t *src = trellis + ((size_t)ti * tiles_j + tj) * (size_t)(8 * K) + c * K;
#pragma unroll
        for (int k = 0; k < K; ++k) wd[k] = __ldg(src + k);
    } else {
#pragma unroll
        for (int k = 0; k < K; ++k) wd[k] = 0u;
    }
    // first word of the next chunk of the same tile (the trellis is tail-biting)
    wd[K] = __shfl_sync(0xffffffffu, wd[0], (lane & 24) | ((c + 1) & 7));

    uint32_t z[32];
    decode_chunk<K>(wd, z);

#pragma unroll
    for (int i = 0; i < 32; ++i)
        stage[warp][tile_row(c, i)][16 * u + tile_col(c, i)] = codeword_to_half(z[i]);
    __syncwarp();

    if (j0 >= tiles_j) return;
    const int cols_live = min(64, (tiles_j - j0) * 16);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 32 + lane;
        const int r = idx >> 3, seg = idx & 7;
        if (seg * 8 < cols_live) {
            const uint4 v = *reinterpret_cast<const uint4 *>(&stage[warp][r][seg * 8]);
            *reinterpret_cast<uint4 *>(w + (size_t)(16 * ti + r) * oc + 16 * j0 + seg * 8) = v;
        }
    }
}

template <int K>
static int launch_reconstruct(void *w, const void *trellis, int ic, int oc, cudaStream_t st) {
    const int tiles_i = ic / 16, tiles_j = oc / 16;
    dim3 grid((tiles_j + kRecWarps * 4 - 1) / (kRecWarps * 4), tiles_i);
    reconstruct_kernel<K><<<grid, kRecWarps * 32, 0, st>>>(
        static_cast<const uint32_t *>(trellis), static_cast<__half *>(w), tiles_j, oc);
    return launch_status();
}

}  // namespace exl3

extern "C" int exl3_reconstruct(void *w, const void *trellis, int ic, int oc, int k_times_2, int mcg,
                                int mul1, void *stream) {
    using namespace exl3;
    if (!w || !trellis) return EXL3_E_NULL;
    if (ic <= 0 || oc <= 0 || (ic & 15) || (oc & 15) || ic / 16 > 65535) return EXL3_E_SHAPE;
    if (mcg || mul1) return EXL3_E_UNSUPPORTED;
    const int K = integer_k(k_times_2);
    if (!K) return EXL3_E_UNSUPPORTED;
    if (!aligned(w, 16) || !aligned(trellis, 16)) return EXL3_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (K) {
        case 1: return launch_reconstruct<1>(w, trellis, ic, oc, st);
        case 2: return launch_reconstruct<2>(w, trellis, ic, oc, st);
        case 3: return launch_reconstruct<3>(w, trellis, ic, oc, st);
        case 4: return launch_reconstruct<4>(w, trellis, ic, oc, st);
        case 5: return launch_reconstruct<5>(w, trellis, ic, oc, st);
        case 6: return launch_reconstruct<6>(w, trellis, ic, oc, st);
        case 7: return launch_reconstruct<7>(w, trellis, ic, oc, st);
        case 8: return launch_reconstruct<8>(w, trellis, ic, oc, st);
    }
    return EXL3_E_UNSUPPORTED;
}
