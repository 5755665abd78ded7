// EXL3 trellis format and codebook, device side.  One statement of the format shared by every
// kernel (reconstruct, fused GEMV, tensor-core GEMM), matching the CPU oracle bit for bit.
//
// Tile = 16x16 weights = 16*K uint16 words = 8 chunks of K 32-bit words (32 weights each).
//   bit n of the tile's circular bit string: (word16[n >> 4] >> (n & 15)) & 1, i.e. the tile is a
//   little-endian integer; as 32-bit little-endian words, bit n = (word32[n >> 5] >> (n & 31)) & 1.
//   state(t) = 16 bits starting at bit t*K (least significant first), wrapping at 256*K.
//   t = 32*c + i; chunk c = 4*p + q is held by one lane: it needs the K words [c*K, c*K+K) plus
//   the first word of chunk (c+1) & 7 for the windows that run over the end.
//   position: row (input channel)  = 8*((i>>2)&1) + 4*((i>>1)&1) + q
//             col (output channel) = 4*(i>>3) + 2*(i&1) + p
//   With lane = 8*u + c holding chunk c of tile u (four tiles side by side along oc), the four
//   weights i = 8a+4b .. 8a+4b+3 are exactly the A-fragment registers a0..a3 of an
//   mma.m16n8k16 whose M index is the lane's group (lane>>2 -> tile u, p) and whose K index
//   pairs (2q, 2q+1), (2q+8, 2q+9) carry the two fp16 halves of one codeword.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace exl3 {

constexpr uint32_t kMul = 89226354u;
constexpr uint32_t kAdd = 64248484u;
constexpr uint32_t kMask = 0x8FFF8FFFu;
constexpr uint32_t kXor = 0x3B603B60u;

// (z & kMask) ^ kXor in one LOP3
__device__ __forceinline__ uint32_t mask_xor(uint32_t z) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(z), "r"(kMask), "r"(kXor));
    return r;
}

// clean 16-bit state -> 32-bit codeword whose two fp16 halves sum to the weight
__device__ __forceinline__ uint32_t codeword(uint32_t state) {
    return mask_xor(state * kMul + kAdd);
}

// codeword -> fp16 weight, rounded exactly as the oracle (one fp16 add)
__device__ __forceinline__ __half codeword_to_half(uint32_t z) {
    __half2 h = *reinterpret_cast<__half2 *>(&z);
    return __hadd(__low2half(h), __high2half(h));
}

// State i (0..31) of a chunk from its K+1 words.
template <int K, int I>
__device__ __forceinline__ uint32_t chunk_state(const uint32_t (&w)[K + 1]) {
    constexpr int off = I * K;
    constexpr int q = off >> 5;
    constexpr int o = off & 31;
    uint32_t v;
    if constexpr (o == 0) {
        v = w[q];
    } else if constexpr (o + 16 <= 32) {
        v = w[q] >> o;
    } else {
        v = __funnelshift_r(w[q], w[q + 1], o);
    }
    if constexpr (o == 16) {
        return v;
    } else {
        return v & 0xFFFFu;
    }
}

template <int K, int I>
struct ChunkDecoder {
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], uint32_t (&z)[32]) {
        z[I] = codeword(chunk_state<K, I>(w));
        ChunkDecoder<K, I + 1>::run(w, z);
    }
};
template <int K>
struct ChunkDecoder<K, 32> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], uint32_t (&)[32]) {}
};

// 32 codewords of one chunk
template <int K>
__device__ __forceinline__ void decode_chunk(const uint32_t (&w)[K + 1], uint32_t (&z)[32]) {
    ChunkDecoder<K, 0>::run(w, z);
}

// K consecutive 32-bit words from shared memory, widest loads the alignment allows.
template <int K>
__device__ __forceinline__ void load_words(const uint32_t *src, uint32_t (&w)[K + 1]) {
    if constexpr (K % 4 == 0) {
#pragma unroll
        for (int k = 0; k < K; k += 4) {
            const uint4 v = *reinterpret_cast<const uint4 *>(src + k);
            w[k] = v.x; w[k + 1] = v.y; w[k + 2] = v.z; w[k + 3] = v.w;
        }
    } else if constexpr (K % 2 == 0) {
#pragma unroll
        for (int k = 0; k < K; k += 2) {
            const uint2 v = *reinterpret_cast<const uint2 *>(src + k);
            w[k] = v.x; w[k + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int k = 0; k < K; ++k) w[k] = src[k];
    }
}

// position of weight i of chunk c inside the 16x16 tile
__device__ __forceinline__ int tile_row(int c, int i) {
    return 8 * ((i >> 2) & 1) + 4 * ((i >> 1) & 1) + (c & 3);
}
__device__ __forceinline__ int tile_col(int c, int i) {
    return 4 * (i >> 3) + 2 * (i & 1) + (c >> 2);
}

}  // namespace exl3
