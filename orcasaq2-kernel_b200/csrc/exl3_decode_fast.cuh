// Pipe-balanced trellis decode for the fused kernels.
//
// Measured on sm_100 (B200), per warp instruction and scheduler: logic / shift / permute
// operations issue every 2 cycles on one pipe, 32-bit multiply-adds every 1-2 cycles on another,
// and the two run side by side; a multiply whose HIGH word is taken costs 3.9 cycles and
// mma.sync.m16n8k16 about 8 that do not overlap with the logic pipe.  A decoder is therefore as
// fast as its count of logic-pipe operations.  The plain form (shift, mask, multiply-add,
// mask-xor) has three per weight; the forms below produce the SAME 32-bit codewords with about
// two:
//
//  * K = 1, 2, 4, 8 (K divides 16): the 32 bits at a weight's window hold two states,
//    Q = [s_b | s_a] with b = a + 16/K.  s_b is one shift away; the codeword of s_a needs no
//    mask at all, because the multiply is linear modulo 2^32:
//        z_a = s_a*A + B = (Q*A + B + (B << 16)) - 65536 * (s_b*A + B)      (mod 2^32)
//    i.e. two multiply-adds instead of a mask and one multiply-add.
//  * every other K: the chunk's words are also kept shifted by 16 bits (K funnel shifts per
//    chunk), so that every window lies inside ONE word of either copy; a multiply by a power of
//    two moves the state to the top half (multiply pipe) and one shift brings it down clean.
//
// Registers only, four warps per scheduler, codewords consumed by mma.sync, cycles per 32
// weights: K = 4 pair form 198 (plain 221); K = 2 182; K = 3 / 5 / 6 split form 210 / 217 / 215
// (plain 239 / 234 / 236).
#pragma once
#include <stdint.h>

#include "exl3_codec.cuh"

namespace exl3 {

// A multiplier that must stay a multiplication (not be strength-reduced into shifts on the busy
// pipe) is passed in a register, derived from a value the compiler cannot see.
struct DecodeConsts {
    uint32_t neg65536;   // -65536 mod 2^32
    __device__ __forceinline__ explicit DecodeConsts(uint32_t one) : neg65536(0u - (one << 16)) {}
};

__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// a * kMul + C with both constants as immediates (no register-file reads for them)
template <uint32_t C>
__device__ __forceinline__ uint32_t mad_code(uint32_t a) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "n"(kMul), "n"(C));
    return d;
}
__device__ __forceinline__ uint32_t mask_xor_v(uint32_t z) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(z), "n"(kMask), "n"(kXor));
    return r;
}

// ---- general K: every window inside one word of w or of its 16-bit-shifted copy v ----------
template <int SH>
__device__ __forceinline__ uint32_t shl_mul(uint32_t x) {
    uint32_t d;
    asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(x), "n"(1u << SH));
    return d;
}
template <int K, int I>
__device__ __forceinline__ uint32_t chunk_state_split(const uint32_t (&w)[K + 1], const uint32_t (&v)[K]) {
    constexpr int off = I * K;
    constexpr int q = off >> 5;
    constexpr int o = off & 31;
    if constexpr (o == 0) return w[q] & 0xFFFFu;
    else if constexpr (o == 16) return w[q] >> 16;
    else if constexpr (o < 16) return shl_mul<16 - o>(w[q]) >> 16;
    else return shl_mul<32 - o>(v[q]) >> 16;
}
template <int K, int I>
struct SplitDecoder {
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], const uint32_t (&v)[K], uint32_t (&z)[32]) {
        z[I] = mask_xor_v(mad_code<kAdd>(chunk_state_split<K, I>(w, v)));
        SplitDecoder<K, I + 1>::run(w, v, z);
    }
};
template <int K>
struct SplitDecoder<K, 32> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], const uint32_t (&)[K], uint32_t (&)[32]) {}
};

// ---- K dividing 16: two states per window -------------------------------------------------
// Pair j of the chunk: weights a = (j / P) * 2P + (j % P) and b = a + P, with P = 16 / K.
template <int K, int J>
struct PairDecoder {
    static constexpr int P = 16 / K;
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], uint32_t (&z)[32], const DecodeConsts &dc) {
        constexpr int a = (J / P) * 2 * P + (J % P);
        constexpr int b = a + P;
        constexpr int off = a * K;
        constexpr int q = off >> 5;
        constexpr int o = off & 31;
        uint32_t Q;
        if constexpr (o == 0) Q = w[q];
        else Q = __funnelshift_r(w[q], w[q + 1], o);
        const uint32_t sb = Q >> 16;
        const uint32_t zb = mad_code<kAdd>(sb);
        const uint32_t t = mad_code<kAdd + (kAdd << 16)>(Q);
        const uint32_t za = mad_u32(zb, dc.neg65536, t);
        z[a] = mask_xor_v(za);
        z[b] = mask_xor_v(zb);
        PairDecoder<K, J + 1>::run(w, z, dc);
    }
};
template <int K>
struct PairDecoder<K, 16> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], uint32_t (&)[32], const DecodeConsts &) {}
};

// Codewords [LO, HI) of one chunk (LO, HI multiples of 16), for callers that consume a chunk in two halves to
// keep fewer codewords alive at a time.  v: the words shifted by 16 bits (shifted_words), unused when K divides 16.
template <int K, int I, int HI>
struct SplitRange {
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], const uint32_t (&v)[K], uint32_t (&z)[32]) {
        z[I] = mask_xor_v(mad_code<kAdd>(chunk_state_split<K, I>(w, v)));
        SplitRange<K, I + 1, HI>::run(w, v, z);
    }
};
template <int K, int HI>
struct SplitRange<K, HI, HI> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], const uint32_t (&)[K], uint32_t (&)[32]) {}
};
template <int K, int J, int JHI>
struct PairRange {
    static constexpr int P = 16 / K;
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], uint32_t (&z)[32], const DecodeConsts &dc) {
        constexpr int a = (J / P) * 2 * P + (J % P);
        constexpr int b = a + P;
        constexpr int off = a * K;
        constexpr int q = off >> 5;
        constexpr int o = off & 31;
        uint32_t Q;
        if constexpr (o == 0) Q = w[q];
        else Q = __funnelshift_r(w[q], w[q + 1], o);
        const uint32_t sb = Q >> 16;
        const uint32_t zb = mad_code<kAdd>(sb);
        const uint32_t t = mad_code<kAdd + (kAdd << 16)>(Q);
        const uint32_t za = mad_u32(zb, dc.neg65536, t);
        z[a] = mask_xor_v(za);
        z[b] = mask_xor_v(zb);
        PairRange<K, J + 1, JHI>::run(w, z, dc);
    }
};
template <int K, int JHI>
struct PairRange<K, JHI, JHI> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], uint32_t (&)[32], const DecodeConsts &) {}
};
template <int K>
__device__ __forceinline__ void shifted_words(const uint32_t (&w)[K + 1], uint32_t (&v)[K]) {
    if constexpr (16 % K != 0) {
#pragma unroll
        for (int q = 0; q < K; ++q) v[q] = __funnelshift_r(w[q], w[q + 1], 16);
    }
}
// pairs of a chunk lie inside blocks of 2 * (16 / K) consecutive weights, so a half chunk holds whole pairs for K >= 2
template <int K, int LO, int HI>
__device__ __forceinline__ void decode_range_fast(const uint32_t (&w)[K + 1], const uint32_t (&v)[K], uint32_t (&z)[32],
                                                  const DecodeConsts &dc) {
    static_assert(LO % 16 == 0 && HI % 16 == 0 && K >= 2, "half chunks only, and not at one bit per weight");
    if constexpr (16 % K == 0) PairRange<K, LO / 2, HI / 2>::run(w, z, dc);
    else SplitRange<K, LO, HI>::run(w, v, z);
}

// 32 codewords of one chunk, identical to decode_chunk<K>
template <int K>
__device__ __forceinline__ void decode_chunk_fast(const uint32_t (&w)[K + 1], uint32_t (&z)[32],
                                                  const DecodeConsts &dc) {
    if constexpr (16 % K == 0) PairDecoder<K, 0>::run(w, z, dc);
    else {
        uint32_t v[K];
#pragma unroll
        for (int q = 0; q < K; ++q) v[q] = __funnelshift_r(w[q], w[q + 1], 16);
        SplitDecoder<K, 0>::run(w, v, z);
    }
}

}  // namespace exl3
