// Pipe-balanced trellis decode for the fused kernels.
//
// On sm_100 the logic/shift/permute pipe and the integer multiply-add pipe each issue one warp
// instruction every two cycles and run side by side, so a decoder is as fast as the busier of
// the two.  The plain form (shift, mask, multiply-add, mask-xor) puts three of its four
// operations on the logic pipe.  The forms below produce the SAME 32-bit codewords with the work
// split evenly:
//
//  * every K: a window that is not already aligned is first moved so that the state sits in the
//    TOP half of a register (multiply by a power of two when it lies inside one word, one funnel
//    shift when it spans two), and the clean state is then the high word of a widening multiply
//    by 65536 -- one operation on each pipe, no mask.
//  * K = 2, 4, 8 (K divides 16): the 32 bits at a weight's window hold two states,
//    Q = [s_b | s_a] with b = a + 16/K.  s_b is one shift away; the codeword of s_a needs no
//    mask at all, because the multiply is linear modulo 2^32:
//        z_a = s_a*A + B = (Q*A + B + (B << 16)) - 65536 * (s_b*A + B)      (mod 2^32)
//    i.e. two multiply-adds instead of a mask and one multiply-add.
//
// Multipliers that must stay multiplications (so that they are not strength-reduced back into
// shifts on the busy pipe) are passed in registers through `DecodeConsts`, derived from a value
// the compiler cannot see.
#pragma once
#include <stdint.h>
#ifndef EXL3_DECODE_VARIANT
#define EXL3_DECODE_VARIANT 0
#endif

#include "exl3_codec.cuh"

namespace exl3 {

struct DecodeConsts {
    uint32_t c65536;     // 65536
    uint32_t neg65536;   // -65536 mod 2^32
    __device__ __forceinline__ explicit DecodeConsts(uint32_t one) : c65536(one << 16), neg65536(0u - (one << 16)) {}
};

// x >> 16 on the multiply pipe: high word of x * 65536
__device__ __forceinline__ uint32_t shr16_mul(uint32_t x, const DecodeConsts &dc) {
    uint32_t hi;
    asm("{\n\t.reg .b64 p;\n\t.reg .b32 lo;\n\tmul.wide.u32 p, %1, %2;\n\tmov.b64 {lo, %0}, p;\n\t}"
        : "=r"(hi)
        : "r"(x), "r"(dc.c65536));
    return hi;
}

__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// a * kMul + C with both constants as immediates (no register-file reads for them)
template <uint32_t C>
__device__ __forceinline__ uint32_t mad_code(uint32_t a) {
#if EXL3_DECODE_VARIANT >= 1
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "n"(kMul), "n"(C));
    return d;
#else
    return mad_u32(a, kMul, C);
#endif
}
__device__ __forceinline__ uint32_t mask_xor_v(uint32_t z) {
#if EXL3_DECODE_VARIANT >= 1
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(z), "n"(kMask), "n"(kXor));
    return r;
#else
    return mask_xor(z);
#endif
}

// ---- general K: one operation per pipe per extraction -------------------------------------
template <int K, int I>
__device__ __forceinline__ uint32_t chunk_state_balanced(const uint32_t (&w)[K + 1], const DecodeConsts &dc) {
    constexpr int off = I * K;
    constexpr int q = off >> 5;
    constexpr int o = off & 31;
    if constexpr (o == 0) {
        return w[q] & 0xFFFFu;
    } else if constexpr (o == 16) {
        // alternate between the pipes for the windows that need a single shift
        if constexpr ((I & 1) != 0) return w[q] >> 16;
        else return shr16_mul(w[q], dc);
    } else if constexpr (o < 16) {
        const uint32_t top = w[q] * (1u << (16 - o));
        return top >> 16;
    } else {
        const uint32_t top = __funnelshift_r(w[q], w[q + 1], o - 16);
        return shr16_mul(top, dc);
    }
}

template <int K, int I>
struct BalancedDecoder {
    static __device__ __forceinline__ void run(const uint32_t (&w)[K + 1], uint32_t (&z)[32], const DecodeConsts &dc) {
        z[I] = mask_xor_v(mad_code<kAdd>(chunk_state_balanced<K, I>(w, dc)));
        BalancedDecoder<K, I + 1>::run(w, z, dc);
    }
};
template <int K>
struct BalancedDecoder<K, 32> {
    static __device__ __forceinline__ void run(const uint32_t (&)[K + 1], uint32_t (&)[32], const DecodeConsts &) {}
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
        uint32_t sb;
        if constexpr ((J & 1) != 0) sb = Q >> 16;
        else sb = shr16_mul(Q, dc);
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

// 32 codewords of one chunk, identical to decode_chunk<K>
template <int K>
__device__ __forceinline__ void decode_chunk_fast(const uint32_t (&w)[K + 1], uint32_t (&z)[32],
                                                  const DecodeConsts &dc) {
    // Measured on B200 (registers only, 4 warps per scheduler, codewords consumed by mma.sync):
    // K = 4: pair form 218 clk per 32 weights, plain form 221; K = 3: balanced form 266, plain
    // 239; K = 5: balanced 272, plain 233.  The compiler's own pipe balancing of the plain form
    // beats the hand-balanced one where no pairing is possible, so that is what runs there.
    if constexpr (K == 2 || K == 4 || K == 8) PairDecoder<K, 0>::run(w, z, dc);
    else decode_chunk<K>(w, z);
}

}  // namespace exl3
