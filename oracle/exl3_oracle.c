/*
 * CPU oracle for the EXL3 trellis-quantized linear layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA library; nothing in the shipped package links,
 * loads or calls it.  Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * PARITY UNPINNED for the trellis decode: the reference plugin holds no kernel, no test and
 * no golden vector for the decode.  It forwards to the pybind11 module
 * `exllamav3.ext.exllamav3_ext` of exllamav3 v1.5.1 (docker/Dockerfile:20,31-38), whose
 * source is not part of the reference tree.  The decode below therefore restates the
 * published "3INST" computed codebook of QTIP (arXiv 2406.11235) on a 16-bit-state
 * tail-biting bitshift trellis, with the packing conventions fixed by this repository's
 * format specification (bit order, window position, order of the 256 weights in a tile).
 *
 * What IS pinned by the reference tree and followed here line by line:
 *   - pipeline order  y = ((x * suh) H) W) H * svh          orcasaq2/ops.py:44-60
 *   - Hadamard: Sylvester order, 128 wide, scaled 1/sqrt(128), along the last dim
 *                                                            orcasaq2/__init__.py:33-46
 *   - deploy-weight identity                                 orcasaq2/__init__.py:49-61
 *   - K = trellis.shape[-1] / 16                             orcasaq2/ops.py:28-34
 *   - int8 embedding gather and int8 head                    orcasaq2/heads.py:61-75
 *                                                            orcasaq2/patches/int8_embedding.py:40-43
 *
 * Format (one 16x16 tile = 16*K uint16 words, trellis[ic/16][oc/16][16*K]):
 *   bit n of the tile's circular bit string, n in [0, 256K):  (word[n >> 4] >> (n & 15)) & 1
 *   state of sequence index t in [0,256):  the 16 bits n = t*K .. t*K+15 (mod 256K), bit
 *   n = t*K being the least significant.
 *   sequence index t -> position inside the tile:
 *       c = t >> 5, i = t & 31, p = c >> 2, q = c & 3
 *       row (input channel)  r   = 8*((i>>2)&1) + 4*((i>>1)&1) + q
 *       col (output channel) col = 4*(i>>3) + 2*(i&1) + p
 *   codebook:  z = state*89226354 + 64248484 (mod 2^32);  z = (z & 0x8FFF8FFF) ^ 0x3B603B60;
 *              weight = fp16(lo16(z) as fp16 + hi16(z) as fp16), one rounding (RN-even).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXL3_MUL 89226354u
#define EXL3_ADD 64248484u
#define EXL3_MASK 0x8FFF8FFFu
#define EXL3_XOR 0x3B603B60u

static inline float half_bits_to_float(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

static inline uint16_t float_to_half_bits(float f) {
    _Float16 v = (_Float16)f; /* round-to-nearest-even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

static inline float bf16_bits_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t float_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u); /* RN-even */
    return (uint16_t)(u >> 16);
}

/* 16-bit state -> fp16 weight bits (QTIP "3INST"). */
uint16_t exl3_oracle_decode_state(uint32_t state) {
    uint32_t z = (state & 0xFFFFu) * EXL3_MUL + EXL3_ADD;
    z = (z & EXL3_MASK) ^ EXL3_XOR;
    float lo = half_bits_to_float((uint16_t)(z & 0xFFFFu));
    float hi = half_bits_to_float((uint16_t)(z >> 16));
    /* both halves have magnitude in [2^-3, 2): the fp32 sum is exact, so one rounding to
       fp16 equals a hardware fp16 add */
    return float_to_half_bits(lo + hi);
}

static inline uint32_t tile_state(const uint16_t *tile, int K, int t) {
    const int nbits = 256 * K;
    const int nwords = 16 * K;
    int n = t * K;
    int q = n >> 4, o = n & 15;
    (void)nbits;
    uint32_t v = (uint32_t)tile[q] | ((uint32_t)tile[(q + 1) % nwords] << 16);
    return (v >> o) & 0xFFFFu;
}

static inline void tile_pos(int t, int *r, int *col) {
    int c = t >> 5, i = t & 31, p = c >> 2, q = c & 3;
    *r = 8 * ((i >> 2) & 1) + 4 * ((i >> 1) & 1) + q;
    *col = 4 * (i >> 3) + 2 * (i & 1) + p;
}

/* exported for tests: the 256 sequence states of one tile */
void exl3_oracle_tile_states(const uint16_t *tile, int K, uint16_t *states) {
    for (int t = 0; t < 256; ++t) states[t] = (uint16_t)tile_state(tile, K, t);
}

/* exported for tests: sequence index -> (row, col) */
void exl3_oracle_tile_perm(int32_t *rows, int32_t *cols) {
    for (int t = 0; t < 256; ++t) {
        int r, c;
        tile_pos(t, &r, &c);
        rows[t] = r;
        cols[t] = c;
    }
}

/*
 * trellis [ic/16][oc/16][16K] uint16  ->  w [ic][oc] fp16 bits (the inner weight, before
 * Hadamard and signs).  Stands for ext.reconstruct(w, trellis, k, mcg, mul1),
 * orcasaq2/ops.py:56 and orcasaq2/__init__.py:57.  Returns 0, or -1 on a bad shape / K.
 */
int exl3_oracle_reconstruct(const uint16_t *trellis, int ic, int oc, int K, uint16_t *w) {
    if (ic <= 0 || oc <= 0 || (ic & 15) || (oc & 15) || K < 1 || K > 8) return -1;
    const int ti = ic / 16, tj = oc / 16;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < ti; ++i)
        for (int j = 0; j < tj; ++j) {
            const uint16_t *tile = trellis + ((size_t)i * tj + j) * (size_t)(16 * K);
            for (int t = 0; t < 256; ++t) {
                int r, c;
                tile_pos(t, &r, &c);
                w[(size_t)(16 * i + r) * oc + (16 * j + c)] =
                    exl3_oracle_decode_state(tile_state(tile, K, t));
            }
        }
    return 0;
}

/* In-place 128-point Walsh-Hadamard transform in Sylvester (natural) order, scaled by
   1/sqrt(128): the matrix of orcasaq2/__init__.py:33-40 (symmetric, orthogonal). */
static void fwht128(double *v) {
    for (int h = 1; h < 128; h <<= 1)
        for (int i = 0; i < 128; i += h << 1)
            for (int j = i; j < i + h; ++j) {
                double a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
    const double s = 0.088388347648318440550105545263106; /* 1/sqrt(128) */
    for (int i = 0; i < 128; ++i) v[i] *= s;
}

/*
 * out = H128_blockwise(in * pre) * post * scale along the last dim; fp16 in, fp16 out
 * (rounded once).  Stands for ext.had_r_128(in, out, pre|None, post|None, scale),
 * orcasaq2/ops.py:54,59; the transform itself is _t128 of orcasaq2/__init__.py:43-46.
 * pre / post may be NULL.
 */
int exl3_oracle_had_r_128(const uint16_t *in, uint16_t *out, const uint16_t *pre,
                          const uint16_t *post, float scale, int rows, int n) {
    if (rows < 0 || n <= 0 || (n & 127)) return -1;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        double v[128];
        for (int b = 0; b < n; b += 128) {
            for (int e = 0; e < 128; ++e) {
                double x = half_bits_to_float(in[(size_t)r * n + b + e]);
                if (pre) x *= half_bits_to_float(pre[b + e]);
                v[e] = x;
            }
            fwht128(v);
            for (int e = 0; e < 128; ++e) {
                double y = v[e];
                if (post) y *= half_bits_to_float(post[b + e]);
                y *= scale;
                out[(size_t)r * n + b + e] = float_to_half_bits((float)y);
            }
        }
    }
    return 0;
}

/*
 * The whole layer, "decode, Hadamard, then matmul" in double precision from fp16 inputs,
 * no intermediate rounding:  y = (((x*suh) H) W) H * svh.   y is written as float.
 * Follows orcasaq2/ops.py:44-60 (both branches compute this same function).
 * w is the [ic][oc] fp16 inner weight from exl3_oracle_reconstruct.
 */
int exl3_oracle_layer(const uint16_t *x, int rows, const uint16_t *w, int ic, int oc,
                      const uint16_t *suh, const uint16_t *svh, float *y) {
    if (rows < 0 || (ic & 127) || (oc & 127) || ic <= 0 || oc <= 0) return -1;
    double *xh = (double *)malloc(sizeof(double) * (size_t)ic);
    double *acc = (double *)malloc(sizeof(double) * (size_t)oc);
    if (!xh || !acc) { free(xh); free(acc); return -2; }
    for (int r = 0; r < rows; ++r) {
        for (int e = 0; e < ic; ++e)
            xh[e] = (double)half_bits_to_float(x[(size_t)r * ic + e]) *
                    (double)half_bits_to_float(suh[e]);
        for (int b = 0; b < ic; b += 128) fwht128(xh + b);
#pragma omp parallel for schedule(static)
        for (int o = 0; o < oc; ++o) acc[o] = 0.0;
        /* row-major sweep over w so the inner loop streams */
#pragma omp parallel
        {
            double *loc = (double *)calloc((size_t)oc, sizeof(double));
#pragma omp for schedule(static)
            for (int e = 0; e < ic; ++e) {
                const uint16_t *wr = w + (size_t)e * oc;
                const double xe = xh[e];
                for (int o = 0; o < oc; ++o) loc[o] += xe * (double)half_bits_to_float(wr[o]);
            }
#pragma omp critical
            for (int o = 0; o < oc; ++o) acc[o] += loc[o];
            free(loc);
        }
        for (int b = 0; b < oc; b += 128) fwht128(acc + b);
        for (int o = 0; o < oc; ++o)
            y[(size_t)r * oc + o] = (float)(acc[o] * (double)half_bits_to_float(svh[o]));
    }
    free(xh);
    free(acc);
    return 0;
}

/* y[rows][oc] (fp16, one rounding) = a[rows][ic] @ w[ic][oc], double accumulate.
   Stands for ext.hgemm_recon(a, w, y), orcasaq2/ops.py:57. */
int exl3_oracle_hgemm(const uint16_t *a, const uint16_t *w, uint16_t *y, int rows, int ic,
                      int oc) {
    if (rows < 0 || ic <= 0 || oc <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        double *acc = (double *)calloc((size_t)oc, sizeof(double));
        for (int e = 0; e < ic; ++e) {
            const double xe = half_bits_to_float(a[(size_t)r * ic + e]);
            const uint16_t *wr = w + (size_t)e * oc;
            for (int o = 0; o < oc; ++o) acc[o] += xe * (double)half_bits_to_float(wr[o]);
        }
        for (int o = 0; o < oc; ++o) y[(size_t)r * oc + o] = float_to_half_bits((float)acc[o]);
        free(acc);
    }
    return 0;
}

/*
 * int8 embedding gather: out[t][h] = dt(q[id][h]) * s[id], rounded once to dt.
 * orcasaq2/heads.py:61-67, orcasaq2/patches/int8_embedding.py:40-43.
 * is_bf16 selects dt (0 = fp16, 1 = bf16); s and out hold dt bit patterns.
 */
int exl3_oracle_int8_embed(const int8_t *q, const uint16_t *s, const int64_t *ids, int tokens,
                           int vocab, int hidden, int is_bf16, uint16_t *out) {
    for (int t = 0; t < tokens; ++t)
        if (ids[t] < 0 || ids[t] >= vocab) return -1;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < tokens; ++t) {
        const int64_t id = ids[t];
        const float sc = is_bf16 ? bf16_bits_to_float(s[id]) : half_bits_to_float(s[id]);
        for (int h = 0; h < hidden; ++h) {
            /* int8 -> dt is exact; the product of two dt values is exact in fp32 */
            float v = (float)q[(size_t)id * hidden + h] * sc;
            out[(size_t)t * hidden + h] = is_bf16 ? float_to_bf16_bits(v) : float_to_half_bits(v);
        }
    }
    return 0;
}

/*
 * int8 head: w = dt(q * s) (the weight is rounded to dt first, heads.py:73), then
 * logits[r][v] = sum_h x[r][h] * w[v][h] in double; written as float.  heads.py:69-75.
 */
int exl3_oracle_int8_head(const int8_t *q, const uint16_t *s, const uint16_t *x, int rows,
                          int vocab, int hidden, int is_bf16, float *logits) {
#pragma omp parallel for schedule(static)
    for (int v = 0; v < vocab; ++v) {
        const float sc = is_bf16 ? bf16_bits_to_float(s[v]) : half_bits_to_float(s[v]);
        for (int r = 0; r < rows; ++r) {
            double acc = 0.0;
            for (int h = 0; h < hidden; ++h) {
                float wv = (float)q[(size_t)v * hidden + h] * sc;
                wv = is_bf16 ? bf16_bits_to_float(float_to_bf16_bits(wv))
                             : half_bits_to_float(float_to_half_bits(wv));
                const float xv = is_bf16 ? bf16_bits_to_float(x[(size_t)r * hidden + h])
                                         : half_bits_to_float(x[(size_t)r * hidden + h]);
                acc += (double)xv * (double)wv;
            }
            logits[(size_t)r * vocab + v] = (float)acc;
        }
    }
    return 0;
}
