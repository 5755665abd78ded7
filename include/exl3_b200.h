/*
 * exl3_b200 -- C ABI of the sm_100a kernels for the EXL3 trellis-quantized linear layer.
 *
 * This is the boundary a host runtime binds instead of the pybind11 module
 * `exllamav3.ext.exllamav3_ext` that the orcasaq2 plugin calls.  Every function takes plain
 * device pointers, integer sizes and a CUDA stream (a `cudaStream_t` passed as `void*`,
 * NULL = the legacy default stream), launches asynchronously on that stream, and returns 0
 * or a negative EXL3_E_* code.  Unless a function says otherwise the library allocates
 * nothing, never synchronises the device and keeps no reference to any buffer: the caller
 * owns inputs, outputs and scratch.  There is no CPU fallback.
 *
 * Common conventions
 *   trellis   [ic/16][oc/16][16*K] uint16 words (int16 storage is the same bits), contiguous,
 *             16-byte aligned.  K = bits per weight; passed as k_times_2 (= 2*K) because the
 *             reference API lets K be x.5 (orcasaq2/ops.py:28-34).  Supported here: integer
 *             K in 1..8.  Half rates return EXL3_E_UNSUPPORTED.
 *   fp16      IEEE binary16 bit patterns; activations row-major, contiguous.
 *   mcg, mul1 alternative codebooks selected by flag in the reference
 *             (orcasaq2/ops.py:38, orcasaq2/config.py:218); only the default "3INST"
 *             codebook is defined here, so a non-zero flag returns EXL3_E_UNSUPPORTED.
 *   ic, oc    multiples of 128 wherever a Hadamard is involved (orcasaq2/__init__.py:29,46),
 *             multiples of 16 for exl3_reconstruct.
 */
#ifndef EXL3_B200_H
#define EXL3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EXL3_ABI_VERSION 1

enum {
    EXL3_OK = 0,
    EXL3_E_SHAPE = -1,       /* bad dimension, row count or packed size */
    EXL3_E_ALIGN = -2,       /* pointer not aligned as required */
    EXL3_E_UNSUPPORTED = -3, /* K, codebook flag or mode not implemented */
    EXL3_E_LAUNCH = -4,      /* CUDA reported an error on launch */
    EXL3_E_WORKSPACE = -5,   /* scratch buffer missing or too small */
    EXL3_E_NULL = -6,        /* required pointer is NULL */
    EXL3_E_DEVICE = -7       /* a tensor lives on another device than the current one */
};

int exl3_abi_version(void);
const char *exl3_strerror(int code);

/*
 * Trellis -> dense fp16 inner weight  w[ic][oc]  (before Hadamard and sign vectors).
 * Replaces ext.reconstruct(w, trellis, k, mcg, mul1): orcasaq2/ops.py:56,
 * orcasaq2/__init__.py:57.  Bit-exact against the CPU oracle.
 */
int exl3_reconstruct(void *w, const void *trellis, int ic, int oc, int k_times_2, int mcg,
                     int mul1, void *stream);

/*
 * out = H128(in * pre) * post * scale, blockwise over the last dimension n (a multiple of
 * 128), rows x n fp16, one rounding.  pre / post are fp16 [n] or NULL; in == out is allowed.
 * Replaces ext.had_r_128(in, out, pre, post, scale): orcasaq2/ops.py:54,59.
 * Pointers must be 8-byte aligned; when all of them are 16-byte aligned a kernel with 32 bytes per lane runs
 * (same results, 5.3 against 4.6 TB/s on B200 for 8192 x 17408).
 */
int exl3_had_r_128(const void *in, void *out, const void *pre, const void *post, float scale,
                   int rows, int n, void *stream);

/* One shard of a (possibly fused) layer for exl3_gemv_grouped. */
typedef struct exl3_shard {
    const void *trellis; /* [ic/16][oc/16][16K] uint16 */
    const void *suh;     /* [ic] fp16 */
    const void *svh;     /* [oc] fp16 */
    int oc;              /* output features of this shard (multiple of 128) */
    int k_times_2;       /* 2 * bits per weight */
    int mcg, mul1;       /* codebook flags; must be 0 */
    int out_col;         /* first column of this shard inside y */
} exl3_shard;

#define EXL3_MAX_SHARDS 8
#define EXL3_GEMV_MAX_ROWS 16

/*
 * Fused decode GEMV for 1..16 rows:   y[:, out_col : out_col+oc] = H(H(x*suh) W) * svh
 * for every shard, in ONE launch.  All shards read the same x [rows][ic]; y is [rows][ldy]
 * fp16 (ldy >= the widest out_col+oc), so a fused qkv_proj / gate_up_proj needs no
 * concatenation.  Replaces ext.exl3_gemm(A, trellis, C, suh, A_had, svh, kernel, mcg, mul1,
 * acc_mode) for small row counts (orcasaq2/ops.py:46-49) and the per-shard loop plus
 * torch.cat of orcasaq2/config.py:236-243.
 *
 * workspace: device scratch of at least exl3_gemv_workspace_bytes(...) bytes, 256-byte
 * aligned, ZERO-FILLED ONCE by the caller before its first use (its first word is a sticky
 * status word, the rest holds the rotated activations between the two launches of a call).
 * Calls that share a workspace must not overlap on the device.
 */
size_t exl3_gemv_workspace_bytes(const exl3_shard *shards, int nshards, int rows, int ic);
/* How exl3_gemv_grouped would cut this launch on the current device: CTAs of the grid, and input slices per
 * 128-column block (= CTAs per thread-block cluster; 1 = no cluster).  For diagnosis and tests. */
int exl3_gemv_plan(const exl3_shard *shards, int nshards, int rows, int ic, int *ctas_out, int *slices_out);
int exl3_gemv_grouped(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                      int ic, int ldy, void *workspace, size_t workspace_bytes, void *stream);

/*
 * exl3_gemv_grouped with the elementwise neighbours of the layer folded in (no counterpart in the
 * reference plugin, which leaves these to the serving engine): the input transform runs inside the
 * activation pre-pass, the residual add inside the output epilogue.
 *   in_mode 0  x is used as it is ([rows][ldx], ldx >= ic)
 *   in_mode 1  RMSNorm first: x * rsqrt(mean(x^2) + eps) * norm_weight (norm_weight fp16 [ic] or NULL
 *              for all ones), rounded to fp16 as a stand-alone norm would
 *   in_mode 2  gated activation first: silu(x[:, 0:ic]) * x[:, ic:2ic]  (x is [rows][ldx], ldx >= 2*ic)
 *   residual   optional fp16 [rows][ld_residual] added to every output before its single rounding;
 *              may alias y (in-place residual update)
 * ldx / ld_residual: 0 selects the natural value.  fusion == NULL is exl3_gemv_grouped.
 */
typedef struct exl3_gemv_fusion {
    int in_mode;
    const void *norm_weight;
    float eps;
    int ldx;
    const void *residual;
    int ld_residual;
} exl3_gemv_fusion;
int exl3_gemv_grouped_ex(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                         int ic, int ldy, void *workspace, size_t workspace_bytes,
                         const exl3_gemv_fusion *fusion, void *stream);

/* Single-shard convenience form of exl3_gemv_grouped (y is [rows][oc]). */
int exl3_gemv(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
              int rows, int ic, int oc, int k_times_2, int mcg, int mul1, void *workspace,
              size_t workspace_bytes, void *stream);

/*
 * Many-row form (mid-batch and prefill):  y[rows][oc] = H(H(x*suh) W) * svh  on tcgen05.mma (fp32
 * accumulators in tensor memory).  Up to 1023 rows the trellis is decoded inside the kernel (into tensor
 * memory up to 128 rows, into shared-memory fp16 tiles above) and the decoded weight is never written to
 * global memory.  From 1024 rows (from 384 .. 640 rows for wide layers), when oc / 128 is even, the weight is rebuilt ONCE per call into the scratch
 * (transposed) and a dense GEMM runs on CTA pairs (tcgen05.mma.cta_group::2): the reference's own many-row idea,
 * orcasaq2/ops.py:50-59, with this library's GEMM in the place of hgemm_recon.  That GEMM keeps the tokens in the
 * accumulator's lanes, so its epilogue applies the output rotation and svh to the fp32 sums in registers and writes
 * the final fp16 result (no pass over the output, one rounding); this needs y and svh 16-byte aligned and ldy a
 * multiple of 8.  With an output that is only 8-byte aligned the rotation is folded into the rebuilt weight or runs
 * as a pass over y, whichever is cheaper (folding changes the rounding by about one fp16 ulp of the weights).
 * x is fp16 (or bf16 when x_is_bf16; it is narrowed to fp16 as the reference does,
 * orcasaq2/config.py:233), y fp16, scratch a caller buffer of exl3_gemm_tc_scratch_bytes() bytes,
 * 256-byte aligned: the rotated activations (the reference's `xh`, orcasaq2/ops.py:53) and, when the
 * output grid alone cannot fill the GPU, fp32 partial sums of the input slices; from 1024 rows the rebuilt
 * weight (ic*oc*2 bytes, the reference's `w`, ops.py:55-56).  Replaces the rows > GEMM_MAX_ROWS branch
 * had_r_128 -> reconstruct -> hgemm_recon -> had_r_128 of orcasaq2/ops.py:50-59 (and serves
 * 17..144 rows, which the reference sends to exl3_gemm).  Three or four launches on `stream`.
 * exl3_gemm_tc_status() returns a sticky device word that is non-zero only if a bounded wait
 * inside the kernel ran out (it synchronises the device; for diagnosis and tests).
 */
size_t exl3_gemm_tc_scratch_bytes(int rows, int ic, int oc);
int exl3_gemm_tc(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
                 void *scratch, size_t scratch_bytes, int rows, int ic, int oc, int k_times_2, int mcg,
                 int mul1, int x_is_bf16, void *stream);
/*
 * exl3_gemm_tc with the elementwise neighbours of the layer folded in, as exl3_gemv_grouped_ex does
 * for few rows (no counterpart in the reference plugin): the input transform (fusion->in_mode, see
 * exl3_gemv_fusion) runs inside the activation pre-pass, the residual add inside the output
 * post-pass, and y may be a column block of a wider matrix: row pitch ldy >= oc elements, a multiple
 * of 4 (this is what removes the torch.cat of orcasaq2/config.py:236-242 for fused layers).
 * fusion == NULL and ldy == oc is exl3_gemm_tc.  Up to 128 rows every
 * combination is served; beyond that a pitch or a residual is refused with EXL3_E_UNSUPPORTED when
 * the shape runs unsplit (the caller then applies them itself); the pair kernel (from 1024 rows) takes
 * a pitch, no residual.
 */
int exl3_gemm_tc_ex(const void *x, const void *trellis, void *y, const void *suh, const void *svh,
                    void *scratch, size_t scratch_bytes, int rows, int ic, int oc, int k_times_2, int mcg,
                    int mul1, int x_is_bf16, int ldy, const exl3_gemv_fusion *fusion, void *stream);
/*
 * All shards of a fused layer (qkv_proj, gate_up_proj) at up to 128 rows in three launches: the
 * grouped form of exl3_gemm_tc_ex, as exl3_gemv_grouped is of exl3_gemv.  y is [rows][ldy]; shard s
 * writes columns out_col .. out_col + oc.  Above 128 rows:
 * EXL3_E_UNSUPPORTED (scratch size 0) and the caller goes shard by shard.
 * Replaces the per-shard loop + torch.cat of orcasaq2/config.py:236-242.
 */
size_t exl3_gemm_tc_grouped_scratch_bytes(const exl3_shard *shards, int nshards, int rows, int ic);
int exl3_gemm_tc_grouped(const exl3_shard *shards, int nshards, const void *x, void *y, int rows, int ic,
                         int ldy, void *scratch, size_t scratch_bytes, int x_is_bf16,
                         const exl3_gemv_fusion *fusion, void *stream);
unsigned exl3_gemm_tc_status(void);
int exl3_gemm_tc_status_reset(void);

/*
 * Self-tests of the bounded waits (no counterpart in the reference): every wait on an mbarrier inside these
 * kernels gives up after a limit, sets a sticky status word and lets the kernel return.  These entry points
 * launch ONE warp that waits, through the kernels' own wait helpers, on a barrier nothing will ever complete,
 * with a short limit, so that the give-up path can be exercised without any fault: afterwards the status word
 * is non-zero and the device is as usable as before.
 *   exl3_gemv_selftest_wait     the GEMV's poll-counted wait; the word set is the first word of `workspace`
 *                               (any 4-byte-aligned device word, e.g. a scratch of its own); 1 <= polls <= 2^20
 *   exl3_gemm_tc_selftest_wait  the timer-bounded waits of exl3_gemm_tc (which 0: shared-memory-operand kernel,
 *                               1: tensor-memory kernel); limit in microseconds; sets the word exl3_gemm_tc_status
 *                               reports (clear it with exl3_gemm_tc_status_reset)
 */
int exl3_gemv_selftest_wait(void *workspace, int polls, void *stream);
int exl3_gemm_tc_selftest_wait(int which, unsigned limit_us, void *stream);

/*
 * exl3_gemv_grouped without a caller-supplied workspace.  This entry point has no counterpart
 * in the reference.  It exists for hosts that cannot allocate device memory where the layer
 * runs: a serving process that has already handed every free byte to its KV-cache pool, an
 * engine whose hot path is forbidden to call the allocator (no cudaMalloc, no torch caching
 * allocator) for latency or fragmentation reasons, or a plugin loaded into a runtime that owns
 * all memory.  The rotated activations that pass from the first launch of a call to the second, and the status word, live in a fixed array
 * inside the library (exl3_gemv_static_capacity() bytes, currently 2 MiB, held on every GPU
 * that loads the library until the process exits); the call itself allocates nothing and calls
 * no allocating routine.
 *
 *   - Inputs, outputs and all argument rules are those of exl3_gemv_grouped.
 *   - A launch whose scratch need (exl3_gemv_workspace_bytes) exceeds the capacity returns
 *     EXL3_E_WORKSPACE and launches nothing; use exl3_gemv_grouped with your own buffer then.
 *   - The scratch used is the copy of the array on the CURRENT device.  x and y must live on that
 *     device; a call made with another device current returns EXL3_E_DEVICE and launches nothing.
 *   - The FIRST call on each device looks up the array's device address (once, under a lock, so
 *     host threads may race to it); make that first call with the device current and before any
 *     stream capture begins.  Nothing is cleared at that point: the loader hands the array over
 *     zero-filled, which is the state the status word needs.
 *   - All calls on a device share the one array, which keeps what the last call left in it
 *     (every call overwrites what it reads; only the status word is sticky): two calls that
 *     overlap on the GPU (different streams without ordering, or two host threads launching
 *     without ordering between their streams) race on it.  Serialise them.
 *   - exl3_gemv_static_status(&word) copies the sticky status word of the current device's array
 *     to the host (it waits for the device; for diagnosis and tests): 0, or non-zero after a
 *     bounded wait inside a kernel launched through this entry point ran out.
 */
size_t exl3_gemv_static_capacity(void);
int exl3_gemv_grouped_static(const exl3_shard *shards, int nshards, const void *x, void *y, int rows,
                             int ic, int ldy, void *stream);
int exl3_gemv_static_status(unsigned *status_out);

/*
 * The word at byte offset 0 of a GEMV workspace is a sticky device-side status: 0, or
 * non-zero after a bounded wait inside a kernel ran out.  Read it with a device-to-host copy
 * when diagnosing; it is never set in normal operation.
 */
#define EXL3_WS_STATUS_OFFSET 0

/*
 * int8 embedding gather:  out[t][:] = dt(q[ids[t]][:]) * scales[ids[t]], one rounding to dt
 * (dt = fp16, or bf16 when is_bf16).  qweight [vocab][hidden] int8 (hidden a multiple of 16),
 * scales [vocab] dt, ids [tokens] int64 (int32 when ids_are_i32), out [tokens][hidden] dt.
 * An id outside [0, vocab) yields a zero row and, if bad_id_flag (a device uint32) is not
 * NULL, sets it to 1.  Replaces Exl3EmbeddingMethod.embedding (orcasaq2/heads.py:61-67) and
 * Int8EmbeddingTable.forward (orcasaq2/patches/int8_embedding.py:40-43).  Bit-exact.
 */
int exl3_int8_embed(const void *qweight, const void *scales, const void *ids, void *out, int tokens,
                    int vocab, int hidden, int is_bf16, int ids_are_i32, void *bad_id_flag,
                    void *stream);

/*
 * int8 head:  logits[r][v] = scales[v] * sum_h x[r][h] * q[v][h]  for 1..64 rows per call, written as dt
 * with leading dimension ld_logits.  hidden must be a multiple of 64 (of 256, with x 16-byte aligned,
 * above 16 rows).  The table is streamed ONCE per call as int8 and never dequantised into memory: up to 16
 * rows the activations stay resident in shared memory, above that they are staged chunk by chunk.  Replaces Exl3EmbeddingMethod.apply
 * (orcasaq2/heads.py:69-75), which materialises the dt table on every call; that version
 * rounds q*s to dt before the product, this one scales the exact integer dot product, so the
 * two agree within the layer tolerance, not bit for bit.
 */
#define EXL3_INT8_HEAD_MAX_ROWS 64
int exl3_int8_head(const void *qweight, const void *scales, const void *x, void *logits, int rows,
                   int vocab, int hidden, long long ld_logits, int is_bf16, void *stream);

/*
 * Decode attention over a contiguous fp16 KV cache: one query token per sequence,
 *     out[b][h][:] = softmax(q[b][h] . K[b][h / G]^T * scale) . V[b][h / G],   G = q_heads / kv_heads.
 * The reference has no attention code of its own: it leaves this step to the serving engine
 * (presets/16gb.env:17-18 pick the engine's attention backend), and it is the largest HBM stream
 * of a decode step next to the quantised weights, so the model-level benchmark needs it.
 *   q, out       [batch][q_heads][256] fp16, batches q_batch_stride / out_batch_stride elements apart
 *   k_cache, v_cache   [batch][kv_heads][capacity][256] fp16: element strides kv_batch_stride and
 *                kv_head_stride (multiples of 8), 16-byte aligned; tokens 0 .. seq_len-1 are read
 *   head_dim     must be 256; G must be 1..8
 *   workspace    exl3_decode_attn_workspace_bytes(...) bytes, 16-byte aligned (partial results of
 *                the sequence splits); may be NULL when that size is 0
 * Query head h uses KV head h / G (consecutive query heads share a KV head).  fp32 accumulation,
 * probabilities rounded to fp16 before the product with V.
 */
size_t exl3_decode_attn_workspace_bytes(int batch, int q_heads, int kv_heads, int seq_len);
int exl3_decode_attn(const void *q, const void *k_cache, const void *v_cache, void *out,
                     void *workspace, size_t workspace_bytes, int batch, int q_heads, int kv_heads,
                     int head_dim, int seq_len, long long q_batch_stride, long long out_batch_stride,
                     long long kv_batch_stride, long long kv_head_stride, float scale, void *stream);

/*
 * exl3_decode_attn over a paged cache.  k_pages / v_pages are page pools of equal layout; a page
 * holds page_size tokens (a multiple of 16) of every KV head: the element of (page p, head h, token
 * t, dimension d) is at p*page_stride + h*head_stride + t*token_stride + d, all strides multiples
 * of 8, which covers both [pages][heads][page_size][256] and [pages][page_size][heads][256].
 *   block_table  int32 [batch][block_table_stride]: the page of tokens i*page_size ... of a sequence
 *   seq_lens     int32 [batch] tokens to read per sequence, each <= max_seq_len, or NULL when every
 *                sequence has max_seq_len tokens; a sequence of length 0 yields a zero row
 *   workspace    exl3_decode_attn_workspace_bytes(batch, q_heads, kv_heads, max_seq_len) bytes
 * block_table must cover ceil(max_seq_len / page_size) entries per sequence; entries beyond a
 * sequence's own length are not read.  Everything else as for exl3_decode_attn.
 */
int exl3_decode_attn_paged(const void *q, const void *k_pages, const void *v_pages, const void *block_table,
                           const void *seq_lens, void *out, void *workspace, size_t workspace_bytes,
                           int batch, int q_heads, int kv_heads, int head_dim, int max_seq_len,
                           int page_size, int block_table_stride, long long q_batch_stride,
                           long long out_batch_stride, long long page_stride, long long head_stride,
                           long long token_stride, float scale, void *stream);

/*
 * The step before exl3_decode_attn, in one launch: rotary embedding (rotate-half form, fp32 math,
 * one rounding) of the query and key heads of one new token per sequence, and the append of the
 * rotated key and of the value to the caches at token index pos.  Like the attention itself this
 * has no counterpart in the reference (the serving engine does it there).
 *   qkv      [batch][ld_qkv] fp16: q_heads, then kv_heads key heads, then kv_heads value heads, 256
 *            elements each; the query heads are rotated in place
 *   cos, sin [128] fp16 of this position, or one row per sequence cos_sin_batch_stride elements
 *            apart (0 = the same row for every sequence)
 *   k_cache, v_cache   as for exl3_decode_attn; capacity must exceed pos
 */
int exl3_rope_append(void *qkv, int ld_qkv, const void *cos, const void *sin, int cos_sin_batch_stride,
                     void *k_cache, void *v_cache, int batch, int q_heads, int kv_heads, int head_dim,
                     int pos, long long kv_batch_stride, long long kv_head_stride, void *stream);

/*
 * The same three steps over an fp8 cache (e4m3 bytes, one positive scale per tensor for K and one for V: the
 * cache holds value / scale; the form the engine keeps under `--kv-cache-dtype fp8`, reference
 * presets/16gb.env:17).  q and out stay fp16.  Arguments as for the fp16 entry points, except: cache strides are in
 * elements = bytes and must be multiples of 16; the workspace size comes from exl3_decode_attn_fp8_workspace_bytes
 * (rings are half as large, two CTAs share an SM, so the sequence is cut differently); k_scale and v_scale must be
 * > 0.  The bytes are widened to fp16 exactly in registers, so the result equals the fp16 kernel's arithmetic on
 * the dequantised cache (K . k_scale folded into the softmax scale, V . v_scale into the normalisation).
 * exl3_rope_append_fp8 rounds the rotated key to fp16 first, then value / scale to e4m3 with saturation.
 */
size_t exl3_decode_attn_fp8_workspace_bytes(int batch, int q_heads, int kv_heads, int seq_len);
int exl3_decode_attn_fp8(const void *q, const void *k_cache, const void *v_cache, void *out,
                         void *workspace, size_t workspace_bytes, int batch, int q_heads, int kv_heads,
                         int head_dim, int seq_len, long long q_batch_stride, long long out_batch_stride,
                         long long kv_batch_stride, long long kv_head_stride, float scale, float k_scale,
                         float v_scale, void *stream);
int exl3_decode_attn_paged_fp8(const void *q, const void *k_pages, const void *v_pages, const void *block_table,
                               const void *seq_lens, void *out, void *workspace, size_t workspace_bytes,
                               int batch, int q_heads, int kv_heads, int head_dim, int max_seq_len,
                               int page_size, int block_table_stride, long long q_batch_stride,
                               long long out_batch_stride, long long page_stride, long long head_stride,
                               long long token_stride, float scale, float k_scale, float v_scale, void *stream);
int exl3_rope_append_fp8(void *qkv, int ld_qkv, const void *cos, const void *sin, int cos_sin_batch_stride,
                         void *k_cache, void *v_cache, int batch, int q_heads, int kv_heads, int head_dim,
                         int pos, long long kv_batch_stride, long long kv_head_stride, float k_scale,
                         float v_scale, void *stream);

/*
 * Measurement probe (no counterpart in the reference, not on the layer's path): the rate at which the GPU can
 * decode the 3INST codebook with this library's decode routines and consume the codewords with mma.sync, on every
 * SM.  mode 0: words never leave registers (the ceiling the integer decode sets for any kernel of this design);
 * mode 1: words come from a shared-memory ring refilled by bulk async copies from a small L2-resident buffer,
 * with the waits and loads of a real streaming loop.  Launches one kernel of `iters` iterations on `stream`;
 * *weights_out receives the number of weights it decodes (time it with events).  scratch: at least 1 MiB + 8.5
 * KiB of device memory, 256-byte aligned, first word zero (set non-zero if a bounded wait ran out).
 */
int exl3_probe_decode_rate(int k, int mode, int iters, void *scratch, size_t scratch_bytes, double *weights_out,
                           void *stream);

/*
 * One-shot all-reduce (sum) of fp16 partial results over peer memory, for the outputs of row-parallel layers
 * under tensor parallelism: one launch, no library collective.  The reference refuses tensor parallelism
 * (orcasaq2/config.py:173-177); the engine around it would call a library all-reduce after every row-parallel
 * projection (vllm/model_executor/layers/linear.py:1556-1559), which at decode sizes is pure latency.
 *
 * Every rank owns one communication buffer of exl3_allreduce_buffer_bytes(max_values) bytes that every other
 * rank has mapped; peer_buffers[r] is rank r's buffer as THIS process addresses it (peer_buffers[rank] is the
 * own one).  exl3_comm_alloc makes such a buffer (the one place this library allocates device memory: a
 * zero-filled cudaMalloc block, plus its 64-byte CUDA IPC handle for the other processes of the node),
 * exl3_comm_open maps a peer's buffer from its handle, exl3_comm_close / exl3_comm_free undo them.  All ranks
 * must have finished allocating and mapping (a host barrier) before the first call.
 *
 * exl3_allreduce_oneshot: out[i] = sum over ranks of in[i], i < n_values (a multiple of 8; in, out 16-byte
 * aligned; out == in allowed), added in fp32 in rank order, so all ranks get bitwise the same result.  Every
 * rank must make the same sequence of calls with the same n_values on buffers of the same size.  Peers are
 * reached with plain loads and stores only.  A wait inside the kernel gives up after spin_limit polls (0 = a
 * default worth a fraction of a second): the kernel then sets the buffer's sticky status word (exl3_comm_status, which waits for
 * the device), leaves that part of out untouched and returns.
 */
#define EXL3_AR_MAX_RANKS 8
size_t exl3_allreduce_buffer_bytes(size_t max_values);
int exl3_allreduce_oneshot(void *const *peer_buffers, int rank, int world, size_t buffer_bytes, const void *in,
                           void *out, long long n_values, int spin_limit, void *stream);
int exl3_comm_alloc(size_t bytes, void **ptr_out, void *ipc_handle_out64);
int exl3_comm_open(const void *ipc_handle64, void **ptr_out);
int exl3_comm_close(void *ptr);
int exl3_comm_free(void *ptr);
int exl3_comm_status(const void *own_buffer, unsigned *status_out);

#ifdef __cplusplus
}
#endif
#endif /* EXL3_B200_H */
