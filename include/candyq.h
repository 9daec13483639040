/*
 * candyq.h -- C ABI of libcandyq: block-quantized (Q4_0 / Q8_0) matmul for gocnn/candy
 * on NVIDIA B200 (sm_100a).
 *
 * The reference (gocnn/candy) has no FFI for its tensor backends: its CUDA backend is
 * an empty Go package (tensor/internal/cuda/device.go:1, storage.go:1) beside unlaunched
 * kernel sources and a registry of kernel names (tensor/internal/cuda/kernels/kernels.go:
 * 482-631).  This header is the boundary a cgo file in tensor/internal/cuda binds to make
 * that backend real for the quantized linear.  The only C-ABI precedent in the reference
 * is llm/internal/flashattn/flash_api.h:71-117 (extern "C", raw device pointers, strides
 * in elements); unlike it, every entry point here returns a status and never aborts.
 *
 * Conventions
 *  - All pointers named *_dev are device pointers on the context's GPU; *_host are host
 *    pointers.  Sizes are in elements unless the name says bytes.
 *  - A weight matrix W[n,k] is n*k/32 blocks, row-major: row r = blocks r*k/32 ...
 *    (r+1)*k/32-1 (same layout the reference kernels index, quantized.cu:1279, :2827).
 *    Q4_0 block = 18 bytes {f16 d; u8 qs[16]}; Q8_0 block = 34 bytes {f16 d; i8 qs[32]}
 *    (tensor/internal/cpu/kernels/quantized.go:8-11, :34-37).  Little-endian, no padding.
 *  - Launches are asynchronous on the context's stream; cq_synchronize waits and reports
 *    deferred device-side errors.  One context must not be used from two threads at once.
 *  - The library has no CPU fallback: without a usable GPU every compute entry fails.
 */
#ifndef CANDYQ_H
#define CANDYQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t cq_status;
enum {
    CQ_OK = 0,
    CQ_ERR_INVALID_ARG = -1, /* null pointer, k % 32 != 0, ld too small, unknown enum ...   */
    CQ_ERR_CUDA = -2,        /* a CUDA runtime call failed; cq_last_error has the text      */
    CQ_ERR_UNSUPPORTED = -3, /* valid request this build has no kernel for                   */
    CQ_ERR_TIMEOUT = -4,     /* a bounded device-side wait gave up (reported at synchronize) */
    CQ_ERR_NOMEM = -5,
    CQ_ERR_TOO_LARGE = -6    /* beyond a stated fixed limit of the entry point               */
};

typedef struct cq_ctx cq_ctx;

/* Block formats; values follow the GGML type ids the reference's registry names use. */
enum cq_qtype {
    CQ_Q4_0 = 2,
    CQ_Q4_1 = 3, /* 20 bytes {f16 d; f16 m; u8 qs[16]}: d*q + m         quantized.go:13-17, :107-116        */
    CQ_Q5_0 = 6, /* 22 bytes {f16 d; u32 qh; u8 qs[16]}: d*(q-16)       quantized.go:19-24, quantized.cu:749-771 */
    CQ_Q5_1 = 7, /* 24 bytes {f16 d; f16 m; u32 qh; u8 qs[16]}: d*q + m quantized.go:26-31, quantized.cu:773-795 */
    CQ_Q8_0 = 8,
    /* 256-value super-blocks, defined by the reference's CUDA dequantizers (quantized.cu:366-436 layouts, :899-1147):
     * dequantize (bit-exact), decode GEMV with f32 activations, tensor-core GEMM through an f16 copy; no quantizer
     * (the reference has none), k % 256 == 0, order CQ_ORDER_GGML_SPLIT only. */
    CQ_Q2_K = 10, /* 84 bytes  */
    CQ_Q3_K = 11, /* 110 bytes */
    CQ_Q4_K = 12, /* 144 bytes */
    CQ_Q5_K = 13, /* 176 bytes */
    CQ_Q6_K = 14  /* 210 bytes */
};
/* Q4_1 / Q5_0 / Q5_1: dequantize, quantize and matmul with CQ_ACT_F32 (a plain GEMV) or CQ_ACT_F16
 * (tensor-core GEMM through an f16 copy); CQ_ACT_Q8_1 and the fused / multi-GPU entries answer
 * CQ_ERR_UNSUPPORTED.  The 5-bit formats exist in the split order only. */

/* Which of the 32 values each Q4_0 nibble is.  The reference disagrees with itself:
 * CQ_ORDER_GO_INTERLEAVED  byte j -> values 2j (low), 2j+1 (high)   quantized.go:87-92
 * CQ_ORDER_GGML_SPLIT      byte j -> values j (low), j+16 (high)    quantized.cu:862-866
 * Ignored for Q8_0. */
enum cq_order { CQ_ORDER_GO_INTERLEAVED = 0, CQ_ORDER_GGML_SPLIT = 1 };

/* How activations enter the dot products.
 * CQ_ACT_F32   f32 activations in, f32 out, no quantization the caller can see: the mode that
 *              stands in for candy's CPU path (dequantize, then conv.go:373-389).  Inside the
 *              decode GEMV each 32-block of activations is held as 16-bit block fixed point
 *              (X = rint(x * 32767 / max|x|)), the dots are exact integers and blocks are summed
 *              in f32: within about 1e-5 of max|y| of the CPU path (bar 1e-3).  The context
 *              option gemv_variant = 3 (three int8 residual slices) or 1 (plain f32 FMAs)
 *              resolves activations to f32 level, about 1e-6, at a lower rate.
 * CQ_ACT_Q8_1  activations quantized per 32 to int8 exactly as quantize_q8_1
 *              (quantized.cu:3521-3558), integer dots scaled per block as
 *              vec_dot_q4_0_q8_1 / vec_dot_q8_0_q8_1 (quantized.cu:1919-1941, :2058-2073).
 * CQ_ACT_F16   activations and dequantized weights rounded to f16, f32 accumulate on
 *              the tensor cores (prefill GEMM). */
enum cq_actmode { CQ_ACT_F32 = 0, CQ_ACT_Q8_1 = 1, CQ_ACT_F16 = 2 };

const char *cq_status_string(cq_status s);
/* Text of the most recent failure on this context ("" if none).  Owned by the context. */
const char *cq_last_error(const cq_ctx *ctx);
/* Library build tag, e.g. "candyq sm_100a". */
const char *cq_version(void);

/* ---- device / memory: what candy.BackendDevice needs (device.go:49-82) -------------- */
cq_status cq_device_count(int *count);
cq_status cq_ctx_create(int device, cq_ctx **out);
cq_status cq_ctx_destroy(cq_ctx *ctx);
/* Run subsequent launches on a caller-owned cudaStream_t (0 restores the context's own). */
cq_status cq_ctx_set_stream(cq_ctx *ctx, void *cuda_stream);
/* Tuning knobs (launch geometry, decoder choice); unknown keys -> CQ_ERR_INVALID_ARG.  Results stay
 * inside each activation mode's stated distance from the CPU path whatever the options are. */
cq_status cq_ctx_set_option(cq_ctx *ctx, const char *key, int64_t value);
/* Options: gemv_warps, gemv_stages, gemv_ctas_per_sm, gemv_rpt, gemv_coop, gemv_pdl, gemv_early (launch geometry of the
 * decode GEMV); gemv_variant (0 default, see CQ_ACT_F32); gemv_multirow (0: one weight pass per activation
 * row); gemv_chain (0, default; 1: the GEMVs launched while it is set are links of a chain with small kernels in
 * between, as in a decode step: unless gemv_warps was set explicitly they run as one CTA of twelve warps per SM);
 * gemv_independent (0, default; 1: the caller promises that the one-row GEMVs launched while it is set neither
 * read nor overwrite anything an earlier launch still in flight writes -- q / k / v or gate / up projections of one x --
 * so they skip the wait on the previous kernel and overlap its last rows; undefined results if the promise does not
 * hold); gemv_q81_inline (1, default: one or two rows in CQ_ACT_Q8_1 quantize their activations inside the GEMV's
 * set-up; 0: in a launch of their own first; the same bits either way); gemv_mma (3, default: CQ_ACT_F32 and CQ_ACT_Q8_1 batches of this many rows up to eight against Q4_0 run the
 * single-launch kernel with mma.sync block dots, two rows too against large weights, and CQ_ACT_F16 batches of up to
 * eight rows its f16 form; 0: never); gemv_force_simple; gemm_variant, gemm_cache_weights (keep an f16 copy of each weight matrix the wide
 * GEMM has seen: the weights must then stay unchanged, or be rewritten only through cq_* entry points, or
 * cq_invalidate_weight_cache must be called); gemm_pair (1, default: CQ_ACT_F16 batches beyond 384 rows run 256 x 256
 * tiles on CTA pairs; 0: 128 x 256 tiles per CTA); gemm_fused_dequant (1, default: Q4_0 batches of 129..384 rows in
 * CQ_ACT_F16 dequantize the raw blocks inside the GEMM instead of making an f16 copy of W; 2: at every batch size;
 * 0: never); gemm_int8 (1, default: batches of i8_min_rows_q8_1 (3) or more
 * rows in CQ_ACT_Q8_1 and of i8_min_rows_f32 (3) or more in CQ_ACT_F32 run the int8 tensor-core kernel, one
 * weight pass per batch; 0: the decode kernels, up to eight rows a pass); attn_variant (decode attention: 1 = one CTA per 32-key chunk for grouped heads instead of split contexts, 2 = never the
 * single-launch cluster kernel of short contexts); comm_poll_limit (polls before the reducing
 * norm gives up on a peer's data, default about one second's worth); comm_cluster; host_zero_copy (see
 * cq_qmatmul_host); fa_transpose_v (1: cq_flash_attention always transposes V into scratch first; 0, default: V tiles
 * are read in place when V is 16-byte aligned with strides that are multiples of 8 elements). */
/* Grows the context's scratch memory to at least `bytes` now, so that no later call has to (scratch cannot
 * grow while the stream is being captured: such a call fails with CQ_ERR_INVALID_ARG and leaves the capture
 * intact).  A block outgrown while graphs made by cq_capture_end exist is kept until the last of them is
 * destroyed, because they point into it; graphs the caller captured by other means are the caller's to
 * protect (reserve up front). */
cq_status cq_reserve(cq_ctx *ctx, size_t bytes);
/* Drops cached f16 copies (option gemm_cache_weights) of weight matrices whose blocks start inside
 * [blocks_dev, blocks_dev + bytes): call after rewriting such blocks by any means other than cq_quantize_rows,
 * cq_memcpy_h2d / _d2d or cq_memset, which do it themselves. */
cq_status cq_invalidate_weight_cache(cq_ctx *ctx, const void *blocks_dev, size_t bytes);
cq_status cq_malloc(cq_ctx *ctx, size_t bytes, void **dptr);     /* BackendDevice.Alloc   */
cq_status cq_free(cq_ctx *ctx, void *dptr);
cq_status cq_malloc_host(cq_ctx *ctx, size_t bytes, void **hptr); /* pinned host memory   */
cq_status cq_free_host(cq_ctx *ctx, void *hptr);
cq_status cq_memset(cq_ctx *ctx, void *dptr, int byte, size_t bytes);            /* Zeros */
cq_status cq_memcpy_h2d(cq_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
                                                          /* BackendDevice.StorageFromSlice */
cq_status cq_memcpy_d2h(cq_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
                                                          /* BackendStorage.Data, backend.go:9 */
cq_status cq_memcpy_d2d(cq_ctx *ctx, void *dst_dev, const void *src_dev, size_t bytes);
                                                          /* BackendStorage.Clone, backend.go:6 */
cq_status cq_synchronize(cq_ctx *ctx);                    /* BackendDevice.Synchronize, device.go:80-81 */

/* ---- block formats ------------------------------------------------------------------ */
/* Bytes of n*k/32 blocks of `qtype`, or 0 for bad arguments. */
size_t cq_blocks_bytes(int qtype, int64_t n, int64_t k);

/* f32 W[n,k] (row-major, contiguous) -> blocks.  Replaces the reference's only weight
 * quantizers, the Metal shaders kernel_cpy_f32_q4_0 / kernel_cpy_f32_q8_0
 * (tensor/internal/metal/kernels/quantized.metal:4149-4214, :4091-4147).  For Q4_0,
 * `order` picks the nibble packing so that cq_dequantize with the same order returns
 * the values in source order. */
cq_status cq_quantize_rows(cq_ctx *ctx, int qtype, int order, const float *w_dev, int64_t n,
                           int64_t k, void *blocks_dev);

/* blocks -> f32, bit-exact (nblocks counts 32-value blocks, or 256-value super-blocks for the K formats).  Replaces DequantizeBlockQ4_0F32 / DequantizeBlockQ8_0F32
 * (tensor/internal/cpu/kernels/quantized.go:85-93, :131-136, f16 decode :149-173) and the
 * kernels dequantize_block_q4_0_f32 / dequantize_block_q8_0_f32 (quantized.cu:838-867,
 * :1149-1175). */
cq_status cq_dequantize(cq_ctx *ctx, int qtype, int order, const void *blocks_dev,
                        int64_t nblocks, float *y_dev);

/* f32 x[m,k] (row stride ldx) -> m*k/32 Q8_1 blocks of 36 bytes {f16 d; f16 sum; i8 q[32]}.
 * Replaces quantize_q8_1 (quantized.cu:3521-3558). */
cq_status cq_quantize_q8_1(cq_ctx *ctx, const float *x_dev, int64_t m, int64_t k, int64_t ldx,
                           void *q8_1_dev);

/* ---- the hot path ------------------------------------------------------------------- */
/* y[m,n] = x[m,k] . W[n,k]^T, f32 in / f32 out, row-major with row strides ldx, ldy.
 * This is BackendStorage.MatMul (backend.go:77-78) for a quantized right-hand side, i.e.
 * what nn.Linear.Forward (nn/linear.go:58-112) reaches through MatMulForward
 * (tensor/ops.go:1238-1266) and, on the CPU, NaiveBatchedMatMulStridedF32
 * (tensor/internal/cpu/kernels/conv.go:373-389) after dequantizing.  It also stands in
 * for the reference's unlaunched CUDA entry points dequantize_mul_mat_vec_q4_0_cuda
 * (quantized.cu:1323), mul_mat_vec_q4_0_q8_1_cuda1..8 (quantized.cu:2874-3519) and
 * mul_mat_q4_0 / mul_mat_q8_0 (quantized.cu:4477, :4529).
 * One row runs the streaming decode GEMV; batches in CQ_ACT_F32 / CQ_ACT_Q8_1 run integer dots per quant block on
 * the tensor cores, scaled per block as the mode says (CQ_ACT_F32 batches hold each activation block as 15-bit
 * block fixed point, about 2e-5 of max|y| from the CPU path; CQ_ACT_Q8_1 batches quantize exactly as quantize_q8_1
 * does; up to eight rows against Q4_0 run in a single-launch streaming kernel, larger batches in the int8 GEMM);
 * CQ_ACT_F16 runs the f16 tensor-core GEMMs (up to eight rows against Q4_0: the single-launch streaming kernel with
 * f16 operands, same rounding of the operands).
 * Preconditions: k % 32 == 0, k >= 32, m, n >= 1, ldx >= k, ldy >= n. */
cq_status cq_qmatmul(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_dev,
                     int64_t m, int64_t k, int64_t ldx, const void *w_blocks_dev, int64_t n,
                     float *y_dev, int64_t ldy);

/* nn.Linear.Forward (nn/linear.go:58-112) on the device: y = x . W^T + bias, bias[n] broadcast over the
 * rows (BroadcastAdd, nn/linear.go:105-110); bias_dev may be NULL.  The decode GEMV adds the bias in its
 * epilogue; the other routes add it with a small kernel behind the matmul. */
cq_status cq_qlinear(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_dev, int64_t m, int64_t k, int64_t ldx,
                     const void *w_blocks_dev, int64_t n, const float *bias_dev, float *y_dev, int64_t ldy);

/* Same product with HOST activations and HOST result: copies x up, runs cq_qmatmul, copies
 * y back and waits.  Weights stay resident on the device (they are the layer's state).
 * x_host / y_host should be pinned (cq_malloc_host) for full copy speed.  With at most eight rows and a
 * pinned y_host of up to host_zero_copy bytes (option, default 256 KiB; 0 turns it off) the kernel stores the
 * result into y_host directly and nothing is copied back; the bits are the same either way. */
cq_status cq_qmatmul_host(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_host,
                          int64_t m, int64_t k, const void *w_blocks_dev, int64_t n,
                          float *y_host);

/* Same product as cq_qmatmul(..., CQ_ACT_Q8_1, ...) for m <= 8, for callers that cannot let
 * the library allocate: hosts that gave all device memory to their own arena at start-up, or
 * language runtimes (cgo, JNI) whose GPU glue may not call the CUDA allocator.  It has no
 * counterpart in the reference.  The quantized activations go to a fixed 294,912-byte array
 * that is part of the library image on every GPU (held from load to process exit), so:
 *  - limits: m <= 8 and k <= 32768, beyond which it returns CQ_ERR_TOO_LARGE;
 *  - it never calls cudaMalloc / cudaFree or any allocating routine;
 *  - the first call on each device looks the array's address up (cudaGetSymbolAddress) --
 *    make that first call outside any stream capture;
 *  - all calls on one GPU, from any context or stream, share the array: two calls that may
 *    overlap on the GPU race on it.  Issue them on one stream, or order them yourself.
 *    Every call overwrites the part of the array it reads, so no clearing is ever needed. */
cq_status cq_qmatmul_q8_1_static(cq_ctx *ctx, int qtype, int order, const float *x_dev, int64_t m,
                                 int64_t k, int64_t ldx, const void *w_blocks_dev, int64_t n,
                                 float *y_dev, int64_t ldy);

/* ---- the operators around the linears in a decoder step ---------------------------------
 * f32, row-major, asynchronous on the context's stream.  Each follows candy's CPU kernel of the
 * same name (file:line in tensor/internal/cpu/kernels/). */
/* BackendDevice.RandNormal / RandUniform (device.go:60-66): counter-based, value i depends only
 * on (seed, i).  The reference's CPU device cannot be seeded (cpu/device.go:48-51). */
cq_status cq_rand_normal(cq_ctx *ctx, float *out_dev, int64_t n, float mean, float std, uint64_t seed);
cq_status cq_rand_uniform(cq_ctx *ctx, float *out_dev, int64_t n, float lo, float hi, uint64_t seed);
/* BackendStorage.FastRmsNorm (backend.go:158-159; FastRmsNormF32, reduce.go:3071-3092):
 * y = x / sqrt(mean(x^2) + eps) * alpha over the last dimension; alpha may be NULL. */
cq_status cq_rmsnorm(cq_ctx *ctx, const float *x_dev, const float *alpha_dev, int64_t rows, int64_t cols,
                     float eps, float *y_dev);
/* x += delta (BackendStorage.Add, backend.go:20), then y = rmsnorm(x): the residual add and the
 * norm that follows it in a decoder layer, in one pass. */
cq_status cq_add_rmsnorm(cq_ctx *ctx, float *x_dev, const float *delta_dev, const float *alpha_dev,
                         int64_t rows, int64_t cols, float eps, float *y_dev);
/* BackendStorage.Rope (backend.go:152-153; RopeF32, reduce.go:3987-4006: pairs (i, i + d/2), cos/sin
 * tables [max_ctx, d/2]) applied at position *pos_dev to the q and k heads of
 * qkv[batch, (n_q + 2 n_kv) * head_dim]; the rotated k and the v of every sequence are then
 * stored at that position of the caches [batch][max_ctx][n_kv * head_dim]. */
cq_status cq_rope_store_kv(cq_ctx *ctx, float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads,
                           int head_dim, const float *cos_dev, const float *sin_dev, const int *pos_dev,
                           float *k_cache_dev, float *v_cache_dev, int max_ctx);
/* The rotary step for the prompt: rows t = 0 .. tokens-1 of qkv[tokens, (n_q + 2 n_kv) * head_dim] belong to positions
 * pos0 + t of ONE sequence.  Same arithmetic as cq_rope_store_kv per row; rotated k and plain v go to the f32 caches
 * [max_ctx][n_kv * head_dim] (what the decode entries read afterwards), and 16-bit copies (f16, or bf16 with is_bf16) of
 * rotated q [tokens][n_q * head_dim], rotated k and v [tokens][n_kv * head_dim] are written for cq_flash_attention /
 * run_mha.  pos0 is a host value: positions outside [0, max_ctx) are refused here.  qkv itself is left unrotated. */
cq_status cq_rope_prefill(cq_ctx *ctx, const float *qkv_dev, int64_t tokens, int n_q_heads, int n_kv_heads, int head_dim, const float *cos_dev,
                          const float *sin_dev, int pos0, float *k_cache_dev, float *v_cache_dev, int max_ctx, void *q16_dev, void *k16_dev,
                          void *v16_dev, int is_bf16);
/* f16 / bf16 -> f32, element by element (the attention output back into the f32 residual stream), and f32 -> f16 / bf16,
 * round to nearest even (the cached keys and values of earlier positions, when a prompt continues a sequence). */
cq_status cq_cast_f32_to_16(cq_ctx *ctx, const float *src_dev, int64_t count, int is_bf16, void *dst16_dev);
cq_status cq_cast16_to_f32(cq_ctx *ctx, const void *src16_dev, int64_t count, int is_bf16, float *dst_dev);
/* One query per sequence against keys 0..*pos_dev of its cache: scores q.k / sqrt(head_dim),
 * softmax as FastSoftmaxF32 (reduce.go:2855-2879), weighted sum of v.  Grouped-query heads
 * (n_q_heads a multiple of n_kv_heads), head_dim <= 256.  scratch_dev needs
 * cq_decode_attention_scratch_floats(...) floats.  out[batch, n_q_heads * head_dim]. */
size_t cq_decode_attention_scratch_floats(int64_t batch, int n_q_heads, int head_dim, int max_ctx);
cq_status cq_decode_attention(cq_ctx *ctx, const float *qkv_dev, int64_t batch, int n_q_heads,
                              int n_kv_heads, int head_dim, const int *pos_dev, const float *k_cache_dev,
                              const float *v_cache_dev, int max_ctx, float *scratch_dev, float *out_dev);
/* cq_rope_store_kv followed by cq_decode_attention, with the rotary step done inside the attention
 * kernels: q is rotated as it is loaded, the newest key / value (position *pos) are taken from qkv and
 * stored to the caches by the CTA that consumes them.  qkv is left unrotated unless the shape takes the
 * route without a fused rotary step (then it is rotated in place, as cq_rope_store_kv does). */
cq_status cq_decode_attention_rope(cq_ctx *ctx, float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads, int head_dim,
                                   const float *cos_dev, const float *sin_dev, const int *pos_dev, float *k_cache_dev,
                                   float *v_cache_dev, int max_ctx, float *scratch_dev, float *out_dev);
/* out[r * ld_out + i] = silu(gu[r, i]) * gu[r, n + i]: BackendStorage.Silu (USiluF32,
 * unary.go:3353-3365, evaluated in f64) fused with the Mul of a SwiGLU feed-forward.  ld_out >= n
 * lets the result sit in rows padded for the next linear. */
cq_status cq_silu_mul(cq_ctx *ctx, const float *gate_up_dev, int64_t rows, int64_t n, float *out_dev,
                      int64_t ld_out);
/* The same with gate and up interleaved: out[r, i] = silu(gate_up[r, 2i]) * gate_up[r, 2i+1]. */
cq_status cq_silu_mul_pairs(cq_ctx *ctx, const float *gate_up_dev, int64_t rows, int64_t n, float *out_dev, int64_t ld_out);
/* BackendStorage.FastArgmax (backend.go:128-129; FastArgmaxF32, reduce.go:846-862): the lowest
 * index among equal maxima. */
cq_status cq_argmax(cq_ctx *ctx, const float *x_dev, int64_t rows, int64_t cols, uint32_t *out_dev);
/* Row gather, out[r, :] = table[ids[r], :] (index select; indexing.go:8-26). */
cq_status cq_embedding(cq_ctx *ctx, const float *table_dev, int64_t vocab, int64_t dim,
                       const uint32_t *ids_dev, int64_t rows, float *out_dev);
/* *value_dev += delta on the stream (advances a decode position inside a captured graph). */
cq_status cq_add_int(cq_ctx *ctx, int *value_dev, int delta);

/* One decode linear with its neighbours fused in (m <= 8, f32 activations, shapes the streaming GEMV
 * takes: k % 256 == 0; CQ_ERR_UNSUPPORTED otherwise, and the caller issues the separate operators):
 *   prologue  x' = x + delta (delta nullable); x_out (nullable, must not alias x) receives x';
 *             x'' = x' / sqrt(mean(x'^2) + eps) * alpha when alpha is given (RMSNorm, reduce.go:3071-3092);
 *   linear    t[m,n] = x''[m,k] . W[n,k]^T;
 *   epilogue  0: y[r, c] = t[r, c], n columns; 1: rows of W come in (gate, up) pairs and
 *             y[r, c] = silu(t[r, 2c]) * t[r, 2c+1], n/2 columns (SiLU as unary.go:3353-3365, but expf in
 *             f32: within 2 ulp of the reference's double evaluation).
 * x, delta, x_out have row pitch k; y has row pitch ldy.  No reference counterpart: candy runs
 * these operators one by one. */
cq_status cq_qlinear_fused(cq_ctx *ctx, int qtype, int order, const float *x_dev, const float *delta_dev,
                           const float *alpha_dev, float eps, float *x_out_dev, int64_t m, int64_t k,
                           const void *w_blocks_dev, int64_t n, int epilogue, float *y_dev, int64_t ldy);

/* ---- tensor-parallel exchange fused into the kernels around it ---------------------------
 * One process per GPU.  A row-parallel linear (o / down projection split along k) needs the sum
 * of every rank's partial output.  Instead of a collective call, cq_qmatmul_push makes the decode
 * GEMV store each result directly into every rank's receive buffer (peer stores over NVLink) as
 * an 8-byte (value, tag) pair; cq_add_rmsnorm_reduce, the residual-add + RMSNorm that follows the
 * linear anyway, polls (bounded; CQ_ERR_TIMEOUT at the next cq_synchronize on give-up) its own
 * memory until every pair carries this exchange's tag, sums the partials in rank order
 * (bit-identical on every rank), adds the sum to x, and advances the tag (kept on the device, so a
 * captured graph replays).  Use set 0 and set 1 alternately (o: 0, down: 1).  Every rank must
 * issue the same sequence of calls.  The reference has no multi-device code; no counterpart.
 *   create:  allocates this rank's buffers; handle64 receives a 64-byte CUDA IPC handle;
 *   connect: takes all ranks' handles (world x 64 bytes, rank order) gathered by the host.  With
 *            all_handles = NULL the communicator is a single-process stand-in: every "peer" is this rank's
 *            own buffer, so pushes land only in this rank's slot and the other ranks' data never arrives
 *            (how a missing peer looks; used to exercise the bounded wait on one GPU).
 * A push into a set that still holds an unconsumed push is refused (CQ_ERR_INVALID_ARG). */
typedef struct cq_comm cq_comm;
cq_status cq_comm_create(cq_ctx *ctx, int rank, int world, int64_t max_floats, cq_comm **out, void *handle64);
cq_status cq_comm_connect(cq_ctx *ctx, cq_comm *comm, const void *all_handles);
cq_status cq_comm_destroy(cq_ctx *ctx, cq_comm *comm);
/* partial[m,n] = x[m,k] . W[n,k]^T (f32 activations, m <= 8), pushed into slot `rank` of `set` on
 * every rank instead of being written locally.  m*n <= max_floats. */
cq_status cq_qmatmul_push(cq_ctx *ctx, cq_comm *comm, int set, int qtype, int order, const float *x_dev,
                          int64_t m, int64_t k, int64_t ldx, const void *w_blocks_dev, int64_t n);
/* x[rows,cols] += sum over ranks of the partials pushed into `set`; y = rmsnorm(x) * alpha. */
cq_status cq_add_rmsnorm_reduce(cq_ctx *ctx, cq_comm *comm, int set, float *x_dev, const float *alpha_dev,
                                int64_t rows, int64_t cols, float eps, float *y_dev);

/* ---- a whole decode step as one persistent kernel (batch 1) --------------------------------------------
 * Embedding row -> per layer [residual + RMSNorm -> QKV linear -> rotary step, KV-cache write, attention ->
 * o linear -> residual + RMSNorm -> gate/up linear with SiLU(gate)*up -> down linear] -> final norm -> output
 * linear -> arg-max, in ONE cooperative launch: every SM keeps one CTA for the whole step, a producer warp
 * streams the weight rows of all linears through one shared-memory ring without stopping at phase boundaries,
 * and the phases are separated by bounded grid-wide barriers (a wait that gives up -> CQ_ERR_TIMEOUT at
 * cq_synchronize; the decoder must then be destroyed).  Numerics of each phase are those of the separate entry
 * points (cq_qlinear_fused, cq_decode_attention_rope, cq_argmax).  No counterpart in the reference.
 * The description's pointer arrays are host arrays of n_layers device pointers, read at create time only.
 *   wqkv[l]  [(n_heads + 2 n_kv_heads) * 128, dim] blocks (q heads, then k heads, then v heads)
 *   wo[l]    [dim, n_heads * 128]      wgu[l] [2 * ffn, dim], gate and up rows interleaved (g0, u0, g1, u1, ...)
 *   wdown[l] [dim, ffn_pad], ffn_pad = ffn rounded up to 256 (padding columns multiply zeros)
 *   k_cache[l], v_cache[l] f32 [max_ctx][n_kv_heads * 128]; cos / sin tables [max_ctx][64]; embed f32 [vocab][dim]
 * Built for head_dim 128, Q4_0 / Q8_0, dim and n_heads * 128 multiples of 256, batch 1.
 * cq_decoder_step consumes *ids_dev (the token to feed) at position *pos_dev and leaves the arg-max token in
 * *ids_dev and the position advanced, so repeated launches (or one captured launch replayed) decode greedily;
 * cq_decoder_logits is the step's logits row (f32 [vocab], device memory owned by the decoder). */
typedef struct cq_decoder cq_decoder;
typedef struct cq_decoder_desc {
    int n_layers, dim, n_heads, n_kv_heads, head_dim, ffn, ffn_pad, vocab, max_ctx;
    float eps;
    int qtype, order;
    const void *const *wqkv, *const *wo, *const *wgu, *const *wdown;
    const float *const *attn_norm, *const *ffn_norm;
    float *const *k_cache, *const *v_cache;
    const float *embed;
    const void *wout;
    const float *final_norm, *cos_table, *sin_table;
} cq_decoder_desc;
cq_status cq_decoder_create(cq_ctx *ctx, const cq_decoder_desc *desc, cq_decoder **out);
cq_status cq_decoder_step(cq_ctx *ctx, cq_decoder *dec, uint32_t *ids_dev, int *pos_dev);
const float *cq_decoder_logits(const cq_decoder *dec);
cq_status cq_decoder_destroy(cq_ctx *ctx, cq_decoder *dec);

/* ---- prefill attention: the FlashAttention binding's replacement ------------------------------------
 * O = softmax(Q K^T * softmax_scale) V per (batch, head) on the sm_100a tensor cores (tcgen05, tensor
 * memory, TMA).  Arguments, their order and meaning are those of run_mha in the reference
 * (llm/internal/flashattn/flash_api.h:71-117; flashattn.go:145-205 is its caller): 16-bit tensors
 * [batch][row][head][d] addressed through batch / row / head strides in ELEMENTS, h a multiple of h_k
 * (grouped-query heads), is_bf16 0 = f16 / 1 = bf16, is_causal with the mask aligned to the bottom right
 * (key j visible to row i iff j <= i + seqlen_k - seqlen_q, kernels/mask.h:61-62), softmax_lse (nullable)
 * [batch][h][seqlen_q] f32 = max * scale + log(sum) (kernels/softmax.h:206).  Built: head dimensions 64 and
 * 128, strides that are multiples of 8 elements.  Not built (CQ_ERR_UNSUPPORTED): other head dimensions,
 * ALiBi, cu_seqlens (variable-length batches), sliding windows, soft-capping, the unpadded LSE layout.
 * V is read in place when it is 16-byte aligned with strides that are multiples of 8 elements; any other V is
 * transposed into context scratch first (then cq_reserve(b * h_k * d * roundup(seqlen_k, 8) * 2) up front when
 * capturing).  cq_flash_attention returns a status and runs on the context's stream; run_mha is the
 * reference's own symbol and signature (void, default stream), for hosts that already bind it, with
 * cq_run_mha_last_status() to read the outcome. */
cq_status cq_flash_attention(cq_ctx *ctx, void *q_ptr, void *k_ptr, void *v_ptr, void *o_ptr, void *softmax_lse_ptr, void *alibi_slopes_ptr,
                             int32_t *cu_seqlens_q_ptr, int32_t *cu_seqlens_k_ptr, uint32_t q_batch_stride, uint32_t k_batch_stride,
                             uint32_t v_batch_stride, uint32_t o_batch_stride, uint32_t alibi_slopes_batch_stride, uint32_t q_row_stride,
                             uint32_t k_row_stride, uint32_t v_row_stride, uint32_t o_row_stride, uint32_t q_head_stride, uint32_t k_head_stride,
                             uint32_t v_head_stride, uint32_t o_head_stride, uint32_t b, uint32_t h, uint32_t h_k, uint32_t d, uint32_t d_rounded,
                             float softmax_scale, uint32_t seqlen_q, uint32_t seqlen_k, uint32_t seqlen_q_rounded, uint32_t seqlen_k_rounded,
                             int is_bf16, int is_causal, int unpadded_lse, int window_size_left, int window_size_right, float softcap);
void run_mha(void *q_ptr, void *k_ptr, void *v_ptr, void *o_ptr, void *softmax_lse_ptr, void *alibi_slopes_ptr, int32_t *cu_seqlens_q_ptr,
             int32_t *cu_seqlens_k_ptr, uint32_t q_batch_stride, uint32_t k_batch_stride, uint32_t v_batch_stride, uint32_t o_batch_stride,
             uint32_t alibi_slopes_batch_stride, uint32_t q_row_stride, uint32_t k_row_stride, uint32_t v_row_stride, uint32_t o_row_stride,
             uint32_t q_head_stride, uint32_t k_head_stride, uint32_t v_head_stride, uint32_t o_head_stride, uint32_t b, uint32_t h, uint32_t h_k,
             uint32_t d, uint32_t d_rounded, float softmax_scale, uint32_t seqlen_q, uint32_t seqlen_k, uint32_t seqlen_q_rounded,
             uint32_t seqlen_k_rounded, int is_bf16, int is_causal, int unpadded_lse, int window_size_left, int window_size_right, float softcap);
cq_status cq_run_mha_last_status(void);

/* ---- NCCL all-reduce: the baseline exchange, and the one for batches beyond eight rows ---------
 * No counterpart in the reference.  NCCL is opened at run time (libnccl.so.2; $CANDYQ_NCCL_LIBRARY
 * overrides), not linked: without it these entries answer CQ_ERR_UNSUPPORTED and everything else works.
 *   cq_tp_unique_id       rank 0 makes the 128-byte id and hands it to the other ranks by any means it has;
 *   cq_tp_init            every rank joins (collective: returns when all `world` ranks have called it);
 *   cq_allreduce_sum_f32  buf[count] = sum over ranks, in place, asynchronous on the context's stream
 *                         (may be recorded into a graph between cq_capture_begin / _end);
 *   cq_tp_wait            waits for the stream, at most timeout_ms: if the work has not finished by then (a
 *                         rank is late or gone) or NCCL reports an asynchronous error, the communicator is
 *                         aborted -- which releases the collective kernels still waiting on the GPU -- and
 *                         CQ_ERR_TIMEOUT (or CQ_ERR_CUDA) comes back; the context stays usable, the
 *                         communicator does not.  Use it instead of cq_synchronize wherever a peer may fail. */
typedef struct cq_tp cq_tp;
cq_status cq_tp_unique_id(cq_ctx *ctx, void *id128);
cq_status cq_tp_init(cq_ctx *ctx, int rank, int world, const void *nccl_unique_id, size_t id_bytes, cq_tp **out);
cq_status cq_tp_destroy(cq_ctx *ctx, cq_tp *tp);
cq_status cq_allreduce_sum_f32(cq_ctx *ctx, cq_tp *tp, float *buf_dev, int64_t count);
cq_status cq_tp_wait(cq_ctx *ctx, cq_tp *tp, int timeout_ms);

/* ---- CUDA graphs and device timing ----------------------------------------------------
 * Decode loops are launch-bound: a GEMV lasts a few microseconds.  These wrap stream capture
 * so a host in any language can record a sequence of cq_* launches once and replay it.
 * The reference has no counterpart (its CUDA backend never launches anything).
 * Between begin and end only asynchronous entry points may be called on this context
 * (no cq_memcpy_h2d/d2h, cq_synchronize, cq_qmatmul_host, nor a first call that has to grow
 * the context's scratch memory). */
typedef struct cq_graph cq_graph;
cq_status cq_capture_begin(cq_ctx *ctx);
cq_status cq_capture_end(cq_ctx *ctx, cq_graph **out);
cq_status cq_graph_launch(cq_ctx *ctx, cq_graph *g);
cq_status cq_graph_destroy(cq_ctx *ctx, cq_graph *g);
/* Measures the int8 tensor-pipe ceiling on this GPU: every SM issues `iters` x 4 back-to-back
 * tcgen05.mma kind::i8 (s8 x s8 -> s32, M 128, N 256, K 32) on operands resident in shared memory, no
 * global traffic and no epilogue.  *tera_ops receives 10^12 integer operations per second (2 per
 * multiply-add).  A plain GEMM can only reach less; it is the denominator for the int8 prefill figures. */
cq_status cq_measure_i8_mma_peak(cq_ctx *ctx, int iters, double *tera_ops);
/* CUDA-event stopwatch on the context's stream: stop waits for the stream and returns the
 * device time in milliseconds between the two marks. */
cq_status cq_timer_start(cq_ctx *ctx);
cq_status cq_timer_stop(cq_ctx *ctx, float *ms);

#ifdef __cplusplus
}
#endif
#endif /* CANDYQ_H */
