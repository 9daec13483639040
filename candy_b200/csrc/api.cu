// libcandyq: context, memory and dispatch entry points of the C ABI (include/candyq.h).
#include <cstring>

#include "common.cuh"

cq_status cq_fail(cq_ctx *ctx, cq_status s, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return s;
}

cq_status cq_cuda_fail(cq_ctx *ctx, cudaError_t e, const char *what) {
    std::string msg = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return cq_fail(ctx, e == cudaErrorMemoryAllocation ? CQ_ERR_NOMEM : CQ_ERR_CUDA, msg);
}

cq_status cq_reserve_scratch(cq_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return CQ_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (ctx->capturing || (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone))
        return cq_fail(ctx, CQ_ERR_INVALID_ARG,
                       "this call needs " + std::to_string(bytes) + " bytes of context scratch but only " + std::to_string(ctx->scratch_bytes) +
                           " are reserved, and scratch cannot grow during stream capture: call cq_reserve first, or run the call once before capturing");
    if (ctx->scratch) {
        CQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->graphs_alive > 0) ctx->retired_scratch.push_back(ctx->scratch);  // graphs may still point into it
        else CQ_CUDA(ctx, cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
    }
    size_t want = (bytes + 0xFFFFF) & ~size_t(0xFFFFF);
    CQ_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return CQ_OK;
}

void cq_w16_invalidate(cq_ctx *ctx, const void *begin, size_t bytes) {
    if (ctx->w16_cache.empty() || !begin || bytes == 0) return;
    const uintptr_t lo = reinterpret_cast<uintptr_t>(begin), hi = lo + bytes;
    bool synced = false;
    for (auto it = ctx->w16_cache.begin(); it != ctx->w16_cache.end();) {
        const uintptr_t w = reinterpret_cast<uintptr_t>(std::get<0>(it->first));
        if (w >= lo && w < hi) {
            if (!synced) cudaStreamSynchronize(ctx->stream), synced = true;  // a GEMM still reading the copy finishes first
            cudaFree(it->second);
            ctx->w16_cache_bytes -= (size_t)std::get<1>(it->first) * (size_t)std::get<2>(it->first) * 2;
            it = ctx->w16_cache.erase(it);
        } else {
            ++it;
        }
    }
}

extern "C" {

const char *cq_status_string(cq_status s) {
    switch (s) {
        case CQ_OK: return "ok";
        case CQ_ERR_INVALID_ARG: return "invalid argument";
        case CQ_ERR_CUDA: return "CUDA runtime error";
        case CQ_ERR_UNSUPPORTED: return "unsupported configuration";
        case CQ_ERR_TIMEOUT: return "device-side wait timed out";
        case CQ_ERR_NOMEM: return "out of memory";
        case CQ_ERR_TOO_LARGE: return "size beyond the entry point's fixed limit";
        default: return "unknown status";
    }
}

const char *cq_last_error(const cq_ctx *ctx) { return ctx ? ctx->last_error.c_str() : ""; }

const char *cq_version(void) { return "candyq 0.1 sm_100a"; }

cq_status cq_device_count(int *count) {
    if (!count) return CQ_ERR_INVALID_ARG;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return CQ_ERR_CUDA;
    }
    *count = n;
    return CQ_OK;
}

cq_status cq_ctx_create(int device, cq_ctx **out) {
    if (!out) return CQ_ERR_INVALID_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return CQ_ERR_CUDA;  // no GPU: there is no CPU fallback
    }
    if (device < 0 || device >= n) return CQ_ERR_INVALID_ARG;
    if (cudaSetDevice(device) != cudaSuccess) return CQ_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return CQ_ERR_CUDA;
    if (prop.major != 10) return CQ_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
    cq_ctx *ctx = new cq_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return CQ_ERR_CUDA;
    }
    ctx->stream = ctx->own_stream;
    if (cudaHostAlloc((void **)&ctx->dev_err, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void **)&ctx->dev_err_devptr, ctx->dev_err, 0) != cudaSuccess) {
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return CQ_ERR_CUDA;
    }
    *ctx->dev_err = 0;
    *out = ctx;
    return CQ_OK;
}

cq_status cq_ctx_destroy(cq_ctx *ctx) {
    if (!ctx) return CQ_ERR_INVALID_ARG;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (void *p : ctx->retired_scratch) cudaFree(p);
    for (auto &kv : ctx->w16_cache) cudaFree(kv.second);
    if (ctx->xfer_x) cudaFree(ctx->xfer_x);
    if (ctx->xfer_y) cudaFree(ctx->xfer_y);
    if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
    if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
    if (ctx->dev_err) cudaFreeHost(ctx->dev_err);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return CQ_OK;
}

cq_status cq_ctx_set_stream(cq_ctx *ctx, void *cuda_stream) {
    if (!ctx) return CQ_ERR_INVALID_ARG;
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
    return CQ_OK;
}

cq_status cq_ctx_set_option(cq_ctx *ctx, const char *key, int64_t value) {
    if (!ctx || !key) return CQ_ERR_INVALID_ARG;
    GemvTuning &t = ctx->tune;
    if (!strcmp(key, "gemv_warps")) t.target_warps = (int)value;
    else if (!strcmp(key, "gemv_stages")) t.stages = (int)value;
    else if (!strcmp(key, "gemv_ctas_per_sm")) t.ctas_per_sm = (int)value;
    else if (!strcmp(key, "host_zero_copy")) t.host_zero_copy = value < 0 ? 0 : value;
    else if (!strcmp(key, "gemm_pair")) t.gemm_pair = value ? 1 : 0;
    else if (!strcmp(key, "gemm_fused_dequant")) t.gemm_fused_dequant = value < 0 ? 0 : (value > 2 ? 2 : (int)value);
    else if (!strcmp(key, "gemv_early")) t.early = value ? 1 : 0;
    else if (!strcmp(key, "gemv_force_simple")) t.force_simple = (int)value;
    else if (!strcmp(key, "gemv_pdl")) t.pdl = (int)value;
    else if (!strcmp(key, "gemm_variant")) t.gemm_variant = (int)value;
    else if (!strcmp(key, "attn_variant")) t.attn_variant = (int)value;
    else if (!strcmp(key, "gemm_cache_weights")) t.gemm_cache_weights = (int)value;
    else if (!strcmp(key, "gemv_variant")) t.gemv_variant = (int)value;
    else if (!strcmp(key, "comm_poll_limit")) t.comm_poll_limit = (int)value;
    else if (!strcmp(key, "comm_cluster")) t.comm_cluster = (int)value;
    else if (!strcmp(key, "gemm_int8")) t.gemm_int8 = (int)value;
    else if (!strcmp(key, "i8_min_rows_f32")) t.i8_min_rows_f32 = (int)value;
    else if (!strcmp(key, "i8_min_rows_q8_1")) t.i8_min_rows_q8_1 = (int)value;
    else if (!strcmp(key, "gemv_mma")) t.gemv_mma = (int)value;
    else if (!strcmp(key, "fa_transpose_v")) t.fa_transpose_v = (int)value;
    else if (!strcmp(key, "gemv_chain")) t.gemv_chain = value ? 1 : 0;
    else if (!strcmp(key, "gemv_independent")) t.gemv_independent = value ? 1 : 0;
    else if (!strcmp(key, "gemv_q81_inline")) t.gemv_q81_inline = (int)value;
    else if (!strcmp(key, "gemv_multirow")) t.gemv_multirow = (int)value;
    else if (!strcmp(key, "gemv_coop")) t.gemv_coop = (int)value;
    else if (!strcmp(key, "gemv_rpt")) t.gemv_rpt = (int)value;
    else return cq_fail(ctx, CQ_ERR_INVALID_ARG, std::string("unknown option ") + key);
    return CQ_OK;
}

cq_status cq_reserve(cq_ctx *ctx, size_t bytes) {
    CQ_ENTER(ctx);
    return cq_reserve_scratch(ctx, bytes);
}

cq_status cq_malloc(cq_ctx *ctx, size_t bytes, void **dptr) {
    CQ_ENTER(ctx);
    if (!dptr) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_malloc: null out pointer");
    *dptr = nullptr;
    if (bytes == 0) return CQ_OK;
    CQ_CUDA(ctx, cudaMalloc(dptr, bytes));
    ctx->allocs[*dptr] = bytes;
    return CQ_OK;
}

cq_status cq_free(cq_ctx *ctx, void *dptr) {
    CQ_ENTER(ctx);
    if (!dptr) return CQ_OK;
    // cached f16 copies of weights that lived anywhere in this allocation die with it
    auto a = ctx->allocs.find(dptr);
    cq_w16_invalidate(ctx, dptr, a != ctx->allocs.end() ? a->second : 1);
    if (a != ctx->allocs.end()) ctx->allocs.erase(a);
    CQ_CUDA(ctx, cudaFree(dptr));
    return CQ_OK;
}

cq_status cq_invalidate_weight_cache(cq_ctx *ctx, const void *blocks_dev, size_t bytes) {
    CQ_ENTER(ctx);
    cq_w16_invalidate(ctx, blocks_dev, bytes);
    return CQ_OK;
}

cq_status cq_malloc_host(cq_ctx *ctx, size_t bytes, void **hptr) {
    CQ_ENTER(ctx);
    if (!hptr) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_malloc_host: null out pointer");
    *hptr = nullptr;
    if (bytes == 0) return CQ_OK;
    CQ_CUDA(ctx, cudaHostAlloc(hptr, bytes, cudaHostAllocDefault));
    return CQ_OK;
}

cq_status cq_free_host(cq_ctx *ctx, void *hptr) {
    CQ_ENTER(ctx);
    if (!hptr) return CQ_OK;
    CQ_CUDA(ctx, cudaFreeHost(hptr));
    return CQ_OK;
}

cq_status cq_memset(cq_ctx *ctx, void *dptr, int byte, size_t bytes) {
    CQ_ENTER(ctx);
    if (!dptr && bytes) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_memset: null pointer");
    cq_w16_invalidate(ctx, dptr, bytes);
    CQ_CUDA(ctx, cudaMemsetAsync(dptr, byte, bytes, ctx->stream));
    return CQ_OK;
}

cq_status cq_memcpy_h2d(cq_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    CQ_ENTER(ctx);
    if ((!dst_dev || !src_host) && bytes) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_memcpy_h2d: null pointer");
    cq_w16_invalidate(ctx, dst_dev, bytes);
    CQ_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    CQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CQ_OK;
}

cq_status cq_memcpy_d2h(cq_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes) {
    CQ_ENTER(ctx);
    if ((!dst_host || !src_dev) && bytes) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_memcpy_d2h: null pointer");
    CQ_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    CQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CQ_OK;
}

cq_status cq_memcpy_d2d(cq_ctx *ctx, void *dst_dev, const void *src_dev, size_t bytes) {
    CQ_ENTER(ctx);
    if ((!dst_dev || !src_dev) && bytes) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_memcpy_d2d: null pointer");
    cq_w16_invalidate(ctx, dst_dev, bytes);
    CQ_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return CQ_OK;
}

cq_status cq_synchronize(cq_ctx *ctx) {
    CQ_ENTER(ctx);
    CQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int e = *(volatile int *)ctx->dev_err;
    if (e != 0) {
        *ctx->dev_err = 0;
        if (e == kDevErrPosition)
            return cq_fail(ctx, CQ_ERR_INVALID_ARG, "a decode kernel found its device-resident position outside [0, max_ctx): it was clamped, the step's results are invalid");
        return cq_fail(ctx, CQ_ERR_TIMEOUT, "a kernel's bounded wait gave up (device error word " + std::to_string(e) + ")");
    }
    return CQ_OK;
}

size_t cq_blocks_bytes(int qtype, int64_t n, int64_t k) {
    if (n <= 0 || k <= 0 || k % kQK != 0) return 0;
    if (cq_is_k_format(qtype)) return k % 256 == 0 ? (size_t)n * (size_t)(k / 256) * (size_t)cq_k_block_bytes(qtype) : 0;
    if (qtype == CQ_Q4_0) return (size_t)n * (size_t)(k / kQK) * kQ4Bytes;
    if (qtype == CQ_Q8_0) return (size_t)n * (size_t)(k / kQK) * kQ8Bytes;
    if (cq_is_more_format(qtype)) return (size_t)n * (size_t)(k / kQK) * (size_t)cq_more_block_bytes(qtype);
    return 0;
}

static cq_status check_qtype_order(cq_ctx *ctx, int qtype, int order) {
    if (qtype != CQ_Q4_0 && qtype != CQ_Q8_0 && !cq_is_more_format(qtype) && !cq_is_k_format(qtype))
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "qtype must be CQ_Q4_0, CQ_Q4_1, CQ_Q5_0, CQ_Q5_1, CQ_Q8_0 or CQ_Q2_K .. CQ_Q6_K");
    if (order != CQ_ORDER_GO_INTERLEAVED && order != CQ_ORDER_GGML_SPLIT)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "order must be 0 (interleaved) or 1 (split)");
    if (cq_is_more_format(qtype) && !cq_more_order_ok(qtype, order))
        return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "Q5_0 / Q5_1 exist in the split order only");
    if (cq_is_k_format(qtype) && order != CQ_ORDER_GGML_SPLIT)
        return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "the K formats have one element order, the reference CUDA kernels': pass CQ_ORDER_GGML_SPLIT");
    return CQ_OK;
}

cq_status cq_quantize_rows(cq_ctx *ctx, int qtype, int order, const float *w_dev, int64_t n, int64_t k,
                           void *blocks_dev) {
    CQ_ENTER(ctx);
    cq_status s = check_qtype_order(ctx, qtype, order);
    if (s != CQ_OK) return s;
    if (!w_dev || !blocks_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_quantize_rows: null pointer");
    if (cq_is_k_format(qtype)) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_quantize_rows: the reference has no quantizer for the K formats and neither has this library; load such weights from a file");
    if (n < 1 || k < kQK || k % kQK != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_quantize_rows: need n >= 1, k >= 32, k % 32 == 0");
    cq_w16_invalidate(ctx, blocks_dev, cq_blocks_bytes(qtype, n, k));
    if (cq_is_more_format(qtype)) return launch_quantize_rows_more(ctx, qtype, order, w_dev, n * (k / kQK), blocks_dev);
    return launch_quantize_rows(ctx, qtype, order, w_dev, n * (k / kQK), blocks_dev);
}

cq_status cq_dequantize(cq_ctx *ctx, int qtype, int order, const void *blocks_dev, int64_t nblocks, float *y_dev) {
    CQ_ENTER(ctx);
    cq_status s = check_qtype_order(ctx, qtype, order);
    if (s != CQ_OK) return s;
    if (nblocks == 0) return CQ_OK;
    if (!blocks_dev || !y_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_dequantize: null pointer");
    if (nblocks < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_dequantize: negative block count");
    if (cq_is_k_format(qtype)) return launch_dequantize_k(ctx, qtype, blocks_dev, nblocks, y_dev);
    if (cq_is_more_format(qtype)) return launch_dequantize_more(ctx, qtype, order, blocks_dev, nblocks, y_dev);
    return launch_dequantize(ctx, qtype, order, blocks_dev, nblocks, y_dev);
}

cq_status cq_quantize_q8_1(cq_ctx *ctx, const float *x_dev, int64_t m, int64_t k, int64_t ldx, void *q8_1_dev) {
    CQ_ENTER(ctx);
    if (!x_dev || !q8_1_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_quantize_q8_1: null pointer");
    if (m < 1 || k < kQK || k % kQK != 0 || ldx < k)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_quantize_q8_1: need m >= 1, k >= 32, k % 32 == 0, ldx >= k");
    return launch_quantize_q8_1(ctx, x_dev, m, k, ldx, q8_1_dev);
}

static cq_status check_matmul_args(cq_ctx *ctx, int qtype, int order, int actmode, const void *x, int64_t m, int64_t k,
                                   int64_t ldx, const void *w, int64_t n, const void *y, int64_t ldy) {
    cq_status s = check_qtype_order(ctx, qtype, order);
    if (s != CQ_OK) return s;
    if (actmode != CQ_ACT_F32 && actmode != CQ_ACT_Q8_1 && actmode != CQ_ACT_F16)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "actmode must be CQ_ACT_F32, CQ_ACT_Q8_1 or CQ_ACT_F16");
    if (!x || !w || !y) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: null pointer");
    if (m < 1 || n < 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: m and n must be >= 1");
    if (k < kQK || k % kQK != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: k must be a positive multiple of 32");
    if (cq_is_k_format(qtype) && k % 256 != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: the K formats need k to be a multiple of 256");
    if (ldx < k) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: ldx < k");
    if (ldy < n) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul: ldy < n");
    if (m > (int64_t(1) << 24) || n > (int64_t(1) << 28) || k > (int64_t(1) << 24))
        return cq_fail(ctx, CQ_ERR_TOO_LARGE, "cq_qmatmul: dimension beyond 2^24 (m, k) / 2^28 (n)");
    return CQ_OK;
}

cq_status cq_qmatmul(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_dev, int64_t m, int64_t k,
                     int64_t ldx, const void *w_blocks_dev, int64_t n, float *y_dev, int64_t ldy) {
    CQ_ENTER(ctx);
    cq_status s = check_matmul_args(ctx, qtype, order, actmode, x_dev, m, k, ldx, w_blocks_dev, n, y_dev, ldy);
    if (s != CQ_OK) return s;
    // Two to eight rows against Q4_0 in CQ_ACT_F32 or CQ_ACT_Q8_1: the streaming kernel with tensor-core block dots, one launch
    // (two rows only against large weights, or in CQ_ACT_Q8_1 long rows: elsewhere the two-row form of the one-row kernel is quicker)
    if (actmode != CQ_ACT_F16 && ctx->tune.gemv_mma > 0 && (m >= ctx->tune.gemv_mma || (m == 2 && (actmode == CQ_ACT_Q8_1 ? (k >= 8192 || n * k >= (int64_t(100) << 20)) : n * k >= (int64_t(40) << 20)))) && m <= 8 &&
        !ctx->fuse.on && ctx->push.world == 0 && ctx->tune.gemv_variant == 0 && !ctx->tune.force_simple &&
        gemv_mma_supported(ctx, qtype, m, k, n, w_blocks_dev, x_dev, ldx)) {
        s = launch_gemv_mma(ctx, order, actmode == CQ_ACT_Q8_1, x_dev, m, k, ldx, w_blocks_dev, n, ctx->bias, y_dev, ldy);
        if (s == CQ_OK && ctx->bias) ctx->bias_done = true;
        return s;
    }
    // Up to eight rows of CQ_ACT_F16 against Q4_0: the same streaming kernel with f16 operands, one launch.
    if (actmode == CQ_ACT_F16 && ctx->tune.gemv_mma > 0 && m <= 8 && !ctx->fuse.on && ctx->push.world == 0 &&
        gemv_mma_f16_supported(ctx, qtype, m, k, n, w_blocks_dev, x_dev, ldx)) {
        s = launch_gemv_mma_f16(ctx, order, x_dev, m, k, ldx, w_blocks_dev, n, ctx->bias, y_dev, ldy);
        if (s == CQ_OK && ctx->bias) ctx->bias_done = true;
        return s;
    }
    // Integer dots on the tensor cores: one weight pass for the whole batch, in the activation mode's own numerics.
    if (actmode != CQ_ACT_F16 && ctx->tune.gemm_int8 && !ctx->fuse.on && ctx->push.world == 0 && ctx->tune.gemv_variant == 0 &&
        m >= (actmode == CQ_ACT_Q8_1 ? ctx->tune.i8_min_rows_q8_1 : ctx->tune.i8_min_rows_f32) &&
        qgemm_i8_supported(qtype, k, w_blocks_dev, x_dev, ldx))
        return launch_qgemm_i8(ctx, qtype, order, actmode == CQ_ACT_Q8_1 ? 1 : 0, x_dev, m, k, ldx, w_blocks_dev, n, y_dev, ldy);
    if (m <= 8 && actmode != CQ_ACT_F16) return launch_gemv(ctx, qtype, order, actmode, x_dev, m, k, ldx, w_blocks_dev, n, y_dev, ldy);
    return launch_gemm(ctx, qtype, order, actmode, x_dev, m, k, ldx, w_blocks_dev, n, y_dev, ldy);
}

// y[r, c] += bias[c] for the routes whose kernels have no bias epilogue (plain GEMV, tensor-core GEMMs).
__global__ void __launch_bounds__(256) add_bias_kernel(float *__restrict__ y, const float *__restrict__ bias, int64_t rows, int64_t n, int64_t ldy) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n, c = i - r * n;
        y[r * ldy + c] += bias[c];
    }
}

cq_status cq_qlinear(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_dev, int64_t m, int64_t k, int64_t ldx,
                     const void *w_blocks_dev, int64_t n, const float *bias_dev, float *y_dev, int64_t ldy) {
    CQ_ENTER(ctx);
    ctx->bias = bias_dev;
    ctx->bias_done = false;
    cq_status s = cq_qmatmul(ctx, qtype, order, actmode, x_dev, m, k, ldx, w_blocks_dev, n, y_dev, ldy);
    const bool done = ctx->bias_done;
    ctx->bias = nullptr;
    ctx->bias_done = false;
    if (s != CQ_OK || !bias_dev || done) return s;
    const int64_t total = m * n;
    const unsigned cap = (unsigned)ctx->sm_count * 8;
    const unsigned grid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
    add_bias_kernel<<<grid, 256, 0, ctx->stream>>>(y_dev, bias_dev, m, n, ldy);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status cq_qlinear_fused(cq_ctx *ctx, int qtype, int order, const float *x_dev, const float *delta_dev, const float *alpha_dev, float eps,
                           float *x_out_dev, int64_t m, int64_t k, const void *w_blocks_dev, int64_t n, int epilogue, float *y_dev,
                           int64_t ldy) {
    CQ_ENTER(ctx);
    const int64_t n_out = epilogue == 1 ? n / 2 : n;
    const int64_t ldy_chk = ldy >= n_out ? (ldy < n ? n : ldy) : -1;  // the shared check wants ldy >= n; here n_out columns are written
    cq_status s = check_matmul_args(ctx, qtype, order, CQ_ACT_F32, x_dev, m, k, k, w_blocks_dev, n, y_dev, ldy_chk);
    if (s != CQ_OK) return s;
    if (m > 8) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qlinear_fused: m must be 1..8 (the decode path)");
    if (epilogue != 0 && epilogue != 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qlinear_fused: epilogue must be 0 or 1");
    if (epilogue == 1 && (n & 1)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qlinear_fused: the pairing epilogue needs an even n");
    if (x_out_dev && x_out_dev == x_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qlinear_fused: x_out must not alias x (other CTAs still read x)");
    for (const void *q : {(const void *)x_dev, (const void *)delta_dev, (const void *)alpha_dev, (const void *)x_out_dev})
        if (reinterpret_cast<uintptr_t>(q) & 15) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qlinear_fused: x, delta, alpha, x_out must be 16-byte aligned");
    FuseSpec f;
    f.on = true, f.delta = delta_dev, f.alpha = alpha_dev, f.x_out = x_out_dev, f.eps = eps, f.norm = alpha_dev != nullptr, f.epilogue = epilogue;
    f.ld_delta = k, f.ld_xout = k;
    ctx->fuse = f;
    s = launch_gemv(ctx, qtype, order, CQ_ACT_F32, x_dev, m, k, k, w_blocks_dev, n, y_dev, ldy);
    ctx->fuse = FuseSpec();
    return s;
}

cq_status cq_qmatmul_host(cq_ctx *ctx, int qtype, int order, int actmode, const float *x_host, int64_t m, int64_t k,
                          const void *w_blocks_dev, int64_t n, float *y_host) {
    CQ_ENTER(ctx);
    cq_status s = check_matmul_args(ctx, qtype, order, actmode, x_host, m, k, k, w_blocks_dev, n, y_host, n);
    if (s != CQ_OK) return s;
    size_t xb = (size_t)m * k * sizeof(float), yb = (size_t)m * n * sizeof(float);
    if (xb > ctx->xfer_x_bytes) {
        if (ctx->xfer_x) CQ_CUDA(ctx, cudaFree(ctx->xfer_x));
        ctx->xfer_x = nullptr, ctx->xfer_x_bytes = 0;
        CQ_CUDA(ctx, cudaMalloc(&ctx->xfer_x, xb));
        ctx->xfer_x_bytes = xb;
    }
    if (yb > ctx->xfer_y_bytes) {
        if (ctx->xfer_y) CQ_CUDA(ctx, cudaFree(ctx->xfer_y));
        ctx->xfer_y = nullptr, ctx->xfer_y_bytes = 0;
        CQ_CUDA(ctx, cudaMalloc(&ctx->xfer_y, yb));
        ctx->xfer_y_bytes = yb;
    }
    CQ_CUDA(ctx, cudaMemcpyAsync(ctx->xfer_x, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    // A result buffer in pinned host memory is written by the kernel itself (it is addressable from the device):
    // no copy out, one submission less.  Only for the row-streaming kernels (m <= 8), which store every result
    // once and coalesced, and only for small results: the stores cross PCIe.
    float *y_direct = nullptr;
    if (m <= 8 && ctx->tune.host_zero_copy > 0 && yb <= (size_t)ctx->tune.host_zero_copy) {
        cudaPointerAttributes pa;
        if (cudaPointerGetAttributes(&pa, y_host) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer)
            y_direct = static_cast<float *>(pa.devicePointer);
        else
            cudaGetLastError();
    }
    s = cq_qmatmul(ctx, qtype, order, actmode, (const float *)ctx->xfer_x, m, k, k, w_blocks_dev, n, y_direct ? y_direct : (float *)ctx->xfer_y, n);
    if (s != CQ_OK) return s;
    if (!y_direct) CQ_CUDA(ctx, cudaMemcpyAsync(y_host, ctx->xfer_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    return cq_synchronize(ctx);
}

struct cq_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

cq_status cq_capture_begin(cq_ctx *ctx) {
    CQ_ENTER(ctx);
    if (ctx->capturing) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_capture_begin: already capturing");
    CQ_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    return CQ_OK;
}

cq_status cq_capture_end(cq_ctx *ctx, cq_graph **out) {
    CQ_ENTER(ctx);
    if (!out) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_capture_end: null out pointer");
    *out = nullptr;
    if (!ctx->capturing) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_capture_end: not capturing");
    ctx->capturing = false;
    cq_graph *g = new cq_graph();
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e == cudaSuccess) e = cudaGraphUpload(g->exec, ctx->stream);  // so the first launch does not pay the upload
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        return cq_cuda_fail(ctx, e, "graph capture/instantiate");
    }
    *out = g;
    ++ctx->graphs_alive;
    return CQ_OK;
}

cq_status cq_graph_launch(cq_ctx *ctx, cq_graph *g) {
    CQ_ENTER(ctx);
    if (!g || !g->exec) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_graph_launch: null graph");
    CQ_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    return CQ_OK;
}

cq_status cq_graph_destroy(cq_ctx *ctx, cq_graph *g) {
    CQ_ENTER(ctx);
    if (!g) return CQ_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    if (--ctx->graphs_alive <= 0) {  // nothing references the outgrown scratch blocks any more
        ctx->graphs_alive = 0;
        cudaStreamSynchronize(ctx->stream);
        for (void *p : ctx->retired_scratch) cudaFree(p);
        ctx->retired_scratch.clear();
    }
    return CQ_OK;
}

cq_status cq_timer_start(cq_ctx *ctx) {
    CQ_ENTER(ctx);
    if (!ctx->ev_start) {
        CQ_CUDA(ctx, cudaEventCreate(&ctx->ev_start));
        CQ_CUDA(ctx, cudaEventCreate(&ctx->ev_stop));
    }
    CQ_CUDA(ctx, cudaEventRecord(ctx->ev_start, ctx->stream));
    return CQ_OK;
}

cq_status cq_timer_stop(cq_ctx *ctx, float *ms) {
    CQ_ENTER(ctx);
    if (!ms || !ctx->ev_start) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_timer_stop: no running timer");
    CQ_CUDA(ctx, cudaEventRecord(ctx->ev_stop, ctx->stream));
    CQ_CUDA(ctx, cudaEventSynchronize(ctx->ev_stop));
    CQ_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_start, ctx->ev_stop));
    return CQ_OK;
}

}  // extern "C"
