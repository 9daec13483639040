// cq_qmatmul_q8_1_static: the quantized-activation decode GEMV for callers that must not
// allocate device memory.
//
// Who that is: a host that has handed all of the GPU's memory to its own arena at start-up
// (an inference server with a pre-sized KV cache, a Go or Java runtime whose cgo/JNI layer is
// forbidden to call the CUDA allocator behind the collector's back), or code running where a
// cudaMalloc would synchronise the device in the middle of a latency-critical decode step.
// The regular entry point, cq_qmatmul with CQ_ACT_Q8_1, keeps the quantized activations in
// context-owned scratch that it grows with cudaMalloc on demand; this one keeps them in a
// fixed array inside the library image instead.
//
// The array below lives in device memory of EVERY GPU that loads the library, from load until
// the process exits: kStaticScratchBytes (288 KiB) per GPU, whether or not this entry is used.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kStaticMaxM = 8;        // activation rows
constexpr int kStaticMaxK = 32768;    // inner dimension
constexpr size_t kStaticScratchBytes = (size_t)kStaticMaxM * (kStaticMaxK / kQK) * kQ81Bytes;  // 294,912 bytes

// Q8_1 activation blocks of the call in flight.  Inside device code this name is the array;
// inside host code it is only a handle for cudaGetSymbolAddress and must never be passed to a
// kernel as if it were a device pointer.
static __device__ __align__(256) unsigned char g_q8_1_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void *g_scratch_addr[kMaxDevices] = {};  // device address of the array on each GPU, looked up once
std::mutex g_scratch_mutex;

// With `device` current: the device address of g_q8_1_scratch on that GPU.
cq_status static_scratch_address(cq_ctx *ctx, void **out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "device ordinal beyond 63");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[ctx->device] == nullptr) {
        // The one-time lookup is a runtime call that must not land inside a stream capture.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (ctx->capturing || (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone))
            return cq_fail(ctx, CQ_ERR_INVALID_ARG,
                           "cq_qmatmul_q8_1_static: the first call on a device looks up the scratch array's address and must be made outside stream capture");
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_q8_1_scratch);
        if (e != cudaSuccess) return cq_cuda_fail(ctx, e, "cudaGetSymbolAddress(g_q8_1_scratch)");
        if (ptr == nullptr) return cq_fail(ctx, CQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[ctx->device] = ptr;
    }
    *out = g_scratch_addr[ctx->device];
    return CQ_OK;
}

}  // namespace

extern "C" cq_status cq_qmatmul_q8_1_static(cq_ctx *ctx, int qtype, int order, const float *x_dev, int64_t m, int64_t k,
                                            int64_t ldx, const void *w_blocks_dev, int64_t n, float *y_dev, int64_t ldy) {
    CQ_ENTER(ctx);  // makes ctx->device current: the symbol lookup below is per device
    if (qtype != CQ_Q4_0 && qtype != CQ_Q8_0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "qtype must be CQ_Q4_0 or CQ_Q8_0");
    if (order != CQ_ORDER_GO_INTERLEAVED && order != CQ_ORDER_GGML_SPLIT)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "order must be 0 (interleaved) or 1 (split)");
    if (!x_dev || !w_blocks_dev || !y_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_q8_1_static: null pointer");
    if (m < 1 || n < 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_q8_1_static: m and n must be >= 1");
    if (k < kQK || k % kQK != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_q8_1_static: k must be a positive multiple of 32");
    if (ldx < k || ldy < n) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_q8_1_static: ldx < k or ldy < n");
    if (m > kStaticMaxM || k > kStaticMaxK)
        return cq_fail(ctx, CQ_ERR_TOO_LARGE,
                       "cq_qmatmul_q8_1_static: limits are m <= 8 and k <= 32768 (the activation blocks must fit the fixed "
                       "294912-byte array); use cq_qmatmul for larger problems");
    if ((reinterpret_cast<uintptr_t>(x_dev) & 3) != 0 || (reinterpret_cast<uintptr_t>(y_dev) & 3) != 0 ||
        (reinterpret_cast<uintptr_t>(w_blocks_dev) & 1) != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_q8_1_static: misaligned pointer");
    void *scratch = nullptr;
    cq_status s = static_scratch_address(ctx, &scratch);
    if (s != CQ_OK) return s;
    // The quantizer rewrites every block the GEMV then reads (m * k/32 of them), so nothing left
    // over from an earlier call is ever consumed and nothing needs clearing.  The GEMV takes the same
    // routes as cq_qmatmul's CQ_ACT_Q8_1 mode (streaming kernel when the shape fits, whose only working
    // memory is shared memory; the plain kernel otherwise): neither allocates.
    s = launch_quantize_q8_1(ctx, x_dev, m, k, ldx, scratch);
    if (s != CQ_OK) return s;
    return launch_gemv_q8_1_blocks(ctx, qtype, order, scratch, m, k, w_blocks_dev, n, y_dev, ldy);
}
