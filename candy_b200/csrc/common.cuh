// Shared internals of libcandyq: context, error plumbing, small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "candyq.h"

constexpr int kQK = 32;         // values per block
constexpr int kQ4Bytes = 18;    // f16 d + 16 nibble bytes
constexpr int kQ8Bytes = 34;    // f16 d + 32 int8
constexpr int kQ81Bytes = 36;   // f16 d + f16 sum + 32 int8

// Device-side error word codes (written by kernels whose bounded waits gave up).
// 1..4: a bounded wait gave up (CQ_ERR_TIMEOUT at cq_synchronize); 5: a device-resident decode position
// was outside [0, max_ctx) (CQ_ERR_INVALID_ARG at cq_synchronize).
enum : int { kDevErrNone = 0, kDevErrFullWait = 1, kDevErrEmptyWait = 2, kDevErrDrain = 3, kDevErrMma = 4, kDevErrPosition = 5 };

struct GemvTuning {
    int target_warps = 8;   // consumer warps per CTA the launcher aims for
    int stages = 4;         // smem ring depth (clamped by capacity)
    int ctas_per_sm = 0;    // 0 = automatic
    // 1: the producer fills the ring before the CTA's first barrier.  Measured slower: the burst of a new CTA's
    // ring fill delays the last loads of the previous kernel's CTAs still running (sweep of four shapes 40.3 us
    // against 37.7), although the same shape back to back gains 0.1-0.2 us per launch.
    int early = 0;
    // 1: the one-row streaming GEMVs launched while this is set neither read nor overwrite anything that an earlier
    // launch on the stream still in flight writes (q / k / v, or gate / up, of one x): they skip the wait on the
    // previous kernel and overlap it.  The caller's promise; results are undefined if it does not hold.
    int gemv_independent = 0;
    int gemv_chain = 0;     // 1: the GEMVs launched while this is set are links of a chain with small kernels in between (a decode step)
    int force_simple = 0;   // 1: always use the plain one-warp-per-row kernel
    int pdl = 1;            // programmatic dependent launch on the streaming kernel
    int gemm_variant = 0;
    int attn_variant = 0;  // 1 = one CTA per 32-key chunk (the earlier grouped-query kernel) instead of split-context
    int gemm_cache_weights = 0;  // keep the f16 copy of every weight matrix the GEMM has seen (4x the Q4_0 bytes)
    int gemv_rpt = 2;       // rows per thread and pass in the streaming kernel (1 or 2)
    int gemv_coop = 1;      // slice activations once per CTA through shared memory when rows share a CTA
    int comm_poll_limit = 0;  // polls before the reducing norm gives up on a (value, tag) pair; 0 = about a second
    int comm_cluster = 0;     // 1: one CTA per row in the reducing norm instead of a cluster of eight
    int gemm_int8 = 1;        // 1: the int8 tensor-core kernel serves CQ_ACT_Q8_1 from i8_min_rows_q8_1 rows and CQ_ACT_F32 from i8_min_rows_f32 rows
    int64_t host_zero_copy = 256 << 10;  // cq_qmatmul_host, m <= 8: a result of up to this many bytes whose buffer is pinned host memory is written in place (0: always copy out)
    int gemm_pair = 1;           // m > 128: 256 x 256 tiles on CTA pairs (cta_group::2) instead of 128 x 256 per CTA
    int gemm_fused_dequant = 1;  // Q4_0, m > 128: dequantize inside the f16 GEMM's producer instead of making an f16 copy of W (1: up to 384 rows, 2: always)
    int i8_min_rows_f32 = 3;
    int i8_min_rows_q8_1 = 3;
    int gemv_mma = 3;       // CQ_ACT_F32, Q4_0: batches of this many rows up to 8 take the single-launch mma.sync kernel (0: never)
    int fa_transpose_v = 0;   // prefill attention: 1 = always transpose V into scratch first (0: read V tiles in place when their strides allow)
    int gemv_q81_inline = 1;  // CQ_ACT_Q8_1, one or two rows: quantize the activations inside the GEMV's set-up (0: a launch of its own first)
    int gemv_multirow = 1;  // 0: one launch (one weight pass) per activation row even for m = 2..8
    int gemv_variant = 0;   // 0: 16-bit block fixed point (default), 1: f32 FMA, 2 / 3: two / three int8 slices
};

// Set by the tensor-parallel entry point around one GEMV launch (see comm.cu).
struct PushSpec {
    uint2 *const *rx = nullptr;    // [world] this rank's slot in each rank's receive buffer: (value bits, tag) pairs
    const unsigned *seq = nullptr; // local word: tag of the last completed exchange on this set
    int world = 0;
    int64_t row_stride = 0;
};

// Operator fusion around one decode GEMV launch (cq_qlinear_fused): residual add + RMSNorm in the
// prologue, SiLU(gate)*up over adjacent output rows in the epilogue.
struct FuseSpec {
    bool on = false;
    const float *delta = nullptr;  // added to x before the norm (nullable)
    const float *alpha = nullptr;  // norm weights (nullable: no norm, only the add)
    float *x_out = nullptr;        // receives x + delta (nullable); must not alias x
    float eps = 0.0f;
    bool norm = false;
    int epilogue = 0;              // 0: y[r] = row r; 1: y[r/2] = silu(row r) * row r+1 for even r
    int64_t ld_delta = 0, ld_xout = 0;
};

struct cq_ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    int *dev_err = nullptr;       // mapped pinned host word the kernels can write
    int *dev_err_devptr = nullptr;
    void *scratch = nullptr;      // activation staging (Q8_1 blocks / f16 copies)
    size_t scratch_bytes = 0;
    std::vector<void *> retired_scratch;  // outgrown blocks that instantiated graphs may still reference
    int graphs_alive = 0;                 // graphs made by cq_capture_end and not yet destroyed
    void *xfer_x = nullptr;       // device staging used by cq_qmatmul_host
    void *xfer_y = nullptr;
    size_t xfer_x_bytes = 0, xfer_y_bytes = 0;
    // f16 shadow copies of weight matrices for the prefill GEMM (option gemm_cache_weights):
    // key = (blocks pointer, n, k, qtype * 2 + order) -> device allocation of n*k halfs.
    std::map<std::tuple<const void *, int64_t, int64_t, int>, void *> w16_cache;
    size_t w16_cache_bytes = 0;
    std::map<const void *, size_t> allocs;  // cq_malloc'ed blocks -> bytes (so cq_free can drop cached copies of weights inside them)
    GemvTuning tune;
    PushSpec push;
    FuseSpec fuse;
    const float *bias = nullptr;  // set by cq_qlinear around one matmul: the streaming GEMV adds it in its epilogue
    bool bias_done = false;       // ... and says so here; other routes leave it to a small kernel afterwards
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    bool capturing = false;
    std::string last_error;
};

cq_status cq_fail(cq_ctx *ctx, cq_status s, const std::string &msg);
cq_status cq_cuda_fail(cq_ctx *ctx, cudaError_t e, const char *what);
// Grows ctx->scratch to at least `bytes` (never shrinks).  Refused while the stream is capturing (growth
// would allocate and synchronise inside the capture); a block outgrown while graphs exist is kept until
// the last graph is destroyed, because their kernel parameters and tensor maps point into it.
cq_status cq_reserve_scratch(cq_ctx *ctx, size_t bytes);

// Drops the cached f16 copies of every weight matrix whose blocks start inside [begin, begin + bytes).
void cq_w16_invalidate(cq_ctx *ctx, const void *begin, size_t bytes);

#define CQ_CUDA(ctx, call)                                              \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return cq_cuda_fail((ctx), e__, #call); \
    } while (0)

#define CQ_ENTER(ctx)                                                          \
    do {                                                                       \
        if ((ctx) == nullptr) return CQ_ERR_INVALID_ARG;                       \
        cudaError_t e__ = cudaSetDevice((ctx)->device);                        \
        if (e__ != cudaSuccess) return cq_cuda_fail((ctx), e__, "cudaSetDevice"); \
    } while (0)

// ---- launchers implemented in the kernel translation units -------------------------
cq_status launch_dequantize(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, float *y);
cq_status launch_quantize_rows(cq_ctx *ctx, int qtype, int order, const float *w, int64_t nblocks, void *blocks);
cq_status launch_quantize_q8_1(cq_ctx *ctx, const float *x, int64_t m, int64_t k, int64_t ldx, void *out);
cq_status launch_gemv(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k,
                      int64_t ldx, const void *w, int64_t n, float *y, int64_t ldy);
cq_status launch_gemv_q8_1_blocks(cq_ctx *ctx, int qtype, int order, const void *act_blocks, int64_t m, int64_t k,
                                  const void *w, int64_t n, float *y, int64_t ldy);
// Q4_1 / Q5_0 / Q5_1 (more_formats.cu)
bool cq_is_more_format(int qtype);
int cq_more_block_bytes(int qtype);
bool cq_more_order_ok(int qtype, int order);
cq_status launch_dequantize_more(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, float *y);
cq_status launch_quantize_rows_more(cq_ctx *ctx, int qtype, int order, const float *w, int64_t nblocks, void *blocks);
cq_status launch_w_to_f16_more(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, void *out_f16);
cq_status launch_gemv_more(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w,
                           int64_t n, float *y, int64_t ldy);
// K super-block formats, 256 values per block (kquants.cu)
bool cq_is_k_format(int qtype);
int cq_k_block_bytes(int qtype);
cq_status launch_dequantize_k(cq_ctx *ctx, int qtype, const void *blocks, int64_t nblocks, float *y);
cq_status launch_w_to_f16_k(cq_ctx *ctx, int qtype, const void *blocks, int64_t nblocks, void *out_f16);
cq_status launch_gemv_k(cq_ctx *ctx, int qtype, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, float *y,
                        int64_t ldy);
// Narrow-batch GEMM that dequantizes raw blocks into tensor memory (gemm_dequant_tmem.cu).
bool qgemm_dequant_tmem_supported(int qtype, int64_t m, int64_t k, const void *w);
cq_status launch_qgemm_dequant_tmem(cq_ctx *ctx, int qtype, int order, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n,
                                    float *y, int64_t ldy);
// Integer-dot GEMM on tcgen05.mma kind::i8 (gemm_i8_tmem.cu): mode 1 = Q8_1 activation columns, mode 0 = 15-bit planes.
bool qgemm_i8_supported(int qtype, int64_t k, const void *w, const float *x, int64_t ldx);
// Q4_0, 2..8 activation rows, one launch, one weight pass (gemv_mma.cu): CQ_ACT_F32 numerics of small batches, or with
// q8_1 set those of CQ_ACT_Q8_1.
bool gemv_mma_supported(cq_ctx *ctx, int qtype, int64_t m, int64_t k, int64_t n, const void *w, const float *x, int64_t ldx);
cq_status launch_gemv_mma(cq_ctx *ctx, int order, int q8_1, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, const float *bias,
                          float *y, int64_t ldy);
// Q4_0, 1..8 activation rows, CQ_ACT_F16 numerics: one launch, one weight pass (gemv_mma_f16.cu).
bool gemv_mma_f16_supported(cq_ctx *ctx, int qtype, int64_t m, int64_t k, int64_t n, const void *w, const float *x, int64_t ldx);
cq_status launch_gemv_mma_f16(cq_ctx *ctx, int order, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, const float *bias,
                              float *y, int64_t ldy);
cq_status launch_qgemm_i8(cq_ctx *ctx, int qtype, int order, int mode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n,
                          float *y, int64_t ldy);
cq_status launch_gemm(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k,
                      int64_t ldx, const void *w, int64_t n, float *y, int64_t ldy);

#ifdef __CUDACC__
// binary16 bits -> f32 exactly as tensor/internal/cpu/kernels/quantized.go:149-173:
// finite values through the hardware conversion (exact), inf/NaN by bit assembly so a
// NaN keeps its payload (mantissa << 13) instead of being quieted.
__device__ __forceinline__ float fp16_bits_to_f32(uint32_t h) {
    h &= 0xFFFFu;
    if ((h & 0x7C00u) == 0x7C00u) return __uint_as_float(((h & 0x8000u) << 16) | 0x7F800000u | ((h & 0x3FFu) << 13));
    return __half2float(__ushort_as_half((unsigned short)h));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false (callers record an error
// word and leave; nothing in this library spins without a limit).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Same, with a sleep between polls: a waiting warp then costs almost no issue slots (the plain
// loop competes with working warps for the integer pipe).  About a second at most.
__device__ __forceinline__ bool mbar_wait_sleep(uint32_t bar, uint32_t parity, uint32_t sleep_ns) {
    const uint32_t limit = sleep_ns >= 512 ? (1u << 21) : (1u << 23);
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(sleep_ns);
    }
    return false;
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 1-D bulk async copy global -> this CTA's shared memory, completion on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Same copy with an L2 eviction-priority hint (a policy word from make_l2_policy_*).
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst_smem),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t make_l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Packed pairs of f32 in a 64-bit register: sm_100 adds, multiplies and fuses two at a time.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t dup2(float v) { return pack2(v, v); }
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif  // __CUDACC__
