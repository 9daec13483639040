// The other 32-value block formats of the reference's kernel registry
// (tensor/internal/cuda/kernels/kernels.go:488-493, :511-513): Q4_1, Q5_0, Q5_1.
//
//   Q4_1  20 bytes {f16 d; f16 m; 16 nibble bytes}          w = d*q + m,       q in 0..15
//   Q5_0  22 bytes {f16 d; u32 qh; 16 nibble bytes}         w = d*(q - 16),    q in 0..31
//   Q5_1  24 bytes {f16 d; f16 m; u32 qh; 16 nibble bytes}  w = d*q + m,       q in 0..31
//
// Element order: Q4_1 has both orders of Q4_0 (interleaved, tensor/internal/cpu/kernels/
// quantized.go:107-116; split, tensor/internal/cuda/kernels/quantized.cu:728-747).  The
// 5-bit formats exist only in the split order (quantized.cu:749-795): value j takes the low
// nibble of qs[j] and bit j of qh, value j+16 the high nibble and bit j+16.
//
// d*q and d*(q-16) are exact in f32 (11 + 5 significant bits), so "+ m" is the only
// rounding and the result does not depend on whether the compiler fuses the two.
//
// This file holds everything these formats need: blocks -> f32, f32 -> blocks, blocks -> f16
// for the tensor-core GEMM, and the plain decode GEMV with f32 activations (four lanes per block,
// one row per warp, about 1.0-1.5 TB/s on a B200) that serves the shapes the streaming kernel
// does not take (k % 256 != 0, misaligned pointers); the streaming decoder for these formats is
// DecMore in gemv_kernels.cu.
#include "common.cuh"

namespace {

template <int QT>
struct Fmt;
template <>
struct Fmt<CQ_Q4_1> {
    static constexpr int kBytes = 20, kQs = 4, kQh = -1, kM = 2;
};
template <>
struct Fmt<CQ_Q5_0> {
    static constexpr int kBytes = 22, kQs = 6, kQh = 2, kM = -1;
};
template <>
struct Fmt<CQ_Q5_1> {
    static constexpr int kBytes = 24, kQs = 8, kQh = 4, kM = 2;
};

__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *reinterpret_cast<const unsigned short *>(p); }
__device__ __forceinline__ void st16(uint8_t *p, uint32_t v) { *reinterpret_cast<unsigned short *>(p) = (unsigned short)v; }

// Values 8p .. 8p+7 (p = 0..3) of one block as their integer codes q[8], plus scale and offset
// (offset = -16 d for Q5_0 is applied as (q - 16) * d by the callers, so `sub` carries the 16).
template <int QT, int ORDER>
__device__ __forceinline__ void codes8(const uint8_t *b, int p, int (&q)[8], float &d, float &m, int &sub) {
    using F = Fmt<QT>;
    // Q4_1 (20 bytes) and Q5_1 (24 bytes) keep every field 4-byte aligned: whole-word loads.  Q5_0
    // (22 bytes) is only 2-byte aligned.
    constexpr bool kWords = (F::kBytes % 4) == 0;
    if (kWords) {
        const uint32_t dm = *reinterpret_cast<const uint32_t *>(b);
        d = fp16_bits_to_f32(dm & 0xFFFFu);
        m = fp16_bits_to_f32(dm >> 16);
    } else {
        d = fp16_bits_to_f32(ld16(b));
        m = 0.0f;
    }
    sub = (QT == CQ_Q5_0) ? 16 : 0;
    if (QT == CQ_Q4_1 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
        const uint32_t four = *reinterpret_cast<const uint32_t *>(b + F::kQs + 4 * p);  // bytes 4p..4p+3 hold values 8p..8p+7
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = (int)((four >> (4 * i)) & 0xF);
    } else {
        const uint8_t *qs = b + F::kQs + 8 * (p & 1);  // low (p < 2) or high nibbles of eight bytes
        uint32_t lo, hi, qh = 0;
        if (kWords) {
            lo = *reinterpret_cast<const uint32_t *>(qs), hi = *reinterpret_cast<const uint32_t *>(qs + 4);
            if (F::kQh >= 0) qh = *reinterpret_cast<const uint32_t *>(b + F::kQh) >> (8 * p);
        } else {
            lo = ld16(qs) | (ld16(qs + 2) << 16), hi = ld16(qs + 4) | (ld16(qs + 6) << 16);
            if (F::kQh >= 0) qh = (ld16(b + F::kQh) | (ld16(b + F::kQh + 2) << 16)) >> (8 * p);  // bits of values 8p..8p+7
        }
        const int sh = (p >= 2) ? 4 : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t word = i < 4 ? lo : hi;
            q[i] = (int)((word >> (8 * (i & 3) + sh)) & 0xF) | (int)(((qh >> i) & 1u) << 4);
        }
    }
}

template <int QT, int ORDER>
__device__ __forceinline__ void values8(const uint8_t *b, int p, float (&v)[8]) {
    int q[8], sub;
    float d, m;
    codes8<QT, ORDER>(b, p, q, d, m, sub);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (QT == CQ_Q5_0) ? __fmul_rn((float)(q[i] - sub), d) : __fadd_rn(__fmul_rn((float)q[i], d), m);
}

// ---- blocks -> f32: one thread writes eight consecutive values --------------------------------
template <int QT, int ORDER, bool VEC>
__global__ void __launch_bounds__(256) dequantize_more_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks, float *__restrict__ y) {
    const int64_t total = nblocks * 4;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        float v[8];
        values8<QT, ORDER>(blocks + (idx >> 2) * Fmt<QT>::kBytes, (int)(idx & 3), v);
        if (VEC) {
            reinterpret_cast<float4 *>(y)[2 * idx] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4 *>(y)[2 * idx + 1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[idx * 8 + i] = v[i];
        }
    }
}

// ---- blocks -> f16 for the tensor-core GEMM (the only further rounding is f32 -> f16) ----------
template <int QT, int ORDER>
__global__ void __launch_bounds__(256) w_to_f16_more_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks, __half *__restrict__ out) {
    const int64_t total = nblocks * 4;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        float v[8];
        values8<QT, ORDER>(blocks + (idx >> 2) * Fmt<QT>::kBytes, (int)(idx & 3), v);
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(out + idx * 8) = *reinterpret_cast<uint4 *>(h);
    }
}

// ---- f32 -> blocks: one thread per block, sequential like the reference shaders ---------------
// tensor/internal/metal/kernels/quantized.metal:4216-4280 (Q4_1: min / max, d = (max-min)/15,
// q = min(15, trunc((x-min)/d + 0.5))), :4282-4345 (Q5_0: first element of largest magnitude,
// d = max/-16, q = min(31, trunc(x/d + 16.5))), :4347-4415 (Q5_1: d = (max-min)/31, no clamp).
// The shaders pair value j with value j+16 (split order); Q4_1 also takes the interleaved pairing.
template <int QT, int ORDER>
__global__ void __launch_bounds__(128) quantize_more_kernel(const float *__restrict__ w, int64_t nblocks, uint8_t *__restrict__ blocks) {
    using F = Fmt<QT>;
    const int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= nblocks) return;
    float v[kQK];
    const float *src = w + blk * kQK;
#pragma unroll
    for (int i = 0; i < kQK; ++i) v[i] = src[i];
    uint8_t *b = blocks + blk * F::kBytes;
    float d, mn = 0.0f, off;
    if (QT == CQ_Q5_0) {
        float amax = 0.0f, mx = 0.0f;
#pragma unroll
        for (int j = 0; j < kQK; ++j)
            if (amax < fabsf(v[j])) amax = fabsf(v[j]), mx = v[j];
        d = __fdiv_rn(mx, -16.0f);
        off = 16.5f;
    } else {
        float lo = v[0], hi = v[0];
#pragma unroll
        for (int j = 1; j < kQK; ++j) lo = v[j] < lo ? v[j] : lo, hi = v[j] > hi ? v[j] : hi;
        d = __fdiv_rn(__fsub_rn(hi, lo), QT == CQ_Q4_1 ? 15.0f : 31.0f);
        mn = lo;
        off = 0.5f;
    }
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    st16(b, __half_as_ushort(__float2half_rn(d)));
    if (F::kM >= 0) st16(b + F::kM, __half_as_ushort(__float2half_rn(mn)));
    uint32_t qh = 0;
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
        uint32_t two = 0;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int jj = j + t;
            const int i0 = (QT == CQ_Q4_1 && ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * jj : jj;
            const int i1 = (QT == CQ_Q4_1 && ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * jj + 1 : jj + 16;
            const float x0 = __fmul_rn(__fsub_rn(v[i0], mn), id), x1 = __fmul_rn(__fsub_rn(v[i1], mn), id);
            int q0 = (int)__fadd_rn(x0, off), q1 = (int)__fadd_rn(x1, off);
            if (QT == CQ_Q4_1) q0 = min(15, (int)(signed char)q0), q1 = min(15, (int)(signed char)q1);
            if (QT == CQ_Q5_0) q0 = min(31, (int)(signed char)q0), q1 = min(31, (int)(signed char)q1);
            q0 &= 0xFF, q1 &= 0xFF;  // Q5_1 converts to an unsigned byte without a clamp
            two |= (uint32_t)((q0 & 0xF) | ((q1 & 0xF) << 4)) << (8 * t);
            qh |= (uint32_t)((q0 >> 4) & 1) << jj;
            qh |= (uint32_t)((q1 >> 4) & 1) << (jj + 16);
        }
        st16(b + F::kQs + j, two);
    }
    if (F::kQh >= 0) st16(b + F::kQh, qh & 0xFFFFu), st16(b + F::kQh + 2, qh >> 16);
}

// ---- decode GEMV, f32 activations ------------------------------------------------------------
// A warp owns R consecutive weight rows (the launcher uses R = 1).  Per trip it covers eight blocks of k: lane l takes
// values 8(l%4) .. +7 of block l/4, so the activation loads of a warp are 1 KB contiguous and the
// block bytes of a row are read in 160..192-byte runs.  The eight activations stay in registers
// for the R rows.  Weights are dequantized to their exact f32 values, then FMA-accumulated.
template <int QT, int ORDER, int R>
__global__ void __launch_bounds__(256) gemv_more_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ y,
                                                      int64_t n, int nb) {
    using F = Fmt<QT>;
    const int lane = threadIdx.x & 31;
    const int64_t row0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
    if (row0 >= n) return;
    const int p = lane & 3;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
#pragma unroll 2
    for (int b = lane >> 2; b < nb; b += 8) {
        const float4 xa = __ldg(reinterpret_cast<const float4 *>(x + (int64_t)b * kQK + 8 * p));
        const float4 xb = __ldg(reinterpret_cast<const float4 *>(x + (int64_t)b * kQK + 8 * p) + 1);
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r < n) {
                float v[8];
                values8<QT, ORDER>(w + ((row0 + r) * nb + b) * F::kBytes, p, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[r] = fmaf(v[i], xv[i], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float t = acc[r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
        if (lane == 0 && row0 + r < n) y[row0 + r] = t;
    }
}

unsigned capped_grid(const cq_ctx *ctx, int64_t items, int threads) {
    const int64_t want = (items + threads - 1) / threads, cap = (int64_t)ctx->sm_count * 64;
    return (unsigned)(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace

bool cq_is_more_format(int qtype) { return qtype == CQ_Q4_1 || qtype == CQ_Q5_0 || qtype == CQ_Q5_1; }

int cq_more_block_bytes(int qtype) { return qtype == CQ_Q4_1 ? 20 : (qtype == CQ_Q5_0 ? 22 : (qtype == CQ_Q5_1 ? 24 : 0)); }

// The 5-bit formats have no interleaved twin in the reference: only the split order is accepted.
bool cq_more_order_ok(int qtype, int order) { return qtype == CQ_Q4_1 || order == CQ_ORDER_GGML_SPLIT; }

#define CQ_MORE_DISPATCH(LAUNCH)                                              \
    do {                                                                      \
        if (qtype == CQ_Q4_1 && order == CQ_ORDER_GO_INTERLEAVED) LAUNCH(CQ_Q4_1, 0); \
        else if (qtype == CQ_Q4_1) LAUNCH(CQ_Q4_1, 1);                        \
        else if (qtype == CQ_Q5_0) LAUNCH(CQ_Q5_0, 1);                        \
        else LAUNCH(CQ_Q5_1, 1);                                              \
    } while (0)

// Q4_1 / Q5_1 blocks are read with whole-word loads, Q5_0 blocks with 2-byte loads.
static bool blocks_aligned(int qtype, const void *p) { return (reinterpret_cast<uintptr_t>(p) & (qtype == CQ_Q5_0 ? 1 : 3)) == 0; }
static const char *kAlignMsg = "blocks must be 4-byte aligned (Q4_1, Q5_1) or 2-byte aligned (Q5_0)";

cq_status launch_dequantize_more(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, float *y) {
    if (!blocks_aligned(qtype, blocks)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, kAlignMsg);
    const bool vec = (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    const unsigned grid = capped_grid(ctx, nblocks * 4, 256);
    const uint8_t *b = static_cast<const uint8_t *>(blocks);
#define CQ_L(QT, ORD)                                                                                   \
    do {                                                                                                \
        if (vec) dequantize_more_kernel<QT, ORD, true><<<grid, 256, 0, ctx->stream>>>(b, nblocks, y);   \
        else dequantize_more_kernel<QT, ORD, false><<<grid, 256, 0, ctx->stream>>>(b, nblocks, y);      \
    } while (0)
    CQ_MORE_DISPATCH(CQ_L);
#undef CQ_L
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_quantize_rows_more(cq_ctx *ctx, int qtype, int order, const float *w, int64_t nblocks, void *blocks) {
    if ((reinterpret_cast<uintptr_t>(blocks) & 1) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "blocks must be 2-byte aligned");
    if ((reinterpret_cast<uintptr_t>(w) & 3) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "w must be 4-byte aligned");
    const unsigned grid = (unsigned)((nblocks + 127) / 128);
    uint8_t *b = static_cast<uint8_t *>(blocks);
#define CQ_L(QT, ORD) quantize_more_kernel<QT, ORD><<<grid, 128, 0, ctx->stream>>>(w, nblocks, b)
    CQ_MORE_DISPATCH(CQ_L);
#undef CQ_L
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_w_to_f16_more(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, void *out_f16) {
    if (!blocks_aligned(qtype, blocks)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, kAlignMsg);
    const unsigned grid = capped_grid(ctx, nblocks * 4, 256);
    const uint8_t *b = static_cast<const uint8_t *>(blocks);
    __half *o = static_cast<__half *>(out_f16);
#define CQ_L(QT, ORD) w_to_f16_more_kernel<QT, ORD><<<grid, 256, 0, ctx->stream>>>(b, nblocks, o)
    CQ_MORE_DISPATCH(CQ_L);
#undef CQ_L
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_gemv_more(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w,
                           int64_t n, float *y, int64_t ldy) {
    if (actmode != CQ_ACT_F32) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "Q4_1 / Q5_0 / Q5_1 take f32 (GEMV) or f16 (GEMM) activations, not Q8_1");
    if (!blocks_aligned(qtype, w)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, kAlignMsg);
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (ldx & 3) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx % 4 == 0");
    // One row per warp: more rows per warp (sharing the activation registers) measured slower at every
    // size tried, 1.0 vs 1.5 TB/s at 32000 x 4096 -- the kernel is bound by decode instructions, not by loads.
    constexpr int kWarps = 8;
    const unsigned grid = (unsigned)((n + kWarps - 1) / kWarps);
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    const int nb = (int)(k / kQK);
    for (int64_t i = 0; i < m; ++i) {
        const float *xi = x + i * ldx;
        float *yi = y + i * ldy;
#define CQ_L(QT, ORD) gemv_more_kernel<QT, ORD, 1><<<grid, kWarps * 32, 0, ctx->stream>>>(wb, xi, yi, n, nb)
        CQ_MORE_DISPATCH(CQ_L);
#undef CQ_L
    }
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}
