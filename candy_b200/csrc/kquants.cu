// The 256-value "K" super-block formats of the reference's kernel registry
// (tensor/internal/cuda/kernels/kernels.go:488-627; layouts tensor/internal/cuda/kernels/quantized.cu:366-436,
// dequantizers :899-1147).  The reference has no CPU code and no quantizer for them: its CUDA dequantizers are
// the definition, restated here value by value.
//
//   Q2_K  84 B {u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}           16 x 16 values: d*(sc&15)*q2 - dmin*(sc>>4)
//   Q3_K 110 B {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}        16 x 16 values: d*(s6-32) * (q2 - (hbit ? 0 : 4))
//   Q4_K 144 B {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]}            8 x 32 values: (d*s6)*q4 - dmin*m6
//   Q5_K 176 B {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} 8 x 32 values: (d*s6)*q5 - dmin*m6
//   Q6_K 210 B {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}          16 x 16 values: d*sc*(q6 - 32)
//
// Every value is computed with exactly the reference's operations in its order; each expression has at most
// one inexact step, so the f32 results do not depend on whether the compiler fuses multiply and add, and they
// equal the reference kernels' bit for bit.
// Here: blocks -> f32, blocks -> f16 (for the tensor-core GEMM), and a decode GEMV with f32 activations (one
// warp per weight row, sixteen values per lane and trip).  No quantizer (the reference has none either).
#include "common.cuh"

namespace {

__device__ __forceinline__ float h2f(const uint8_t *p) { return fp16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

// The 6-bit (scale, min) pair j of the 12-byte packing shared by Q4_K and Q5_K (get_scale_min_k4, quantized.cu:994-1006).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

template <int QT>
struct KFmt;
template <>
struct KFmt<CQ_Q2_K> {
    static constexpr int kBytes = 84;
};
template <>
struct KFmt<CQ_Q3_K> {
    static constexpr int kBytes = 110;
};
template <>
struct KFmt<CQ_Q4_K> {
    static constexpr int kBytes = 144;
};
template <>
struct KFmt<CQ_Q5_K> {
    static constexpr int kBytes = 176;
};
template <>
struct KFmt<CQ_Q6_K> {
    static constexpr int kBytes = 210;
};

// Values 16g .. 16g+15 (g = 0..15) of one super-block.
template <int QT>
__device__ __forceinline__ void dequant16(const uint8_t *b, int g, float (&y)[16]) {
    if (QT == CQ_Q2_K) {
        // value 128n + 32j + l: q = (qs[32n + l] >> 2j) & 3, scale byte 8n + 2j + l/16 = g  (quantized.cu:902-925)
        const int n = g >> 3, j = (g & 7) >> 1, l0 = (g & 1) * 16;
        const float dall = h2f(b + 80), dmin = h2f(b + 82);
        const int sc = b[g];
        const float dl = dall * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
        const uint8_t *qs = b + 16 + 32 * n + l0;
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = dl * (float)((qs[i] >> (2 * j)) & 3) - ml;
    } else if (QT == CQ_Q3_K) {
        // value 128n + 32j + l: low bits (qs[32n + l] >> 2j) & 3, high bit hmask[l] & (1 << (4n + j)), scale g  (quantized.cu:937-969)
        const int n = g >> 3, j = (g & 7) >> 1, l0 = (g & 1) * 16;
        const uint8_t *sc = b + 96;
        const int is = g;
        const int us = is < 4 ? (sc[is] & 0xF) | (((sc[is + 8] >> 0) & 3) << 4)
                     : is < 8 ? (sc[is] & 0xF) | (((sc[is + 4] >> 2) & 3) << 4)
                     : is < 12 ? (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4)
                               : (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
        const float dl = h2f(b + 108) * (float)(us - 32);
        const uint8_t *qs = b + 32 + 32 * n + l0, *hm = b + l0;
        const int mask = 1 << (4 * n + j);
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = dl * (float)((int)((qs[i] >> (2 * j)) & 3) - ((hm[i] & mask) ? 0 : 4));
    } else if (QT == CQ_Q4_K || QT == CQ_Q5_K) {
        // value 64il + 32h + l: nibble h of qs[32il + l], scale pair 2il + h  (quantized.cu:1008-1042, :1049-1082)
        const int il = g >> 2, h = (g & 3) >> 1, l0 = (g & 1) * 16;
        const float dall = h2f(b), dmin = h2f(b + 2);
        int sc, m;
        scale_min_k4(2 * il + h, b + 4, sc, m);
        const float d1 = dall * (float)sc, m1 = dmin * (float)m;
        const uint8_t *qs = b + (QT == CQ_Q4_K ? 16 : 48) + 32 * il + l0;
        const uint8_t *qh = b + 16 + l0;  // Q5_K only
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int q = h ? (qs[i] >> 4) : (qs[i] & 0xF);
            if (QT == CQ_Q5_K) q += ((qh[i] >> (2 * il + h)) & 1) ? 16 : 0;
            y[i] = d1 * (float)q - m1;
        }
    } else {
        // Q6_K, value 128ip + 32t + l: t = 0: ql[64ip + l] & 15, 1: ql[64ip + 32 + l] & 15, 2 / 3: the same bytes' high
        // nibbles; two more bits (qh[32ip + l] >> 2t) & 3; scale 8ip + 2t + l/16 = g  (quantized.cu:1099-1123)
        const int ip = g >> 3, t = (g & 7) >> 1, l0 = (g & 1) * 16;
        const float d = h2f(b + 208);
        const float ds = d * (float)(int)(signed char)b[192 + g];
        const uint8_t *ql = b + 64 * ip + 32 * (t & 1) + l0, *qh = b + 128 + 32 * ip + l0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int lo = (t & 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
            const int q = lo | (((qh[i] >> (2 * t)) & 3) << 4);
            y[i] = ds * (float)(q - 32);
        }
    }
}

template <int QT>
__global__ void __launch_bounds__(256) dequantize_k_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks, float *__restrict__ out) {
    const int64_t total = nblocks * 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float y[16];
        dequant16<QT>(blocks + (i >> 4) * KFmt<QT>::kBytes, (int)(i & 15), y);
        float *dst = out + i * 16;
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = y[j];
    }
}

template <int QT>
__global__ void __launch_bounds__(256) w_to_f16_k_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks, __half *__restrict__ out) {
    const int64_t total = nblocks * 16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float y[16];
        dequant16<QT>(blocks + (i >> 4) * KFmt<QT>::kBytes, (int)(i & 15), y);
        __half2 h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = __floats2half2_rn(y[2 * j], y[2 * j + 1]);
        uint4 *dst = reinterpret_cast<uint4 *>(out + i * 16);  // k % 256 == 0 and the scratch is aligned: 32-byte groups
        dst[0] = reinterpret_cast<uint4 *>(h)[0];
        dst[1] = reinterpret_cast<uint4 *>(h)[1];
    }
}

// y[r, row] = sum over k of x[r, k] * dequant(W[row, k]); one warp per weight row, M activation rows.
template <int QT, int M>
__global__ void __launch_bounds__(256) gemv_k_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, int64_t n, int nsb,
                                                   int64_t ldx, int64_t ldy) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.0f;
    const uint8_t *wr = w + row * (int64_t)nsb * KFmt<QT>::kBytes;
    for (int gi = lane; gi < nsb * 16; gi += 32) {
        float v[16];
        dequant16<QT>(wr + (gi >> 4) * KFmt<QT>::kBytes, gi & 15, v);
        const float *xg = x + (int64_t)gi * 16;
#pragma unroll
        for (int r = 0; r < M; ++r) {
            const float4 *xv = reinterpret_cast<const float4 *>(xg + r * ldx);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const float4 t = xv[q4];
                acc[r] = fmaf(v[4 * q4], t.x, fmaf(v[4 * q4 + 1], t.y, fmaf(v[4 * q4 + 2], t.z, fmaf(v[4 * q4 + 3], t.w, acc[r]))));
            }
        }
    }
#pragma unroll
    for (int r = 0; r < M; ++r) {
        float t = acc[r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
        if (lane == 0) y[r * ldy + row] = t;
    }
}

unsigned k_grid(const cq_ctx *ctx, int64_t items, int threads) {
    int64_t g = (items + threads - 1) / threads;
    const int64_t cap = (int64_t)ctx->sm_count * 32;
    return (unsigned)(g < cap ? (g < 1 ? 1 : g) : cap);
}

}  // namespace

bool cq_is_k_format(int qtype) { return qtype == CQ_Q2_K || qtype == CQ_Q3_K || qtype == CQ_Q4_K || qtype == CQ_Q5_K || qtype == CQ_Q6_K; }

int cq_k_block_bytes(int qtype) {
    switch (qtype) {
        case CQ_Q2_K: return 84;
        case CQ_Q3_K: return 110;
        case CQ_Q4_K: return 144;
        case CQ_Q5_K: return 176;
        case CQ_Q6_K: return 210;
        default: return 0;
    }
}

#define CQ_K_DISPATCH(LAUNCH)               \
    do {                                    \
        switch (qtype) {                    \
            case CQ_Q2_K: LAUNCH(CQ_Q2_K); break; \
            case CQ_Q3_K: LAUNCH(CQ_Q3_K); break; \
            case CQ_Q4_K: LAUNCH(CQ_Q4_K); break; \
            case CQ_Q5_K: LAUNCH(CQ_Q5_K); break; \
            default: LAUNCH(CQ_Q6_K); break;      \
        }                                   \
    } while (0)

cq_status launch_dequantize_k(cq_ctx *ctx, int qtype, const void *blocks, int64_t nblocks, float *y) {
    const unsigned grid = k_grid(ctx, nblocks * 16, 256);
    const uint8_t *b = static_cast<const uint8_t *>(blocks);
#define CQ_L(QT) dequantize_k_kernel<QT><<<grid, 256, 0, ctx->stream>>>(b, nblocks, y)
    CQ_K_DISPATCH(CQ_L);
#undef CQ_L
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_w_to_f16_k(cq_ctx *ctx, int qtype, const void *blocks, int64_t nblocks, void *out_f16) {
    const unsigned grid = k_grid(ctx, nblocks * 16, 256);
    const uint8_t *b = static_cast<const uint8_t *>(blocks);
    __half *o = static_cast<__half *>(out_f16);
#define CQ_L(QT) w_to_f16_k_kernel<QT><<<grid, 256, 0, ctx->stream>>>(b, nblocks, o)
    CQ_K_DISPATCH(CQ_L);
#undef CQ_L
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_gemv_k(cq_ctx *ctx, int qtype, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, float *y,
                        int64_t ldy) {
    if (actmode != CQ_ACT_F32) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "the K formats take f32 (GEMV) or f16 (GEMM) activations, not Q8_1");
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (ldx & 3) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "x must be 16-byte aligned with ldx % 4 == 0");
    constexpr int kWarps = 8;
    const unsigned grid = (unsigned)((n + kWarps - 1) / kWarps);
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    const int nsb = (int)(k / 256);
    for (int64_t r0 = 0; r0 < m; r0 += 4) {  // up to four activation rows share one pass over the weights
        const int rows = (int)((m - r0) < 4 ? (m - r0) : 4);
        const float *xi = x + r0 * ldx;
        float *yi = y + r0 * ldy;
#define CQ_L(QT)                                                                                                       \
    do {                                                                                                               \
        if (rows == 1) gemv_k_kernel<QT, 1><<<grid, kWarps * 32, 0, ctx->stream>>>(wb, xi, yi, n, nsb, ldx, ldy);      \
        else if (rows == 2) gemv_k_kernel<QT, 2><<<grid, kWarps * 32, 0, ctx->stream>>>(wb, xi, yi, n, nsb, ldx, ldy); \
        else if (rows == 3) gemv_k_kernel<QT, 3><<<grid, kWarps * 32, 0, ctx->stream>>>(wb, xi, yi, n, nsb, ldx, ldy); \
        else gemv_k_kernel<QT, 4><<<grid, kWarps * 32, 0, ctx->stream>>>(wb, xi, yi, n, nsb, ldx, ldy);                \
    } while (0)
        CQ_K_DISPATCH(CQ_L);
#undef CQ_L
    }
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}
