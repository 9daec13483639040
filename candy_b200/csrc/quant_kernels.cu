// Block-format conversion kernels: blocks -> f32 (bit-exact), f32 -> Q4_0 / Q8_0 weight
// blocks, f32 -> Q8_1 activation blocks.  All are streaming, HBM-bound kernels; none is
// on the per-token hot path (weights are quantized once, dequantize is a utility).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t ld_u16(const uint8_t *p) { return *reinterpret_cast<const unsigned short *>(p); }

// d * f with the NaN bit patterns the reference's CPU path produces on amd64 (SSE MULSS):
// a NaN scale comes back quieted with its payload, inf * 0 gives the default NaN 0xFFC00000.
// The GPU multiplier would return the canonical 0x7FFFFFFF for both.
__device__ __forceinline__ float mul_like_cpu(float d, float f) {
    float r = __fmul_rn(d, f);
    if (r != r) {
        const uint32_t db = __float_as_uint(d);
        r = ((db & 0x7FFFFFFFu) > 0x7F800000u) ? __uint_as_float(db | 0x00400000u) : __uint_as_float(0xFFC00000u);
    }
    return r;
}

// One thread produces four consecutive f32 values (one 16-byte store), so a warp writes
// 512 contiguous bytes.  Semantics: tensor/internal/cpu/kernels/quantized.go:85-93
// (ORDER 0), tensor/internal/cuda/kernels/quantized.cu:838-867 (ORDER 1), quantized.go:
// 131-136 (Q8_0).  d*(q-8) and d*q are exact in f32, so the results are bit-identical to
// the Go loops for every scale, including subnormal, inf and NaN scales.
template <int QT, int ORDER, bool VEC>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks,
                                                       float *__restrict__ y) {
    const int64_t total = nblocks * 8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t blk = idx >> 3;
        const int p = (int)(idx & 7);
        float v[4];
        if (QT == CQ_Q4_0) {
            const uint8_t *b = blocks + blk * kQ4Bytes;
            const float d = fp16_bits_to_f32(ld_u16(b));
            int q[4];
            if (ORDER == CQ_ORDER_GO_INTERLEAVED) {
                const uint32_t two = ld_u16(b + 2 + 2 * p);  // bytes 2p, 2p+1 -> values 4p..4p+3
                q[0] = two & 0xF, q[1] = (two >> 4) & 0xF, q[2] = (two >> 8) & 0xF, q[3] = (two >> 12) & 0xF;
            } else {
                const uint8_t *qs = b + 2 + 4 * (p & 3);  // values 4p..4p+3 = low (p<4) or high nibbles
                const uint32_t four = ld_u16(qs) | (ld_u16(qs + 2) << 16);
                const int sh = (p >= 4) ? 4 : 0;
                q[0] = (four >> sh) & 0xF, q[1] = (four >> (8 + sh)) & 0xF, q[2] = (four >> (16 + sh)) & 0xF,
                q[3] = (four >> (24 + sh)) & 0xF;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = mul_like_cpu(d, (float)(q[i] - 8));
        } else {
            const uint8_t *b = blocks + blk * kQ8Bytes;
            const float d = fp16_bits_to_f32(ld_u16(b));
            const uint8_t *qs = b + 2 + 4 * p;
            const uint32_t four = ld_u16(qs) | (ld_u16(qs + 2) << 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = mul_like_cpu(d, (float)(int)(signed char)((four >> (8 * i)) & 0xFF));
        }
        if (VEC) {
            reinterpret_cast<float4 *>(y)[idx] = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) y[idx * 4 + i] = v[i];
        }
    }
}

__device__ __forceinline__ void st_u16(uint8_t *p, uint32_t v) { *reinterpret_cast<unsigned short *>(p) = (unsigned short)v; }

// One thread quantizes one block of 32 values, sequentially, so that "first element with
// the largest magnitude" and every rounding follow the reference shaders literally:
// tensor/internal/metal/kernels/quantized.metal:4187-4211 (Q4_0), :4129-4145 (Q8_0).
// Multiplies and adds are issued with explicit rounding intrinsics so the compiler cannot
// contract v*id + 8.5 into one fused operation.
template <int QT, int ORDER>
__global__ void __launch_bounds__(128) quantize_rows_kernel(const float *__restrict__ w, int64_t nblocks,
                                                          uint8_t *__restrict__ blocks) {
    const int64_t blk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (blk >= nblocks) return;
    float v[kQK];
    const float *src = w + blk * kQK;
    if ((reinterpret_cast<uintptr_t>(w) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4 t = reinterpret_cast<const float4 *>(src)[i];
            v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kQK; ++i) v[i] = src[i];
    }
    if (QT == CQ_Q4_0) {
        uint8_t *b = blocks + blk * kQ4Bytes;
        float amax = 0.0f, mx = 0.0f;
#pragma unroll
        for (int j = 0; j < kQK; ++j)
            if (amax < fabsf(v[j])) {
                amax = fabsf(v[j]);
                mx = v[j];
            }
        const float d = __fdiv_rn(mx, -8.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
        st_u16(b, __half_as_ushort(__float2half_rn(d)));
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            uint32_t two = 0;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int jj = j + t;
                const int i0 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * jj : jj;
                const int i1 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * jj + 1 : jj + 16;
                int q0 = (int)__fadd_rn(__fmul_rn(v[i0], id), 8.5f);
                int q1 = (int)__fadd_rn(__fmul_rn(v[i1], id), 8.5f);
                q0 = min(15, (int)(signed char)q0);
                q1 = min(15, (int)(signed char)q1);
                two |= (uint32_t)(((q0 & 0xFF) | ((q1 << 4) & 0xFF)) & 0xFF) << (8 * t);
            }
            st_u16(b + 2 + j, two);
        }
    } else {
        uint8_t *b = blocks + blk * kQ8Bytes;
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < kQK; ++j) {
            const float a = fabsf(v[j]);
            amax = amax > a ? amax : a;
        }
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
        st_u16(b, __half_as_ushort(__float2half_rn(d)));
#pragma unroll
        for (int j = 0; j < kQK; j += 2) {
            const int q0 = (int)roundf(__fmul_rn(v[j], id));
            const int q1 = (int)roundf(__fmul_rn(v[j + 1], id));
            st_u16(b + 2 + j, (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8));
        }
    }
}

// One warp per block of 32 activations, as tensor/internal/cuda/kernels/quantized.cu:
// 3521-3558: xor-butterfly max and sum, d = amax/127, q = roundf(x/d) by true division.
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const float *__restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                          uint8_t *__restrict__ out) {
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= m * k) return;  // m*k is a multiple of 32: whole warps leave together
    const int64_t row = gid / k, col = gid - row * k;
    const float xi = x[row * ldx + col];
    float amax = fabsf(xi), sum = xi;
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask, 32));
        sum += __shfl_xor_sync(0xffffffffu, sum, mask, 32);
    }
    const float d = __fdiv_rn(amax, 127.0f);
    const int q = (amax == 0.0f) ? 0 : (int)roundf(__fdiv_rn(xi, d));
    uint8_t *b = out + (gid >> 5) * kQ81Bytes;
    const int lane = threadIdx.x & 31;
    b[4 + lane] = (uint8_t)(q & 0xFF);
    if (lane == 0) {
        st_u16(b, __half_as_ushort(__float2half_rn(d)));
        st_u16(b + 2, __half_as_ushort(__float2half_rn(sum)));
    }
}

}  // namespace

cq_status launch_dequantize(cq_ctx *ctx, int qtype, int order, const void *blocks, int64_t nblocks, float *y) {
    const bool vec = (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    if ((reinterpret_cast<uintptr_t>(blocks) & 1) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "blocks must be 2-byte aligned");
    const int64_t total = nblocks * 8;
    const int threads = 256;
    int64_t grid64 = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)ctx->sm_count * 64;
    const unsigned grid = (unsigned)(grid64 < cap ? grid64 : cap);
    const uint8_t *b = static_cast<const uint8_t *>(blocks);
#define CQ_DQ(QT, ORD)                                                                                  \
    do {                                                                                                \
        if (vec) dequantize_kernel<QT, ORD, true><<<grid, threads, 0, ctx->stream>>>(b, nblocks, y);    \
        else dequantize_kernel<QT, ORD, false><<<grid, threads, 0, ctx->stream>>>(b, nblocks, y);       \
    } while (0)
    if (qtype == CQ_Q4_0 && order == CQ_ORDER_GO_INTERLEAVED) CQ_DQ(CQ_Q4_0, 0);
    else if (qtype == CQ_Q4_0) CQ_DQ(CQ_Q4_0, 1);
    else CQ_DQ(CQ_Q8_0, 0);
#undef CQ_DQ
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_quantize_rows(cq_ctx *ctx, int qtype, int order, const float *w, int64_t nblocks, void *blocks) {
    if ((reinterpret_cast<uintptr_t>(blocks) & 1) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "blocks must be 2-byte aligned");
    if ((reinterpret_cast<uintptr_t>(w) & 3) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "w must be 4-byte aligned");
    const int threads = 128;
    const unsigned grid = (unsigned)((nblocks + threads - 1) / threads);
    uint8_t *b = static_cast<uint8_t *>(blocks);
    if (qtype == CQ_Q4_0 && order == CQ_ORDER_GO_INTERLEAVED)
        quantize_rows_kernel<CQ_Q4_0, 0><<<grid, threads, 0, ctx->stream>>>(w, nblocks, b);
    else if (qtype == CQ_Q4_0)
        quantize_rows_kernel<CQ_Q4_0, 1><<<grid, threads, 0, ctx->stream>>>(w, nblocks, b);
    else
        quantize_rows_kernel<CQ_Q8_0, 0><<<grid, threads, 0, ctx->stream>>>(w, nblocks, b);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status launch_quantize_q8_1(cq_ctx *ctx, const float *x, int64_t m, int64_t k, int64_t ldx, void *out) {
    if ((reinterpret_cast<uintptr_t>(out) & 1) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "q8_1 output must be 2-byte aligned");
    const int threads = 256;
    const unsigned grid = (unsigned)((m * k + threads - 1) / threads);
    quantize_q8_1_kernel<<<grid, threads, 0, ctx->stream>>>(x, m, k, ldx, static_cast<uint8_t *>(out));
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}
