// The small kernels a decoder step needs around the quantized linears, each following the
// arithmetic of candy's CPU kernels (paths inside a gocnn/candy checkout):
//   RMSNorm        tensor/internal/cpu/kernels/reduce.go:3071-3092  (FastRmsNormF32)
//   softmax        reduce.go:2855-2879 (FastSoftmaxF32), inside the decode-attention kernel
//   RoPE           reduce.go:3987-4006 (RopeF32: half-split pairs (i, i + d/2), cos/sin tables)
//   SiLU           tensor/internal/cpu/kernels/unary.go:3353-3365 (USiluF32, evaluated in f64)
//   argmax         reduce.go:846-862 (FastArgmaxF32: strict >, the lowest index wins ties)
//   embedding      tensor/internal/cpu/kernels/indexing.go:8-26 (index select of rows)
// All are HBM- or latency-bound streaming kernels over a few KB..MB; none touches weights.
// They take part in programmatic dependent launch like the GEMV: trigger the dependents at
// entry, wait for the previous kernel before reading its output.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cooperative_groups.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o, 32);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o, 32));
    return v;
}

// Block-wide sum over blockDim.x threads (multiple of 32, <= 1024); result in every thread.
__device__ __forceinline__ float block_sum(float v, float *sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : 0.0f;
    return warp_sum(t);
}

// y = x * rsqrt(mean(x^2) + eps) * alpha, one CTA per row; optionally x += delta first (the
// residual add that precedes every norm in a decoder layer), written back to x.
template <bool ADD>
__global__ void __launch_bounds__(1024) rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ delta,
                                                     const float *__restrict__ alpha, int cols, float eps, float *__restrict__ y) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    pdl_wait_prior();
    float *xr = x + (int64_t)blockIdx.x * cols;
    const float *dr = ADD ? delta + (int64_t)blockIdx.x * cols : nullptr;
    float *yr = y + (int64_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = xr[c];
        if (ADD) {
            v += dr[c];
            xr[c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, sh);
    const float mean = ss / (float)cols;
    const float scale = 1.0f / sqrtf(mean + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = xr[c];  // own writes above are visible to the same thread
        yr[c] = alpha ? scale * v * alpha[c] : scale * v;
    }
}

// The decode position lives on the device (it is advanced inside captured graphs), so the host cannot
// validate it: every kernel that indexes a cache or a rotary table with it goes through here.  A position
// outside [0, max_ctx) is recorded in the context's error word (reported by cq_synchronize) and clamped,
// so that no access ever leaves the caches or the tables; the step's results are then meaningless.
__device__ __forceinline__ int checked_pos(const int *pos_dev, int max_ctx, int *err) {
    const int pos = *pos_dev;
    if (pos < 0 || pos >= max_ctx) {
        if (threadIdx.x == 0) atomicExch(err, kDevErrPosition);
        return pos < 0 ? 0 : max_ctx - 1;
    }
    return pos;
}

// qkv: [B, (nq + 2 nkv) * hd].  Rotates q in place and k (half-split pairs), then stores k and v
// of every sequence at position *pos of its cache [B][max_ctx][nkv*hd].
__global__ void __launch_bounds__(256) rope_store_kv_kernel(float *__restrict__ qkv, int nq, int nkv, int hd,
                                                          const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                                          const int *__restrict__ pos_dev, float *__restrict__ kc,
                                                          float *__restrict__ vc, int max_ctx, int *err) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int b = blockIdx.y;
    const int pos = checked_pos(pos_dev, max_ctx, err);
    const int half = hd / 2;
    const int row = (nq + 2 * nkv) * hd;
    float *base = qkv + (int64_t)b * row;
    const int npairs = (nq + nkv) * half;
    const int64_t cache_row = ((int64_t)b * max_ctx + pos) * (int64_t)(nkv * hd);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npairs + nkv * hd; i += gridDim.x * blockDim.x) {
        if (i < npairs) {
            const int head = i / half, d = i - head * half;  // heads 0..nq-1 are q, then nkv k heads
            float *p = base + head * hd;
            const float c = cos_t[(int64_t)pos * half + d], s = sin_t[(int64_t)pos * half + d];
            const float a = p[d], bb = p[d + half];
            const float r1 = a * c - bb * s, r2 = a * s + bb * c;
            p[d] = r1;
            p[d + half] = r2;
            if (head >= nq) {
                float *kdst = kc + cache_row + (head - nq) * hd;
                kdst[d] = r1;
                kdst[d + half] = r2;
            }
        } else {
            const int j = i - npairs;  // v values
            vc[cache_row + j] = base[(nq + nkv) * hd + j];
        }
    }
}

// Element d of head vector v (hd values) rotated to position `pos`, half-split pairs (d, d + hd/2),
// the same expression as rope_store_kv_kernel; cos/sin tables are [max_ctx][hd/2].
__device__ __forceinline__ float rope_elem(const float *__restrict__ v, int d, int hd, const float *__restrict__ cos_t,
                                           const float *__restrict__ sin_t, int pos) {
    const int half = hd >> 1;
    if (d < half) {
        const float c = cos_t[(int64_t)pos * half + d], s = sin_t[(int64_t)pos * half + d];
        return v[d] * c - v[d + half] * s;
    }
    const float c = cos_t[(int64_t)pos * half + d - half], s = sin_t[(int64_t)pos * half + d - half];
    return v[d - half] * s + v[d] * c;
}

// ---- prompt phase: the rotary step for T consecutive positions of one sequence -----------------------------
// qkv: [T, (nq + 2 nkv) * hd] f32, row t belongs to position pos0 + t.  The same arithmetic as
// rope_store_kv_kernel per row: q and k rotated (half-split pairs), rotated k and plain v stored to the f32 caches
// [max_ctx][nkv * hd] at their positions -- what the decode kernels read afterwards -- and, for the tensor-core
// attention of the prompt itself, 16-bit copies (f16 or bf16, round to nearest even) of rotated q [T][nq * hd],
// rotated k [T][nkv * hd] and v [T][nkv * hd].
template <bool BF16>
__device__ __forceinline__ uint16_t to16(float v) {
    if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    return __half_as_ushort(__float2half_rn(v));
}
template <bool BF16>
__global__ void __launch_bounds__(256) rope_prefill_kernel(const float *__restrict__ qkv, int T, int nq, int nkv, int hd, const float *__restrict__ cos_t,
                                                         const float *__restrict__ sin_t, int pos0, float *__restrict__ kc, float *__restrict__ vc,
                                                         uint16_t *__restrict__ q16, uint16_t *__restrict__ k16, uint16_t *__restrict__ v16) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int t = blockIdx.y;
    const int pos = pos0 + t;
    const int half = hd / 2;
    const int row = (nq + 2 * nkv) * hd;
    const float *base = qkv + (int64_t)t * row;
    const int npairs = (nq + nkv) * half;
    const int64_t cache_row = (int64_t)pos * (int64_t)(nkv * hd);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < npairs + nkv * hd; i += gridDim.x * blockDim.x) {
        if (i < npairs) {
            const int head = i / half, d = i - head * half;  // heads 0..nq-1 are q, then nkv k heads
            const float *p = base + head * hd;
            const float c = cos_t[(int64_t)pos * half + d], s = sin_t[(int64_t)pos * half + d];
            const float a = p[d], bb = p[d + half];
            const float r1 = a * c - bb * s, r2 = a * s + bb * c;
            if (head < nq) {
                uint16_t *dst = q16 + ((int64_t)t * nq + head) * hd;
                dst[d] = to16<BF16>(r1);
                dst[d + half] = to16<BF16>(r2);
            } else {
                float *kdst = kc + cache_row + (head - nq) * hd;
                kdst[d] = r1;
                kdst[d + half] = r2;
                uint16_t *dst = k16 + ((int64_t)t * nkv + (head - nq)) * hd;
                dst[d] = to16<BF16>(r1);
                dst[d + half] = to16<BF16>(r2);
            }
        } else {
            const int j = i - npairs;  // v values
            const float v = base[(nq + nkv) * hd + j];
            vc[cache_row + j] = v;
            v16[(int64_t)t * nkv * hd + j] = to16<BF16>(v);
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(256) cast_f32_to_16_kernel(const float *__restrict__ src, int64_t n, uint16_t *__restrict__ dst) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = to16<BF16>(src[i]);
}

template <bool BF16>
__global__ void __launch_bounds__(256) cast16_to_f32_kernel(const uint16_t *__restrict__ src, int64_t n, float *__restrict__ dst) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = BF16 ? __bfloat162float(__ushort_as_bfloat16(src[i])) : __half2float(__ushort_as_half(src[i]));
}

constexpr int kAttnChunk = 32;    // keys per CTA: short chunks keep many CTAs in flight at small contexts
constexpr int kAttnThreads = 128;

// One CTA per (query head, sequence, chunk of 32 keys): scores, chunk-local softmax numerators
// and the weighted sum of V; writes (max, sum, acc[hd]) for the combine kernel.  hd <= 256 and a
// multiple of 4.  Latency-bound (a few hundred KB per CTA out of L2/HBM), so every loop keeps
// eight independent loads in flight.
// With cos_t / sin_t given the kernel also does the rotary step: q is rotated as it is loaded, and the
// newest key (position *pos, not yet in the cache) is taken from qkv -- rotated k, plain v -- by the
// chunk that holds it; the first head of each kv group stores it to the caches (kc_w / vc_w).
__global__ void __launch_bounds__(kAttnThreads) attn_partial_kernel(const float *__restrict__ qkv, int nq, int nkv, int hd,
                                                                  const int *__restrict__ pos_dev, const float *kc,
                                                                  const float *vc, int max_ctx, float scale,
                                                                  float *__restrict__ part, int nchunks, const float *__restrict__ cos_t,
                                                                  const float *__restrict__ sin_t, float *kc_w, float *vc_w, int *err) {
    __shared__ float p_s[kAttnChunk];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int head = blockIdx.x, b = blockIdx.y, chunk = blockIdx.z;
    const int nkeys = checked_pos(pos_dev, max_ctx, err) + 1;
    const int t0 = chunk * kAttnChunk;
    float *out = part + (((int64_t)b * nq + head) * nchunks + chunk) * (hd + 2);
    if (t0 >= nkeys) {  // chunk beyond the current length: neutral element
        if (threadIdx.x == 0) {
            out[0] = -3.402823466e38f;
            out[1] = 0.0f;
        }
        for (int d = threadIdx.x; d < hd; d += blockDim.x) out[2 + d] = 0.0f;
        return;
    }
    const int t1 = min(t0 + kAttnChunk, nkeys);
    const int cnt = t1 - t0;
    const int kvh = head / (nq / nkv);
    const int row = (nq + 2 * nkv) * hd;
    const float *q = qkv + (int64_t)b * row + head * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t kv_stride = (int64_t)nkv * hd;
    const float *kbase = kc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    const float *vbase = vc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    // Every global load of the CTA is issued before the first use: q, this warp's 8 keys, and (for
    // hd <= 128) this thread's 32 values of V.  One memory round trip instead of one per phase.
    float4 kreg[8][2];
    float4 qreg[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int d = lane * 4 + 128 * h2;
        qreg[h2] = (d < hd) ? *reinterpret_cast<const float4 *>(q + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (cos_t && d < hd)
            qreg[h2] = make_float4(rope_elem(q, d, hd, cos_t, sin_t, nkeys - 1), rope_elem(q, d + 1, hd, cos_t, sin_t, nkeys - 1),
                                   rope_elem(q, d + 2, hd, cos_t, sin_t, nkeys - 1), rope_elem(q, d + 3, hd, cos_t, sin_t, nkeys - 1));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = t0 + warp * 8 + j;
            const bool newest = cos_t && t == nkeys - 1;  // not in the cache yet: comes from qkv
            kreg[j][h2] = (t < t1 && d < hd && !newest) ? *reinterpret_cast<const float4 *>(kbase + (int64_t)t * kv_stride + d)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
            if (newest && d < hd) {
                const float *kn = qkv + (int64_t)b * row + (nq + kvh) * hd;
                kreg[j][h2] = make_float4(rope_elem(kn, d, hd, cos_t, sin_t, t), rope_elem(kn, d + 1, hd, cos_t, sin_t, t),
                                          rope_elem(kn, d + 2, hd, cos_t, sin_t, t), rope_elem(kn, d + 3, hd, cos_t, sin_t, t));
                if (head % (nq / nkv) == 0)
                    *reinterpret_cast<float4 *>(kc_w + ((int64_t)b * max_ctx + t) * kv_stride + kvh * hd + d) = kreg[j][h2];
            }
        }
    }
    const float *vnew = qkv + (int64_t)b * row + (nq + nkv + kvh) * hd;  // newest value row, straight from qkv
    float vreg[kAttnChunk];
    const bool v_in_regs = hd <= kAttnThreads;
    if (v_in_regs) {
#pragma unroll
        for (int j = 0; j < kAttnChunk; ++j) {
            const bool newest = cos_t && t0 + j == nkeys - 1;
            vreg[j] = (j < cnt && (int)threadIdx.x < hd) ? (newest ? vnew[threadIdx.x] : vbase[(int64_t)(t0 + j) * kv_stride + threadIdx.x]) : 0.0f;
        }
    }
    if (cos_t && t1 == nkeys && head % (nq / nkv) == 0)  // this chunk holds the newest key: its value row goes to the cache
        for (int d = threadIdx.x; d < hd; d += blockDim.x) vc_w[((int64_t)b * max_ctx + nkeys - 1) * kv_stride + kvh * hd + d] = vnew[d];
    {
        float s[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j] = 0.0f;
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
                s[j] = fmaf(qreg[h2].x, kreg[j][h2].x,
                            fmaf(qreg[h2].y, kreg[j][h2].y, fmaf(qreg[h2].z, kreg[j][h2].z, fmaf(qreg[h2].w, kreg[j][h2].w, s[j]))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o, 32);
        if (lane < 8) {
            float v = s[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) v = (lane == j) ? s[j] : v;
            p_s[warp * 8 + lane] = v * scale;
        }
    }
    __syncthreads();
    // chunk softmax numerators: every warp computes the same max / sum over the 32 scores
    const float sc = (lane < cnt) ? p_s[lane] : -3.402823466e38f;
    const float m = warp_max(sc);
    const float e = (lane < cnt) ? expf(sc - m) : 0.0f;
    const float l = warp_sum(e);
    __syncthreads();
    if (warp == 0) p_s[lane] = e;
    __syncthreads();
    if (v_in_regs) {
        if ((int)threadIdx.x < hd) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < kAttnChunk; ++j) acc[j & 3] = fmaf(p_s[j], vreg[j], acc[j & 3]);
            out[2 + threadIdx.x] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
    } else {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
            for (int tb = 0; tb < cnt; tb += 8) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (tb + j < cnt)
                        acc[j] = fmaf(p_s[tb + j], (cos_t && t0 + tb + j == nkeys - 1) ? vnew[d] : vbase[(int64_t)(t0 + tb + j) * kv_stride + d], acc[j]);
            }
            out[2 + d] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        }
    }
    if (threadIdx.x == 0) {
        out[0] = m;
        out[1] = l;
    }
}

// ---- decode attention in ONE launch for short contexts: a cluster of eight CTAs per (head, sequence) --------------
// CTA `rank` of the cluster takes the 32-key chunks rank, rank + 8, ... of the context (the arithmetic of
// attn_partial_kernel per chunk, merged into a running maximum / sum / weighted sum), leaves its partial in its own
// shared memory, and after one cluster barrier rank 0 reads the eight partials through distributed shared memory,
// merges them in rank order and writes the normalised output: no partials in global memory, no second kernel.
// head_dim <= 128 (thread = dim).  With cos_t / sin_t the rotary step is fused as in attn_partial_kernel.
constexpr int kAttnCluster = 8;
__global__ void __launch_bounds__(kAttnThreads) attn_cluster_kernel(const float *__restrict__ qkv, int nq, int nkv, int hd,
                                                                  const int *__restrict__ pos_dev, const float *kc, const float *vc, int max_ctx,
                                                                  float scale, float *__restrict__ out, const float *__restrict__ cos_t,
                                                                  const float *__restrict__ sin_t, float *kc_w, float *vc_w, int *err) {
    namespace cg = cooperative_groups;
    __shared__ float p_s[kAttnChunk];
    __shared__ float part_s[kAttnThreads + 2];  // (max, sum, weighted sum per dim) of this CTA's chunks
    pdl_launch_dependents();
    pdl_wait_prior();
    cg::cluster_group cluster = cg::this_cluster();
    const int head = blockIdx.x, b = blockIdx.y, rank = blockIdx.z;  // the cluster spans z
    const int nkeys = checked_pos(pos_dev, max_ctx, err) + 1;
    const int nchunks = (nkeys + kAttnChunk - 1) / kAttnChunk;
    const int kvh = head / (nq / nkv);
    const int row = (nq + 2 * nkv) * hd;
    const float *q = qkv + (int64_t)b * row + head * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t kv_stride = (int64_t)nkv * hd;
    const float *kbase = kc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    const float *vbase = vc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    const float *vnew = qkv + (int64_t)b * row + (nq + nkv + kvh) * hd;  // newest value row, straight from qkv
    float4 qreg;
    {
        const int d = lane * 4;
        qreg = (d < hd) ? *reinterpret_cast<const float4 *>(q + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (cos_t && d < hd)
            qreg = make_float4(rope_elem(q, d, hd, cos_t, sin_t, nkeys - 1), rope_elem(q, d + 1, hd, cos_t, sin_t, nkeys - 1),
                               rope_elem(q, d + 2, hd, cos_t, sin_t, nkeys - 1), rope_elem(q, d + 3, hd, cos_t, sin_t, nkeys - 1));
    }
    float m_run = -3.402823466e38f, l_run = 0.0f, acc_run = 0.0f;
    for (int chunk = rank; chunk < nchunks; chunk += kAttnCluster) {
        const int t0 = chunk * kAttnChunk;
        const int t1 = min(t0 + kAttnChunk, nkeys);
        const int cnt = t1 - t0;
        // every global load of the chunk is issued before the first use: this warp's 8 keys and this thread's 32 values of V
        float4 kreg[8];
        const int d4 = lane * 4;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int t = t0 + warp * 8 + j;
            const bool newest = cos_t && t == nkeys - 1;  // not in the cache yet: comes from qkv
            kreg[j] = (t < t1 && d4 < hd && !newest) ? *reinterpret_cast<const float4 *>(kbase + (int64_t)t * kv_stride + d4) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (newest && d4 < hd) {
                const float *kn = qkv + (int64_t)b * row + (nq + kvh) * hd;
                kreg[j] = make_float4(rope_elem(kn, d4, hd, cos_t, sin_t, t), rope_elem(kn, d4 + 1, hd, cos_t, sin_t, t),
                                      rope_elem(kn, d4 + 2, hd, cos_t, sin_t, t), rope_elem(kn, d4 + 3, hd, cos_t, sin_t, t));
                if (head % (nq / nkv) == 0) *reinterpret_cast<float4 *>(kc_w + ((int64_t)b * max_ctx + t) * kv_stride + kvh * hd + d4) = kreg[j];
            }
        }
        float vreg[kAttnChunk];
#pragma unroll
        for (int j = 0; j < kAttnChunk; ++j) {
            const bool newest = cos_t && t0 + j == nkeys - 1;
            vreg[j] = (j < cnt && (int)threadIdx.x < hd) ? (newest ? vnew[threadIdx.x] : vbase[(int64_t)(t0 + j) * kv_stride + threadIdx.x]) : 0.0f;
        }
        if (cos_t && t1 == nkeys && head % (nq / nkv) == 0)  // this chunk holds the newest key: its value row goes to the cache
            for (int d = threadIdx.x; d < hd; d += blockDim.x) vc_w[((int64_t)b * max_ctx + nkeys - 1) * kv_stride + kvh * hd + d] = vnew[d];
        {
            float sc8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                sc8[j] = fmaf(qreg.x, kreg[j].x, fmaf(qreg.y, kreg[j].y, fmaf(qreg.z, kreg[j].z, qreg.w * kreg[j].w)));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int j = 0; j < 8; ++j) sc8[j] += __shfl_xor_sync(0xffffffffu, sc8[j], o, 32);
            if (lane < 8) {
                float v = sc8[0];
#pragma unroll
                for (int j = 1; j < 8; ++j) v = (lane == j) ? sc8[j] : v;
                p_s[warp * 8 + lane] = v * scale;
            }
        }
        __syncthreads();
        // chunk softmax numerators: every warp computes the same max / sum over the 32 scores
        const float sc = (lane < cnt) ? p_s[lane] : -3.402823466e38f;
        const float m = warp_max(sc);
        const float e = (lane < cnt) ? expf(sc - m) : 0.0f;
        const float l = warp_sum(e);
        __syncthreads();
        if (warp == 0) p_s[lane] = e;
        __syncthreads();
        float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < kAttnChunk; ++j) acc4[j & 3] = fmaf(p_s[j], vreg[j], acc4[j & 3]);
        const float acc = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
        // merge into the running partial
        const float m_new = fmaxf(m_run, m);
        const float f_old = expf(m_run - m_new), f_new = expf(m - m_new);
        l_run = l_run * f_old + l * f_new;
        acc_run = acc_run * f_old + acc * f_new;
        m_run = m_new;
        __syncthreads();  // p_s is rewritten by the next chunk
    }
    if (threadIdx.x == 0) part_s[0] = m_run, part_s[1] = l_run;
    part_s[2 + threadIdx.x] = acc_run;
    cluster.sync();
    if (rank == 0 && (int)threadIdx.x < hd) {
        float m = -3.402823466e38f, l = 0.0f, acc = 0.0f;
        for (int r = 0; r < kAttnCluster; ++r) {
            const float *ps = cluster.map_shared_rank(part_s, r);
            const float mr = ps[0], lr = ps[1], ar = ps[2 + threadIdx.x];
            const float m_new = fmaxf(m, mr);
            const float f_old = expf(m - m_new), f_r = expf(mr - m_new);
            l = l * f_old + lr * f_r;
            acc = acc * f_old + ar * f_r;
            m = m_new;
        }
        out[((int64_t)b * nq + head) * hd + threadIdx.x] = acc / l;
    }
    cluster.sync();  // the partials are read out of the other CTAs' shared memory: nobody leaves before that
}

// Grouped-query variant: one CTA per (kv head, sequence, chunk of 32 keys) serves all G = nq/nkv
// query heads of the group, so a K/V chunk is read from memory once instead of G times.  K is
// staged transposed in shared memory (lane = key, conflict-free), V row-major (thread = dim).
// hd == 128, G <= 8.  Same partial layout as attn_partial_kernel.
constexpr int kGqaMaxG = 8;
__global__ void __launch_bounds__(128) attn_partial_gqa_kernel(const float *__restrict__ qkv, int nq, int nkv, const int *__restrict__ pos_dev,
                                                             const float *__restrict__ kc, const float *__restrict__ vc, int max_ctx,
                                                             float scale, float *__restrict__ part, int nchunks, int *err) {
    constexpr int hd = 128;
    __shared__ float kt_s[hd][kAttnChunk + 1];       // K transposed, padded
    __shared__ float v_s[kAttnChunk][hd];
    __shared__ float q_s[kGqaMaxG][hd];
    __shared__ float p_s[kGqaMaxG][kAttnChunk];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int kvh = blockIdx.x, b = blockIdx.y, chunk = blockIdx.z;
    const int G = nq / nkv;
    const int nkeys = checked_pos(pos_dev, max_ctx, err) + 1;
    const int t0 = chunk * kAttnChunk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (t0 >= nkeys) {
        for (int g = 0; g < G; ++g) {
            float *out = part + (((int64_t)b * nq + kvh * G + g) * nchunks + chunk) * (hd + 2);
            if (tid == 0) out[0] = -3.402823466e38f, out[1] = 0.0f;
            out[2 + tid] = 0.0f;
        }
        return;
    }
    const int cnt = min(kAttnChunk, nkeys - t0);
    const int row = (nq + 2 * nkv) * hd;
    const int64_t kv_stride = (int64_t)nkv * hd;
    const float *kbase = kc + ((int64_t)b * max_ctx + t0) * kv_stride + kvh * hd;
    const float *vbase = vc + ((int64_t)b * max_ctx + t0) * kv_stride + kvh * hd;
    // all global loads first: 32 K values and 32 V values per thread (thread = dim), plus q
    float kreg[kAttnChunk], vreg[kAttnChunk];
#pragma unroll
    for (int t = 0; t < kAttnChunk; ++t) {
        kreg[t] = (t < cnt) ? kbase[(int64_t)t * kv_stride + tid] : 0.0f;
        vreg[t] = (t < cnt) ? vbase[(int64_t)t * kv_stride + tid] : 0.0f;
    }
    for (int g = 0; g < G; ++g) q_s[g][tid] = qkv[(int64_t)b * row + (kvh * G + g) * hd + tid];
#pragma unroll
    for (int t = 0; t < kAttnChunk; ++t) {
        kt_s[tid][t] = kreg[t];
        v_s[t][tid] = vreg[t];
    }
    __syncthreads();
    // scores: warp w takes heads w, w+4; lane = key
    for (int g = warp; g < G; g += 4) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 8
        for (int d = 0; d < hd; d += 4) {
            s0 = fmaf(q_s[g][d], kt_s[d][lane], s0);
            s1 = fmaf(q_s[g][d + 1], kt_s[d + 1][lane], s1);
            s2 = fmaf(q_s[g][d + 2], kt_s[d + 2][lane], s2);
            s3 = fmaf(q_s[g][d + 3], kt_s[d + 3][lane], s3);
        }
        const float sc = (lane < cnt) ? ((s0 + s1) + (s2 + s3)) * scale : -3.402823466e38f;
        const float m = warp_max(sc);
        const float e = (lane < cnt) ? expf(sc - m) : 0.0f;
        const float l = warp_sum(e);
        p_s[g][lane] = e;
        if (lane == 0) {
            float *out = part + (((int64_t)b * nq + kvh * G + g) * nchunks + chunk) * (hd + 2);
            out[0] = m;
            out[1] = l;
        }
    }
    __syncthreads();
    // weighted V: thread = dim, all heads of the group from the same staged V
    for (int g = 0; g < G; ++g) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int t = 0; t < kAttnChunk; t += 4) {
            a0 = fmaf(p_s[g][t], v_s[t][tid], a0);
            a1 = fmaf(p_s[g][t + 1], v_s[t + 1][tid], a1);
            a2 = fmaf(p_s[g][t + 2], v_s[t + 2][tid], a2);
            a3 = fmaf(p_s[g][t + 3], v_s[t + 3][tid], a3);
        }
        part[(((int64_t)b * nq + kvh * G + g) * nchunks + chunk) * (hd + 2) + 2 + tid] = (a0 + a1) + (a2 + a3);
    }
}

// Split-context grouped-query decode attention, hd == 128, G = nq/nkv <= 8.  One CTA per
// (split of the context, kv head, sequence) walks its keys 64 at a time with a running softmax
// and serves all G query heads of the group from one pass over K and V:
//   load    64 keys and values into shared memory with 16-byte async copies (K rows padded to
//           132 floats so that lane = key reads are conflict-free);
//   scores  warp = quarter of the 128 dims, lane = keys (lane, lane+32): 2 x 8 accumulators,
//           ten 16-byte shared loads per 64 FMAs; the four dim-quarters are summed through
//           shared memory;
//   softmax warp w owns heads 2w, 2w+1: running max and sum in registers, numerators and the
//           rescaling factor to shared memory;
//   values  warp = quarter of the 64 keys, lane = four dims: 8 x 4 accumulators kept in
//           registers across the whole split, three 16-byte shared loads per 32 FMAs.
// Writes (max, sum, acc[128]) per (head, split) in the layout the combine kernel reads.
constexpr int kAttn2Keys = 64;
constexpr int kAttn2KStride = 132;
constexpr size_t kAttn2Smem = (size_t)kAttn2Keys * kAttn2KStride * 4 + (size_t)kAttn2Keys * 128 * 4  // K, V
                              + 8 * 128 * 4                                                          // q
                              + 4 * 8 * kAttn2Keys * 4                                               // score partials [warp][head][key]
                              + kAttn2Keys * 8 * 4 + 64;                                             // numerators [key][head], factors
template <bool ROPE>
__global__ void __launch_bounds__(128) attn_split_gqa_kernel(const float *__restrict__ qkv, int nq, int nkv, const int *__restrict__ pos_dev,
                                                           const float *kc, const float *vc, int max_ctx, float scale,
                                                           float *__restrict__ part, int nsplits, int keys_per_split,
                                                           const float *__restrict__ cos_t, const float *__restrict__ sin_t, float *kc_w,
                                                           float *vc_w, int *err) {
    constexpr int hd = 128;
    extern __shared__ __align__(16) uint8_t attn_smem[];
    float *Ks = reinterpret_cast<float *>(attn_smem);
    float *Vs = Ks + kAttn2Keys * kAttn2KStride;
    float *q_s = Vs + kAttn2Keys * hd;
    float *sp_s = q_s + 8 * hd;                  // [4][8][64]
    float *p_s = sp_s + 4 * 8 * kAttn2Keys;      // [64][8]
    float *alpha_s = p_s + kAttn2Keys * 8;       // [8]
    pdl_launch_dependents();
    pdl_wait_prior();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int G = nq / nkv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkeys = checked_pos(pos_dev, max_ctx, err) + 1;
    const int t_begin = split * keys_per_split;
    const int t_end = min(t_begin + keys_per_split, nkeys);
    const int stride = hd + 2;
    if (t_begin >= t_end) {  // split beyond the current length: neutral element
        for (int g = 0; g < G; ++g) {
            float *out = part + (((int64_t)b * nq + kvh * G + g) * nsplits + split) * stride;
            if (tid == 0) out[0] = -3.402823466e38f, out[1] = 0.0f;
            out[2 + tid] = 0.0f;
        }
        return;
    }
    const int row = (nq + 2 * nkv) * hd;
    const int64_t kv_stride = (int64_t)nkv * hd;
    const float *kbase = kc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    const float *vbase = vc + ((int64_t)b * max_ctx) * kv_stride + kvh * hd;
    // q of the group's heads (rotated here when the rotary step is fused in: cos_t given)
    for (int i = tid; i < 8 * hd; i += 128) {
        const float *qh = qkv + (int64_t)b * row + (kvh * G + i / hd) * hd;
        q_s[i] = (i / hd) < G ? (ROPE ? rope_elem(qh, i % hd, hd, cos_t, sin_t, nkeys - 1) : qh[i % hd]) : 0.0f;
    }

    float m_run[2] = {-3.402823466e38f, -3.402823466e38f}, l_run[2] = {0.0f, 0.0f};  // heads 2*warp, 2*warp+1 (lane-uniform)
    float acc[8][4];
#pragma unroll
    for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[g][i] = 0.0f;

    // 64 rows of K (or V) starting at key t0 into shared memory, as one async-copy group; rows past
    // the end become zeros, so that no stale NaN reaches a product with a zero weight.  A warp copies
    // one 512-byte row per instruction.
    auto load_rows = [&](const float *base, float *dst, int dst_stride, int t0) {
        const int cnt = min(kAttn2Keys, t_end - t0);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int f = tid + 128 * j, r = f >> 5, c4 = f & 31;
            float *d = dst + r * dst_stride + 4 * c4;
            if (ROPE && r < cnt && t0 + r == nkeys - 1) {
                // the newest key is not in the cache yet: rotated k / plain v come from qkv, and this CTA
                // (the only one of its kv head and sequence that sees this row) stores them to the cache
                const bool is_k = base == kbase;
                const float *src = qkv + (int64_t)b * row + (nq + (is_k ? 0 : nkv) + kvh) * hd;
                float4 v4;
                if (is_k) v4 = make_float4(rope_elem(src, 4 * c4, hd, cos_t, sin_t, t0 + r), rope_elem(src, 4 * c4 + 1, hd, cos_t, sin_t, t0 + r),
                                           rope_elem(src, 4 * c4 + 2, hd, cos_t, sin_t, t0 + r), rope_elem(src, 4 * c4 + 3, hd, cos_t, sin_t, t0 + r));
                else v4 = *reinterpret_cast<const float4 *>(src + 4 * c4);
                *reinterpret_cast<float4 *>(d) = v4;
                *reinterpret_cast<float4 *>((is_k ? kc_w : vc_w) + ((int64_t)b * max_ctx + t0 + r) * kv_stride + kvh * hd + 4 * c4) = v4;
            } else if (r < cnt) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(d)),
                             "l"(base + (int64_t)(t0 + r) * kv_stride + 4 * c4)
                             : "memory");
            } else {
                *reinterpret_cast<float4 *>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Software pipeline over two buffers: K of the next chunk streams in during this chunk's softmax
    // and value pass, V of the next chunk during the next chunk's scores.
    load_rows(kbase, Ks, kAttn2KStride, t_begin);
    load_rows(vbase, Vs, hd, t_begin);
    for (int t0 = t_begin; t0 < t_end; t0 += kAttn2Keys) {
        const int cnt = min(kAttn2Keys, t_end - t0);
        const bool more = t0 + kAttn2Keys < t_end;
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // K of this chunk has landed (V may still be in flight)
        __syncthreads();
        // ---- scores: this warp's 32 dims, keys lane and lane+32, all eight heads --------------------
        {
            float s[2][8];
#pragma unroll
            for (int g = 0; g < 8; ++g) s[0][g] = 0.0f, s[1][g] = 0.0f;
            const float *k0 = Ks + lane * kAttn2KStride + 32 * warp, *k1 = k0 + 32 * kAttn2KStride;
            const float *qw = q_s + 32 * warp;
#pragma unroll
            for (int d4 = 0; d4 < 8; ++d4) {
                const float4 a = *reinterpret_cast<const float4 *>(k0 + 4 * d4), c = *reinterpret_cast<const float4 *>(k1 + 4 * d4);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 q = *reinterpret_cast<const float4 *>(qw + g * hd + 4 * d4);
                    s[0][g] = fmaf(q.x, a.x, fmaf(q.y, a.y, fmaf(q.z, a.z, fmaf(q.w, a.w, s[0][g]))));
                    s[1][g] = fmaf(q.x, c.x, fmaf(q.y, c.y, fmaf(q.z, c.z, fmaf(q.w, c.w, s[1][g]))));
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                sp_s[(warp * 8 + g) * kAttn2Keys + lane] = s[0][g];
                sp_s[(warp * 8 + g) * kAttn2Keys + lane + 32] = s[1][g];
            }
        }
        __syncthreads();
        if (more) load_rows(kbase, Ks, kAttn2KStride, t0 + kAttn2Keys);  // K buffer is free
        else asm volatile("cp.async.commit_group;" ::: "memory");         // keep the group count uniform
        // ---- running softmax: warp w owns heads 2w and 2w+1 ------------------------------------------
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int g = 2 * warp + hh;
            float sc[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int t = lane + 32 * half;
                const float v = (sp_s[(0 * 8 + g) * kAttn2Keys + t] + sp_s[(1 * 8 + g) * kAttn2Keys + t]) +
                                (sp_s[(2 * 8 + g) * kAttn2Keys + t] + sp_s[(3 * 8 + g) * kAttn2Keys + t]);
                sc[half] = t < cnt ? v * scale : -3.402823466e38f;
            }
            const float m_new = fmaxf(m_run[hh], warp_max(fmaxf(sc[0], sc[1])));
            const float e0 = lane < cnt ? expf(sc[0] - m_new) : 0.0f;
            const float e1 = lane + 32 < cnt ? expf(sc[1] - m_new) : 0.0f;
            const float a = expf(m_run[hh] - m_new);  // 0 on the first chunk
            l_run[hh] = l_run[hh] * a + warp_sum(e0 + e1);
            m_run[hh] = m_new;
            p_s[lane * 8 + g] = e0;
            p_s[(lane + 32) * 8 + g] = e1;
            if (lane == 0) alpha_s[g] = a;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // V of this chunk has landed (the next K may still be in flight)
        __syncthreads();
        // ---- values: this warp's 16 keys, dims 4*lane .. 4*lane+3, all eight heads ---------------------
        {
            const float4 a0 = *reinterpret_cast<const float4 *>(alpha_s), a1 = *reinterpret_cast<const float4 *>(alpha_s + 4);
            const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int g = 0; g < 8; ++g)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[g][i] *= al[g];
#pragma unroll 4
            for (int tt = 0; tt < 16; ++tt) {
                const int t = 16 * warp + tt;
                const float4 v = *reinterpret_cast<const float4 *>(Vs + t * hd + 4 * lane);
                const float4 p0 = *reinterpret_cast<const float4 *>(p_s + t * 8), p1 = *reinterpret_cast<const float4 *>(p_s + t * 8 + 4);
                const float pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    acc[g][0] = fmaf(pw[g], v.x, acc[g][0]);
                    acc[g][1] = fmaf(pw[g], v.y, acc[g][1]);
                    acc[g][2] = fmaf(pw[g], v.z, acc[g][2]);
                    acc[g][3] = fmaf(pw[g], v.w, acc[g][3]);
                }
            }
        }
        __syncthreads();
        if (more) load_rows(vbase, Vs, hd, t0 + kAttn2Keys);  // V buffer is free
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ---- the four key-quarters' accumulators are summed through shared memory (K region) ---------
    __syncthreads();
    float *red = Ks;  // [4][8][128]
#pragma unroll
    for (int g = 0; g < 8; ++g) *reinterpret_cast<float4 *>(red + (warp * 8 + g) * hd + 4 * lane) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    if (lane == 0) {
        alpha_s[2 * warp] = m_run[0], alpha_s[2 * warp + 1] = m_run[1];
        p_s[2 * warp] = l_run[0], p_s[2 * warp + 1] = l_run[1];
    }
    __syncthreads();
    for (int g = 0; g < G; ++g) {
        float *out = part + (((int64_t)b * nq + kvh * G + g) * nsplits + split) * stride;
        out[2 + tid] = (red[(0 * 8 + g) * hd + tid] + red[(1 * 8 + g) * hd + tid]) + (red[(2 * 8 + g) * hd + tid] + red[(3 * 8 + g) * hd + tid]);
        if (tid == 0) out[0] = alpha_s[g], out[1] = p_s[g];
    }
}

// Combines the chunk partials of one (head, sequence): out[b][head*hd + d].  Lane = four
// consecutive dims, the four warps take every fourth chunk; all loads of a batch of eight chunks
// are unconditional (clamped index, zero weight past the end) so they are in flight together.
__global__ void __launch_bounds__(128) attn_combine_kernel(const float *__restrict__ part, int nq, int hd, int nchunks,
                                                         float *__restrict__ out) {
    __shared__ float w_s[512];  // per-chunk weight exp(m_c - m); nchunks <= 512 (context <= 16384)
    __shared__ float red[32];
    __shared__ float4 acc_s[4][64];  // per-warp partial sums, hd <= 256
    pdl_launch_dependents();
    pdl_wait_prior();
    const int head = blockIdx.x, b = blockIdx.y;
    const int stride = hd + 2;
    const float *p = part + (((int64_t)b * nq + head) * nchunks) * stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    // chunk maxima and sums: one (m, l) pair per thread per trip, both loads issued together
    float m = -3.402823466e38f;
    float mc[4], lc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 128;
        const int cc = c < nchunks ? c : nchunks - 1;
        mc[i] = p[(int64_t)cc * stride];
        lc[i] = p[(int64_t)cc * stride + 1];
        if (c >= nchunks) mc[i] = -3.402823466e38f, lc[i] = 0.0f;
        m = fmaxf(m, mc[i]);
    }
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = (lane < nw) ? red[lane] : -3.402823466e38f;
    m = warp_max(m);
    __syncthreads();
    float l = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 128;
        const float w = (c < nchunks) ? expf(mc[i] - m) : 0.0f;
        if (c < nchunks) w_s[c] = w;
        l = fmaf(w, lc[i], l);
    }
    l = block_sum(l, red);  // has the barriers that publish w_s
    const float inv = 1.0f / l;
    for (int d0 = 0; d0 < hd; d0 += 128) {
        const int d = d0 + lane * 4;
        const bool live = d < hd;
        const float *pd = p + 2 + (live ? d : 0);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c0 = warp; c0 < nchunks; c0 += 32) {
            float a[8][4];
            float w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = c0 + 4 * j;
                const int cc = c < nchunks ? c : nchunks - 1;
                const float *q = pd + (int64_t)cc * stride;  // rows start 8 bytes past a 16-byte boundary: two 8-byte loads
                const float2 lo = *reinterpret_cast<const float2 *>(q), hi = *reinterpret_cast<const float2 *>(q + 2);
                a[j][0] = lo.x, a[j][1] = lo.y, a[j][2] = hi.x, a[j][3] = hi.y;
                w[j] = c < nchunks ? w_s[c] : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc.x = fmaf(a[j][0], w[j], acc.x);
                acc.y = fmaf(a[j][1], w[j], acc.y);
                acc.z = fmaf(a[j][2], w[j], acc.z);
                acc.w = fmaf(a[j][3], w[j], acc.w);
            }
        }
        acc_s[warp][(d0 >> 2) + lane] = acc;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        const float *f = reinterpret_cast<const float *>(&acc_s[0][0]);
        const float v = (f[d] + f[256 + d]) + (f[512 + d] + f[768 + d]);
        out[((int64_t)b * nq + head) * hd + d] = v * inv;
    }
}

// out[b][i] = silu(gu[b][i]) * gu[b][n + i]; silu evaluated in f64 like USiluF32.
__global__ void __launch_bounds__(256) silu_mul_kernel(const float *__restrict__ gu, int n, int64_t total, float *__restrict__ out,
                                                     int64_t ld_out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n, c = i - b * n;
        const double g = (double)gu[b * 2 * n + c];
        const float s = (float)(g / (1.0 + exp(-g)));
        out[b * ld_out + c] = s * gu[b * 2 * n + n + c];
    }
}

// The same on (gate, up) pairs: out[b][i] = silu(gu[b][2i]) * gu[b][2i + 1].
__global__ void __launch_bounds__(256) silu_mul_pairs_kernel(const float *__restrict__ gu, int n, int64_t total, float *__restrict__ out,
                                                           int64_t ld_out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n, c = i - b * n;
        const float2 v = *reinterpret_cast<const float2 *>(gu + b * 2 * n + 2 * c);
        const double g = (double)v.x;
        out[b * ld_out + c] = (float)(g / (1.0 + exp(-g))) * v.y;
    }
}

// One CTA per row; the lowest index among equal maxima wins, as the sequential strict '>' does.
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ x, int cols, uint32_t *__restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait_prior();
    const float *xr = x + (int64_t)blockIdx.x * cols;
    float best = -3.402823466e38f;
    int bi = 0x7FFFFFFF;
    if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0 && cols <= 8 * 4 * (int)blockDim.x) {
        // up to 8 float4 per thread, all loads issued before the first compare; a thread's elements
        // are visited in increasing index order, so strict '>' keeps the lowest index of its maxima
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = (i * blockDim.x + threadIdx.x) * 4;
            v[i] = (c + 3 < cols) ? *reinterpret_cast<const float4 *>(xr + c) : make_float4(-3.402823466e38f, -3.402823466e38f, -3.402823466e38f, -3.402823466e38f);
            if (c < cols && c + 3 >= cols) {  // ragged tail
                v[i].x = xr[c];
                if (c + 1 < cols) v[i].y = xr[c + 1];
                if (c + 2 < cols) v[i].z = xr[c + 2];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = (i * blockDim.x + threadIdx.x) * 4;
            if (v[i].x > best) best = v[i].x, bi = c;
            if (v[i].y > best) best = v[i].y, bi = c + 1;
            if (v[i].z > best) best = v[i].z, bi = c + 2;
            if (v[i].w > best) best = v[i].w, bi = c + 3;
        }
    } else {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float v = xr[c];
            if (v > best) {
                best = v;
                bi = c;
            }
        }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o, 32);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o, 32);
        if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
    }
    if (lane == 0) sv[w] = best, si[w] = bi;
    __syncthreads();
    if (w == 0) {
        best = (lane < nw) ? sv[lane] : -3.402823466e38f;
        bi = (lane < nw) ? si[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o, 32);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o, 32);
            if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
        }
        // every value <= -FLT_MAX (or NaN): the sequential loop never updates and returns index 0
        if (lane == 0) out[blockIdx.x] = (bi == 0x7FFFFFFF) ? 0u : (uint32_t)bi;
    }
}

__global__ void __launch_bounds__(256) embedding_kernel(const float *__restrict__ table, const uint32_t *__restrict__ ids, int dim,
                                                      int64_t vocab, float *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int b = blockIdx.x;
    int64_t id = ids[b];
    if (id >= vocab) id = vocab - 1;  // never read outside the table
    for (int c = threadIdx.x; c < dim; c += blockDim.x) out[(int64_t)b * dim + c] = table[id * dim + c];
}

__global__ void add_int_kernel(int *p, int delta) {
    pdl_launch_dependents();
    pdl_wait_prior();
    if (threadIdx.x == 0 && blockIdx.x == 0) *p += delta;
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Counter-based normal / uniform fill: value i depends only on (seed, i).
__global__ void __launch_bounds__(256) rand_fill_kernel(float *__restrict__ out, int64_t n, uint64_t seed, float a, float b, int normal) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint64_t r = mix64(seed * 0x9E3779B97F4A7C15ull + (uint64_t)i + 0x632BE59BD9B4E019ull);
        const float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
        const float u2 = (float)(uint32_t)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
        if (normal) out[i] = a + b * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        else out[i] = a + (b - a) * u2;
    }
}

template <typename Kern, typename... Args>
cq_status launch_pdl(cq_ctx *ctx, Kern kern, dim3 grid, dim3 block, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, args...));
    return CQ_OK;
}

}  // namespace

extern "C" {

cq_status cq_rand_normal(cq_ctx *ctx, float *out_dev, int64_t n, float mean, float std, uint64_t seed) {
    CQ_ENTER(ctx);
    if (!out_dev || n < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rand_normal: bad arguments");
    if (n == 0) return CQ_OK;
    const unsigned grid = (unsigned)((n + 255) / 256 < (int64_t)ctx->sm_count * 32 ? (n + 255) / 256 : (int64_t)ctx->sm_count * 32);
    rand_fill_kernel<<<grid, 256, 0, ctx->stream>>>(out_dev, n, seed, mean, std, 1);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status cq_rand_uniform(cq_ctx *ctx, float *out_dev, int64_t n, float lo, float hi, uint64_t seed) {
    CQ_ENTER(ctx);
    if (!out_dev || n < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rand_uniform: bad arguments");
    if (n == 0) return CQ_OK;
    const unsigned grid = (unsigned)((n + 255) / 256 < (int64_t)ctx->sm_count * 32 ? (n + 255) / 256 : (int64_t)ctx->sm_count * 32);
    rand_fill_kernel<<<grid, 256, 0, ctx->stream>>>(out_dev, n, seed, lo, hi, 0);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

cq_status cq_rmsnorm(cq_ctx *ctx, const float *x_dev, const float *alpha_dev, int64_t rows, int64_t cols, float eps, float *y_dev) {
    CQ_ENTER(ctx);
    if (!x_dev || !y_dev || rows < 1 || cols < 1 || cols > 0x7FFFFFFF) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rmsnorm: bad arguments");
    const int threads = cols >= 4096 ? 1024 : (cols >= 1024 ? 512 : 256);
    return launch_pdl(ctx, rmsnorm_kernel<false>, dim3((unsigned)rows), dim3(threads), const_cast<float *>(x_dev), (const float *)nullptr,
                      alpha_dev, (int)cols, eps, y_dev);
}

cq_status cq_add_rmsnorm(cq_ctx *ctx, float *x_dev, const float *delta_dev, const float *alpha_dev, int64_t rows, int64_t cols, float eps,
                         float *y_dev) {
    CQ_ENTER(ctx);
    if (!x_dev || !delta_dev || !y_dev || rows < 1 || cols < 1 || cols > 0x7FFFFFFF)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm: bad arguments");
    const int threads = cols >= 4096 ? 1024 : (cols >= 1024 ? 512 : 256);
    return launch_pdl(ctx, rmsnorm_kernel<true>, dim3((unsigned)rows), dim3(threads), x_dev, delta_dev, alpha_dev, (int)cols, eps, y_dev);
}

cq_status cq_rope_store_kv(cq_ctx *ctx, float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads, int head_dim, const float *cos_dev,
                           const float *sin_dev, const int *pos_dev, float *k_cache_dev, float *v_cache_dev, int max_ctx) {
    CQ_ENTER(ctx);
    if (!qkv_dev || !cos_dev || !sin_dev || !pos_dev || !k_cache_dev || !v_cache_dev)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rope_store_kv: null pointer");
    if (batch < 1 || n_q_heads < 1 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || head_dim < 2 || head_dim % 2 != 0 || max_ctx < 1)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rope_store_kv: bad shape");
    const int work = (n_q_heads + n_kv_heads) * head_dim / 2 + n_kv_heads * head_dim;
    return launch_pdl(ctx, rope_store_kv_kernel, dim3((unsigned)((work + 255) / 256), (unsigned)batch), dim3(256), qkv_dev, n_q_heads,
                      n_kv_heads, head_dim, cos_dev, sin_dev, pos_dev, k_cache_dev, v_cache_dev, max_ctx, ctx->dev_err_devptr);
}

cq_status cq_rope_prefill(cq_ctx *ctx, const float *qkv_dev, int64_t tokens, int n_q_heads, int n_kv_heads, int head_dim, const float *cos_dev,
                          const float *sin_dev, int pos0, float *k_cache_dev, float *v_cache_dev, int max_ctx, void *q16_dev, void *k16_dev,
                          void *v16_dev, int is_bf16) {
    CQ_ENTER(ctx);
    if (!qkv_dev || !cos_dev || !sin_dev || !k_cache_dev || !v_cache_dev || !q16_dev || !k16_dev || !v16_dev)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rope_prefill: null pointer");
    if (tokens < 1 || tokens > 65535 || n_q_heads < 1 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || head_dim < 2 || head_dim % 2 != 0 || max_ctx < 1)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rope_prefill: bad shape");
    if (pos0 < 0 || (int64_t)pos0 + tokens > max_ctx)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_rope_prefill: positions pos0 .. pos0 + tokens - 1 must lie inside [0, max_ctx)");
    const int work = (n_q_heads + n_kv_heads) * head_dim / 2 + n_kv_heads * head_dim;
    const dim3 grid((unsigned)((work + 255) / 256), (unsigned)tokens);
    if (is_bf16)
        return launch_pdl(ctx, rope_prefill_kernel<true>, grid, dim3(256), qkv_dev, (int)tokens, n_q_heads, n_kv_heads, head_dim, cos_dev, sin_dev, pos0,
                          k_cache_dev, v_cache_dev, static_cast<uint16_t *>(q16_dev), static_cast<uint16_t *>(k16_dev), static_cast<uint16_t *>(v16_dev));
    return launch_pdl(ctx, rope_prefill_kernel<false>, grid, dim3(256), qkv_dev, (int)tokens, n_q_heads, n_kv_heads, head_dim, cos_dev, sin_dev, pos0,
                      k_cache_dev, v_cache_dev, static_cast<uint16_t *>(q16_dev), static_cast<uint16_t *>(k16_dev), static_cast<uint16_t *>(v16_dev));
}

cq_status cq_cast_f32_to_16(cq_ctx *ctx, const float *src_dev, int64_t count, int is_bf16, void *dst16_dev) {
    CQ_ENTER(ctx);
    if (!src_dev || !dst16_dev || count < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_cast_f32_to_16: bad arguments");
    if (count == 0) return CQ_OK;
    const unsigned cap = (unsigned)ctx->sm_count * 8;
    const unsigned grid = (unsigned)((count + 255) / 256 < cap ? (count + 255) / 256 : cap);
    if (is_bf16) return launch_pdl(ctx, cast_f32_to_16_kernel<true>, dim3(grid), dim3(256), src_dev, count, static_cast<uint16_t *>(dst16_dev));
    return launch_pdl(ctx, cast_f32_to_16_kernel<false>, dim3(grid), dim3(256), src_dev, count, static_cast<uint16_t *>(dst16_dev));
}

cq_status cq_cast16_to_f32(cq_ctx *ctx, const void *src16_dev, int64_t count, int is_bf16, float *dst_dev) {
    CQ_ENTER(ctx);
    if (!src16_dev || !dst_dev || count < 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_cast16_to_f32: bad arguments");
    if (count == 0) return CQ_OK;
    const unsigned cap = (unsigned)ctx->sm_count * 8;
    const unsigned grid = (unsigned)((count + 255) / 256 < cap ? (count + 255) / 256 : cap);
    if (is_bf16) return launch_pdl(ctx, cast16_to_f32_kernel<true>, dim3(grid), dim3(256), static_cast<const uint16_t *>(src16_dev), count, dst_dev);
    return launch_pdl(ctx, cast16_to_f32_kernel<false>, dim3(grid), dim3(256), static_cast<const uint16_t *>(src16_dev), count, dst_dev);
}

size_t cq_decode_attention_scratch_floats(int64_t batch, int n_q_heads, int head_dim, int max_ctx) {
    const int nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    return (size_t)batch * n_q_heads * nchunks * (head_dim + 2);
}

}  // extern "C"

namespace {
// Decode attention; with cos_dev / sin_dev also the rotary step and the cache write of the newest position
// (inside the attention kernels where they support it, as a separate kernel before them otherwise).
cq_status attention_impl(cq_ctx *ctx, float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads, int head_dim, const float *cos_dev,
                         const float *sin_dev, const int *pos_dev, float *k_cache_dev, float *v_cache_dev, int max_ctx, float *scratch_dev,
                         float *out_dev) {
    if (!qkv_dev || !pos_dev || !k_cache_dev || !v_cache_dev || !scratch_dev || !out_dev)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decode_attention: null pointer");
    if (batch < 1 || n_q_heads < 1 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0 || head_dim < 4 || head_dim > 256 || head_dim % 4 != 0 || max_ctx < 1 || max_ctx > 512 * kAttnChunk)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decode_attention: bad shape (head_dim <= 256 and a multiple of 4, max_ctx <= 16384)");
    int nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const int group = n_q_heads / n_kv_heads;
    cq_status s;
    const bool split_route = head_dim == 128 && group >= 2 && group <= 8 && ctx->tune.attn_variant != 1;
    const bool gqa_chunk_route = !split_route && head_dim == 128 && group >= 2 && group <= kGqaMaxG;
    if (cos_dev && gqa_chunk_route) {  // this route has no fused rotary step: run it as its own kernel first
        const int work = (n_q_heads + n_kv_heads) * head_dim / 2 + n_kv_heads * head_dim;
        s = launch_pdl(ctx, rope_store_kv_kernel, dim3((unsigned)((work + 255) / 256), (unsigned)batch), dim3(256), qkv_dev, n_q_heads, n_kv_heads,
                       head_dim, cos_dev, sin_dev, pos_dev, k_cache_dev, v_cache_dev, max_ctx, ctx->dev_err_devptr);
        if (s != CQ_OK) return s;
        cos_dev = sin_dev = nullptr;
    }
    // Short contexts, one launch: a cluster of eight CTAs per (head, sequence) splits the chunks and combines through
    // distributed shared memory (at most four chunks per CTA; longer contexts want more CTAs than that gives).
    if (!split_route && !gqa_chunk_route && head_dim <= kAttnThreads && max_ctx <= 4 * kAttnCluster * kAttnChunk && ctx->tune.attn_variant != 2) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_q_heads, (unsigned)batch, (unsigned)kAttnCluster);
        cfg.blockDim = dim3(kAttnThreads);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = kAttnCluster;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->tune.pdl ? 2 : 1;
        CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, attn_cluster_kernel, (const float *)qkv_dev, n_q_heads, n_kv_heads, head_dim, pos_dev, (const float *)k_cache_dev,
                                        (const float *)v_cache_dev, max_ctx, scale, out_dev, cos_dev, sin_dev, k_cache_dev, v_cache_dev, ctx->dev_err_devptr));
        return CQ_OK;
    }
    if (split_route) {
        // splits of the context sized so that about four CTAs per SM exist, never under 64 keys each
        const int64_t pairs = (int64_t)n_kv_heads * batch;
        int64_t want = ((int64_t)ctx->sm_count * 4 + pairs - 1) / pairs;
        const int max_splits = (max_ctx + kAttn2Keys - 1) / kAttn2Keys;
        if (want > max_splits) want = max_splits;
        if (want < 1) want = 1;
        const int keys_per_split = (int)(((max_ctx + want - 1) / want + kAttn2Keys - 1) / kAttn2Keys) * kAttn2Keys;
        nchunks = (max_ctx + keys_per_split - 1) / keys_per_split;
        static thread_local int configured = -1;
        if (configured != ctx->device) {
            CQ_CUDA(ctx, cudaFuncSetAttribute(attn_split_gqa_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttn2Smem));
            CQ_CUDA(ctx, cudaFuncSetAttribute(attn_split_gqa_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttn2Smem));
            configured = ctx->device;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)nchunks, (unsigned)n_kv_heads, (unsigned)batch);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = kAttn2Smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
        if (cos_dev)
            CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, attn_split_gqa_kernel<true>, (const float *)qkv_dev, n_q_heads, n_kv_heads, pos_dev, (const float *)k_cache_dev,
                                        (const float *)v_cache_dev, max_ctx, scale, scratch_dev, nchunks, keys_per_split, cos_dev, sin_dev,
                                        k_cache_dev, v_cache_dev, ctx->dev_err_devptr));
        else
            CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, attn_split_gqa_kernel<false>, (const float *)qkv_dev, n_q_heads, n_kv_heads, pos_dev, (const float *)k_cache_dev,
                                        (const float *)v_cache_dev, max_ctx, scale, scratch_dev, nchunks, keys_per_split, cos_dev, sin_dev,
                                        k_cache_dev, v_cache_dev, ctx->dev_err_devptr));
        s = CQ_OK;
    } else if (gqa_chunk_route)
        s = launch_pdl(ctx, attn_partial_gqa_kernel, dim3((unsigned)n_kv_heads, (unsigned)batch, (unsigned)nchunks), dim3(128), (const float *)qkv_dev,
                       n_q_heads, n_kv_heads, pos_dev, (const float *)k_cache_dev, (const float *)v_cache_dev, max_ctx, scale, scratch_dev, nchunks, ctx->dev_err_devptr);
    else
        s = launch_pdl(ctx, attn_partial_kernel, dim3((unsigned)n_q_heads, (unsigned)batch, (unsigned)nchunks), dim3(kAttnThreads),
                       (const float *)qkv_dev, n_q_heads, n_kv_heads, head_dim, pos_dev, (const float *)k_cache_dev, (const float *)v_cache_dev, max_ctx,
                       scale, scratch_dev, nchunks, cos_dev, sin_dev, k_cache_dev, v_cache_dev, ctx->dev_err_devptr);
    if (s != CQ_OK) return s;
    return launch_pdl(ctx, attn_combine_kernel, dim3((unsigned)n_q_heads, (unsigned)batch), dim3(128), (const float *)scratch_dev, n_q_heads,
                      head_dim, nchunks, out_dev);
}
}  // namespace

extern "C" {

cq_status cq_decode_attention(cq_ctx *ctx, const float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads, int head_dim,
                              const int *pos_dev, const float *k_cache_dev, const float *v_cache_dev, int max_ctx, float *scratch_dev,
                              float *out_dev) {
    CQ_ENTER(ctx);
    return attention_impl(ctx, const_cast<float *>(qkv_dev), batch, n_q_heads, n_kv_heads, head_dim, nullptr, nullptr, pos_dev,
                          const_cast<float *>(k_cache_dev), const_cast<float *>(v_cache_dev), max_ctx, scratch_dev, out_dev);
}

cq_status cq_decode_attention_rope(cq_ctx *ctx, float *qkv_dev, int64_t batch, int n_q_heads, int n_kv_heads, int head_dim, const float *cos_dev,
                                   const float *sin_dev, const int *pos_dev, float *k_cache_dev, float *v_cache_dev, int max_ctx,
                                   float *scratch_dev, float *out_dev) {
    CQ_ENTER(ctx);
    if (!cos_dev || !sin_dev || head_dim % 2 != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decode_attention_rope: cos / sin tables and an even head_dim are required");
    return attention_impl(ctx, qkv_dev, batch, n_q_heads, n_kv_heads, head_dim, cos_dev, sin_dev, pos_dev, k_cache_dev, v_cache_dev, max_ctx,
                          scratch_dev, out_dev);
}

cq_status cq_silu_mul(cq_ctx *ctx, const float *gate_up_dev, int64_t rows, int64_t n, float *out_dev, int64_t ld_out) {
    CQ_ENTER(ctx);
    if (!gate_up_dev || !out_dev || rows < 1 || n < 1 || n > 0x7FFFFFFF || ld_out < n)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_silu_mul: bad arguments");
    const int64_t total = rows * n;
    const unsigned grid = (unsigned)((total + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (total + 255) / 256 : (int64_t)ctx->sm_count * 8);
    return launch_pdl(ctx, silu_mul_kernel, dim3(grid), dim3(256), gate_up_dev, (int)n, total, out_dev, ld_out);
}

cq_status cq_silu_mul_pairs(cq_ctx *ctx, const float *gate_up_dev, int64_t rows, int64_t n, float *out_dev, int64_t ld_out) {
    CQ_ENTER(ctx);
    if (!gate_up_dev || !out_dev || rows < 1 || n < 1 || n > 0x7FFFFFFF || ld_out < n || (reinterpret_cast<uintptr_t>(gate_up_dev) & 7))
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_silu_mul_pairs: bad arguments");
    const int64_t total = rows * n;
    const unsigned grid = (unsigned)((total + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (total + 255) / 256 : (int64_t)ctx->sm_count * 8);
    return launch_pdl(ctx, silu_mul_pairs_kernel, dim3(grid), dim3(256), gate_up_dev, (int)n, total, out_dev, ld_out);
}

cq_status cq_argmax(cq_ctx *ctx, const float *x_dev, int64_t rows, int64_t cols, uint32_t *out_dev) {
    CQ_ENTER(ctx);
    if (!x_dev || !out_dev || rows < 1 || cols < 1 || cols > 0x7FFFFFFF) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_argmax: bad arguments");
    return launch_pdl(ctx, argmax_kernel, dim3((unsigned)rows), dim3(1024), x_dev, (int)cols, out_dev);
}

cq_status cq_embedding(cq_ctx *ctx, const float *table_dev, int64_t vocab, int64_t dim, const uint32_t *ids_dev, int64_t rows, float *out_dev) {
    CQ_ENTER(ctx);
    if (!table_dev || !ids_dev || !out_dev || vocab < 1 || dim < 1 || rows < 1 || dim > 0x7FFFFFFF)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_embedding: bad arguments");
    return launch_pdl(ctx, embedding_kernel, dim3((unsigned)rows), dim3(256), table_dev, ids_dev, (int)dim, vocab, out_dev);
}

cq_status cq_add_int(cq_ctx *ctx, int *value_dev, int delta) {
    CQ_ENTER(ctx);
    if (!value_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_int: null pointer");
    return launch_pdl(ctx, add_int_kernel, dim3(1), dim3(32), value_dev, delta);
}

}  // extern "C"
