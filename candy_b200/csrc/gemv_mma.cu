// Small batches (2..8 activation rows) against Q4_0 weights in ONE weight pass and ONE launch: the weights stream
// through a shared-memory ring exactly as in the one-row kernel, and the dot products of a quant block against all
// activation rows are one pair of integer tensor-core instructions (mma.sync m16n8k32, u8 x s8 -> s32) instead of
// 32 x 8 multiply-adds on the CUDA cores, so the kernel stays bound by HBM at eight rows as it is at one.
//
// CQ_ACT_F32 numerics (ACT = 0) are those of the int8 tensor-core GEMM's plane columns (gemm_i8_tmem.cu): every activation block is
// 15-bit block fixed point, X = rint(x * 16383 / amax) = 128 * hi + lo (hi in [-128, 127], lo in [0, 127]); with the
// unsigned nibbles n of a weight block the block's term is (d_w * amax / 16383) * (128 * sum(n * hi) + sum(n * lo)
// - 8 * sum(X)), integer sums exact.  The reference path is QMatMul's dequantize + f32 matmul
// (tensor/cpu_backend.go:419-481); this lands about 2e-5 of max|y| from it.
//
// With ACT = 1 the same kernel runs CQ_ACT_Q8_1: one int8 plane quantized exactly as quantize_q8_1
// (tensor/internal/cuda/kernels/quantized.cu:3521-3558), block terms d4 * (sumi * d8 - 8 * s8) as vec_dot_q4_0_q8_1
// (quantized.cu:1919-1941), each step a fused multiply-add.
//
// Shape of the work:
//   * the CTAs of a cluster of `ks` (1, 2, 4 or 8) share a range of weight rows and split k between them, so that a
//     CTA's part of every activation row fits its registers as ready-made B fragments (16 warps x BPW blocks);
//   * a stage of the ring is 16 weight rows (the M of the instruction) by the CTA's k slice, one bulk copy per row
//     into a pitch that keeps the eight rows a warp reads at once in different banks;
//   * warp w owns blocks [w * BPW, (w + 1) * BPW) of the slice.  Lane (g = lane / 4, q = lane % 4) holds, per block,
//     four nibble bytes of weight rows g and g + 8 (A fragment: low nibbles = k positions 4q.., high nibbles =
//     16 + 4q..) and the matching eight activation values of activation row g (B fragment).  Which four bytes a lane
//     takes is free as long as both operands agree: odd blocks start on a word boundary (bytes 4q .. 4q + 3), even
//     blocks start two bytes past one, so there lanes 0..2 take bytes 2 + 4q .. 5 + 4q and lane 3 bytes 0, 1, 14, 15;
//   * the accumulator of the low-plane instruction starts at (bias + 0x4B400000): after t = 128 * S_hi + S_lo the
//     register read as a float is 12582912 + T exactly (|T| <= 8 * 16383 * 32 < 2^22), so the conversion is one
//     subtraction and no int-to-float instruction is on the path;
//   * the sixteen warps' partial 16 x 8 tiles are parked in shared memory and added in warp order by a warp of its
//     own (deterministic; the workers only arrive at a named barrier and go on with the next stage), the cluster's
//     k slices in rank order through distributed shared memory at the end.
// Every wait is bounded and records an error word.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int MM_WARPS = 16;       // consumer warps
constexpr int MM_ROWS = 16;        // weight rows per stage
constexpr int MM_MAX_STAGES = 8;
constexpr int MM_RED_BYTES = 2 * MM_WARPS * 128 * 4;
constexpr int MM_COLSC_BYTES = MM_WARPS * 8 * 4 * 32;  // per (warp, block, q): the accumulator seeds as a ready quad, then the two scales
constexpr int MM_THREADS = (MM_WARPS + 2) * 32;   // workers, the producer warp, the reducer warp
constexpr int kMagicBits = 0x4B400000;  // 1.5 * 2^23 as a float
constexpr float kMagic = 12582912.0f;

struct MmaGemvParams {
    const uint8_t *w;
    const float *x;
    float *y;
    const float *bias;
    int64_t ldx, ldy, n;
    int nb;        // blocks per weight row
    int m;         // activation rows (<= 8)
    int ks;        // CTAs per cluster = k slices
    int ranges;    // row ranges = clusters
    int order;     // 0: interleaved nibbles (elements 2j, 2j+1 in byte j), 1: split (elements j, j+16)
    int act;       // 0: 15-bit plane columns (CQ_ACT_F32), 1: Q8_1 columns (CQ_ACT_Q8_1); host-side dispatch only
    int stages, pitch, stage_bytes;
    int ypart_off;  // byte offset of the cluster-reduction buffer in dynamic shared memory
    int *err;
};

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int c0, int c1, int c2, int c3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
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

template <int BPW, int ORDER, int ACT>
__global__ void __launch_bounds__(MM_THREADS, 1) gemv_mma_kernel(const MmaGemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[MM_MAX_STAGES];
    __shared__ uint64_t bar_empty[MM_MAX_STAGES];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ks = p.ks > 1 ? (int)(blockIdx.x % p.ks) : 0;  // rank in the cluster (clusters are consecutive CTAs)
    const int range = (int)(blockIdx.x / p.ks);
    const int64_t row_begin = p.n * range / p.ranges, row_end = p.n * (range + 1) / p.ranges;
    const int nrows = (int)(row_end - row_begin);
    const int npass = (nrows + MM_ROWS - 1) / MM_ROWS;
    const int units = p.nb >> 3;  // slices are cut in units of eight blocks (144 bytes: copies stay 16-byte aligned)
    const int u0 = units * ks / p.ks, u1 = units * (ks + 1) / p.ks;
    const int sblocks = (u1 - u0) * 8;
    const uint32_t slice_bytes = (uint32_t)sblocks * kQ4Bytes;
    const int64_t row_bytes = (int64_t)p.nb * kQ4Bytes;
    float *red = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);
    float4 *colsc = reinterpret_cast<float4 *>(smem + (size_t)p.stages * p.stage_bytes + MM_RED_BYTES);  // [warp][block][q] entries of 32 bytes
    float *ypart = reinterpret_cast<float *>(smem + p.ypart_off);

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), MM_WARPS);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (warp == MM_WARPS) {
        // ---- producer: the weights do not depend on the previous kernel, so the ring fills at once ----
        const uint64_t policy = make_l2_policy_evict_first();
        const uint8_t *src0 = p.w + row_begin * row_bytes + (int64_t)u0 * (8 * kQ4Bytes);
        int issued = 0;
        for (int ps = 0; ps < npass; ++ps) {
            const int s = ps % p.stages;
            if (ps >= p.stages && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ((ps / p.stages) - 1) & 1)) {
                if (lane == 0) atomicExch(p.err, kDevErrEmptyWait);
                break;
            }
            const int rows = min(MM_ROWS, nrows - ps * MM_ROWS);
            if (lane == 0) mbar_expect_tx(smem_u32(&bar_full[s]), (uint32_t)rows * slice_bytes);
            __syncwarp();
            if (lane < rows)
                bulk_g2s_hint(smem_u32(smem + (size_t)s * p.stage_bytes + (size_t)lane * p.pitch), src0 + (int64_t)(ps * MM_ROWS + lane) * row_bytes,
                              slice_bytes, smem_u32(&bar_full[s]), policy);
            issued = ps + 1;
        }
        // never leave with copies in flight into this CTA's shared memory
        for (int ps = issued > p.stages ? issued - p.stages : 0; ps < issued; ++ps) {
            if (!mbar_wait_bounded(smem_u32(&bar_full[ps % p.stages]), (ps / p.stages) & 1)) {
                if (lane == 0) atomicExch(p.err, kDevErrDrain);
                break;
            }
        }
    } else if (warp == MM_WARPS + 1) {
        // ---- reducer: adds the sixteen partial tiles of a pass in warp order while the others work on the next ----
        pdl_wait_prior();
        for (int ps = 0; ps < npass; ++ps) {
            const int buf = ps & 1;
            asm volatile("bar.sync %0, %1;" ::"r"(2 + buf), "n"(MM_WARPS * 32 + 32) : "memory");  // the tile is parked
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = e * 32 + lane;  // value t of the tile: lane t / 4 of the fragment, register t % 4
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < MM_WARPS; ++w) tot += red[(buf * MM_WARPS + w) * 128 + t];
                const int l = t >> 2, c = t & 3;
                const int wrow = ps * MM_ROWS + (l >> 2) + ((c >> 1) << 3), col = 2 * (l & 3) + (c & 1);
                if (wrow < nrows && col < p.m) {
                    if (p.ks > 1) ypart[wrow * 8 + col] = tot;
                    else p.y[(int64_t)col * p.ldy + row_begin + wrow] = p.bias ? tot + p.bias[row_begin + wrow] : tot;
                }
            }
            if (ps + 2 < npass) asm volatile("bar.arrive %0, %1;" ::"r"(4 + buf), "n"(MM_WARPS * 32 + 32) : "memory");  // the buffer is free again
        }
    } else {
        // ---- workers ----
        const int g = lane >> 2, q = lane & 3;
        pdl_wait_prior();  // the activations come from the previous kernel in the stream

        // B fragments of this warp's blocks for activation row g, in registers; the scale and the accumulator seed of
        // every (block, activation row) go to shared memory, where the lane that owns result columns 2q, 2q+1 finds them.
        uint32_t bh[BPW][2], bl[BPW][2];  // ACT 1: bh holds the single int8 plane, bl is unused
        if (ACT == 0) {
            float v[BPW][8];  // 0..3: the elements under the low nibbles of the lane's four bytes, 4..7: under the high nibbles
#pragma unroll
            for (int j = 0; j < BPW; ++j) {  // every load first: one trip to L2 for the whole warp's share
                const int lb = warp * BPW + j;
                const bool live = lb < sblocks && g < p.m;
                const float *xb = p.x + (int64_t)(live ? g : 0) * p.ldx + (int64_t)(u0 * 8 + (lb < sblocks ? lb : 0)) * kQK;
                // the lane's four bytes are two byte pairs, starting at bytes b0 and b1 (both even)
                const int b0 = (j & 1) ? 4 * q : (q < 3 ? 2 + 4 * q : 0), b1 = (j & 1) ? 4 * q + 2 : (q < 3 ? 4 + 4 * q : 14);
                if (ORDER == 0) {  // byte b holds elements 2b (low nibble) and 2b + 1: a pair of bytes is four consecutive floats
                    const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    const float4 f0 = live ? __ldg(reinterpret_cast<const float4 *>(xb + 2 * b0)) : z;
                    const float4 f1 = live ? __ldg(reinterpret_cast<const float4 *>(xb + 2 * b1)) : z;
                    v[j][0] = f0.x, v[j][4] = f0.y, v[j][1] = f0.z, v[j][5] = f0.w;
                    v[j][2] = f1.x, v[j][6] = f1.y, v[j][3] = f1.z, v[j][7] = f1.w;
                } else {  // byte b holds elements b (low nibble) and b + 16
                    const float2 z = make_float2(0.0f, 0.0f);
                    const float2 l0 = live ? __ldg(reinterpret_cast<const float2 *>(xb + b0)) : z;
                    const float2 l1 = live ? __ldg(reinterpret_cast<const float2 *>(xb + b1)) : z;
                    const float2 h0 = live ? __ldg(reinterpret_cast<const float2 *>(xb + 16 + b0)) : z;
                    const float2 h1 = live ? __ldg(reinterpret_cast<const float2 *>(xb + 16 + b1)) : z;
                    v[j][0] = l0.x, v[j][1] = l0.y, v[j][2] = l1.x, v[j][3] = l1.y;
                    v[j][4] = h0.x, v[j][5] = h0.y, v[j][6] = h1.x, v[j][7] = h1.y;
                }
            }
            float *sc = reinterpret_cast<float *>(colsc) + (size_t)warp * BPW * 32;
#pragma unroll
            for (int j = 0; j < BPW; ++j) {
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                const float inv = amax > 0.0f ? 16383.0f / amax : 0.0f;
                int xsum = 0;
                uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int t = __float2int_rn(v[j][i] * inv);  // |v * inv| <= 16383 * (1 + 2^-23): never rounds to 16384
                    xsum += t;
                    hi[i >> 2] |= (uint32_t)((t >> 7) & 0xFF) << (8 * (i & 3));
                    lo[i >> 2] |= (uint32_t)(t & 0x7F) << (8 * (i & 3));
                }
                xsum += __shfl_xor_sync(0xffffffffu, xsum, 1);
                xsum += __shfl_xor_sync(0xffffffffu, xsum, 2);
                bh[j][0] = hi[0], bh[j][1] = hi[1];
                bl[j][0] = lo[0], bl[j][1] = lo[1];
                // entry (block j, q') of 8 words = (seed of row 2q', seed of row 2q'+1, the same two again: the accumulator
                // quad of the low-plane instruction as one 16-byte load), (scale of row 2q', scale of row 2q'+1), padding
                if (q == 0) {
                    float *dst = sc + (j * 4 + (g >> 1)) * 8 + (g & 1);
                    dst[0] = dst[2] = __int_as_float(kMagicBits - 8 * xsum);
                    dst[4] = amax * (1.0f / 16383.0f);
                }
            }
        }
        else {
            // Q8_1 columns, exactly quantize_q8_1 (tensor/internal/cuda/kernels/quantized.cu:3521-3558): eight lanes per
            // (block, activation row) in natural element order, d = amax / 127 and q = round(x / d) by true division, d and
            // the block's f32 sum (the reference's xor butterfly: offsets 16, 8, 4 across the lanes here, 2 and 1 inside a
            // lane) rounded to f16.  The bytes go through this warp's kilobyte of the reduction buffer (not yet in use), from
            // where every lane picks the eight that match its weight bytes.
            uint8_t *stg = reinterpret_cast<uint8_t *>(red) + (size_t)warp * 1024;  // [block of the chunk][row][32 positions]
            float *sc = reinterpret_cast<float *>(colsc) + (size_t)warp * BPW * 32;
            const int l8 = lane & 7;
#pragma unroll
            for (int c0 = 0; c0 < BPW; c0 += 4) {
                constexpr int kChunkMax = 4;
                const int cb = BPW - c0 < kChunkMax ? BPW - c0 : kChunkMax;  // blocks in this chunk
                // up to four rows: rows 4..7 take no turns, their entries and bytes are zeroed first (the MMA still reads them)
                const int rsh = p.m <= 4 ? 2 : 3, mrows = 1 << rsh;
                if (mrows < 8) {
                    for (int i = lane; i < cb * 8 * 8; i += 32) reinterpret_cast<uint32_t *>(stg)[i] = 0u;
                    for (int i = lane; i < cb * 4 * 4; i += 32) sc[(c0 * 4 + (i >> 2)) * 8 + (i & 3)] = 0.0f;
                    __syncwarp();
                }
                const int turns = (cb * mrows + 3) >> 2;
                float4 vin[kChunkMax * 2];
#pragma unroll
                for (int it = 0; it < kChunkMax * 2; ++it) {  // every load of the chunk first: one trip to L2
                    const int pairi = it * 4 + (lane >> 3);
                    const int bj = pairi >> rsh, row = pairi & (mrows - 1);
                    const int lb = warp * BPW + c0 + bj;
                    vin[it] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (it < turns && bj < cb && lb < sblocks && row < p.m)
                        vin[it] = __ldg(reinterpret_cast<const float4 *>(p.x + (int64_t)row * p.ldx + (int64_t)(u0 * 8 + lb) * kQK) + l8);
                }
#pragma unroll
                for (int it = 0; it < kChunkMax * 2; ++it) {
                    if (it >= turns) break;
                    const int pairi = it * 4 + (lane >> 3);  // (block of the chunk, activation row)
                    const int bj = pairi >> rsh, row = pairi & (mrows - 1);
                    const float4 v = vin[it];
                    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                    float s0 = v.x, s1 = v.y, s2 = v.z, s3 = v.w;
#pragma unroll
                    for (int o = 4; o > 0; o >>= 1) {
                        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
                        s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, o, 8));
                        s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, o, 8));
                        s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, o, 8));
                        s3 = __fadd_rn(s3, __shfl_xor_sync(0xffffffffu, s3, o, 8));
                    }
                    const float sum = __fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3));
                    const float d = __fdiv_rn(amax, 127.0f);
                    // round(x / d) by true division only where the quick quotient lies within 1e-3 of a tie: elsewhere both
                    // round to the same integer (the quick quotient is off by less than 127 * 2^-21)
                    const float rd = amax == 0.0f ? 0.0f : __frcp_rn(d);
                    auto q8 = [&](float xv) -> uint32_t {
                        const float t = xv * rd;
                        float r = roundf(t);
                        if (!(fabsf(fabsf(t - r) - 0.5f) >= 1e-3f)) r = roundf(__fdiv_rn(xv, d));  // also when the quick quotient is not finite
                        return (uint32_t)((int)r & 0xFF);
                    };
                    uint32_t byte[4];
                    byte[0] = amax == 0.0f ? 0u : q8(v.x);
                    byte[1] = amax == 0.0f ? 0u : q8(v.y);
                    byte[2] = amax == 0.0f ? 0u : q8(v.z);
                    byte[3] = amax == 0.0f ? 0u : q8(v.w);
                    // positions 0..15: the elements under the low nibbles of bytes 0..15, positions 16..31: under the high nibbles
                    uint8_t *dst = stg + ((bj < cb ? bj : 0) * 8 + row) * 32;
                    if (bj >= cb) {
                    } else if (ORDER == 0) {  // elements 4l, 4l+2 are the low nibbles of bytes 2l, 2l+1; elements 4l+1, 4l+3 the high ones
                        *reinterpret_cast<uint16_t *>(dst + 2 * l8) = (uint16_t)(byte[0] | (byte[2] << 8));
                        *reinterpret_cast<uint16_t *>(dst + 16 + 2 * l8) = (uint16_t)(byte[1] | (byte[3] << 8));
                    } else {           // element e is the low nibble of byte e (e < 16) or the high nibble of byte e - 16
                        *reinterpret_cast<uint32_t *>(dst + 4 * l8) = byte[0] | (byte[1] << 8) | (byte[2] << 16) | (byte[3] << 24);
                    }
                    // entry (block, q') = (d8 of rows 2q', 2q'+1, then -8 * s8 of the same rows)
                    if (l8 == 0 && bj < cb) {
                        float *e = sc + ((c0 + bj) * 4 + (row >> 1)) * 8 + (row & 1);
                        e[0] = __half2float(__float2half_rn(d));
                        e[2] = -8.0f * __half2float(__float2half_rn(sum));
                    }
                }
                __syncwarp();
#pragma unroll
                for (int bj = 0; bj < cb; ++bj) {
                    const int j = c0 + bj;
                    const int b0 = (j & 1) ? 4 * q : (q < 3 ? 2 + 4 * q : 0), b1 = (j & 1) ? 4 * q + 2 : (q < 3 ? 4 + 4 * q : 14);
                    const uint8_t *src = stg + (bj * 8 + g) * 32;
                    bh[j][0] = (uint32_t)*reinterpret_cast<const uint16_t *>(src + b0) | ((uint32_t)*reinterpret_cast<const uint16_t *>(src + b1) << 16);
                    bh[j][1] = (uint32_t)*reinterpret_cast<const uint16_t *>(src + 16 + b0) | ((uint32_t)*reinterpret_cast<const uint16_t *>(src + 16 + b1) << 16);
                    bl[j][0] = bl[j][1] = 0;
                }
                __syncwarp();
            }
            // the staging bytes lie where other warps will park their partial tiles
            asm volatile("bar.sync 1, %0;" ::"n"(MM_WARPS * 32) : "memory");
        }
        __syncwarp();

        const uint64_t neg_magic = dup2(-kMagic);
        const uint32_t sel = q < 3 ? 0x3210u : 0x5432u;  // lane 3 of an even block: the upper half of word 0 and the lower half of word 4
        const int word_even = q < 3 ? 1 + q : 0, word_odd = 5 + q;
        const float *mysc = reinterpret_cast<const float *>(colsc) + ((size_t)warp * BPW * 4 + q) * 8;
        const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
        int stage = 0;
        uint32_t phase = 0;
        bool dead = false;
        for (int ps = 0; ps < npass; ++ps) {
            const int buf = ps & 1;
            // a warp whose wait gave up keeps walking the loop so that the reducer's barriers still fill up
            if (!dead && !mbar_wait_bounded(full0 + 8 * stage, phase)) {
                if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                dead = true;
            }
            uint64_t acc01 = 0, acc23 = 0;  // packed f32 pairs: (row g, col 2q), (g, 2q+1) and (g+8, 2q), (g+8, 2q+1)
            if (!dead) {
                // word pointers of weight rows g and g + 8 at this warp's first block: the head word of a pair of blocks
                // (scale of the even block, its bytes 0, 1), the lane's word of the even block and of the odd block
                const uint32_t *h0p = reinterpret_cast<const uint32_t *>(smem + (size_t)stage * p.stage_bytes + (size_t)g * p.pitch + (size_t)warp * (BPW * kQ4Bytes));
                const uint32_t *h1p = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(h0p) + 8 * (size_t)p.pitch);
                const uint32_t *e0p = h0p + word_even, *e1p = h1p + word_even, *o0p = h0p + word_odd, *o1p = h1p + word_odd;
#pragma unroll
                for (int j = 0; j < BPW; j += 2) {
                    if (warp * BPW + j < sblocks) {  // slices are multiples of eight blocks: a pair is whole or absent
                        constexpr int kPairWords = 2 * kQ4Bytes / 4;  // a pair of blocks is nine words
                        const int wo = (j / 2) * kPairWords;
                        const uint32_t h0 = h0p[wo], t0 = h0p[wo + 4], e0 = e0p[wo], o0 = o0p[wo];
                        const uint32_t h1 = h1p[wo], t1 = h1p[wo + 4], e1 = e1p[wo], o1 = o1p[wo];
                        const uint32_t wv[2][2] = {{__byte_perm(e0, t0, sel), __byte_perm(e1, t1, sel)}, {o0, o1}};
                        // scales of (even block, odd block) x (row g, row g + 8), each twice in a register pair
                        const uint64_t dw[2][2] = {{dup2(__low2float(*reinterpret_cast<const __half2 *>(&h0))),
                                                    dup2(__low2float(*reinterpret_cast<const __half2 *>(&h1)))},
                                                   {dup2(__high2float(*reinterpret_cast<const __half2 *>(&t0))),
                                                    dup2(__high2float(*reinterpret_cast<const __half2 *>(&t1)))}};
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            const uint32_t a[4] = {wv[b][0] & 0x0F0F0F0Fu, wv[b][1] & 0x0F0F0F0Fu, (wv[b][0] >> 4) & 0x0F0F0F0Fu,
                                                   (wv[b][1] >> 4) & 0x0F0F0F0Fu};
                            if (ACT == 0) {
                                const int4 sd = *reinterpret_cast<const int4 *>(mysc + (j + b) * 32);
                                const uint64_t csxy = *reinterpret_cast<const uint64_t *>(mysc + (j + b) * 32 + 4);
                                int sh[4], sl[4];
                                mma_u8s8(sh, a, bh[j + b][0], bh[j + b][1], 0, 0, 0, 0);
                                mma_u8s8(sl, a, bl[j + b][0], bl[j + b][1], sd.x, sd.y, sd.z, sd.w);
                                // two results per instruction (packed f32): (T - magic) * (activation scales), then * weight scale
                                const uint64_t u01 = mul2(add2(pack2(__int_as_float(sh[0] * 128 + sl[0]), __int_as_float(sh[1] * 128 + sl[1])), neg_magic), csxy);
                                const uint64_t u23 = mul2(add2(pack2(__int_as_float(sh[2] * 128 + sl[2]), __int_as_float(sh[3] * 128 + sl[3])), neg_magic), csxy);
                                acc01 = fma2(dw[b][0], u01, acc01);
                                acc23 = fma2(dw[b][1], u23, acc23);
                            } else {
                                // vec_dot_q4_0_q8_1 (quantized.cu:1919-1941) with the block scale applied as at :4434-4453:
                                // acc += d4 * (sumi * d8 - 8 * s8), each step a fused multiply-add
                                const ulonglong2 cs = *reinterpret_cast<const ulonglong2 *>(mysc + (j + b) * 32);  // (d8, d8'), (-8 s8, -8 s8')
                                int si[4];
                                mma_u8s8(si, a, bh[j + b][0], bh[j + b][1], kMagicBits, kMagicBits, kMagicBits, kMagicBits);
                                const uint64_t f01 = add2(pack2(__int_as_float(si[0]), __int_as_float(si[1])), neg_magic);
                                const uint64_t f23 = add2(pack2(__int_as_float(si[2]), __int_as_float(si[3])), neg_magic);
                                acc01 = fma2(dw[b][0], fma2(f01, cs.x, cs.y), acc01);
                                acc23 = fma2(dw[b][1], fma2(f23, cs.x, cs.y), acc23);
                            }
                        }
                    }
                }
            }
            float acc[4];
            unpack2(acc01, acc[0], acc[1]);
            unpack2(acc23, acc[2], acc[3]);
            // The tile of pass ps - 2 has left this buffer once the reducer says so.  The partial tile depends on every
            // word read from the stage, so the stage can be released once it is parked.
            if (ps >= 2) asm volatile("bar.sync %0, %1;" ::"r"(4 + buf), "n"(MM_WARPS * 32 + 32) : "memory");
            reinterpret_cast<float4 *>(red)[(buf * MM_WARPS + warp) * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);
            asm volatile("bar.arrive %0, %1;" ::"r"(2 + buf), "n"(MM_WARPS * 32 + 32) : "memory");
            if (++stage == p.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
    }

    if (p.ks > 1) {
        // add the cluster's k slices in rank order; every rank finishes the rows r with r % ks == its rank
        cg::cluster_group cluster = cg::this_cluster();
        pdl_wait_prior();  // the producer warp writes results below and has not waited yet
        cluster.sync();
        for (int i = tid; i < nrows * 8; i += MM_THREADS) {
            const int wrow = i >> 3, col = i & 7;
            if (col < p.m && wrow % p.ks == ks) {
                float tot = 0.0f;
                for (int r = 0; r < p.ks; ++r) tot += cluster.map_shared_rank(ypart, r)[i];
                p.y[(int64_t)col * p.ldy + row_begin + wrow] = p.bias ? tot + p.bias[row_begin + wrow] : tot;
            }
        }
        cluster.sync();  // nobody leaves while its shared memory may still be read
    }
}

struct MmaPlan {
    int ks, bpw, ranges, stages, pitch, stage_bytes, ypart_off;
    size_t smem;
};

// ranges = 0: one row range per group of ks SMs; otherwise that many row ranges.
bool plan_mma(cq_ctx *ctx, int64_t k, int64_t n, int ranges, MmaPlan &pl) {
    const int nb = (int)(k / kQK), units = nb / 8;
    for (int ks = 1; ks <= 8; ks *= 2) {
        if (ks > units) return false;
        const int max_blocks = ((units + ks - 1) / ks) * 8;
        if (max_blocks > MM_WARPS * 8) continue;
        int bpw = (max_blocks + MM_WARPS - 1) / MM_WARPS;
        bpw += bpw & 1;
        if (ranges <= 0) ranges = ctx->sm_count / ks;
        if (ranges < 1) return false;
        // eight rows read at once must fall in different banks: pitch = 16 (mod 32) bytes
        const int slice = max_blocks * kQ4Bytes;
        const int pitch = (slice % 32 == 16) ? slice : slice + 16;
        const int stage_bytes = MM_ROWS * pitch;
        const int rows_max = (int)((n + ranges - 1) / ranges);
        const int ypart = ks > 1 ? ((rows_max + MM_ROWS) * 8 * 4) : 0;
        const int budget = 225 * 1024 - MM_RED_BYTES - MM_COLSC_BYTES - ypart;
        int stages = budget / stage_bytes;
        if (stages > MM_MAX_STAGES) stages = MM_MAX_STAGES;
        if (stages < 2) return false;
        pl.ks = ks, pl.bpw = bpw, pl.ranges = ranges, pl.stages = stages, pl.pitch = pitch, pl.stage_bytes = stage_bytes;
        pl.ypart_off = stages * stage_bytes + MM_RED_BYTES + MM_COLSC_BYTES;
        pl.smem = (size_t)pl.ypart_off + ypart;
        return true;
    }
    return false;
}

template <int BPW, int ORDER, int ACT>
cq_status run_mma_o(cq_ctx *ctx, MmaGemvParams p, MmaPlan pl, int64_t k) {
    auto kern = gemv_mma_kernel<BPW, ORDER, ACT>;
    static thread_local size_t configured = 0;
    static thread_local int configured_dev = -1;
    static thread_local std::map<std::pair<int, size_t>, int> resident;  // (cluster size, shared memory) -> clusters resident at once
    if (configured_dev != ctx->device) configured = 0, resident.clear(), configured_dev = ctx->device;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    for (int round = 0; round < 3; ++round) {
        if (configured < pl.smem) {
            CQ_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
            configured = pl.smem;
        }
        cfg.gridDim = dim3((unsigned)(pl.ranges * pl.ks));
        cfg.blockDim = dim3(MM_THREADS);
        cfg.dynamicSmemBytes = pl.smem;
        cfg.stream = ctx->stream;
        cfg.attrs = attr;
        cfg.numAttrs = 0;
        if (pl.ks == 1) break;
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)pl.ks, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.numAttrs = 1;
        // Every cluster must be resident at once: the SMs of a GPC do not always divide by the cluster size, and a second
        // wave of a few clusters would double the time.  Fewer, longer row ranges instead.
        const auto key = std::make_pair(pl.ks, pl.smem);
        auto it = resident.find(key);
        if (it == resident.end()) {
            int nc = 0;
            CQ_CUDA(ctx, cudaOccupancyMaxActiveClusters(&nc, kern, &cfg));
            it = resident.emplace(key, nc).first;
        }
        if (it->second >= pl.ranges) break;
        if (it->second < 1 || !plan_mma(ctx, k, p.n, it->second, pl)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "small-batch kernel: clusters do not fit");
    }
    p.ks = pl.ks, p.ranges = pl.ranges, p.stages = pl.stages, p.pitch = pl.pitch, p.stage_bytes = pl.stage_bytes, p.ypart_off = pl.ypart_off;
    if (ctx->tune.pdl) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return CQ_OK;
}

template <int BPW>
cq_status run_mma(cq_ctx *ctx, const MmaGemvParams &p, const MmaPlan &pl, int64_t k) {
    if (p.act == 0) return p.order == 0 ? run_mma_o<BPW, 0, 0>(ctx, p, pl, k) : run_mma_o<BPW, 1, 0>(ctx, p, pl, k);
    return p.order == 0 ? run_mma_o<BPW, 0, 1>(ctx, p, pl, k) : run_mma_o<BPW, 1, 1>(ctx, p, pl, k);
}

}  // namespace

bool gemv_mma_supported(cq_ctx *ctx, int qtype, int64_t m, int64_t k, int64_t n, const void *w, const float *x, int64_t ldx) {
    MmaPlan pl;
    return qtype == CQ_Q4_0 && m >= 2 && m <= 8 && k % 256 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ldx % 4 == 0 && plan_mma(ctx, k, n, 0, pl);
}

cq_status launch_gemv_mma(cq_ctx *ctx, int order, int q8_1, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, const float *bias,
                          float *y, int64_t ldy) {
    MmaPlan pl;
    if (!plan_mma(ctx, k, n, 0, pl)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "small-batch kernel: shape not supported");
    MmaGemvParams p = {};
    p.w = static_cast<const uint8_t *>(w);
    p.x = x, p.y = y, p.bias = bias;
    p.ldx = ldx, p.ldy = ldy, p.n = n;
    p.nb = (int)(k / kQK), p.m = (int)m, p.order = order == CQ_ORDER_GGML_SPLIT ? 1 : 0, p.act = q8_1 ? 1 : 0;
    p.err = ctx->dev_err_devptr;
    switch (pl.bpw) {  // the plan may still change its row ranges and stages, never its k slices
    case 2: return run_mma<2>(ctx, p, pl, k);
    case 4: return run_mma<4>(ctx, p, pl, k);
    case 6: return run_mma<6>(ctx, p, pl, k);
    default: return run_mma<8>(ctx, p, pl, k);
    }
}
