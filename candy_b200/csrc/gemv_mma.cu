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
#include "gemv_mma.cuh"

using namespace mma_gemv;

namespace {

constexpr int kMagicBits = 0x4B400000;  // 1.5 * 2^23 as a float
constexpr float kMagic = 12582912.0f;

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int c0, int c1, int c2, int c3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

template <int BPW, int ORDER, int ACT>
__global__ void __launch_bounds__(MM_THREADS, 1) gemv_mma_kernel(const MmaGemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[MM_MAX_STAGES];
    __shared__ uint64_t bar_empty[MM_MAX_STAGES];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const Geometry geo = geometry(p);
    const int npass = geo.npass, u0 = geo.u0, sblocks = geo.sblocks;
    float *red = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);
    float4 *colsc = reinterpret_cast<float4 *>(smem + p.aux_off);  // [warp][block][q] entries of 32 bytes
    float *ypart = reinterpret_cast<float *>(smem + p.ypart_off);

    pdl_launch_dependents();
    init_ring(p, bar_full, bar_empty);

    if (warp == MM_WARPS) {
        produce(p, geo, smem, bar_full, bar_empty);
    } else if (warp == MM_WARPS + 1) {
        reduce<1>(p, geo, red, ypart);
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
            float acc[1][4];
            unpack2(acc01, acc[0][0], acc[0][1]);
            unpack2(acc23, acc[0][2], acc[0][3]);
            park<1>(red, ps, warp, lane, acc, empty0 + 8 * stage);
            if (++stage == p.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
    }

    if (p.ks > 1) cluster_sum<1>(p, geo, ypart);
}

template <int BPW>
cq_status run_mma(cq_ctx *ctx, const MmaGemvParams &p, const MmaPlan &pl, int64_t k) {
    if (p.act == 0) {
        if (p.order == 0) return launch_planned(ctx, gemv_mma_kernel<BPW, 0, 0>, p, pl, k, 1, 8);
        return launch_planned(ctx, gemv_mma_kernel<BPW, 1, 0>, p, pl, k, 1, 8);
    }
    if (p.order == 0) return launch_planned(ctx, gemv_mma_kernel<BPW, 0, 1>, p, pl, k, 1, 8);
    return launch_planned(ctx, gemv_mma_kernel<BPW, 1, 1>, p, pl, k, 1, 8);
}

}  // namespace

bool gemv_mma_supported(cq_ctx *ctx, int qtype, int64_t m, int64_t k, int64_t n, const void *w, const float *x, int64_t ldx) {
    MmaPlan pl;
    return qtype == CQ_Q4_0 && m >= 2 && m <= 8 && k % 256 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ldx % 4 == 0 && plan_mma(ctx, k, n, 0, 1, 8, pl);
}

cq_status launch_gemv_mma(cq_ctx *ctx, int order, int q8_1, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, const float *bias,
                          float *y, int64_t ldy) {
    MmaPlan pl;
    if (!plan_mma(ctx, k, n, 0, 1, 8, pl)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "small-batch kernel: shape not supported");
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
