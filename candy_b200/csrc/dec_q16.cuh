// The default activation decoder of the decode GEMV kernels: 16-bit block fixed point (see gemv_kernels.cu).
// Shared by the streaming GEMV kernels and the persistent decode-step kernel.
#pragma once
#include "common.cuh"

namespace {

constexpr int kXPerThread = 64;  // activations a consumer thread keeps in registers

// Which activation (0..31 of its block) meets byte lane t of packed word wi: Q4_0 low / high
// nibble vectors, or Q8_0 bytes (hi unused).
template <int QT, int ORDER>
__host__ __device__ constexpr int act_elem(int wi, int t, int hi) {
    if (QT == CQ_Q8_0) return 4 * wi + t;
    const int j = 4 * wi + t;  // data byte inside the block
    return (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j + hi : j + 16 * hi;
}

// ---- default decoder: 16-bit block fixed point --------------------------------------------
// Every 32-block of activations is scaled once to 16-bit integers,  X = rint(x * 32767 / amax),
// |x - X * amax/32767| <= amax / 65534, and split into a signed high byte and an unsigned low
// byte (X = 256 * hi + lo).  A block's dot product is then exact integer arithmetic,
//     sum_i n_i X_i = 256 * dp4a(n, hi) + dp4a(n, lo),
// four weights per instruction and byte plane, followed by one int -> float conversion and two
// multiplies per block.  Against candy's CPU path the result differs by the 16-bit rounding
// of the activations (about 1e-5 of max|y| on Gaussian data) and by summation order.
// Setting the state up costs ~5 instructions per activation, a third of the slice decoder.
template <int QT, int ORDER>
struct DecQ16 {
    static constexpr int kWords = (QT == CQ_Q4_0) ? 9 : 17;
    static constexpr int kBlkWords = (QT == CQ_Q4_0) ? 4 : 8;
    static constexpr int kVecs = (QT == CQ_Q4_0) ? 2 : 1;
    static constexpr bool kCoop = true;
    static constexpr bool kSplitStage = true;
    // 8 hi words, 8 lo words, scale, bias.  A thread's two blocks are 36 words: 16-byte aligned, and at this
    // stride the eight lanes of a 128-bit shared-memory load phase fall on disjoint banks (40 words collide two ways).
    static constexpr int kStateWordsPerBlock = 18;
    int qh[2][kBlkWords][kVecs];  // high bytes (signed), lane order matching the weight bytes
    int ql[2][kBlkWords][kVecs];  // low bytes (unsigned)
    float d16[2];                 // amax / 32767 per block
    int bias[2];                  // -8 * sum X for Q4_0, 0 for Q8_0

    // low 16 bits of each input = X (two's complement): returns the packed low / high bytes
    __device__ __forceinline__ static void pack_planes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t &lo, uint32_t &hi) {
        const uint32_t ab = __byte_perm(a, b, 0x5410), cd = __byte_perm(c, d, 0x5410);
        lo = __byte_perm(ab, cd, 0x6420);
        hi = __byte_perm(ab, cd, 0x7531);
    }
    __device__ __forceinline__ static int plane_sum(uint32_t lo, uint32_t hi) {  // sum of the four X
        return 256 * __dp4a((int)hi, 0x01010101, 0) + (int)__dp4a(lo, 0x01010101u, 0u);
    }
    __device__ __forceinline__ static uint32_t to_fixed(float x, float inv) {
        return __float_as_uint(fminf(x * inv, 32767.0f) + 12582912.0f);  // 1.5 * 2^23: rint into the mantissa
    }

    // Cooperative set-up: item = block * 4 + quarter, 8 activations per lane, four adjacent
    // lanes make one block.  All 32 lanes of the warp must call this together.
    __device__ __forceinline__ static void load_quarter(const float *x, int item, bool valid, float (&r)[8]) {
        if (valid) {
            // plain loads: the source is global memory or, with a fused norm, this CTA's shared memory
            const float4 a = reinterpret_cast<const float4 *>(x)[2 * item];
            const float4 b = reinterpret_cast<const float4 *>(x)[2 * item + 1];
            r[0] = a.x, r[1] = a.y, r[2] = a.z, r[3] = a.w, r[4] = b.x, r[5] = b.y, r[6] = b.z, r[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = 0.0f;
        }
    }
    __device__ __forceinline__ static void stage_quarter(const float *x, int item, bool valid, uint32_t *area) {
        float r[8];
        load_quarter(x, item, valid, r);
        stage_quarter_regs(r, item, valid, area);
    }
    __device__ __forceinline__ static void stage_quarter_regs(const float (&r)[8], int item, bool valid, uint32_t *area) {
        const int blk = item >> 2, qd = item & 3;
        int idxA, idxB;  // which of the block's 8 packed words this quarter fills
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) idxA = 2 * qd, idxB = 2 * qd + 1;
        else if (QT == CQ_Q4_0) idxA = (qd < 2) ? 4 * qd : 4 * (qd - 2) + 1, idxB = idxA + 2;
        else idxA = 2 * qd, idxB = 2 * qd + 1;
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(r[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1, 32));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2, 32));
        const float inv = amax > 0.0f ? __fdividef(32767.0f, amax) : 0.0f;
        uint32_t xi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xi[i] = to_fixed(r[i], inv);
        uint32_t la, ha, lb, hb;
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
            pack_planes(xi[0], xi[2], xi[4], xi[6], la, ha);  // low nibbles meet the even values
            pack_planes(xi[1], xi[3], xi[5], xi[7], lb, hb);
        } else {
            pack_planes(xi[0], xi[1], xi[2], xi[3], la, ha);
            pack_planes(xi[4], xi[5], xi[6], xi[7], lb, hb);
        }
        int xsum = plane_sum(la, ha) + plane_sum(lb, hb);
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 1, 32);
        xsum += __shfl_xor_sync(0xffffffffu, xsum, 2, 32);
        if (valid) {
            uint32_t *dst = area + blk * kStateWordsPerBlock;
            dst[idxA] = ha, dst[idxB] = hb;
            dst[8 + idxA] = la, dst[8 + idxB] = lb;
            if (qd == 0) {
                dst[16] = __float_as_uint(amax * (1.0f / 32767.0f));
                dst[17] = (QT == CQ_Q4_0) ? (uint32_t)(-8 * xsum) : 0u;
            }
        }
    }

    // src: this thread's two consecutive block states (16-byte aligned).
    __device__ __forceinline__ void load(const uint32_t *src) {
        uint32_t t[2 * kStateWordsPerBlock];
#pragma unroll
        for (int i = 0; i < 2 * kStateWordsPerBlock / 4; ++i) {
            const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
            t[4 * i] = v.x, t[4 * i + 1] = v.y, t[4 * i + 2] = v.z, t[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                qh[blk][j / kVecs][j % kVecs] = (int)t[blk * kStateWordsPerBlock + j];
                ql[blk][j / kVecs][j % kVecs] = (int)t[blk * kStateWordsPerBlock + 8 + j];
            }
            d16[blk] = __uint_as_float(t[blk * kStateWordsPerBlock + 16]);
            bias[blk] = (int)t[blk * kStateWordsPerBlock + 17];
        }
    }

    // Per-thread set-up from the thread's own 64 activations (used when rows do not share a CTA).
    __device__ __forceinline__ void init(const float (&x)[kXPerThread]) {
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < kQK; ++i) amax = fmaxf(amax, fabsf(x[blk * kQK + i]));
            const float inv = amax > 0.0f ? __fdividef(32767.0f, amax) : 0.0f;
            d16[blk] = amax * (1.0f / 32767.0f);
            uint32_t xi[kQK];
#pragma unroll
            for (int i = 0; i < kQK; ++i) xi[i] = to_fixed(x[blk * kQK + i], inv);
            int xsum = 0;
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi)
#pragma unroll
                for (int v = 0; v < kVecs; ++v) {
                    uint32_t lo, hi;
                    pack_planes(xi[act_elem<QT, ORDER>(wi, 0, v)], xi[act_elem<QT, ORDER>(wi, 1, v)],
                                xi[act_elem<QT, ORDER>(wi, 2, v)], xi[act_elem<QT, ORDER>(wi, 3, v)], lo, hi);
                    qh[blk][wi][v] = (int)hi;
                    ql[blk][wi][v] = (int)lo;
                    xsum += plane_sum(lo, hi);
                }
            bias[blk] = (QT == CQ_Q4_0) ? -8 * xsum : 0;
        }
    }

    // weights (signed for Q8_0, small non-negative for Q4_0) times unsigned low bytes
    __device__ __forceinline__ static int dp4a_wu(int w, int lo, int acc) {
        int r;
        asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(lo), "r"(acc));
        return r;
    }

    __device__ __forceinline__ float pass(const uint32_t *sw) const {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
        // data words of block A start 2 bytes into the slice: realign with funnel shifts
        uint32_t dw[2][kBlkWords];
#pragma unroll
        for (int i = 0; i < kBlkWords; ++i) {
            dw[0][i] = __funnelshift_r(w[i], w[i + 1], 16);
            dw[1][i] = w[kBlkWords + 1 + i];
        }
        // plain hardware conversion: a NaN scale gives a NaN sum either way
        const float scale[2] = {__half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu))),
                                __half2float(__ushort_as_half((unsigned short)(w[kBlkWords] >> 16)))};
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            int ah = 0, al = bias[blk];
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi) {
                if (QT == CQ_Q4_0) {
                    const int lo = (int)(dw[blk][wi] & 0x0F0F0F0Fu);
                    const int hi = (int)((dw[blk][wi] >> 4) & 0x0F0F0F0Fu);
                    ah = __dp4a(hi, qh[blk][wi][1], __dp4a(lo, qh[blk][wi][0], ah));
                    al = dp4a_wu(hi, ql[blk][wi][1], dp4a_wu(lo, ql[blk][wi][0], al));
                } else {
                    ah = __dp4a((int)dw[blk][wi], qh[blk][wi][0], ah);
                    al = dp4a_wu((int)dw[blk][wi], ql[blk][wi][0], al);
                }
            }
            const float v = (float)(ah * 256 + al);  // |.| < 2^24: exact
            total = fmaf(scale[blk] * d16[blk], v, total);
        }
        return total;
    }

    // Set-up in two steps for the multi-row kernel, which issues several items' loads before using the first.
    struct QRegs {
        float r[8];
    };
    __device__ __forceinline__ static void qload(const float *x, int item, bool valid, QRegs &q) { load_quarter(x, item, valid, q.r); }
    __device__ __forceinline__ static void qstage(const QRegs &q, int item, bool valid, uint32_t *area) { stage_quarter_regs(q.r, item, valid, area); }

    // The same arithmetic as pass(), split in two for the multi-row kernel: the weight words of a thread's
    // two blocks are loaded and unpacked once (WBlk) and then meet the state of each activation row.
    struct WBlk {
        int a[2][kBlkWords];  // Q4_0: low nibbles, Q8_0: the signed bytes
        int b[2][kBlkWords];  // Q4_0: high nibbles, Q8_0: unused
        float scale[2];
    };
    __device__ __forceinline__ static void unpack(const uint32_t *sw, WBlk &o) {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
#pragma unroll
        for (int i = 0; i < kBlkWords; ++i) {
            const uint32_t d0 = __funnelshift_r(w[i], w[i + 1], 16), d1 = w[kBlkWords + 1 + i];
            if (QT == CQ_Q4_0) {
                o.a[0][i] = (int)(d0 & 0x0F0F0F0Fu), o.b[0][i] = (int)((d0 >> 4) & 0x0F0F0F0Fu);
                o.a[1][i] = (int)(d1 & 0x0F0F0F0Fu), o.b[1][i] = (int)((d1 >> 4) & 0x0F0F0F0Fu);
            } else {
                o.a[0][i] = (int)d0, o.a[1][i] = (int)d1;
                o.b[0][i] = 0, o.b[1][i] = 0;
            }
        }
        o.scale[0] = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
        o.scale[1] = __half2float(__ushort_as_half((unsigned short)(w[kBlkWords] >> 16)));
    }
    __device__ __forceinline__ float dot(const WBlk &wb) const {
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            int ah = 0, al = bias[blk];
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi) {
                if (QT == CQ_Q4_0) {
                    ah = __dp4a(wb.b[blk][wi], qh[blk][wi][1], __dp4a(wb.a[blk][wi], qh[blk][wi][0], ah));
                    al = dp4a_wu(wb.b[blk][wi], ql[blk][wi][1], dp4a_wu(wb.a[blk][wi], ql[blk][wi][0], al));
                } else {
                    ah = __dp4a(wb.a[blk][wi], qh[blk][wi][0], ah);
                    al = dp4a_wu(wb.a[blk][wi], ql[blk][wi][0], al);
                }
            }
            const float v = (float)(ah * 256 + al);  // |.| < 2^24: exact
            total = fmaf(wb.scale[blk] * d16[blk], v, total);
        }
        return total;
    }
};

}  // namespace
