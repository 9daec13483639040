// Batches of up to eight activation rows in CQ_ACT_F16 against Q4_0 weights in ONE launch and one weight pass: the
// small-batch streaming skeleton (gemv_mma.cuh) with f16 operands on mma.sync m16n8k16, f32 accumulate.
//
// Numerics are those of the f16 tensor-core GEMMs (gemm_tcgen05.cu, gemm_dequant_tmem.cu): activations rounded to
// f16, every weight dequantized to f16 as (n - 8) * d with ONE rounding, products exact in f32, sums in f32.  The
// reference path is QMatMul's dequantize + f32 matmul (tensor/cpu_backend.go:419-481).
//
//   * A fragments come straight from the raw block in registers.  A word w of eight nibbles n0..n7 gives four f16
//     pairs without a single shift per value: (w & 0x000F000F) | 0x64006400 read as f16 pair is (1024 + n0,
//     1024 + n4), minus 1032 -> (n0 - 8, n4 - 8) exactly; (w & 0x00F000F0) | 0x64006400 is (1024 + 16 n1, 1024 + 16 n5),
//     times 1/16 minus 72 -> (n1 - 8, n5 - 8) exactly; the same on w >> 8 for (n2, n6) and (n3, n7); each pair is then
//     multiplied by (d, d), the one rounding.  The k positions inside an instruction are therefore nibble order
//     (0, 4), (1, 5) for the first and (2, 6), (3, 7) for the second of a block's two instructions, and the activation
//     fragments are built in the same order.
//   * The accumulators run across all blocks of a stage (the scale is inside the operand), so there is no per-block
//     epilogue at all: a block and 16 rows cost the unpacking and two (NG = 1) or four (NG = 2) instructions.
//   * NG column groups of eight rows: only NG = 1 is dispatched.  Two groups (9..16 rows) were measured: the activation
//     fragments of 16 rows take twice the registers, k = 4096 then has to be split over a cluster of two, and the
//     result (19.6 us at 11008 x 4096, 43.6 at 32000 x 4096) loses to the narrow tensor-memory GEMM (17.9 / 29.9).
#include "gemv_mma.cuh"

using namespace mma_gemv;

namespace {

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// The four f16 pairs of a word of eight nibbles, dequantized: (n0, n4), (n1, n5), (n2, n6), (n3, n7), each (n - 8) * d.
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 d2, uint32_t (&out)[4]) {
    const uint32_t w8 = w >> 8;
    uint32_t p0 = (w & 0x000F000Fu) | 0x64006400u, p1 = (w & 0x00F000F0u) | 0x64006400u;
    uint32_t p2 = (w8 & 0x000F000Fu) | 0x64006400u, p3 = (w8 & 0x00F000F0u) | 0x64006400u;
    const __half2 m1032 = __half2half2(__ushort_as_half((unsigned short)0xE408));      // -1032
    const __half2 sixteenth = __half2half2(__ushort_as_half((unsigned short)0x2C00));  // 1/16
    const __half2 m72 = __half2half2(__ushort_as_half((unsigned short)0xD480));        // -72
    const __half2 v0 = __hmul2(__hadd2(*reinterpret_cast<__half2 *>(&p0), m1032), d2);
    const __half2 v1 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p1), sixteenth, m72), d2);
    const __half2 v2 = __hmul2(__hadd2(*reinterpret_cast<__half2 *>(&p2), m1032), d2);
    const __half2 v3 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p3), sixteenth, m72), d2);
    out[0] = *reinterpret_cast<const uint32_t *>(&v0), out[1] = *reinterpret_cast<const uint32_t *>(&v1);
    out[2] = *reinterpret_cast<const uint32_t *>(&v2), out[3] = *reinterpret_cast<const uint32_t *>(&v3);
}

template <int BPW, int ORDER, int NG>
__global__ void __launch_bounds__(MM_THREADS, 1) gemv_mma_f16_kernel(const MmaGemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[MM_MAX_STAGES];
    __shared__ uint64_t bar_empty[MM_MAX_STAGES];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const Geometry geo = geometry(p);
    float *red = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);
    float *ypart = reinterpret_cast<float *>(smem + p.ypart_off);

    pdl_launch_dependents();
    init_ring(p, bar_full, bar_empty);

    if (warp == MM_WARPS) {
        produce(p, geo, smem, bar_full, bar_empty);
    } else if (warp == MM_WARPS + 1) {
        reduce<NG>(p, geo, red, ypart);
    } else {
        // ---- workers ----
        const int g = lane >> 2, q = lane & 3;
        pdl_wait_prior();  // the activations come from the previous kernel in the stream

        // B fragments of this warp's blocks: lane (g, q) holds, per block and column group, the eight activations of
        // row g (+ 8 per group) that stand against its four weight bytes c0..c3, as f16 pairs in the order of the two
        // instructions: (c0.lo, c2.lo), (c0.hi, c2.hi) and (c1.lo, c3.lo), (c1.hi, c3.hi).
        uint32_t bf[BPW][NG][4];
#pragma unroll
        for (int j = 0; j < BPW; ++j) {
            const int lb = warp * BPW + j;
            // the lane's four bytes are two byte pairs, starting at bytes b0 and b1 (both even)
            const int b0 = (j & 1) ? 4 * q : (q < 3 ? 2 + 4 * q : 0), b1 = (j & 1) ? 4 * q + 2 : (q < 3 ? 4 + 4 * q : 14);
#pragma unroll
            for (int gr = 0; gr < NG; ++gr) {
                const int row = gr * 8 + g;
                const bool live = lb < geo.sblocks && row < p.m;
                const float *xb = p.x + (int64_t)(live ? row : 0) * p.ldx + (int64_t)(geo.u0 * 8 + (lb < geo.sblocks ? lb : 0)) * kQK;
                if (ORDER == 0) {  // byte b holds elements 2b (low nibble) and 2b + 1: a pair of bytes is four consecutive floats
                    const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    const float4 f0 = live ? __ldg(reinterpret_cast<const float4 *>(xb + 2 * b0)) : z;  // c0.lo, c0.hi, c1.lo, c1.hi
                    const float4 f1 = live ? __ldg(reinterpret_cast<const float4 *>(xb + 2 * b1)) : z;  // c2.lo, c2.hi, c3.lo, c3.hi
                    bf[j][gr][0] = h2(f0.x, f1.x), bf[j][gr][1] = h2(f0.y, f1.y);
                    bf[j][gr][2] = h2(f0.z, f1.z), bf[j][gr][3] = h2(f0.w, f1.w);
                } else {  // byte b holds elements b (low nibble) and b + 16
                    const float2 z = make_float2(0.0f, 0.0f);
                    const float2 l0 = live ? __ldg(reinterpret_cast<const float2 *>(xb + b0)) : z;       // c0.lo, c1.lo
                    const float2 l1 = live ? __ldg(reinterpret_cast<const float2 *>(xb + b1)) : z;       // c2.lo, c3.lo
                    const float2 h0 = live ? __ldg(reinterpret_cast<const float2 *>(xb + 16 + b0)) : z;  // c0.hi, c1.hi
                    const float2 h1 = live ? __ldg(reinterpret_cast<const float2 *>(xb + 16 + b1)) : z;  // c2.hi, c3.hi
                    bf[j][gr][0] = h2(l0.x, l1.x), bf[j][gr][1] = h2(h0.x, h1.x);
                    bf[j][gr][2] = h2(l0.y, l1.y), bf[j][gr][3] = h2(h0.y, h1.y);
                }
            }
        }

        const uint32_t sel = q < 3 ? 0x3210u : 0x5432u;  // lane 3 of an even block: the upper half of word 0 and the lower half of word 4
        const int word_even = q < 3 ? 1 + q : 0, word_odd = 5 + q;
        const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
        int stage = 0;
        uint32_t phase = 0;
        bool dead = false;
        for (int ps = 0; ps < geo.npass; ++ps) {
            // a warp whose wait gave up keeps walking the loop so that the reducer's barriers still fill up
            if (!dead && !mbar_wait_bounded(full0 + 8 * stage, phase)) {
                if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                dead = true;
            }
            float acc[NG][4];
#pragma unroll
            for (int gr = 0; gr < NG; ++gr) acc[gr][0] = acc[gr][1] = acc[gr][2] = acc[gr][3] = 0.0f;
            if (!dead) {
                const uint32_t *h0p = reinterpret_cast<const uint32_t *>(smem + (size_t)stage * p.stage_bytes + (size_t)g * p.pitch + (size_t)warp * (BPW * kQ4Bytes));
                const uint32_t *h1p = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(h0p) + 8 * (size_t)p.pitch);
                const uint32_t *e0p = h0p + word_even, *e1p = h1p + word_even, *o0p = h0p + word_odd, *o1p = h1p + word_odd;
#pragma unroll
                for (int j = 0; j < BPW; j += 2) {
                    if (warp * BPW + j < geo.sblocks) {  // slices are multiples of eight blocks: a pair is whole or absent
                        constexpr int kPairWords = 2 * kQ4Bytes / 4;  // a pair of blocks is nine words
                        const int wo = (j / 2) * kPairWords;
                        const uint32_t h0 = h0p[wo], t0 = h0p[wo + 4], e0 = e0p[wo], o0 = o0p[wo];
                        const uint32_t h1 = h1p[wo], t1 = h1p[wo + 4], e1 = e1p[wo], o1 = o1p[wo];
                        const uint32_t wv[2][2] = {{__byte_perm(e0, t0, sel), __byte_perm(e1, t1, sel)}, {o0, o1}};
                        // (d, d) of (even block, odd block) x (row g, row g + 8): the scale is the low half of the pair's
                        // first word and the high half of its fifth
                        const uint32_t dd[2][2] = {{__byte_perm(h0, 0u, 0x1010u), __byte_perm(h1, 0u, 0x1010u)},
                                                   {__byte_perm(t0, 0u, 0x3232u), __byte_perm(t1, 0u, 0x3232u)}};
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            uint32_t r0[4], r1[4];
                            dequant_word(wv[b][0], *reinterpret_cast<const __half2 *>(&dd[b][0]), r0);
                            dequant_word(wv[b][1], *reinterpret_cast<const __half2 *>(&dd[b][1]), r1);
                            const uint32_t a0[4] = {r0[0], r1[0], r0[1], r1[1]};  // k = (n0, n4) | (n1, n5)
                            const uint32_t a1[4] = {r0[2], r1[2], r0[3], r1[3]};  // k = (n2, n6) | (n3, n7)
#pragma unroll
                            for (int gr = 0; gr < NG; ++gr) {
                                mma_f16(acc[gr], a0, bf[j + b][gr][0], bf[j + b][gr][1]);
                                mma_f16(acc[gr], a1, bf[j + b][gr][2], bf[j + b][gr][3]);
                            }
                        }
                    }
                }
            }
            park<NG>(red, ps, warp, lane, acc, empty0 + 8 * stage);
            if (++stage == p.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
    }

    if (p.ks > 1) cluster_sum<NG>(p, geo, ypart);
}

template <int BPW, int NG>
cq_status run_f16(cq_ctx *ctx, const MmaGemvParams &p, const MmaPlan &pl, int64_t k) {
    if (p.order == 0) return launch_planned(ctx, gemv_mma_f16_kernel<BPW, 0, NG>, p, pl, k, NG, 8 / NG);
    return launch_planned(ctx, gemv_mma_f16_kernel<BPW, 1, NG>, p, pl, k, NG, 8 / NG);
}

}  // namespace

bool gemv_mma_f16_supported(cq_ctx *ctx, int qtype, int64_t m, int64_t k, int64_t n, const void *w, const float *x, int64_t ldx) {
    MmaPlan pl;
    return qtype == CQ_Q4_0 && m >= 1 && m <= 8 && k % 256 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ldx % 4 == 0 && plan_mma(ctx, k, n, 0, 1, 8, pl);
}

cq_status launch_gemv_mma_f16(cq_ctx *ctx, int order, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, const float *bias,
                              float *y, int64_t ldy) {
    MmaPlan pl;
    if (m > 8 || !plan_mma(ctx, k, n, 0, 1, 8, pl)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "small-batch kernel: shape not supported");
    MmaGemvParams p = {};
    p.w = static_cast<const uint8_t *>(w);
    p.x = x, p.y = y, p.bias = bias;
    p.ldx = ldx, p.ldy = ldy, p.n = n;
    p.nb = (int)(k / kQK), p.m = (int)m, p.order = order == CQ_ORDER_GGML_SPLIT ? 1 : 0, p.act = 2;
    p.err = ctx->dev_err_devptr;
    switch (pl.bpw) {  // the plan may still change its row ranges and stages, never its k slices
    case 2: return run_f16<2, 1>(ctx, p, pl, k);
    case 4: return run_f16<4, 1>(ctx, p, pl, k);
    case 6: return run_f16<6, 1>(ctx, p, pl, k);
    default: return run_f16<8, 1>(ctx, p, pl, k);
    }
}
