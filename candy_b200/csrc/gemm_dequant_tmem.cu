// Quantized GEMM for narrow batches (8 < m <= 128 for Q4_0, <= 64 for Q8_0): Y[m,n] = X[m,k] . W[n,k]^T with the
// weights read from HBM once, as the 18-byte blocks they are stored in.
//
// Same CQ_ACT_F16 numerics as the wide GEMM (f16 activations, weights d*(q-8) rounded once to
// f16, f32 accumulation in the tensor core) but no f16 copy of W ever exists in memory: the
// copy is 3.6 times the size of the blocks and at these batch sizes the GEMM is bound by weight
// bytes, not by the tensor pipe.  Roles are swapped against the wide kernel: the WEIGHT rows are
// the M side of the MMA (128 rows = 128 tensor-memory lanes) and the batch is the N side.
//
// A CTA runs three (two for m > 32) independent pipes, one per 128-row tile of a group of tiles
// that share each slab of X:
//
//   warp 0        TMA: per step one [MPAD x 256] f16 slab of X (four 64-wide boxes, 128-byte
//                 swizzle) and, per pipe, one [128 rows x 144 B] tile of raw blocks (256 values of
//                 k per row; 2-D byte tensor map, no swizzle).  Separate rings, so a stage of raw
//                 blocks is free again as soon as it has been read into registers.
//   4 warps/pipe  dequantize, thread = weight row: nine 16-byte shared loads fetch the row's eight
//                 blocks (row pitch 144 B = 9 x 16 B, odd, so quarter-warps hit eight different
//                 bank groups); nibbles become f16 pairs with one mask-or each (0x6400 | q =
//                 1024 + q), one HSUB2/HFMA2 takes off the 1032 and one HMUL2 applies the block
//                 scale; packed registers go to tensor memory with tcgen05.st as the A operand,
//                 in two halves of 64 columns so the second half is converted while the first
//                 is multiplied.
//   1 lane/pipe   issues tcgen05.mma (A from tensor memory, B = X slab through a shared-memory
//                 descriptor), M=128, N=MPAD, K=16, sixteen per item, into the pipe's own f32
//                 accumulator.  A single thread can start an MMA only every ~90 cycles whatever
//                 its shape -- far too slow for narrow N -- hence one issuer per pipe.
//   4 warps       epilogue: tcgen05.ld, store.  Lane = weight row, so for each batch row a warp
//                 writes 32 consecutive floats.
//
// Every mbarrier is waited on by the same threads for each of its phases, in order: a parity
// wait cannot tell phase k from phase k-2, so no barrier is shared between alternating waiters.
//
// Inside a 32-block the nibble extraction yields the values in a fixed permuted order; X is
// written to f16 scratch in the same order by the conversion pre-pass (a dot product does not
// care), which also serves the ggml element order with a different table.
//
// Work is the list of (group of tiles, 256-wide chunk of k) steps, group-major; every CTA takes
// an equal contiguous share, so the SMs finish together whatever n and k are.  A share is cut
// into segments at group boundaries: a segment that spans a group's whole k range is written to
// y, the others (at most two per CTA) go to scratch and a small kernel adds them in CTA order.
// The rings, the A buffers and the accumulators keep cycling across segments.  Every wait is
// bounded.
#include "common.cuh"
#include "tcgen05.cuh"


namespace {

constexpr int FT_ROWS = 128;                   // weight rows per tile = tensor-memory lanes
constexpr int FT_KCHUNK = 256;                 // values of k per item
constexpr int FT_ACOLS = FT_KCHUNK / 2;        // 128 columns of A per pipe (two halves of 64)

template <int QT, int MPAD>
struct FtCfg {
    static constexpr int kBlockBytes = QT == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    static constexpr int kRowChunk = 8 * kBlockBytes;        // bytes of one row per item: 144 (Q4_0) / 272 (Q8_0)
    static constexpr int kWBytes = FT_ROWS * kRowChunk;      // one stage of raw blocks: 18 432 / 34 816
    static constexpr int kHalfWords = kRowChunk / 8;         // 32-bit words a thread loads: four blocks = 18 / 34
    // Independent pipes per CTA, each = (tile of the group, a TMA warp, four dequantizing warps, two
    // MMA-issuing lanes with an accumulator each, 128 columns of A in two halves).
    static constexpr int kPipes = 2;
    static constexpr int kGroupRows = kPipes * FT_ROWS;
    static constexpr int kXBytes = 4 * MPAD * 128;  // one slab of X: four 64-wide boxes of MPAD rows
    static constexpr int kIssuers = MPAD >= 128 ? 1 : 2;  // MMA-issuing lanes per pipe, an accumulator each
    static constexpr int kXStages = MPAD >= 64 ? 2 : 3;
    static constexpr int kWStages = (MPAD >= 128 || QT == CQ_Q8_0) ? 2 : 4;  // per pipe
    static constexpr size_t kSmem = (size_t)kPipes * kWStages * kWBytes + (size_t)kXStages * kXBytes + 1024 + 512;
    static_assert(kSmem <= 232448, "shared memory");
    // tensor memory: 128 columns of A per pipe, then two accumulators of MPAD columns per pipe
    static constexpr int kDCol0 = kPipes * FT_ACOLS;
    static constexpr int kWarpW0 = 2;                        // warps 0,1 load X; then one TMA warp per pipe
    static constexpr int kWarpMma0 = kWarpW0 + kPipes;       // two issuing warps per pipe
    static constexpr int kWarpDq0 = kWarpMma0 + kIssuers * kPipes;  // eight dequantizing warps per pipe: four per half of an item
    static constexpr int kWarpEp0 = kWarpDq0 + 8 * kPipes;   // four epilogue warps
    static constexpr int kThreads = 32 * (kWarpEp0 + 4);
    static_assert(kDCol0 + kIssuers * kPipes * MPAD <= 512, "tensor memory");
};

// Position p of a block's 32 values, in the order the dequantizing threads emit them, holds
// original element kPerm[order][p].
__constant__ uint8_t kPerm[3][32] = {
    {0, 4, 1, 5, 2, 6, 3, 7, 8, 12, 9, 13, 10, 14, 11, 15, 16, 20, 17, 21, 18, 22, 19, 23, 24, 28, 25, 29, 26, 30, 27, 31},
    {0, 2, 16, 18, 1, 3, 17, 19, 4, 6, 20, 22, 5, 7, 21, 23, 8, 10, 24, 26, 9, 11, 25, 27, 12, 14, 28, 30, 13, 15, 29, 31},
    // Q8_0: bytes convert in place, natural order
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24, 25, 26, 27, 28, 29, 30, 31}};

// X [m,k] f32 -> f16 with each 32-group permuted; one thread per eight output positions.
__global__ void __launch_bounds__(256) x_to_f16_perm_kernel(const float *__restrict__ x, int64_t m, int64_t k, int64_t ldx, int order,
                                                          __half *__restrict__ out) {
    pdl_launch_dependents();  // the GEMM behind this kernel starts fetching weights meanwhile
    pdl_wait_prior();         // x comes from the previous kernel; the scratch this writes may still be read by it
    const int64_t per_row = k / 8, total = m * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / per_row, o8 = i - row * per_row;  // output positions 8*o8 .. 8*o8+7 of the row
        const float *src = x + row * ldx + (o8 >> 2) * 32;
        const uint8_t *perm = kPerm[order] + (o8 & 3) * 8;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(src[perm[2 * j]], src[perm[2 * j + 1]]);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(out + row * k + o8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Groups of tiles whose k range was shared between CTAs: y[m][j] = sum of the CTAs' partials, in
// CTA order.  CTA i owns steps [i*per_cta, (i+1)*per_cta); a group's steps are [t*nchunks, (t+1)*nchunks).
// One block per (group, batch row), one thread per four columns.
__global__ void __launch_bounds__(64) shared_group_sum_kernel(const float *__restrict__ part, int64_t m, int64_t n, int nchunks, int per_cta,
                                                            float *__restrict__ y, int64_t ldy) {
    constexpr int kGroupRows = 256;
    pdl_launch_dependents();
    pdl_wait_prior();
    const int t = blockIdx.x, row = blockIdx.y;
    const int first = (t * nchunks) / per_cta, last = ((t + 1) * nchunks - 1) / per_cta;
    if (first == last) return;  // one CTA had the group's whole k range and wrote y itself
    const int r = threadIdx.x * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = first; c <= last; ++c) {
        const int slot = 2 * c + (((c * per_cta) / nchunks == t) ? 0 : 1);
        const float4 v = *reinterpret_cast<const float4 *>(part + ((int64_t)slot * m + row) * kGroupRows + r);
        acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    const int64_t j = (int64_t)t * kGroupRows + r;
    float *dst = y + (int64_t)row * ldy + j;
    if (j + 3 < n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<float4 *>(dst) = acc;
    } else {
        if (j < n) dst[0] = acc.x;
        if (j + 1 < n) dst[1] = acc.y;
        if (j + 2 < n) dst[2] = acc.z;
        if (j + 3 < n) dst[3] = acc.w;
    }
}

// Eight nibbles of one word -> four f16 pairs d*(q-8), in the order (v0,v4)(v1,v5)(v2,v6)(v3,v7).
__device__ __forceinline__ void dequant_word(uint32_t n, __half2 d2, uint32_t *out) {
    const __half2 k1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 k16th = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));
    const __half2 km72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));
    const uint32_t n8 = n >> 8;
    uint32_t t0 = (n & 0x000F000Fu) | 0x64006400u;   // 1024 + q
    uint32_t t1 = (n & 0x00F000F0u) | 0x64006400u;   // 1024 + 16 q
    uint32_t t2 = (n8 & 0x000F000Fu) | 0x64006400u;
    uint32_t t3 = (n8 & 0x00F000F0u) | 0x64006400u;
    __half2 q0 = __hsub2(*reinterpret_cast<__half2 *>(&t0), k1032);
    __half2 q1 = __hfma2(*reinterpret_cast<__half2 *>(&t1), k16th, km72);
    __half2 q2 = __hsub2(*reinterpret_cast<__half2 *>(&t2), k1032);
    __half2 q3 = __hfma2(*reinterpret_cast<__half2 *>(&t3), k16th, km72);
    q0 = __hmul2(q0, d2), q1 = __hmul2(q1, d2), q2 = __hmul2(q2, d2), q3 = __hmul2(q3, d2);
    out[0] = *reinterpret_cast<uint32_t *>(&q0);
    out[1] = *reinterpret_cast<uint32_t *>(&q1);
    out[2] = *reinterpret_cast<uint32_t *>(&q2);
    out[3] = *reinterpret_cast<uint32_t *>(&q3);
}

// Four int8 of one word -> two f16 pairs d*q, natural order: q ^ 0x80 = q + 128 as an unsigned byte,
// a byte permute puts it under a 0x64 high byte (1024 + 128 + q), one HSUB2 removes the 1152.
__device__ __forceinline__ void dequant_word_q8(uint32_t n, __half2 d2, uint32_t *out) {
    const __half2 k1152 = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
    const uint32_t u = n ^ 0x80808080u;
    uint32_t t0 = __byte_perm(u, 0x64646464u, 0x4140);  // bytes: u0, 0x64, u1, 0x64
    uint32_t t1 = __byte_perm(u, 0x64646464u, 0x4342);  // bytes: u2, 0x64, u3, 0x64
    __half2 q0 = __hsub2(*reinterpret_cast<__half2 *>(&t0), k1152);
    __half2 q1 = __hsub2(*reinterpret_cast<__half2 *>(&t1), k1152);
    q0 = __hmul2(q0, d2), q1 = __hmul2(q1, d2);
    out[0] = *reinterpret_cast<uint32_t *>(&q0);
    out[1] = *reinterpret_cast<uint32_t *>(&q1);
}

struct FtParams {
    float *y;          // [m, n], row pitch ldy: groups whose whole k range one CTA owns are written here directly
    int64_t ldy;
    float *part;       // partial sums of groups shared between CTAs: [2 * ctas][m][group rows]
    int m, n, nchunks;
    int total, per_cta;  // (group, chunk) steps in all and per CTA
    int *err;
};

template <int QT, int MPAD>
__global__ void __launch_bounds__(FtCfg<QT, MPAD>::kThreads, 1)
    qgemm_tmem_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const FtParams p) {
    using Cfg = FtCfg<QT, MPAD>;
    constexpr int FT_WBYTES = Cfg::kWBytes, ROWCHUNK = Cfg::kRowChunk, HW = Cfg::kHalfWords;
    constexpr int WSP = Cfg::kWStages, XST = Cfg::kXStages, PIPES = Cfg::kPipes, DCOL0 = Cfg::kDCol0, GROUP_ROWS = Cfg::kGroupRows;
    constexpr int IPP = Cfg::kIssuers, NISS = IPP * PIPES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_w = smem;                                          // per pipe WSP stages of raw blocks
    uint8_t *smem_x = smem + (size_t)PIPES * WSP * FT_WBYTES;        // XST slabs of X
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_x + (size_t)XST * Cfg::kXBytes);
    uint64_t *w_full = bars, *w_empty = w_full + PIPES * WSP, *x_full = w_empty + PIPES * WSP, *x_empty = x_full + XST;
    uint64_t *a_full = x_empty + XST, *a_empty = a_full + 2 * PIPES, *d_full = a_empty + 2 * PIPES, *d_empty = d_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(d_empty + 1);
    uint32_t *sink = tmem_slot + 1;  // one word per warp: target of the stores that pin load completion (see the dequantizing warps)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Chained launch: the next kernel may become resident now.  Here, only the warps that touch what
    // earlier kernels produce or still read wait for them: the X loaders (X scratch) and the epilogue
    // (y, partial sums).  The raw blocks are nobody's output, so their TMA warps start at once.
    pdl_launch_dependents();
    // this CTA's steps [g0, g1) of the (group, chunk) list: equal shares, so the SMs finish together
    const int g0 = blockIdx.x * p.per_cta, g1 = min(g0 + p.per_cta, p.total);
    const int nsteps = g1 - g0;

    // Every barrier below is waited on by the same threads for each of its phases, in order
    // (a parity wait cannot tell phase k from phase k-2).
    if (threadIdx.x == 0) {
        for (int s = 0; s < PIPES * WSP; ++s) {
            mbar_init(smem_u32(&w_full[s]), 1);
            mbar_init(smem_u32(&w_empty[s]), 8);  // the pipe's eight dequantizing warps
        }
        for (int s = 0; s < XST; ++s) {
            mbar_init(smem_u32(&x_full[s]), 2);   // the two X-loading warps
            mbar_init(smem_u32(&x_empty[s]), NISS);
        }
        for (int b = 0; b < 2 * PIPES; ++b) {  // per pipe: one per half of an item
            mbar_init(smem_u32(&a_full[b]), 4);
            mbar_init(smem_u32(&a_empty[b]), IPP);  // the pipe's issuers
        }
        mbar_init(smem_u32(&d_full[0]), NISS);
        mbar_init(smem_u32(&d_empty[0]), 4);
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // the segment of the list that starts at step g: stays inside one group of tiles
    auto segment = [&](int g, int &group, int &c0, int &cn) {
        group = g / p.nchunks;
        c0 = g - group * p.nchunks;
        cn = min(p.nchunks - c0, g1 - g);
    };

    // One thread can start a TMA copy or a tcgen05.mma only every few hundred / ~100 cycles, so
    // both jobs are spread over several warps: two for X, one per pipe for the raw blocks, two
    // issuers per pipe (each with its own accumulator: MMAs of different threads are unordered).
    if (warp < Cfg::kWarpW0) {
        // ---- TMA, X: warp 0 loads boxes 0,1 of every slab, warp 1 boxes 2,3 -------------------------
        if (lane == 0) {
            pdl_wait_prior();
            int step = 0;
            bool ok = true;
            for (int g = g0; g < g1 && ok;) {
                int group, c0, cn;
                segment(g, group, c0, cn);
                g += cn;
                for (int c = 0; c < cn; ++c, ++step) {
                    const int xs = step % XST;
                    if (step >= XST && !mbar_wait_sleep(smem_u32(&x_empty[xs]), ((step / XST) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    const uint32_t xbar = smem_u32(&x_full[xs]);
                    mbar_expect_tx(xbar, Cfg::kXBytes / 2);
#pragma unroll
                    for (int a = 2 * warp; a < 2 * warp + 2; ++a)
                        tma_load_2d(smem_u32(smem_x + (size_t)xs * Cfg::kXBytes + a * MPAD * 128), &tmX, (c0 + c) * FT_KCHUNK + a * 64, 0, xbar);
                }
            }
            if (ok)  // leave only when nothing is in flight into this CTA's shared memory
                for (int i = step > XST ? step - XST : 0; i < step; ++i)
                    if (!mbar_wait_sleep(smem_u32(&x_full[i % XST]), (i / XST) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        break;
                    }
        }
    } else if (warp < Cfg::kWarpMma0) {
        // ---- TMA, raw blocks of pipe q: one [128 x 144 B] tile per step ------------------------------
        if (lane == 0) {
            const int q = warp - Cfg::kWarpW0;
            int step = 0;
            bool ok = true;
            for (int g = g0; g < g1 && ok;) {
                int group, c0, cn;
                segment(g, group, c0, cn);
                g += cn;
                for (int c = 0; c < cn; ++c, ++step) {
                    const int s = q * WSP + step % WSP;
                    if (step >= WSP && !mbar_wait_sleep(smem_u32(&w_empty[s]), ((step / WSP) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&w_full[s]);
                    mbar_expect_tx(bar, FT_WBYTES);
                    // tiles past the last row are outside the tensor: zero fill, no traffic
                    tma_load_2d(smem_u32(smem_w + (size_t)s * FT_WBYTES), &tmW, (c0 + c) * (ROWCHUNK / 2), (group * PIPES + q) * FT_ROWS, bar);  // x in 2-byte elements
                }
            }
            if (ok)
                for (int i = step > WSP ? step - WSP : 0; i < step; ++i)
                    if (!mbar_wait_sleep(smem_u32(&w_full[q * WSP + i % WSP]), (i / WSP) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        break;
                    }
        }
    } else if (warp < Cfg::kWarpDq0) {
        // ---- MMA: issuer (pipe q, parity e) takes every second K=16 step of both halves ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(FT_ROWS, MPAD);
            const int iss = warp - Cfg::kWarpMma0, q = iss / IPP, e = iss % IPP;
            int step = 0, seg = 0;
            bool ok = true;
            const uint32_t acc = tmem_base + (uint32_t)(DCOL0 + iss * MPAD);
            for (int g = g0; g < g1 && ok; ++seg) {
                int group, c0, cn;
                segment(g, group, c0, cn);
                g += cn;
                if (seg >= 1 && !mbar_wait_sleep(smem_u32(&d_empty[0]), (seg - 1) & 1, 100)) {  // epilogue has read the accumulators
                    atomicExch(p.err, kDevErrMma);
                    break;
                }
                tc_fence_after();
                for (int c = 0; c < cn && ok; ++c, ++step) {
                    const int xs = step % XST;
                    if (!mbar_wait_sleep(smem_u32(&x_full[xs]), (step / XST) & 1, 40)) {
                        atomicExch(p.err, kDevErrFullWait);
                        ok = false;
                        break;
                    }
                    const uint64_t bdesc = smem_desc_k128(smem_u32(smem_x + (size_t)xs * Cfg::kXBytes));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (!mbar_wait_sleep(smem_u32(&a_full[2 * q + h]), step & 1, 20)) {
                            atomicExch(p.err, kDevErrFullWait);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t a_t = tmem_base + (uint32_t)(q * FT_ACOLS + h * 64);
                        {
#pragma unroll
                            for (int j2 = 0; j2 < 8 / IPP; ++j2) {
                                const int j = IPP * j2 + e;  // K=16 step inside the half
                                const int jj = 8 * h + j;  // ... inside the item: X box jj/4, 32-byte column jj%4
                                tc_mma_f16_ts(acc, a_t + 8 * j, bdesc + (uint64_t)((jj >> 2) * (MPAD * 128 / 16) + (jj & 3) * 2), idesc, (c | h | j2) != 0);
                            }
                        }
                        tc_commit(smem_u32(&a_empty[2 * q + h]));
                    }
                    tc_commit(smem_u32(&x_empty[xs]));
                }
                tc_commit(smem_u32(&d_full[0]));
            }
        }
    } else if (warp < Cfg::kWarpEp0) {
        // ---- dequantize: per pipe four warps for each half of an item, thread = weight row ----------
        const int dw = warp - Cfg::kWarpDq0, q = dw >> 3, h = (dw >> 2) & 1;
        const int quarter = warp & 3;  // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        for (int step = 0; step < nsteps; ++step) {
            const int s = q * WSP + step % WSP;
            if (!mbar_wait_sleep(smem_u32(&w_full[s]), (step / WSP) & 1, 60)) {
                if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                break;
            }
            // Four blocks = 72 / 136 bytes, 8-byte aligned.
            uint32_t w[HW];
            const uint32_t src = smem_u32(smem_w + (size_t)s * FT_WBYTES + r * ROWCHUNK + h * (ROWCHUNK / 2));
#pragma unroll
            for (int i = 0; i < HW / 2; ++i)
                asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w[2 * i]), "=r"(w[2 * i + 1]) : "r"(src + 8 * i) : "memory");
            // The stage may be refilled once the raw blocks are in registers -- really in registers.
            // Neither the compiler nor the arrive waits for shared-memory loads that are still in
            // flight (observed: rows read from a stage the next TMA copy was already overwriting), so
            // an instruction that needs every loaded word, and that cannot be dropped, goes first:
            // instructions issue in order, and this store cannot issue before its operand exists.
            {
                uint32_t all = w[0];
#pragma unroll
                for (int i = 1; i < HW; ++i) all ^= w[i];
                asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem_u32(&sink[warp])), "r"(all) : "memory");
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&w_empty[s]));
            if (step >= 1 && !mbar_wait_sleep(smem_u32(&a_empty[2 * q + h]), (step - 1) & 1, 20)) {
                if (lane == 0) atomicExch(p.err, kDevErrMma);
                break;
            }
            tc_fence_after();
            const uint32_t a_t = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(q * FT_ACOLS + h * 64);
            {
#pragma unroll
                for (int pr = 0; pr < 2; ++pr) {
                    // two blocks in 9 (Q4_0) / 17 (Q8_0) words: the first starts on a word, its values two
                    // bytes in; the second starts two bytes into the middle word, its values on the next one
                    constexpr int PW = HW / 2, VW = (PW - 1) / 2;  // words per pair, words of values per block
                    const uint32_t *wq = w + PW * pr;
                    uint32_t o[16];
                    {
                        const __half dh = __ushort_as_half((unsigned short)(wq[0] & 0xFFFFu));
                        const __half2 d2 = __halves2half2(dh, dh);
#pragma unroll
                        for (int j = 0; j < VW; ++j) {
                            const uint32_t v = __funnelshift_r(wq[j], wq[j + 1], 16);
                            if (QT == CQ_Q4_0) dequant_word(v, d2, o + 4 * j);
                            else dequant_word_q8(v, d2, o + 2 * j);
                        }
                        tmem_st16(a_t + (uint32_t)((2 * pr) * 16), o);
                    }
                    {
                        const __half dh = __ushort_as_half((unsigned short)(wq[VW] >> 16));
                        const __half2 d2 = __halves2half2(dh, dh);
#pragma unroll
                        for (int j = 0; j < VW; ++j) {
                            if (QT == CQ_Q4_0) dequant_word(wq[VW + 1 + j], d2, o + 4 * j);
                            else dequant_word_q8(wq[VW + 1 + j], d2, o + 2 * j);
                        }
                        tmem_st16(a_t + (uint32_t)((2 * pr + 1) * 16), o);
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&a_full[2 * q + h]));
        }
    } else {
        // ---- epilogue: two accumulators per tile of the group, lane = weight row ---------------------
        pdl_wait_prior();
        const int quarter = warp & 3;
        int seg = 0;
        for (int g = g0; g < g1; ++seg) {
            int group, c0, cn;
            segment(g, group, c0, cn);
            const bool first_seg = g == g0;
            g += cn;
            if (!mbar_wait_sleep(smem_u32(&d_full[0]), seg & 1, 500)) {
                if (lane == 0) atomicExch(p.err, kDevErrMma);
                break;
            }
            tc_fence_after();
            // whole k range -> y; otherwise one of this CTA's two partial slots (0: the segment its share starts with)
            const bool direct = cn == p.nchunks;
            const int64_t ld = direct ? p.ldy : GROUP_ROWS;
#pragma unroll 1
            for (int t = 0; t < PIPES; ++t) {
                const int row_in_group = t * FT_ROWS + quarter * 32 + lane;
                const int row = group * GROUP_ROWS + row_in_group;
                float *dst = direct ? p.y + row : p.part + ((int64_t)(2 * blockIdx.x + (first_seg ? 0 : 1)) * p.m) * GROUP_ROWS + row_in_group;
#pragma unroll 1
                for (int c = 0; c < MPAD / 16; ++c) {
                    uint32_t v0[16], v1[16];
                    const uint32_t col = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(DCOL0 + IPP * t * MPAD + c * 16);
                    tmem_ld16(col, v0);
                    if (IPP == 2) {
                        tmem_ld16(col + MPAD, v1);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v1[i] = 0u;
                    }
                    if (t == PIPES - 1 && c == MPAD / 16 - 1) {  // everything is in registers: the issuers may overwrite the accumulators
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&d_empty[0]));
                    }
                    if (row < p.n) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c * 16 + i < p.m) dst[(int64_t)(c * 16 + i) * ld] = __uint_as_float(v0[i]) + __uint_as_float(v1[i]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// The raw blocks as a 2-D tensor of 2-byte elements (a Q8_0 item is 272 bytes per row, more than the 256
// elements a box may span in 1-byte elements): box = one item of 128 rows.
bool make_w_map(CUtensorMap *map, const void *w, int64_t n, int64_t row_bytes, int row_chunk) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 2), (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(row_chunk / 2), (cuuint32_t)FT_ROWS};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_x_map(CUtensorMap *map, const void *x16, int64_t m, int64_t k, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launch with programmatic stream serialization: the kernel may become resident while its predecessor
// is still running; whatever depends on earlier work waits with griddepcontrol.wait inside the kernel.
template <typename Kern, typename... Args>
cq_status launch_chained(cq_ctx *ctx, Kern kern, dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, args...));
    return CQ_OK;
}

template <int QT, int MPAD>
cq_status run_ft(cq_ctx *ctx, const CUtensorMap &tmW, const CUtensorMap &tmX, const FtParams &p, unsigned ctas) {
    static thread_local int configured = -1;
    if (configured != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(qgemm_tmem_kernel<QT, MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FtCfg<QT, MPAD>::kSmem));
        configured = ctx->device;
    }
    return launch_chained(ctx, qgemm_tmem_kernel<QT, MPAD>, dim3(ctas), dim3(FtCfg<QT, MPAD>::kThreads), FtCfg<QT, MPAD>::kSmem, tmW, tmX, p);
}

}  // namespace

bool qgemm_dequant_tmem_supported(int qtype, int64_t m, int64_t k, const void *w) {
    // Q8_0 stages are twice as large: no room for the 128-row X slabs next to them, so a Q8_0 batch of
    // 65..128 rows runs as two 64-row passes (the second pass finds the weights in L2)
    return (qtype == CQ_Q4_0 || qtype == CQ_Q8_0) && m >= 1 && m <= 128 && k % FT_KCHUNK == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

cq_status launch_qgemm_dequant_tmem(cq_ctx *ctx, int qtype, int order, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, float *y,
                                    int64_t ldy) {
    if ((reinterpret_cast<uintptr_t>(x) & 3) != 0 || (reinterpret_cast<uintptr_t>(y) & 3) != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemm: misaligned pointer");
    if (n > 0x7FFFFFFF || k > 0x7FFFFFFF) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: dimension beyond 2^31");
    if (qtype == CQ_Q8_0 && m > 64) {
        cq_status s = launch_qgemm_dequant_tmem(ctx, qtype, order, x, 64, k, ldx, w, n, y, ldy);
        if (s != CQ_OK) return s;
        return launch_qgemm_dequant_tmem(ctx, qtype, order, x + 64 * ldx, m - 64, k, ldx, w, n, y + 64 * ldy, ldy);
    }
    const int mpad = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
    const int group_rows = FtCfg<CQ_Q4_0, 32>::kGroupRows;
    const int ngroups = (int)((n + group_rows - 1) / group_rows);
    const int nchunks = (int)(k / FT_KCHUNK);
    const int64_t total = (int64_t)ngroups * nchunks;
    if (total > 0x3FFFFFFF) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: too many tiles");
    // equal shares of the (group, chunk) list per CTA; at least two steps (eight tile-chunks) each
    int64_t per_cta = (total + ctx->sm_count - 1) / ctx->sm_count;
    if (per_cta < 2) per_cta = total < 2 ? total : 2;
    const unsigned ctas = (unsigned)((total + per_cta - 1) / per_cta);
    const bool shared_tiles = per_cta % nchunks != 0;
    const size_t x16_bytes = (((size_t)m * k * 2) + 1023) & ~size_t(1023);
    const size_t part_bytes = shared_tiles ? (size_t)2 * ctas * m * group_rows * 4 : 0;
    cq_status s = cq_reserve_scratch(ctx, x16_bytes + part_bytes);
    if (s != CQ_OK) return s;
    __half *x16 = static_cast<__half *>(ctx->scratch);
    float *part = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->scratch) + x16_bytes);
    {
        const int64_t items = m * (k / 8);
        const unsigned cap = (unsigned)ctx->sm_count * 8;
        const unsigned grid = (unsigned)((items + 255) / 256 < cap ? (items + 255) / 256 : cap);
        s = launch_chained(ctx, x_to_f16_perm_kernel, dim3(grid), dim3(256), 0, x, m, k, ldx, qtype == CQ_Q4_0 ? order : 2, x16);
        if (s != CQ_OK) return s;
    }
    CUtensorMap tmW, tmX;
    const int bb = qtype == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    if (!make_w_map(&tmW, w, n, (k / 32) * bb, 8 * bb) || !make_x_map(&tmX, x16, m, k, mpad))
        return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
    FtParams p;
    p.y = y, p.ldy = ldy, p.part = part;
    p.m = (int)m, p.n = (int)n, p.nchunks = nchunks, p.total = (int)total, p.per_cta = (int)per_cta;
    p.err = ctx->dev_err_devptr;
    if (qtype == CQ_Q4_0) {
        if (mpad == 16) s = run_ft<CQ_Q4_0, 16>(ctx, tmW, tmX, p, ctas);
        else if (mpad == 32) s = run_ft<CQ_Q4_0, 32>(ctx, tmW, tmX, p, ctas);
        else if (mpad == 64) s = run_ft<CQ_Q4_0, 64>(ctx, tmW, tmX, p, ctas);
        else s = run_ft<CQ_Q4_0, 128>(ctx, tmW, tmX, p, ctas);
    } else {
        if (mpad == 16) s = run_ft<CQ_Q8_0, 16>(ctx, tmW, tmX, p, ctas);
        else if (mpad == 32) s = run_ft<CQ_Q8_0, 32>(ctx, tmW, tmX, p, ctas);
        else s = run_ft<CQ_Q8_0, 64>(ctx, tmW, tmX, p, ctas);
    }
    if (s != CQ_OK) return s;
    if (shared_tiles) {
        static_assert(FtCfg<CQ_Q4_0, 16>::kGroupRows == 256 && FtCfg<CQ_Q8_0, 64>::kGroupRows == 256 && FtCfg<CQ_Q4_0, 128>::kGroupRows == 256, "sum kernel layout");
        s = launch_chained(ctx, shared_group_sum_kernel, dim3((unsigned)ngroups, (unsigned)m), dim3(64), 0, (const float *)part, m, n, nchunks, (int)per_cta, y, ldy);
        if (s != CQ_OK) return s;
    }
    return CQ_OK;
}
