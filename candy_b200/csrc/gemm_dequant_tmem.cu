// Quantized GEMM for narrow batches (8 < m <= 64, Q4_0): Y[m,n] = X[m,k] . W[n,k]^T with the
// weights read from HBM once, as the 18-byte blocks they are stored in.
//
// Same CQ_ACT_F16 numerics as the wide GEMM (f16 activations, weights d*(q-8) rounded once to
// f16, f32 accumulation in the tensor core) but no f16 copy of W ever exists in memory: the
// copy is 3.6 times the size of the blocks and at these batch sizes the GEMM is bound by weight
// bytes, not by the tensor pipe.  Roles are swapped against the wide kernel: the WEIGHT rows are
// the M side of the MMA (128 rows = 128 tensor-memory lanes) and the batch is the N side.
//
//   warp 0        TMA: per stage one [128 rows x 144 B] tile of raw blocks (256 values of k per
//                 row; 2-D byte tensor map, no swizzle) and the matching [MPAD x 256] f16 slab of X
//                 (four 64-wide boxes, 128-byte swizzle).
//   warps 5-20    four groups of 128 threads, thread = (weight row, half a stage): nine 8-byte shared
//                 loads fetch four blocks of the row, nibbles become f16 pairs with one mask-or each
//                 (0x6400 | q = 1024 + q), one HSUB2/HFMA2 takes off the 1032 and one HMUL2
//                 applies the block scale; the 64 packed registers go to tensor memory with
//                 tcgen05.st as the A operand.  Two groups share a stage, pairs of groups alternate
//                 stages; three A buffers.
//   warps 1-4     one lane each issues tcgen05.mma (A from tensor memory, B = X slab through a
//                 shared-memory descriptor), M=128, N=MPAD, K=16: four of a stage's sixteen steps
//                 per issuer, each issuer into its own f32 accumulator (a single thread can start
//                 an MMA only every ~90 cycles, too slow for narrow N); commits free the stage,
//                 the A buffer and, at the end of a unit, hand the accumulators to the epilogue.
//   warps 21-24   epilogue: tcgen05.ld of the four accumulators, add, store.  Lane = weight row, so for each batch row a warp
//                 writes 32 consecutive floats.
//
// Inside a 32-block the nibble extraction yields the values in a fixed permuted order; X is
// written to f16 scratch in the same order by the conversion pre-pass (a dot product does not
// care), which also serves the ggml element order with a different table.
//
// A unit of work is (128-row tile, range of k).  k is split when the tiles alone would not fill
// the SMs; partial sums then go to scratch and a small kernel adds them in a fixed order.  CTAs
// are persistent: units u = blockIdx.x, +gridDim.x, ...; the stage ring, the A buffers and the
// accumulators keep cycling across units.  Every wait is bounded.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int FT_ROWS = 128;                   // weight rows per unit
constexpr int FT_KCHUNK = 256;                 // values of k per stage
constexpr int FT_ROWCHUNK_Q4 = 8 * kQ4Bytes;   // 144 bytes of one row per stage
constexpr int FT_WBYTES = FT_ROWS * FT_ROWCHUNK_Q4;  // 18432
constexpr int FT_ACOLS = FT_KCHUNK / 2;        // 128 columns per A buffer
constexpr int FT_ISSUERS = 4;                  // MMA-issuing warps, each with its own accumulator
constexpr int FT_DQ_WARPS = 16;                // four groups of four warps (one per lane quarter)
constexpr int FT_WARP_DQ0 = 1 + FT_ISSUERS;     // first dequantizing warp
constexpr int FT_WARP_EP0 = FT_WARP_DQ0 + FT_DQ_WARPS;
constexpr int FT_THREADS = 32 * (FT_WARP_EP0 + 4);

template <int MPAD>
struct FtCfg {
    static constexpr int kXBytes = 4 * MPAD * 128;  // four 64-wide boxes of MPAD rows
    static constexpr int kStageBytes = FT_WBYTES + kXBytes;
    static constexpr int kStages = MPAD >= 64 ? 4 : (MPAD >= 32 ? 6 : 8);
    static constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 + 256;
    // tensor memory: A buffers of 128 columns, then one accumulator of MPAD columns per issuing warp
    static constexpr int kABufs = (512 - FT_ISSUERS * MPAD) / FT_ACOLS;  // 3 (MPAD <= 32) or 2 (MPAD = 64)
    static constexpr int kDCol0 = kABufs * FT_ACOLS;
};

// Position p of a block's 32 values, in the order the dequantizing threads emit them, holds
// original element kPerm[order][p].
__constant__ uint8_t kPerm[2][32] = {
    {0, 4, 1, 5, 2, 6, 3, 7, 8, 12, 9, 13, 10, 14, 11, 15, 16, 20, 17, 21, 18, 22, 19, 23, 24, 28, 25, 29, 26, 30, 27, 31},
    {0, 2, 16, 18, 1, 3, 17, 19, 4, 6, 20, 22, 5, 7, 21, 23, 8, 10, 24, 26, 9, 11, 25, 27, 12, 14, 28, 30, 13, 15, 29, 31}};

// X [m,k] f32 -> f16 with each 32-group permuted; one thread per eight output positions.
__global__ void __launch_bounds__(256) x_to_f16_perm_kernel(const float *__restrict__ x, int64_t m, int64_t k, int64_t ldx, int order,
                                                          __half *__restrict__ out) {
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

// y[m][j] = sum over splits of part[s][m][j], in split order.
__global__ void __launch_bounds__(256) splitk_sum_kernel(const float *__restrict__ part, int splits, int64_t m, int64_t n, float *__restrict__ y,
                                                       int64_t ldy) {
    const int64_t total = m * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = part[i];
        for (int s = 1; s < splits; ++s) acc += part[(int64_t)s * total + i];
        const int64_t row = i / n;
        y[row * ldy + (i - row * n)] = acc;
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

struct FtParams {
    float *out;        // y, or the split partials [splits][m][n]
    int64_t ld_out;    // row pitch of out in floats
    int64_t split_stride;  // floats between two splits' partials (0 when not split)
    int m, n, ntiles, nchunks, splits, chunks_per_split;
    int *err;
};

template <int MPAD>
__global__ void __launch_bounds__(FT_THREADS, 1)
    qgemm_q4_0_tmem_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const FtParams p) {
    using Cfg = FtCfg<MPAD>;
    constexpr int STAGES = Cfg::kStages, FT_ABUFS = Cfg::kABufs, FT_DCOL0 = Cfg::kDCol0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * Cfg::kStageBytes);
    uint64_t *w_full = bars, *w_empty = bars + STAGES, *a_full = bars + 2 * STAGES, *a_empty = a_full + FT_ABUFS;
    uint64_t *d_full = a_empty + FT_ABUFS, *d_empty = d_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(d_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nunits = p.ntiles * p.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&w_full[s]), 1);
            mbar_init(smem_u32(&w_empty[s]), 8 + FT_ISSUERS);  // eight dequantizing warps + one commit per issuing warp
        }
        for (int b = 0; b < FT_ABUFS; ++b) {
            mbar_init(smem_u32(&a_full[b]), 8);
            mbar_init(smem_u32(&a_empty[b]), FT_ISSUERS);
        }
        mbar_init(smem_u32(&d_full[0]), FT_ISSUERS);
        mbar_init(smem_u32(&d_empty[0]), 4);
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // unit -> (tile, first chunk, chunk count)
    auto unit_chunks = [&](int u, int &tile, int &c0, int &cn) {
        const int split = u / p.ntiles;
        tile = u - split * p.ntiles;
        c0 = split * p.chunks_per_split;
        cn = min(p.chunks_per_split, p.nchunks - c0);
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
                int tile, c0, cn;
                unit_chunks(u, tile, c0, cn);
                for (int c = 0; c < cn; ++c, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_bounded(smem_u32(&w_empty[s]), ((it / STAGES) - 1) & 1)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    uint8_t *st = smem + (size_t)s * Cfg::kStageBytes;
                    const uint32_t bar = smem_u32(&w_full[s]);
                    mbar_expect_tx(bar, Cfg::kStageBytes);
                    tma_load_2d(smem_u32(st), &tmW, (c0 + c) * FT_ROWCHUNK_Q4, tile * FT_ROWS, bar);
#pragma unroll
                    for (int a = 0; a < 4; ++a)
                        tma_load_2d(smem_u32(st + FT_WBYTES + a * MPAD * 128), &tmX, (c0 + c) * FT_KCHUNK + a * 64, 0, bar);
                }
            }
            const int first = it > STAGES ? it - STAGES : 0;
            for (int i = first; i < it; ++i)
                if (!mbar_wait_bounded(smem_u32(&w_full[i % STAGES]), (i / STAGES) & 1)) {
                    atomicExch(p.err, kDevErrDrain);
                    break;
                }
        }
    } else if (warp < FT_WARP_DQ0) {
        // ---- MMA: four issuing lanes (one per warp), each takes a quarter of a stage's sixteen
        // K=16 steps into its own accumulator.  One thread can start a tcgen05.mma only every ~90
        // cycles whatever its shape, so narrow MMAs need several issuers to keep the pipe fed.
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(FT_ROWS, MPAD);
            const int q = warp - 1;
            int it = 0, ui = 0;
            bool ok = true;
            const uint32_t acc = tmem_base + (uint32_t)(FT_DCOL0 + q * MPAD);
            for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++ui) {
                int tile, c0, cn;
                unit_chunks(u, tile, c0, cn);
                if (ui >= 1 && !mbar_wait_bounded(smem_u32(&d_empty[0]), (ui - 1) & 1)) {  // epilogue has read the accumulators
                    atomicExch(p.err, kDevErrMma);
                    break;
                }
                tc_fence_after();
                for (int c = 0; c < cn; ++c, ++it) {
                    const int s = it % STAGES, ab = it % FT_ABUFS;
                    if (!mbar_wait_bounded(smem_u32(&w_full[s]), (it / STAGES) & 1) ||
                        !mbar_wait_bounded(smem_u32(&a_full[ab]), (it / FT_ABUFS) & 1)) {
                        atomicExch(p.err, kDevErrFullWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    // this issuer's 64 values of k: one 128-byte-swizzled box of X, 32 columns of A
                    const uint64_t bdesc = smem_desc_k128(smem_u32(smem + (size_t)s * Cfg::kStageBytes + FT_WBYTES + q * (MPAD * 128)));
                    const uint32_t a_t = tmem_base + (uint32_t)(ab * FT_ACOLS + q * 32);
#pragma unroll
                    for (int j = 0; j < 4; ++j) tc_mma_f16_ts(acc, a_t + 8 * j, bdesc + 2 * j, idesc, (c | j) != 0);
                    tc_commit(smem_u32(&w_empty[s]));
                    tc_commit(smem_u32(&a_empty[ab]));
                }
                tc_commit(smem_u32(&d_full[0]));
            }
        }
    } else if (warp < FT_WARP_EP0) {
        // ---- dequantize: thread = (weight row, half of the stage's 256 values); a group of four
        // warps covers the 128 rows, groups 0/1 take the two halves of even stages, 2/3 of odd ones
        const int g = (warp - FT_WARP_DQ0) >> 2;
        const int half = g & 1, parity = g >> 1;
        const int quarter = warp & 3;  // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        int it = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
            int tile, c0, cn;
            unit_chunks(u, tile, c0, cn);
            for (int c = 0; c < cn; ++c, ++it) {
                if ((it & 1) != parity) continue;
                const int s = it % STAGES, ab = it % FT_ABUFS;
                if (!mbar_wait_bounded(smem_u32(&w_full[s]), (it / STAGES) & 1)) {
                    if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                    ok = false;
                    break;
                }
                uint32_t w[18];  // four blocks = 72 bytes, 8-byte aligned
                const uint2 *src = reinterpret_cast<const uint2 *>(smem + (size_t)s * Cfg::kStageBytes + r * FT_ROWCHUNK_Q4 + half * 72);
#pragma unroll
                for (int i = 0; i < 9; ++i) {
                    const uint2 t = src[i];
                    w[2 * i] = t.x, w[2 * i + 1] = t.y;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&w_empty[s]));  // the raw blocks are in registers: the stage may be refilled
                if (it >= FT_ABUFS && !mbar_wait_bounded(smem_u32(&a_empty[ab]), ((it / FT_ABUFS) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.err, kDevErrMma);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_t = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * FT_ACOLS + half * 64);
#pragma unroll
                for (int pr = 0; pr < 2; ++pr) {
                    // two blocks in nine words: the first starts on a word, its nibbles two bytes in;
                    // the second starts two bytes into word 4, its nibbles on word 5
                    const uint32_t *q = w + 9 * pr;
                    uint32_t o[16];
                    {
                        const __half dh = __ushort_as_half((unsigned short)(q[0] & 0xFFFFu));
                        const __half2 d2 = __halves2half2(dh, dh);
#pragma unroll
                        for (int j = 0; j < 4; ++j) dequant_word(__funnelshift_r(q[j], q[j + 1], 16), d2, o + 4 * j);
                        tmem_st16(a_t + (uint32_t)((2 * pr) * 16), o);
                    }
                    {
                        const __half dh = __ushort_as_half((unsigned short)(q[4] >> 16));
                        const __half2 d2 = __halves2half2(dh, dh);
#pragma unroll
                        for (int j = 0; j < 4; ++j) dequant_word(q[5 + j], d2, o + 4 * j);
                        tmem_st16(a_t + (uint32_t)((2 * pr + 1) * 16), o);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&a_full[ab]));
            }
        }
    } else {
        // ---- epilogue: adds the issuers' accumulators, lane = weight row ----------------------
        const int quarter = warp & 3;
        int ui = 0;
        for (int u = blockIdx.x; u < nunits; u += gridDim.x, ++ui) {
            const int split = u / p.ntiles, tile = u - split * p.ntiles;
            if (!mbar_wait_bounded(smem_u32(&d_full[0]), ui & 1)) {
                if (lane == 0) atomicExch(p.err, kDevErrMma);
                break;
            }
            tc_fence_after();
            const int row = tile * FT_ROWS + quarter * 32 + lane;
            float *dst = p.out + (int64_t)split * p.split_stride + row;
#pragma unroll 1
            for (int c = 0; c < MPAD / 16; ++c) {
                float v[16];
#pragma unroll
                for (int q = 0; q < FT_ISSUERS; ++q) {
                    uint32_t t[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(FT_DCOL0 + q * MPAD + c * 16), t);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = q == 0 ? __uint_as_float(t[i]) : v[i] + __uint_as_float(t[i]);
                }
                if (c == MPAD / 16 - 1) {  // everything is in registers: the issuers may overwrite the accumulators
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&d_empty[0]));
                }
                if (row < p.n) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c * 16 + i < p.m) dst[(int64_t)(c * 16 + i) * p.ld_out] = v[i];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

bool make_w_map(CUtensorMap *map, const void *w, int64_t n, int64_t row_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)FT_ROWCHUNK_Q4, (cuuint32_t)FT_ROWS};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
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

template <int MPAD>
cq_status run_ft(cq_ctx *ctx, const CUtensorMap &tmW, const CUtensorMap &tmX, const FtParams &p, unsigned ctas) {
    static thread_local int configured = -1;
    if (configured != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(qgemm_q4_0_tmem_kernel<MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FtCfg<MPAD>::kSmem));
        configured = ctx->device;
    }
    qgemm_q4_0_tmem_kernel<MPAD><<<ctas, FT_THREADS, FtCfg<MPAD>::kSmem, ctx->stream>>>(tmW, tmX, p);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

}  // namespace

bool qgemm_dequant_tmem_supported(int qtype, int64_t m, int64_t k, const void *w) {
    return qtype == CQ_Q4_0 && m >= 1 && m <= 64 && k % FT_KCHUNK == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

cq_status launch_qgemm_dequant_tmem(cq_ctx *ctx, int order, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, float *y,
                                    int64_t ldy) {
    if ((reinterpret_cast<uintptr_t>(x) & 3) != 0 || (reinterpret_cast<uintptr_t>(y) & 3) != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemm: misaligned pointer");
    if (n > 0x7FFFFFFF || k > 0x7FFFFFFF) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: dimension beyond 2^31");
    const int ntiles = (int)((n + FT_ROWS - 1) / FT_ROWS);
    const int nchunks = (int)(k / FT_KCHUNK);
    // split k until the units cover the SMs about one and a half times, keeping at least two chunks per unit
    int splits = 1;
    while (ntiles * splits < ctx->sm_count * 3 / 2 && nchunks / (splits * 2) >= 2 && splits < 16) splits *= 2;
    int cps = (nchunks + splits - 1) / splits;
    splits = (nchunks + cps - 1) / cps;  // no empty split
    const size_t x16_bytes = (((size_t)m * k * 2) + 1023) & ~size_t(1023);
    const size_t part_bytes = splits > 1 ? (size_t)splits * m * n * 4 : 0;
    cq_status s = cq_reserve_scratch(ctx, x16_bytes + part_bytes);
    if (s != CQ_OK) return s;
    __half *x16 = static_cast<__half *>(ctx->scratch);
    float *part = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->scratch) + x16_bytes);
    {
        const int64_t total = m * (k / 32);
        const unsigned cap = (unsigned)ctx->sm_count * 8;
        const unsigned grid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        x_to_f16_perm_kernel<<<grid, 256, 0, ctx->stream>>>(x, m, k, ldx, order, x16);
    }
    const int mpad = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    CUtensorMap tmW, tmX;
    if (!make_w_map(&tmW, w, n, (k / 32) * kQ4Bytes) || !make_x_map(&tmX, x16, m, k, mpad))
        return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
    FtParams p;
    p.out = splits > 1 ? part : y;
    p.ld_out = splits > 1 ? n : ldy;
    p.split_stride = splits > 1 ? m * n : 0;
    p.m = (int)m, p.n = (int)n, p.ntiles = ntiles, p.nchunks = nchunks, p.splits = splits, p.chunks_per_split = cps;
    p.err = ctx->dev_err_devptr;
    const int64_t nunits = (int64_t)ntiles * splits;
    const unsigned ctas = (unsigned)(nunits < ctx->sm_count ? nunits : ctx->sm_count);
    if (mpad == 16) s = run_ft<16>(ctx, tmW, tmX, p, ctas);
    else if (mpad == 32) s = run_ft<32>(ctx, tmW, tmX, p, ctas);
    else s = run_ft<64>(ctx, tmW, tmX, p, ctas);
    if (s != CQ_OK) return s;
    if (splits > 1) {
        const int64_t total = m * n;
        const unsigned grid = (unsigned)((total + 255) / 256 < (int64_t)ctx->sm_count * 8 ? (total + 255) / 256 : (int64_t)ctx->sm_count * 8);
        splitk_sum_kernel<<<grid, 256, 0, ctx->stream>>>(part, splits, m, n, y, ldy);
        CQ_CUDA(ctx, cudaGetLastError());
    }
    return CQ_OK;
}
