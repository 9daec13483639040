// Prefill GEMM (m > 8): Y[m,n] = X[m,k] . W[n,k]^T on the 5th-generation tensor cores.
//
// CQ_ACT_F16 numerics: activations rounded to f16, weights dequantized (exactly, in f32) and
// rounded once to f16, products exact, accumulation in f32 inside the tensor core.  Against
// candy's CPU path (f32 activations, conv.go:373-389) this differs by the two f16 roundings:
// ~3e-4 of max|y| on the benchmark's distributions, inside the 1e-3 bar.  Why not int8 MMAs:
// each 32-block carries its own scale on BOTH operands (d_w[n,b] * d_x[m,b]), a rank-1 factor per
// block that no single int8 operand can absorb, so an int8 design has to drain the accumulator
// every 32 values of k and rescale on CUDA cores -- about 4 CUDA-core instructions per 32 MACs,
// which caps it near one eighth of the int8 pipe, below this f16 kernel, and single-slice int8
// activations miss the 1e-3 bar against the CPU path (5.8e-3) anyway.
//
// Two steps.  (1) streaming conversion kernels write f16 copies of X [m,k] and W [n,k] into
// context scratch (HBM-bound: 18/34 B in, 64 B out per block).  (2) gemm_f16_tn_kernel: one CTA
// per 128 x 256 (or, for m <= 64, 128 x 64) output tile; a producer lane feeds a shared-memory ring with TMA tensor
// loads (128-byte swizzle, K-major tiles of 64 values); one lane issues tcgen05.mma
// (cta_group::1, kind::f16, M=128, N=256, K=16 x 4 per stage) into a 256-column f32 accumulator
// in tensor memory; tcgen05.commit hands stages back to the producer and, at the end, the
// accumulator to four epilogue warps that read it with tcgen05.ld and store f32 rows.
// Every mbarrier wait is bounded; a give-up sets the context's error word and the CTA still
// reaches the final barrier and frees its tensor memory.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int GEMM_THREADS = 192;     // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
// Two tile shapes: 128 x 256 (4 stages) for wide batches, 128 x 64 (8 stages) for batches of at
// most 64 rows, where the number of n-tiles is what fills the SMs.
template <int BN>
struct GemmCfg {
    static constexpr int kStages = BN >= 256 ? 4 : 8;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr size_t kSmem = (size_t)kStages * (A_BYTES + kBBytes) + 1024 /* alignment slack */ + 256 /* barriers */;
};

// ---- f16 conversion kernels -------------------------------------------------------------
__global__ void __launch_bounds__(256) x_to_f16_kernel(const float *__restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                     __half *__restrict__ out) {
    const int64_t total = m * (k / 4);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / (k / 4), c4 = i - row * (k / 4);
        const float *src = x + row * ldx + c4 * 4;
        __half2 a = __floats2half2_rn(src[0], src[1]), b = __floats2half2_rn(src[2], src[3]);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t *>(&a);
        v.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(out + row * k + c4 * 4) = v;
    }
}

// One thread converts 8 consecutive values of a block (one 16-byte store).  The f32 value
// d*(q-8) (or d*q) is exact, so the only rounding is f32 -> f16, round-to-nearest-even.
template <int QT, int ORDER>
__global__ void __launch_bounds__(256) w_to_f16_kernel(const uint8_t *__restrict__ blocks, int64_t nblocks,
                                                     __half *__restrict__ out) {
    const int64_t total = nblocks * 4;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t blk = idx >> 2;
        const int p = (int)(idx & 3);  // values 8p .. 8p+7
        float v[8];
        if (QT == CQ_Q4_0) {
            const uint8_t *b = blocks + blk * kQ4Bytes;
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b)));
            if (ORDER == CQ_ORDER_GO_INTERLEAVED) {
                const uint8_t *qs = b + 2 + 4 * p;  // bytes 4p..4p+3 -> values 8p..8p+7
                const uint32_t four = *reinterpret_cast<const unsigned short *>(qs) |
                                      ((uint32_t) * reinterpret_cast<const unsigned short *>(qs + 2) << 16);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = d * (float)((int)((four >> (4 * i)) & 0xF) - 8);
            } else {
                const uint8_t *qs = b + 2 + 8 * (p & 1);  // values 8p..8p+7 = low (p<2) or high nibbles of 8 bytes
                const int sh = (p >= 2) ? 4 : 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = d * (float)((int)((qs[i] >> sh) & 0xF) - 8);
            }
        } else {
            const uint8_t *b = blocks + blk * kQ8Bytes;
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b)));
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = d * (float)(int)(signed char)b[2 + 8 * p + i];
        }
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(out + idx * 8) = *reinterpret_cast<uint4 *>(h);
    }
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_f16_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, float *__restrict__ y, int M,
                       int N, int K, int64_t ldy, int *err) {
    constexpr int STAGES = GemmCfg<BN>::kStages, B_BYTES = GemmCfg<BN>::kBBytes, TMEM_COLS = GemmCfg<BN>::kTmemCols;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smA = smem;                              // [STAGES][A_BYTES]
    uint8_t *smB = smem + (size_t)STAGES * A_BYTES;   // [STAGES][B_BYTES]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * (A_BYTES + B_BYTES));
    uint64_t *full = bars, *empty = bars + STAGES, *acc_full = bars + 2 * STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // m-tiles vary fastest across the grid: a wave of CTAs then shares a handful of B tiles (and all
    // of A), so the f16 weight copy crosses HBM about once instead of once per few m-tiles.
    const int tile_m = blockIdx.x, tile_n = blockIdx.y;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(acc_full), 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < nk; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ((kb / STAGES) - 1) & 1)) {
                    atomicExch(err, kDevErrEmptyWait);
                    break;
                }
                mbar_expect_tx(smem_u32(&full[s]), A_BYTES + B_BYTES);
                tma_load_2d(smem_u32(smA + (size_t)s * A_BYTES), &tmA, kb * BK, tile_m * BM, smem_u32(&full[s]));
                tma_load_2d(smem_u32(smB + (size_t)s * B_BYTES), &tmB, kb * BK, tile_n * BN, smem_u32(&full[s]));
                issued = kb + 1;
            }
            // never leave with copies in flight into this CTA's shared memory
            const int first = issued > STAGES ? issued - STAGES : 0;
            for (int kb = first; kb < issued; ++kb)
                if (!mbar_wait_bounded(smem_u32(&full[kb % STAGES]), (kb / STAGES) & 1)) {
                    atomicExch(err, kDevErrDrain);
                    break;
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < nk && ok; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait_bounded(smem_u32(&full[s]), (kb / STAGES) & 1)) {
                    atomicExch(err, kDevErrFullWait);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a0 = smem_u32(smA + (size_t)s * A_BYTES), b0 = smem_u32(smB + (size_t)s * B_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)  // 16 values of k = 32 bytes inside the 128-byte swizzled row
                    tc_mma_f16(tmem_base, smem_desc_k128(a0 + 32 * k), smem_desc_k128(b0 + 32 * k), idesc, (kb | k) != 0);
                tc_commit(smem_u32(&empty[s]));  // arrives when these MMAs have finished reading the stage
            }
            tc_commit(smem_u32(acc_full));  // arrives when every MMA issued so far has completed
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31 only
        const int q = warp & 3;
        if (mbar_wait_bounded(smem_u32(acc_full), 0)) {
            tc_fence_after();
            const int64_t row = (int64_t)tile_m * BM + q * 32 + lane;
            const int col0 = tile_n * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
                const int col = col0 + c * 32;
                if (row < M) {
                    float *dst = y + row * ldy + col;
                    if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4 *>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                             __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < N) dst[i] = __uint_as_float(r[i]);
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(err, kDevErrMma);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Persistent variant of the 128 x 256 kernel: one CTA per SM walks tiles t = blockIdx.x, +gridDim.x, ...
// (m-tiles fastest).  The shared-memory ring keeps running across tile boundaries and the
// accumulator is double-buffered in tensor memory (2 x 256 columns), so the epilogue of tile i
// overlaps the MMAs of tile i+1 and no tile pays the pipeline fill again.
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_f16_tn_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, float *__restrict__ y,
                                  int M, int N, int K, int64_t ldy, int *err) {
    constexpr int BN = 256;
    constexpr int STAGES = GemmCfg<BN>::kStages, B_BYTES = GemmCfg<BN>::kBBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smA = smem;
    uint8_t *smB = smem + (size_t)STAGES * A_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * (A_BYTES + B_BYTES));
    uint64_t *full = bars, *empty = bars + STAGES, *acc_full = bars + 2 * STAGES, *acc_empty = bars + 2 * STAGES + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = (M + BM - 1) / BM, nt = (N + BN - 1) / BN;
    const int ntiles = mt * nt;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);  // one arrival per epilogue warp
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;  // k-blocks issued so far, across tiles
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const int tile_m = t % mt, tile_n = t / mt;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ((it / STAGES) - 1) & 1)) {
                        atomicExch(err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&full[s]), A_BYTES + B_BYTES);
                    tma_load_2d(smem_u32(smA + (size_t)s * A_BYTES), &tmA, kb * BK, tile_m * BM, smem_u32(&full[s]));
                    tma_load_2d(smem_u32(smB + (size_t)s * B_BYTES), &tmB, kb * BK, tile_n * BN, smem_u32(&full[s]));
                }
            }
            // never leave with copies in flight into this CTA's shared memory
            const int first = it > STAGES ? it - STAGES : 0;
            for (int i = first; i < it; ++i)
                if (!mbar_wait_bounded(smem_u32(&full[i % STAGES]), (i / STAGES) & 1)) {
                    atomicExch(err, kDevErrDrain);
                    break;
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(BM, BN);
            int it = 0, ti = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !mbar_wait_bounded(smem_u32(&acc_empty[buf]), ((ti >> 1) - 1) & 1)) {  // epilogue done with this buffer
                    atomicExch(err, kDevErrMma);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(smem_u32(&full[s]), (it / STAGES) & 1)) {
                        atomicExch(err, kDevErrFullWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smA + (size_t)s * A_BYTES), b0 = smem_u32(smB + (size_t)s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma_f16(acc, smem_desc_k128(a0 + 32 * k), smem_desc_k128(b0 + 32 * k), idesc, (kb | k) != 0);
                    tc_commit(smem_u32(&empty[s]));
                }
                tc_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        const int q = warp & 3;
        int ti = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++ti) {
            const int buf = ti & 1;
            const int tile_m = t % mt, tile_n = t / mt;
            if (!mbar_wait_bounded(smem_u32(&acc_full[buf]), (ti >> 1) & 1)) {
                if (lane == 0) atomicExch(err, kDevErrMma);
                break;
            }
            tc_fence_after();
            const int64_t row = (int64_t)tile_m * BM + q * 32 + lane;
            const int col0 = tile_n * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
                const int col = col0 + c * 32;
                if (row < M) {
                    float *dst = y + row * ldy + col;
                    if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4 *>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                             __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < N) dst[i] = __uint_as_float(r[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));  // this warp's quarter of the buffer is free
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}


// ---- CTA pairs: one 256 x 256 output tile per two SMs (cta_group::2) -----------------------------------
// The persistent kernel above is bound by shared-memory bandwidth, not by the tensor pipe: per K = 16 step a
// 128 x 256 MMA reads 4 KB of A and 8 KB of B from the CTA's shared memory, 96 bytes per clock at the pipe's
// rate, next to the TMA writes of the same bytes.  With cta_group::2 the two CTAs of a cluster (the two SMs
// of a TPC) issue ONE MMA of M = 256: each CTA supplies its own 128 rows of A and HALF of the B tile (128 of
// the 256 weight rows) from its own shared memory and keeps the 128 x 256 accumulators of its rows in its own
// tensor memory, so each SM stages and reads 8 KB per step instead of 12 for the same work.
// Protocol (every barrier wait bounded): both CTAs' producer lanes issue their TMA loads with the LEADER's
// (cluster rank 0) full barrier as the completion barrier; the leader's producer arms it with the byte count of
// both; the leader's MMA lane waits on it, issues the pair's MMAs and commits to the empty barrier of BOTH CTAs
// (and, at the end of a tile, to both accumulator-full barriers); the epilogue warps of both CTAs drain their own
// tensor memory and arrive on the leader's accumulator-empty barrier.  Cluster barriers after the barrier set-up
// and before the end keep either CTA from touching the other's barriers too early or leaving too soon.
constexpr int P2_STAGES = 6;
constexpr int P2_BH_BYTES = 128 * BK * 2;  // this CTA's half of the B tile: 16 KB
constexpr int P2_STAGE_BYTES = A_BYTES + P2_BH_BYTES;
constexpr size_t P2_SMEM = (size_t)P2_STAGES * P2_STAGE_BYTES + 1024 + 256;

__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_f16_tn_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, float *__restrict__ y, int M,
                            int N, int K, int64_t ldy, int *err) {
    constexpr int BN = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smA = smem;                                    // [P2_STAGES][A_BYTES]
    uint8_t *smB = smem + (size_t)P2_STAGES * A_BYTES;      // [P2_STAGES][P2_BH_BYTES]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)P2_STAGES * P2_STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + P2_STAGES, *acc_full = bars + 2 * P2_STAGES, *acc_empty = bars + 2 * P2_STAGES + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * P2_STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int mt = (M + 255) / 256, nt = (N + BN - 1) / BN;
    const int ntiles = mt * nt;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P2_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 8);  // four epilogue warps of each CTA
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything of this CTA can signal them
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = pair; t < ntiles && ok; t += npairs) {
                const int tile_m = t % mt, tile_n = t / mt;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % P2_STAGES;
                    if (it >= P2_STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ((it / P2_STAGES) - 1) & 1)) {
                        atomicExch(err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    const uint32_t lead_full = mapa_shared(smem_u32(&full[s]), 0);
                    if (rank == 0) mbar_expect_tx(smem_u32(&full[s]), 2 * P2_STAGE_BYTES);
                    tma_load_2d_pair(smem_u32(smA + (size_t)s * A_BYTES), &tmA, kb * BK, tile_m * 256 + (int)rank * 128, lead_full);
                    tma_load_2d_pair(smem_u32(smB + (size_t)s * P2_BH_BYTES), &tmB, kb * BK, tile_n * BN + (int)rank * 128, lead_full);
                }
            }
            if (rank == 0 && ok) {  // the leader's full barriers count the bytes of both CTAs: wait for the last ones
                const int first = it > P2_STAGES ? it - P2_STAGES : 0;
                for (int i = first; i < it; ++i)
                    if (!mbar_wait_bounded(smem_u32(&full[i % P2_STAGES]), (i / P2_STAGES) & 1)) {
                        atomicExch(err, kDevErrDrain);
                        break;
                    }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_f16(256, BN);
            int it = 0, ti = 0;
            bool ok = true;
            for (int t = pair; t < ntiles && ok; t += npairs, ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !mbar_wait_bounded(smem_u32(&acc_empty[buf]), ((ti >> 1) - 1) & 1)) {
                    atomicExch(err, kDevErrMma);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % P2_STAGES;
                    if (!mbar_wait_bounded(smem_u32(&full[s]), (it / P2_STAGES) & 1)) {
                        atomicExch(err, kDevErrFullWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smA + (size_t)s * A_BYTES), b0 = smem_u32(smB + (size_t)s * P2_BH_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma_f16_pair(acc, smem_desc_k128(a0 + 32 * k), smem_desc_k128(b0 + 32 * k), idesc, (kb | k) != 0);
                    tc_commit_pair(smem_u32(&empty[s]), 3);
                }
                if (ok) tc_commit_pair(smem_u32(&acc_full[buf]), 3);
            }
        }
    } else {
        const int q = warp & 3;
        const uint32_t lead_acc_empty0 = mapa_shared(smem_u32(&acc_empty[0]), 0);
        int ti = 0;
        for (int t = pair; t < ntiles; t += npairs, ++ti) {
            const int buf = ti & 1;
            const int tile_m = t % mt, tile_n = t / mt;
            if (!mbar_wait_bounded(smem_u32(&acc_full[buf]), (ti >> 1) & 1)) {
                if (lane == 0) atomicExch(err, kDevErrMma);
                break;
            }
            tc_fence_after();
            const int64_t row = (int64_t)tile_m * 256 + (int)rank * 128 + q * 32 + lane;
            const int col0 = tile_n * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
                const int col = col0 + c * 32;
                if (row < M) {
                    float *dst = y + row * ldy + col;
                    if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4 *>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                             __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < N) dst[i] = __uint_as_float(r[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_acc_empty0 + 8 * buf);  // this warp's quarter of this CTA's buffer is free
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the pair's MMAs may still use it
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ---- wide batches without an f16 copy of W (Q4_0) --------------------------------------------------
// The persistent 128 x 256 kernel above with its B operand made in place: a TMA lane streams the RAW
// blocks of the tile's 256 weight rows (144 bytes per row and 256 values of k) into a two-stage ring,
// sixteen dequantize warps (two threads per weight row) turn each row's nibbles into f16 with exact arithmetic --
// (1024 + n) assembled by one LOP3, minus 1032 (or times 1/16 minus 72 for the nibble four bits up)
// gives n - 8 exactly, then one f16 multiply by the block's scale, the single rounding the f16 copy also
// had -- and store them as the K-major, 128-byte-swizzled tile the MMA reads (the layout a TMA load with
// CU_TENSOR_MAP_SWIZZLE_128B would have written).  A 32-bit word of nibbles yields the pairs
// (n0,n4) (n1,n5) (n2,n6) (n3,n7): the values of k inside each group of eight are therefore stored
// in that order, and the activation pre-pass writes X in the same order (a contraction does not care
// how k is numbered as long as both operands agree).  W crosses HBM once (the CTAs that share a weight
// tile run side by side); each CTA dequantizes the tile again for its own 128 activation rows, under
// the MMAs of the previous stage.
constexpr int FD_STAGES = 3;                       // MMA stages: A 16 KB + B 32 KB each
constexpr int FD_RAW_STAGES = 2;
constexpr int FD_RAW_ROW = 8 * kQ4Bytes;           // 144 bytes: one row's blocks for 256 values of k
constexpr int FD_RAW_BYTES = 256 * FD_RAW_ROW;     // 36 KB
constexpr int FD_B_BYTES = 256 * BK * 2;           // 32 KB
constexpr int FD_DQ_WARPS = 16;                    // dequantize warps: thread = (weight row, one of its two blocks per 64 values of k)
constexpr int FD_THREADS = (7 + FD_DQ_WARPS) * 32;  // warp 0 TMA(A), 1 MMA, 2-5 epilogue, 6 TMA(raw W), 7.. dequantize
constexpr size_t FD_SMEM = (size_t)FD_STAGES * (A_BYTES + FD_B_BYTES) + (size_t)FD_RAW_STAGES * FD_RAW_BYTES + 1024 + 256;

// Where value `slot` (0..7) of 16-byte chunk `cw` (0..3) of a 32-block sits in the block (see above).
template <int ORDER>
__host__ __device__ constexpr int fd_elem(int cw, int slot) {
    // slots hold the nibbles (n0, n4, n1, n5, n2, n6, n3, n7) of word cw
    const int nib = (slot & 1) * 4 + (slot >> 1);
    const int byte = 4 * cw + (nib >> 1), hi = nib & 1;
    return ORDER == CQ_ORDER_GO_INTERLEAVED ? 2 * byte + hi : byte + 16 * hi;
}

template <int ORDER>
__global__ void __launch_bounds__(256) x_to_f16_perm_kernel(const float *__restrict__ x, int64_t m, int64_t k, int64_t ldx,
                                                          __half *__restrict__ out) {
    const int64_t total = m * (k / 8);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / (k / 8), c8 = i - row * (k / 8);
        const float *src = x + row * ldx + (c8 >> 2) * 32;
        const int cw = (int)(c8 & 3);
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // selected at run time by cw only: the four candidates per slot are compile-time offsets
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (c == cw) a = src[fd_elem<ORDER>(c, 2 * j)], b = src[fd_elem<ORDER>(c, 2 * j + 1)];
            h[j] = __floats2half2_rn(a, b);
        }
        *reinterpret_cast<uint4 *>(out + row * k + c8 * 8) = *reinterpret_cast<uint4 *>(h);
    }
}

// eight nibbles of `w` times the scale pair d2 -> four f16 pairs in the order (n0,n4) (n1,n5) (n2,n6) (n3,n7)
__device__ __forceinline__ uint4 fd_dequant_word(uint32_t w, __half2 d2) {
    const uint32_t w8 = w >> 8;
    uint32_t p0 = (w & 0x000F000Fu) | 0x64006400u, p1 = (w & 0x00F000F0u) | 0x64006400u;
    uint32_t p2 = (w8 & 0x000F000Fu) | 0x64006400u, p3 = (w8 & 0x00F000F0u) | 0x64006400u;
    const __half2 m1032 = __half2half2(__ushort_as_half((unsigned short)0xE408));  // -1032
    const __half2 sixteenth = __half2half2(__ushort_as_half((unsigned short)0x2C00));  // 1/16
    const __half2 m72 = __half2half2(__ushort_as_half((unsigned short)0xD480));  // -72
    __half2 v0 = __hmul2(__hadd2(*reinterpret_cast<__half2 *>(&p0), m1032), d2);
    __half2 v1 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p1), sixteenth, m72), d2);
    __half2 v2 = __hmul2(__hadd2(*reinterpret_cast<__half2 *>(&p2), m1032), d2);
    __half2 v3 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p3), sixteenth, m72), d2);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t *>(&v0), o.y = *reinterpret_cast<uint32_t *>(&v1);
    o.z = *reinterpret_cast<uint32_t *>(&v2), o.w = *reinterpret_cast<uint32_t *>(&v3);
    return o;
}

__global__ void __launch_bounds__(FD_THREADS, 1)
    gemm_f16_fused_dequant_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, float *__restrict__ y,
                                  int M, int N, int K, int64_t ldy, int *err) {
    constexpr int BN = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smA = smem;                                        // [FD_STAGES][A_BYTES]
    uint8_t *smB = smem + (size_t)FD_STAGES * A_BYTES;          // [FD_STAGES][FD_B_BYTES]
    uint8_t *smR = smB + (size_t)FD_STAGES * FD_B_BYTES;        // [FD_RAW_STAGES][FD_RAW_BYTES]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smR + (size_t)FD_RAW_STAGES * FD_RAW_BYTES);
    uint64_t *full = bars, *empty = full + FD_STAGES, *raw_full = empty + FD_STAGES, *raw_empty = raw_full + FD_RAW_STAGES;
    uint64_t *acc_full = raw_empty + FD_RAW_STAGES, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = (M + BM - 1) / BM, nt = (N + BN - 1) / BN;
    const int ntiles = mt * nt;
    const int nk = K / BK;           // K % 256 == 0
    const int nchunks = K / 256;

    if (threadIdx.x == 0) {
        for (int s = 0; s < FD_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1 + FD_DQ_WARPS);  // the TMA lane's expect_tx arrival + one per dequantize warp
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int s = 0; s < FD_RAW_STAGES; ++s) {
            mbar_init(smem_u32(&raw_full[s]), 1);
            mbar_init(smem_u32(&raw_empty[s]), FD_DQ_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- activation tiles ----
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const int tile_m = t % mt;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % FD_STAGES;
                    if (it >= FD_STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ((it / FD_STAGES) - 1) & 1)) {
                        atomicExch(err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&full[s]), A_BYTES);
                    tma_load_2d(smem_u32(smA + (size_t)s * A_BYTES), &tmA, kb * BK, tile_m * BM, smem_u32(&full[s]));
                }
            }
            // never leave with copies in flight into this CTA's shared memory: the MMA lane waits on every
            // full barrier it uses, and it only skips one after an error; wait here for the last stages too
            const int first = it > FD_STAGES ? it - FD_STAGES : 0;
            for (int i = first; i < it && ok; ++i)
                if (!mbar_wait_bounded(smem_u32(&full[i % FD_STAGES]), (i / FD_STAGES) & 1)) {
                    atomicExch(err, kDevErrDrain);
                    break;
                }
        }
    } else if (warp == 6) {
        // ---- raw weight blocks ----
        if (lane == 0) {
            int ic = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const int tile_n = t / mt;
                for (int c = 0; c < nchunks; ++c, ++ic) {
                    const int rs = ic % FD_RAW_STAGES;
                    if (ic >= FD_RAW_STAGES && !mbar_wait_bounded(smem_u32(&raw_empty[rs]), ((ic / FD_RAW_STAGES) - 1) & 1)) {
                        atomicExch(err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&raw_full[rs]), FD_RAW_BYTES);
                    tma_load_2d(smem_u32(smR + (size_t)rs * FD_RAW_BYTES), &tmW, c * (FD_RAW_ROW / 2), tile_n * BN, smem_u32(&raw_full[rs]));
                }
            }
            const int first = ic > FD_RAW_STAGES ? ic - FD_RAW_STAGES : 0;
            for (int i = first; i < ic && ok; ++i)
                if (!mbar_wait_bounded(smem_u32(&raw_full[i % FD_RAW_STAGES]), (i / FD_RAW_STAGES) & 1)) {
                    atomicExch(err, kDevErrDrain);
                    break;
                }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(BM, BN);
            int it = 0, ti = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !mbar_wait_bounded(smem_u32(&acc_empty[buf]), ((ti >> 1) - 1) & 1)) {
                    atomicExch(err, kDevErrMma);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % FD_STAGES;
                    if (!mbar_wait_bounded(smem_u32(&full[s]), (it / FD_STAGES) & 1)) {
                        atomicExch(err, kDevErrFullWait);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(smA + (size_t)s * A_BYTES), b0 = smem_u32(smB + (size_t)s * FD_B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tc_mma_f16(acc, smem_desc_k128(a0 + 32 * k), smem_desc_k128(b0 + 32 * k), idesc, (kb | k) != 0);
                    tc_commit(smem_u32(&empty[s]));
                }
                if (ok) tc_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else if (warp >= 7) {
        // ---- dequantize: thread = (weight row of the tile, first or second block of each 64 values of k) ----
        const int dw = warp - 7;
        const int row = (dw & 7) * 32 + lane, half = dw >> 3;
        const uint32_t sw = (uint32_t)(row & 7);
        int it = 0, ic = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
            for (int c = 0; c < nchunks && ok; ++c, ++ic) {
                const int rs = ic % FD_RAW_STAGES;
                if (!mbar_wait_bounded(smem_u32(&raw_full[rs]), (ic / FD_RAW_STAGES) & 1)) {
                    if (lane == 0) atomicExch(err, kDevErrFullWait);
                    ok = false;
                    break;
                }
                uint32_t R[36];
                const uint4 *rp = reinterpret_cast<const uint4 *>(smR + (size_t)rs * FD_RAW_BYTES + (size_t)row * FD_RAW_ROW);
#pragma unroll
                for (int i = 0; i < 9; ++i) {
                    const uint4 v = rp[i];
                    R[4 * i] = v.x, R[4 * i + 1] = v.y, R[4 * i + 2] = v.z, R[4 * i + 3] = v.w;
                }
                // this thread's block of each of the four 64-value stages: scale pair and four aligned nibble words
                uint32_t wq[4][4], dd[4];
#pragma unroll
                for (int sub = 0; sub < 4; ++sub) {
                    const uint32_t *W9 = R + 9 * sub;  // [dA:2][qsA:16][dB:2][qsB:16]
                    dd[sub] = half == 0 ? __byte_perm(W9[0], 0, 0x1010) : __byte_perm(W9[4], 0, 0x3232);
#pragma unroll
                    for (int i = 0; i < 4; ++i) wq[sub][i] = half == 0 ? __funnelshift_r(W9[i], W9[i + 1], 16) : W9[5 + i];
                }
                // the words are in registers: the raw stage can be refilled while they are converted
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&raw_empty[rs]));
#pragma unroll
                for (int sub = 0; sub < 4; ++sub, ++it) {
                    const int s = it % FD_STAGES;
                    if (ok && it >= FD_STAGES && !mbar_wait_bounded(smem_u32(&empty[s]), ((it / FD_STAGES) - 1) & 1)) {
                        if (lane == 0) atomicExch(err, kDevErrEmptyWait);
                        ok = false;
                    }
                    if (ok) {
                        const __half2 d2 = *reinterpret_cast<__half2 *>(&dd[sub]);
                        uint8_t *brow = smB + (size_t)s * FD_B_BYTES + (size_t)row * 128;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *reinterpret_cast<uint4 *>(brow + (((uint32_t)(4 * half + i) ^ sw) << 4)) = fd_dequant_word(wq[sub][i], d2);
                        fence_proxy_async();  // these generic-proxy stores are read by the tensor core (async proxy)
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(smem_u32(&full[s]));
                }
            }
        }
    } else {
        // ---- epilogue warps 2..5 (as in the kernel above) ----
        const int q = warp & 3;
        int ti = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++ti) {
            const int buf = ti & 1;
            const int tile_m = t % mt, tile_n = t / mt;
            if (!mbar_wait_bounded(smem_u32(&acc_full[buf]), (ti >> 1) & 1)) {
                if (lane == 0) atomicExch(err, kDevErrMma);
                break;
            }
            tc_fence_after();
            const int64_t row = (int64_t)tile_m * BM + q * 32 + lane;
            const int col0 = tile_n * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
                const int col = col0 + c * 32;
                if (row < M) {
                    float *dst = y + row * ldy + col;
                    if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4 *>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                             __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col + i < N) dst[i] = __uint_as_float(r[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// raw Q4_0 blocks [n rows][row_bytes]; box = 144 bytes (256 values of k) x 256 rows, no swizzle, zero fill outside
bool make_raw_w_map(CUtensorMap *map, const void *w, int64_t n, int64_t row_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 2), (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(FD_RAW_ROW / 2), 256u};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- host side ----------------------------------------------------------------------------
// f16 [rows, k] row-major; box = 64 values of k x box_rows rows, 128-byte swizzle, zero fill outside.
bool make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t k, int box_rows) {  // box_rows <= 256
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cq_status launch_gemm(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx,
                      const void *w, int64_t n, float *y, int64_t ldy) {
    if (actmode != CQ_ACT_F16) {
        // f32 / Q8_1 activation numerics for m > 8: the decode kernels, eight rows at a time
        // (weights are re-read once per eight rows; the tensor-core path is CQ_ACT_F16).
        for (int64_t r = 0; r < m; r += 8) {
            const int64_t rows = (m - r) < 8 ? (m - r) : 8;
            cq_status s = launch_gemv(ctx, qtype, order, actmode, x + r * ldx, rows, k, ldx, w, n, y + r * ldy, ldy);
            if (s != CQ_OK) return s;
        }
        return CQ_OK;
    }
    if ((reinterpret_cast<uintptr_t>(w) & 1) != 0 || (reinterpret_cast<uintptr_t>(x) & 3) != 0 || (reinterpret_cast<uintptr_t>(y) & 3) != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemm: misaligned pointer");
    if (m > 0x7FFFFFFF || n > 0x7FFFFFFF || k > 0x7FFFFFFF) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: dimension beyond 2^31");
    // narrow batches stream the raw blocks and dequantize into tensor memory: no f16 copy of W
    if (!cq_is_more_format(qtype) && !cq_is_k_format(qtype) && ctx->tune.gemm_variant != 3 && !ctx->tune.gemm_cache_weights && qgemm_dequant_tmem_supported(qtype, m, k, w))
        return launch_qgemm_dequant_tmem(ctx, qtype, order, x, m, k, ldx, w, n, y, ldy);
    const size_t x16_bytes = (((size_t)m * k * 2) + 1023) & ~size_t(1023);
    // Q4_0, wide batch: no f16 copy of W at all (the dequantization happens inside the GEMM's producer)
    // (taken up to 384 rows unless forced with gemm_fused_dequant = 2: beyond that the two-step route on CTA pairs is
    // faster.  A CTA-pair form of this kernel -- each CTA dequantizing its half of the B tile -- was built and measured
    // too: correct, but 207 us against 171 at m = 2048, and still 189 us with the conversion arithmetic removed, so it
    // is not kept.)
    if (qtype == CQ_Q4_0 && (ctx->tune.gemm_fused_dequant == 2 || (ctx->tune.gemm_fused_dequant == 1 && m <= 384)) && !ctx->tune.gemm_cache_weights &&
        ctx->tune.gemm_variant == 0 && k % 256 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        cq_status s = cq_reserve_scratch(ctx, x16_bytes);
        if (s != CQ_OK) return s;
        __half *x16 = static_cast<__half *>(ctx->scratch);
        const unsigned cap = (unsigned)ctx->sm_count * 16;
        const int64_t total = m * (k / 8);
        const unsigned xgrid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        if (order == CQ_ORDER_GO_INTERLEAVED) x_to_f16_perm_kernel<0><<<xgrid, 256, 0, ctx->stream>>>(x, m, k, ldx, x16);
        else x_to_f16_perm_kernel<1><<<xgrid, 256, 0, ctx->stream>>>(x, m, k, ldx, x16);
        CQ_CUDA(ctx, cudaGetLastError());
        CUtensorMap tmA, tmW;
        if (!make_map(&tmA, x16, m, k, BM) || !make_raw_w_map(&tmW, w, n, (k / kQK) * kQ4Bytes))
            return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
        static thread_local int configured_f = -1;
        if (configured_f != ctx->device) {
            CQ_CUDA(ctx, cudaFuncSetAttribute(gemm_f16_fused_dequant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FD_SMEM));
            configured_f = ctx->device;
        }
        const int64_t ntiles = ((m + BM - 1) / BM) * ((n + 255) / 256);
        const unsigned ctas = (unsigned)(ntiles < ctx->sm_count ? ntiles : ctx->sm_count);
        gemm_f16_fused_dequant_kernel<<<ctas, FD_THREADS, FD_SMEM, ctx->stream>>>(tmA, tmW, y, (int)m, (int)n, (int)k, ldy, ctx->dev_err_devptr);
        CQ_CUDA(ctx, cudaGetLastError());
        return CQ_OK;
    }
    const size_t w16_bytes = (size_t)n * k * 2;
    // With gemm_cache_weights the f16 copy of a weight matrix is made once and kept (the caller
    // promises not to rewrite those blocks in place): later calls skip the conversion kernel.
    __half *w16 = nullptr;
    bool need_convert = true;
    const auto key = std::make_tuple(w, n, k, qtype * 2 + order);
    if (ctx->tune.gemm_cache_weights) {
        auto it = ctx->w16_cache.find(key);
        if (it != ctx->w16_cache.end()) {
            w16 = static_cast<__half *>(it->second);
            need_convert = false;
        } else {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (ctx->capturing || (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone))
                return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemm: the cached f16 copy of this weight matrix does not exist yet and cannot be allocated during stream capture: run the call once before capturing");
            void *p = nullptr;
            CQ_CUDA(ctx, cudaMalloc(&p, w16_bytes));
            ctx->w16_cache[key] = p;
            ctx->w16_cache_bytes += w16_bytes;
            w16 = static_cast<__half *>(p);
        }
    }
    cq_status s = cq_reserve_scratch(ctx, x16_bytes + (w16 ? 0 : w16_bytes));
    if (s != CQ_OK) return s;
    __half *x16 = static_cast<__half *>(ctx->scratch);
    if (!w16) w16 = reinterpret_cast<__half *>(static_cast<uint8_t *>(ctx->scratch) + x16_bytes);
    const unsigned cap = (unsigned)ctx->sm_count * 16;
    {
        const int64_t total = m * (k / 4);
        const unsigned grid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        x_to_f16_kernel<<<grid, 256, 0, ctx->stream>>>(x, m, k, ldx, x16);
    }
    if (need_convert) {
        const int64_t nblocks = n * (k / kQK);
        const int64_t total = nblocks * 4;
        const unsigned grid = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        const uint8_t *wb = static_cast<const uint8_t *>(w);
        if (cq_is_k_format(qtype)) {
            cq_status s2 = launch_w_to_f16_k(ctx, qtype, w, n * (k / 256), w16);
            if (s2 != CQ_OK) return s2;
        } else if (cq_is_more_format(qtype)) {
            cq_status s2 = launch_w_to_f16_more(ctx, qtype, order, w, nblocks, w16);
            if (s2 != CQ_OK) return s2;
        } else if (qtype == CQ_Q4_0 && order == CQ_ORDER_GO_INTERLEAVED) w_to_f16_kernel<CQ_Q4_0, 0><<<grid, 256, 0, ctx->stream>>>(wb, nblocks, w16);
        else if (qtype == CQ_Q4_0) w_to_f16_kernel<CQ_Q4_0, 1><<<grid, 256, 0, ctx->stream>>>(wb, nblocks, w16);
        else w_to_f16_kernel<CQ_Q8_0, 0><<<grid, 256, 0, ctx->stream>>>(wb, nblocks, w16);
    }
    CQ_CUDA(ctx, cudaGetLastError());
    CUtensorMap tmA, tmB;
    const int bn = (m <= 64 && ctx->tune.gemm_variant != 1) ? 64 : 256;
    if (!make_map(&tmA, x16, m, k, BM) || !make_map(&tmB, w16, n, k, bn))
        return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(gemm_f16_tn_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<256>::kSmem));
        CQ_CUDA(ctx, cudaFuncSetAttribute(gemm_f16_tn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<64>::kSmem));
        configured_device = ctx->device;
    }
    dim3 grid((unsigned)((m + BM - 1) / BM), (unsigned)((n + bn - 1) / bn));
    if (bn == 256 && ctx->tune.gemm_variant == 0 && ctx->tune.gemm_pair) {
        // CTA pairs: 256 x 256 tiles, one per two SMs
        CUtensorMap tmBh;
        if (!make_map(&tmBh, w16, n, k, 128)) return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
        static thread_local int configured_pair = -1;
        static thread_local int max_clusters = 0;
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = P2_SMEM;
        cfg.stream = ctx->stream;
        if (configured_pair != ctx->device) {
            CQ_CUDA(ctx, cudaFuncSetAttribute(gemm_f16_tn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_SMEM));
            cfg.gridDim = dim3((unsigned)ctx->sm_count & ~1u);
            int nc = 0;
            CQ_CUDA(ctx, cudaOccupancyMaxActiveClusters(&nc, gemm_f16_tn_pair_kernel, &cfg));
            max_clusters = nc;
            configured_pair = ctx->device;
        }
        if (max_clusters > 0) {
            const int64_t ntiles = ((m + 255) / 256) * ((n + 255) / 256);
            const int64_t pairs = ntiles < max_clusters ? ntiles : max_clusters;
            cfg.gridDim = dim3((unsigned)(2 * pairs));
            CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_f16_tn_pair_kernel, tmA, tmBh, y, (int)m, (int)n, (int)k, ldy, ctx->dev_err_devptr));
            return CQ_OK;
        }
    }
    if (bn == 256 && ctx->tune.gemm_variant != 2) {
        static thread_local int configured_p = -1;
        if (configured_p != ctx->device) {
            CQ_CUDA(ctx, cudaFuncSetAttribute(gemm_f16_tn_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<256>::kSmem));
            configured_p = ctx->device;
        }
        const int64_t ntiles = (int64_t)grid.x * grid.y;
        const unsigned ctas = (unsigned)(ntiles < ctx->sm_count ? ntiles : ctx->sm_count);
        gemm_f16_tn_persistent_kernel<<<ctas, GEMM_THREADS, GemmCfg<256>::kSmem, ctx->stream>>>(tmA, tmB, y, (int)m, (int)n, (int)k, ldy,
                                                                                               ctx->dev_err_devptr);
    } else if (bn == 64)
        gemm_f16_tn_kernel<64><<<grid, GEMM_THREADS, GemmCfg<64>::kSmem, ctx->stream>>>(tmA, tmB, y, (int)m, (int)n, (int)k, ldy, ctx->dev_err_devptr);
    else
        gemm_f16_tn_kernel<256><<<grid, GEMM_THREADS, GemmCfg<256>::kSmem, ctx->stream>>>(tmA, tmB, y, (int)m, (int)n, (int)k, ldy, ctx->dev_err_devptr);
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}
