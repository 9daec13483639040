// Shared skeleton of the small-batch streaming kernels (gemv_mma.cu: integer block dots for CQ_ACT_F32 / CQ_ACT_Q8_1;
// gemv_mma_f16.cu: f16 operands for CQ_ACT_F16): the geometry of row ranges and k slices, the producer warp's ring of
// bulk copies, the reducer warp that adds the worker warps' partial tiles, the cluster's final sum over k slices, the
// host-side plan and launch.  A kernel built on it has MM_WARPS worker warps, then the producer warp, then the reducer
// warp; NG column groups of eight activation rows each.
#pragma once
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace mma_gemv {

namespace cg = cooperative_groups;

constexpr int MM_WARPS = 16;       // worker warps
constexpr int MM_ROWS = 16;        // weight rows per stage (the M of the instructions)
constexpr int MM_MAX_STAGES = 8;
constexpr int MM_RED_BYTES = 2 * MM_WARPS * 128 * 4;   // per column group: two buffers of one 16 x 8 tile per worker warp
constexpr int MM_COLSC_BYTES = MM_WARPS * 8 * 4 * 32;  // per (warp, block, q): 32 bytes of per-column constants (integer kernels)
constexpr int MM_THREADS = (MM_WARPS + 2) * 32;

struct MmaGemvParams {
    const uint8_t *w;
    const float *x;
    float *y;
    const float *bias;
    int64_t ldx, ldy, n;
    int nb;        // blocks per weight row
    int m;         // activation rows (<= 8 per column group)
    int ks;        // CTAs per cluster = k slices
    int ranges;    // row ranges = clusters
    int order;     // 0: interleaved nibbles (elements 2j, 2j+1 in byte j), 1: split (elements j, j+16); host-side dispatch only
    int act;       // 0: 15-bit plane columns (CQ_ACT_F32), 1: Q8_1 columns (CQ_ACT_Q8_1), 2: f16 operands; host-side dispatch only
    int stages, pitch, stage_bytes;
    int aux_off;    // byte offset of the kernel's own area (MM_COLSC_BYTES) in dynamic shared memory
    int ypart_off;  // byte offset of the cluster-reduction buffer
    int *err;
};

// What one CTA works on.
struct Geometry {
    int ks;              // rank in the cluster = index of the k slice
    int64_t row_begin;
    int nrows, npass;
    int u0;              // first unit (eight blocks) of the slice
    int sblocks;         // blocks of the slice
};

__device__ __forceinline__ Geometry geometry(const MmaGemvParams &p) {
    Geometry g;
    g.ks = p.ks > 1 ? (int)(blockIdx.x % p.ks) : 0;  // clusters are consecutive CTAs
    const int range = (int)(blockIdx.x / p.ks);
    g.row_begin = p.n * range / p.ranges;
    g.nrows = (int)(p.n * (range + 1) / p.ranges - g.row_begin);
    g.npass = (g.nrows + MM_ROWS - 1) / MM_ROWS;
    const int units = p.nb >> 3;  // slices are cut in units of eight blocks (144 bytes: copies stay 16-byte aligned)
    g.u0 = units * g.ks / p.ks;
    g.sblocks = (units * (g.ks + 1) / p.ks - g.u0) * 8;
    return g;
}

__device__ __forceinline__ void init_ring(const MmaGemvParams &p, uint64_t *bar_full, uint64_t *bar_empty) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), MM_WARPS);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
}

// Producer warp: a stage is 16 weight rows by the CTA's k slice, one bulk copy per row.  The weights do not depend on
// the previous kernel, so the ring fills at once.
__device__ __forceinline__ void produce(const MmaGemvParams &p, const Geometry &g, uint8_t *smem, uint64_t *bar_full, uint64_t *bar_empty) {
    const int lane = threadIdx.x & 31;
    const uint64_t policy = make_l2_policy_evict_first();
    const int64_t row_bytes = (int64_t)p.nb * kQ4Bytes;
    const uint32_t slice_bytes = (uint32_t)g.sblocks * kQ4Bytes;
    const uint8_t *src0 = p.w + g.row_begin * row_bytes + (int64_t)g.u0 * (8 * kQ4Bytes);
    int issued = 0;
    for (int ps = 0; ps < g.npass; ++ps) {
        const int s = ps % p.stages;
        if (ps >= p.stages && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ((ps / p.stages) - 1) & 1)) {
            if (lane == 0) atomicExch(p.err, kDevErrEmptyWait);
            break;
        }
        const int rows = min(MM_ROWS, g.nrows - ps * MM_ROWS);
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
}

// Worker side of the hand-over: park this warp's partial tile(s) of pass ps (acc[group][4]: rows g, g; g+8, g+8 by
// columns 2q, 2q+1), release the stage, tell the reducer.  The tile of pass ps - 2 has left the buffer once the
// reducer says so; the partial tile depends on every word read from the stage, so the stage can be released once it
// is parked.
template <int NG>
__device__ __forceinline__ void park(float *red, int ps, int warp, int lane, const float (&acc)[NG][4], uint32_t empty_bar) {
    const int buf = ps & 1;
    if (ps >= 2) asm volatile("bar.sync %0, %1;" ::"r"(4 + buf), "n"(MM_WARPS * 32 + 32) : "memory");
#pragma unroll
    for (int gr = 0; gr < NG; ++gr)
        reinterpret_cast<float4 *>(red)[((buf * MM_WARPS + warp) * NG + gr) * 32 + lane] = make_float4(acc[gr][0], acc[gr][1], acc[gr][2], acc[gr][3]);
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar);
    asm volatile("bar.arrive %0, %1;" ::"r"(2 + buf), "n"(MM_WARPS * 32 + 32) : "memory");
}

// Reducer warp: adds the worker warps' partial tiles of a pass in warp order (deterministic) while the workers are on the
// next stage; results go to y, or with k slices to this CTA's part of the cluster sum.
template <int NG>
__device__ __forceinline__ void reduce(const MmaGemvParams &p, const Geometry &g, const float *red, float *ypart) {
    const int lane = threadIdx.x & 31;
    pdl_wait_prior();
    for (int ps = 0; ps < g.npass; ++ps) {
        const int buf = ps & 1;
        asm volatile("bar.sync %0, %1;" ::"r"(2 + buf), "n"(MM_WARPS * 32 + 32) : "memory");  // the tiles are parked
#pragma unroll
        for (int e = 0; e < 4 * NG; ++e) {
            const int gr = e >> 2, t = (e & 3) * 32 + lane;  // value t of group gr's tile: lane t / 4 of the fragment, register t % 4
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < MM_WARPS; ++w) tot += red[((buf * MM_WARPS + w) * NG + gr) * 128 + t];
            const int l = t >> 2, c = t & 3;
            const int wrow = ps * MM_ROWS + (l >> 2) + ((c >> 1) << 3), col = gr * 8 + 2 * (l & 3) + (c & 1);
            if (wrow < g.nrows && col < p.m) {
                if (p.ks > 1) ypart[wrow * (8 * NG) + col] = tot;
                else p.y[(int64_t)col * p.ldy + g.row_begin + wrow] = p.bias ? tot + p.bias[g.row_begin + wrow] : tot;
            }
        }
        if (ps + 2 < g.npass) asm volatile("bar.arrive %0, %1;" ::"r"(4 + buf), "n"(MM_WARPS * 32 + 32) : "memory");  // the buffer is free again
    }
}

// All threads of all CTAs of the cluster: add the k slices in rank order; every rank finishes the rows r with
// r % ks == its rank.
template <int NG>
__device__ __forceinline__ void cluster_sum(const MmaGemvParams &p, const Geometry &g, float *ypart) {
    cg::cluster_group cluster = cg::this_cluster();
    pdl_wait_prior();  // the producer warp writes results below and has not waited yet
    cluster.sync();
    for (int i = threadIdx.x; i < g.nrows * 8 * NG; i += MM_THREADS) {
        const int wrow = i / (8 * NG), col = i % (8 * NG);
        if (col < p.m && wrow % p.ks == g.ks) {
            float tot = 0.0f;
            for (int r = 0; r < p.ks; ++r) tot += cluster.map_shared_rank(ypart, r)[i];
            p.y[(int64_t)col * p.ldy + g.row_begin + wrow] = p.bias ? tot + p.bias[g.row_begin + wrow] : tot;
        }
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
}

// ---- host side ------------------------------------------------------------------------------------------
struct MmaPlan {
    int ks, bpw, ranges, stages, pitch, stage_bytes, aux_off, ypart_off;
    size_t smem;
};

// ranges = 0: one row range per group of ks SMs; otherwise that many row ranges.  ng column groups; a worker warp
// holds at most max_bpw blocks of every activation row as fragments.
inline bool plan_mma(cq_ctx *ctx, int64_t k, int64_t n, int ranges, int ng, int max_bpw, MmaPlan &pl) {
    const int nb = (int)(k / kQK), units = nb / 8;
    for (int ks = 1; ks <= 8; ks *= 2) {
        if (ks > units) return false;
        const int max_blocks = ((units + ks - 1) / ks) * 8;
        if (max_blocks > MM_WARPS * max_bpw) continue;
        int bpw = (max_blocks + MM_WARPS - 1) / MM_WARPS;
        bpw += bpw & 1;
        if (ranges <= 0) ranges = ctx->sm_count / ks;
        if (ranges < 1) return false;
        // eight rows read at once must fall in different banks: pitch = 16 (mod 32) bytes
        const int slice = max_blocks * kQ4Bytes;
        const int pitch = (slice % 32 == 16) ? slice : slice + 16;
        const int stage_bytes = MM_ROWS * pitch;
        const int rows_max = (int)((n + ranges - 1) / ranges);
        const int ypart = ks > 1 ? ((rows_max + MM_ROWS) * 8 * ng * 4) : 0;
        const int budget = 225 * 1024 - MM_RED_BYTES * ng - MM_COLSC_BYTES - ypart;
        int stages = budget / stage_bytes;
        if (stages > MM_MAX_STAGES) stages = MM_MAX_STAGES;
        if (stages < 2) return false;
        pl.ks = ks, pl.bpw = bpw, pl.ranges = ranges, pl.stages = stages, pl.pitch = pitch, pl.stage_bytes = stage_bytes;
        pl.aux_off = stages * stage_bytes + MM_RED_BYTES * ng;
        pl.ypart_off = pl.aux_off + MM_COLSC_BYTES;
        pl.smem = (size_t)pl.ypart_off + ypart;
        return true;
    }
    return false;
}

// Launches `kern` (one instantiation per call site: the caches below are per instantiation) on the plan, re-planning
// when fewer clusters can be resident than the plan has row ranges.
template <class Kern>
cq_status launch_planned(cq_ctx *ctx, Kern kern, MmaGemvParams p, MmaPlan pl, int64_t k, int ng, int max_bpw) {
    static thread_local size_t configured = 0;
    static thread_local int configured_dev = -1;
    static thread_local Kern configured_kern = nullptr;
    static thread_local std::map<std::pair<int, size_t>, int> resident;  // (cluster size, shared memory) -> clusters resident at once
    if (configured_dev != ctx->device || configured_kern != kern) configured = 0, resident.clear(), configured_dev = ctx->device, configured_kern = kern;
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
        if (it->second < 1 || !plan_mma(ctx, k, p.n, it->second, ng, max_bpw, pl)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "small-batch kernel: clusters do not fit");
    }
    p.ks = pl.ks, p.ranges = pl.ranges, p.stages = pl.stages, p.pitch = pl.pitch, p.stage_bytes = pl.stage_bytes;
    p.aux_off = pl.aux_off, p.ypart_off = pl.ypart_off;
    if (ctx->tune.pdl) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        ++cfg.numAttrs;
    }
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return CQ_OK;
}

}  // namespace mma_gemv
