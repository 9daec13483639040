// Tensor-parallel exchange without a collective library: the row-parallel linear's all-reduce is
// split between the kernel before it and the kernel after it.
//
//   producer  cq_qmatmul_push      the decode GEMV writes each partial result straight into every
//                                  rank's receive buffer (plain peer stores over NVLink/NVSwitch) as
//                                  one 8-byte pair (value bits, tag).
//   consumer  cq_add_rmsnorm_reduce polls (bounded) each pair in its OWN memory until the tag is the
//                                  one this exchange carries, sums the world partials in rank order,
//                                  adds the sum to the residual, applies RMSNorm, and advances the tag.
//
// Value and tag travel as ONE 64-bit element (st.relaxed.sys.b64 / ld.relaxed.sys.v2.b64: each 64-bit
// element is single-copy atomic; a .v2.u32 access would be two 32-bit elements in no stated order), so the data is
// usable one NVLink hop after it was produced: no fence, no separate flag, no extra kernel, no
// NCCL call, nothing loaded from a peer.  The tag is a per-set counter kept in each rank's own
// memory and advanced by the consumer, so a captured CUDA graph replays correctly.
// Buffers come in two sets used alternately (o-projection: set 0, down-projection: set 1); a rank
// can only push into a set again after it consumed the other set, which needs every rank's push
// there, which every rank issues after consuming this set -- so reuse is ordered by the data flow
// itself.  One process per GPU; peers are mapped with CUDA IPC handles that the host exchanges
// through whatever transport it has (torch.distributed object gather in the benchmark).
// The reference has no multi-device code at all; nothing here has a counterpart in it.
#include <cooperative_groups.h>

#include <vector>

#include "common.cuh"

namespace cg = cooperative_groups;

constexpr int kMaxWorld = 16;

struct cq_comm {
    int rank = 0, world = 1;
    size_t max_floats = 0;          // capacity of one slot
    void *local = nullptr;          // [2 sets][world slots][max_floats] (value, tag) pairs, then [2] tags, then [2] "done" counters
    void *peer_base[kMaxWorld] = {};
    bool opened[kMaxWorld] = {};
    uint2 **d_push_rx[2] = {};      // device arrays [world]: my slot on each rank, per set
    bool pushed[2] = {false, false};  // a push into the set awaits its reducing norm
    bool loopback = false;            // single-process stand-in: every "peer" is this rank's own buffer
};

namespace {

size_t comm_bytes(int world, size_t max_floats) { return 2 * (size_t)world * max_floats * 8 + 64; }
uint2 *slot_ptr(void *base, int world, size_t max_floats, int set, int slot) {
    return reinterpret_cast<uint2 *>(base) + ((size_t)set * world + slot) * max_floats;
}
unsigned *seq_ptr(void *base, int world, size_t max_floats, int set) {
    return reinterpret_cast<unsigned *>(reinterpret_cast<uint8_t *>(base) + 2 * (size_t)world * max_floats * 8) + set;
}
unsigned *done_ptr(void *base, int world, size_t max_floats, int set) { return seq_ptr(base, world, max_floats, 0) + 2 + set; }

// two adjacent (value, tag) pairs in one 16-byte load; each pair is one 64-bit element (tag in the high half)
__device__ __forceinline__ void ld_pair2(const uint2 *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned tag_of(unsigned long long v) { return (unsigned)(v >> 32); }
__device__ __forceinline__ float val_of(unsigned long long v) { return __uint_as_float((unsigned)v); }

// x[row] += sum over ranks of rx[rank][row]; y[row] = rmsnorm(x[row]) * alpha.
// A row is shared by the CTAs of one thread-block cluster (1 or 8): each CTA polls, sums and stores its
// slice of the columns, the sums of squares meet through distributed shared memory across one hardware
// cluster barrier, and each CTA normalises its own slice.  With eight CTAs a thread of an 8192-column row
// has one column pair and `world` 16-byte loads in flight at once: a single memory round trip.
__global__ void __launch_bounds__(512) add_rmsnorm_reduce_kernel(float *__restrict__ x, const uint2 *rx, int world, int64_t slot_stride,
                                                                unsigned *seq, unsigned *done, const float *__restrict__ alpha, int cols,
                                                                float eps, float *__restrict__ y, int *err, unsigned poll_limit) {
    __shared__ float sh[32];
    __shared__ float cta_ss;
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    const int row = blockIdx.x / csize;
    pdl_launch_dependents();
    pdl_wait_prior();
    const unsigned tag = *seq + 1u;  // advanced only after every CTA of this grid has read it (below)
    float *xr = x + (int64_t)row * cols;
    float *yr = y + (int64_t)row * cols;
    const uint2 *r0 = rx + (int64_t)row * cols;
    const int slice = cols / csize, c_begin = crank * slice, c_end = c_begin + slice;  // slice is even (host checks)
    float ss = 0.0f;
    bool timed_out = false;
    // Two adjacent columns per trip, and every rank's 16-byte (value, tag, value, tag) load issued before
    // the first tag is looked at: `world` loads in flight per thread instead of one.
    for (int c = c_begin + 2 * threadIdx.x; c < c_end; c += 2 * blockDim.x) {
        float d0 = 0.0f, d1 = 0.0f;  // partials first, in rank order (identical on every rank), then the residual: what an all-reduce would give
        for (int rb = 0; rb < world; rb += 8) {  // eight ranks' loads in flight at a time
            unsigned long long va[8], vb[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (rb + i < world) ld_pair2(r0 + (int64_t)(rb + i) * slot_stride + c, va[i], vb[i]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (rb + i < world) {
                    // bounded wait for this pair, then give up and flag it
                    for (unsigned it = 0; (tag_of(va[i]) != tag || tag_of(vb[i]) != tag) && it < poll_limit && !timed_out; ++it) {
                        if (it >= 32) __nanosleep(it < 1024 ? 100 : 400);
                        ld_pair2(r0 + (int64_t)(rb + i) * slot_stride + c, va[i], vb[i]);
                    }
                    if (tag_of(va[i]) != tag || tag_of(vb[i]) != tag) timed_out = true;
                    d0 = (rb + i) == 0 ? val_of(va[i]) : d0 + val_of(va[i]);
                    d1 = (rb + i) == 0 ? val_of(vb[i]) : d1 + val_of(vb[i]);
                }
            }
        }
        const float2 xv = *reinterpret_cast<const float2 *>(xr + c);
        const float v0 = xv.x + d0, v1 = xv.y + d1;
        *reinterpret_cast<float2 *>(xr + c) = make_float2(v0, v1);
        ss = fmaf(v0, v0, fmaf(v1, v1, ss));
    }
    if (timed_out) atomicExch(err, kDevErrFullWait);
    // CTA sum, then the cluster's sum in CTA-rank order (the same order, hence the same bits, on every rank)
    {
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
        if (lane == 0) sh[w] = ss;
        __syncthreads();
        ss = (lane < nw) ? sh[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
        if (threadIdx.x == 0) cta_ss = ss;
    }
    cluster.sync();
    float tot = 0.0f;
    for (int r = 0; r < csize; ++r) tot += *cluster.map_shared_rank(&cta_ss, r);
    cluster.sync();  // nobody leaves while a neighbour may still read its shared memory
    const float scale = 1.0f / sqrtf(tot / (float)cols + eps);
    for (int c = c_begin + threadIdx.x; c < c_end; c += blockDim.x) yr[c] = alpha ? scale * xr[c] * alpha[c] : scale * xr[c];
    // the last CTA of the grid advances the tag for the next use of this set
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(done, 1u);
        if (prev == gridDim.x - 1) {
            atomicExch(done, 0u);
            atomicExch(seq, tag);
        }
    }
}

}  // namespace

extern "C" {

cq_status cq_comm_create(cq_ctx *ctx, int rank, int world, int64_t max_floats, cq_comm **out, void *handle64) {
    CQ_ENTER(ctx);
    if (!out || !handle64 || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_floats < 1)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_comm_create: bad arguments (world <= 16)");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cq_comm *c = new cq_comm();
    c->rank = rank, c->world = world, c->max_floats = (size_t)max_floats;
    const size_t bytes = comm_bytes(world, c->max_floats);
    cudaError_t e = cudaMalloc(&c->local, bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(handle64), c->local);
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        delete c;
        return cq_cuda_fail(ctx, e, "cq_comm_create");
    }
    *out = c;
    return CQ_OK;
}

// all_handles: world x 64 bytes, rank order (this rank's own entry is ignored).
cq_status cq_comm_connect(cq_ctx *ctx, cq_comm *c, const void *all_handles) {
    CQ_ENTER(ctx);
    if (!c) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_comm_connect: null pointer");
    if (c->d_push_rx[0]) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_comm_connect: already connected");
    const cudaIpcMemHandle_t *h = reinterpret_cast<const cudaIpcMemHandle_t *>(all_handles);
    c->loopback = all_handles == nullptr;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank || c->loopback) {
            c->peer_base[r] = c->local;
            continue;
        }
        CQ_CUDA(ctx, cudaIpcOpenMemHandle(&c->peer_base[r], h[r], cudaIpcMemLazyEnablePeerAccess));
        c->opened[r] = true;
    }
    for (int set = 0; set < 2; ++set) {
        std::vector<uint2 *> rx(c->world);
        for (int r = 0; r < c->world; ++r) rx[r] = slot_ptr(c->peer_base[r], c->world, c->max_floats, set, c->rank);
        CQ_CUDA(ctx, cudaMalloc((void **)&c->d_push_rx[set], sizeof(uint2 *) * c->world));
        CQ_CUDA(ctx, cudaMemcpy(c->d_push_rx[set], rx.data(), sizeof(uint2 *) * c->world, cudaMemcpyHostToDevice));
    }
    return CQ_OK;
}

cq_status cq_comm_destroy(cq_ctx *ctx, cq_comm *c) {
    CQ_ENTER(ctx);
    if (!c) return CQ_OK;
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
    for (int set = 0; set < 2; ++set) {
        if (c->d_push_rx[set]) cudaFree(c->d_push_rx[set]);
    }
    if (c->local) cudaFree(c->local);
    delete c;
    return CQ_OK;
}

cq_status cq_qmatmul_push(cq_ctx *ctx, cq_comm *c, int set, int qtype, int order, const float *x_dev, int64_t m, int64_t k, int64_t ldx,
                          const void *w_blocks_dev, int64_t n) {
    CQ_ENTER(ctx);
    if (!c || (set != 0 && set != 1) || !x_dev || !w_blocks_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_push: bad arguments");
    if (qtype != CQ_Q4_0 && qtype != CQ_Q8_0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "qtype must be CQ_Q4_0 or CQ_Q8_0");
    if (order != 0 && order != 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "order must be 0 or 1");
    if (m < 1 || m > 8 || n < 1 || k < kQK || k % kQK != 0 || ldx < k)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_push: need 1 <= m <= 8, k % 32 == 0, ldx >= k");
    if ((size_t)(m * n) > c->max_floats) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "cq_qmatmul_push: m*n exceeds the communicator's slot size");
    if (!c->d_push_rx[set]) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_push: communicator is not connected");
    if (c->pushed[set])
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_qmatmul_push: this set already holds a push that no cq_add_rmsnorm_reduce has consumed (it would reuse the tag and overwrite data peers may still read)");
    ctx->push.rx = c->d_push_rx[set];
    ctx->push.seq = seq_ptr(c->local, c->world, c->max_floats, set);
    ctx->push.world = c->world;
    ctx->push.row_stride = n;
    cq_status s = launch_gemv(ctx, qtype, order, CQ_ACT_F32, x_dev, m, k, ldx, w_blocks_dev, n, /*y unused*/ const_cast<float *>(x_dev), n);
    c->pushed[set] = s == CQ_OK;
    ctx->push = PushSpec();
    return s;
}

cq_status cq_add_rmsnorm_reduce(cq_ctx *ctx, cq_comm *c, int set, float *x_dev, const float *alpha_dev, int64_t rows, int64_t cols, float eps,
                                float *y_dev) {
    CQ_ENTER(ctx);
    if (!c || (set != 0 && set != 1) || !x_dev || !y_dev || rows < 1 || rows > 8 || cols < 1 || cols > 0x7FFFFFFF)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm_reduce: bad arguments");
    if ((size_t)(rows * cols) > c->max_floats) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "cq_add_rmsnorm_reduce: rows*cols exceeds the slot size");
    if ((cols & 1) || (reinterpret_cast<uintptr_t>(x_dev) & 7)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm_reduce: cols must be even and x 8-byte aligned");
    if (!c->pushed[set]) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm_reduce: no cq_qmatmul_push was issued into this set");
    c->pushed[set] = false;
    // eight CTAs (one cluster) per row when the row is long enough to share out in even slices
    const int csize = (cols >= 2048 && cols % 16 == 0 && ctx->tune.comm_cluster != 1) ? 8 : 1;
    const int slice = (int)cols / csize;
    const int threads = slice >= 1024 ? 512 : 256;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows * csize));
    cfg.blockDim = dim3(threads);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 2 : 1;
    const uint2 *rx = slot_ptr(c->local, c->world, c->max_floats, set, 0);
    const unsigned poll_limit = ctx->tune.comm_poll_limit > 0 ? (unsigned)ctx->tune.comm_poll_limit : (1u << 22);
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, add_rmsnorm_reduce_kernel, x_dev, rx, c->world, (int64_t)c->max_floats,
                                    seq_ptr(c->local, c->world, c->max_floats, set), done_ptr(c->local, c->world, c->max_floats, set), alpha_dev,
                                    (int)cols, eps, y_dev, ctx->dev_err_devptr, poll_limit));
    return CQ_OK;
}

}  // extern "C"
