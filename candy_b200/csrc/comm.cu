// Tensor-parallel exchange without a collective library: the row-parallel linear's all-reduce is
// split between the kernel before it and the kernel after it.
//
//   producer  cq_qmatmul_push      the decode GEMV writes its partial results straight into every
//                                  rank's receive buffer (plain peer stores over NVLink/NVSwitch) and,
//                                  per CTA, bumps one counter on each peer (red.release.sys).
//   consumer  cq_add_rmsnorm_reduce waits (bounded) until every rank's counter shows all of that
//                                  rank's CTAs, sums the world partials from its OWN memory into the
//                                  residual, applies RMSNorm, and re-arms the counters.
//
// No extra kernel, no NCCL call, nothing loaded from a peer (data is pushed, then read locally).
// Buffers come in two sets used alternately (o-projection: set 0, down-projection: set 1); a rank
// can only push into a set again after it consumed the other set, which needs every rank's push
// there, which every rank issues after consuming (and re-arming) this set -- so reuse is ordered
// by the data flow itself.  One process per GPU; peers are mapped with CUDA IPC handles that the
// host exchanges through whatever transport it has (torch.distributed object gather in bench.py).
// The reference has no multi-device code at all; nothing here has a counterpart in it.
#include <vector>

#include "common.cuh"

constexpr int kMaxWorld = 16;

struct cq_comm {
    int rank = 0, world = 1;
    size_t max_floats = 0;          // capacity of one slot
    void *local = nullptr;          // [2 sets][world slots][max_floats] f32, then [2][kMaxWorld] u32 counters, then [2] u32 "done"
    void *peer_base[kMaxWorld] = {};
    bool opened[kMaxWorld] = {};
    float **d_push_rx[2] = {};      // device arrays [world]: my slot on each peer, per set
    unsigned **d_push_cnt[2] = {};  // device arrays [world]: my counter on each peer, per set
    int64_t expected[2] = {0, 0};   // arrivals per peer the consumer of each set waits for
};

namespace {

size_t comm_bytes(int world, size_t max_floats) { return 2 * (size_t)world * max_floats * 4 + 2 * kMaxWorld * 4 + 64; }
float *slot_ptr(void *base, int world, size_t max_floats, int set, int slot) {
    return reinterpret_cast<float *>(base) + ((size_t)set * world + slot) * max_floats;
}
unsigned *cnt_ptr(void *base, int world, size_t max_floats, int set, int slot) {
    return reinterpret_cast<unsigned *>(reinterpret_cast<uint8_t *>(base) + 2 * (size_t)world * max_floats * 4) + set * kMaxWorld + slot;
}
unsigned *done_ptr(void *base, int world, size_t max_floats, int set) {
    return reinterpret_cast<unsigned *>(reinterpret_cast<uint8_t *>(base) + 2 * (size_t)world * max_floats * 4 + 2 * kMaxWorld * 4) + set;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA per row.  x[row] += sum over ranks of rx[rank][row]; y[row] = rmsnorm(x[row]) * alpha.
__global__ void __launch_bounds__(1024) add_rmsnorm_reduce_kernel(float *__restrict__ x, const float *rx, int world, int64_t slot_stride,
                                                                const unsigned *cnt, unsigned *cnt_rw, unsigned *done, unsigned expected,
                                                                const float *__restrict__ alpha, int cols, float eps, float *__restrict__ y,
                                                                int *err) {
    __shared__ float sh[32];
    __shared__ int ok_s;
    pdl_launch_dependents();
    pdl_wait_prior();
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        // bounded wait for rank threadIdx.x's pushes (about two seconds at most, then give up)
        bool ok = false;
        for (unsigned it = 0; it < (1u << 22); ++it) {
            if (ld_acquire_sys(cnt + threadIdx.x) >= expected) {
                ok = true;
                break;
            }
            __nanosleep(it < 64 ? 0 : 200);
        }
        if (!ok) {
            atomicExch(err, kDevErrFullWait);
            ok_s = 0;
        }
    }
    __syncthreads();
    float *xr = x + (int64_t)blockIdx.x * cols;
    float *yr = y + (int64_t)blockIdx.x * cols;
    const float *r0 = rx + (int64_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = xr[c];
        for (int r = 0; r < world; ++r) v += r0[(int64_t)r * slot_stride + c];  // rank order: identical sums on every rank
        xr[c] = v;
        ss = fmaf(v, v, ss);
    }
    // block sum
    {
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
        if (lane == 0) sh[w] = ss;
        __syncthreads();
        ss = (lane < nw) ? sh[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
    }
    const float scale = 1.0f / sqrtf(ss / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = alpha ? scale * xr[c] * alpha[c] : scale * xr[c];
    // the last row's CTA re-arms the counters for the next use of this set
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(done, 1u);
        if (prev == gridDim.x - 1) {
            for (int r = 0; r < world; ++r) atomicSub(cnt_rw + r, expected);  // subtract, not clear: early arrivals of a later use survive
            atomicExch(done, 0u);
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
    if (!c || !all_handles) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_comm_connect: null pointer");
    const cudaIpcMemHandle_t *h = reinterpret_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) {
            c->peer_base[r] = c->local;
            continue;
        }
        CQ_CUDA(ctx, cudaIpcOpenMemHandle(&c->peer_base[r], h[r], cudaIpcMemLazyEnablePeerAccess));
        c->opened[r] = true;
    }
    for (int set = 0; set < 2; ++set) {
        std::vector<float *> rx(c->world);
        std::vector<unsigned *> cnt(c->world);
        for (int r = 0; r < c->world; ++r) {
            rx[r] = slot_ptr(c->peer_base[r], c->world, c->max_floats, set, c->rank);
            cnt[r] = cnt_ptr(c->peer_base[r], c->world, c->max_floats, set, c->rank);
        }
        CQ_CUDA(ctx, cudaMalloc((void **)&c->d_push_rx[set], sizeof(float *) * c->world));
        CQ_CUDA(ctx, cudaMalloc((void **)&c->d_push_cnt[set], sizeof(unsigned *) * c->world));
        CQ_CUDA(ctx, cudaMemcpy(c->d_push_rx[set], rx.data(), sizeof(float *) * c->world, cudaMemcpyHostToDevice));
        CQ_CUDA(ctx, cudaMemcpy(c->d_push_cnt[set], cnt.data(), sizeof(unsigned *) * c->world, cudaMemcpyHostToDevice));
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
        if (c->d_push_cnt[set]) cudaFree(c->d_push_cnt[set]);
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
    ctx->push.rx = c->d_push_rx[set];
    ctx->push.cnt = c->d_push_cnt[set];
    ctx->push.world = c->world;
    ctx->push.row_stride = n;
    ctx->push.arrivals = 0;
    cq_status s = launch_gemv(ctx, qtype, order, CQ_ACT_F32, x_dev, m, k, ldx, w_blocks_dev, n, /*y unused*/ const_cast<float *>(x_dev), n);
    c->expected[set] = ctx->push.arrivals;
    ctx->push = PushSpec();
    return s;
}

cq_status cq_add_rmsnorm_reduce(cq_ctx *ctx, cq_comm *c, int set, float *x_dev, const float *alpha_dev, int64_t rows, int64_t cols, float eps,
                                float *y_dev) {
    CQ_ENTER(ctx);
    if (!c || (set != 0 && set != 1) || !x_dev || !y_dev || rows < 1 || rows > 8 || cols < 1 || cols > 0x7FFFFFFF)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm_reduce: bad arguments");
    if ((size_t)(rows * cols) > c->max_floats) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "cq_add_rmsnorm_reduce: rows*cols exceeds the slot size");
    if (c->expected[set] <= 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_add_rmsnorm_reduce: no cq_qmatmul_push was issued into this set");
    const int threads = cols >= 4096 ? 1024 : (cols >= 1024 ? 512 : 256);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(threads);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    const float *rx = slot_ptr(c->local, c->world, c->max_floats, set, 0);
    unsigned *cnt = cnt_ptr(c->local, c->world, c->max_floats, set, 0);
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, add_rmsnorm_reduce_kernel, x_dev, rx, c->world, (int64_t)c->max_floats, (const unsigned *)cnt, cnt,
                                    done_ptr(c->local, c->world, c->max_floats, set), (unsigned)c->expected[set], alpha_dev, (int)cols, eps,
                                    y_dev, ctx->dev_err_devptr));
    return CQ_OK;
}

}  // extern "C"
