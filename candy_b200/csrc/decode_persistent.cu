// One decode step of a Llama-shape decoder as ONE persistent kernel (batch 1, f32-activation numerics of the
// streaming GEMV: 16-bit block fixed-point activations, exact integer dots per block, f32 sums).
//
// Why: a decode step is a chain of ~200 small dependent launches; each GEMV in the chain pays a fixed few
// microseconds (launch boundary, pipeline fill and drain) on top of its weight bytes, and the step ends up at a
// third of the HBM roofline.  Here every SM runs one CTA for the whole step (a cooperative launch, so that all
// CTAs are resident together):
//   warp 0       producer: streams this CTA's share of the weight rows of EVERY linear of the step, in order,
//                through one shared-memory ring with 1-D bulk copies.  Weights depend on nothing, so the producer
//                never waits for a phase boundary: while the consumers sit in a barrier or set activations up,
//                the ring keeps filling with the next linear's rows and HBM stays busy.
//   warps 1-15   consumers: walk the list of phases
//                  linear    prologue (embedding row | residual add + RMSNorm | attention partials combined)
//                            -> activation state -> passes over the ring -> epilogue (store | SiLU(gate)*up |
//                            store + arg-max partial)
//                  attention rotary step on q and the newest k, KV-cache write, chunked softmax partials
//                  finish    arg-max of the logits -> next token id, position += 1
//                with a grid-wide barrier between phases: one atomic counter that only grows (its base is read
//                from a generation word at kernel entry and advanced at exit, so a captured graph replays), polled
//                with a BOUNDED spin; a poll that gives up records an error word, stops waiting for the rest of
//                the kernel and lets every CTA run to the end (results are then meaningless and the decoder must
//                be recreated), so nothing can hang.
// Numerically each phase computes what the separate kernels compute (cq_qlinear_fused, cq_decode_attention_rope,
// cq_argmax); the parity tests compare both against the CPU oracle.
// The reference has no decoder and no counterpart for any of this.
#include <vector>

#include "common.cuh"
#include "dec_q16.cuh"

namespace {

constexpr int PS_THREADS = 512;
constexpr int PS_CWARPS = 15;            // consumer warps
constexpr int PS_CTHREADS = PS_CWARPS * 32;
constexpr int PS_MAX_STAGES = 12;
constexpr int PS_PASS_GROUP = 4;         // passes reduced together (two rows per thread and pass: eight partial sums)
constexpr int PS_ATT_CHUNK = 64;         // keys per attention work item
constexpr int PS_HD = 128;               // head dimension this kernel is built for

enum : int { PS_LINEAR = 0, PS_ATTENTION = 1, PS_FINISH = 2 };
// prologues: activations straight from global memory | RMSNorm of a residual whose sum of squares the previous
// linear's epilogue left as per-CTA partials | attention partials combined | the token's embedding row, normed
enum : int { PS_PRO_PLAIN = 0, PS_PRO_NORM = 1, PS_PRO_ATT_COMBINE = 2, PS_PRO_EMBED_NORM = 3 };
// epilogues: store | SiLU(gate) * up over row pairs | store + arg-max partial | residual update: x_out = x_in + result,
// with this CTA's share of sum(x_out^2) for the norm that follows
enum : int { PS_EPI_STORE = 0, PS_EPI_SILU_PAIRS = 1, PS_EPI_STORE_ARGMAX = 2, PS_EPI_RESID = 3 };

struct PsOp {
    int kind;
    // linear
    const uint8_t *w;
    int n, nb, row_bytes;
    int tpr, lanes, wpr, rpp, cwarps;   // consumer geometry: threads per row, lanes of a warp on one row, warps per row, rows per pass and row slot, active warps
    int prologue, epilogue;
    const float *x, *alpha;             // activations (or the residual to norm), norm weights
    const float *x_in;                  // PS_EPI_RESID: the residual the result is added to
    float *x_out, *y;                   // new residual (PS_EPI_RESID, PS_PRO_EMBED_NORM) / output vector
    int ss_slot;                        // which of the two sum-of-squares partial arrays this phase writes (epilogue) or reads (prologue)
    // attention
    float *k_cache, *v_cache;
};

struct PsParams {
    const PsOp *ops;
    int nops;
    int stages, stage_bytes, stash_off, coop_off, xs_off;  // dynamic shared memory layout
    int dim, nq, nkv, max_ctx, nch_max, vocab;
    float eps, att_scale;
    const float *embed, *cos_t, *sin_t;
    float *qkv, *part;                  // [(nq + 2 nkv) * 128], [nq][nch_max][130]
    float2 *argmax_part;                // per CTA (value, index bits)
    float *ss_part;                     // [2][CTAs] partial sums of squares of a residual
    uint32_t *ids;                      // in: the token to feed; out: the arg-max token
    int *pos;                           // in: its position; out: + 1
    unsigned long long *bar_count;
    unsigned *gen;
    unsigned poll_limit;
    int *err;
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(PS_CTHREADS) : "memory"); }

__device__ __forceinline__ float ps_rope_elem(const float *__restrict__ v, int d, const float *__restrict__ cos_t, const float *__restrict__ sin_t, int pos) {
    constexpr int half = PS_HD / 2;
    if (d < half) {
        const float c = cos_t[pos * half + d], s = sin_t[pos * half + d];
        return v[d] * c - v[d + half] * s;
    }
    const float c = cos_t[pos * half + d - half], s = sin_t[pos * half + d - half];
    return v[d - half] * s + v[d] * c;
}

template <class Dec>
__global__ void __launch_bounds__(PS_THREADS, 1) decode_step_kernel(const PsParams p) {
    constexpr int kWords = Dec::kWords;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[PS_MAX_STAGES];
    __shared__ uint64_t bar_empty[PS_MAX_STAGES];
    __shared__ float red[2][8][64];
    __shared__ float att_s[PS_ATT_CHUNK + 4];
    __shared__ float att_acc[2][PS_HD];
    __shared__ float best_val[PS_CWARPS];
    __shared__ uint32_t best_idx[PS_CWARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), PS_CWARPS);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    // this CTA's rows of a linear: an even split of [0, n) (on even rows when outputs pair up)
    auto row_range = [&](const PsOp &op, int64_t &rb, int &nrows) {
        const int64_t unit = op.epilogue == PS_EPI_SILU_PAIRS ? 2 : 1;
        rb = unit * (((op.n / unit) * (int64_t)cta) / G);
        const int64_t re = unit * (((op.n / unit) * (int64_t)(cta + 1)) / G);
        nrows = (int)(re - rb);
    };

    if (warp == 0) {
        // ---- producer: every linear's rows, back to back ------------------------------------------------------
        if (lane == 0) {
            const uint64_t policy = make_l2_policy_evict_first();
            unsigned it = 0;  // passes issued so far, over all phases
            bool ok = true;
            for (int oi = 0; oi < p.nops && ok; ++oi) {
                const PsOp &op = p.ops[oi];
                if (op.kind != PS_LINEAR) continue;
                int64_t rb;
                int nrows;
                row_range(op, rb, nrows);
                const int rows_per_pass = 2 * op.rpp;
                for (int r0 = 0; r0 < nrows; r0 += rows_per_pass, ++it) {
                    const int s = it % p.stages;
                    if (it >= (unsigned)p.stages && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ((it / p.stages) - 1) & 1)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    const int rows = min(rows_per_pass, nrows - r0);
                    const uint32_t bytes = (uint32_t)rows * (uint32_t)op.row_bytes;
                    mbar_expect_tx(smem_u32(&bar_full[s]), bytes);
                    bulk_g2s_hint(smem_u32(smem + (size_t)s * p.stage_bytes), op.w + (rb + r0) * (int64_t)op.row_bytes, bytes, smem_u32(&bar_full[s]), policy);
                }
            }
            if (ok) {  // never leave with copies in flight into this CTA's shared memory
                const unsigned first = it > (unsigned)p.stages ? it - p.stages : 0;
                for (unsigned i = first; i < it; ++i)
                    if (!mbar_wait_bounded(smem_u32(&bar_full[i % p.stages]), (i / p.stages) & 1)) {
                        atomicExch(p.err, kDevErrDrain);
                        break;
                    }
            }
        }
        return;
    }

    // ---- consumers -------------------------------------------------------------------------------------------
    const int ctid = tid - 32, cw = warp - 1;   // index among the consumer threads / warps
    float *stash = reinterpret_cast<float *>(smem + p.stash_off);    // [8][PS_CTHREADS]
    uint32_t *area = reinterpret_cast<uint32_t *>(smem + p.coop_off);  // activation state of the current linear
    float *xs = reinterpret_cast<float *>(smem + p.xs_off);          // activations a prologue produces
    const unsigned long long base = (unsigned long long)(*p.gen) * (unsigned long long)p.nops * (unsigned long long)G;
    bool dead = false;     // a bounded wait gave up: no more waiting, run to the end
    unsigned it = 0;       // passes consumed so far (mirrors the producer's counter)
    float my_best = -INFINITY, my_ss = 0.0f;
    uint32_t my_best_idx = 0xFFFFFFFFu;

    // all CTAs have finished phases 0 .. oi-1 (their global writes are visible after this)
    auto grid_wait = [&](int oi) {
        if (oi == 0) return;
        if (ctid == 0 && !dead) {
            const unsigned long long target = base + (unsigned long long)oi * (unsigned long long)G;
            unsigned n = 0;
            while (ld_acquire_u64(p.bar_count) < target) {
                if (++n > p.poll_limit) {
                    atomicExch(p.err, kDevErrFullWait);
                    dead = true;
                    break;
                }
                if (n > 64) __nanosleep(40);
            }
        }
        consumer_sync();
    };
    // this CTA has finished the current phase
    auto grid_arrive = [&]() {
        consumer_sync();
        if (ctid == 0) asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(p.bar_count) : "memory");
    };

    const int pos_raw = *p.pos;
    const int pos = pos_raw < 0 ? 0 : (pos_raw >= p.max_ctx ? p.max_ctx - 1 : pos_raw);
    if ((pos_raw < 0 || pos_raw >= p.max_ctx) && ctid == 0) atomicExch(p.err, kDevErrPosition);
    const int nkeys = pos + 1;
    const int nch = (nkeys + PS_ATT_CHUNK - 1) / PS_ATT_CHUNK;

    for (int oi = 0; oi < p.nops; ++oi) {
        const PsOp &op = p.ops[oi];
        grid_wait(oi);
        if (op.kind == PS_ATTENTION) {
            // ---- work items (query head, chunk of 64 keys): scores, chunk-local softmax, weighted sum of V ------
            const int group = p.nq / p.nkv;
            const int64_t kv_stride = (int64_t)p.nkv * PS_HD;
            for (int item = cta; item < p.nq * nch; item += G) {
                const int head = item / nch, chunk = item - head * nch;
                const int kvh = head / group;
                const int t0 = chunk * PS_ATT_CHUNK, t1 = min(t0 + PS_ATT_CHUNK, nkeys), cnt = t1 - t0;
                const float *q = p.qkv + head * PS_HD;
                const float *kn = p.qkv + (p.nq + kvh) * PS_HD;            // newest key (unrotated) and value, straight from qkv
                const float *vn = p.qkv + (p.nq + p.nkv + kvh) * PS_HD;
                const float *kbase = op.k_cache + kvh * PS_HD, *vbase = op.v_cache + kvh * PS_HD;
                if (cw < 8) {
                    // warp cw scores keys t0 + cw*8 .. +7; lane holds four dimensions
                    const int d = lane * 4;
                    const float4 qv = make_float4(ps_rope_elem(q, d, p.cos_t, p.sin_t, pos), ps_rope_elem(q, d + 1, p.cos_t, p.sin_t, pos),
                                                  ps_rope_elem(q, d + 2, p.cos_t, p.sin_t, pos), ps_rope_elem(q, d + 3, p.cos_t, p.sin_t, pos));
                    float4 kreg[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int t = t0 + cw * 8 + j;
                        if (t < t1 && t != pos) {
                            kreg[j] = *reinterpret_cast<const float4 *>(kbase + (int64_t)t * kv_stride + d);
                        } else if (t == pos) {  // not in the cache yet: rotate it here; the group's first head stores it
                            kreg[j] = make_float4(ps_rope_elem(kn, d, p.cos_t, p.sin_t, pos), ps_rope_elem(kn, d + 1, p.cos_t, p.sin_t, pos),
                                                  ps_rope_elem(kn, d + 2, p.cos_t, p.sin_t, pos), ps_rope_elem(kn, d + 3, p.cos_t, p.sin_t, pos));
                            if (head % group == 0) *reinterpret_cast<float4 *>(op.k_cache + (int64_t)t * kv_stride + kvh * PS_HD + d) = kreg[j];
                        } else {
                            kreg[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                    float s[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) s[j] = fmaf(qv.x, kreg[j].x, fmaf(qv.y, kreg[j].y, fmaf(qv.z, kreg[j].z, qv.w * kreg[j].w)));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                        for (int j = 0; j < 8; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o, 32);
                    if (lane < 8) {
                        float v = s[0];
#pragma unroll
                        for (int j = 1; j < 8; ++j) v = (lane == j) ? s[j] : v;
                        att_s[cw * 8 + lane] = v * p.att_scale;
                    }
                }
                if (t1 == nkeys && head % group == 0)  // this item holds the newest position: its value row goes to the cache
                    for (int d = ctid; d < PS_HD; d += PS_CTHREADS) op.v_cache[(int64_t)pos * kv_stride + kvh * PS_HD + d] = vn[d];
                consumer_sync();
                // chunk softmax numerators (FastSoftmax, reduce.go:2855-2879: subtract the maximum, exponentiate); every warp the same
                const float s0 = lane < cnt ? att_s[lane] : -INFINITY, s1 = lane + 32 < cnt ? att_s[lane + 32] : -INFINITY;
                float m = fmaxf(s0, s1);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o, 32));
                const float e0 = lane < cnt ? expf(s0 - m) : 0.0f, e1 = lane + 32 < cnt ? expf(s1 - m) : 0.0f;
                float l = e0 + e1;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o, 32);
                consumer_sync();
                if (cw == 0) att_s[lane] = e0, att_s[lane + 32] = e1;
                consumer_sync();
                if (ctid < 2 * PS_HD) {  // two halves of the chunk's keys, thread = dimension
                    const int d = ctid & (PS_HD - 1), hf = ctid >> 7;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
                    for (int j = hf * 32; j < hf * 32 + 32; ++j) {
                        const int t = t0 + j;
                        const float v = j < cnt ? (t == pos ? vn[d] : vbase[(int64_t)t * kv_stride + d]) : 0.0f;
                        acc[j & 3] = fmaf(att_s[j], v, acc[j & 3]);
                    }
                    att_acc[hf][d] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                }
                consumer_sync();
                float *out = p.part + ((int64_t)head * p.nch_max + chunk) * (PS_HD + 2);
                if (ctid < PS_HD) out[2 + ctid] = att_acc[0][ctid] + att_acc[1][ctid];
                if (ctid == 0) out[0] = m, out[1] = l;
                consumer_sync();
            }
            grid_arrive();
            continue;
        }
        if (op.kind == PS_FINISH) {
            // ---- arg-max over the CTAs' partials (lowest index among equal maxima, reduce.go:846-862), position += 1 ---
            if (cta == 0 && cw == 0) {
                float bv = -INFINITY;
                uint32_t bi = 0xFFFFFFFFu;
                for (int c = lane; c < G; c += 32) {
                    const float2 pr = p.argmax_part[c];
                    const uint32_t idx = __float_as_uint(pr.y);
                    if (pr.x > bv || (pr.x == bv && idx < bi)) bv = pr.x, bi = idx;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o, 32);
                    const uint32_t oi2 = __shfl_xor_sync(0xffffffffu, bi, o, 32);
                    if (ov > bv || (ov == bv && oi2 < bi)) bv = ov, bi = oi2;
                }
                if (lane == 0) {
                    p.ids[0] = bi == 0xFFFFFFFFu ? 0u : bi;
                    *p.pos = pos_raw + 1;
                }
            }
            grid_arrive();
            continue;
        }
        // ---- linear -----------------------------------------------------------------------------------------------
        int64_t row_begin;
        int nrows;
        row_range(op, row_begin, nrows);
        const int rows_per_pass = 2 * op.rpp;
        const int npass = (nrows + rows_per_pass - 1) / rows_per_pass;
        const int k4 = op.nb * 8;  // float4 groups in an activation row
        const float *xsrc = op.x;
        if (op.prologue == PS_PRO_EMBED_NORM) {
            // x = the embedding row of the current token (CTA 0 stores it as the residual);
            // x' = x / sqrt(mean(x^2) + eps) * alpha in shared memory.  Every CTA computes the same numbers in the same order.
            const float *src = p.embed + (int64_t)min(p.ids[0], (uint32_t)(p.vocab - 1)) * p.dim;
            float ss = 0.0f;
            for (int i = ctid; i < k4; i += PS_CTHREADS) {
                const float4 v = reinterpret_cast<const float4 *>(src)[i];
                if (cta == 0) reinterpret_cast<float4 *>(op.x_out)[i] = v;
                reinterpret_cast<float4 *>(xs)[i] = v;
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
            if (lane == 0) red[0][0][cw] = ss;
            consumer_sync();
            float tot = 0.0f;
            for (int w = 0; w < PS_CWARPS; ++w) tot += red[0][0][w];
            consumer_sync();
            const float scale = 1.0f / sqrtf(tot / (float)(op.nb * kQK) + p.eps);
            for (int i = ctid; i < k4; i += PS_CTHREADS) {  // each thread rescales what it wrote itself
                float4 v = reinterpret_cast<float4 *>(xs)[i];
                const float4 a = __ldg(reinterpret_cast<const float4 *>(op.alpha) + i);
                v.x = scale * v.x * a.x, v.y = scale * v.y * a.y, v.z = scale * v.z * a.z, v.w = scale * v.w * a.w;
                reinterpret_cast<float4 *>(xs)[i] = v;
            }
            consumer_sync();
            xsrc = xs;
        } else if (op.prologue == PS_PRO_NORM) {
            // RMSNorm of the residual the previous linear's epilogue wrote (row by row, across the CTAs) together with each
            // CTA's share of its sum of squares: everything this needs is issued as one batch of loads -- the residual, the
            // norm weights and the partial sums -- so the prologue costs one round trip to L2.
            constexpr int kMaxV = 6;  // float4 groups per thread: k <= 6 * 480 * 4 = 11520 activations
            float4 v[kMaxV], a[kMaxV];
#pragma unroll
            for (int u = 0; u < kMaxV; ++u) {
                const int i = ctid + u * PS_CTHREADS;
                if (i < k4) {
                    v[u] = reinterpret_cast<const float4 *>(op.x)[i];
                    a[u] = __ldg(reinterpret_cast<const float4 *>(op.alpha) + i);
                }
            }
            // the CTAs' partial sums in CTA order (the same order, hence the same bits, in every warp of every CTA)
            const float *sp = p.ss_part + (size_t)op.ss_slot * G;
            float part = 0.0f;
            for (int c = lane; c < G; c += 32) part += sp[c];
            float tot = 0.0f;
            for (int l2 = 0; l2 < 32; ++l2) tot += __shfl_sync(0xffffffffu, part, l2, 32);
            const float scale = 1.0f / sqrtf(tot / (float)(op.nb * kQK) + p.eps);
#pragma unroll
            for (int u = 0; u < kMaxV; ++u) {
                const int i = ctid + u * PS_CTHREADS;
                if (i < k4)
                    reinterpret_cast<float4 *>(xs)[i] = make_float4(scale * v[u].x * a[u].x, scale * v[u].y * a[u].y, scale * v[u].z * a[u].z, scale * v[u].w * a[u].w);
            }
            consumer_sync();
            xsrc = xs;
        } else if (op.prologue == PS_PRO_ATT_COMBINE) {
            // attention output = the chunks' partial sums rescaled to a common maximum; every CTA combines all heads.
            // Weights first (one thread per (head, chunk) pair, then one per head), then the sums with their loads batched.
            float *wgt = reinterpret_cast<float *>(area);  // [2][nq][nch_max]: the activation-state area is free until the set-up below
            float *lsm = wgt + p.nq * p.nch_max;
            for (int i = ctid; i < p.nq * p.nch_max; i += PS_CTHREADS) {
                const int c = i % p.nch_max;
                const float2 ml = c < nch ? *reinterpret_cast<const float2 *>(p.part + (int64_t)i * (PS_HD + 2)) : make_float2(-INFINITY, 0.0f);
                wgt[i] = ml.x;  // chunk maximum
                lsm[i] = ml.y;  // chunk sum
            }
            consumer_sync();
            for (int head = ctid; head < p.nq; head += PS_CTHREADS) {
                float M = -INFINITY;
                for (int c = 0; c < nch; ++c) M = fmaxf(M, wgt[head * p.nch_max + c]);
                float den = 0.0f;
                for (int c = 0; c < nch; ++c) {
                    const float e = expf(wgt[head * p.nch_max + c] - M);
                    den = fmaf(e, lsm[head * p.nch_max + c], den);
                    wgt[head * p.nch_max + c] = e;
                }
                const float inv = 1.0f / den;
                for (int c = 0; c < nch; ++c) wgt[head * p.nch_max + c] *= inv;
            }
            consumer_sync();
            for (int idx = ctid; idx < p.nq * PS_HD; idx += PS_CTHREADS) {
                const int head = idx >> 7, d = idx & (PS_HD - 1);
                const float *pp = p.part + (int64_t)head * p.nch_max * (PS_HD + 2) + 2 + d;
                const float *wh = wgt + head * p.nch_max;
                float num = 0.0f;
                for (int c0 = 0; c0 < nch; c0 += 8) {
                    float t[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) t[j] = c0 + j < nch ? pp[(c0 + j) * (PS_HD + 2)] : 0.0f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) num = fmaf(c0 + j < nch ? wh[c0 + j] : 0.0f, t[j], num);
                }
                xs[idx] = num;
            }
            consumer_sync();
            xsrc = xs;
        }
        // activation state, once per CTA: four lanes per 32-block, two items per trip with both loads issued first
        {
            const int nitems = op.nb * 4;
            for (int b0 = 0; b0 < nitems; b0 += 2 * PS_CTHREADS) {
                const int i0 = b0 + ctid, i1 = b0 + PS_CTHREADS + ctid;
                float r0[8], r1[8];
                Dec::load_quarter(xsrc, i0, i0 < nitems, r0);
                Dec::load_quarter(xsrc, i1, i1 < nitems, r1);
                Dec::stage_quarter_regs(r0, i0, i0 < nitems, area);
                Dec::stage_quarter_regs(r1, i1, i1 < nitems, area);
            }
            consumer_sync();
        }
        const int rows_per_warp = 32 / op.lanes;
        const int rsub = (cw / op.wpr) * rows_per_warp + lane / op.lanes;
        const int wir = cw % op.wpr;
        const int pair = wir * 32 + (lane % op.lanes);
        const bool active = cw < op.cwarps && pair < op.tpr;
        Dec dec;
        dec.load(area + (size_t)(active ? pair : 0) * 2 * Dec::kStateWordsPerBlock);

        const uint8_t *my_words = smem + 4 * (rsub * (op.row_bytes >> 2) + pair * kWords);
        const int sub_bytes = op.rpp * op.row_bytes;  // distance between a thread's two rows of a pass
        int rows_left = nrows, buf = 0;
        for (int pbase = 0; pbase < npass; pbase += PS_PASS_GROUP) {
            const int ucount = min(PS_PASS_GROUP, npass - pbase);
#pragma unroll 1
            for (int u = 0; u < ucount; ++u, ++it) {
                const int stage = it % p.stages;
                if (!dead && !mbar_wait_bounded(smem_u32(&bar_full[stage]), (it / p.stages) & 1)) {
                    atomicExch(p.err, kDevErrFullWait);
                    dead = true;
                }
                float v0 = 0.0f, v1 = 0.0f;
                const uint8_t *sw = my_words + (size_t)stage * p.stage_bytes;
                const bool go = !dead && active;
                if (go && rsub + op.rpp < rows_left) {
                    v0 = dec.pass(reinterpret_cast<const uint32_t *>(sw));
                    v1 = dec.pass(reinterpret_cast<const uint32_t *>(sw + sub_bytes));
                } else if (go && rsub < rows_left) {
                    v0 = dec.pass(reinterpret_cast<const uint32_t *>(sw));
                }
                // parked BEFORE the stage is released: these stores need every word the pass loaded
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_u32(&stash[(u * 2) * PS_CTHREADS + ctid])), "f"(v0) : "memory");
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_u32(&stash[(u * 2 + 1) * PS_CTHREADS + ctid])), "f"(v1) : "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_empty[stage]));
                rows_left -= rows_per_pass;
            }
            float part[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) part[i] = (i < ucount * 2) ? stash[i * PS_CTHREADS + ctid] : 0.0f;
            // reduce the 8 partials over the lanes of each row segment: three exchange steps halve the live values
            const int L = op.lanes;
            if (L >= 8) {
                const int lr = lane % L;
                int vidx = 0;
                float v4[4], v2[2], v1r;
                {
                    const int off = L >> 1;
                    const bool up = (lr & off) != 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float keep = up ? part[i + 4] : part[i];
                        const float send = up ? part[i] : part[i + 4];
                        v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, off, 32);
                    }
                    vidx = up ? 4 : 0;
                }
                {
                    const int off = L >> 2;
                    const bool up = (lr & off) != 0;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float keep = up ? v4[i + 2] : v4[i];
                        const float send = up ? v4[i] : v4[i + 2];
                        v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, off, 32);
                    }
                    vidx += up ? 2 : 0;
                }
                {
                    const int off = L >> 3;
                    const bool up = (lr & off) != 0;
                    const float keep = up ? v2[1] : v2[0];
                    const float send = up ? v2[0] : v2[1];
                    v1r = keep + __shfl_xor_sync(0xffffffffu, send, off, 32);
                    vidx += up ? 1 : 0;
                }
                for (int off = L >> 4; off > 0; off >>= 1) v1r += __shfl_xor_sync(0xffffffffu, v1r, off, 32);
                const bool writer = (lr & ((L >> 3) - 1)) == 0;
                if (writer && cw < op.cwarps) red[buf][vidx][rsub * op.wpr + wir] = v1r;
            } else {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float t = part[u];
                    for (int off = L >> 1; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
                    if ((lane % L) == 0 && cw < op.cwarps) red[buf][u][rsub * op.wpr + wir] = t;
                }
            }
            consumer_sync();
            for (int t = ctid; t < 8 * op.rpp; t += PS_CTHREADS) {
                const int i = t / op.rpp, rs = t % op.rpp;  // i = pass-in-group * 2 + row-of-thread
                const int u = i >> 1, j = i & 1;
                const int r = (pbase + u) * rows_per_pass + j * op.rpp + rs;
                if (u < ucount && r < nrows) {
                    float tot = 0.0f;
                    for (int w = 0; w < op.wpr; ++w) tot += red[buf][i][rs * op.wpr + w];
                    if (op.epilogue == PS_EPI_SILU_PAIRS) {
                        if ((rs & 1) == 0) {  // rows come in (gate, up) pairs: the even row's thread writes silu(gate) * up
                            float up = 0.0f;
                            for (int w = 0; w < op.wpr; ++w) up += red[buf][i][(rs + 1) * op.wpr + w];
                            op.y[(row_begin + r) >> 1] = tot / (1.0f + expf(-tot)) * up;
                        }
                    } else if (op.epilogue == PS_EPI_RESID) {
                        const float xv = op.x_in[row_begin + r] + tot;
                        op.x_out[row_begin + r] = xv;
                        my_ss = fmaf(xv, xv, my_ss);
                    } else {
                        op.y[row_begin + r] = tot;
                        if (op.epilogue == PS_EPI_STORE_ARGMAX) {
                            const uint32_t idx = (uint32_t)(row_begin + r);
                            if (tot > my_best || (tot == my_best && idx < my_best_idx)) my_best = tot, my_best_idx = idx;
                        }
                    }
                }
            }
            buf ^= 1;
        }
        if (op.epilogue == PS_EPI_RESID) {
            // this CTA's share of sum(x_out^2), summed in a fixed order -> global, for the norm of the next phase
            float t = my_ss;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o, 32);
            if (lane == 0) best_val[cw] = t;
            consumer_sync();
            if (ctid == 0) {
                float tot = 0.0f;
                for (int w = 0; w < PS_CWARPS; ++w) tot += best_val[w];
                p.ss_part[(size_t)op.ss_slot * G + cta] = tot;
            }
            my_ss = 0.0f;
        }
        if (op.epilogue == PS_EPI_STORE_ARGMAX) {
            // this CTA's best (value, lowest index) -> global
            float bv = my_best;
            uint32_t bi = my_best_idx;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o, 32);
                const uint32_t oi2 = __shfl_xor_sync(0xffffffffu, bi, o, 32);
                if (ov > bv || (ov == bv && oi2 < bi)) bv = ov, bi = oi2;
            }
            if (lane == 0) best_val[cw] = bv, best_idx[cw] = bi;
            consumer_sync();
            if (ctid == 0) {
                for (int w = 1; w < PS_CWARPS; ++w)
                    if (best_val[w] > bv || (best_val[w] == bv && best_idx[w] < bi)) bv = best_val[w], bi = best_idx[w];
                p.argmax_part[cta] = make_float2(bv, __uint_as_float(bi));
            }
        }
        grid_arrive();
    }
    // the step is complete on every CTA that CTA 0 has seen arrive: advance the generation for the next launch
    if (cta == 0) {
        grid_wait(p.nops);
        if (ctid == 0) atomicAdd(p.gen, 1u);
    }
}

bool ps_is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

struct cq_decoder {
    cq_decoder_desc d;
    std::vector<PsOp> ops;
    PsOp *ops_dev = nullptr;
    float *qkv = nullptr, *part = nullptr, *xa = nullptr, *xb = nullptr, *o = nullptr, *h = nullptr, *dd = nullptr, *logits = nullptr;
    float2 *argmax_part = nullptr;
    float *ss_part = nullptr;
    unsigned long long *bar_count = nullptr;
    unsigned *gen = nullptr;
    PsParams params;
    size_t smem = 0;
    int grid = 0;
    std::vector<void *> owned;
};

namespace {

// consumer geometry of one linear (the streaming GEMV's rule: a thread owns 64 values of k)
bool ps_plan_linear(PsOp &op, int n, int k, int block_bytes, bool even_rows) {
    const int nb = k / kQK;
    if (nb % 8 != 0) return false;
    const int tpr = nb / 2;
    int lanes, wpr;
    if (tpr >= 32) {
        lanes = 32;
        wpr = (tpr + 31) / 32;
    } else {
        if (!ps_is_pow2(tpr)) return false;
        lanes = tpr;
        wpr = 1;
    }
    if (wpr > PS_CWARPS) return false;
    int row_groups = PS_CWARPS / wpr;
    const int rows_per_warp = 32 / lanes;
    while (row_groups > 1 && (row_groups * rows_per_warp * wpr > 64 || (even_rows && (row_groups * rows_per_warp) % 2 != 0))) --row_groups;
    if (row_groups * rows_per_warp * wpr > 64) return false;
    op.n = n, op.nb = nb, op.row_bytes = nb * block_bytes, op.tpr = tpr, op.lanes = lanes, op.wpr = wpr;
    op.rpp = row_groups * rows_per_warp;
    op.cwarps = row_groups * wpr;
    return true;
}

template <typename T>
cq_status ps_alloc(cq_ctx *ctx, cq_decoder *dec, T **out, size_t count, bool zero) {
    void *ptr = nullptr;
    CQ_CUDA(ctx, cudaMalloc(&ptr, count * sizeof(T)));
    dec->owned.push_back(ptr);
    if (zero) CQ_CUDA(ctx, cudaMemsetAsync(ptr, 0, count * sizeof(T), ctx->stream));
    *out = static_cast<T *>(ptr);
    return CQ_OK;
}

template <class Dec>
cq_status ps_launch(cq_ctx *ctx, cq_decoder *dec) {
    static thread_local int configured = -1;
    auto kern = decode_step_kernel<Dec>;
    if (configured != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - 8192)));
        configured = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(dec->grid);
    cfg.blockDim = dim3(PS_THREADS);
    cfg.dynamicSmemBytes = dec->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: the grid barriers rely on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, dec->params));
    return CQ_OK;
}

}  // namespace

extern "C" {

cq_status cq_decoder_create(cq_ctx *ctx, const cq_decoder_desc *desc, cq_decoder **out) {
    CQ_ENTER(ctx);
    if (!desc || !out) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decoder_create: null pointer");
    *out = nullptr;
    const cq_decoder_desc &d = *desc;
    if (d.qtype != CQ_Q4_0 && d.qtype != CQ_Q8_0) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_decoder_create: Q4_0 / Q8_0 weights only");
    if (d.head_dim != PS_HD) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_decoder_create: head dimension 128 only");
    if (d.n_layers < 1 || d.dim < 256 || d.dim % 256 != 0 || d.ffn < 1 || d.ffn_pad % 256 != 0 || d.ffn_pad < d.ffn || d.vocab < 1 || d.max_ctx < 1 ||
        d.n_heads < 1 || d.n_kv_heads < 1 || d.n_heads % d.n_kv_heads != 0 || d.n_heads * d.head_dim % 256 != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decoder_create: bad shape (dim, heads * 128 and ffn_pad must be multiples of 256)");
    if (!d.wqkv || !d.wo || !d.wgu || !d.wdown || !d.attn_norm || !d.ffn_norm || !d.k_cache || !d.v_cache || !d.embed || !d.wout || !d.final_norm || !d.cos_table || !d.sin_table)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decoder_create: null pointer in the description");
    const int bb = d.qtype == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    const int order = d.order;
    if (order != 0 && order != 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decoder_create: order must be 0 or 1");
    cq_decoder *dec = new cq_decoder();
    dec->d = d;
    auto fail = [&](cq_status s) {
        for (void *ptr : dec->owned) cudaFree(ptr);
        delete dec;
        return s;
    };
    const int qkv_rows = (d.n_heads + 2 * d.n_kv_heads) * d.head_dim, att_dim = d.n_heads * d.head_dim;
    const int nch_max = (d.max_ctx + PS_ATT_CHUNK - 1) / PS_ATT_CHUNK;
    cq_status s = CQ_OK;
    if ((s = ps_alloc(ctx, dec, &dec->qkv, (size_t)qkv_rows, true)) != CQ_OK || (s = ps_alloc(ctx, dec, &dec->part, (size_t)d.n_heads * nch_max * (PS_HD + 2), true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->xa, (size_t)d.dim, true)) != CQ_OK || (s = ps_alloc(ctx, dec, &dec->xb, (size_t)d.dim, true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->o, (size_t)d.dim, true)) != CQ_OK || (s = ps_alloc(ctx, dec, &dec->h, (size_t)d.ffn_pad, true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->dd, (size_t)d.dim, true)) != CQ_OK || (s = ps_alloc(ctx, dec, &dec->logits, (size_t)d.vocab, true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->argmax_part, (size_t)ctx->sm_count, true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->ss_part, (size_t)2 * ctx->sm_count, true)) != CQ_OK || (s = ps_alloc(ctx, dec, &dec->bar_count, (size_t)1, true)) != CQ_OK ||
        (s = ps_alloc(ctx, dec, &dec->gen, (size_t)1, true)) != CQ_OK)
        return fail(s);
    // ---- the step as a list of phases ---------------------------------------------------------------------------
    bool ok = true;
    int max_stage = 0, max_nb = 0;
    auto linear = [&](const void *w, int n, int k, int prologue, int epilogue, const float *x, const float *alpha, const float *x_in, float *x_out, float *y,
                      int ss_slot) {
        PsOp op = {};
        op.kind = PS_LINEAR;
        op.w = static_cast<const uint8_t *>(w);
        ok = ok && w && ps_plan_linear(op, n, k, bb, epilogue == PS_EPI_SILU_PAIRS) && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
        if (epilogue == PS_EPI_SILU_PAIRS) ok = ok && (op.rpp % 2 == 0) && (n % 2 == 0);
        if (prologue == PS_PRO_NORM) ok = ok && k <= 6 * PS_CTHREADS * 4;
        op.prologue = prologue, op.epilogue = epilogue, op.x = x, op.alpha = alpha, op.x_in = x_in, op.x_out = x_out, op.y = y, op.ss_slot = ss_slot;
        if (ok) {
            max_stage = std::max(max_stage, 2 * op.rpp * op.row_bytes);
            max_nb = std::max(max_nb, op.nb);
        }
        dec->ops.push_back(op);
    };
    // The residual stream alternates between two buffers: a linear whose output is added to the stream reads one and
    // writes the other, row by row, in its epilogue; the norm of the next phase reads the new one.
    float *cur = dec->xa, *other = dec->xb;
    int slot = 0;
    for (int l = 0; l < d.n_layers; ++l) {
        if (l == 0) linear(d.wqkv[l], qkv_rows, d.dim, PS_PRO_EMBED_NORM, PS_EPI_STORE, nullptr, d.attn_norm[l], nullptr, cur, dec->qkv, 0);
        else linear(d.wqkv[l], qkv_rows, d.dim, PS_PRO_NORM, PS_EPI_STORE, cur, d.attn_norm[l], nullptr, nullptr, dec->qkv, slot ^ 1);
        PsOp att = {};
        att.kind = PS_ATTENTION;
        att.k_cache = d.k_cache[l], att.v_cache = d.v_cache[l];
        ok = ok && att.k_cache && att.v_cache;
        dec->ops.push_back(att);
        linear(d.wo[l], d.dim, att_dim, PS_PRO_ATT_COMBINE, PS_EPI_RESID, nullptr, nullptr, cur, other, nullptr, slot);
        std::swap(cur, other);
        linear(d.wgu[l], 2 * d.ffn, d.dim, PS_PRO_NORM, PS_EPI_SILU_PAIRS, cur, d.ffn_norm[l], nullptr, nullptr, dec->h, slot);
        slot ^= 1;
        linear(d.wdown[l], d.dim, d.ffn_pad, PS_PRO_PLAIN, PS_EPI_RESID, dec->h, nullptr, cur, other, nullptr, slot);
        std::swap(cur, other);
        slot ^= 1;
    }
    linear(d.wout, d.vocab, d.dim, PS_PRO_NORM, PS_EPI_STORE_ARGMAX, cur, d.final_norm, nullptr, nullptr, dec->logits, slot ^ 1);
    PsOp fin = {};
    fin.kind = PS_FINISH;
    dec->ops.push_back(fin);
    if (!ok) {
        cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_decoder_create: a linear's shape does not fit the persistent kernel (k % 256, k <= 30720, aligned weights, paired rows)");
        return fail(CQ_ERR_UNSUPPORTED);
    }
    // ---- shared memory: ring, partial sums, activation state, prologue activations --------------------------------
    const size_t stash_bytes = (size_t)8 * PS_CTHREADS * sizeof(float);
    size_t coop_bytes = (size_t)max_nb * DecQ16<CQ_Q4_0, 0>::kStateWordsPerBlock * sizeof(uint32_t);
    coop_bytes = std::max(coop_bytes, (size_t)2 * d.n_heads * nch_max * sizeof(float));  // the attention combine's weights live there too
    const size_t xs_bytes = (size_t)std::max(d.dim, att_dim) * sizeof(float);
    const size_t cap = ctx->smem_optin - 8192;  // static shared memory of the kernel, rounded up
    const size_t stage_bytes = ((size_t)max_stage + 127) & ~size_t(127);
    if (cap < stash_bytes + coop_bytes + xs_bytes + 2 * stage_bytes) {
        cq_fail(ctx, CQ_ERR_UNSUPPORTED, "cq_decoder_create: the model's rows do not leave room for a two-stage ring in shared memory");
        return fail(CQ_ERR_UNSUPPORTED);
    }
    int stages = (int)((cap - stash_bytes - coop_bytes - xs_bytes) / stage_bytes);
    if (stages > PS_MAX_STAGES) stages = PS_MAX_STAGES;
    PsParams &p = dec->params;
    p = PsParams{};
    p.stages = stages, p.stage_bytes = (int)stage_bytes;
    p.stash_off = (int)(stages * stage_bytes), p.coop_off = p.stash_off + (int)stash_bytes, p.xs_off = p.coop_off + (int)coop_bytes;
    dec->smem = (size_t)p.xs_off + xs_bytes;
    dec->grid = ctx->sm_count;
    CQ_CUDA(ctx, cudaMalloc((void **)&dec->ops_dev, dec->ops.size() * sizeof(PsOp)));
    dec->owned.push_back(dec->ops_dev);
    CQ_CUDA(ctx, cudaMemcpyAsync(dec->ops_dev, dec->ops.data(), dec->ops.size() * sizeof(PsOp), cudaMemcpyHostToDevice, ctx->stream));
    CQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    p.ops = dec->ops_dev, p.nops = (int)dec->ops.size();
    p.dim = d.dim, p.nq = d.n_heads, p.nkv = d.n_kv_heads, p.max_ctx = d.max_ctx, p.nch_max = nch_max, p.vocab = d.vocab;
    p.eps = d.eps, p.att_scale = 1.0f / sqrtf((float)d.head_dim);
    p.embed = d.embed, p.cos_t = d.cos_table, p.sin_t = d.sin_table;
    p.qkv = dec->qkv, p.part = dec->part, p.argmax_part = dec->argmax_part, p.ss_part = dec->ss_part;
    p.bar_count = dec->bar_count, p.gen = dec->gen;
    p.err = ctx->dev_err_devptr;
    *out = dec;
    return CQ_OK;
}

cq_status cq_decoder_step(cq_ctx *ctx, cq_decoder *dec, uint32_t *ids_dev, int *pos_dev) {
    CQ_ENTER(ctx);
    if (!dec || !ids_dev || !pos_dev) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_decoder_step: null pointer");
    dec->params.ids = ids_dev, dec->params.pos = pos_dev;
    dec->params.poll_limit = ctx->tune.comm_poll_limit > 0 ? (unsigned)ctx->tune.comm_poll_limit : (1u << 22);
    const cq_decoder_desc &d = dec->d;
    if (d.qtype == CQ_Q4_0 && d.order == 0) return ps_launch<DecQ16<CQ_Q4_0, 0>>(ctx, dec);
    if (d.qtype == CQ_Q4_0) return ps_launch<DecQ16<CQ_Q4_0, 1>>(ctx, dec);
    return ps_launch<DecQ16<CQ_Q8_0, 0>>(ctx, dec);
}

const float *cq_decoder_logits(const cq_decoder *dec) { return dec ? dec->logits : nullptr; }

cq_status cq_decoder_destroy(cq_ctx *ctx, cq_decoder *dec) {
    CQ_ENTER(ctx);
    if (!dec) return CQ_OK;
    cudaStreamSynchronize(ctx->stream);
    for (void *ptr : dec->owned) cudaFree(ptr);
    delete dec;
    return CQ_OK;
}

}  // extern "C"
