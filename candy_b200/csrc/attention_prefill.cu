// Prefill attention on the 5th-generation tensor cores: O = softmax(Q K^T * scale) V per (batch, head), f16 or bf16
// in and out, f32 accumulate, behind the interface of the reference's FlashAttention binding
// (llm/internal/flashattn/flash_api.h:71-117 run_mha; semantics of kernels/flash_api.cu:13-147: one split, causal
// switch, grouped-query heads, strides in elements, softmax_lse = max * scale + log(sum)).  The reference ships
// FlashAttention-2 for sm_80 built on CUTLASS (a submodule that is absent from the checkout); this is a from-scratch
// sm_100a kernel with the same contract for the cases a decoder's prompt phase needs.
//
// A work item is (128 query rows, head, batch); keys and values stream through in tiles of 128 keys.  One persistent CTA
// per SM walks its share of the items (heavy first, dealt out in alternating directions): the rings, the barriers'
// phases and the tensor memory carry on from one item to the next, so the next item's Q, first keys and first score
// tile overlap the previous item's normalization and store (measured against one CTA per item: 32 heads x 2048 causal
// 95.8 -> 79.6 us, 2 x 64 heads x 4096 858 -> 760 us; a plain round-robin instead of alternating directions: 89.8 us).
//   warp 0        TMA: the item's Q tile, then K tiles into a three-stage ring and V tiles into a two-stage ring of
//                 its own (128-byte swizzle); a K tile is free as soon as its scores exist, long before its V
//   warp 1        tcgen05.mma issue of S = Q K^T into a 128-column f32 slot of tensor memory (one slot: the compute
//                 warps release it once the scores sit in their registers)
//   warp 10       tcgen05.mma issue of O_tile = P V, with P read from tensor memory as the A operand, into one of two
//                 product slots; one commit per product.  Two issuing threads because one thread issues an
//                 M 128 x N 128 x K 16 instruction every ~100 cycles while the tensor pipe needs 64: with both products on
//                 one thread the issue was the longest role of a tile (2 x 64/8 heads x 4096: 732 -> 659 us)
//   warps 2-9     compute: thread = (query row, half of the columns): warps 2-5 take keys 0-63 of a tile and the first
//                 half of the output row, warps 6-9 the other halves (two warps per tensor-memory lane quarter, two per
//                 scheduler).  Softmax of the half: scores read once (tcgen05.ld, loads in flight together), masked
//                 only on a tile the causal diagonal or the end of the keys cuts (key >= seqlen_k; causal: key > row +
//                 seqlen_k - seqlen_q, the bottom-right alignment of kernels/mask.h:61-62); the two halves of a row
//                 agree on the maximum through shared memory and a 64-thread named barrier; p = ex2.approx of the
//                 scaled difference, written as packed f16 / bf16 pairs into one of two P slots (tcgen05.st).  Then the
//                 previous tile's product is folded into f32 registers, acc = acc * factor + tile, so nothing in
//                 tensor memory is ever rescaled in place and the factor never leaves its thread; at the end
//                 acc / (sum of both halves) goes out as f16 / bf16
// Measured per tile with ONE issuing thread (clock64 counters in an instrumented build): the MMA lane busy ~2400 of
// ~3600 cycles (the tensor pipe itself ~1450 by the profiler's count), the compute warps waiting for scores a third of
// the time; that is what the second issuer removed (a tile now takes ~2800 cycles at 4096 keys).
// Keeping Q in tensor memory as the A operand of S, so that only K is read from shared memory, changed nothing
// (measured, not kept), and so did two S slots with one product slot: the MMAs are neither starved for operands
// nor held back by the S slot.
// V is [key][d] in memory, i.e. N-major for the P V product: the tile is loaded like a K tile and handed to the tensor
// core with an N-major operand descriptor (8-row groups along the keys, 64-wide slabs of d a tile's 16 KB apart).  A V
// the tensor maps cannot address (rows not 16-byte aligned) is transposed into context scratch by a small kernel first
// and read as a K-major V^T (the first form of this kernel did that always: 79.6 us against 58.5 at 32 heads x 2048).
// Every wait is bounded; tensor memory is always freed.
#include <cuda_bf16.h>

#include <cmath>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int FA_M = 128;   // query rows per CTA
constexpr int FA_N = 128;   // keys per tile
constexpr int FA_THREADS = 352;  // TMA warp, first MMA issuer, eight compute warps, second MMA issuer

struct FaParams {
    void *o;
    float *lse;             // [b][h][seqlen_q] or null
    int64_t o_batch_stride, o_row_stride, o_head_stride;
    int b, h, h_k, seqlen_q, seqlen_k;
    int causal;
    float scale_log2;       // softmax_scale * log2(e)
    float scale;            // softmax_scale
    int *err;
};

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(smem_dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
// kind::f16 instruction descriptor with the operand type: f16 (0) or bf16 (1); D f32; both operands K-major.
__host__ __device__ constexpr uint32_t idesc_16(int mm, int nn, bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(nn >> 3) << 17) | ((uint32_t)(mm >> 4) << 24);
}

// 2^x by the special-function unit (relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t *>(&v);
    }
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// V [b][key][h_k][d] (strides in elements) -> Vt [b * h_k][d][sk_pad], 16-bit elements moved as they are.
__global__ void __launch_bounds__(256) fa_transpose_v_kernel(const uint16_t *__restrict__ v, int64_t bs, int64_t rs, int64_t hs, int h_k, int d, int sk,
                                                           int sk_pad, uint16_t *__restrict__ vt) {
    __shared__ uint16_t tile[32][33];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int bh = blockIdx.z, b = bh / h_k, hh = bh - b * h_k;
    const int k0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const uint16_t *src = v + (int64_t)b * bs + (int64_t)hh * hs;
    for (int i = ty; i < 32; i += 8) {
        const int key = k0 + i, dd = d0 + tx;
        tile[i][tx] = (key < sk && dd < d) ? src[(int64_t)key * rs + dd] : (uint16_t)0;
    }
    __syncthreads();
    uint16_t *dst = vt + (int64_t)bh * d * sk_pad;
    for (int i = ty; i < 32; i += 8) {
        const int dd = d0 + i, key = k0 + tx;
        if (dd < d && key < sk_pad) dst[(int64_t)dd * sk_pad + key] = tile[tx][i];
    }
}

template <int D, bool BF16>
struct FaCfg {
    static constexpr int kSlabs = D / 64;                       // 64-wide slabs of the head dimension
    static constexpr int kQBytes = kSlabs * FA_M * 128;         // Q tile
    static constexpr int kKBytes = kSlabs * FA_N * 128;         // K tile
    static constexpr int kVBytes = 2 * D * 128;                 // V^T tile: two 64-key slabs of D rows
    // K and V^T have rings of their own: a K tile is free again as soon as its scores are computed, long before the
    // same tile's V^T (needed only after the softmax) is; with one ring for both, the next K could not be fetched
    // until the previous tile's second product had finished, and that load sat on the critical path of every tile.
    static constexpr int kKStages = 3, kVStages = 2;  // kVStages must stay 2 (see the V^T loads)
    static constexpr size_t kSmem = (size_t)kQBytes + (size_t)kKStages * kKBytes + (size_t)kVStages * kVBytes + 4 * FA_M * 4 /* half-row maxima */ + 2 * FA_M * 4 /* half-row sums */ +
                                    1024 /* alignment */ + 256 /* barriers */;
    // tensor memory columns: S (read into registers as soon as it is complete, so one slot is enough), two P slots
    // (64 columns each: 128 16-bit values), two slots for the tile's P V product
    static constexpr uint32_t kColS = 0, kColP = 128, kColO = 256;
    static_assert(kColO + 2 * D <= 512, "tensor memory");
};

template <int D, bool BF16, bool VT>
__global__ void __launch_bounds__(FA_THREADS, 1)
    fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmVt, const FaParams p) {
    using Cfg = FaCfg<D, BF16>;
    constexpr int SLABS = Cfg::kSlabs, KS = Cfg::kKStages, VS = Cfg::kVStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sm_q = smem;
    uint8_t *sm_k = sm_q + Cfg::kQBytes;                         // [KS][kKBytes]
    uint8_t *sm_v = sm_k + (size_t)KS * Cfg::kKBytes;            // [VS][kVBytes]
    float *sm_mx = reinterpret_cast<float *>(sm_v + (size_t)VS * Cfg::kVBytes);  // [2 tile parities][2 halves][128]: maxima of half rows
    float *sm_l = sm_mx + 4 * FA_M;                              // [2 halves][128] final sums
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm_l + 2 * FA_M);
    uint64_t *q_full = bars, *q_empty = q_full + 1, *k_full = q_empty + 1, *k_empty = k_full + KS, *v_full = k_empty + KS, *s_full = v_full + VS, *s_empty = s_full + 1, *p_full = s_empty + 1,
             *o_full = p_full + 2, *o_empty = o_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A CTA stays on its SM and takes one work item per round: an item is one tile of 128 query rows of one (head, batch).
    // Items are numbered heavy first (late query rows under a causal mask have the most key tiles) and dealt out in
    // alternating directions, which gives every CTA a similar load.  Between items nothing is torn down: the next
    // item's Q and first K tiles are loaded, and its first score tile computed, while the compute warps still normalize
    // and store the previous item's rows.  Every role walks the same list and keeps a running tile count g: stage
    // indices and barrier phases follow g, not the tile's number inside its item.
    const int off = p.seqlen_k - p.seqlen_q;  // causal: key j is visible to row i iff j <= i + off
    const int nq = (p.seqlen_q + FA_M - 1) / FA_M, hb = p.h * p.b, items = nq * hb;
    auto item_at = [&](int w, int &q0, int &head, int &batch, int &ntiles) {
        const int qt = nq - 1 - w / hb, rem = w % hb;
        head = rem % p.h, batch = rem / p.h;
        q0 = qt * FA_M;
        ntiles = (p.seqlen_k + FA_N - 1) / FA_N;
        if (p.causal) {
            const int lim = q0 + FA_M + off;  // keys >= lim are masked for every row of this tile
            const int t = lim <= 0 ? 0 : (lim + FA_N - 1) / FA_N;
            ntiles = t < ntiles ? t : ntiles;
        }
    };
    const int kv_group = p.h / p.h_k;
    // round rd hands out items rd * G .. rd * G + G - 1, forwards on even rounds and backwards on odd ones: the CTA that
    // got the heaviest item of a round gets the lightest of the next
    auto item_of_round = [&](int rd) { return (rd & 1) ? (rd + 1) * (int)gridDim.x - 1 - (int)blockIdx.x : rd * (int)gridDim.x + (int)blockIdx.x; };

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        mbar_init(smem_u32(q_empty), 1);
        for (int s = 0; s < KS; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(smem_u32(&v_full[s]), 1);
        }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(s_empty), 8);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&p_full[s]), 8);
            mbar_init(smem_u32(&o_full[s]), 1);
            mbar_init(smem_u32(&o_empty[s]), 8);
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
            pdl_wait_prior();  // Q, K come from earlier kernels, V^T from the transpose just before this one
            bool ok = true;
            int g = 0, qi = 0;  // key tiles and (non-empty) items loaded so far
            for (int rd = 0; rd * (int)gridDim.x < items && ok; ++rd) {
                const int w = item_of_round(rd);
                if (w >= items) continue;
                int q0, head, batch, ntiles;
                item_at(w, q0, head, batch, ntiles);
                if (ntiles == 0) continue;
                const int kv_head = head / kv_group;
                // Q has one buffer: free once the previous item's last score tile has been computed
                if (qi >= 1 && !mbar_wait_sleep(smem_u32(q_empty), (qi - 1) & 1, 100)) {
                    atomicExch(p.err, kDevErrEmptyWait);
                    ok = false;
                    break;
                }
                mbar_expect_tx(smem_u32(q_full), Cfg::kQBytes);
#pragma unroll
                for (int c = 0; c < SLABS; ++c) tma_load_4d(smem_u32(sm_q + c * (FA_M * 128)), &tmQ, c * 64, head, q0, batch, smem_u32(q_full));
                auto load_k = [&](int t) {  // t: tile of this item; its stage and phase follow g + t
                    const int gt = g + t, s = gt % KS;
                    if (gt >= KS && !mbar_wait_sleep(smem_u32(&k_empty[s]), ((gt / KS) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        return;
                    }
                    mbar_expect_tx(smem_u32(&k_full[s]), Cfg::kKBytes);
#pragma unroll
                    for (int c = 0; c < SLABS; ++c)
                        tma_load_4d(smem_u32(sm_k + (size_t)s * Cfg::kKBytes + c * (FA_N * 128)), &tmK, c * 64, kv_head, t * FA_N, batch, smem_u32(&k_full[s]));
                };
                auto load_v = [&](int t) {
                    const int gt = g + t, s = gt % VS;
                    // a V^T stage is free when the product that read it has finished: the barrier the compute warps wait on
                    // for that product (one commit per tile serves all three uses; VS == 2 == the number of product slots)
                    if (gt >= VS && !mbar_wait_sleep(smem_u32(&o_full[s]), ((gt / VS) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        return;
                    }
                    mbar_expect_tx(smem_u32(&v_full[s]), Cfg::kVBytes);
                    if (VT) {
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf)
                            tma_load_3d(smem_u32(sm_v + (size_t)s * Cfg::kVBytes + hf * (D * 128)), &tmVt, t * FA_N + hf * 64, 0, batch * p.h_k + kv_head,
                                        smem_u32(&v_full[s]));
                    } else {  // the V tile as it lies in memory, [key][d], loaded like a K tile
#pragma unroll
                        for (int c = 0; c < SLABS; ++c)
                            tma_load_4d(smem_u32(sm_v + (size_t)s * Cfg::kVBytes + c * (FA_N * 128)), &tmVt, c * 64, kv_head, t * FA_N, batch, smem_u32(&v_full[s]));
                    }
                };
                // K runs one tile ahead of V^T: K(0), K(1), V(0), K(2), V(1), ...
                load_k(0);
                for (int j = 0; j < ntiles && ok; ++j) {
                    if (j + 1 < ntiles) load_k(j + 1);
                    if (ok) load_v(j);
                }
                g += ntiles;
                ++qi;
            }
            if (ok && qi > 0) {  // leave only when nothing is in flight into this CTA's shared memory
                if (!mbar_wait_sleep(smem_u32(q_full), (qi - 1) & 1, 100)) atomicExch(p.err, kDevErrDrain);
                for (int j = g > KS ? g - KS : 0; j < g && ok; ++j)
                    if (!mbar_wait_sleep(smem_u32(&k_full[j % KS]), (j / KS) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        ok = false;
                    }
                for (int j = g > VS ? g - VS : 0; j < g && ok; ++j)
                    if (!mbar_wait_sleep(smem_u32(&v_full[j % VS]), (j / VS) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        ok = false;
                    }
            }
        }
    } else if (warp == 1) {
        // ---- first MMA issuer: S(t) = Q K(t)^T, as far ahead as the K ring and the score slot allow ----------------------
        // (one thread issues an M 128 x N 128 x K 16 instruction every ~100 cycles, the tensor pipe needs 64: with the two
        // products on one thread the issue was the tile's longest role, with a thread each they run side by side)
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_16(FA_M, FA_N, BF16);
            const uint32_t q_addr = smem_u32(sm_q);
            bool ok = true;
            int g = 0, qi = 0;
            for (int rd = 0; rd * (int)gridDim.x < items && ok; ++rd) {
                const int w = item_of_round(rd);
                if (w >= items) continue;
                int q0, head, batch, ntiles;
                item_at(w, q0, head, batch, ntiles);
                if (ntiles == 0) continue;
                if (!mbar_wait_bounded(smem_u32(q_full), qi & 1)) {
                    ok = false;
                    break;
                }
                for (int t = 0; t < ntiles && ok; ++t) {
                    const int gt = g + t, s = gt % KS;
                    // the K tile has landed; the score slot is free (one slot: the softmax warps free it as soon as they hold
                    // the previous tile's scores in registers)
                    if (!mbar_wait_bounded(smem_u32(&k_full[s]), (gt / KS) & 1) || (gt >= 1 && !mbar_wait_bounded(smem_u32(s_empty), (gt - 1) & 1))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sm_k + (size_t)s * Cfg::kKBytes);
#pragma unroll
                    for (int c = 0; c < SLABS; ++c)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            tc_mma_f16(tmem_base + Cfg::kColS, smem_desc_k128(q_addr + c * (FA_M * 128) + kk * 32),
                                       smem_desc_k128(k_addr + c * (FA_N * 128) + kk * 32), idesc_s, (c | kk) != 0);
                    tc_commit(smem_u32(s_full));
                    tc_commit(smem_u32(&k_empty[s]));  // the K tile is free once these MMAs have read it
                    if (t == ntiles - 1) tc_commit(smem_u32(q_empty));  // and so is Q after the item's last score tile
                }
                g += ntiles;
                ++qi;
            }
            if (!ok) atomicExch(p.err, kDevErrMma);
        }
    } else if (warp == FA_THREADS / 32 - 1) {
        // ---- second MMA issuer: O_tile(t) = P(t) V(t), P from tensor memory as the A operand ----------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_o = idesc_16(FA_M, D, BF16);
            bool ok = true;
            int g = 0;
            for (int rd = 0; rd * (int)gridDim.x < items && ok; ++rd) {
                const int w = item_of_round(rd);
                if (w >= items) continue;
                int q0, head, batch, ntiles;
                item_at(w, q0, head, batch, ntiles);
                for (int j = 0; j < ntiles && ok; ++j) {
                    const int gj = g + j, s = gj % VS, slot = gj & 1;
                    // V and P in place, and the product slot free (the compute warps have folded the tile two back)
                    if (!mbar_wait_bounded(smem_u32(&v_full[s]), (gj / VS) & 1) || !mbar_wait_bounded(smem_u32(&p_full[slot]), (gj >> 1) & 1) ||
                        (gj >= 2 && !mbar_wait_bounded(smem_u32(&o_empty[slot]), ((gj >> 1) - 1) & 1))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t v_addr = smem_u32(sm_v + (size_t)s * Cfg::kVBytes);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step: 8 tensor-memory columns of P
                            // V^T: 32 bytes further along a row of 64 keys (K-major operand).  V itself: 16 rows of 128 bytes further
                            // down (the operand is N-major: d runs along a row, 64-wide slabs of d lie FA_N * 128 bytes apart)
                            const uint64_t bdesc = VT ? smem_desc_k128(v_addr + hf * (D * 128) + kk * 32) : smem_desc_mn128(v_addr + (hf * 4 + kk) * 2048, FA_N * 128);
                            tc_mma_f16_ts(tmem_base + Cfg::kColO + (uint32_t)(slot * D), tmem_base + Cfg::kColP + (uint32_t)(slot * 64 + (hf * 4 + kk) * 8), bdesc,
                                          VT ? idesc_o : (idesc_o | (1u << 16)), (hf | kk) != 0);
                        }
                    tc_commit(smem_u32(&o_full[slot]));  // product ready; its P slot and V stage free
                }
                g += ntiles;
            }
            if (!ok) atomicExch(p.err, kDevErrMma);
        }
    } else {
        // ---- eight compute warps: thread = (query row, one half of the columns) ------------------------------------------
        // Warps 2-5 take key columns 0-63 of a tile's scores and the first half of the output row, warps 6-9 the other
        // halves (a warp may touch only the tensor-memory lanes of its quarter, warp & 3: two warps per quarter).
        // Each does the softmax of its half -- the two halves of a row agree on the maximum through shared memory and
        // a 64-thread named barrier -- and folds its half of the previous tile's P V product into registers
        // (acc = acc * factor + tile).  Two warps per scheduler instead of one hide each other's latencies, and the
        // factor never leaves the thread that computed it.
        constexpr int HC = FA_N / 2, HD = D / 2;
        const int quarter = warp & 3, half = (warp - 2) >> 2, r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        bool ok = true, waited_prior = false;
        int g = 0;
        auto fold = [&](int gt, float alpha, float (&acc)[HD]) -> bool {  // acc = acc * alpha + (P V)(gt), this thread's half of the columns
            if (!mbar_wait_bounded(smem_u32(&o_full[gt & 1]), (gt >> 1) & 1)) {
                if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                return false;
            }
            tc_fence_after();
            const uint32_t o_addr = lane_addr + Cfg::kColO + (uint32_t)((gt & 1) * D + half * HD);
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(o_addr + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(acc[c * 32 + i], alpha, __uint_as_float(v[i]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&o_empty[gt & 1]));
            return true;
        };
        for (int rd = 0; rd * (int)gridDim.x < items; ++rd) {
            const int w = item_of_round(rd);
            if (w >= items) continue;
            int q0, head, batch, ntiles;
            item_at(w, q0, head, batch, ntiles);
            const int row = q0 + r;                                    // global query index
            const int causal_lim = p.causal ? row + off : 0x7FFFFFFF;  // last visible key
            float m_run = -INFINITY, l_run = 0.0f;  // running max of the raw scores (whole row), running sum (this half)
            float alpha_prev = 0.0f;                // the factor of the tile whose product is folded next
            float acc[HD];
#pragma unroll
            for (int i = 0; i < HD; ++i) acc[i] = 0.0f;
            for (int j = 0; j < ntiles; ++j) {
                const int gj = g + j, buf = gj & 1;
                // A warp whose wait gave up keeps walking the tiles without waiting or computing, so that its partner
                // (the other half of the rows' columns) still finds it at the named barrier below.
                if (ok && !mbar_wait_bounded(smem_u32(s_full), gj & 1)) {
                    if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                    ok = false;
                }
                if (!ok) {
                    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
                    continue;
                }
                tc_fence_after();
                const int kmax = min(p.seqlen_k - 1, causal_lim) - j * FA_N - half * HC;  // columns > kmax of this half are masked
                // this half of the row's scores: read out of tensor memory once, kept in registers for both steps
                uint32_t sv[HC];
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) tmem_ld32_async(lane_addr + Cfg::kColS + (uint32_t)(half * HC + c * 32), sv + c * 32);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(s_empty));  // the scores are in registers: the next tile's may be computed
                const bool cut = kmax < HC - 1;  // only a tile that the causal diagonal or the end of the keys cuts needs the mask
                float m_half = -INFINITY;
                if (!cut) {
                    float m8[8];  // eight independent chains
#pragma unroll
                    for (int i = 0; i < 8; ++i) m8[i] = __uint_as_float(sv[i]);
#pragma unroll
                    for (int i = 8; i < HC; i += 8) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) m8[u] = fmaxf(m8[u], __uint_as_float(sv[i + u]));
                    }
                    m_half = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
                } else {
#pragma unroll
                    for (int i = 0; i < HC; ++i)
                        if (i <= kmax) m_half = fmaxf(m_half, __uint_as_float(sv[i]));
                }
                // the row's maximum over both halves
                sm_mx[(buf * 2 + half) * FA_M + r] = m_half;
                asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
                const float m_tile = fmaxf(m_half, sm_mx[(buf * 2 + (half ^ 1)) * FA_M + r]);
                const float m_new = fmaxf(m_run, m_tile);
                const float m_use = m_new == -INFINITY ? 0.0f : m_new;  // a row with no visible key yet: every p is 0
                const float alpha = fast_ex2((m_run - m_use) * p.scale_log2);  // m_run = -inf gives 0: nothing accumulated yet
                const float mb = m_use * p.scale_log2;
                // P has two slots: the product that read this one (two tiles back) has finished -- this warp folded it
                // at the end of the previous iteration (the last tile of the previous item right after its loop).
                // p = exp2(s * scale_log2 - max * scale_log2), summed in f32, stored as 16-bit pairs
                float l2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < HC / 32; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c0 = c * 32 + 2 * i;
                        float p0 = fast_ex2(fmaf(__uint_as_float(sv[c0]), p.scale_log2, -mb));
                        float p1 = fast_ex2(fmaf(__uint_as_float(sv[c0 + 1]), p.scale_log2, -mb));
                        if (cut) {
                            p0 = c0 <= kmax ? p0 : 0.0f;
                            p1 = c0 + 1 <= kmax ? p1 : 0.0f;
                        }
                        l2[(i & 1) * 2] += p0, l2[(i & 1) * 2 + 1] += p1;
                        pk[i] = pack2<BF16>(p0, p1);
                    }
                    tmem_st16(lane_addr + Cfg::kColP + (uint32_t)(buf * (FA_N / 2) + half * (HC / 2) + c * 16), pk);
                }
                tmem_wait_st();
                l_run = l_run * alpha + ((l2[0] + l2[1]) + (l2[2] + l2[3]));
                m_run = m_new;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));  // this warp's part of P is in place
                // the previous tile's product, while the tensor core works on this tile's
                if (j >= 1) ok = fold(gj - 1, alpha_prev, acc);
                alpha_prev = alpha;
            }
            if (ok && ntiles > 0) ok = fold(g + ntiles - 1, alpha_prev, acc);
            g += ntiles;
            // the row's sum over both halves (both used the same maxima); the second barrier keeps the next item's sums
            // out of the buffer until the partner has read this item's
            sm_l[half * FA_M + r] = l_run;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            const float l = l_run + sm_l[(half ^ 1) * FA_M + r];
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            if (!waited_prior) {
                pdl_wait_prior();  // the output buffers may still be read by an earlier kernel
                waited_prior = true;
            }
            if (half == 0 && p.lse && row < p.seqlen_q)  // kernels/softmax.h:206: max * scale + log(sum); +inf for a row with nothing to attend to
                p.lse[((int64_t)batch * p.h + head) * p.seqlen_q + row] = (l == 0.0f || l != l) ? INFINITY : m_run * p.scale + logf(l);
            if (ok && row < p.seqlen_q) {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;  // nothing to attend to: zeros, as the reference writes
                uint16_t *dst = reinterpret_cast<uint16_t *>(p.o) + (int64_t)batch * p.o_batch_stride + (int64_t)row * p.o_row_stride + (int64_t)head * p.o_head_stride +
                                half * HD;
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) {
                    uint4 wv;
                    wv.x = pack2<BF16>(acc[8 * c] * inv, acc[8 * c + 1] * inv);
                    wv.y = pack2<BF16>(acc[8 * c + 2] * inv, acc[8 * c + 3] * inv);
                    wv.z = pack2<BF16>(acc[8 * c + 4] * inv, acc[8 * c + 5] * inv);
                    wv.w = pack2<BF16>(acc[8 * c + 6] * inv, acc[8 * c + 7] * inv);
                    reinterpret_cast<uint4 *>(dst)[c] = wv;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Q / K: [b][row][head][d] with strides in elements -> 4-D map (d, head, row, batch); box = 64 x 1 x 128 x 1.
bool make_qk_map(CUtensorMap *map, const void *base, bool bf16, int d, int heads, int rows, int batches, int64_t hs, int64_t rs, int64_t bs) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batches};
    cuuint64_t strides[3] = {(cuuint64_t)hs * 2, (cuuint64_t)rs * 2, (cuuint64_t)bs * 2};
    cuuint32_t box[4] = {64u, 1u, 128u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// V^T: [b * h_k][d][sk_pad] -> 3-D map (key, d, b * h_k) whose key extent is seqlen_k (keys beyond read as zero); box = 64 keys x d x 1.
bool make_vt_map(CUtensorMap *map, const void *base, bool bf16, int d, int sk, int sk_pad, int planes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)sk, (cuuint64_t)d, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)sk_pad * 2, (cuuint64_t)d * sk_pad * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)d, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool BF16, bool VT>
cq_status run_fa(cq_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const FaParams &p, dim3 grid) {
    static thread_local int configured = -1;
    if (configured != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(fmha_fwd_kernel<D, BF16, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FaCfg<D, BF16>::kSmem));
        configured = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(FA_THREADS);
    cfg.dynamicSmemBytes = FaCfg<D, BF16>::kSmem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, fmha_fwd_kernel<D, BF16, VT>, tq, tk, tv, p));
    return CQ_OK;
}

}  // namespace

extern "C" {

cq_status cq_flash_attention(cq_ctx *ctx, void *q_ptr, void *k_ptr, void *v_ptr, void *o_ptr, void *softmax_lse_ptr, void *alibi_slopes_ptr,
                             int32_t *cu_seqlens_q_ptr, int32_t *cu_seqlens_k_ptr, uint32_t q_batch_stride, uint32_t k_batch_stride,
                             uint32_t v_batch_stride, uint32_t o_batch_stride, uint32_t alibi_slopes_batch_stride, uint32_t q_row_stride,
                             uint32_t k_row_stride, uint32_t v_row_stride, uint32_t o_row_stride, uint32_t q_head_stride, uint32_t k_head_stride,
                             uint32_t v_head_stride, uint32_t o_head_stride, uint32_t b, uint32_t h, uint32_t h_k, uint32_t d, uint32_t d_rounded,
                             float softmax_scale, uint32_t seqlen_q, uint32_t seqlen_k, uint32_t seqlen_q_rounded, uint32_t seqlen_k_rounded, int is_bf16,
                             int is_causal, int unpadded_lse, int window_size_left, int window_size_right, float softcap) {
    CQ_ENTER(ctx);
    (void)alibi_slopes_batch_stride, (void)d_rounded, (void)seqlen_q_rounded, (void)seqlen_k_rounded;
    if (!q_ptr || !k_ptr || !v_ptr || !o_ptr) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: query, key, value, and output tensors must be non-nil");
    if (b == 0 || h == 0 || h_k == 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: batch size, number of heads, and number of KV heads must be positive");
    if (d == 0 || seqlen_q == 0 || seqlen_k == 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: head dimension and sequence lengths must be positive");
    if (h % h_k != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: num_heads must be divisible by num_heads_kv");
    if (d != 64 && d != 128) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "flash attention: this build has kernels for head dimensions 64 and 128");
    if (alibi_slopes_ptr || cu_seqlens_q_ptr || cu_seqlens_k_ptr || window_size_left >= 0 || window_size_right >= 0 || softcap > 0.0f || unpadded_lse)
        return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "flash attention: ALiBi, variable-length batches, sliding windows, soft-capping and the unpadded LSE layout are not built");
    const uint32_t str[] = {q_batch_stride, k_batch_stride, v_batch_stride, o_batch_stride, q_row_stride, k_row_stride, o_row_stride,
                            q_head_stride, k_head_stride, o_head_stride};
    for (uint32_t sv : str)
        if (sv % 8 != 0) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "flash attention: q / k / o strides must be multiples of 8 elements (16-byte rows for the tensor maps)");
    for (const void *ptr : {(const void *)q_ptr, (const void *)k_ptr, (const void *)o_ptr})
        if (reinterpret_cast<uintptr_t>(ptr) & 15) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: q, k, o must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(v_ptr) & 1) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "flash attention: v must be 2-byte aligned");
    if (seqlen_q > (1u << 24) || seqlen_k > (1u << 24) || (uint64_t)b * h > 65535u * 65535ull) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "flash attention: sequence beyond 2^24");
    // V tiles are read where they lie when the tensor maps can address them (16-byte rows); otherwise, or on request
    // (option fa_transpose_v), V is transposed into context scratch first and read as V^T
    const bool v_direct = !ctx->tune.fa_transpose_v && v_batch_stride % 8 == 0 && v_row_stride % 8 == 0 && v_head_stride % 8 == 0 &&
                          (reinterpret_cast<uintptr_t>(v_ptr) & 15) == 0;
    CUtensorMap tq, tk, tv;
    const bool bf = is_bf16 != 0;
    if (!v_direct) {
        const int sk_pad = (int)((seqlen_k + 7) & ~7u);
        const size_t vt_bytes = (size_t)b * h_k * d * sk_pad * 2;
        cq_status s = cq_reserve_scratch(ctx, vt_bytes);
        if (s != CQ_OK) return s;
        uint16_t *vt = static_cast<uint16_t *>(ctx->scratch);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((sk_pad + 31) / 32), (unsigned)((d + 31) / 32), (unsigned)(b * h_k));
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
        CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, fa_transpose_v_kernel, (const uint16_t *)v_ptr, (int64_t)v_batch_stride, (int64_t)v_row_stride,
                                        (int64_t)v_head_stride, (int)h_k, (int)d, (int)seqlen_k, sk_pad, vt));
        if (!make_vt_map(&tv, vt, bf, (int)d, (int)seqlen_k, sk_pad, (int)(b * h_k)))
            return cq_fail(ctx, CQ_ERR_CUDA, "flash attention: cuTensorMapEncodeTiled failed or is unavailable");
    } else if (!make_qk_map(&tv, v_ptr, bf, (int)d, (int)h_k, (int)seqlen_k, (int)b, v_head_stride, v_row_stride, v_batch_stride)) {
        return cq_fail(ctx, CQ_ERR_CUDA, "flash attention: cuTensorMapEncodeTiled failed or is unavailable");
    }
    if (!make_qk_map(&tq, q_ptr, bf, (int)d, (int)h, (int)seqlen_q, (int)b, q_head_stride, q_row_stride, q_batch_stride) ||
        !make_qk_map(&tk, k_ptr, bf, (int)d, (int)h_k, (int)seqlen_k, (int)b, k_head_stride, k_row_stride, k_batch_stride))
        return cq_fail(ctx, CQ_ERR_CUDA, "flash attention: cuTensorMapEncodeTiled failed or is unavailable");
    FaParams p;
    p.o = o_ptr, p.lse = static_cast<float *>(softmax_lse_ptr);
    p.o_batch_stride = o_batch_stride, p.o_row_stride = o_row_stride, p.o_head_stride = o_head_stride;
    p.b = (int)b, p.h = (int)h, p.h_k = (int)h_k, p.seqlen_q = (int)seqlen_q, p.seqlen_k = (int)seqlen_k, p.causal = is_causal ? 1 : 0;
    p.scale = softmax_scale, p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.err = ctx->dev_err_devptr;
    // persistent CTAs, one per SM (the kernel's shared memory allows no more), each walking its share of the work items
    const int64_t items = (int64_t)((seqlen_q + FA_M - 1) / FA_M) * h * b;
    const dim3 grid((unsigned)(items < ctx->sm_count ? items : ctx->sm_count));
    if (v_direct) {
        if (d == 128) return bf ? run_fa<128, true, false>(ctx, tq, tk, tv, p, grid) : run_fa<128, false, false>(ctx, tq, tk, tv, p, grid);
        return bf ? run_fa<64, true, false>(ctx, tq, tk, tv, p, grid) : run_fa<64, false, false>(ctx, tq, tk, tv, p, grid);
    }
    if (d == 128) return bf ? run_fa<128, true, true>(ctx, tq, tk, tv, p, grid) : run_fa<128, false, true>(ctx, tq, tk, tv, p, grid);
    return bf ? run_fa<64, true, true>(ctx, tq, tk, tv, p, grid) : run_fa<64, false, true>(ctx, tq, tk, tv, p, grid);
}

// The reference's own entry point, same symbol and signature (flash_api.h:71-117): a host that binds run_mha
// (llm/internal/flashattn/flashattn.go:145-205) can link this library instead of the reference's static one.  Like the
// reference it returns nothing and runs on the default stream; it keeps one context per device and the status of
// the last call can be read with cq_run_mha_last_status().
static cq_status g_run_mha_status = CQ_OK;
static cq_ctx *g_run_mha_ctx[64] = {};

cq_status cq_run_mha_last_status(void) { return g_run_mha_status; }

void run_mha(void *q_ptr, void *k_ptr, void *v_ptr, void *o_ptr, void *softmax_lse_ptr, void *alibi_slopes_ptr, int32_t *cu_seqlens_q_ptr,
             int32_t *cu_seqlens_k_ptr, uint32_t q_batch_stride, uint32_t k_batch_stride, uint32_t v_batch_stride, uint32_t o_batch_stride,
             uint32_t alibi_slopes_batch_stride, uint32_t q_row_stride, uint32_t k_row_stride, uint32_t v_row_stride, uint32_t o_row_stride,
             uint32_t q_head_stride, uint32_t k_head_stride, uint32_t v_head_stride, uint32_t o_head_stride, uint32_t b, uint32_t h, uint32_t h_k,
             uint32_t d, uint32_t d_rounded, float softmax_scale, uint32_t seqlen_q, uint32_t seqlen_k, uint32_t seqlen_q_rounded,
             uint32_t seqlen_k_rounded, int is_bf16, int is_causal, int unpadded_lse, int window_size_left, int window_size_right, float softcap) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        g_run_mha_status = CQ_ERR_CUDA;
        return;
    }
    if (!g_run_mha_ctx[dev]) {
        g_run_mha_status = cq_ctx_create(dev, &g_run_mha_ctx[dev]);
        if (g_run_mha_status != CQ_OK) return;
        g_run_mha_ctx[dev]->stream = cudaStreamLegacy;  // the reference launches on the default stream (flash_api.cu:145)
    }
    g_run_mha_status = cq_flash_attention(g_run_mha_ctx[dev], q_ptr, k_ptr, v_ptr, o_ptr, softmax_lse_ptr, alibi_slopes_ptr, cu_seqlens_q_ptr,
                                          cu_seqlens_k_ptr, q_batch_stride, k_batch_stride, v_batch_stride, o_batch_stride, alibi_slopes_batch_stride,
                                          q_row_stride, k_row_stride, v_row_stride, o_row_stride, q_head_stride, k_head_stride, v_head_stride,
                                          o_head_stride, b, h, h_k, d, d_rounded, softmax_scale, seqlen_q, seqlen_k, seqlen_q_rounded,
                                          seqlen_k_rounded, is_bf16, is_causal, unpadded_lse, window_size_left, window_size_right, softcap);
}

}  // extern "C"
