// Integer-dot GEMM on the tensor cores: Y[m,n] = X[m,k] . W[n,k]^T with int8 activations, the design of the
// reference's mul_mat_q kernels (tensor/internal/cuda/kernels/quantized.cu:455-578, per-block scales applied at
// :4434-4453) carried onto tcgen05.mma kind::i8.
//
// Every 32-block of k has its own scale on BOTH operands, so an integer accumulator cannot run across blocks:
// one MMA (K = 32) per quant block writes a fresh s32 tile into a rotating tensor-memory slot, epilogue warps
// drain the slot, scale it and accumulate in f32 registers.
//
// Roles are swapped against a textbook GEMM: the 128 weight rows of a tile are the M side (128 tensor-memory
// lanes, thread = weight row in the unpacking and epilogue warps), the activations are the N side (NC columns).
//   warp 0      TMA: raw weight blocks of (tile, 256-wide chunk of k), a [128 rows x 144 / 272 B] byte box
//   warp 1      TMA: the chunk's int8 activation columns, two [NC x 128 B] boxes, 128-byte swizzle
//   warp 2      MMA issue: eight tcgen05.mma.kind::i8 per chunk (M 128, N NC, K 32), one per quant block
//   warps 4-7   unpack: nibbles -> bytes 0..15 (u8) or Q8_0 bytes (s8) into the swizzled K-major A tile in
//               shared memory, the blocks' f16 scales into a side array
//   warps 8..   epilogue: tcgen05.ld of each block's slot, then per column
//                 Q8_1 columns   acc += d4 * (sumi * d8 - 8 * s8)        (vec_dot_q4_0_q8_1, quantized.cu:1919-1941)
//                                acc += (d8_0 * d8_1) * sumi              (vec_dot_q8_0_q8_1, :2058-2073)
//                 plane columns  acc += (d4 * dx) * (128 * S_hi + S_lo + bias)   (15-bit block fixed point, below)
// Two activation encodings share the kernel:
//   Q8_1 columns (CQ_ACT_Q8_1): exactly quantize_q8_1 (quantized.cu:3521-3558): q = round(x / (amax/127)), d and
//     the block's sum kept as f16.
//   plane columns (CQ_ACT_F32 for small batches): each activation block is 15-bit block fixed point,
//     X = rint(x * 16383 / amax) = 128 * hi + lo with hi in [-128, 127] and lo in [0, 127], two int8 columns per
//     activation row; the integer dots are exact and |x - X * amax/16383| <= amax/32766, which lands about 2e-5 of
//     max|y| from candy's CPU path (bar 1e-3).
// Work is the list of (tile, chunk) items, tile-major, cut into equal contiguous shares per CTA; a share that
// holds only part of a tile's k range writes a partial tile to scratch and a small kernel adds the partials in
// CTA order (deterministic).  Every wait is bounded; tensor memory is always freed.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int I8_ROWS = 128;     // weight rows per tile
constexpr int I8_KCHUNK = 256;   // values of k per item (eight quant blocks)
constexpr int I8_BLOCKS = 8;

template <int QT, int NC>
struct I8Cfg {
    static constexpr int kBlockBytes = QT == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    static constexpr int kRowChunk = I8_BLOCKS * kBlockBytes;     // raw bytes of one row per item: 144 / 272
    static constexpr int kWBytes = I8_ROWS * kRowChunk;           // 18 432 / 34 816
    static constexpr int kWStages = QT == CQ_Q4_0 ? 3 : 2;
    static constexpr int kABytes = I8_ROWS * I8_KCHUNK;           // unpacked A tile: two [128 x 128 B] halves
    static constexpr int kAStages = 2;
    static constexpr int kWScaleBytes = I8_BLOCKS * I8_ROWS * 4;  // f32 scale per (block, row)
    static constexpr int kBBytes = NC * I8_KCHUNK;                // activation columns: two [NC x 128 B] halves
    static constexpr int kBStages = NC <= 32 ? 4 : (NC <= 64 ? 3 : 2);  // the epilogue holds a stage (its scales) to the end of the chunk
    static constexpr int kXScaleBytes = I8_BLOCKS * NC * 8;       // float2 per (block, column) (plane mode uses half)
    static constexpr int kEpWarps = NC >= 128 ? 8 : 4;
    static constexpr int kColsPerWarp = NC / (kEpWarps / 4);
    // Accumulator slots in tensor memory, handed over in two groups: the MMAs of a group are committed once and
    // the epilogue takes a whole group per barrier round (NC <= 32: a group is a chunk's eight blocks).
    static constexpr int kSlots = (512 / NC) < 16 ? (512 / NC) : 16;
    static constexpr int kGroup = kSlots / 2;
    static constexpr int kWarpUnpack0 = 4, kWarpEp0 = 8;
    static constexpr int kThreads = 32 * (kWarpEp0 + kEpWarps);
    static constexpr size_t kSmem = (size_t)kWStages * kWBytes + (size_t)kAStages * (kABytes + kWScaleBytes) +
                                    (size_t)kBStages * (kBBytes + kXScaleBytes) + 1024 /* alignment */ + 512 /* barriers */;
    static_assert(kSmem <= 232448, "shared memory");
};

struct I8Params {
    float *y;            // [cols, n] with row pitch ldy (an activation row is a row of y)
    int64_t ldy;
    float *part;         // partial tiles: [2 * ctas][logical cols of this launch][128]
    const float2 *xscale;  // this launch's activation scales, [chunk][8 blocks][logical columns of a launch]: Q8_1 (d8, s8); planes (amax/16383, bias)
    int col0;            // first logical column of this launch (column tile)
    int ncols;           // valid logical columns in this launch
    int n, nchunks;
    int total, per_cta;  // (tile, chunk) items in all and per CTA
    int *err;
};

// ---- activation pre-pass -------------------------------------------------------------------------------
// Eight lanes per (activation row, block), four values each.  MODE 1: Q8_1 columns.  MODE 0: hi / lo plane columns.
// planes: int8 [rows_total][k]; scale: float2 [launch][chunk][8 blocks][ncl] (launch = row / ncl), so that the
// scales one (launch, chunk) item needs are one contiguous run.  Rows >= m are zero (written here).
template <int MODE>
__global__ void __launch_bounds__(256) i8_prepass_kernel(const float *__restrict__ x, int m, int m_pad, int k, int64_t ldx, int order, int is_q4,
                                                       int8_t *__restrict__ planes, float2 *__restrict__ scale, int ncl) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int nb = k / kQK;
    const int64_t total = (int64_t)m_pad * nb * 8;  // a multiple of 8: the eight lanes of a block stay together
    const int l = threadIdx.x & 7;                  // values 4l .. 4l+3 of the block
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t blk = i >> 3;
        const int row = (int)(blk / nb), b = (int)(blk - (int64_t)row * nb);
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (row < m) v = reinterpret_cast<const float4 *>(x + (int64_t)row * ldx + (int64_t)b * kQK)[l];
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
        int q[4];
        float2 sc = make_float2(0.0f, 0.0f);
        if (MODE == 1) {
            // quantize_q8_1 (quantized.cu:3521-3558): d = amax / 127, q = round(x / d) by true division (0 when
            // amax == 0); d and the sum of the block's f32 values are stored as f16 and read back rounded.  The sum
            // follows the reference's xor butterfly over the 32 values (offsets 16, 8, 4 across the lanes here, 2 and 1
            // inside a lane), so its bits agree with the reference kernel's.
            float s0 = v.x, s1 = v.y, s2 = v.z, s3 = v.w;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
                s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, o, 8));
                s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, o, 8));
                s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, o, 8));
                s3 = __fadd_rn(s3, __shfl_xor_sync(0xffffffffu, s3, o, 8));
            }
            const float sum = __fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3));
            const float d = __fdiv_rn(amax, 127.0f);
            q[0] = amax == 0.0f ? 0 : (int)roundf(__fdiv_rn(v.x, d));
            q[1] = amax == 0.0f ? 0 : (int)roundf(__fdiv_rn(v.y, d));
            q[2] = amax == 0.0f ? 0 : (int)roundf(__fdiv_rn(v.z, d));
            q[3] = amax == 0.0f ? 0 : (int)roundf(__fdiv_rn(v.w, d));
            sc.x = __half2float(__float2half_rn(d));
            sc.y = __half2float(__float2half_rn(sum));
        } else {
            const float inv = amax > 0.0f ? 16383.0f / amax : 0.0f;
            q[0] = __float2int_rn(fminf(fmaxf(v.x * inv, -16383.0f), 16383.0f));
            q[1] = __float2int_rn(fminf(fmaxf(v.y * inv, -16383.0f), 16383.0f));
            q[2] = __float2int_rn(fminf(fmaxf(v.z * inv, -16383.0f), 16383.0f));
            q[3] = __float2int_rn(fminf(fmaxf(v.w * inv, -16383.0f), 16383.0f));
            int xsum = q[0] + q[1] + q[2] + q[3];
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) xsum += __shfl_xor_sync(0xffffffffu, xsum, o, 8);
            sc.x = amax * (1.0f / 16383.0f);
            sc.y = __int_as_float(is_q4 ? -8 * xsum : 0);  // an integer carried in the float2's second word
        }
        // Where the four values go inside the block's 32 positions.  Natural order: positions 4l .. 4l+3.  Go
        // (interleaved) order: the unpacking threads emit the low nibbles (even elements) as positions 0..15 and
        // the high nibbles (odd elements) as positions 16..31, so elements 4l, 4l+2 land at 2l, 2l+1 and elements
        // 4l+1, 4l+3 at 16+2l, 16+2l+1.
        const int planes_per_row = MODE == 1 ? 1 : 2;
#pragma unroll
        for (int pl = 0; pl < planes_per_row; ++pl) {
            uint32_t byte[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) byte[t] = MODE == 1 ? (uint32_t)(q[t] & 0xFF) : (pl == 0 ? (uint32_t)((q[t] >> 7) & 0xFF) : (uint32_t)(q[t] & 0x7F));
            int8_t *dst = planes + (int64_t)(planes_per_row * row + pl) * k + (int64_t)b * kQK;
            if (order == 0) {
                *reinterpret_cast<uint16_t *>(dst + 2 * l) = (uint16_t)(byte[0] | (byte[2] << 8));
                *reinterpret_cast<uint16_t *>(dst + 16 + 2 * l) = (uint16_t)(byte[1] | (byte[3] << 8));
            } else {
                *reinterpret_cast<uint32_t *>(dst + 4 * l) = byte[0] | (byte[1] << 8) | (byte[2] << 16) | (byte[3] << 24);
            }
        }
        if (l == 0) scale[((int64_t)(row / ncl) * nb + b) * ncl + (row % ncl)] = sc;
    }
}

// Tiles whose k range was shared between CTAs: y[col][row] = sum of the CTAs' partial tiles, in CTA order.
// CTA i owns items [i*per_cta, (i+1)*per_cta); tile t's items are [t*nchunks, (t+1)*nchunks).
__global__ void __launch_bounds__(128) i8_tile_sum_kernel(const float *__restrict__ part, int ncols, int n, int nchunks, int per_cta,
                                                        float *__restrict__ y, int64_t ldy) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int t = blockIdx.x, col = blockIdx.y;
    const int first = (t * nchunks) / per_cta, last = ((t + 1) * nchunks - 1) / per_cta;
    if (first == last) return;  // one CTA had the tile's whole k range and wrote y itself
    const int row = t * I8_ROWS + threadIdx.x;
    float acc = 0.0f;
    for (int c = first; c <= last; ++c) {
        const int slot = 2 * c + (((c * per_cta) / nchunks == t) ? 0 : 1);  // 0: the tile the CTA's share starts in
        acc += part[((int64_t)slot * ncols + col) * I8_ROWS + threadIdx.x];
    }
    if (row < n) y[(int64_t)col * ldy + row] = acc;
}

__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"  // never accumulate: every quant block gets a fresh tile
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
// kind::i8 instruction descriptor: D s32; A (weights) u8 for Q4_0 nibbles, s8 for Q8_0; B (activations) s8; both K-major.
__host__ __device__ constexpr uint32_t idesc_i8(int mm, int nn, bool a_signed) {
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(nn >> 3) << 17) | ((uint32_t)(mm >> 4) << 24);
}

// NW consecutive 32-bit words that start at 16-bit unit `hw` (a compile-time constant after unrolling) of a row
// held in registers as 32-bit words.
template <int NW, int ROWW>
__device__ __forceinline__ void row_words(const uint32_t (&row)[ROWW], int hw, uint32_t (&out)[NW]) {
    if ((hw & 1) == 0) {
#pragma unroll
        for (int i = 0; i < NW; ++i) out[i] = row[hw / 2 + i];
    } else {
#pragma unroll
        for (int i = 0; i < NW; ++i) out[i] = __funnelshift_r(row[(hw - 1) / 2 + i], row[(hw - 1) / 2 + i + 1], 16);
    }
}

// MODE 1: Q8_1 columns, MODE 0: hi / lo plane columns (NC tensor-memory columns = NC / 2 activation rows).
template <int QT, int MODE, int NC>
__global__ void __launch_bounds__(I8Cfg<QT, NC>::kThreads, 1)
    qgemm_i8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const I8Params p) {
    using Cfg = I8Cfg<QT, NC>;
    constexpr int WST = Cfg::kWStages, AST = Cfg::kAStages, BST = Cfg::kBStages, GROUP = Cfg::kGroup, EPW = Cfg::kEpWarps;
    constexpr int NCL = MODE == 1 ? NC : NC / 2;  // logical columns (activation rows) of the launch
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sm_a = smem;                                            // AST unpacked A tiles (1024-byte aligned halves)
    uint8_t *sm_b = sm_a + (size_t)AST * Cfg::kABytes;               // BST activation tiles
    uint8_t *sm_w = sm_b + (size_t)BST * Cfg::kBBytes;               // WST raw weight stages
    float *sm_ws = reinterpret_cast<float *>(sm_w + (size_t)WST * Cfg::kWBytes);            // [AST][8][128]
    float2 *sm_xs = reinterpret_cast<float2 *>(reinterpret_cast<uint8_t *>(sm_ws) + (size_t)AST * Cfg::kWScaleBytes);  // [BST][8][NCL]
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sm_xs) + (size_t)BST * Cfg::kXScaleBytes);
    uint64_t *w_full = bars, *w_empty = w_full + WST, *a_full = w_empty + WST, *a_empty = a_full + AST, *b_full = a_empty + AST,
             *b_empty = b_full + BST, *s_full = b_empty + BST, *s_empty = s_full + 2;  // one pair per group of slots
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(s_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    const int g0 = blockIdx.x * p.per_cta, g1 = min(g0 + p.per_cta, p.total);

    if (threadIdx.x == 0) {
        for (int s = 0; s < WST; ++s) {
            mbar_init(smem_u32(&w_full[s]), 1);
            mbar_init(smem_u32(&w_empty[s]), 4);          // the unpacking warps
        }
        for (int s = 0; s < AST; ++s) {
            mbar_init(smem_u32(&a_full[s]), 4);           // the unpacking warps
            mbar_init(smem_u32(&a_empty[s]), 1 + EPW);    // the MMAs' commit + every epilogue warp (weight scales read)
        }
        for (int s = 0; s < BST; ++s) {
            mbar_init(smem_u32(&b_full[s]), 1);
            mbar_init(smem_u32(&b_empty[s]), 1 + EPW);    // the MMAs' commit + every epilogue warp (activation scales read)
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);           // the group's MMA commit
            mbar_init(smem_u32(&s_empty[s]), EPW);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 2) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // the segment of the item list that starts at item g: stays inside one tile
    auto segment = [&](int g, int &tile, int &c0, int &cn) {
        tile = g / p.nchunks;
        c0 = g - tile * p.nchunks;
        cn = min(p.nchunks - c0, g1 - g);
    };

    if (warp == 0) {
        // ---- TMA, raw weight blocks (nobody's output: starts at once) -------------------------------
        if (lane == 0) {
            int st = 0;
            bool ok = true;
            for (int g = g0; g < g1 && ok;) {
                int tile, c0, cn;
                segment(g, tile, c0, cn);
                g += cn;
                for (int c = 0; c < cn; ++c, ++st) {
                    const int s = st % WST;
                    if (st >= WST && !mbar_wait_sleep(smem_u32(&w_empty[s]), ((st / WST) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&w_full[s]), Cfg::kWBytes);
                    // rows past n are outside the tensor: zero fill
                    tma_load_2d(smem_u32(sm_w + (size_t)s * Cfg::kWBytes), &tmW, (c0 + c) * (Cfg::kRowChunk / 2), tile * I8_ROWS, smem_u32(&w_full[s]));
                }
            }
            if (ok)  // leave only when nothing is in flight into this CTA's shared memory
                for (int i = st > WST ? st - WST : 0; i < st; ++i)
                    if (!mbar_wait_sleep(smem_u32(&w_full[i % WST]), (i / WST) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        break;
                    }
        }
    } else if (warp == 1) {
        // ---- TMA, int8 activation columns of the chunk (written by the pre-pass before this kernel) -----
        if (lane == 0) {
            pdl_wait_prior();
            int st = 0;
            bool ok = true;
            for (int g = g0; g < g1 && ok;) {
                int tile, c0, cn;
                segment(g, tile, c0, cn);
                g += cn;
                for (int c = 0; c < cn; ++c, ++st) {
                    const int s = st % BST;
                    if (st >= BST && !mbar_wait_sleep(smem_u32(&b_empty[s]), ((st / BST) - 1) & 1, 100)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        ok = false;
                        break;
                    }
                    constexpr uint32_t XS_BYTES = I8_BLOCKS * NCL * 8;
                    mbar_expect_tx(smem_u32(&b_full[s]), Cfg::kBBytes + XS_BYTES);
                    bulk_g2s(smem_u32(sm_xs + (size_t)s * (I8_BLOCKS * NCL)), p.xscale + (int64_t)(c0 + c) * (I8_BLOCKS * NCL), XS_BYTES, smem_u32(&b_full[s]));
                    const int row0 = (MODE == 1 ? p.col0 : 2 * p.col0);
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        tma_load_2d(smem_u32(sm_b + (size_t)s * Cfg::kBBytes + h * (NC * 128)), &tmX, (c0 + c) * I8_KCHUNK + h * 128, row0, smem_u32(&b_full[s]));
                }
            }
            if (ok)
                for (int i = st > BST ? st - BST : 0; i < st; ++i)
                    if (!mbar_wait_sleep(smem_u32(&b_full[i % BST]), (i / BST) & 1, 100)) {
                        atomicExch(p.err, kDevErrDrain);
                        break;
                    }
        }
    } else if (warp == 2) {
        // ---- MMA: one K = 32 instruction per quant block, each into its own tensor-memory slot ----------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_i8(I8_ROWS, NC, QT == CQ_Q8_0);
            int st = 0, gi = 0;  // chunks and groups of blocks issued so far
            bool ok = true;
            for (int g = g0; g < g1 && ok; ++g, ++st) {
                const int sa = st % AST, sb = st % BST;
                if (!mbar_wait_sleep(smem_u32(&a_full[sa]), (st / AST) & 1, 40) || !mbar_wait_sleep(smem_u32(&b_full[sb]), (st / BST) & 1, 40)) {
                    atomicExch(p.err, kDevErrFullWait);
                    break;
                }
                tc_fence_after();
                const uint32_t a0 = smem_u32(sm_a + (size_t)sa * Cfg::kABytes), b0 = smem_u32(sm_b + (size_t)sb * Cfg::kBBytes);
#pragma unroll 1
                for (int j0 = 0; j0 < I8_BLOCKS; j0 += GROUP, ++gi) {
                    const int grp = gi & 1;
                    if (gi >= 2 && !mbar_wait_sleep(smem_u32(&s_empty[grp]), ((gi >> 1) - 1) & 1, 40)) {  // the epilogue has drained this group's slots
                        atomicExch(p.err, kDevErrMma);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int jg = 0; jg < GROUP; ++jg) {
                        const int j = j0 + jg;
                        // block j: half j/4 of the tile (a [rows x 128 B] swizzled slab), 32 bytes of k inside the 128-byte row
                        tc_mma_i8(tmem_base + (uint32_t)((grp * GROUP + jg) * NC), smem_desc_k128(a0 + (j >> 2) * (I8_ROWS * 128) + (j & 3) * 32),
                                  smem_desc_k128(b0 + (j >> 2) * (NC * 128) + (j & 3) * 32), idesc);
                    }
                    tc_commit(smem_u32(&s_full[grp]));  // arrives when the group's MMAs (and all before) have completed
                }
                if (!ok) break;
                tc_commit(smem_u32(&a_empty[sa]));  // arrive when the chunk's MMAs have finished reading shared memory
                tc_commit(smem_u32(&b_empty[sb]));
            }
        }
    } else if (warp >= Cfg::kWarpUnpack0 && warp < Cfg::kWarpEp0) {
        // ---- unpack: thread = weight row of the tile ----------------------------------------------------
        const int r = (warp - Cfg::kWarpUnpack0) * 32 + lane;
        int st = 0;
        for (int g = g0; g < g1; ++g, ++st) {  // (weights are nobody's output: no wait for earlier kernels here)
            const int sw = st % WST, sa = st % AST;
            if (!mbar_wait_sleep(smem_u32(&w_full[sw]), (st / WST) & 1, 60)) {
                if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                break;
            }
            if (st >= AST && !mbar_wait_sleep(smem_u32(&a_empty[sa]), ((st / AST) - 1) & 1, 60)) {
                if (lane == 0) atomicExch(p.err, kDevErrEmptyWait);
                break;
            }
            // The thread's row of the stage, 144 / 272 bytes, in 16-byte loads: at this row pitch eight lanes' 16 bytes
            // fall into distinct banks (32-bit loads would collide four ways).
            constexpr int ROWW = Cfg::kRowChunk / 4;  // 36 / 68 words
            uint32_t row[ROWW];
            {
                const uint4 *src = reinterpret_cast<const uint4 *>(sm_w + (size_t)sw * Cfg::kWBytes + (size_t)r * Cfg::kRowChunk);
#pragma unroll
                for (int i = 0; i < ROWW / 4; ++i) {
                    const uint4 t = src[i];
                    row[4 * i] = t.x, row[4 * i + 1] = t.y, row[4 * i + 2] = t.z, row[4 * i + 3] = t.w;
                }
            }
            uint8_t *a_tile = sm_a + (size_t)sa * Cfg::kABytes;
            float *ws = sm_ws + (size_t)sa * (I8_BLOCKS * I8_ROWS);
#pragma unroll
            for (int j = 0; j < I8_BLOCKS; ++j) {
                constexpr int HWB = Cfg::kBlockBytes / 2;  // 16-bit units per block: 9 / 17
                const uint32_t dword = row[(HWB * j) / 2];
                const uint32_t dbits = ((HWB * j) & 1) ? (dword >> 16) : (dword & 0xFFFFu);
                ws[j * I8_ROWS + r] = __half2float(__ushort_as_half((unsigned short)dbits));
                uint32_t o[8];
                if (QT == CQ_Q4_0) {
                    uint32_t q[4];
                    row_words<4, ROWW>(row, HWB * j + 1, q);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] = q[i] & 0x0F0F0F0Fu, o[4 + i] = (q[i] >> 4) & 0x0F0F0F0Fu;
                } else {
                    row_words<8, ROWW>(row, HWB * j + 1, o);
                }
                // block j -> bytes [32 (j & 3), +32) of the 128-byte row of half j >> 2; 16-byte chunk c sits at c ^ (r & 7)
                uint8_t *dst = a_tile + (j >> 2) * (I8_ROWS * 128) + r * 128;
                const int c = 2 * (j & 3);
                *reinterpret_cast<uint4 *>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<uint4 *>(dst + (((c + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            }
            fence_proxy_async();  // the A tile is read by the tensor core's asynchronous proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&w_empty[sw]));
                mbar_arrive(smem_u32(&a_full[sa]));
            }
        }
    } else if (warp >= Cfg::kWarpEp0) {
        // ---- epilogue: lane = weight row; this warp's share of the columns in registers --------------------
        const int ew = warp - Cfg::kWarpEp0, quarter = warp & 3, chalf = ew >> 2;
        constexpr int CPW = Cfg::kColsPerWarp;               // tensor-memory columns this warp drains
        constexpr int LPW = MODE == 1 ? CPW : CPW / 2;       // logical columns
        const int lcol0 = chalf * LPW;                       // first logical column of this warp inside the launch
        const int r = quarter * 32 + lane;
        pdl_wait_prior();  // y and the partial tiles may still be read by earlier kernels
        float acc[LPW];
#pragma unroll
        for (int i = 0; i < LPW; ++i) acc[i] = 0.0f;
        int st = 0, gi = 0;  // chunks and groups of blocks drained so far
        bool ok = true, first_seg = true;
        for (int g = g0; g < g1 && ok;) {
            int tile, c0, cn;
            segment(g, tile, c0, cn);
            g += cn;
            for (int c = 0; c < cn && ok; ++c, ++st) {
                const int sa = st % AST, sb = st % BST;
                // the weight scales (written by the unpacking warps) and the activation scales (bulk copy) of this chunk are in place
                if (!mbar_wait_sleep(smem_u32(&a_full[sa]), (st / AST) & 1, 60) || !mbar_wait_sleep(smem_u32(&b_full[sb]), (st / BST) & 1, 60)) {
                    if (lane == 0) atomicExch(p.err, kDevErrFullWait);
                    ok = false;
                    break;
                }
                const float *ws = sm_ws + (size_t)sa * (I8_BLOCKS * I8_ROWS);
                const float2 *xs = sm_xs + (size_t)sb * (I8_BLOCKS * NCL);
                // A group of slots is drained in pieces of 16 columns, two register sets in turn: the load of the next
                // piece is in flight while the current one is scaled and accumulated.
                constexpr int PPB = CPW / 16;             // pieces per block
                constexpr int PIECES = GROUP * PPB;       // pieces per group (even)
                const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(chalf * CPW);
#pragma unroll 1
                for (int j0 = 0; j0 < I8_BLOCKS && ok; j0 += GROUP, ++gi) {
                    const int grp = gi & 1;
                    if (!mbar_wait_sleep(smem_u32(&s_full[grp]), (gi >> 1) & 1, 20)) {
                        if (lane == 0) atomicExch(p.err, kDevErrMma);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t gbase = lane_base + (uint32_t)(grp * GROUP * NC);
                    auto fetch = [&](uint32_t (&dst)[16], int e) { tmem_ld16_async(gbase + (uint32_t)((e / PPB) * NC + (e % PPB) * 16), dst); };
                    auto consume = [&](const uint32_t (&v)[16], int e) {
                        const int j = j0 + e / PPB, cb = e % PPB;
                        const float dw = ws[j * I8_ROWS + r];
                        if (MODE == 1) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float2 sc = xs[j * NCL + lcol0 + cb * 16 + i];  // (d8, s8): the same address in every lane
                                const float sumi = (float)(int)v[i];
                                if (QT == CQ_Q4_0) acc[cb * 16 + i] = fmaf(dw, fmaf(sumi, sc.x, -8.0f * sc.y), acc[cb * 16 + i]);
                                else acc[cb * 16 + i] = fmaf(dw * sc.x, sumi, acc[cb * 16 + i]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float2 sc = xs[j * NCL + lcol0 + cb * 8 + i];   // (amax / 16383, bias as an integer)
                                const int t = ((int)v[2 * i] << 7) + (int)v[2 * i + 1] + __float_as_int(sc.y);
                                acc[cb * 8 + i] = fmaf(dw * sc.x, (float)t, acc[cb * 8 + i]);
                            }
                        }
                    };
                    uint32_t va[16], vb[16];
                    fetch(va, 0);
                    tmem_wait_ld();
#pragma unroll
                    for (int u = 0; u < PIECES / 2; ++u) {
                        fetch(vb, 2 * u + 1);
                        consume(va, 2 * u);
                        tmem_wait_ld();
                        if (2 * u + 2 < PIECES) fetch(va, 2 * u + 2);
                        consume(vb, 2 * u + 1);
                        tmem_wait_ld();
                    }
                    // every piece of the group is in registers or already used: its slots may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&s_empty[grp]));
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) {  // this warp has read the chunk's scales
                    mbar_arrive(smem_u32(&a_empty[sa]));
                    mbar_arrive(smem_u32(&b_empty[sb]));
                }
            }
            if (!ok) break;
            // the segment is complete: whole k range -> y, otherwise one of this CTA's two partial slots
            const bool direct = cn == p.nchunks;
            const int row = tile * I8_ROWS + r;
#pragma unroll
            for (int i = 0; i < LPW; ++i) {
                const int lc = lcol0 + i;
                if (lc < p.ncols) {
                    if (direct) {
                        if (row < p.n) p.y[(int64_t)lc * p.ldy + row] = acc[i];
                    } else {
                        p.part[((int64_t)(2 * blockIdx.x + (first_seg ? 0 : 1)) * p.ncols + lc) * I8_ROWS + r] = acc[i];
                    }
                }
                acc[i] = 0.0f;
            }
            first_seg = false;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, 512);
}

// ---- tensor-pipe probe: back-to-back kind::i8 MMAs on operands resident in shared memory ---------------
__global__ void __launch_bounds__(128, 1) i8_mma_peak_kernel(int iters, int *err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sa = smem, *sb = smem + I8_ROWS * 128;  // A [128 x 128 B], B [256 x 128 B]
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_slot;
    for (int i = threadIdx.x; i < (I8_ROWS + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u * (uint32_t)(i & 3);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done), 1);
        fence_mbar_init();
    }
    fence_proxy_async();
    if (threadIdx.x < 32) tmem_alloc(smem_u32(&tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = idesc_i8(I8_ROWS, 256, true);
        for (int it = 0; it < iters; ++it)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                tc_mma_i8(tmem_base + (uint32_t)((it & 1) * 256), smem_desc_k128(smem_u32(sa) + kk * 32), smem_desc_k128(smem_u32(sb) + kk * 32), idesc);
        tc_commit(smem_u32(&done));
        if (!mbar_wait_sleep(smem_u32(&done), 0, 200)) atomicExch(err, kDevErrMma);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

// The raw blocks as a 2-D tensor of 2-byte elements (a Q8_0 item is 272 bytes per row, more than the 256 elements
// a box may span in 1-byte elements): box = one item of 128 rows, no swizzle.
bool make_i8_w_map(CUtensorMap *map, const void *w, int64_t n, int64_t row_bytes, int row_chunk) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 2), (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(row_chunk / 2), (cuuint32_t)I8_ROWS};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// int8 activation columns [rows][k], box = 128 bytes of k x NC rows, 128-byte swizzle.
bool make_i8_x_map(CUtensorMap *map, const void *planes, int64_t rows, int64_t k, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(planes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename Kern, typename... Args>
cq_status i8_launch_chained(cq_ctx *ctx, Kern kern, dim3 grid, dim3 block, size_t smem, Args... args) {
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

template <int QT, int MODE, int NC>
cq_status run_i8(cq_ctx *ctx, const CUtensorMap &tmW, const CUtensorMap &tmX, const I8Params &p, unsigned ctas) {
    static thread_local int configured = -1;
    if (configured != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(qgemm_i8_kernel<QT, MODE, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)I8Cfg<QT, NC>::kSmem));
        configured = ctx->device;
    }
    return i8_launch_chained(ctx, qgemm_i8_kernel<QT, MODE, NC>, dim3(ctas), dim3(I8Cfg<QT, NC>::kThreads), I8Cfg<QT, NC>::kSmem, tmW, tmX, p);
}

template <int QT, int MODE>
cq_status run_i8_nc(cq_ctx *ctx, int nc, const CUtensorMap &tmW, const CUtensorMap &tmX, const I8Params &p, unsigned ctas) {
    switch (nc) {
        case 16: return run_i8<QT, MODE, 16>(ctx, tmW, tmX, p, ctas);
        case 32: return run_i8<QT, MODE, 32>(ctx, tmW, tmX, p, ctas);
        case 64: return run_i8<QT, MODE, 64>(ctx, tmW, tmX, p, ctas);
        default: return run_i8<QT, MODE, 128>(ctx, tmW, tmX, p, ctas);
    }
}

}  // namespace

bool qgemm_i8_supported(int qtype, int64_t k, const void *w, const float *x, int64_t ldx) {
    return (qtype == CQ_Q4_0 || qtype == CQ_Q8_0) && k % I8_KCHUNK == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ldx % 4 == 0;
}

// mode 1: Q8_1 activation columns (CQ_ACT_Q8_1 numerics); mode 0: 15-bit plane columns (CQ_ACT_F32 numerics).
cq_status launch_qgemm_i8(cq_ctx *ctx, int qtype, int order, int mode, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n,
                          float *y, int64_t ldy) {
    if ((reinterpret_cast<uintptr_t>(y) & 3) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemm: misaligned pointer");
    if (n > 0x7FFFFFFF || k > 0x7FFFFFFF || m > (1 << 22)) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: dimension beyond the int8 kernel's limits");
    const int cols_per_row = mode == 1 ? 1 : 2;
    const int64_t tcols = m * cols_per_row;  // tensor-memory columns needed in all
    const int nc = tcols <= 16 ? 16 : (tcols <= 32 ? 32 : (tcols <= 64 ? 64 : 128));
    const int ncl = nc / cols_per_row;       // activation rows per launch
    const int launches = (int)((m + ncl - 1) / ncl);
    const int64_t m_pad = (int64_t)launches * ncl;
    const int nb = (int)(k / kQK);
    const int ntiles = (int)((n + I8_ROWS - 1) / I8_ROWS), nchunks = (int)(k / I8_KCHUNK);
    const int64_t total = (int64_t)ntiles * nchunks;
    if (total > 0x3FFFFFFF) return cq_fail(ctx, CQ_ERR_TOO_LARGE, "gemm: too many tiles");
    int64_t per_cta = (total + ctx->sm_count - 1) / ctx->sm_count;
    if (per_cta < 2) per_cta = total < 2 ? total : 2;
    const unsigned ctas = (unsigned)((total + per_cta - 1) / per_cta);
    const bool shared_tiles = per_cta % nchunks != 0;
    const size_t planes_bytes = (((size_t)m_pad * cols_per_row * k) + 1023) & ~size_t(1023);
    const size_t scale_bytes = (((size_t)nb * m_pad * sizeof(float2)) + 1023) & ~size_t(1023);
    const size_t part_bytes = shared_tiles ? (size_t)2 * ctas * ncl * I8_ROWS * 4 : 0;
    cq_status s = cq_reserve_scratch(ctx, planes_bytes + scale_bytes + part_bytes);
    if (s != CQ_OK) return s;
    int8_t *planes = static_cast<int8_t *>(ctx->scratch);
    float2 *scale = reinterpret_cast<float2 *>(static_cast<uint8_t *>(ctx->scratch) + planes_bytes);
    float *part = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->scratch) + planes_bytes + scale_bytes);
    {
        const int64_t items = m_pad * nb * 8;
        const unsigned cap = (unsigned)ctx->sm_count * 8;
        const unsigned grid = (unsigned)((items + 255) / 256 < cap ? (items + 255) / 256 : cap);
        const int ord = qtype == CQ_Q4_0 ? order : 1;
        if (mode == 1) s = i8_launch_chained(ctx, i8_prepass_kernel<1>, dim3(grid), dim3(256), 0, x, (int)m, (int)m_pad, (int)k, ldx, ord, qtype == CQ_Q4_0 ? 1 : 0, planes, scale, ncl);
        else s = i8_launch_chained(ctx, i8_prepass_kernel<0>, dim3(grid), dim3(256), 0, x, (int)m, (int)m_pad, (int)k, ldx, ord, qtype == CQ_Q4_0 ? 1 : 0, planes, scale, ncl);
        if (s != CQ_OK) return s;
    }
    CUtensorMap tmW, tmX;
    const int bb = qtype == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    if (!make_i8_w_map(&tmW, w, n, (int64_t)nb * bb, I8_BLOCKS * bb) || !make_i8_x_map(&tmX, planes, m_pad * cols_per_row, k, nc))
        return cq_fail(ctx, CQ_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed or is unavailable");
    for (int l = 0; l < launches; ++l) {
        I8Params p;
        p.y = y + (int64_t)l * ncl * ldy, p.ldy = ldy, p.part = part, p.xscale = scale + (int64_t)l * nb * ncl;
        p.col0 = l * ncl;
        p.ncols = (int)((m - (int64_t)l * ncl) < ncl ? (m - (int64_t)l * ncl) : ncl);
        p.n = (int)n, p.nchunks = nchunks, p.total = (int)total, p.per_cta = (int)per_cta;
        p.err = ctx->dev_err_devptr;
        if (qtype == CQ_Q4_0) s = mode == 1 ? run_i8_nc<CQ_Q4_0, 1>(ctx, nc, tmW, tmX, p, ctas) : run_i8_nc<CQ_Q4_0, 0>(ctx, nc, tmW, tmX, p, ctas);
        else s = mode == 1 ? run_i8_nc<CQ_Q8_0, 1>(ctx, nc, tmW, tmX, p, ctas) : run_i8_nc<CQ_Q8_0, 0>(ctx, nc, tmW, tmX, p, ctas);
        if (s != CQ_OK) return s;
        if (shared_tiles) {
            s = i8_launch_chained(ctx, i8_tile_sum_kernel, dim3((unsigned)ntiles, (unsigned)p.ncols), dim3(I8_ROWS), 0, (const float *)part, p.ncols, (int)n,
                                  nchunks, (int)per_cta, p.y, ldy);
            if (s != CQ_OK) return s;
        }
    }
    return CQ_OK;
}

extern "C" cq_status cq_measure_i8_mma_peak(cq_ctx *ctx, int iters, double *tera_ops) {
    CQ_ENTER(ctx);
    if (!tera_ops || iters < 1 || iters > (1 << 20)) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "cq_measure_i8_mma_peak: bad arguments");
    *tera_ops = 0.0;
    const size_t smem = (size_t)(I8_ROWS + 256) * 128 + 1024;
    CQ_CUDA(ctx, cudaFuncSetAttribute(i8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    CQ_CUDA(ctx, cudaEventCreate(&e0));
    CQ_CUDA(ctx, cudaEventCreate(&e1));
    float best = 0.0f;
    for (int rep = 0; rep < 4; ++rep) {  // first repetition warms up
        cudaEventRecord(e0, ctx->stream);
        i8_mma_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->dev_err_devptr);
        cudaEventRecord(e1, ctx->stream);
        cudaEventSynchronize(e1);
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && (best == 0.0f || ms < best)) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    CQ_CUDA(ctx, cudaGetLastError());
    const double ops = 2.0 * I8_ROWS * 256.0 * 32.0 * 4.0 * (double)iters * (double)ctx->sm_count;
    *tera_ops = ops / ((double)best * 1e-3) / 1e12;
    return cq_synchronize(ctx);
}
