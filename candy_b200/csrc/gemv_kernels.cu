// Decode GEMV: y[m,n] = x[m,k] . W[n,k]^T for m <= 8 with Q4_0 / Q8_0 weights.
//
// Streaming kernel (the hot path, HBM-bound).  The weight matrix is one contiguous byte
// stream of n rows x (k/32) blocks.  Each CTA owns a contiguous range of rows and pulls it
// through a ring of shared-memory stages with 1-D bulk async copies (cp.async.bulk,
// completion on mbarriers) issued by a dedicated producer warp; the consumer warps never
// touch global memory for weights.  A consumer thread owns a fixed 64-value slice of k for
// the whole kernel: its 64 activations live in registers (pre-scaled, see below) and every
// pass it reads the two blocks of that slice for one row from shared memory as 32-bit
// words at a lane stride of 9 (Q4_0) or 17 (Q8_0) words -- odd, hence bank-conflict-free.
//
// Decoders (how a consumer thread turns its 64 activations and its 9 / 17 words into a dot product):
//
// DecQ16, the default for CQ_ACT_F32: every 32-block of activations becomes 16-bit block fixed
// point once per CTA (X = rint(x * 32767 / amax), split into a signed high and an unsigned low
// byte plane), and a block's dot product is exact integer arithmetic on packed nibbles / bytes,
// 256 * dp4a(n, hi) + dp4a(n, lo): four weights per instruction and plane, one int -> float
// conversion and two multiplies per block.  Against candy's CPU path (dequantize, then
// tensor/internal/cpu/kernels/conv.go:373-389) the result differs by the 16-bit rounding of the
// activations (about 1e-5 of max|y| on Gaussian data) and by summation order.
//
// DecSlices<S> (option gemv_variant = 2 / 3): S int8 residual slices per block,
// x = d1*q1 + d2*q2 (+ d3*q3) + r; three slices resolve x to f32 level (~1e-6 of max|y|).
//
// DecFma (gemv_variant = 1): plain f32.  A nibble n at bit position 4p of a word is masked in
// place and OR-ed into the mantissa of 2^23, giving the float 2^23 + n*16^p; subtracting
// 2^23 + 8*16^p leaves (n-8)*16^p exactly, and the power of 16 is cancelled by scaling the
// thread's activation by 16^-p once.  Every product x*(q-8) is formed exactly inside an FMA and
// summed in f32 per block: the values of the CPU path in another summation order (~1e-6).  About
// five issued instructions per weight, which caps it near 1.8 TB/s.
//
// DecQ81 (CQ_ACT_Q8_1): activations already quantized by quantize_q8_1, exact integer dots scaled
// per block as the reference's CUDA kernels do.  DecMore: Q4_1 / Q5_0 / Q5_1 on DecQ16's state.
//
// Plain kernel: one warp per row, byte loads, any k % 32 == 0, any alignment, m <= 8.  It is
// the route for shapes the streaming kernel does not take and a second implementation the
// tests compare against.
#include <type_traits>

#include "common.cuh"
#include "dec_q16.cuh"

namespace {

constexpr int kPassUnroll = 8;   // passes whose partial sums are reduced together
constexpr int kMaxStages = 16;
constexpr size_t kStaticSmemReserve = 8192;  // static shared memory of the streaming kernel, rounded up

struct GemvParams {
    const uint8_t *w;
    const float *x;
    float *y;
    int64_t n;
    int nb;            // blocks per row
    int row_bytes;     // nb * block bytes (multiple of 16)
    int tpr;           // threads that cover one row (nb / 2)
    int lanes_per_row; // lanes of a warp on one row: 32, or tpr when tpr < 32 (power of two)
    int wpr;           // warps per row
    int rpp;           // rows per pass
    int cwarps;        // consumer warps
    int stages;
    int stage_bytes;
    int coop_off;      // byte offset of the cooperative activation staging area in dynamic smem, or -1
    // Row-parallel tensor parallelism: instead of y, the results go straight into every rank's
    // receive buffer (peer stores over NVLink), then one counter per peer is bumped per CTA.
    uint2 *const *push_rx;      // [world] this rank's slot in each rank's receive buffer: (value bits, tag)
    const unsigned *push_seq;   // tag of the last completed exchange; this launch tags its values with +1
    int push_world;             // 0 = ordinary launch
    int64_t push_off;           // element offset of this activation row inside the slot
    // Fused prologue / epilogue (0 / null = off): x' = x + delta (written to x_out by CTA 0), then
    // x'' = rmsnorm(x') * alpha, kept in shared memory at xs_off; epilogue 1 pairs adjacent rows.
    const float *delta;
    const float *alpha;
    float *x_out;
    float eps;
    int norm;
    int xs_off;
    int epilogue;
    // Multi-row launches (gemv_stream_mr_kernel): m activation rows against one pass over the weights.
    int m;               // activation rows (<= MR * xg)
    int xg;              // groups of warps that take the same weight rows against different activation rows
    int64_t x_row_bytes; // distance between activation rows (f32 rows, or rows of Q8_1 blocks)
    int64_t ldy;
    const float *bias;   // added to every output row in the epilogue (nn.Linear's bias), or null
    int *err;
    int early;           // 1: the producer fills the ring before the CTA's first barrier
    int independent;     // 1: the caller promises that this launch reads and overwrites nothing an earlier launch still in flight writes
};

// ---- compile-time description of where each value of a thread's two blocks sits --------
// A thread's slice is 36 bytes (Q4_0) = 9 words: [dA:2][qsA:16][dB:2][qsB:16], or 68 bytes
// (Q8_0) = 17 words: [dA:2][qA:32][dB:2][qB:32].
struct Slot {
    int word;   // which 32-bit word
    int shift;  // 0: take from the word, 1: take from word >> 16
    int pos;    // nibble (Q4_0) or byte (Q8_0) position inside the (shifted) word
    int elem;   // index 0..63 of the activation it multiplies (block A: 0..31, block B: 32..63)
    int blk;    // 0 = block A, 1 = block B
};

template <int ORDER>
__host__ __device__ constexpr Slot q4_slot(int s) {
    // s enumerates the 64 nibbles of the 32 data bytes in stream order: data byte = s/2.
    const int db = s / 2, hi = s & 1;
    const int blk = db / 16, j = db % 16;          // byte j of block blk
    const int sbyte = (blk == 0) ? 2 + j : 20 + j; // byte offset inside the 36-byte slice
    const int word = sbyte / 4;
    const int nib = (sbyte % 4) * 2 + hi;          // nibble index 0..7 inside the word
    const int e = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j + hi : j + 16 * hi;
    return Slot{word, nib >= 5 ? 1 : 0, nib >= 5 ? nib - 4 : nib, blk * 32 + e, blk};
}

__host__ __device__ constexpr Slot q8_slot(int s) {
    const int blk = s / 32, j = s % 32;
    const int sbyte = (blk == 0) ? 2 + j : 36 + j;
    const int word = sbyte / 4, b = sbyte % 4;
    return Slot{word, b >= 2 ? 1 : 0, b >= 2 ? b - 2 : b, blk * 32 + j, blk};
}

template <int QT, int ORDER>
__host__ __device__ constexpr Slot slot_of(int s) {
    return QT == CQ_Q4_0 ? q4_slot<ORDER>(s) : q8_slot(s);
}

__host__ __device__ constexpr float pow2i(int e) {  // 2^e for small |e|
    float r = 1.0f;
    for (int i = 0; i < (e < 0 ? -e : e); ++i) r = (e < 0) ? r * 0.5f : r * 2.0f;
    return r;
}

template <int QT>
__host__ __device__ constexpr int bits_per_pos() { return QT == CQ_Q4_0 ? 4 : 8; }

// (v & mask) | magic for Q4_0, (v & mask) ^ (magic | signbit) for Q8_0: one LOP3 either way.
template <int QT>
__device__ __forceinline__ float magic_float(uint32_t v, int pos) {
    if (QT == CQ_Q4_0) return __uint_as_float((v & (0xFu << (4 * pos))) | 0x4B000000u);
    return __uint_as_float((v & (0xFFu << (8 * pos))) ^ (0x4B000000u | (0x80u << (8 * pos))));
}
// The constant to subtract: 2^23 + 8*16^pos (Q4_0) or 2^23 + 128*256^pos (Q8_0).
template <int QT>
__host__ __device__ constexpr float magic_bias(int pos) {
    return 8388608.0f + (QT == CQ_Q4_0 ? 8.0f * pow2i(4 * pos) : 128.0f * pow2i(8 * pos));
}

// ---- decoders: how a consumer thread turns its 64 activations and 9/17 words into a dot ----
template <int QT, int ORDER>
struct DecFma {
    static constexpr bool kCoop = false;
    static constexpr int kStateWordsPerBlock = 0;
    static constexpr int kWords = (QT == CQ_Q4_0) ? 9 : 17;
    static constexpr bool kSplitStage = false;
    __device__ __forceinline__ static void stage_quarter(const float *, int, bool, uint32_t *) {}
    __device__ __forceinline__ static void load_quarter(const float *, int, bool, float (&)[8]) {}
    __device__ __forceinline__ static void stage_quarter_regs(const float (&)[8], int, bool, uint32_t *) {}
    __device__ __forceinline__ void load(const uint32_t *) {}
    static constexpr int kDBWord = (QT == CQ_Q4_0) ? 4 : 8;  // word whose high half is block B's scale
    float xr[kXPerThread];  // xr[s] multiplies slot s; already divided by 16^pos / 256^pos

    __device__ __forceinline__ void init(const float (&x)[kXPerThread]) {
#pragma unroll
        for (int s = 0; s < kXPerThread; ++s) {
            constexpr int bpp = bits_per_pos<QT>();
            const Slot sl = slot_of<QT, ORDER>(s);
            xr[s] = x[sl.elem] * pow2i(-bpp * sl.pos);
        }
    }

    __device__ __forceinline__ float pass(const uint32_t *sw) const {
        uint32_t wv[kWords], ws[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) wv[i] = sw[i];
#pragma unroll
        for (int i = 0; i < kWords; ++i) ws[i] = wv[i] >> 16;
        float2 acc[2][2];
        acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int sidx = 0; sidx < kXPerThread; sidx += 2) {
            const Slot a = slot_of<QT, ORDER>(sidx), b = slot_of<QT, ORDER>(sidx + 1);
            // both slots of a pair come from the same data byte, hence the same block
            float2 f = make_float2(magic_float<QT>(a.shift ? ws[a.word] : wv[a.word], a.pos),
                                   magic_float<QT>(b.shift ? ws[b.word] : wv[b.word], b.pos));
            f = __fadd2_rn(f, make_float2(-magic_bias<QT>(a.pos), -magic_bias<QT>(b.pos)));
            float2 &dst = acc[a.blk][(sidx >> 1) & 1];
            dst = __ffma2_rn(f, make_float2(xr[sidx], xr[sidx + 1]), dst);
        }
        const float dA = fp16_bits_to_f32(wv[0] & 0xFFFFu);
        const float dB = fp16_bits_to_f32(ws[kDBWord]);
        const float sA = (acc[0][0].x + acc[0][0].y) + (acc[0][1].x + acc[0][1].y);
        const float sB = (acc[1][0].x + acc[1][0].y) + (acc[1][1].x + acc[1][1].y);
        return fmaf(dA, sA, dB * sB);
    }
};

template <int QT, int ORDER, int S>
struct DecSlices {
    static constexpr int kWords = (QT == CQ_Q4_0) ? 9 : 17;
    static constexpr int kBlkWords = (QT == CQ_Q4_0) ? 4 : 8;  // data words per block
    static constexpr int kVecs = (QT == CQ_Q4_0) ? 2 : 1;      // low + high nibble vectors, or bytes
    int q[2][kBlkWords][kVecs][S];  // packed int8 activations, lane order matching the weight bytes
    float ds[2][S];                 // slice scales per block
    int bias[2][S];                 // -8 * sum of the slice's int8 values (Q4_0's "-8"), 0 for Q8_0

    // Cooperative set-up.  When a CTA works on several rows at once, its threads would each
    // slice the same activations again; instead every activation block is sliced once per CTA
    // by four adjacent lanes (8 values each) into shared memory, in exactly the register layout
    // the owner threads need, and each thread then loads its two blocks' state.
    // Per block: S x 8 packed words, then S scales, then S biases.
    static constexpr bool kCoop = true;
    static constexpr bool kSplitStage = false;
    static constexpr int kStateWordsPerBlock = S * 10;
    __device__ __forceinline__ static void load_quarter(const float *, int, bool, float (&)[8]) {}
    __device__ __forceinline__ static void stage_quarter_regs(const float (&)[8], int, bool, uint32_t *) {}

    __device__ __forceinline__ static uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
    }

    // item = block * 4 + quarter; all 32 lanes of the warp must call this together.
    __device__ __forceinline__ static void stage_quarter(const float *x, int item, bool valid, uint32_t *area) {
        const int blk = item >> 2, qd = item & 3;
        float r[8];
        if (valid) {
            // plain loads: the source is global memory or, with a fused norm, this CTA's shared memory
            const float4 a = reinterpret_cast<const float4 *>(x)[2 * item];
            const float4 b = reinterpret_cast<const float4 *>(x)[2 * item + 1];
            r[0] = a.x, r[1] = a.y, r[2] = a.z, r[3] = a.w, r[4] = b.x, r[5] = b.y, r[6] = b.z, r[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = 0.0f;
        }
        int idxA, idxB;
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) idxA = 2 * qd, idxB = 2 * qd + 1;
        else if (QT == CQ_Q4_0) idxA = (qd < 2) ? 4 * qd : 4 * (qd - 2) + 1, idxB = idxA + 2;
        else idxA = 2 * qd, idxB = 2 * qd + 1;
        uint32_t *dst = area + blk * kStateWordsPerBlock;
#pragma unroll
        for (int s = 0; s < S; ++s) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(r[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1, 32));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2, 32));
            const float d = amax * (1.0f / 127.0f);
            const float inv = amax > 0.0f ? __fdividef(127.0f, amax) : 0.0f;
            uint32_t qi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float tm = fminf(r[i] * inv, 127.0f) + 12582912.0f;  // 1.5 * 2^23: round to nearest integer
                qi[i] = __float_as_uint(tm);
                if (s + 1 < S) r[i] = fmaf(-(tm - 12582912.0f), d, r[i]);
            }
            uint32_t wa, wb;
            if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
                wa = pack4(qi[0], qi[2], qi[4], qi[6]);  // low nibbles meet the even values
                wb = pack4(qi[1], qi[3], qi[5], qi[7]);
            } else {
                wa = pack4(qi[0], qi[1], qi[2], qi[3]);
                wb = pack4(qi[4], qi[5], qi[6], qi[7]);
            }
            int qsum = __dp4a((int)wa, 0x01010101, __dp4a((int)wb, 0x01010101, 0));
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 1, 32);
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 2, 32);
            if (valid) {
                dst[s * 8 + idxA] = wa;
                dst[s * 8 + idxB] = wb;
                if (qd == 0) {
                    dst[S * 8 + s] = __float_as_uint(d);
                    dst[S * 8 + S + s] = (QT == CQ_Q4_0) ? (uint32_t)(-8 * qsum) : 0u;
                }
            }
        }
    }

    // src: this thread's two consecutive block states (16-byte aligned).
    __device__ __forceinline__ void load(const uint32_t *src) {
        uint32_t t[2 * kStateWordsPerBlock];
#pragma unroll
        for (int i = 0; i < 2 * kStateWordsPerBlock / 4; ++i) {
            const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
            t[4 * i] = v.x, t[4 * i + 1] = v.y, t[4 * i + 2] = v.z, t[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int blk = 0; blk < 2; ++blk)
#pragma unroll
            for (int sl = 0; sl < S; ++sl) {
#pragma unroll
                for (int j = 0; j < 8; ++j) q[blk][j / kVecs][j % kVecs][sl] = (int)t[blk * kStateWordsPerBlock + sl * 8 + j];
                ds[blk][sl] = __uint_as_float(t[blk * kStateWordsPerBlock + S * 8 + sl]);
                bias[blk][sl] = (int)t[blk * kStateWordsPerBlock + S * 8 + S + sl];
            }
    }

    __device__ __forceinline__ void init(const float (&x)[kXPerThread]) {
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            float r[kQK];
#pragma unroll
            for (int i = 0; i < kQK; ++i) r[i] = x[blk * kQK + i];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < kQK; ++i) amax = fmaxf(amax, fabsf(r[i]));
                const float d = amax * (1.0f / 127.0f);
                const float inv = amax > 0.0f ? __fdividef(127.0f, amax) : 0.0f;
                ds[blk][s] = d;
                uint32_t qi[kQK];  // low byte = the int8 value (two's complement)
#pragma unroll
                for (int i = 0; i < kQK; ++i) {
                    const float t = fminf(fmaxf(r[i] * inv, -127.0f), 127.0f);
                    const float tm = t + 12582912.0f;  // 1.5 * 2^23: rounds to nearest integer
                    qi[i] = __float_as_uint(tm);
                    r[i] = fmaf(-(tm - 12582912.0f), d, r[i]);  // residual for the next slice
                }
                int qsum = 0;
#pragma unroll
                for (int wi = 0; wi < kBlkWords; ++wi)
#pragma unroll
                    for (int v = 0; v < kVecs; ++v) {
                        const uint32_t p01 = __byte_perm(qi[act_elem<QT, ORDER>(wi, 0, v)], qi[act_elem<QT, ORDER>(wi, 1, v)], 0x0040);
                        const uint32_t p23 = __byte_perm(qi[act_elem<QT, ORDER>(wi, 2, v)], qi[act_elem<QT, ORDER>(wi, 3, v)], 0x0040);
                        const int packed = (int)__byte_perm(p01, p23, 0x5410);
                        q[blk][wi][v][s] = packed;
                        qsum = __dp4a(packed, 0x01010101, qsum);
                    }
                bias[blk][s] = (QT == CQ_Q4_0) ? -8 * qsum : 0;
            }
        }
    }

    __device__ __forceinline__ float pass(const uint32_t *sw) const {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
        // data words of block A start 2 bytes into the slice: realign with funnel shifts
        uint32_t dw[2][kBlkWords];
#pragma unroll
        for (int i = 0; i < kBlkWords; ++i) {
            dw[0][i] = __funnelshift_r(w[i], w[i + 1], 16);
            dw[1][i] = w[kBlkWords + 1 + i];
        }
        // plain hardware conversion: a NaN scale gives a NaN sum either way
        const float scale[2] = {__half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu))),
                                __half2float(__ushort_as_half((unsigned short)(w[kBlkWords] >> 16)))};
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            int acc[S];
#pragma unroll
            for (int s = 0; s < S; ++s) acc[s] = bias[blk][s];
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi) {
                if (QT == CQ_Q4_0) {
                    const int lo = (int)(dw[blk][wi] & 0x0F0F0F0Fu);
                    const int hi = (int)((dw[blk][wi] >> 4) & 0x0F0F0F0Fu);
#pragma unroll
                    for (int s = 0; s < S; ++s) acc[s] = __dp4a(hi, q[blk][wi][1][s], __dp4a(lo, q[blk][wi][0][s], acc[s]));
                } else {
#pragma unroll
                    for (int s = 0; s < S; ++s) acc[s] = __dp4a((int)dw[blk][wi], q[blk][wi][0][s], acc[s]);
                }
            }
            float v = 0.0f;
#pragma unroll
            for (int s = S - 1; s >= 0; --s) v = fmaf(ds[blk][s], (float)acc[s], v);  // smallest slice first
            total = fmaf(scale[blk], v, total);
        }
        return total;
    }
};

// Q4_1 / Q5_0 / Q5_1 with the 16-bit block fixed point of DecQ16.  The nibble bytes of these formats
// pair with the activations exactly like Q4_0's, so the activation state (and its cooperative set-up)
// is DecQ16<CQ_Q4_0, ORDER>'s; only the slice layout and the per-block closing arithmetic differ:
//   Q4_1, Q5_1:  sum_i (d q_i + m) x_i = d16 * (d * sum q_i X_i + m * sum X_i)
//   Q5_0:        sum_i d (q_i - 16) x_i = d16 * d * (sum q_i X_i - 16 sum X_i)
// with sum X_i recovered from DecQ16's Q4_0 bias (-8 sum X_i).  A fifth bit is spread from qh into
// bit 4 of its byte before the dp4a.  Two consecutive blocks are 40 / 44 / 48 bytes: every field of
// Q4_1 and Q5_1 is word aligned; Q5_0's first block sits 2 bytes off and is realigned by funnel shifts.
template <int QT, int ORDER>
struct DecMore {
    using Base = DecQ16<CQ_Q4_0, ORDER>;
    static constexpr int kBlockBytes = QT == CQ_Q4_1 ? 20 : (QT == CQ_Q5_0 ? 22 : 24);
    static constexpr int kWords = kBlockBytes / 2;  // words of two blocks
    static constexpr bool kCoop = true;
    static constexpr bool kSplitStage = true;
    static constexpr int kStateWordsPerBlock = Base::kStateWordsPerBlock;
    Base b;

    __device__ __forceinline__ static void load_quarter(const float *x, int item, bool valid, float (&r)[8]) { Base::load_quarter(x, item, valid, r); }
    __device__ __forceinline__ static void stage_quarter(const float *x, int item, bool valid, uint32_t *area) { Base::stage_quarter(x, item, valid, area); }
    __device__ __forceinline__ static void stage_quarter_regs(const float (&r)[8], int item, bool valid, uint32_t *area) {
        Base::stage_quarter_regs(r, item, valid, area);
    }
    __device__ __forceinline__ void load(const uint32_t *src) { b.load(src); }
    __device__ __forceinline__ void init(const float (&x)[kXPerThread]) { b.init(x); }

    // four qh bits -> bit 4 of four bytes
    __device__ __forceinline__ static uint32_t spread4(uint32_t bits) { return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) << 4; }

    __device__ __forceinline__ float pass(const uint32_t *sw) const {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
        uint32_t dw[2][4], qh[2] = {0u, 0u};
        float d[2], mn[2] = {0.0f, 0.0f};
        if (QT == CQ_Q4_1) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                d[blk] = __half2float(__ushort_as_half((unsigned short)(w[5 * blk] & 0xFFFFu)));
                mn[blk] = __half2float(__ushort_as_half((unsigned short)(w[5 * blk] >> 16)));
#pragma unroll
                for (int i = 0; i < 4; ++i) dw[blk][i] = w[5 * blk + 1 + i];
            }
        } else if (QT == CQ_Q5_1) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                d[blk] = __half2float(__ushort_as_half((unsigned short)(w[6 * blk] & 0xFFFFu)));
                mn[blk] = __half2float(__ushort_as_half((unsigned short)(w[6 * blk] >> 16)));
                qh[blk] = w[6 * blk + 1];
#pragma unroll
                for (int i = 0; i < 4; ++i) dw[blk][i] = w[6 * blk + 2 + i];
            }
        } else {  // Q5_0: block A at byte 0 (d 0-1, qh 2-5, qs 6-21), block B at byte 22 (d 22-23, qh 24-27, qs 28-43)
            d[0] = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
            qh[0] = __funnelshift_r(w[0], w[1], 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) dw[0][i] = __funnelshift_r(w[1 + i], w[2 + i], 16);
            d[1] = __half2float(__ushort_as_half((unsigned short)(w[5] >> 16)));
            qh[1] = w[6];
#pragma unroll
            for (int i = 0; i < 4; ++i) dw[1][i] = w[7 + i];
        }
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const int xsum = b.bias[blk] / -8;  // exact: the bias is -8 * sum X
            int ah = 0, al = (QT == CQ_Q5_0) ? -16 * xsum : 0;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                int lo = (int)(dw[blk][wi] & 0x0F0F0F0Fu);
                int hi = (int)((dw[blk][wi] >> 4) & 0x0F0F0F0Fu);
                if (QT != CQ_Q4_1) {
                    lo |= (int)spread4(qh[blk] >> (4 * wi));
                    hi |= (int)spread4(qh[blk] >> (16 + 4 * wi));
                }
                ah = __dp4a(hi, b.qh[blk][wi][1], __dp4a(lo, b.qh[blk][wi][0], ah));
                al = Base::dp4a_wu(hi, b.ql[blk][wi][1], Base::dp4a_wu(lo, b.ql[blk][wi][0], al));
            }
            const float v = (float)(ah * 256 + al);
            if (QT == CQ_Q5_0) total = fmaf(d[blk] * b.d16[blk], v, total);
            else total = fmaf(b.d16[blk], fmaf(d[blk], v, mn[blk] * (float)xsum), total);
        }
        return total;
    }
};

// Q8_1 activations, the reference CUDA kernels' numerics (quantized.cu:3521-3558 quantizer, :1919-1941
// and :2058-2073 dots): the activations arrive already quantized by quantize_q8_1 (36-byte blocks:
// f16 d, f16 sum of the block's f32 values, 32 int8) and are only permuted here into the order of
// the weight nibbles; a block contributes d4 * (sumi * d8 - 8 * s8) (Q4_0) or d8_0 * d8_1 * sumi
// (Q8_0) with an exact integer dot sumi.  Cooperative set-up only (p.x points at the Q8_1 blocks).
template <int QT, int ORDER>
struct DecQ81 {
    static constexpr int kWords = (QT == CQ_Q4_0) ? 9 : 17;
    static constexpr int kBlkWords = (QT == CQ_Q4_0) ? 4 : 8;
    static constexpr int kVecs = (QT == CQ_Q4_0) ? 2 : 1;
    static constexpr bool kCoop = true;
    static constexpr bool kSplitStage = false;
    static constexpr int kStateWordsPerBlock = 10;  // 8 packed words, d8, s8
    int q[2][kBlkWords][kVecs];
    float d8[2], s8[2];

    __device__ __forceinline__ static void load_quarter(const float *, int, bool, float (&)[8]) {}
    __device__ __forceinline__ static void stage_quarter_regs(const float (&)[8], int, bool, uint32_t *) {}

    // item = block * 4 + quarter: eight int8 of one Q8_1 block -> two packed words in weight order
    __device__ __forceinline__ static void stage_quarter(const float *x, int item, bool valid, uint32_t *area) {
        if (!valid) return;
        const int blk = item >> 2, qd = item & 3;
        const uint32_t *src = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(x) + (size_t)blk * kQ81Bytes);
        const uint32_t w0 = src[1 + 2 * qd], w1 = src[2 + 2 * qd];  // values 8qd..8qd+3, 8qd+4..8qd+7
        uint32_t wa, wb;
        int idxA, idxB;
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
            wa = __byte_perm(w0, w1, 0x6420), wb = __byte_perm(w0, w1, 0x7531);  // low nibbles meet the even values
            idxA = 2 * qd, idxB = 2 * qd + 1;
        } else if (QT == CQ_Q4_0) {
            wa = w0, wb = w1;
            idxA = (qd < 2) ? 4 * qd : 4 * (qd - 2) + 1, idxB = idxA + 2;
        } else {
            wa = w0, wb = w1;
            idxA = 2 * qd, idxB = 2 * qd + 1;
        }
        uint32_t *dst = area + blk * kStateWordsPerBlock;
        dst[idxA] = wa;
        dst[idxB] = wb;
        if (qd == 0) {
            dst[8] = __float_as_uint(__half2float(__ushort_as_half((unsigned short)(src[0] & 0xFFFFu))));
            dst[9] = __float_as_uint(__half2float(__ushort_as_half((unsigned short)(src[0] >> 16))));
        }
    }

    __device__ __forceinline__ void load(const uint32_t *src) {
        uint32_t t[2 * kStateWordsPerBlock];
#pragma unroll
        for (int i = 0; i < 2 * kStateWordsPerBlock / 4; ++i) {
            const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
            t[4 * i] = v.x, t[4 * i + 1] = v.y, t[4 * i + 2] = v.z, t[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[blk][j / kVecs][j % kVecs] = (int)t[blk * kStateWordsPerBlock + j];
            d8[blk] = __uint_as_float(t[blk * kStateWordsPerBlock + 8]);
            s8[blk] = __uint_as_float(t[blk * kStateWordsPerBlock + 9]);
        }
    }

    __device__ __forceinline__ void init(const float (&)[kXPerThread]) {}  // never used: the planner insists on the cooperative set-up

    __device__ __forceinline__ float pass(const uint32_t *sw) const {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
        uint32_t dw[2][kBlkWords];
#pragma unroll
        for (int i = 0; i < kBlkWords; ++i) {
            dw[0][i] = __funnelshift_r(w[i], w[i + 1], 16);
            dw[1][i] = w[kBlkWords + 1 + i];
        }
        const float scale[2] = {__half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu))),
                                __half2float(__ushort_as_half((unsigned short)(w[kBlkWords] >> 16)))};
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            int acc = 0;
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi) {
                if (QT == CQ_Q4_0) {
                    const int lo = (int)(dw[blk][wi] & 0x0F0F0F0Fu);
                    const int hi = (int)((dw[blk][wi] >> 4) & 0x0F0F0F0Fu);
                    acc = __dp4a(hi, q[blk][wi][1], __dp4a(lo, q[blk][wi][0], acc));
                } else {
                    acc = __dp4a((int)dw[blk][wi], q[blk][wi][0], acc);
                }
            }
            if (QT == CQ_Q4_0) total += __fmul_rn(scale[blk], __fsub_rn(__fmul_rn((float)acc, d8[blk]), __fmul_rn(8.0f, s8[blk])));
            else total += __fmul_rn(__fmul_rn(scale[blk], d8[blk]), (float)acc);
        }
        return total;
    }

    // Set-up in two steps for the multi-row kernel (loads of several items in flight together).
    struct QRegs {
        uint32_t w[3];  // the block's (d, s) word and the quarter's two data words
    };
    __device__ __forceinline__ static void qload(const float *x, int item, bool valid, QRegs &q) {
        if (!valid) {
            q.w[0] = q.w[1] = q.w[2] = 0u;
            return;
        }
        const int blk = item >> 2, qd = item & 3;
        const uint32_t *src = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(x) + (size_t)blk * kQ81Bytes);
        q.w[0] = src[0], q.w[1] = src[1 + 2 * qd], q.w[2] = src[2 + 2 * qd];
    }
    __device__ __forceinline__ static void qstage(const QRegs &q, int item, bool valid, uint32_t *area) {
        if (!valid) return;
        const int blk = item >> 2, qd = item & 3;
        const uint32_t w0 = q.w[1], w1 = q.w[2];
        uint32_t wa, wb;
        int idxA, idxB;
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
            wa = __byte_perm(w0, w1, 0x6420), wb = __byte_perm(w0, w1, 0x7531);
            idxA = 2 * qd, idxB = 2 * qd + 1;
        } else if (QT == CQ_Q4_0) {
            wa = w0, wb = w1;
            idxA = (qd < 2) ? 4 * qd : 4 * (qd - 2) + 1, idxB = idxA + 2;
        } else {
            wa = w0, wb = w1;
            idxA = 2 * qd, idxB = 2 * qd + 1;
        }
        uint32_t *dst = area + blk * kStateWordsPerBlock;
        dst[idxA] = wa;
        dst[idxB] = wb;
        if (qd == 0) {
            dst[8] = __float_as_uint(__half2float(__ushort_as_half((unsigned short)(q.w[0] & 0xFFFFu))));
            dst[9] = __float_as_uint(__half2float(__ushort_as_half((unsigned short)(q.w[0] >> 16))));
        }
    }

    // pass() split in two for the multi-row kernel (see DecQ16::WBlk).
    struct WBlk {
        int a[2][kBlkWords];
        int b[2][kBlkWords];
        float scale[2];
    };
    __device__ __forceinline__ static void unpack(const uint32_t *sw, WBlk &o) {
        uint32_t w[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) w[i] = sw[i];
#pragma unroll
        for (int i = 0; i < kBlkWords; ++i) {
            const uint32_t d0 = __funnelshift_r(w[i], w[i + 1], 16), d1 = w[kBlkWords + 1 + i];
            if (QT == CQ_Q4_0) {
                o.a[0][i] = (int)(d0 & 0x0F0F0F0Fu), o.b[0][i] = (int)((d0 >> 4) & 0x0F0F0F0Fu);
                o.a[1][i] = (int)(d1 & 0x0F0F0F0Fu), o.b[1][i] = (int)((d1 >> 4) & 0x0F0F0F0Fu);
            } else {
                o.a[0][i] = (int)d0, o.a[1][i] = (int)d1;
                o.b[0][i] = 0, o.b[1][i] = 0;
            }
        }
        o.scale[0] = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
        o.scale[1] = __half2float(__ushort_as_half((unsigned short)(w[kBlkWords] >> 16)));
    }
    __device__ __forceinline__ float dot(const WBlk &wb) const {
        float total = 0.0f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            int acc = 0;
#pragma unroll
            for (int wi = 0; wi < kBlkWords; ++wi) {
                if (QT == CQ_Q4_0) acc = __dp4a(wb.b[blk][wi], q[blk][wi][1], __dp4a(wb.a[blk][wi], q[blk][wi][0], acc));
                else acc = __dp4a(wb.a[blk][wi], q[blk][wi][0], acc);
            }
            if (QT == CQ_Q4_0) total += __fmul_rn(wb.scale[blk], __fsub_rn(__fmul_rn((float)acc, d8[blk]), __fmul_rn(8.0f, s8[blk])));
            else total += __fmul_rn(__fmul_rn(wb.scale[blk], d8[blk]), (float)acc);
        }
        return total;
    }
};

// The same numerics straight from f32 activations: quantize_q8_1's arithmetic (quantized.cu:3521-3558) runs in the
// kernel's cooperative set-up instead of a launch of its own.  Four adjacent lanes hold a block, eight values each:
// d = amax / 127 and q = round(x / d) by true division (taken only where the quick quotient x * rcp(d) lies within
// 1e-3 of a rounding tie or is not finite: elsewhere both round to the same integer), d and the block's f32 sum rounded
// to f16; the sum follows the reference's xor butterfly over the 32 values (offsets 16 and 8 across the lanes here,
// 4, 2, 1 inside a lane), so its bits agree with the reference kernel's.  All 32 lanes call the staging together.
template <int QT, int ORDER>
struct DecQ81F : DecQ81<QT, ORDER> {
    using Base = DecQ81<QT, ORDER>;
    static constexpr bool kSplitStage = true;
    __device__ __forceinline__ static void load_quarter(const float *x, int item, bool valid, float (&r)[8]) {
        if (valid) {
            const float4 a = reinterpret_cast<const float4 *>(x)[2 * item];
            const float4 b = reinterpret_cast<const float4 *>(x)[2 * item + 1];
            r[0] = a.x, r[1] = a.y, r[2] = a.z, r[3] = a.w, r[4] = b.x, r[5] = b.y, r[6] = b.z, r[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = 0.0f;
        }
    }
    __device__ __forceinline__ static void stage_quarter_regs(const float (&r)[8], int item, bool valid, uint32_t *area) {
        const int blk = item >> 2, qd = item & 3;
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(r[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1, 32));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2, 32));
        float s[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s[i] = __fadd_rn(r[i], __shfl_xor_sync(0xffffffffu, r[i], 2, 32));   // values 16 apart
            s[i] = __fadd_rn(s[i], __shfl_xor_sync(0xffffffffu, s[i], 1, 32));   // values 8 apart
        }
        const float c0 = __fadd_rn(s[0], s[4]), c1 = __fadd_rn(s[1], s[5]), c2 = __fadd_rn(s[2], s[6]), c3 = __fadd_rn(s[3], s[7]);
        const float sum = __fadd_rn(__fadd_rn(c0, c2), __fadd_rn(c1, c3));
        const float d = __fdiv_rn(amax, 127.0f);
        const float rd = amax == 0.0f ? 0.0f : __frcp_rn(d);
        uint32_t w01[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = r[i] * rd;
            float q = roundf(t);
            if (!(fabsf(fabsf(t - q) - 0.5f) >= 1e-3f)) q = roundf(__fdiv_rn(r[i], d));
            const uint32_t byte = amax == 0.0f ? 0u : (uint32_t)((int)q & 0xFF);
            w01[i >> 2] |= byte << (8 * (i & 3));
        }
        if (!valid) return;
        const uint32_t w0 = w01[0], w1 = w01[1];  // values 8qd .. 8qd+3, 8qd+4 .. 8qd+7
        uint32_t wa, wb;
        int idxA, idxB;
        if (QT == CQ_Q4_0 && ORDER == CQ_ORDER_GO_INTERLEAVED) {
            wa = __byte_perm(w0, w1, 0x6420), wb = __byte_perm(w0, w1, 0x7531);  // low nibbles meet the even values
            idxA = 2 * qd, idxB = 2 * qd + 1;
        } else if (QT == CQ_Q4_0) {
            wa = w0, wb = w1;
            idxA = (qd < 2) ? 4 * qd : 4 * (qd - 2) + 1, idxB = idxA + 2;
        } else {
            wa = w0, wb = w1;
            idxA = 2 * qd, idxB = 2 * qd + 1;
        }
        uint32_t *dst = area + blk * Base::kStateWordsPerBlock;
        dst[idxA] = wa;
        dst[idxB] = wb;
        if (qd == 0) {
            dst[8] = __float_as_uint(__half2float(__float2half_rn(d)));
            dst[9] = __float_as_uint(__half2float(__float2half_rn(sum)));
        }
    }
    __device__ __forceinline__ static void stage_quarter(const float *x, int item, bool valid, uint32_t *area) {
        float r[8];
        load_quarter(x, item, valid, r);
        stage_quarter_regs(r, item, valid, area);
    }
    struct QRegs {
        float r[8];
    };
    __device__ __forceinline__ static void qload(const float *x, int item, bool valid, QRegs &q) { load_quarter(x, item, valid, q.r); }
    __device__ __forceinline__ static void qstage(const QRegs &q, int item, bool valid, uint32_t *area) { stage_quarter_regs(q.r, item, valid, area); }
};

// MAXT / MINB are launch bounds only: geometries of at most 288 threads are compiled to fit two
// CTAs per SM, so that under programmatic dependent launch the next GEMV of the stream can be
// resident (and prefetching its weights) while this one is still computing.
// RPT: rows a thread handles per pass (1 or 2).  Two rows give the scheduler two independent
// instruction streams per warp that share the thread's activation registers.
template <class Dec, int RPT, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) gemv_stream_kernel(const GemvParams p) {
    constexpr int kWords = Dec::kWords;
    constexpr int kPassGroup = kPassUnroll / RPT;  // passes per reduction group (8 partial sums)
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[kMaxStages];
    __shared__ uint64_t bar_empty[kMaxStages];
    __shared__ float red[2][kPassUnroll][64];  // [buffer][pass][rsub * wpr + warp-in-row], rpp*wpr <= 64

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int cthreads = p.cwarps * 32;
    float *stash = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);  // [8][cthreads] partial sums
    const bool is_producer = warp == p.cwarps;

    // Rows of this CTA: an even split of [0, n).
    // (with the pairing epilogue the split falls on even rows)
    const int64_t unit = p.epilogue == 1 ? 2 : 1;
    int64_t row_begin, row_end;
    {
        const int64_t units = p.n / unit;
        if (units * (int64_t)gridDim.x < (int64_t)1 << 32) {  // the usual case: 32-bit divisions (a 64-bit one is a long subroutine on the way to the first copy)
            row_begin = unit * (int64_t)(((uint32_t)units * blockIdx.x) / gridDim.x);
            row_end = unit * (int64_t)(((uint32_t)units * (blockIdx.x + 1)) / gridDim.x);
        } else {
            row_begin = unit * ((units * (int64_t)blockIdx.x) / gridDim.x);
            row_end = unit * ((units * (int64_t)(blockIdx.x + 1)) / gridDim.x);
        }
    }
    const int nrows = (int)(row_end - row_begin);
    const int rows_per_pass = p.rpp * RPT;
    const int npass = (nrows + rows_per_pass - 1) / rows_per_pass;

    // Let the next kernel in the stream become resident as soon as every CTA of this one is:
    // its producer warp may prefetch weights, everything else there waits for this grid.
    pdl_launch_dependents();

    // Weights are read exactly once: mark them evict-first so that the stream does not push
    // the activations (re-read by every CTA) and the outputs out of L2.
    uint64_t policy = 0;
    int issued = 0;
    auto issue_pass = [&](int ps) {
        const int s = ps % p.stages;
        const int r0 = ps * rows_per_pass;
        const int rows = min(rows_per_pass, nrows - r0);
        const uint32_t bytes = (uint32_t)rows * (uint32_t)p.row_bytes;
        mbar_expect_tx(smem_u32(&bar_full[s]), bytes);
        bulk_g2s_hint(smem_u32(smem + (size_t)s * p.stage_bytes), p.w + (row_begin + r0) * (int64_t)p.row_bytes, bytes,
                      smem_u32(&bar_full[s]), policy);
        issued = ps + 1;
    };
    // The producer lane initialises the barriers (and, with the `early` option, fills the ring before the CTA
    // meets).  Weights do not depend on the previous kernel in the stream, so under programmatic dependent
    // launch the ring fills while that kernel is still draining.
    if (is_producer && lane == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), p.cwarps);
        }
        fence_mbar_init();
        fence_proxy_async();
        policy = make_l2_policy_evict_first();
        if (p.early) {
            const int first = min(npass, p.stages);
            for (int ps = 0; ps < first; ++ps) issue_pass(ps);
        }
    }
    __syncthreads();

    if (is_producer) {
        // ---- producer warp: one lane streams this CTA's rows into the ring ---------------
        if (lane == 0) {
            for (int ps = issued; ps < npass; ++ps) {
                const int s = ps % p.stages;
                if (ps >= p.stages && !mbar_wait_bounded(smem_u32(&bar_empty[s]), ((ps / p.stages) - 1) & 1)) {
                    atomicExch(p.err, kDevErrEmptyWait);
                    break;
                }
                issue_pass(ps);
            }
            // Do not leave while copies into this CTA's shared memory may still be in flight:
            // wait (bounded) for the last use of every stage that was issued.
            const int first = issued > p.stages ? issued - p.stages : 0;
            for (int ps = first; ps < issued; ++ps) {
                if (!mbar_wait_bounded(smem_u32(&bar_full[ps % p.stages]), (ps / p.stages) & 1)) {
                    atomicExch(p.err, kDevErrDrain);
                    break;
                }
            }
        }
        return;
    }

    // ---- consumer warps ---------------------------------------------------------------------
    // Thread -> (row inside a pass, 64-value slice of k).
    const int rows_per_warp = 32 / p.lanes_per_row;
    const int rsub = (warp / p.wpr) * rows_per_warp + lane / p.lanes_per_row;
    const int wir = warp % p.wpr;  // warp index inside the row
    const int pair = wir * 32 + (lane % p.lanes_per_row);
    const bool active = pair < p.tpr;

    // Activations depend on the previous kernel in the stream, unless the caller has said otherwise (option
    // gemv_independent): then this launch's set-up and first rows overlap the previous launch's last ones.
    if (!p.independent) pdl_wait_prior();

    // Fused prologue: x' = x + delta (CTA 0 also stores it to x_out: the caller ping-pongs two residual
    // buffers, every other CTA keeps reading the old one), x'' = x' / sqrt(mean(x'^2) + eps) * alpha.
    // Every CTA computes the same numbers in the same order; the result lives in shared memory and
    // the activation set-up below reads it from there.
    const float *xsrc = p.x;
    if (p.xs_off >= 0) {
        float *xs = reinterpret_cast<float *>(smem + p.xs_off);
        const int k4 = p.nb * 8;  // float4 groups in a row
        float ss = 0.0f;
        for (int i = tid; i < k4; i += cthreads) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(p.x) + i);
            if (p.delta) {
                const float4 d = __ldg(reinterpret_cast<const float4 *>(p.delta) + i);
                v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
            }
            if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[i] = v;
            reinterpret_cast<float4 *>(xs)[i] = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        if (p.norm) {
            // consumer-only block sum (the producer warp is not part of barrier 1)
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, 32);
            if (lane == 0) red[0][0][warp] = ss;
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            float tot = 0.0f;
            for (int w = 0; w < p.cwarps; ++w) tot += red[0][0][w];
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");  // red is reused by the reduction below
            const float scale = 1.0f / sqrtf(tot / (float)(p.nb * kQK) + p.eps);
            for (int i = tid; i < k4; i += cthreads) {  // each thread rescales what it wrote itself
                float4 v = reinterpret_cast<float4 *>(xs)[i];
                const float4 a = __ldg(reinterpret_cast<const float4 *>(p.alpha) + i);
                v.x = scale * v.x * a.x, v.y = scale * v.y * a.y, v.z = scale * v.z * a.z, v.w = scale * v.w * a.w;
                reinterpret_cast<float4 *>(xs)[i] = v;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        xsrc = xs;
    }

    Dec dec;
    if (Dec::kCoop && p.coop_off >= 0) {
        uint32_t *area = reinterpret_cast<uint32_t *>(smem + p.coop_off);
        const int nitems = p.nb * 4;
        if (Dec::kSplitStage) {
            // two items per trip with both loads issued first: one L2 round trip for k <= 16 * threads
            for (int base = 0; base < nitems; base += 2 * cthreads) {  // uniform trip count: the shuffles need whole warps
                const int i0 = base + tid, i1 = base + cthreads + tid;
                float r0[8], r1[8];
                Dec::load_quarter(xsrc, i0, i0 < nitems, r0);
                Dec::load_quarter(xsrc, i1, i1 < nitems, r1);
                Dec::stage_quarter_regs(r0, i0, i0 < nitems, area);
                Dec::stage_quarter_regs(r1, i1, i1 < nitems, area);
            }
        } else {
            for (int base = 0; base < nitems; base += cthreads) {
                const int item = base + tid;
                Dec::stage_quarter(xsrc, item, item < nitems, area);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        if (active) dec.load(area + (size_t)pair * 2 * Dec::kStateWordsPerBlock);
        else dec.load(area);  // idle lanes: any valid state, their results are never used
    } else {
        float tmp[kXPerThread];
        if (active) {
            const float4 *xv = reinterpret_cast<const float4 *>(xsrc + (int64_t)pair * kXPerThread);
#pragma unroll
            for (int i = 0; i < kXPerThread / 4; ++i) {
                float4 t = xv[i];
                tmp[4 * i] = t.x, tmp[4 * i + 1] = t.y, tmp[4 * i + 2] = t.z, tmp[4 * i + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < kXPerThread; ++i) tmp[i] = 0.0f;
        }
        dec.init(tmp);
    }

    // Loop state is kept incremental (stage index, phase bit, rows left): an integer divide or
    // modulo per pass costs more ALU-pipe slots than the pass's own mask instructions.
    const uint8_t *my_words = smem + 4 * (rsub * (p.row_bytes >> 2) + pair * kWords);
    const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
    int stage = 0;
    uint32_t phase = 0;
    int rows_left = nrows;
    int buf = 0;
    bool dead = false;
    const unsigned push_tag = p.push_world > 0 ? *p.push_seq + 1u : 0u;

    const int sub_bytes = p.rpp * p.row_bytes;  // distance between a thread's two rows of a pass
    for (int pbase = 0; pbase < npass; pbase += kPassGroup) {
        const int ucount = min(kPassGroup, npass - pbase);
        // One copy of the pass body; each pass parks its partial sums in shared memory and the
        // eight are read back below (a chain of predicated moves per pass costs more).
#pragma unroll 1
        for (int u = 0; u < ucount; ++u) {
            // A warp whose wait gave up keeps walking the loop without waiting or computing,
            // so that every consumer still reaches the barriers below and the CTA can exit.
            if (!dead && !mbar_wait_bounded(full0 + 8 * stage, phase)) {
                atomicExch(p.err, kDevErrFullWait);
                dead = true;
            }
            float v[RPT];
#pragma unroll
            for (int j = 0; j < RPT; ++j) v[j] = 0.0f;
            const uint8_t *sw = my_words + stage * p.stage_bytes;
            const bool go = !dead && active;
            if (RPT == 2 && go && rsub + p.rpp < rows_left) {
                // both rows present: one basic block, so the two streams interleave
                v[0] = dec.pass(reinterpret_cast<const uint32_t *>(sw));
                v[RPT - 1] = dec.pass(reinterpret_cast<const uint32_t *>(sw + sub_bytes));
            } else if (go && rsub < rows_left) {
                v[0] = dec.pass(reinterpret_cast<const uint32_t *>(sw));
            }
            // The partial sums are parked BEFORE the stage is released: these stores need every word
            // the pass loaded, and instructions issue in order, so the release below cannot be issued
            // while a shared-memory load of this stage is still in flight (the arrive by itself does
            // not wait for such loads, and the producer would start overwriting the stage).
#pragma unroll
            for (int j = 0; j < RPT; ++j) asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_u32(&stash[(u * RPT + j) * cthreads + tid])), "f"(v[j]) : "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);
            rows_left -= rows_per_pass;
            if (++stage == p.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        float part[kPassUnroll];
#pragma unroll
        for (int i = 0; i < kPassUnroll; ++i) part[i] = (i < ucount * RPT) ? stash[i * cthreads + tid] : 0.0f;

        // ---- reduce the 8 partials over the lanes of each row segment ---------------------
        // Three exchange steps halve the number of live values (8 -> 4 -> 2 -> 1) while
        // summing over the three highest lane bits of the segment; the remaining lane bits are
        // a plain butterfly.  Afterwards a lane holds the total of pass index `vidx`.
        const int L = p.lanes_per_row;
        int vidx = 0;
        float v1;
        if (L >= 8) {
            const int lr = lane % L;
            float v4[4], v2[2];
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
                v1 = keep + __shfl_xor_sync(0xffffffffu, send, off, 32);
                vidx += up ? 1 : 0;
            }
            for (int off = L >> 4; off > 0; off >>= 1) v1 += __shfl_xor_sync(0xffffffffu, v1, off, 32);
            const bool writer = (lr & ((L >> 3) - 1)) == 0;
            if (writer) red[buf][vidx][rsub * p.wpr + wir] = v1;
        } else {
            // narrow rows (k <= 128): plain butterflies, lane 0 of the segment writes all eight
#pragma unroll
            for (int u = 0; u < kPassUnroll; ++u) {
                float t = part[u];
                for (int off = L >> 1; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
                if ((lane % L) == 0) red[buf][u][rsub * p.wpr + wir] = t;
            }
        }
        // consumer-only barrier (the producer warp is not part of it)
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        for (int t = tid; t < kPassUnroll * p.rpp; t += cthreads) {
            const int i = t / p.rpp, rs = t % p.rpp;  // i = partial index = pass-in-group * RPT + row-of-thread
            const int u = i / RPT, j = i % RPT;
            const int r = (pbase + u) * rows_per_pass + j * p.rpp + rs;
            if (pbase + u < npass && r < nrows) {
                float tot = 0.0f;
                for (int w = 0; w < p.wpr; ++w) tot += red[buf][i][rs * p.wpr + w];
                if (p.epilogue == 1) {
                    // rows come in (gate, up) pairs: the even row's thread writes silu(gate) * up.  The
                    // reference evaluates the sigmoid in double and rounds (unary.go:3353-3365); here it is
                    // expf in f32 (within 2 ulp of that) because this sits on every consumer's critical path.
                    if ((rs & 1) == 0) {
                        float up = 0.0f;
                        for (int w = 0; w < p.wpr; ++w) up += red[buf][i][(rs + 1) * p.wpr + w];
                        p.y[(row_begin + r) >> 1] = tot / (1.0f + expf(-tot)) * up;
                    }
                } else if (p.push_world > 0) {
                    // value and tag travel in one 8-byte store: the receiver polls the data itself, so
                    // nothing but one NVLink hop lies between this store and its use (no fence, no flag)
                    // (one 64-bit element, tag in the high half: single-copy atomic, never seen torn)
                    const unsigned long long v = ((unsigned long long)push_tag << 32) | (unsigned long long)__float_as_uint(tot);
                    for (int pr = 0; pr < p.push_world; ++pr)
                        asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p.push_rx[pr] + p.push_off + row_begin + r), "l"(v) : "memory");
                } else {
                    p.y[row_begin + r] = p.bias ? tot + p.bias[row_begin + r] : tot;
                }
            }
        }
        buf ^= 1;
    }
}

// ---- several activation rows per weight pass (m = 2..8) ------------------------------------
// Same ring, producer and reduction as gemv_stream_kernel; a consumer thread keeps the state of MR
// activation rows in registers, unpacks its two weight blocks once per pass and forms MR dot products
// from them, so the weights cross HBM (and shared memory) once for all rows.  When MR rows of state do
// not cover m, xg groups of warps take the same weight rows against different activation rows
// (group g: rows g*MR .. g*MR+MR-1).  One weight row per thread and pass; no fused prologue / epilogue.
template <class Dec, int MR>
__global__ void __launch_bounds__(384, 1) gemv_stream_mr_kernel(const GemvParams p) {
    constexpr int kWords = Dec::kWords;
    constexpr int kPassGroup = kPassUnroll / MR;  // passes per reduction group (8 partial sums)
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bar_full[kMaxStages];
    __shared__ uint64_t bar_empty[kMaxStages];
    __shared__ float red[2][kPassUnroll][64];  // [buffer][partial][(group * rpp + rsub) * wpr + warp-in-row]

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int cthreads = p.cwarps * 32;
    float *stash = reinterpret_cast<float *>(smem + (size_t)p.stages * p.stage_bytes);  // [8][cthreads] partial sums
    const bool is_producer = warp == p.cwarps;

    int64_t row_begin, row_end;
    if (p.n * (int64_t)gridDim.x < (int64_t)1 << 32) {  // 32-bit divisions where they are exact (see gemv_stream_kernel)
        row_begin = (int64_t)(((uint32_t)p.n * blockIdx.x) / gridDim.x);
        row_end = (int64_t)(((uint32_t)p.n * (blockIdx.x + 1)) / gridDim.x);
    } else {
        row_begin = (p.n * (int64_t)blockIdx.x) / gridDim.x;
        row_end = (p.n * (int64_t)(blockIdx.x + 1)) / gridDim.x;
    }
    const int nrows = (int)(row_end - row_begin);
    const int npass = (nrows + p.rpp - 1) / p.rpp;

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), p.cwarps);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (is_producer) {
        if (lane == 0) {
            const uint64_t policy = make_l2_policy_evict_first();
            int issued = 0;
            for (int ps = 0; ps < npass; ++ps) {
                const int s = ps % p.stages;
                if (ps >= p.stages) {
                    if (!mbar_wait_bounded(smem_u32(&bar_empty[s]), ((ps / p.stages) - 1) & 1)) {
                        atomicExch(p.err, kDevErrEmptyWait);
                        break;
                    }
                }
                const int r0 = ps * p.rpp;
                const int rows = min(p.rpp, nrows - r0);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)p.row_bytes;
                mbar_expect_tx(smem_u32(&bar_full[s]), bytes);
                bulk_g2s_hint(smem_u32(smem + (size_t)s * p.stage_bytes), p.w + (row_begin + r0) * (int64_t)p.row_bytes, bytes,
                              smem_u32(&bar_full[s]), policy);
                issued = ps + 1;
            }
            // never leave with copies in flight into this CTA's shared memory
            const int first = issued > p.stages ? issued - p.stages : 0;
            for (int ps = first; ps < issued; ++ps) {
                if (!mbar_wait_bounded(smem_u32(&bar_full[ps % p.stages]), (ps / p.stages) & 1)) {
                    atomicExch(p.err, kDevErrDrain);
                    break;
                }
            }
        }
        return;
    }

    // ---- consumer warps: warp -> (row group, activation-row group, warp inside the row) ----
    const int rows_per_warp = 32 / p.lanes_per_row;
    const int wir = warp % p.wpr;
    const int xgi = (warp / p.wpr) % p.xg;
    const int rsub = (warp / (p.wpr * p.xg)) * rows_per_warp + lane / p.lanes_per_row;
    const int pair = wir * 32 + (lane % p.lanes_per_row);
    const bool active = pair < p.tpr;

    pdl_wait_prior();  // activations depend on the previous kernel in the stream

    // Activation state of all m rows, built once per CTA into shared memory (four lanes per block).
    uint32_t *area = reinterpret_cast<uint32_t *>(smem + p.coop_off);
    const int nitems = p.nb * 4;
    const int row_words = p.nb * Dec::kStateWordsPerBlock;
    const int total_items = p.m * nitems;
    // Four items per trip with all four loads issued before the first is used: a trip costs one L2 round trip, and
    // 4 rows of k = 4096 take two trips instead of eight.  Uniform trip count: the shuffles inside need whole warps.
    for (int base = 0; base < total_items; base += 4 * cthreads) {
        typename Dec::QRegs q[4];
        int rr[4], it[4];
        bool vd[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = base + u * cthreads + tid;
            vd[u] = idx < total_items;
            rr[u] = vd[u] ? idx / nitems : 0;
            it[u] = vd[u] ? idx - rr[u] * nitems : 0;
            Dec::qload(reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(p.x) + (int64_t)rr[u] * p.x_row_bytes), it[u], vd[u], q[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) Dec::qstage(q[u], it[u], vd[u], area + (size_t)rr[u] * row_words);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
    Dec dec[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) {
        const int xr = xgi * MR + r;
        // rows beyond m and idle lanes: any valid state, their results are never stored
        dec[r].load(area + (size_t)(xr < p.m ? xr : 0) * row_words + (size_t)(active ? pair : 0) * 2 * Dec::kStateWordsPerBlock);
    }

    const uint8_t *my_words = smem + 4 * (rsub * (p.row_bytes >> 2) + pair * kWords);
    const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
    int stage = 0;
    uint32_t phase = 0;
    int rows_left = nrows;
    int buf = 0;
    bool dead = false;
    const int slots = p.rpp * p.xg;  // (group, weight row of the pass) pairs

    for (int pbase = 0; pbase < npass; pbase += kPassGroup) {
        const int ucount = min(kPassGroup, npass - pbase);
#pragma unroll 1
        for (int u = 0; u < ucount; ++u) {
            // a warp whose wait gave up keeps walking the loop so that every consumer reaches the barriers below
            if (!dead && !mbar_wait_bounded(full0 + 8 * stage, phase)) {
                atomicExch(p.err, kDevErrFullWait);
                dead = true;
            }
            float v[MR];
#pragma unroll
            for (int r = 0; r < MR; ++r) v[r] = 0.0f;
            if (!dead && active && rsub < rows_left) {
                typename Dec::WBlk wb;
                Dec::unpack(reinterpret_cast<const uint32_t *>(my_words + stage * p.stage_bytes), wb);
#pragma unroll
                for (int r = 0; r < MR; ++r) v[r] = dec[r].dot(wb);
            }
            // parked BEFORE the stage is released: these stores need every word the pass loaded (an
            // mbarrier arrive by itself does not wait for shared-memory loads still in flight)
#pragma unroll
            for (int r = 0; r < MR; ++r) asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_u32(&stash[(u * MR + r) * cthreads + tid])), "f"(v[r]) : "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);
            rows_left -= p.rpp;
            if (++stage == p.stages) {
                stage = 0;
                phase ^= 1;
            }
        }
        float part[kPassUnroll];
#pragma unroll
        for (int i = 0; i < kPassUnroll; ++i) part[i] = (i < ucount * MR) ? stash[i * cthreads + tid] : 0.0f;

        // reduce the 8 partials over the lanes of each row segment (as in gemv_stream_kernel)
        const int L = p.lanes_per_row;
        const int slot = (xgi * p.rpp + rsub) * p.wpr + wir;
        if (L >= 8) {
            const int lr = lane % L;
            int vidx = 0;
            float v4[4], v2[2], v1;
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
                v1 = keep + __shfl_xor_sync(0xffffffffu, send, off, 32);
                vidx += up ? 1 : 0;
            }
            for (int off = L >> 4; off > 0; off >>= 1) v1 += __shfl_xor_sync(0xffffffffu, v1, off, 32);
            const bool writer = (lr & ((L >> 3) - 1)) == 0;
            if (writer) red[buf][vidx][slot] = v1;
        } else {
#pragma unroll
            for (int u = 0; u < kPassUnroll; ++u) {
                float t = part[u];
                for (int off = L >> 1; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
                if ((lane % L) == 0) red[buf][u][slot] = t;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
        for (int t = tid; t < kPassUnroll * slots; t += cthreads) {
            const int i = t / slots, sl = t - i * slots;   // i = pass-in-group * MR + activation row of the thread
            const int g = sl / p.rpp, rs = sl - g * p.rpp;
            const int u = i / MR, r = i - u * MR;
            const int wrow = (pbase + u) * p.rpp + rs;
            const int xr = g * MR + r;
            if (u < ucount && wrow < nrows && xr < p.m) {
                float tot = 0.0f;
                for (int w = 0; w < p.wpr; ++w) tot += red[buf][i][sl * p.wpr + w];
                p.y[(int64_t)xr * p.ldy + row_begin + wrow] = p.bias ? tot + p.bias[row_begin + wrow] : tot;
            }
        }
        buf ^= 1;
    }
}

// ---- plain kernel ------------------------------------------------------------------------
template <int QT, int ORDER, int M>
__global__ void __launch_bounds__(256) gemv_simple_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                                                        float *__restrict__ y, int64_t n, int nb, int64_t ldx, int64_t ldy) {
    constexpr int BB = (QT == CQ_Q4_0) ? kQ4Bytes : kQ8Bytes;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.0f;
    for (int b = lane; b < nb; b += 32) {
        const uint8_t *blk = w + (row * nb + b) * BB;
        const float d = fp16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
        const float *xb = x + (int64_t)b * kQK;
        if (QT == CQ_Q4_0) {
#pragma unroll 4
            for (int j = 0; j < 16; ++j) {
                const uint32_t q = blk[2 + j];
                const float w0 = d * (float)((int)(q & 0xF) - 8);
                const float w1 = d * (float)((int)(q >> 4) - 8);
                const int e0 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j : j;
                const int e1 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j + 1 : j + 16;
#pragma unroll
                for (int i = 0; i < M; ++i) acc[i] = fmaf(w1, xb[i * ldx + e1], fmaf(w0, xb[i * ldx + e0], acc[i]));
            }
        } else {
#pragma unroll 4
            for (int j = 0; j < kQK; ++j) {
                const float wv = d * (float)(int)(signed char)blk[2 + j];
#pragma unroll
                for (int i = 0; i < M; ++i) acc[i] = fmaf(wv, xb[i * ldx + j], acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < M; ++i) {
        float t = acc[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
        if (lane == 0) y[i * ldy + row] = t;
    }
}

// Q8_1 activations: per-block integer dots scaled in f32, the arithmetic of
// tensor/internal/cuda/kernels/quantized.cu:1919-1941 (Q4_0) and :2058-2073 (Q8_0) with the
// work split of mul_mat_vec_q (quantized.cu:2806-2824): a Q4_0 block is two half-block dots,
// each d4 * (sumi * d8 - 4 * s8); a Q8_0 block is four quarter-block dots d8_0 * d8_1 * sumi.
// One warp per row; lane handles blocks lane, lane+32, ...
template <int QT, int ORDER, int M>
__global__ void __launch_bounds__(256) gemv_q8_1_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ act,
                                                      float *__restrict__ y, int64_t n, int nb, int64_t ldy) {
    constexpr int BB = (QT == CQ_Q4_0) ? kQ4Bytes : kQ8Bytes;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.0f;
    for (int b = lane; b < nb; b += 32) {
        const uint8_t *blk = w + (row * nb + b) * BB;
        const float dw = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
#pragma unroll
        for (int i = 0; i < M; ++i) {
            const uint8_t *ab = act + ((int64_t)i * nb + b) * kQ81Bytes;  // 4-byte aligned: 36 | base
            const float d8 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(ab)));
            const float s8 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(ab + 2)));
            const signed char *q8 = reinterpret_cast<const signed char *>(ab + 4);
            if (QT == CQ_Q4_0) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    int sumi = 0;
#pragma unroll
                    for (int j = 8 * half; j < 8 * half + 8; ++j) {
                        const int q = blk[2 + j];
                        const int e0 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j : j;
                        const int e1 = (ORDER == CQ_ORDER_GO_INTERLEAVED) ? 2 * j + 1 : j + 16;
                        sumi += (q & 0xF) * q8[e0] + (q >> 4) * q8[e1];
                    }
                    acc[i] += __fmul_rn(dw, __fsub_rn(__fmul_rn((float)sumi, d8), __fmul_rn(4.0f, s8)));
                }
            } else {
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    int sumi = 0;
#pragma unroll
                    for (int j = 8 * part; j < 8 * part + 8; ++j) sumi += (int)(signed char)blk[2 + j] * q8[j];
                    acc[i] += __fmul_rn(__fmul_rn(dw, d8), (float)sumi);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < M; ++i) {
        float t = acc[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off, 32);
        if (lane == 0) y[i * ldy + row] = t;
    }
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Chooses the streaming kernel's geometry; returns false when the shape must take the plain
// kernel (row bytes not a multiple of 16, misaligned pointers, k > 32768, no room for 2 stages).
bool plan_stream(const cq_ctx *ctx, int qtype, const void *w, const float *x, int64_t n, int64_t k, GemvParams &p,
                 int &rpt, int &grid, int &threads, size_t &smem) {
    const int bb = cq_is_more_format(qtype) ? cq_more_block_bytes(qtype) : (qtype == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes);
    const int64_t nb = k / kQK;
    if (nb % 8 != 0) return false;  // row bytes % 16 == 0 and an even block count
    if ((reinterpret_cast<uintptr_t>(w) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
    const int tpr = (int)(nb / 2);
    int lanes, wpr;
    if (tpr >= 32) {
        lanes = 32;
        wpr = (tpr + 31) / 32;
    } else {
        if (!is_pow2(tpr)) return false;
        lanes = tpr;
        wpr = 1;
    }
    if (wpr > 15) return false;  // 15 consumer warps + the producer warp = 512 threads
    int target = ctx->tune.target_warps < 1 ? 1 : (ctx->tune.target_warps > 15 ? 15 : ctx->tune.target_warps);
    // In a chain of GEMVs with small kernels in between (a decode step; the caller says so) one CTA of twelve warps per
    // SM beats two of eight (7B-shape step: 1154 -> 1194 tok/s at 16 layers), while GEMVs back to back prefer the latter
    // (74 MB shape: 15.1 against 16.7 us).  An explicit gemv_warps setting wins.
    if (ctx->tune.gemv_chain && ctx->tune.target_warps == 8) target = 12;
    int row_groups = (target + wpr - 1) / wpr;  // warp groups, each covering 32/lanes rows
    if (row_groups < 1) row_groups = 1;
    while (row_groups > 1 && row_groups * wpr > 15) --row_groups;
    int cwarps = row_groups * wpr;
    int rpp = row_groups * (32 / lanes);
    if (rpp * wpr > 64) {  // reduction scratch holds 64 entries per pass
        rpp = 64 / wpr;
        row_groups = rpp / (32 / lanes);
        if (row_groups < 1) return false;
        cwarps = row_groups * wpr;
        rpp = row_groups * (32 / lanes);
    }
    const int64_t row_bytes = nb * bb;
    rpt = ctx->tune.gemv_rpt == 2 ? 2 : 1;
    const int64_t stage_bytes = (int64_t)rpp * rpt * row_bytes;
    threads = (cwarps + 1) * 32;
    const size_t stash_bytes = (size_t)kPassUnroll * cwarps * 32 * sizeof(float);
    // Small geometries share the SM with the next kernel of the stream: half the shared memory each.
    const bool two_per_sm = threads <= 288;
    const size_t per_cta = two_per_sm ? (ctx->smem_optin + 1024) / 2 - 1024 : ctx->smem_optin;  // 1 KB is reserved per CTA
    // Cooperative activation slicing pays off when several row groups share the CTA; its staging
    // area holds 10 words per block and slice (sized for three slices).
    size_t coop_bytes = (size_t)nb * 3 * 10 * sizeof(uint32_t);
    if (rpp <= 1 || coop_bytes > 49152 || ctx->tune.gemv_coop == 0) coop_bytes = 0;
    // the activations a fused prologue produces (nothing when only the epilogue is fused)
    const bool prologue = ctx->fuse.on && (ctx->fuse.delta || ctx->fuse.alpha || ctx->fuse.x_out);
    const size_t xs_bytes = prologue ? (size_t)k * sizeof(float) : 0;
    const size_t budget = per_cta > kStaticSmemReserve + stash_bytes + coop_bytes + xs_bytes ? per_cta - kStaticSmemReserve - stash_bytes - coop_bytes - xs_bytes : 0;
    // A prologue that would crowd the ring out of a half-SM launch is refused (the caller then runs
    // the norm as its own kernel): one CTA per SM costs a large GEMV more than the fusion saves.
    int stages = ctx->tune.stages < 2 ? 2 : (ctx->tune.stages > kMaxStages ? kMaxStages : ctx->tune.stages);
    if ((size_t)stage_bytes * 2 > budget) return false;
    while ((size_t)stage_bytes * stages > budget) --stages;
    p.early = ctx->tune.early;
    p.independent = (ctx->tune.gemv_independent && !ctx->fuse.on && ctx->push.world == 0) ? 1 : 0;
    p.n = n;
    p.nb = (int)nb;
    p.row_bytes = (int)row_bytes;
    p.tpr = tpr;
    p.lanes_per_row = lanes;
    p.wpr = wpr;
    p.rpp = rpp;
    p.cwarps = cwarps;
    p.stages = stages;
    p.stage_bytes = (int)stage_bytes;
    smem = (size_t)stage_bytes * stages + stash_bytes + coop_bytes + xs_bytes;
    p.coop_off = coop_bytes ? (int)((size_t)stage_bytes * stages + stash_bytes) : -1;
    p.xs_off = xs_bytes ? (int)((size_t)stage_bytes * stages + stash_bytes + coop_bytes) : -1;
    if (ctx->fuse.on && ctx->fuse.epilogue == 1 && ((rpp & 1) != 0 || (n & 1) != 0)) return false;  // pairs must share a pass
    const int64_t max_ctas = (n + rpp * rpt - 1) / (rpp * rpt);
    // 0 = automatic: geometries that fit two CTAs per SM use both slots (more warps in flight).
    // (One CTA per SM is faster when the SAME small shape runs back to back -- the next launch
    // becomes resident at once and prefetches during this one -- but slower in a real decode
    // step, where small kernels sit between the GEMVs: 59 vs 56 us per 7B-shape layer.)
    const int per_sm = ctx->tune.ctas_per_sm > 0 ? ctx->tune.ctas_per_sm : (two_per_sm ? 2 : 1);
    int64_t g = (int64_t)ctx->sm_count * per_sm;
    if (g > max_ctas) g = max_ctas;
    grid = (int)g;
    return true;
}

// Geometry of the multi-row kernel for `m` activation rows with `mr` rows of state per thread; false when
// the shape does not fit (then the caller falls back to one launch per row or per smaller group).
bool plan_stream_mr(const cq_ctx *ctx, int qtype, const void *w, const void *x, int64_t n, int64_t k, int m, int mr, int state_words,
                    GemvParams &p, int &grid, int &threads, size_t &smem) {
    const int bb = qtype == CQ_Q4_0 ? kQ4Bytes : kQ8Bytes;
    const int64_t nb = k / kQK;
    if (nb % 8 != 0 || k > 32768) return false;
    if ((reinterpret_cast<uintptr_t>(w) & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return false;
    const int tpr = (int)(nb / 2);
    int lanes, wpr;
    if (tpr >= 32) {
        lanes = 32;
        wpr = (tpr + 31) / 32;
    } else {
        if (!is_pow2(tpr)) return false;
        lanes = tpr;
        wpr = 1;
    }
    const int xg = (m + mr - 1) / mr;
    constexpr int kMaxCWarps = 11;  // 11 consumer warps + the producer = 384 threads: 168 registers each
    if (wpr * xg > kMaxCWarps) return false;
    int row_groups = kMaxCWarps / (wpr * xg);
    const int rows_per_warp = 32 / lanes;
    while (row_groups > 1 && row_groups * rows_per_warp * xg * wpr > 64) --row_groups;  // reduction scratch: 64 slots per partial
    if (row_groups * rows_per_warp * xg * wpr > 64) return false;
    const int cwarps = row_groups * xg * wpr;
    const int rpp = row_groups * rows_per_warp;
    const int64_t row_bytes = nb * bb;
    const int64_t stage_bytes = (int64_t)rpp * row_bytes;
    threads = (cwarps + 1) * 32;
    const size_t stash_bytes = (size_t)kPassUnroll * cwarps * 32 * sizeof(float);
    const size_t coop_bytes = (size_t)m * nb * state_words * sizeof(uint32_t);
    const size_t fixed = kStaticSmemReserve + stash_bytes + coop_bytes;
    if (ctx->smem_optin < fixed + 2 * (size_t)stage_bytes) return false;
    const size_t budget = ctx->smem_optin - fixed;
    int stages = 8;
    while ((size_t)stage_bytes * stages > budget) --stages;
    p.n = n;
    p.nb = (int)nb;
    p.row_bytes = (int)row_bytes;
    p.tpr = tpr;
    p.lanes_per_row = lanes;
    p.wpr = wpr;
    p.rpp = rpp;
    p.cwarps = cwarps;
    p.stages = stages;
    p.stage_bytes = (int)stage_bytes;
    p.coop_off = (int)((size_t)stage_bytes * stages + stash_bytes);
    p.xs_off = -1;
    p.m = m;
    p.xg = xg;
    smem = (size_t)stage_bytes * stages + stash_bytes + coop_bytes;
    const int64_t max_ctas = (n + rpp - 1) / rpp;
    grid = (int)(max_ctas < ctx->sm_count ? max_ctas : ctx->sm_count);
    return true;
}

template <class Dec, int MR>
cq_status run_stream_mr(cq_ctx *ctx, const GemvParams &p, int grid, int threads, size_t smem) {
    static thread_local int configured_device = -1;
    auto kern = gemv_stream_mr_kernel<Dec, MR>;
    if (configured_device != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - kStaticSmemReserve)));
        configured_device = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return CQ_OK;
}

// m (2..8) rows in as few weight passes as the register budget allows.  `x` is f32 rows (Q16 state, at
// most 4 rows of state per thread, two warp groups for 5..8 rows when the row is short enough) or rows of
// Q8_1 blocks (Q81 state, up to 8 rows per thread).  Returns how many leading rows were launched (0 when
// the shape does not fit; a single left-over row is left to the one-row kernel).
// DECK: 0 = f32 rows, Q16 state; 1 = rows of Q8_1 blocks; 2 = f32 rows quantized to Q8_1 in the set-up (two rows a pass only).
template <int QT, int ORDER, int DECK>
int64_t try_stream_mr(cq_ctx *ctx, const void *x, int64_t x_row_bytes, int64_t m, int64_t k, const uint8_t *w, int64_t n, float *y, int64_t ldy,
                      cq_status &s) {
    constexpr bool Q81 = DECK == 1;
    using Dec = typename std::conditional<DECK == 2, DecQ81F<QT, ORDER>, typename std::conditional<DECK == 1, DecQ81<QT, ORDER>, DecQ16<QT, ORDER>>::type>::type;
    s = CQ_OK;
    if (ctx->tune.force_simple || ctx->tune.gemv_multirow == 0 || m < 2 || m > 8 || (x_row_bytes & 15) != 0) return 0;
    int64_t r0 = 0;
    while (m - r0 >= 2) {
        GemvParams p{};
        int grid = 0, threads = 0;
        size_t smem = 0;
        const uint8_t *xr = static_cast<const uint8_t *>(x) + r0 * x_row_bytes;
        int rows = (int)(m - r0);
        if (DECK == 2 && rows > 2) rows = 2;
        const int mr = Q81 ? (rows <= 2 ? 2 : (rows <= 4 ? 4 : 8)) : (rows <= 2 ? 2 : 4);
        bool ok = plan_stream_mr(ctx, QT, w, xr, n, k, rows, mr, Dec::kStateWordsPerBlock, p, grid, threads, smem);
        if (!ok && rows > mr) {  // not enough warps for two activation-row groups: mr rows now, the rest in another pass
            rows = mr;
            ok = plan_stream_mr(ctx, QT, w, xr, n, k, rows, mr, Dec::kStateWordsPerBlock, p, grid, threads, smem);
        }
        if (!ok) break;
        p.w = w;
        p.x = reinterpret_cast<const float *>(xr);
        p.x_row_bytes = x_row_bytes;
        p.y = y + r0 * ldy;
        p.ldy = ldy;
        p.err = ctx->dev_err_devptr;
        p.bias = ctx->bias;
        if (mr == 2 || DECK == 2) s = run_stream_mr<Dec, 2>(ctx, p, grid, threads, smem);
        else if (mr == 4) s = run_stream_mr<Dec, DECK == 2 ? 2 : 4>(ctx, p, grid, threads, smem);
        else s = run_stream_mr<Dec, DECK == 2 ? 2 : (Q81 ? 8 : 4)>(ctx, p, grid, threads, smem);
        if (s != CQ_OK) return r0 + rows;
        r0 += rows;
    }
    return r0;
}

template <class Dec, int RPT, int MAXT, int MINB>
cq_status run_stream_b(cq_ctx *ctx, GemvParams p, int grid, int threads, size_t smem) {
    static thread_local int configured_device = -1;
    auto kern = gemv_stream_kernel<Dec, RPT, MAXT, MINB>;
    if (configured_device != ctx->device) {
        CQ_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - kStaticSmemReserve)));
        configured_device = ctx->device;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    CQ_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return CQ_OK;
}

template <class Dec>
cq_status run_stream(cq_ctx *ctx, GemvParams p, int rpt, int grid, int threads, size_t smem) {
    if (rpt == 2) {
        if (threads <= 288) return run_stream_b<Dec, 2, 288, 2>(ctx, p, grid, threads, smem);
        return run_stream_b<Dec, 2, 512, 1>(ctx, p, grid, threads, smem);
    }
    if (threads <= 288) return run_stream_b<Dec, 1, 288, 2>(ctx, p, grid, threads, smem);
    return run_stream_b<Dec, 1, 512, 1>(ctx, p, grid, threads, smem);
}

template <int QT, int ORDER>
cq_status run_simple(cq_ctx *ctx, const uint8_t *w, const float *x, float *y, int64_t m, int64_t n, int nb, int64_t ldx,
                     int64_t ldy) {
    const int threads = 256, rows_per_cta = threads / 32;
    const unsigned grid = (unsigned)((n + rows_per_cta - 1) / rows_per_cta);
    switch (m) {
#define CQ_CASE(MM)                                                                                            \
    case MM:                                                                                                   \
        gemv_simple_kernel<QT, ORDER, MM><<<grid, threads, 0, ctx->stream>>>(w, x, y, n, nb, ldx, ldy);        \
        break;
        CQ_CASE(1) CQ_CASE(2) CQ_CASE(3) CQ_CASE(4) CQ_CASE(5) CQ_CASE(6) CQ_CASE(7) CQ_CASE(8)
#undef CQ_CASE
        default: return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemv: m must be 1..8");
    }
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

template <int QT, int ORDER>
cq_status run_q8_1(cq_ctx *ctx, const uint8_t *w, const uint8_t *act, float *y, int64_t m, int64_t n, int nb, int64_t ldy) {
    const int threads = 256, rows_per_cta = threads / 32;
    const unsigned grid = (unsigned)((n + rows_per_cta - 1) / rows_per_cta);
    switch (m) {
#define CQ_CASE(MM)                                                                                      \
    case MM:                                                                                             \
        gemv_q8_1_kernel<QT, ORDER, MM><<<grid, threads, 0, ctx->stream>>>(w, act, y, n, nb, ldy);       \
        break;
        CQ_CASE(1) CQ_CASE(2) CQ_CASE(3) CQ_CASE(4) CQ_CASE(5) CQ_CASE(6) CQ_CASE(7) CQ_CASE(8)
#undef CQ_CASE
        default: return cq_fail(ctx, CQ_ERR_INVALID_ARG, "gemv: m must be 1..8");
    }
    CQ_CUDA(ctx, cudaGetLastError());
    return CQ_OK;
}

// The Q8_1-activation GEMV on m rows of already quantized activation blocks (36 bytes each, 16-byte aligned
// base): the streaming kernel with the Q8_1 decoder when the shape fits it (one weight pass for all rows),
// else the plain one-warp-per-row kernel.  Allocates nothing.
template <int QT, int ORDER>
cq_status q8_1_on_blocks(cq_ctx *ctx, const void *act_blocks, int64_t m, int64_t k, const uint8_t *w, int64_t n, float *y, int64_t ldy) {
    const int nb = (int)(k / kQK);
    GemvParams p{};
    int rpt = 1, grid = 0, threads = 0;
    size_t smem = 0;
    if (!ctx->tune.force_simple && ctx->push.world == 0 && !ctx->fuse.on &&
        plan_stream(ctx, QT, w, static_cast<const float *>(act_blocks), n, k, p, rpt, grid, threads, smem) && p.coop_off >= 0) {
        p.w = w;
        p.err = ctx->dev_err_devptr;
        p.bias = ctx->bias;
        ctx->bias_done = true;
        cq_status s = CQ_OK;
        const int64_t done = try_stream_mr<QT, ORDER, 1>(ctx, act_blocks, (int64_t)nb * kQ81Bytes, m, k, w, n, y, ldy, s);
        if (s != CQ_OK) return s;
        for (int64_t i = done; i < m; ++i) {
            p.x = reinterpret_cast<const float *>(static_cast<const uint8_t *>(act_blocks) + (size_t)i * nb * kQ81Bytes);
            p.y = y + i * ldy;
            s = run_stream<DecQ81<QT, ORDER>>(ctx, p, rpt, grid, threads, smem);
            if (s != CQ_OK) return s;
        }
        return CQ_OK;
    }
    return run_q8_1<QT, ORDER>(ctx, w, static_cast<const uint8_t *>(act_blocks), y, m, n, nb, ldy);
}

template <int QT, int ORDER>
cq_status gemv_dispatch(cq_ctx *ctx, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx, const uint8_t *w,
                        int64_t n, float *y, int64_t ldy) {
    const int nb = (int)(k / kQK);
    if (actmode == CQ_ACT_Q8_1) {
        // One or two rows: the activations are quantized inside the GEMV's set-up, no launch of their own.
        if (m <= 2 && ctx->tune.gemv_q81_inline && !ctx->tune.force_simple && ctx->push.world == 0 && !ctx->fuse.on && ldx % 4 == 0 &&
            (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            GemvParams p{};
            int rpt = 1, grid = 0, threads = 0;
            size_t smem = 0;
            if (plan_stream(ctx, QT, w, x, n, k, p, rpt, grid, threads, smem) && p.coop_off >= 0) {
                p.w = w;
                p.err = ctx->dev_err_devptr;
                p.bias = ctx->bias;
                ctx->bias_done = true;
                cq_status s = CQ_OK;
                const int64_t done = try_stream_mr<QT, ORDER, 2>(ctx, x, ldx * (int64_t)sizeof(float), m, k, w, n, y, ldy, s);
                if (s != CQ_OK) return s;
                for (int64_t i = done; i < m; ++i) {
                    p.x = x + i * ldx;
                    p.y = y + i * ldy;
                    s = run_stream<DecQ81F<QT, ORDER>>(ctx, p, rpt, grid, threads, smem);
                    if (s != CQ_OK) return s;
                }
                return CQ_OK;
            }
        }
        const size_t bytes = (size_t)m * nb * kQ81Bytes;
        cq_status s = cq_reserve_scratch(ctx, bytes);
        if (s != CQ_OK) return s;
        s = launch_quantize_q8_1(ctx, x, m, k, ldx, ctx->scratch);
        if (s != CQ_OK) return s;
        return q8_1_on_blocks<QT, ORDER>(ctx, ctx->scratch, m, k, w, n, y, ldy);
    }
    GemvParams p{};
    int rpt = 1, grid = 0, threads = 0;
    size_t smem = 0;
    if (!ctx->tune.force_simple && plan_stream(ctx, QT, w, x, n, k, p, rpt, grid, threads, smem) && (ldx % 4 == 0)) {
        p.w = w;
        p.err = ctx->dev_err_devptr;
        p.bias = (ctx->push.world == 0 && !(ctx->fuse.on && ctx->fuse.epilogue == 1)) ? ctx->bias : nullptr;
        ctx->bias_done = p.bias != nullptr;
        p.push_world = ctx->push.world;
        p.push_rx = ctx->push.rx;
        p.push_seq = ctx->push.seq;
        const FuseSpec &f = ctx->fuse;
        p.norm = f.on && f.norm ? 1 : 0;
        p.eps = f.eps;
        p.epilogue = f.on ? f.epilogue : 0;
        int64_t done = 0;
        if (!f.on && ctx->push.world == 0 && ctx->tune.gemv_variant == 0) {  // two or more plain rows: one weight pass for up to 4 (8) of them
            cq_status s = CQ_OK;
            done = try_stream_mr<QT, ORDER, 0>(ctx, x, ldx * (int64_t)sizeof(float), m, k, w, n, y, ldy, s);
            if (s != CQ_OK) return s;
        }
        for (int64_t i = done; i < m; ++i) {  // one pass over the weights per remaining activation row
            p.x = x + i * ldx;
            p.y = y + i * ldy;
            p.delta = f.on && f.delta ? f.delta + i * f.ld_delta : nullptr;
            p.alpha = f.on ? f.alpha : nullptr;
            p.x_out = f.on && f.x_out ? f.x_out + i * f.ld_xout : nullptr;
            p.push_off = i * ctx->push.row_stride;
            cq_status s;
            switch (ctx->tune.gemv_variant) {
                case 1: s = run_stream<DecFma<QT, ORDER>>(ctx, p, rpt, grid, threads, smem); break;
                case 3: s = run_stream<DecSlices<QT, ORDER, 3>>(ctx, p, rpt, grid, threads, smem); break;
                case 2: s = run_stream<DecSlices<QT, ORDER, 2>>(ctx, p, rpt, grid, threads, smem); break;
                default: s = run_stream<DecQ16<QT, ORDER>>(ctx, p, rpt, grid, threads, smem); break;
            }
            if (s != CQ_OK) return s;
        }
        return CQ_OK;
    }
    if (ctx->push.world > 0) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "pushing GEMV needs a shape the streaming kernel takes (k % 256 == 0, aligned pointers)");
    if (ctx->fuse.on) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "fused linear needs a shape the streaming kernel takes (k % 256 == 0, aligned pointers, an even row-group count for the pairing epilogue)");
    return run_simple<QT, ORDER>(ctx, w, x, y, m, n, nb, ldx, ldy);
}

}  // namespace

// Q4_1 / Q5_0 / Q5_1 on the streaming kernel; false when the shape must take the plain kernel.
template <int QT, int ORDER>
bool try_stream_more(cq_ctx *ctx, const float *x, int64_t m, int64_t k, int64_t ldx, const void *w, int64_t n, float *y, int64_t ldy, cq_status &s) {
    GemvParams p{};
    int rpt = 1, grid = 0, threads = 0;
    size_t smem = 0;
    if (ctx->tune.force_simple || (ldx % 4) != 0 || !plan_stream(ctx, QT, w, x, n, k, p, rpt, grid, threads, smem)) return false;
    p.w = static_cast<const uint8_t *>(w);
    p.err = ctx->dev_err_devptr;
    s = CQ_OK;
    for (int64_t i = 0; i < m && s == CQ_OK; ++i) {
        p.x = x + i * ldx;
        p.y = y + i * ldy;
        s = run_stream<DecMore<QT, ORDER>>(ctx, p, rpt, grid, threads, smem);
    }
    return true;
}

cq_status launch_gemv(cq_ctx *ctx, int qtype, int order, int actmode, const float *x, int64_t m, int64_t k, int64_t ldx,
                      const void *w, int64_t n, float *y, int64_t ldy) {
    if (cq_is_k_format(qtype)) {
        if (ctx->fuse.on || ctx->push.world != 0) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "fused and multi-GPU GEMVs take Q4_0 / Q8_0 only");
        return launch_gemv_k(ctx, qtype, actmode, x, m, k, ldx, w, n, y, ldy);
    }
    if (cq_is_more_format(qtype)) {
        if (ctx->fuse.on || ctx->push.world != 0) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "fused and multi-GPU GEMVs take Q4_0 / Q8_0 only");
        if (actmode == CQ_ACT_F32) {
            cq_status s = CQ_OK;
            bool taken;
            if (qtype == CQ_Q4_1 && order == CQ_ORDER_GO_INTERLEAVED) taken = try_stream_more<CQ_Q4_1, 0>(ctx, x, m, k, ldx, w, n, y, ldy, s);
            else if (qtype == CQ_Q4_1) taken = try_stream_more<CQ_Q4_1, 1>(ctx, x, m, k, ldx, w, n, y, ldy, s);
            else if (qtype == CQ_Q5_0) taken = try_stream_more<CQ_Q5_0, 1>(ctx, x, m, k, ldx, w, n, y, ldy, s);
            else taken = try_stream_more<CQ_Q5_1, 1>(ctx, x, m, k, ldx, w, n, y, ldy, s);
            if (taken) return s;
        }
        return launch_gemv_more(ctx, qtype, order, actmode, x, m, k, ldx, w, n, y, ldy);
    }
    if ((reinterpret_cast<uintptr_t>(w) & 1) != 0) return cq_fail(ctx, CQ_ERR_INVALID_ARG, "weight blocks must be 2-byte aligned");
    if ((reinterpret_cast<uintptr_t>(x) & 3) != 0 || (reinterpret_cast<uintptr_t>(y) & 3) != 0)
        return cq_fail(ctx, CQ_ERR_INVALID_ARG, "x and y must be 4-byte aligned");
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    if (qtype == CQ_Q4_0 && order == CQ_ORDER_GO_INTERLEAVED)
        return gemv_dispatch<CQ_Q4_0, 0>(ctx, actmode, x, m, k, ldx, wb, n, y, ldy);
    if (qtype == CQ_Q4_0) return gemv_dispatch<CQ_Q4_0, 1>(ctx, actmode, x, m, k, ldx, wb, n, y, ldy);
    return gemv_dispatch<CQ_Q8_0, 0>(ctx, actmode, x, m, k, ldx, wb, n, y, ldy);
}

// The Q8_1-activation GEMV on activation blocks the caller has already quantized (36-byte blocks, m rows of
// k/32, base 16-byte aligned for the streaming route).  The same routes as cq_qmatmul's CQ_ACT_Q8_1 mode; nothing is allocated.
cq_status launch_gemv_q8_1_blocks(cq_ctx *ctx, int qtype, int order, const void *act_blocks, int64_t m, int64_t k,
                                  const void *w, int64_t n, float *y, int64_t ldy) {
    if (cq_is_more_format(qtype)) return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "Q8_1 activations take Q4_0 / Q8_0 weights only");
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    if (qtype == CQ_Q4_0 && order == CQ_ORDER_GO_INTERLEAVED) return q8_1_on_blocks<CQ_Q4_0, 0>(ctx, act_blocks, m, k, wb, n, y, ldy);
    if (qtype == CQ_Q4_0) return q8_1_on_blocks<CQ_Q4_0, 1>(ctx, act_blocks, m, k, wb, n, y, ldy);
    return q8_1_on_blocks<CQ_Q8_0, 0>(ctx, act_blocks, m, k, wb, n, y, ldy);
}
