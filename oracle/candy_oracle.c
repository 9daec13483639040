/*
 * candy_oracle.c -- CPU restatement of gocnn/candy's block-quantized matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared
 * against; nothing in the shipped library links, imports or calls it.  It may be used
 * from tests, from the smoke check and from the CPU-baseline leg of the benchmark.
 *
 * PARITY UNPINNED: the reference ships no test, fixture or golden vector for any of
 * the functions restated here, and its Go sources cannot be compiled in this build
 * environment (no Go toolchain).  The restatement is pinned only by (1) hand-derived
 * known answers, (2) an independent NumPy twin that must agree bit for bit, (3) a
 * third-party GGUF codec for the split-order block formats, and (4) the reference's own
 * CUDA kernels run on a GPU for the split-order dequantizers, the Q8_1 quantizer and
 * the integer dot products.
 *
 * Every function cites the reference file:line (paths relative to the gocnn/candy
 * checkout) whose arithmetic it follows.  Build with
 *     gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * so that every f32 multiply and add rounds separately, as the Go compiler emits on
 * amd64 (Go only fuses multiply-add on arm64/ppc64/s390x/riscv64).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CO_QK 32
#define CO_Q4_0_BYTES 18
#define CO_Q8_0_BYTES 34
#define CO_Q8_1_BYTES 36

/* element order of the 32 values inside a Q4_0 block */
#define CO_ORDER_GO_INTERLEAVED 0 /* tensor/internal/cpu/kernels/quantized.go:87-92 */
#define CO_ORDER_GGML_SPLIT 1     /* tensor/internal/cuda/kernels/quantized.cu:862-866 */

static float bits_to_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static uint32_t f32_to_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

/* tensor/internal/cpu/kernels/quantized.go:149-173 (fp16ToFloat32).
 * Inf/NaN keep the mantissa payload shifted left by 13 (a signalling NaN is not
 * quieted); subnormals are normalised with the same shift loop. */
uint32_t co_fp16_to_f32_bits(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (uint32_t)(h & 0x7C00u);
    uint32_t mant = (uint32_t)(h & 0x03FFu);
    if (exp == 0x7C00u) return sign | 0x7F800000u | (mant << 13);
    if (exp == 0) {
        if (mant == 0) return sign;
        exp = (127u - 14u) << 23;
        while ((mant & 0x400u) == 0) {
            mant <<= 1;
            exp -= 1u << 23;
        }
        mant &= 0x3FFu;
        return sign | exp | (mant << 13);
    }
    return sign | ((((exp >> 10) - 15u + 127u) << 23)) | (mant << 13);
}

float co_fp16_to_f32(uint16_t h) { return bits_to_f32(co_fp16_to_f32_bits(h)); }

/* f32 -> binary16, IEEE round-to-nearest-even.  This is the conversion performed by
 * the assignment `dst.d = d` (float -> half) in the reference's weight quantizers
 * (tensor/internal/metal/kernels/quantized.metal:4132 and :4198) and by the half
 * stores of the Q8_1 quantizer (tensor/internal/cuda/kernels/quantized.cu:3556-3557).
 * The Go side of the reference has no f32 -> f16 encoder at all. */
uint16_t co_f32_to_fp16(float f) {
    uint32_t x = f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((absx >> 13) & 0x3FFu)); /* NaN */
    if (absx >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536 -> inf (also inf) */
    if (absx >= 0x38800000u) {                                  /* normal half range */
        uint32_t mant = absx & 0x7FFFFFu;
        uint32_t e = (absx >> 23) - 112u; /* rebias 127 -> 15 */
        uint32_t hbits = (e << 10) | (mant >> 13);
        uint32_t rem = mant & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (hbits & 1u))) hbits++; /* may carry into inf */
        return (uint16_t)(sign | hbits);
    }
    if (absx < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to zero */
    /* subnormal half: value = m * 2^-24, m in [0,1024] */
    {
        uint32_t e = absx >> 23;                        /* 102..112 */
        uint32_t mant = (absx & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
        uint32_t shift = 126u - e;                      /* 14..24 */
        uint32_t hbits = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hbits & 1u))) hbits++;
        return (uint16_t)(sign | hbits);
    }
}

static uint16_t load_u16(const uint8_t *p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }
static void store_u16(uint8_t *p, uint16_t v) {
    p[0] = (uint8_t)(v & 0xFF);
    p[1] = (uint8_t)(v >> 8);
}

/* Q4_0 block (18 bytes: f16 scale, 16 bytes of nibbles) -> 32 f32.
 * order 0: tensor/internal/cpu/kernels/quantized.go:85-93  (y[2j]=lo, y[2j+1]=hi).
 * order 1: tensor/internal/cuda/kernels/quantized.cu:838-867 (y[j]=lo, y[j+16]=hi;
 *          the CUDA form d*q + (-8d) and the Go form d*(q-8) are both exact in f32
 *          and therefore equal, so one expression serves both). */
void co_dequantize_q4_0(const uint8_t *blocks, int64_t nblocks, int order, float *y) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t *blk = blocks + b * CO_Q4_0_BYTES;
        float d = co_fp16_to_f32(load_u16(blk));
        const uint8_t *qs = blk + 2;
        float *yb = y + b * CO_QK;
        for (int j = 0; j < 16; ++j) {
            int q1 = qs[j] & 0xF;
            int q2 = qs[j] >> 4;
            float v1 = d * ((float)q1 - 8.0f);
            float v2 = d * ((float)q2 - 8.0f);
            if (order == CO_ORDER_GO_INTERLEAVED) {
                yb[2 * j] = v1;
                yb[2 * j + 1] = v2;
            } else {
                yb[j] = v1;
                yb[j + 16] = v2;
            }
        }
    }
}

/* Q8_0 block (34 bytes) -> 32 f32: tensor/internal/cpu/kernels/quantized.go:131-136. */
void co_dequantize_q8_0(const uint8_t *blocks, int64_t nblocks, float *y) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t *blk = blocks + b * CO_Q8_0_BYTES;
        float d = co_fp16_to_f32(load_u16(blk));
        const int8_t *qs = (const int8_t *)(blk + 2);
        for (int i = 0; i < CO_QK; ++i) y[b * CO_QK + i] = d * (float)qs[i];
    }
}

/* f32 -> Q4_0, tensor/internal/metal/kernels/quantized.metal:4187-4211
 * (kernel_cpy_f32_q4_0): the first element with the largest |v| gives `max` with its
 * sign; d = max / -8; id = d ? 1/d : 0 from the unrounded f32 d; q = min(15,
 * (int8)(v*id + 8.5)) with a truncating cast.  The shader packs in split order
 * (qs[j] = q(v[j]) | q(v[j+16]) << 4); `order` selects which element goes to which
 * nibble so that the matching dequantizer returns the values in their source order. */
void co_quantize_q4_0(const float *w, int64_t nblocks, int order, uint8_t *blocks) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const float *src = w + b * CO_QK;
        uint8_t *blk = blocks + b * CO_Q4_0_BYTES;
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < CO_QK; ++j) {
            float v = src[j];
            if (amax < fabsf(v)) {
                amax = fabsf(v);
                max = v;
            }
        }
        float d = max / -8.0f;
        float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        store_u16(blk, co_f32_to_fp16(d));
        for (int j = 0; j < 16; ++j) {
            int i0 = (order == CO_ORDER_GO_INTERLEAVED) ? 2 * j : j;
            int i1 = (order == CO_ORDER_GO_INTERLEAVED) ? 2 * j + 1 : j + 16;
            float x0 = src[i0] * id;
            float x1 = src[i1] * id;
            int q0 = (int)(int8_t)(x0 + 8.5f);
            int q1 = (int)(int8_t)(x1 + 8.5f);
            uint8_t xi0 = (uint8_t)(q0 < 15 ? q0 : 15);
            uint8_t xi1 = (uint8_t)(q1 < 15 ? q1 : 15);
            blk[2 + j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}

/* f32 -> Q8_0, tensor/internal/metal/kernels/quantized.metal:4129-4145
 * (kernel_cpy_f32_q8_0): d = amax/127; id = d ? 1/d : 0; q = round(v*id), ties away
 * from zero. */
void co_quantize_q8_0(const float *w, int64_t nblocks, uint8_t *blocks) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const float *src = w + b * CO_QK;
        uint8_t *blk = blocks + b * CO_Q8_0_BYTES;
        float amax = 0.0f;
        for (int j = 0; j < CO_QK; ++j) {
            float a = fabsf(src[j]);
            amax = amax > a ? amax : a;
        }
        float d = amax / 127.0f;
        float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        store_u16(blk, co_f32_to_fp16(d));
        for (int j = 0; j < CO_QK; ++j) {
            float x0 = src[j] * id;
            blk[2 + j] = (uint8_t)(int8_t)roundf(x0);
        }
    }
}

/* ---- Q4_1 / Q5_0 / Q5_1: the other 32-value formats of the reference's registry ------------
 * Block layouts: tensor/internal/cpu/kernels/quantized.go:13-31.  qtype ids follow GGML:
 * 3 = Q4_1 (20 bytes), 6 = Q5_0 (22 bytes), 7 = Q5_1 (24 bytes). */
#define CO_Q4_1_BYTES 20
#define CO_Q5_0_BYTES 22
#define CO_Q5_1_BYTES 24

static int64_t co_block_bytes(int qtype) {
    switch (qtype) {
    case 2: return CO_Q4_0_BYTES;
    case 3: return CO_Q4_1_BYTES;
    case 6: return CO_Q5_0_BYTES;
    case 7: return CO_Q5_1_BYTES;
    case 8: return CO_Q8_0_BYTES;
    default: return 0;
    }
}

/* Q4_1 -> f32.  order 0: tensor/internal/cpu/kernels/quantized.go:107-116 (y[2j] = d*lo + m,
 * y[2j+1] = d*hi + m).  order 1: tensor/internal/cuda/kernels/quantized.cu:728-747 with the
 * element placement of dequantize_block (y[j], y[j+16]).  d*q is exact, "+ m" rounds once. */
void co_dequantize_q4_1(const uint8_t *blocks, int64_t nblocks, int order, float *y) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t *blk = blocks + b * CO_Q4_1_BYTES;
        float d = co_fp16_to_f32(load_u16(blk));
        float m = co_fp16_to_f32(load_u16(blk + 2));
        const uint8_t *qs = blk + 4;
        float *yb = y + b * CO_QK;
        for (int j = 0; j < 16; ++j) {
            float t1 = d * (float)(qs[j] & 0xF);
            float t2 = d * (float)(qs[j] >> 4);
            float v1 = t1 + m, v2 = t2 + m;
            if (order == CO_ORDER_GO_INTERLEAVED) {
                yb[2 * j] = v1;
                yb[2 * j + 1] = v2;
            } else {
                yb[j] = v1;
                yb[j + 16] = v2;
            }
        }
    }
}

/* Q5_0 / Q5_1 -> f32, tensor/internal/cuda/kernels/quantized.cu:749-771 and :773-795: value j
 * is the low nibble of qs[j] with bit j of qh as its fifth bit, value j+16 the high nibble
 * with bit j+16.  Q5_0: (q - 16) * d;  Q5_1: q * d + m. */
void co_dequantize_q5(int qtype, const uint8_t *blocks, int64_t nblocks, float *y) {
    const int with_min = qtype == 7;
    const int64_t bb = with_min ? CO_Q5_1_BYTES : CO_Q5_0_BYTES;
    for (int64_t b = 0; b < nblocks; ++b) {
        const uint8_t *blk = blocks + b * bb;
        float d = co_fp16_to_f32(load_u16(blk));
        float m = with_min ? co_fp16_to_f32(load_u16(blk + 2)) : 0.0f;
        const uint8_t *qhp = blk + (with_min ? 4 : 2);
        uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
        const uint8_t *qs = qhp + 4;
        float *yb = y + b * CO_QK;
        for (int j = 0; j < 16; ++j) {
            int q0 = (qs[j] & 0xF) | (int)(((qh >> j) & 1u) << 4);
            int q1 = (qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
            if (with_min) {
                float t0 = (float)q0 * d, t1 = (float)q1 * d;
                yb[j] = t0 + m;
                yb[j + 16] = t1 + m;
            } else {
                yb[j] = ((float)q0 - 16.0f) * d;
                yb[j + 16] = ((float)q1 - 16.0f) * d;
            }
        }
    }
}

/* f32 -> Q4_1 / Q5_0 / Q5_1, tensor/internal/metal/kernels/quantized.metal:4216-4280 (Q4_1:
 * min and max of the block, d = (max - min) / 15, id = d ? 1/d : 0, q = min(15, (int8)((v - min)
 * * id + 0.5))), :4282-4345 (Q5_0: first element of largest |v| gives max with its sign, d =
 * max / -16, q = min(31, (int8)(v * id + 16.5))), :4347-4415 (Q5_1: d = (max - min) / 31, q =
 * (uint8)((v - min) * id + 0.5), no clamp).  d and min are stored rounded to f16; id comes from
 * the unrounded d.  The shaders pair value j with value j+16 in byte j (split order); for Q4_1
 * `order` 0 pairs values 2j, 2j+1 instead so that the Go dequantizer returns source order. */
void co_quantize_more(int qtype, const float *w, int64_t nblocks, int order, uint8_t *blocks) {
    const int64_t bb = co_block_bytes(qtype);
    const int interleaved = (qtype == 3 && order == CO_ORDER_GO_INTERLEAVED);
    for (int64_t b = 0; b < nblocks; ++b) {
        const float *src = w + b * CO_QK;
        uint8_t *blk = blocks + b * bb;
        float d, mn = 0.0f, off;
        if (qtype == 6) {
            float amax = 0.0f, max = 0.0f;
            for (int j = 0; j < CO_QK; ++j)
                if (amax < fabsf(src[j])) {
                    amax = fabsf(src[j]);
                    max = src[j];
                }
            d = max / -16.0f;
            off = 16.5f;
        } else {
            float lo = src[0], hi = src[0];
            for (int j = 1; j < CO_QK; ++j) {
                lo = src[j] < lo ? src[j] : lo;
                hi = src[j] > hi ? src[j] : hi;
            }
            float range = hi - lo;
            d = range / (qtype == 3 ? 15.0f : 31.0f);
            mn = lo;
            off = 0.5f;
        }
        float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        store_u16(blk, co_f32_to_fp16(d));
        uint8_t *qs = blk + 2;
        if (qtype != 6) {
            store_u16(blk + 2, co_f32_to_fp16(mn));
            qs += 2;
        }
        uint8_t *qhp = qs;
        if (qtype != 3) qs += 4;
        uint32_t qh = 0;
        for (int j = 0; j < 16; ++j) {
            int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + 16;
            float s0 = src[i0] - mn, s1 = src[i1] - mn;
            float x0 = s0 * id, x1 = s1 * id;
            float r0 = x0 + off, r1 = x1 + off;
            int q0, q1;
            if (qtype == 7) {
                q0 = (int)(uint8_t)(int)r0;
                q1 = (int)(uint8_t)(int)r1;
            } else {
                const int top = qtype == 3 ? 15 : 31;
                q0 = (int)(int8_t)(int)r0;
                q1 = (int)(int8_t)(int)r1;
                q0 = q0 < top ? q0 : top;
                q1 = q1 < top ? q1 : top;
                q0 &= 0xFF;
                q1 &= 0xFF;
            }
            qs[j] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
            qh |= (uint32_t)((q0 >> 4) & 1) << j;
            qh |= (uint32_t)((q1 >> 4) & 1) << (j + 16);
        }
        if (qtype != 3) {
            qhp[0] = (uint8_t)qh, qhp[1] = (uint8_t)(qh >> 8), qhp[2] = (uint8_t)(qh >> 16), qhp[3] = (uint8_t)(qh >> 24);
        }
    }
}

/* tensor/internal/cpu/kernels/conv.go:373-389 (NaiveBatchedMatMulStridedF32):
 * c[i,j] = sum over l = 0..k-1, in that order, of a*b with the product and the sum
 * each rounded to f32, starting from +0.  Strides are {batch,row,col} in elements. */
void co_matmul_strided_f32(int64_t bsize, int64_t m, int64_t n, int64_t k, const float *a,
                           const float *b, float *c, const int64_t *as, const int64_t *bs,
                           const int64_t *cs) {
    for (int64_t bb = 0; bb < bsize; ++bb)
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) {
                float sum = 0.0f;
                for (int64_t l = 0; l < k; ++l) {
                    float prod = a[bb * as[0] + i * as[1] + l * as[2]] *
                                 b[bb * bs[0] + l * bs[1] + j * bs[2]];
                    sum = sum + prod;
                }
                c[bb * cs[0] + i * cs[1] + j * cs[2]] = sum;
            }
}

static void dequant_row(int qtype, int order, const uint8_t *row, int64_t nb, float *out) {
    if (qtype == 2)
        co_dequantize_q4_0(row, nb, order, out);
    else if (qtype == 3)
        co_dequantize_q4_1(row, nb, order, out);
    else if (qtype == 6 || qtype == 7)
        co_dequantize_q5(qtype, row, nb, out);
    else
        co_dequantize_q8_0(row, nb, out);
}

/* "candy's CPU quantized linear": dequantize every block of W [n,k]
 * (quantized.go:85-93 / :131-136), then y = x . W^T through the strided naive matmul
 * with rhs strides {0,1,K} -- the branch CpuStorage.MatMul takes for a transposed
 * weight view (tensor/internal/cpu/storage.go:892-909) as reached from
 * nn/linear.go:58-112.  Rows of W are dequantized one at a time into a scratch row;
 * the per-element arithmetic and its order are unchanged.  qtype: 2 = Q4_0, 8 = Q8_0; 3 / 6 / 7 =
 * Q4_1 / Q5_0 / Q5_1 follow the same rule (the reference's CPU side holds only their dequantizers).
 * nthreads > 1 splits the rows of W across OpenMP threads (each output element is
 * still one sequential sum, so results do not depend on nthreads). */
int co_qmatmul(int qtype, int order, const float *x, int64_t m, int64_t k, int64_t ldx,
               const uint8_t *wblocks, int64_t n, float *y, int64_t ldy, int nthreads) {
    if (k <= 0 || k % CO_QK != 0 || m <= 0 || n <= 0) return -1;
    if (co_block_bytes(qtype) == 0) return -2;
    if ((qtype == 6 || qtype == 7) && order != CO_ORDER_GGML_SPLIT) return -3;
    const int64_t nb = k / CO_QK;
    const int64_t bpb = co_block_bytes(qtype);
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel num_threads(nthreads)
    {
        float *wrow = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t j = 0; j < n; ++j) {
            dequant_row(qtype, order, wblocks + j * nb * bpb, nb, wrow);
            for (int64_t i = 0; i < m; ++i) {
                float sum = 0.0f;
                const float *xi = x + i * ldx;
                for (int64_t l = 0; l < k; ++l) {
                    float prod = xi[l] * wrow[l];
                    sum = sum + prod;
                }
                y[i * ldy + j] = sum;
            }
        }
        free(wrow);
    }
    return 0;
}

/* ---- K super-block formats (256 values), tensor/internal/cuda/kernels/quantized.cu:366-436 (layouts) and
 * :899-1147 (dequantizers): the reference's only code for them is CUDA, restated here value by value, in
 * value order, with each kernel's expression and operation order.  GGML type ids 10..14.  Pinned bit for bit
 * against the third-party gguf package's dequantizers (tests/test_kquants.py). */
static int64_t co_k_block_bytes(int qtype) {
    switch (qtype) {
    case 10: return 84;
    case 11: return 110;
    case 12: return 144;
    case 13: return 176;
    case 14: return 210;
    default: return 0;
    }
}

/* get_scale_min_k4, quantized.cu:994-1006 */
static void co_scale_min_k4(int j, const uint8_t *q, int *d, int *m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

void co_dequantize_k(int qtype, const uint8_t *blocks, int64_t nblocks, float *y) {
    const int64_t bb = co_k_block_bytes(qtype);
    for (int64_t ib = 0; ib < nblocks; ++ib) {
        const uint8_t *b = blocks + ib * bb;
        float *out = y + ib * 256;
        if (qtype == 10) { /* dequantize_block_q2_K, quantized.cu:902-925 */
            const float dall = co_fp16_to_f32(load_u16(b + 80)), dmin = co_fp16_to_f32(load_u16(b + 82));
            const uint8_t *scales = b, *qs = b + 16;
            for (int n = 0; n < 2; ++n)
                for (int l = 0; l < 32; ++l) {
                    const int is = 8 * n + l / 16;
                    const uint8_t q = qs[32 * n + l];
                    for (int j = 0; j < 4; ++j) {
                        const uint8_t sc = scales[is + 2 * j];
                        float t = dall * (float)(sc & 0xF);
                        t = t * (float)((q >> (2 * j)) & 3);
                        const float mn = dmin * (float)(sc >> 4);
                        out[128 * n + 32 * j + l] = t - mn;
                    }
                }
        } else if (qtype == 11) { /* dequantize_block_q3_K, quantized.cu:937-969 */
            const uint8_t *hm = b, *qs = b + 32, *sc = b + 96;
            const float d_all = co_fp16_to_f32(load_u16(b + 108));
            for (int n = 0; n < 2; ++n)
                for (int j = 0; j < 4; ++j)
                    for (int is0 = 0; is0 < 2; ++is0) {
                        const int is = 8 * n + 2 * j + is0;
                        const int us = is < 4 ? (sc[is] & 0xF) | (((sc[is + 8] >> 0) & 3) << 4)
                                     : is < 8 ? (sc[is] & 0xF) | (((sc[is + 4] >> 2) & 3) << 4)
                                     : is < 12 ? (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4)
                                               : (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
                        const float dl = d_all * (float)((int)(int8_t)us - 32);
                        const uint8_t m = (uint8_t)(1 << (4 * n + j));
                        for (int l = 16 * is0; l < 16 * is0 + 16; ++l)
                            out[128 * n + 32 * j + l] = dl * (float)((int)(int8_t)((qs[32 * n + l] >> (2 * j)) & 3) - ((hm[l] & m) ? 0 : 4));
                    }
        } else if (qtype == 12 || qtype == 13) { /* dequantize_block_q4_K :1008-1042, _q5_K :1049-1082 */
            const float dall = co_fp16_to_f32(load_u16(b)), dmin = co_fp16_to_f32(load_u16(b + 2));
            const uint8_t *scales = b + 4;
            const uint8_t *qh = b + 16;                         /* Q5_K only */
            const uint8_t *qs = b + (qtype == 12 ? 16 : 48);
            for (int il = 0; il < 4; ++il)
                for (int h = 0; h < 2; ++h) {
                    int sc, m;
                    co_scale_min_k4(2 * il + h, scales, &sc, &m);
                    const float d1 = dall * (float)sc, m1 = dmin * (float)m;
                    for (int l = 0; l < 32; ++l) {
                        int q = h ? (qs[32 * il + l] >> 4) : (qs[32 * il + l] & 0xF);
                        if (qtype == 13) q += (qh[l] & (1 << (2 * il + h))) ? 16 : 0;
                        const float t = d1 * (float)q;
                        out[64 * il + 32 * h + l] = t - m1;
                    }
                }
        } else { /* dequantize_block_q6_K, quantized.cu:1099-1123 */
            const uint8_t *ql = b, *qh = b + 128;
            const int8_t *sc = (const int8_t *)(b + 192);
            const float d = co_fp16_to_f32(load_u16(b + 208));
            for (int ip = 0; ip < 2; ++ip)
                for (int il = 0; il < 32; ++il) {
                    const int is = 8 * ip + il / 16;
                    const uint8_t h = qh[32 * ip + il];
                    const uint8_t *q = ql + 64 * ip + il;
                    const int v[4] = {(int)(int8_t)((q[0] & 0xF) | (((h >> 0) & 3) << 4)) - 32, (int)(int8_t)((q[32] & 0xF) | (((h >> 2) & 3) << 4)) - 32,
                                      (int)(int8_t)((q[0] >> 4) | (((h >> 4) & 3) << 4)) - 32, (int)(int8_t)((q[32] >> 4) | (((h >> 6) & 3) << 4)) - 32};
                    for (int t = 0; t < 4; ++t) {
                        const float ds = d * (float)sc[is + 2 * t];
                        out[128 * ip + 32 * t + il] = ds * (float)v[t];
                    }
                }
        }
    }
}

/* y = x . W^T for a K-format W [n,k] (k % 256 == 0): dequantize each row, then the sequential f32 dot of
 * candy's CPU matmul (conv.go:373-389), as co_qmatmul does for the 32-value formats. */
int co_qmatmul_k(int qtype, const float *x, int64_t m, int64_t k, int64_t ldx, const uint8_t *wblocks, int64_t n, float *y, int64_t ldy,
                 int nthreads) {
    const int64_t bb = co_k_block_bytes(qtype);
    if (bb == 0) return -2;
    if (k <= 0 || k % 256 != 0 || m <= 0 || n <= 0) return -1;
    const int64_t nsb = k / 256;
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel num_threads(nthreads)
    {
        float *wrow = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t j = 0; j < n; ++j) {
            co_dequantize_k(qtype, wblocks + j * nsb * bb, nsb, wrow);
            for (int64_t i = 0; i < m; ++i) {
                float sum = 0.0f;
                const float *xi = x + i * ldx;
                for (int64_t l = 0; l < k; ++l) {
                    float prod = xi[l] * wrow[l];
                    sum = sum + prod;
                }
                y[i * ldy + j] = sum;
            }
        }
        free(wrow);
    }
    return 0;
}

/* f32 activations -> Q8_1 blocks {half d; half sum; int8 q[32]},
 * tensor/internal/cuda/kernels/quantized.cu:3521-3558 (struct at :349-357):
 * d = amax/127; q = amax==0 ? 0 : roundf(x/d) (true division by the f32 d);
 * sum = sum of the unquantized x.  The kernel reduces both with xor-butterfly
 * shuffles (offsets 16,8,4,2,1: quantized.cu:22-46); the same pairing is used here so
 * that the f32 sum is rounded identically. */
void co_quantize_q8_1(const float *x, int64_t nblocks, uint8_t *out) {
    for (int64_t b = 0; b < nblocks; ++b) {
        const float *src = x + b * CO_QK;
        uint8_t *blk = out + b * CO_Q8_1_BYTES;
        float s[CO_QK], amax = 0.0f;
        for (int i = 0; i < CO_QK; ++i) {
            s[i] = src[i];
            float a = fabsf(src[i]);
            amax = amax > a ? amax : a;
        }
        for (int mask = 16; mask > 0; mask >>= 1) {
            float t[CO_QK];
            for (int i = 0; i < CO_QK; ++i) t[i] = s[i] + s[i ^ mask];
            memcpy(s, t, sizeof(s));
        }
        float d = amax / 127.0f;
        store_u16(blk, co_f32_to_fp16(d));
        store_u16(blk + 2, co_f32_to_fp16(s[0]));
        for (int i = 0; i < CO_QK; ++i) {
            int8_t q = (amax == 0.0f) ? 0 : (int8_t)roundf(src[i] / d);
            blk[4 + i] = (uint8_t)q;
        }
    }
}

/* One Q4_0 block against one Q8_1 block with the reference's CUDA arithmetic:
 * vec_dot_q4_0_q8_1 (quantized.cu:2420-2438) is called twice per block by
 * mul_mat_vec_q (quantized.cu:2806-2824; vdr = 2, so iqs = 0 and 2), each call taking
 * 8 bytes of nibbles: low nibbles pair with q8[4*iqs ..], high nibbles with
 * q8[4*(iqs+4) ..] (split order), and each returns
 *     d4 * (sumi * d8 - (8*vdr/QI4_0) * s8)         (quantized.cu:1919-1941)
 * with d8 and s8 read back from their half storage. */
static float o2_block_q4_0(const uint8_t *wblk, const uint8_t *ablk, int order) {
    float d4 = co_fp16_to_f32(load_u16(wblk));
    float d8 = co_fp16_to_f32(load_u16(ablk));
    float s8 = co_fp16_to_f32(load_u16(ablk + 2));
    const uint8_t *qs = wblk + 2;
    const int8_t *q8 = (const int8_t *)(ablk + 4);
    float acc = 0.0f;
    for (int half = 0; half < 2; ++half) {
        int32_t sumi = 0;
        for (int j = 8 * half; j < 8 * half + 8; ++j) {
            int lo = qs[j] & 0xF, hi = qs[j] >> 4;
            int e_lo = (order == CO_ORDER_GO_INTERLEAVED) ? 2 * j : j;
            int e_hi = (order == CO_ORDER_GO_INTERLEAVED) ? 2 * j + 1 : j + 16;
            sumi += lo * q8[e_lo] + hi * q8[e_hi];
        }
        float part = d4 * ((float)sumi * d8 - 4.0f * s8);
        acc = acc + part;
    }
    return acc;
}

/* vec_dot_q8_0_q8_1 (quantized.cu:2504-2521, impl :2058-2073): four calls per block
 * (vdr = 2 ints = 8 values each), each d8_0 * d8_1 * sumi. */
static float o2_block_q8_0(const uint8_t *wblk, const uint8_t *ablk) {
    float d0 = co_fp16_to_f32(load_u16(wblk));
    float d1 = co_fp16_to_f32(load_u16(ablk));
    const int8_t *qw = (const int8_t *)(wblk + 2);
    const int8_t *qa = (const int8_t *)(ablk + 4);
    float acc = 0.0f;
    for (int part = 0; part < 4; ++part) {
        int32_t sumi = 0;
        for (int i = 8 * part; i < 8 * part + 8; ++i) sumi += (int32_t)qw[i] * (int32_t)qa[i];
        float v = d0 * d1 * (float)sumi;
        acc = acc + v;
    }
    return acc;
}

/* The reference's CUDA quantized matmul numerics: activations through the Q8_1
 * quantizer, per-block integer dots scaled in f32 (quantized.cu:2787-2871).  The
 * kernel's thread-level summation order is an implementation detail; here the
 * per-block values are added in block order.  For order 0 the activation element
 * that pairs with each nibble follows the Go element order instead of the split one. */
int co_qmatmul_q8_1(int qtype, int order, const float *x, int64_t m, int64_t k, int64_t ldx,
                    const uint8_t *wblocks, int64_t n, float *y, int64_t ldy, int nthreads) {
    if (k <= 0 || k % CO_QK != 0 || m <= 0 || n <= 0) return -1;
    if (qtype != 2 && qtype != 8) return -2;
    const int64_t nb = k / CO_QK;
    const int64_t bpb = (qtype == 2) ? CO_Q4_0_BYTES : CO_Q8_0_BYTES;
    uint8_t *act = (uint8_t *)malloc((size_t)(m * nb) * CO_Q8_1_BYTES);
    if (!act) return -3;
    for (int64_t i = 0; i < m; ++i) co_quantize_q8_1(x + i * ldx, nb, act + i * nb * CO_Q8_1_BYTES);
    if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads)
    for (int64_t j = 0; j < n; ++j) {
        for (int64_t i = 0; i < m; ++i) {
            float sum = 0.0f;
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t *wb = wblocks + (j * nb + b) * bpb;
                const uint8_t *ab = act + (i * nb + b) * CO_Q8_1_BYTES;
                float v = (qtype == 2) ? o2_block_q4_0(wb, ab, order) : o2_block_q8_0(wb, ab);
                sum = sum + v;
            }
            y[i * ldy + j] = sum;
        }
    }
    free(act);
    return 0;
}
