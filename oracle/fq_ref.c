/*
 * CPU oracle for the K-quant dequantize-and-multiply path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls anything in this file; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Every function restates, operation for operation, CPU code that the reference
 * (austinwells-dev/ferrum) itself uses as the expected value in its kernel tests.
 * The reference is a macOS-only Rust crate whose implementation of this path is Metal
 * shader code, so it cannot be compiled here; parity is pinned against the reference's
 * closed-form test fixtures (src/ops/transformer.rs:2833-2980, 4102-4189, 1683-1728),
 * which this repository's tests re-derive independently of the block decoders below.
 * The reference stores no golden output vectors for this path.
 *
 * Compile with -ffp-contract=off: the dequantizers are a fixed sequence of IEEE
 * single-precision operations and must not be fused.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FQO_Q8_0 8
#define FQO_Q3_K 11
#define FQO_Q4_K 12
#define FQO_Q5_K 13
#define FQO_IQ4_NL 20
#define FQO_IQ4_XS 23
#define FQO_Q6_K 14

/* ---------------------------------------------------------------- scalar conversions */

/* IEEE binary16 -> binary32, exact (the reference uses the `half` crate 2.7.1,
 * `f16::from_le_bytes(..).to_f32()`, e.g. src/diffusion/tests.rs:765-767). */
float fqo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (`half::f16::from_f32`). */
uint16_t fqo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mag = x & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (mag > 0x7F800000u ? 0x200u | ((mag >> 13) & 0x3FFu) : 0));
    if (mag >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to infinity */
    if (mag < 0x33000001u) return (uint16_t)sign;               /* rounds to zero */
    int32_t e = (int32_t)(mag >> 23) - 127;
    uint32_t m = (mag & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1))) q++;
    return (uint16_t)(sign | (half_bits + q));
}

/* Round to the nearest BF16, ties to even, NaN quieted: src/hybrid/draft/gguf.rs:362-369. */
uint16_t fqo_f32_to_bf16(float v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    if (v != v) return (uint16_t)((bits >> 16) | 0x40u);
    return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

float fqo_bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static float f16_at(const uint8_t *b, int at) {
    return fqo_f16_to_f32((uint16_t)(b[at] | (b[at + 1] << 8)));
}

/* ---------------------------------------------------------------- block layouts */

/* (elements, bytes) of a block: src/loader/gguf.rs:99-105, src/quantization.rs:50-73. */
int fqo_block_layout(int format, int *elements, int *bytes) {
    switch (format) {
    case FQO_Q8_0: *elements = 32; *bytes = 34; return 0;
    case FQO_Q4_K: *elements = 256; *bytes = 144; return 0;
    case FQO_Q5_K: *elements = 256; *bytes = 176; return 0;
    case FQO_Q3_K: *elements = 256; *bytes = 110; return 0;
    case FQO_Q6_K: *elements = 256; *bytes = 210; return 0;
    case FQO_IQ4_NL: *elements = 32; *bytes = 18; return 0;   /* src/loader/gguf.rs:110 */
    case FQO_IQ4_XS: *elements = 256; *bytes = 136; return 0; /* src/loader/gguf.rs:111 */
    default: return -1;
    }
}

/* Payload validation before blocks are kept as packed storage:
 * src/quantization.rs:212-261.  0 = ok, 1 = stream ends inside a block,
 * 2 = non-finite (or, for Q8_0, negative) scale, 3 = Q8_0 value -128. */
int fqo_validate(int format, const uint8_t *p, size_t len) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb)) return -1;
    if (len % (size_t)bb) return 1;
    for (size_t o = 0; o < len; o += (size_t)bb) {
        const uint8_t *b = p + o;
        if (format == FQO_Q3_K) {
            continue; /* no check in the reference: Q3_K is rewritten as Q6_K before it is kept */
        } else if (format == FQO_Q4_K || format == FQO_Q5_K) {
            if (!isfinite(f16_at(b, 0)) || !isfinite(f16_at(b, 2))) return 2;
        } else if (format == FQO_Q6_K) {
            if (!isfinite(f16_at(b, 208))) return 2;
        } else if (format == FQO_IQ4_NL || format == FQO_IQ4_XS) {
            if (!isfinite(f16_at(b, 0))) return 2; /* no check in the reference; the one scale of the block, as for Q4_0 */
        } else {
            float s = f16_at(b, 0);
            if (!isfinite(s) || s < 0.0f) return 2;
            for (int i = 2; i < 34; i++)
                if (b[i] == 0x80) return 3;
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- dequantizers */

/* Sub-block j's 6-bit scale and minimum: src/diffusion/tests.rs:797-807
 * (same as src/ops/transformer.rs:2905-2918 and hybrid.metal:417-420). */
static void scale_min(int j, const uint8_t *q, float *sc, float *m) {
    uint8_t s, mn;
    if (j < 4) {
        s = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        s = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
    *sc = (float)s;
    *m = (float)mn;
}

/* One Q4_K block: src/diffusion/tests.rs:811-832 (`q45_k` with high = false).
 * Value order and evaluation order ((d*sc)*q) - (dmin*m) are the reference's. */
static void dequant_q4_k(const uint8_t *b, float *out) {
    float d = f16_at(b, 0), dmin = f16_at(b, 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
    for (int j = 0; j < 4; j++) {
        const uint8_t *q = qs + 32 * j;
        for (int half = 0; half < 2; half++) {
            float sc, m;
            scale_min(2 * j + half, scales, &sc, &m);
            for (int l = 0; l < 32; l++) {
                uint8_t low = half == 0 ? (q[l] & 0xF) : (q[l] >> 4);
                float ds = d * sc;
                float t = ds * (float)low;
                float mm = dmin * m;
                *out++ = t - mm;
            }
        }
    }
}

/* One Q5_K block: src/diffusion/tests.rs:811-840 (`q45_k` with high = true): 32 bytes of fifth bits between the
 * scales and the nibbles; bit (2 j + half) of qh[l] belongs to value l of that sub-block. */
static void dequant_q5_k(const uint8_t *b, float *out) {
    float d = f16_at(b, 0), dmin = f16_at(b, 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + 48;
    for (int j = 0; j < 4; j++) {
        const uint8_t *q = qs + 32 * j;
        for (int half = 0; half < 2; half++) {
            float sc, m;
            scale_min(2 * j + half, scales, &sc, &m);
            uint8_t bit = (uint8_t)(1u << (2 * j + half));
            for (int l = 0; l < 32; l++) {
                uint8_t low = half == 0 ? (q[l] & 0xF) : (q[l] >> 4);
                uint8_t top = (qh[l] & bit) ? 16 : 0;
                float ds = d * sc;
                float t = ds * (float)(low + top);
                float mm = dmin * m;
                *out++ = t - mm;
            }
        }
    }
}

/* One Q3_K block (hmask[32], qs[64], scales[12], d): llama.cpp's `dequantize_row_q3_K` as the reference's tests
 * restate it, src/hybrid/iq_tests.rs:1441-1478.  Used to check the Q3_K -> Q6_K rewrite of the loader. */
static void dequant_q3_k(const uint8_t *b, float *out) {
    const uint8_t *hm = b, *q = b + 32;
    float d_all = f16_at(b, 108);
    uint32_t aux[4] = {0, 0, 0, 0};
    for (int k = 0; k < 3; k++) aux[k] = (uint32_t)b[96 + 4 * k] | ((uint32_t)b[97 + 4 * k] << 8) | ((uint32_t)b[98 + 4 * k] << 16) | ((uint32_t)b[99 + 4 * k] << 24);
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu, tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
    aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
    aux[0] = (aux[0] & kmask2) | ((tmp & kmask1) << 4);
    aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
    int8_t scales[16];
    for (int k = 0; k < 16; k++) scales[k] = (int8_t)((aux[k / 4] >> (8 * (k % 4))) & 0xFF);
    int is = 0, at = 0;
    uint8_t m = 1;
    for (int n = 0; n < 2; n++) {
        const uint8_t *qq = q + 32 * n;
        for (int shift = 0; shift < 8; shift += 2) {
            for (int half = 0; half < 2; half++) {
                float dl = d_all * ((float)scales[is++] - 32.0f);
                for (int l = 16 * half; l < 16 * half + 16; l++) {
                    int v = (int)((qq[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4);
                    out[at++] = dl * (float)v;
                }
            }
            m = (uint8_t)(m << 1);
        }
    }
}

/* One Q6_K block: src/diffusion/tests.rs:842-864 (= src/hybrid/iq_tests.rs:1481-1500). */
static void dequant_q6_k(const uint8_t *b, float *out) {
    const uint8_t *ql0 = b, *qh0 = b + 128;
    const int8_t *sc0 = (const int8_t *)(b + 192);
    float d = f16_at(b, 208);
    for (int n = 0; n < 2; n++) {
        const uint8_t *ql = ql0 + 64 * n, *qh = qh0 + 32 * n;
        const int8_t *sc = sc0 + 8 * n;
        float *y = out + 128 * n;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            uint8_t q[4] = {
                (uint8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)),
                (uint8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)),
                (uint8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)),
                (uint8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)),
            };
            for (int i = 0; i < 4; i++) {
                float scale = (float)sc[is + 2 * i];
                float ds = d * scale;
                y[l + 32 * i] = ds * ((float)q[i] - 32.0f);
            }
        }
    }
}

/* The non-linear 4-bit codebook of the IQ4 formats (`kvalues_iq4nl`, src/hybrid/iq_tests.rs:1608-1610). */
static const int8_t IQ4_VALUES[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* One IQ4_NL block (d f16, qs[16]): `dequant_iq4_nl`, src/hybrid/iq_tests.rs:1606-1618: byte j holds values j and
 * j + 16. */
static void dequant_iq4_nl(const uint8_t *b, float *out) {
    float d = f16_at(b, 0);
    for (int j = 0; j < 16; j++) {
        out[j] = d * (float)IQ4_VALUES[b[2 + j] & 15];
        out[j + 16] = d * (float)IQ4_VALUES[b[2 + j] >> 4];
    }
}

/* One IQ4_XS block (d f16, scales_h u16, scales_l[4], qs[128]): `dequantize_iq4_xs`,
 * src/metal/shaders/hybrid.metal:580-596: sub-block ib of 32 values has the 6-bit scale
 * ls = (scales_l[ib / 2] >> 4 (ib % 2) & 15) | (scales_h >> 2 ib & 3) << 4 and the factor d (ls - 32); byte j of
 * its 16 bytes holds values j and j + 16. */
static void dequant_iq4_xs(const uint8_t *b, float *out) {
    float d = f16_at(b, 0);
    unsigned scales_h = (unsigned)b[2] | ((unsigned)b[3] << 8);
    for (int ib = 0; ib < 8; ib++) {
        int ls = (int)((b[4 + ib / 2] >> (4 * (ib % 2))) & 15) | (int)(((scales_h >> (2 * ib)) & 3) << 4);
        float dl = d * (float)(ls - 32);
        const uint8_t *q = b + 8 + 16 * ib;
        for (int j = 0; j < 16; j++) {
            out[32 * ib + j] = dl * (float)IQ4_VALUES[q[j] & 15];
            out[32 * ib + j + 16] = dl * (float)IQ4_VALUES[q[j] >> 4];
        }
    }
}

/* One Q8_0 block: src/hybrid/draft/gguf.rs:336-343. */
static void dequant_q8_0(const uint8_t *b, float *out) {
    float d = f16_at(b, 0);
    for (int i = 0; i < 32; i++) out[i] = (float)(int8_t)b[2 + i] * d;
}

/* Decode `blocks` consecutive blocks. */
int fqo_dequant(int format, const uint8_t *src, size_t blocks, float *out) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb)) return -1;
    for (size_t i = 0; i < blocks; i++) {
        const uint8_t *b = src + i * (size_t)bb;
        float *o = out + i * (size_t)el;
        if (format == FQO_Q4_K) dequant_q4_k(b, o);
        else if (format == FQO_Q5_K) dequant_q5_k(b, o);
        else if (format == FQO_Q3_K) dequant_q3_k(b, o);
        else if (format == FQO_Q6_K) dequant_q6_k(b, o);
        else if (format == FQO_IQ4_NL) dequant_iq4_nl(b, o);
        else if (format == FQO_IQ4_XS) dequant_iq4_xs(b, o);
        else dequant_q8_0(b, o);
    }
    return 0;
}

/* ---------------------------------------------------------------- matmul oracles */

/* y[m][n] = sum_k x[m][k] * W[n][k], W given as dequantized `dense` [rows, cols].
 * mode 0: f64 accumulate, cast to f32 (src/hybrid/iq_tests.rs:1317-1325,
 *         src/diffusion/tests.rs:741-748, src/reference.rs:57-66);
 * mode 1: f32 left-to-right sum (src/ops/transformer.rs:2964-2980);
 * mode 2: bf16(x) * bf16(w) in f32, left-to-right f32 sum, result rounded to bf16
 *         and widened (src/ops/transformer.rs:3683-3694). */
void fqo_matmul_dense(const float *dense, size_t rows, size_t cols, const float *x, size_t m,
                      int mode, float *y) {
    for (size_t i = 0; i < m; i++) {
        const float *xi = x + i * cols;
        for (size_t r = 0; r < rows; r++) {
            const float *w = dense + r * cols;
            if (mode == 0) {
                double acc = 0.0;
                for (size_t c = 0; c < cols; c++) acc += (double)xi[c] * (double)w[c];
                y[i * rows + r] = (float)acc;
            } else if (mode == 1) {
                float acc = 0.0f;
                for (size_t c = 0; c < cols; c++) {
                    float p = xi[c] * w[c];
                    acc = acc + p;
                }
                y[i * rows + r] = acc;
            } else {
                float acc = 0.0f;
                for (size_t c = 0; c < cols; c++) {
                    float p = fqo_bf16_to_f32(fqo_f32_to_bf16(xi[c])) *
                              fqo_bf16_to_f32(fqo_f32_to_bf16(w[c]));
                    acc = acc + p;
                }
                y[i * rows + r] = fqo_bf16_to_f32(fqo_f32_to_bf16(acc));
            }
        }
    }
}

/* Dequantize then multiply; `W` is `rows` rows of cols/elements blocks. */
int fqo_matmul(int format, const uint8_t *W, size_t rows, size_t cols, const float *x, size_t m,
               int mode, float *y) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb) || cols % (size_t)el) return -1;
    size_t row_bytes = cols / (size_t)el * (size_t)bb;
    float *dense = (float *)malloc(sizeof(float) * cols);
    if (!dense) return -2;
    for (size_t r = 0; r < rows; r++) {
        fqo_dequant(format, W + r * row_bytes, cols / (size_t)el, dense);
        for (size_t i = 0; i < m; i++) {
            float out;
            fqo_matmul_dense(dense, 1, cols, x + i * cols, 1, mode, &out);
            y[i * rows + r] = out;
        }
    }
    free(dense);
    return 0;
}

/* Expert GEMV: route r multiplies activation row r / x_div by the rows of expert ids[r]
 * (src/hybrid/iq_tests.rs:1398-1439; kernel contract hybrid.metal:2390-2428). */
int fqo_matmul_id(int format, const uint8_t *W, size_t rows_e, size_t cols, const float *x,
                  const uint32_t *ids, size_t routes, size_t x_div, int mode, float *y) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb) || cols % (size_t)el || x_div == 0) return -1;
    size_t row_bytes = cols / (size_t)el * (size_t)bb;
    for (size_t r = 0; r < routes; r++) {
        int rc = fqo_matmul(format, W + (size_t)ids[r] * rows_e * row_bytes, rows_e, cols,
                            x + (r / x_div) * cols, 1, mode, y + r * rows_e);
        if (rc) return rc;
    }
    return 0;
}

/* Expert GEMM over expert-sorted rows: group z covers rows offsets[z]..offsets[z+1] and
 * uses the expert stored at slots[z] (or z when slots is NULL)
 * (src/hybrid/iq_tests.rs:1766-1800; kernel contract hybrid.metal:2430-2523). */
int fqo_matmul_grouped(int format, const uint8_t *W, size_t rows_e, size_t cols, const float *x,
                       const uint32_t *offsets, const uint32_t *slots, size_t groups, int mode,
                       float *y) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb) || cols % (size_t)el) return -1;
    size_t row_bytes = cols / (size_t)el * (size_t)bb;
    for (size_t z = 0; z < groups; z++) {
        size_t e = slots ? slots[z] : z;
        for (size_t row = offsets[z]; row < offsets[z + 1]; row++) {
            int rc = fqo_matmul(format, W + e * rows_e * row_bytes, rows_e, cols, x + row * cols, 1,
                                mode, y + row * rows_e);
            if (rc) return rc;
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- MoE glue */

/* Routing oracle: src/hybrid/engine.rs:5001-5033 (the test's expected values), which is the
 * same selection as the shipping CPU router src/nn/moe.rs:392-458.  Scores are softmax in f32
 * (max, exp, left-to-right sum, divide) or a logistic per logit; order is score descending,
 * then expert index ascending; weights are divided by the picked sum when `norm`. */
void fqo_moe_route(const float *logits, const float *x, const float *shared_w, int experts,
                   int used, int hidden, int tokens, int sigmoid, int norm, int shared_gate,
                   uint32_t *ids, float *weights, float *gate) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)experts);
    char *taken = (char *)malloc((size_t)experts);
    for (int t = 0; t < tokens; t++) {
        const float *row = logits + (size_t)t * experts;
        if (sigmoid) {
            for (int e = 0; e < experts; e++) scores[e] = 1.0f / (1.0f + expf(-row[e]));
        } else {
            float mx = -INFINITY;
            for (int e = 0; e < experts; e++) mx = row[e] > mx ? row[e] : mx;
            float total = 0.0f;
            for (int e = 0; e < experts; e++) {
                scores[e] = expf(row[e] - mx);
                total = total + scores[e];
            }
            for (int e = 0; e < experts; e++) scores[e] = scores[e] / total;
        }
        memset(taken, 0, (size_t)experts);
        float sum = 0.0f;
        for (int k = 0; k < used; k++) {
            int best = -1;
            for (int e = 0; e < experts; e++) {
                if (taken[e]) continue;
                if (best < 0 || scores[e] > scores[best]) best = e; /* ties keep the lower index */
            }
            taken[best] = 1;
            ids[(size_t)t * used + k] = (uint32_t)best;
            weights[(size_t)t * used + k] = scores[best];
            sum = sum + scores[best];
        }
        if (norm)
            for (int k = 0; k < used; k++) weights[(size_t)t * used + k] /= sum;
        if (shared_gate) {
            float dot = 0.0f;
            for (int i = 0; i < hidden; i++) {
                float p = x[(size_t)t * hidden + i] * shared_w[i];
                dot = dot + p;
            }
            gate[t] = 1.0f / (1.0f + expf(-dot));
        } else {
            gate[t] = 1.0f;
        }
    }
    free(scores);
    free(taken);
}

/* Deterministic expert-major ordering of routes (hybrid.metal:2321-2358): offsets[e]..offsets[e+1]
 * are expert e's rows, sorted[p] the route at row p, position[r] the row of route r; routes of
 * one expert keep their route order. */
void fqo_moe_map(const uint32_t *ids, int experts, int routes, uint32_t *offsets, uint32_t *sorted,
                 uint32_t *position) {
    uint32_t acc = 0;
    for (int e = 0; e < experts; e++) {
        offsets[e] = acc;
        for (int r = 0; r < routes; r++)
            if (ids[r] == (uint32_t)e) {
                sorted[acc] = (uint32_t)r;
                position[r] = acc;
                acc++;
            }
    }
    offsets[experts] = acc;
}

/* xg[row] = x[token of sorted[row]] (hybrid.metal:2360-2369). */
void fqo_moe_gather(const float *x, const uint32_t *sorted, int hidden, int used, int routes,
                    float *xg) {
    for (int r = 0; r < routes; r++)
        memcpy(xg + (size_t)r * hidden, x + (size_t)(sorted[r] / (uint32_t)used) * hidden,
               sizeof(float) * (size_t)hidden);
}

/* out[t] = sum_s w[t][s] * down[row(t,s)] + gate[t] * shared[t] (hybrid.metal:2371-2388);
 * row(t,s) is the route itself when `identity`, else position[route]. */
void fqo_moe_combine(const float *down, const float *weights, const uint32_t *position,
                     const float *shared, const float *gate, int hidden, int used, int tokens,
                     int identity, float *out) {
    for (int t = 0; t < tokens; t++)
        for (int i = 0; i < hidden; i++) {
            float acc = 0.0f;
            for (int s = 0; s < used; s++) {
                uint32_t r = (uint32_t)(t * used + s);
                uint32_t row = identity ? r : position[r];
                float p = weights[r] * down[(size_t)row * hidden + i];
                acc = acc + p;
            }
            float g = gate[t] * shared[(size_t)t * hidden + i];
            out[(size_t)t * hidden + i] = acc + g;
        }
}

/* out = silu(gate) * up, as the kernel writes it: x / (1 + exp(-x)) * u (hybrid.metal:1606-1613). */
void fqo_swiglu(const float *g, const float *u, size_t n, float *y) {
    for (size_t i = 0; i < n; i++) {
        float x = g[i];
        y[i] = x / (1.0f + expf(-x)) * u[i];
    }
}

/* ---------------------------------------------------------------- timed CPU baseline */

/* y = dequant(W) x for m activation rows, output rows split over `threads` host threads.  Each
 * thread dequantizes one block at a time to fp32 and accumulates in fp32 (the per-block decode of
 * the functions above, src/diffusion/tests.rs:795-864).  Used only to time the CPU path. */
typedef struct {
    int format;
    const uint8_t *W;
    size_t row0, row1, rows, cols, m;
    const float *x;
    float *y;
} gemv_job;

static void *gemv_worker(void *arg) {
    gemv_job *j = (gemv_job *)arg;
    int el, bb;
    fqo_block_layout(j->format, &el, &bb);
    size_t blocks = j->cols / (size_t)el;
    size_t row_bytes = blocks * (size_t)bb;
    float w[256];
    float acc[64];
    for (size_t r = j->row0; r < j->row1; r++) {
        const uint8_t *row = j->W + r * row_bytes;
        for (size_t i = 0; i < j->m; i++) acc[i] = 0.0f;
        for (size_t b = 0; b < blocks; b++) {
            fqo_dequant(j->format, row + b * (size_t)bb, 1, w);
            for (size_t i = 0; i < j->m; i++) {
                const float *xi = j->x + i * j->cols + b * (size_t)el;
                float s = 0.0f;
                for (int c = 0; c < el; c++) s += xi[c] * w[c];
                acc[i] += s;
            }
        }
        for (size_t i = 0; i < j->m; i++) j->y[i * j->rows + r] = acc[i];
    }
    return NULL;
}

int fqo_gemv_threads(int format, const uint8_t *W, size_t rows, size_t cols, const float *x,
                     size_t m, int threads, float *y) {
    int el, bb;
    if (fqo_block_layout(format, &el, &bb) || cols % (size_t)el || m > 64 || threads < 1) return -1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    gemv_job jobs[256];
    size_t per = (rows + (size_t)threads - 1) / (size_t)threads;
    int started = 0;
    for (int t = 0; t < threads; t++) {
        size_t r0 = (size_t)t * per, r1 = r0 + per;
        if (r0 >= rows) break;
        if (r1 > rows) r1 = rows;
        jobs[t] = (gemv_job){format, W, r0, r1, rows, cols, m, x, y};
        if (pthread_create(&tid[t], NULL, gemv_worker, &jobs[t])) return -3;
        started++;
    }
    for (int t = 0; t < started; t++) pthread_join(tid[t], NULL);
    return 0;
}
