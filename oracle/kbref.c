/*
 * kbref.c — CPU oracle (test infrastructure, never on the product path).
 * See kbref.h for scope and parity status.  Build with -ffp-contract=off so
 * every "mul then add" below stays two roundings, as in the reference's scalar
 * Rust code.
 */
#include "kbref.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ codecs */

/* crates/kore-btes/src/encoder.rs:73-86 — digit = trit+1, trit 0 least significant */
uint8_t kbref_encode_trits5(const int8_t trits[5]) {
    unsigned val = 0, mult = 1;
    for (int i = 0; i < 5; ++i) {
        unsigned digit = (unsigned)(trits[i] + 1);
        val += digit * mult;
        mult *= 3;
    }
    return (uint8_t)val;
}

/* encoder.rs:50-70 (LUT) and :89-95 (bytes >= 243 decode to five zeros) */
void kbref_decode_trits5(uint8_t byte, int8_t trits[5]) {
    if (byte >= 243) {
        memset(trits, 0, 5);
        return;
    }
    unsigned v = byte;
    for (int j = 0; j < 5; ++j) {
        trits[j] = (int8_t)((int)(v % 3) - 1);
        v /= 3;
    }
}

/* encoder.rs:98-100 — element i in bits [2i+1:2i] */
uint8_t kbref_pack_quats4(const uint8_t c[4]) {
    return (uint8_t)((c[0] & 3) | ((c[1] & 3) << 2) | ((c[2] & 3) << 4) | ((c[3] & 3) << 6));
}

void kbref_unpack_quats4(uint8_t byte, uint8_t c[4]) {
    for (int i = 0; i < 4; ++i) c[i] = (uint8_t)((byte >> (2 * i)) & 3);
}

/* encoder.rs:27-34 and cpu_quat_matmul.rs:11 */
float kbref_quat_value(uint8_t code) {
    static const float v[4] = {-3.0f, -1.0f, 1.0f, 3.0f};
    return v[code & 3];
}

/* crates/kore-btes/src/packing.rs:7-20 — last block padded with Zero */
size_t kbref_pack_ternary(const int8_t *trits, size_t n, uint8_t *out) {
    size_t nb = (n + 4) / 5;
    for (size_t b = 0; b < nb; ++b) {
        int8_t blk[5] = {0, 0, 0, 0, 0};
        for (size_t i = 0; i < 5 && b * 5 + i < n; ++i) blk[i] = trits[b * 5 + i];
        out[b] = kbref_encode_trits5(blk);
    }
    return nb;
}

/* packing.rs:40-53 — last block padded with Pos1 (code 2) */
size_t kbref_pack_quaternary(const uint8_t *codes, size_t n, uint8_t *out) {
    size_t nb = (n + 3) / 4;
    for (size_t b = 0; b < nb; ++b) {
        uint8_t blk[4] = {2, 2, 2, 2};
        for (size_t i = 0; i < 4 && b * 4 + i < n; ++i) blk[i] = codes[b * 4 + i];
        out[b] = kbref_pack_quats4(blk);
    }
    return nb;
}

/* -------------------------------------------------------------- quantisers */

static float absmax_f32(const float *w, size_t n) {
    float m = 0.0f; /* fold(0.0, f32::max): NaNs are ignored like fmaxf */
    for (size_t i = 0; i < n; ++i) m = fmaxf(m, fabsf(w[i]));
    return m;
}

static int8_t trit_of(float w, float scale, float thr) {
    float nrm = w / scale;
    if (nrm > thr) return 1;
    if (nrm < -thr) return -1;
    return 0;
}

static uint8_t quat_code_of(float w, float scale) {
    float nrm = w / scale;
    if (nrm < -2.0f) return 0;
    if (nrm < 0.0f) return 1;
    if (nrm < 2.0f) return 2;
    return 3;
}

/* crates/kore-btes/src/quantize.rs:8-27 */
float kbref_quantize_ternary(const float *w, size_t n, float thr, int8_t *trits) {
    float am = absmax_f32(w, n);
    float scale = am < 1e-8f ? 1.0f : am;
    for (size_t i = 0; i < n; ++i) trits[i] = trit_of(w[i], scale, thr);
    return scale;
}

/* quantize.rs:32-53 */
float kbref_quantize_quaternary(const float *w, size_t n, uint8_t *codes) {
    float am = absmax_f32(w, n);
    float scale = am < 1e-8f ? 1.0f : am / 3.0f;
    for (size_t i = 0; i < n; ++i) codes[i] = quat_code_of(w[i], scale);
    return scale;
}

/* crates/kore-kernels/src/cpu_ternary_matmul.rs:198-240 */
void kbref_pack_weights_ternary(const float *w, size_t m, size_t k, float thr, uint8_t *packed,
                                float *scales) {
    size_t kp = (k + 4) / 5;
    int8_t *tr = (int8_t *)malloc(k + 5);
    for (size_t r = 0; r < m; ++r) {
        scales[r] = kbref_quantize_ternary(w + r * k, k, thr, tr);
        kbref_pack_ternary(tr, k, packed + r * kp);
    }
    free(tr);
}

/* crates/kore-kernels/src/cpu_quat_matmul.rs:174-214 — unused tail slots stay code 0 */
void kbref_pack_weights_quaternary(const float *w, size_t m, size_t k, uint8_t *packed,
                                   float *scales) {
    size_t kp = (k + 3) / 4;
    for (size_t r = 0; r < m; ++r) {
        const float *row = w + r * k;
        float am = absmax_f32(row, k);
        float scale = am < 1e-8f ? 1.0f : am / 3.0f;
        scales[r] = scale;
        for (size_t b = 0; b < kp; ++b) {
            uint8_t byte = 0;
            for (size_t i = 0; i < 4; ++i) {
                size_t ki = b * 4 + i;
                if (ki >= k) break;
                byte |= (uint8_t)(quat_code_of(row[ki], scale) << (2 * i));
            }
            packed[r * kp + b] = byte;
        }
    }
}

/* Benchmark-specified absmean ternariser (not in the reference). */
void kbref_pack_weights_ternary_absmean(const float *w, size_t m, size_t k, uint8_t *packed,
                                        float *scales) {
    size_t kp = (k + 4) / 5;
    double total = 0.0;
    for (size_t r = 0; r < m; ++r) {
        double rs = 0.0;
        for (size_t i = 0; i < k; ++i) rs += (double)fabsf(w[r * k + i]);
        total += rs;
    }
    float s = (float)(total / (double)(m * k));
    if (s < 1e-8f) s = 1.0f;
    int8_t *tr = (int8_t *)malloc(k + 5);
    for (size_t r = 0; r < m; ++r) {
        for (size_t i = 0; i < k; ++i) {
            float q = rintf(w[r * k + i] / s); /* round half to even */
            tr[i] = (int8_t)(q > 1.0f ? 1 : (q < -1.0f ? -1 : (int)q));
        }
        kbref_pack_ternary(tr, k, packed + r * kp);
        scales[r] = s;
    }
    free(tr);
}

/* ------------------------------------------------------------- R matmuls */

static void unpack_row_trits(const uint8_t *row, size_t kp, size_t k, int8_t *out) {
    /* cpu_ternary_matmul.rs:91-101 — decode all bytes, truncate to k */
    int8_t t5[5];
    size_t pos = 0;
    for (size_t b = 0; b < kp; ++b) {
        kbref_decode_trits5(row[b], t5);
        for (int j = 0; j < 5 && pos < k; ++j) out[pos++] = t5[j];
    }
}

static void ternary_compute_row(const int8_t *trits, const float *b, float *c_row, float scale,
                                size_t n, size_t k) {
    /* cpu_ternary_matmul.rs:105-124 — zero trits skipped, k ascending, scale after sum */
    for (size_t ki = 0; ki < k; ++ki) {
        int8_t t = trits[ki];
        if (t == 0) continue;
        float tf = (float)t;
        const float *b_row = b + ki * n;
        for (size_t col = 0; col < n; ++col) c_row[col] += tf * b_row[col];
    }
    for (size_t col = 0; col < n; ++col) c_row[col] *= scale;
}

int kbref_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                         size_t scales_len, const float *b, float *c, size_t m, size_t n,
                         size_t k, int threads) {
    size_t kp = (k + 4) / 5;
    if (a_len < m * kp) return KBREF_ERR_STORAGE;   /* :44-50 */
    if (scales_len < m) return KBREF_ERR_STORAGE;   /* :51-57 */
    memset(c, 0, m * n * sizeof(float));
    int par = (m >= 16) && threads > 1;             /* PAR_ROW_THRESHOLD :19 */
#pragma omp parallel num_threads(par ? threads : 1)
    {
        int8_t *tr = (int8_t *)malloc(k + 5);
#pragma omp for schedule(dynamic, 8)
        for (long r = 0; r < (long)m; ++r) {
            unpack_row_trits(a_packed + (size_t)r * kp, kp, k, tr);
            ternary_compute_row(tr, b, c + (size_t)r * n, a_scales[r], n, k);
        }
        free(tr);
    }
    return KBREF_OK;
}

int kbref_quat_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                      size_t scales_len, const float *b, float *c, size_t m, size_t n,
                      size_t k, int use_fma) {
    size_t kp = (k + 3) / 4;
    if (a_len < m * kp) return KBREF_ERR_STORAGE;   /* cpu_quat_matmul.rs:37-43 */
    if (scales_len < m) return KBREF_ERR_STORAGE;   /* :44-50 */
    memset(c, 0, m * n * sizeof(float));
    float *q = (float *)malloc((k + 4) * sizeof(float));
    for (size_t r = 0; r < m; ++r) {                /* single-threaded, :84 */
        float scale = a_scales[r];
        const uint8_t *a_row = a_packed + r * kp;
        float *c_row = c + r * n;
        for (size_t bi = 0; bi < kp; ++bi)
            for (int i = 0; i < 4; ++i) q[bi * 4 + i] = kbref_quat_value((a_row[bi] >> (2 * i)) & 3);
        for (size_t ki = 0; ki < k; ++ki) {
            float w = q[ki] * scale;                /* scale folded in first, :101 */
            const float *b_row = b + ki * n;
            if (!use_fma) {
                for (size_t col = 0; col < n; ++col) c_row[col] += w * b_row[col];
            } else {
                /* AVX2 path :133-166: full blocks of 8 columns use fused multiply-add,
                 * a trailing partial block uses mul-then-add */
                size_t full = n - (n % 8);
                for (size_t col = 0; col < full; ++col) c_row[col] = fmaf(w, b_row[col], c_row[col]);
                for (size_t col = full; col < n; ++col) c_row[col] += w * b_row[col];
            }
        }
    }
    free(q);
    return KBREF_OK;
}

int kbref_ternary_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                                 const uint8_t *b_packed, size_t b_len, const float *b_scales,
                                 float *c, size_t m, size_t n, size_t k) {
    size_t kp = (k + 4) / 5;
    if (a_len < m * kp || b_len < n * kp) return KBREF_ERR_STORAGE; /* :142-146 */
    int8_t *ta = (int8_t *)malloc(m * k + 5), *tb = (int8_t *)malloc(n * k + 5);
    for (size_t r = 0; r < m; ++r) unpack_row_trits(a_packed + r * kp, kp, k, ta + r * k);
    for (size_t r = 0; r < n; ++r) unpack_row_trits(b_packed + r * kp, kp, k, tb + r * k);
    for (size_t r = 0; r < m; ++r)
        for (size_t col = 0; col < n; ++col) {
            int64_t acc = 0; /* TernaryWord64::dot summed over words == plain integer dot */
            for (size_t i = 0; i < k; ++i) acc += (int64_t)ta[r * k + i] * tb[col * k + i];
            c[r * n + col] = (float)acc * a_scales[r] * b_scales[col]; /* :188 */
        }
    free(ta);
    free(tb);
    return KBREF_OK;
}

void kbref_edge_matmul_ternary(const uint8_t *a_packed, const float *a_scales, const float *b,
                               float *c, size_t m, size_t n, size_t k) {
    /* crates/kore-edge/src/ops/matmul.rs:49-93 — same arithmetic as ternary_matmul */
    size_t kp = (k + 4) / 5;
    kbref_ternary_matmul(a_packed, m * kp, a_scales, m, b, c, m, n, k, 1);
}

void kbref_edge_matmul_quaternary(const uint8_t *a_packed, const float *a_scales,
                                  const float *b, float *c, size_t m, size_t n, size_t k) {
    /* crates/kore-edge/src/ops/matmul.rs:101-142 and dequant_matmul.cu:34-92:
     * unscaled sum first, then one multiply by the row scale */
    size_t kp = (k + 3) / 4;
    memset(c, 0, m * n * sizeof(float));
    for (size_t r = 0; r < m; ++r) {
        const uint8_t *a_row = a_packed + r * kp;
        float *c_row = c + r * n;
        for (size_t ki = 0; ki < k; ++ki) {
            float w = kbref_quat_value((a_row[ki / 4] >> (2 * (ki % 4))) & 3);
            const float *b_row = b + ki * n;
            for (size_t col = 0; col < n; ++col) c_row[col] += w * b_row[col];
        }
        for (size_t col = 0; col < n; ++col) c_row[col] *= a_scales[r];
    }
}

/* ------------------------------------------------------------ module level */

static void transpose_f32(const float *src, size_t rows, size_t cols, float *dst) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t c2 = 0; c2 < cols; ++c2) dst[c2 * rows + r] = src[r * cols + c2];
}

static int linear_forward(int kind, const uint8_t *packed, const float *scales,
                          const float *bias, size_t m, size_t k, const float *x, size_t nt,
                          size_t in_dim, float *y, int threads) {
    if (in_dim != k) return KBREF_ERR_SHAPE;        /* bit_linear.rs:179-184 */
    float *xt = (float *)malloc((nt * k + 1) * sizeof(float));
    float *ct = (float *)malloc((m * nt + 1) * sizeof(float));
    transpose_f32(x, nt, k, xt);                    /* :207 input^T [K, batch] */
    int rc;
    if (kind == 0)
        rc = kbref_ternary_matmul(packed, m * ((k + 4) / 5), scales, m, xt, ct, m, nt, k, threads);
    else
        rc = kbref_quat_matmul(packed, m * ((k + 3) / 4), scales, m, xt, ct, m, nt, k, 0);
    if (rc == KBREF_OK) {
        transpose_f32(ct, m, nt, y);                /* :219 back to [batch, out] */
        if (bias)                                   /* :222-224 broadcast add */
            for (size_t t = 0; t < nt; ++t)
                for (size_t r = 0; r < m; ++r) y[t * m + r] += bias[r];
    }
    free(xt);
    free(ct);
    return rc;
}

int kbref_bitlinear_forward(const uint8_t *packed, const float *scales, const float *bias,
                            size_t m, size_t k, const float *x, size_t nt, size_t in_dim,
                            float *y, int threads) {
    return linear_forward(0, packed, scales, bias, m, k, x, nt, in_dim, y, threads);
}

int kbref_quatlinear_forward(const uint8_t *packed, const float *scales, const float *bias,
                             size_t m, size_t k, const float *x, size_t nt, size_t in_dim,
                             float *y) {
    return linear_forward(1, packed, scales, bias, m, k, x, nt, in_dim, y, 1);
}

void kbref_dequantize_ternary(const uint8_t *packed, const float *scales, size_t m, size_t k,
                              float *w) {
    size_t kp = (k + 4) / 5;
    int8_t *tr = (int8_t *)malloc(k + 5);
    for (size_t r = 0; r < m; ++r) {
        unpack_row_trits(packed + r * kp, kp, k, tr);
        for (size_t i = 0; i < k; ++i) w[r * k + i] = (float)tr[i] * scales[r];
    }
    free(tr);
}

void kbref_dequantize_quaternary(const uint8_t *packed, const float *scales, size_t m, size_t k,
                                 float *w) {
    size_t kp = (k + 3) / 4;
    for (size_t r = 0; r < m; ++r)
        for (size_t i = 0; i < k; ++i)
            w[r * k + i] = kbref_quat_value((packed[r * kp + i / 4] >> (2 * (i % 4))) & 3) * scales[r];
}

/* ----------------------------------------------------------------- Q level */

void kbref_quantize_act_i8(const float *x, size_t nt, size_t k, int8_t *xq, size_t ldq,
                           float *sx, int32_t *sumq) {
    for (size_t t = 0; t < nt; ++t) {
        const float *row = x + t * k;
        float am = absmax_f32(row, k);
        float s = am < 1e-8f ? 1.0f : am / 127.0f;
        int32_t sum = 0;
        for (size_t i = 0; i < k; ++i) {
            float q = rintf(row[i] / s);
            if (q > 127.0f) q = 127.0f;
            if (q < -127.0f) q = -127.0f;
            if (q != q) q = 0.0f;
            xq[t * ldq + i] = (int8_t)q;
            sum += (int32_t)q;
        }
        for (size_t i = k; i < ldq; ++i) xq[t * ldq + i] = 0;
        sx[t] = s;
        if (sumq) sumq[t] = sum;
    }
}

void kbref_decode_weights_i8(int kind, const uint8_t *packed, size_t m, size_t k, int8_t *w) {
    if (kind == 0) {
        size_t kp = (k + 4) / 5;
        for (size_t r = 0; r < m; ++r) unpack_row_trits(packed + r * kp, kp, k, w + r * k);
    } else {
        size_t kp = (k + 3) / 4;
        for (size_t r = 0; r < m; ++r)
            for (size_t i = 0; i < k; ++i)
                w[r * k + i] = (int8_t)(2 * (int)((packed[r * kp + i / 4] >> (2 * (i % 4))) & 3) - 3);
    }
}

void kbref_acc_i32(const int8_t *w, size_t m, size_t k, const int8_t *xq, size_t ldq, size_t nt,
                   int32_t *acc, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
    for (long r = 0; r < (long)m; ++r) {
        const int8_t *wr = w + (size_t)r * k;
        for (size_t t = 0; t < nt; ++t) {
            const int8_t *xr = xq + t * ldq;
            int32_t a = 0;
            for (size_t i = 0; i < k; ++i) a += (int32_t)wr[i] * (int32_t)xr[i];
            acc[t * m + (size_t)r] = a;
        }
    }
}

void kbref_dequant_epilogue(const int32_t *acc, const float *sw, const float *sx,
                            const float *bias, size_t nt, size_t m, float *y) {
    for (size_t t = 0; t < nt; ++t)
        for (size_t r = 0; r < m; ++r) {
            float v = (float)acc[t * m + r] * sw[r];
            v = v * sx[t];
            if (bias) v = v + bias[r];
            y[t * m + r] = v;
        }
}

int kbref_q_forward(int kind, const uint8_t *packed, const float *scales, const float *bias,
                    size_t m, size_t k, const float *x, size_t nt, float *y, int32_t *acc_out,
                    int threads) {
    int8_t *w = (int8_t *)malloc(m * k + 8);
    int8_t *xq = (int8_t *)malloc(nt * k + 8);
    float *sx = (float *)malloc((nt + 1) * sizeof(float));
    int32_t *acc = acc_out ? acc_out : (int32_t *)malloc((nt * m + 1) * sizeof(int32_t));
    kbref_decode_weights_i8(kind, packed, m, k, w);
    kbref_quantize_act_i8(x, nt, k, xq, k, sx, NULL);
    kbref_acc_i32(w, m, k, xq, k, nt, acc, threads);
    kbref_dequant_epilogue(acc, scales, sx, bias, nt, m, y);
    if (!acc_out) free(acc);
    free(w);
    free(xq);
    free(sx);
    return KBREF_OK;
}

int kbref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
