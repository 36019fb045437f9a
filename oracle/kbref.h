/*
 * kbref — CPU oracle for the BitLinear / QuatLinear forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in plain C, the arithmetic
 * of KORE's CPU implementation of the quantized-linear forward so that the
 * CUDA kernels can be checked against it.  Nothing in the shipped package may
 * call it; only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark load it.
 *
 * Parity status: the reference is Rust and cannot be compiled in an image
 * without a Rust toolchain, so this restatement is pinned against the known
 * answers written in the reference's own unit tests (byte 121 for five zero
 * trits, the 0..242 round trip, the exact matmul answers 10 / 4 / -3 / 24,48 /
 * 0,12 ...), not against outputs of the reference binary.
 *
 * Two levels are provided:
 *   R  — reference-faithful: f32 activations, f32 sequential accumulation,
 *        per-row absmax ternary quantiser, base-243 wire format.
 *   Q  — the W2A8 integer path the accelerated kernels implement: per-token
 *        absmax int8 activations, int32 accumulation, fixed-order f32 epilogue.
 *        (Its activation quantiser and the per-tensor absmean weight quantiser
 *        are defined by the benchmark specification, not by the reference.)
 *
 * Orientation follows the reference kernels: M = out_features (weight rows),
 * K = in_features, N = tokens.  "b" is [K,N], "c" is [M,N]; the module-level
 * functions take x as [N,K] and return y as [N,M].
 */
#ifndef KBREF_H
#define KBREF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (mirror KoreError variants used on this path) */
#define KBREF_OK 0
#define KBREF_ERR_SHAPE 1   /* KoreError::ShapeMismatch   */
#define KBREF_ERR_STORAGE 2 /* KoreError::StorageError    */

/* ---- codecs: crates/kore-btes/src/encoder.rs ---- */
uint8_t kbref_encode_trits5(const int8_t trits[5]);              /* :73-86  */
void kbref_decode_trits5(uint8_t byte, int8_t trits[5]);         /* :50-70,89-95 */
uint8_t kbref_pack_quats4(const uint8_t codes[4]);               /* :98-100 */
void kbref_unpack_quats4(uint8_t byte, uint8_t codes[4]);        /* :103-110 */
float kbref_quat_value(uint8_t code);                            /* :27-34 */
/* whole-slice packers: crates/kore-btes/src/packing.rs (pad last block with Zero / code 0) */
size_t kbref_pack_ternary(const int8_t *trits, size_t n, uint8_t *out);
size_t kbref_pack_quaternary(const uint8_t *codes, size_t n, uint8_t *out);

/* ---- slice quantisers: crates/kore-btes/src/quantize.rs:8-53 ---- */
float kbref_quantize_ternary(const float *w, size_t n, float threshold, int8_t *trits);
float kbref_quantize_quaternary(const float *w, size_t n, uint8_t *codes);

/* ---- weight packers ---- */
/* crates/kore-kernels/src/cpu_ternary_matmul.rs:198-240 */
void kbref_pack_weights_ternary(const float *w, size_t m, size_t k, float threshold,
                                uint8_t *packed /*[m*ceil(k/5)]*/, float *scales /*[m]*/);
/* crates/kore-kernels/src/cpu_quat_matmul.rs:174-214 */
void kbref_pack_weights_quaternary(const float *w, size_t m, size_t k,
                                   uint8_t *packed /*[m*ceil(k/4)]*/, float *scales /*[m]*/);
/* benchmark-specified absmean ternariser: s = mean|W| (f64: each row summed in
 * ascending k, then rows summed in ascending m), t = clamp(rne(w/s),-1,1),
 * scales[m] = s for every row; packed as base-243 like the reference. */
void kbref_pack_weights_ternary_absmean(const float *w, size_t m, size_t k,
                                        uint8_t *packed, float *scales);

/* ---- R level matmuls ---- */
/* crates/kore-kernels/src/cpu_ternary_matmul.rs:29-124 ; threads<=1 = serial,
 * otherwise rows are spread over `threads` workers when m >= 16 (rayon rule :19,66). */
int kbref_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                         size_t scales_len, const float *b, float *c, size_t m, size_t n,
                         size_t k, int threads);
/* crates/kore-kernels/src/cpu_quat_matmul.rs:22-108 (scalar path; use_fma=1 mimics the
 * fused multiply-add of the AVX2 path :153 for full 8-column blocks) */
int kbref_quat_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                      size_t scales_len, const float *b, float *c, size_t m, size_t n,
                      size_t k, int use_fma);
/* crates/kore-kernels/src/cpu_ternary_matmul.rs:131-193 */
int kbref_ternary_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                                 const uint8_t *b_packed, size_t b_len, const float *b_scales,
                                 float *c, size_t m, size_t n, size_t k);
/* scale-after-sum statements of the same op:
 * crates/kore-edge/src/ops/matmul.rs:49-93,101-142 and
 * crates/kore-kernels/src/cuda/kernels/dequant_matmul.cu:34-92 */
void kbref_edge_matmul_ternary(const uint8_t *a_packed, const float *a_scales, const float *b,
                               float *c, size_t m, size_t n, size_t k);
void kbref_edge_matmul_quaternary(const uint8_t *a_packed, const float *a_scales,
                                  const float *b, float *c, size_t m, size_t n, size_t k);

/* ---- module level: crates/kore-nn/src/bit_linear.rs:175-237, quat_linear.rs:245-319 ----
 * x is [n_tokens, in_dim]; in_dim must equal k or KBREF_ERR_SHAPE is returned. */
int kbref_bitlinear_forward(const uint8_t *packed, const float *scales, const float *bias,
                            size_t m, size_t k, const float *x, size_t n_tokens, size_t in_dim,
                            float *y, int threads);
int kbref_quatlinear_forward(const uint8_t *packed, const float *scales, const float *bias,
                             size_t m, size_t k, const float *x, size_t n_tokens,
                             size_t in_dim, float *y);
/* bit_linear.rs:145-167 / quat_linear.rs:134-157 */
void kbref_dequantize_ternary(const uint8_t *packed, const float *scales, size_t m, size_t k,
                              float *w);
void kbref_dequantize_quaternary(const uint8_t *packed, const float *scales, size_t m, size_t k,
                                 float *w);

/* ---- Q level (W2A8) ---- */
/* per-token absmax int8: s = max|x|/127 (1.0 if max < 1e-8), q = clamp(rne(x/s),-127,127);
 * xq row stride = ldq (>= k, tail zero-filled); sumq[n] = sum of the row's q. */
void kbref_quantize_act_i8(const float *x, size_t n_tokens, size_t k, int8_t *xq, size_t ldq,
                           float *sx, int32_t *sumq);
/* integer weights decoded from the wire format: kind 0 = ternary base-243, 1 = quaternary */
void kbref_decode_weights_i8(int kind, const uint8_t *packed, size_t m, size_t k, int8_t *w);
/* acc[n,m] = sum_k w[m,k]*xq[n,k]  (int32), threads as above */
void kbref_acc_i32(const int8_t *w, size_t m, size_t k, const int8_t *xq, size_t ldq,
                   size_t n_tokens, int32_t *acc, int threads);
/* y[n,m] = (float(acc)*sw[m])*sx[n] (+ bias[m]) — two separately rounded multiplies */
void kbref_dequant_epilogue(const int32_t *acc, const float *sw, const float *sx,
                            const float *bias, size_t n_tokens, size_t m, float *y);
/* whole Q forward from wire-format weights; acc_out may be NULL */
int kbref_q_forward(int kind, const uint8_t *packed, const float *scales, const float *bias,
                    size_t m, size_t k, const float *x, size_t n_tokens, float *y,
                    int32_t *acc_out, int threads);

int kbref_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
