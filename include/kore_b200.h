/*
 * kore_b200 — C ABI of the B200-native BitLinear / QuatLinear forward path.
 *
 * This is the boundary a KORE maintainer binds from Rust (or any FFI): plain
 * pointers and sizes, integer status codes, an opaque weight handle with a paired
 * destroy.  Each entry point names the KORE interface it stands in for (path inside
 * the KORE source tree : lines).
 *
 * Orientation follows KORE's kernels: M = out_features (weight rows),
 * K = in_features, N = tokens.  Module-shaped calls take x as [N,K] and write
 * y as [N,M]; the kernel-shaped one-shots take b as [K,N] and write c as [M,N].
 *
 * Arithmetic (W2A8): activations are quantised per token to int8 by absmax
 * (s = max|x|/127, or 1.0 when max|x| < 1e-8; q = clamp(rne(x/s), -127, 127)),
 * accumulated against the 2-bit weights in int32, and dequantised as
 * y = (float(acc) * w_scale[m]) * s[n] (+ bias[m]) with separately rounded
 * multiplies.  There is no CPU fallback anywhere behind this header: every entry
 * point that computes runs CUDA kernels for sm_100a or fails with a status code.
 *
 * Threading: a handle is immutable after creation; any number of host threads may
 * call the forward entry points on one handle concurrently, each on its own stream.
 * Per-call scratch comes from the stream-ordered allocator unless the caller passes
 * a workspace.  Calls return after enqueueing work on the given stream unless they
 * take host pointers, in which case they synchronise before returning.
 */
#ifndef KORE_B200_H
#define KORE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  Names follow KoreError (crates/kore-core/src/error.rs:6-51) and
 * CudaError (crates/kore-kernels/src/cuda/context.rs:58-80). */
enum {
    KB_OK = 0,
    KB_ERR_SHAPE = 1,       /* KoreError::ShapeMismatch                      */
    KB_ERR_STORAGE = 2,     /* KoreError::StorageError ("... too small")     */
    KB_ERR_DTYPE = 3,       /* KoreError::UnsupportedDType                   */
    KB_ERR_CUDA = 4,        /* CudaError::{DeviceInit,LaunchError,MemoryError} */
    KB_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up             */
    KB_ERR_BAD_HANDLE = 7,  /* null or destroyed handle                      */
    KB_ERR_INVALID = 8,     /* null pointer / unknown enum / zero dimension  */
    KB_ERR_UNSUPPORTED = 9  /* shape outside what the chosen kernel accepts   */
};

enum { KB_TERNARY = 0, KB_QUATERNARY = 1 };

/* weight quantiser used by *_from_f32 */
enum {
    KB_QUANT_REFERENCE = 0, /* KORE's: per-row absmax (ternary: +-1 beyond threshold; quaternary: absmax/3) */
    KB_QUANT_ABSMEAN = 1    /* ternary only: per-tensor s = mean|W|, clamp(rne(W/s),-1,1) */
};

/* kernel choice for the forward entry points that take `path` (AUTO picks by N).
 * KB_PATH_GEMV_SHARED is the GEMV launched with about half the CTAs (two row groups per warp):
 * a single launch finishes later, but independent layers issued on several streams share the
 * SMs better and their aggregate bandwidth is higher.  Use it when several GEMVs are in
 * flight at once; use KB_PATH_GEMV (or AUTO) for a chain of dependent layers.
 * KB_PATH_GEMV_MMA is the small-batch kernel (up to 32 tokens whose int8 activations fit in
 * shared memory): weights stream global -> registers -> warp-level int8 MMA.
 * KB_PATH_GEMV_STREAM is the streaming decode kernel (1..32 tokens): every warp runs its own ring
 * of bulk-copied 16-row stages in shared memory and contracts them with the warp-level int8 MMA. */
enum { KB_PATH_AUTO = 0, KB_PATH_GEMV = 1, KB_PATH_GEMM_TC = 2, KB_PATH_GEMV_SHARED = 3, KB_PATH_GEMV_MMA = 4, KB_PATH_GEMV_STREAM = 5 };

/* epilogue activation of kb_linear_forward_act */
enum { KB_ACT_NONE = 0, KB_ACT_RELU = 1 };

typedef struct kb_linear kb_linear; /* opaque: device-resident 2-bit weights + scales + bias */
typedef struct kb_linear_group kb_linear_group; /* opaque: a set of same-shaped layers run in one launch */
typedef void *kb_stream;            /* a cudaStream_t; NULL = the legacy default stream */

/* ---- library ---- */
const char *kb_version(void);
/* Thread-local description of the last failure on the calling thread, worded like
 * the KoreError it mirrors (e.g. "a_packed too small: need 52 bytes, got 51"). */
const char *kb_last_error(void);
int kb_device_count(int *count);

/* ---- weights: construction (one-time upload + repack into the device layout) ---- */

/* Takes BitLinear::packed_weights()/scales() or QuatLinear::packed_weights()/scales()
 * unchanged: ternary base-243 [M,ceil(K/5)] or quaternary 2-bit LSB-first
 * [M,ceil(K/4)], f32 per-row scales [M], optional bias [M] (host pointers).
 * Stands in for the per-call upload in QuatLinear::try_cuda_forward
 * (crates/kore-nn/src/quat_linear.rs:166-197) and the per-call row decode in
 * ternary_matmul (crates/kore-kernels/src/cpu_ternary_matmul.rs:59-62). */
int kb_linear_create_from_ref_packed(int kind, const uint8_t *packed, size_t packed_len,
                                     const float *scales, size_t scales_len, const float *bias,
                                     size_t m, size_t k, int device, kb_linear **out);

/* BitLinear::new / QuatLinear::new (crates/kore-nn/src/bit_linear.rs:48-77,
 * quat_linear.rs:46-73): quantise f32 weights [M,K] (host) on the device. */
int kb_linear_create_from_f32(int kind, int quantiser, const float *w, const float *bias, size_t m,
                              size_t k, float threshold, int device, kb_linear **out);

/* Null-tolerant, like the frees of crates/kore-edge/src/ffi.rs:131-161. */
void kb_linear_destroy(kb_linear *h);

/* in_features()/out_features()/weight_memory_bytes() (bit_linear.rs:104-132);
 * weight_bytes reports the reference's own formula: wire-format bytes + 4*M. */
int kb_linear_info(const kb_linear *h, size_t *m, size_t *k, int *kind, int *device,
                   size_t *weight_bytes);
/* scales() (bit_linear.rs:124-127): copies the M per-row scales to the host. */
int kb_linear_scales(const kb_linear *h, float *scales, size_t scales_len);
/* packed_weights() (bit_linear.rs:119-122): re-encodes the device layout into the
 * reference wire format on the device and copies it to the host. */
int kb_linear_packed_weights(const kb_linear *h, uint8_t *packed, size_t packed_len);
/* dequantize_weights() (bit_linear.rs:145-167, quat_linear.rs:134-157): f32 [M,K] to the host. */
int kb_linear_dequantize_weights(const kb_linear *h, float *w, size_t w_len);

/* ---- activations ---- */

/* Fused per-token absmax int8 quantiser (device pointers).  xq is [N,ldq] with
 * ldq >= K, ldq % 16 == 0, columns K..ldq-1 written as zero; sx[N] scales;
 * sumq[N] = sum of each row's codes (nullable).  No counterpart in the reference,
 * whose activations stay f32 (cpu_ternary_matmul.rs:37-40). */
int kb_quantize_act_i8(const float *x, size_t n, size_t k, int8_t *xq, size_t ldq, float *sx,
                       int32_t *sumq, kb_stream stream);
/* Leading dimension the forward entry points expect for pre-quantised activations. */
size_t kb_act_ld(size_t k);

/* ---- forward (device pointers) ---- */

/* Module::forward for BitLinear / QuatLinear (bit_linear.rs:175-237,
 * quat_linear.rs:245-319): x [N,K] f32 -> y [N,M] f32, bias added when present.
 * Picks the decode GEMV for small N and the tcgen05 GEMM otherwise. */
int kb_linear_forward(const kb_linear *h, const float *x, size_t n, float *y, kb_stream stream);

/* Same with an explicit kernel choice, an optional raw-accumulator output
 * acc [N,M] int32 (nullable) and an optional caller workspace (nullable; size from
 * kb_linear_workspace_bytes).  in_dim is checked against K like the ShapeMismatch
 * test of bit_linear.rs:179-184.  ldy is the row stride of y and acc in elements
 * (0 = M), which lets a column-sharded layer write straight into its slice. */
int kb_linear_forward_ex(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y,
                         size_t ldy, int32_t *acc, int path, void *workspace,
                         size_t workspace_bytes, kb_stream stream);
size_t kb_linear_workspace_bytes(const kb_linear *h, size_t n);

/* Forward with an activation in the epilogue: y = act(dequant(acc) + bias), act = KB_ACT_RELU
 * gives max(., 0).  The layer-shaped form of the reference's fused bias + ReLU variant of its
 * dequantising matmul (crates/kore-kernels/src/cuda/ops.rs:828-878, kernel
 * cuda/kernels/dequant_matmul.cu:210-264).  bias is the handle's own, one value per output
 * feature.  Other arguments as kb_linear_forward_ex. */
int kb_linear_forward_act(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y,
                          size_t ldy, int act, int path, void *workspace, size_t workspace_bytes,
                          kb_stream stream);

/* Forward from activations the caller already quantised (kb_quantize_act_i8 layout,
 * ldq = kb_act_ld(K)).  y and acc are each nullable (not both). */
int kb_linear_forward_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx,
                         const int32_t *sumq, size_t n, float *y, size_t ldy, int32_t *acc,
                         int path, kb_stream stream);

/* Forward for a decoder step: input either f32 x [N,K] or pre-quantised (xq, sx, sumq),
 * and an optional residual resid [N,ldy] (may be y itself) added after the bias:
 * y = ((float(acc) * w_scale) * s + bias) + resid.  Stands in for the project() +
 * residual_add() pairs of the reference's decoder loop
 * (crates/kore-edge/src/runtime.rs:197-212,254-265).  With f32 input and the GEMM path a
 * caller workspace (kb_linear_workspace_bytes) is required; nothing is allocated per call (the
 * medium-batch GEMM creates one scratch buffer per stream the first time it splits K, see
 * kb_linear_forward_static for the entry that never allocates). */
int kb_linear_forward_fused(const kb_linear *h, const float *x, const int8_t *xq, size_t ldq,
                            const float *sx, const int32_t *sumq, size_t n, const float *resid,
                            float *y, size_t ldy, int path, void *workspace,
                            size_t workspace_bytes, kb_stream stream);

/* ---- projections fused with their neighbours in a decode step (1..8 tokens, GEMV kernel) ----
 *
 * kb_linear_forward_rmsnorm: y = W . quantise(rmsnorm(x) * gamma) — the RMSNorm of
 * crates/kore-kernels/src/cpu_fused.rs:160-190 and the activation quantiser run in the GEMV's
 * prologue (every CTA normalises the L2-resident row itself), so norm + projection is one
 * launch.  With swiglu != 0 (1 or 2 tokens) the weight rows must alternate gate_i, up_i
 * (runtime.rs:232-252 computes the two projections separately); the epilogue writes
 * h_i = silu(gate_i) * up_i into y [N][M/2] and, when absmax_out is given, folds max|h| of each
 * token into absmax_out[N] with an atomic max — the caller keeps that word at zero beforehand.
 *
 * kb_linear_forward_scaled: the projection of f32 activations whose per-token max|x| is already
 * known (x_absmax[N], e.g. from the SwiGLU epilogue above): the prologue quantises without its
 * own reduction.  resid as in kb_linear_forward_fused.  clear_words (nullable): N floats the
 * launch sets to zero, so two absmax arrays can alternate between layers without a memset. */
int kb_linear_forward_rmsnorm(const kb_linear *h, const float *x, const float *gamma, float eps, size_t n,
                              float *y, size_t ldy, int swiglu, float *absmax_out, kb_stream stream);
int kb_linear_forward_scaled(const kb_linear *h, const float *x, const float *x_absmax, size_t n,
                             const float *resid, float *y, size_t ldy, float *clear_words, kb_stream stream);

/* ---- glue kernels of the decoder step; each ends in the per-token int8 quantiser so the
 * next projection reads codes.  Device pointers.  xn / h receive the f32 values when
 * not NULL; xq may be NULL to get only the f32 result. ---- */
/* RMSNorm (crates/kore-kernels/src/cpu_fused.rs:160-190): (x * (1/sqrt(mean(x^2)+eps))) * gamma */
int kb_rmsnorm_quant(const float *x, const float *gamma, size_t n, size_t d, float eps, float *xn,
                     int8_t *xq, size_t ldq, float *sx, int32_t *sumq, kb_stream stream);
/* SwiGLU (crates/kore-edge/src/runtime.rs:232-252, ops/activation.rs:21-26): rows of
 * gate_up are [gate(f) | up(f)] with row stride ld; h = (g / (1 + exp(-g))) * u */
int kb_swiglu_quant(const float *gate_up, size_t n, size_t f, size_t ld, float *h, int8_t *xq,
                    size_t ldq, float *sx, int32_t *sumq, kb_stream stream);
/* the same for rows that alternate gate_0, up_0, gate_1, up_1, ... (the output of a projection
 * whose weight rows are interleaved for the SwiGLU epilogue of kb_linear_forward_rmsnorm) */
int kb_swiglu_quant_pairs(const float *gate_up, size_t n, size_t f, size_t ld, float *h, int8_t *xq,
                          size_t ldq, float *sx, int32_t *sumq, kb_stream stream);
/* Half-split RoPE (crates/kore-edge/src/ops/rope.rs:9-36) on the q and k parts of rows
 * [q|k|v] with cos/sin tables [max_pos][head_dim/2]; k and v go to the caches, which are laid
 * out head-major, [sequence][n_heads][lmax][head_dim] (a head's keys are contiguous, so decode
 * attention streams them page by page); cache_rows[t] = sequence * lmax + position. */
int kb_rope_kv(const float *qkv, const int *positions, const long long *cache_rows,
               const float *cos_table, const float *sin_table, size_t n, int n_heads, int head_dim,
               int lmax, float *q_out, float *k_cache, float *v_cache, kb_stream stream);
/* Dense f32 head of a greedy decode step for up to 16 sequences (the reference's lm_head is a dense f32 matmul
 * followed by an argmax, crates/kore-edge/src/runtime.rs:283-294): logits[n][vocab] = x[n][d] . w[vocab][d]^T
 * (logits nullable), and per token an argmax key folded into keys[n] (device words, zero before the call) by
 * atomic max: the largest logit wins and, among equal ones, the lowest index.  d a multiple of 4 up to 4096. */
int kb_lm_head_argmax(const float *x, size_t n, size_t d, const float *w, size_t vocab, float *logits,
                      unsigned long long *keys, kb_stream stream);
/* End of a greedy step: tokens[t] = the index in keys[t], keys[t] = 0, and positions / lens / cache_rows (each
 * nullable) advance by one. */
int kb_decode_advance(unsigned long long *keys, size_t n, long long *tokens, int *positions, int *lens,
                      long long *cache_rows, kb_stream stream);
/* One query token per sequence against its cache [batch][n_heads][lmax][head_dim]
 * (crates/kore-edge/src/ops/attention.rs:74-135); lens[b] counts the current token. */
int kb_attn_decode(const float *q, const float *k_cache, const float *v_cache, const int *lens,
                   size_t batch, int n_heads, int head_dim, int lmax, float *out, float *scratch,
                   size_t scratch_bytes, kb_stream stream);
/* scratch (zero-initialised once by the caller, reusable across calls on one stream) lets the
 * kernel split long caches over several CTAs per head; without it one CTA serves a head. */
size_t kb_attn_decode_scratch_bytes(size_t batch, int n_heads);

/* ---- persistent decode step: one greedy step of the decoder loop of
 * crates/kore-edge/src/runtime.rs:106-294 (pre-norm, q/k/v, half-split RoPE, KV cache, causal attention,
 * output projection + residual, SwiGLU feed-forward + residual, final norm, lm_head, argmax) for one or two
 * sequences as ONE cooperative kernel: a grid of one CTA per SM walks the phases of every layer, separated by a
 * bounded device-side grid barrier, and streams the next phase's weights while it waits.  Device pointers.
 *   qkv[l]      [3d, d] rows q | k | v;  o[l] [d, d];  gate_up[l] [2f, d] rows gate_0, up_0, gate_1, ...;
 *   down[l]     [d, f] — ternary handles without bias, all on one device (borrowed: destroy the decoder first)
 *   norm1/2[l]  RMSNorm weights [d];  k_cache/v_cache[l]  [batch, n_heads, max_len, head_dim] f32
 *   embed, lm_head [vocab, d] f32 dense;  norm_f [d];  cos/sin tables [max_len, head_dim / 2]
 * kb_decoder_step consumes tokens[b] (int64) at positions[b] (cache row cache_rows[b] = b * max_len + position,
 * lens[b] = position + 1) and leaves the chosen tokens in tokens[b], the logits in logits [batch, vocab]
 * (nullable) and all four counters advanced by one.  hidden is a [batch, d] f32 work buffer of the caller. */
typedef struct kb_decoder kb_decoder;
int kb_decoder_create(const kb_linear *const *qkv, const kb_linear *const *o, const kb_linear *const *gate_up,
                      const kb_linear *const *down, const float *const *norm1, const float *const *norm2,
                      float *const *k_cache, float *const *v_cache, size_t n_layers, size_t batch,
                      size_t n_heads, size_t max_len, size_t vocab, float eps, const float *embed,
                      const float *lm_head, const float *norm_f, const float *cos_table,
                      const float *sin_table, kb_decoder **out);
void kb_decoder_destroy(kb_decoder *h);
int kb_decoder_step(kb_decoder *h, long long *tokens, int *positions, int *lens, long long *cache_rows,
                    float *hidden, float *logits, kb_stream stream);
/* 0 = clean; otherwise KB_ERR_TIMEOUT and the code of the bounded wait that gave up (the word is cleared) */
int kb_decoder_status(kb_decoder *h, kb_stream stream, int *status);

/* ---- forward (host pointers; what a Tensor-in/Tensor-out caller uses) ---- */

/* Copies x to the device, runs kb_linear_forward, copies y back, synchronises.
 * Replaces the H2D/launch/D2H sequence of quat_linear.rs:183-212. */
int kb_linear_forward_host(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y);

/* ---- forward without any allocation (device pointers) ----
 * No counterpart in the reference (its CUDA path allocates a fresh output and three
 * upload buffers on every call, quat_linear.rs:183-199, cuda/ops.rs:778-780).
 *
 * For callers that may not allocate device memory while they run — a latency-critical
 * loop with a fixed memory budget, a plugin inside a process whose own allocator has
 * claimed the GPU, an engine whose pools are frozen after start-up.  Same result as
 * kb_linear_forward, but the quantised activations live in a fixed array inside the
 * library (kb_static_scratch_bytes() = 1 MiB, resident on every GPU that loads the
 * library until the process exits) instead of stream-ordered scratch, and the call
 * performs no cudaMalloc/cudaFree of any kind; x and y stay caller-owned.
 *   - needs round_up(N*Kp,256) + 2*round_up(4*N,256) <= kb_static_scratch_bytes(),
 *     Kp = kb_act_ld(K); larger requests fail with KB_ERR_UNSUPPORTED and a message
 *     stating both sizes;
 *   - the first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress), and the first launch of each kernel it can pick (token
 *     counts 1, 2, 3..4, 5..8, 9..128, 129..256 and above 256 each take a different one)
 *     loads that kernel and sets its shared-memory limit, which the driver may back with
 *     memory of its own.  Make one warm-up call per token-count class you will use during
 *     set-up, before any stream capture and before the process's memory budget is frozen;
 *   - all calls on a device share the array and it keeps the previous call's bytes.
 *     Each call overwrites everything it reads, so nothing has to be cleared, but calls
 *     that overlap on the GPU (two streams, two threads) race: serialise them. */
int kb_linear_forward_static(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y,
                             kb_stream stream);
size_t kb_static_scratch_bytes(void);

/* ---- grouped decode: one token through each of several independent layers ----
 *
 * `count` BitLinear / QuatLinear layers of the same kind, shape and device, each called once
 * with its own single-token input (Module::forward, bit_linear.rs:175-237 /
 * quat_linear.rs:245-319, called once per layer: independent projections such as the experts
 * or heads of a block, or the same projection of several models).  One launch streams all their
 * weights: a 4 MiB layer is shorter than any kernel's launch, ramp-up and tail, so launching them
 * one by one leaves HBM bandwidth unused.  Layer i reads token row i of (xq, sx, sumq) — one
 * kb_quantize_act_i8 call over the [count, K] matrix of inputs produces all three — and writes
 * y[i, 0..M) (ldy = 0 means M).  Results are bit-identical to kb_linear_forward_q8 per layer.
 * kb_linear_group_forward takes the f32 inputs x [count, ldx] (ldx = 0 means K) instead and
 * quantises them in the kernel's prologue (bit-identical to kb_quantize_act_i8 + the q8 entry):
 * the whole group is then a single launch.
 * The group borrows the handles' device memory: destroy the group before its members. */
int kb_linear_group_create(const kb_linear *const *handles, size_t count, kb_linear_group **out);
void kb_linear_group_destroy(kb_linear_group *g);
size_t kb_linear_group_count(const kb_linear_group *g);
int kb_linear_group_forward_q8(const kb_linear_group *g, const int8_t *xq, size_t ldq, const float *sx,
                               const int32_t *sumq, float *y, size_t ldy, kb_stream stream);
int kb_linear_group_forward(const kb_linear_group *g, const float *x, size_t ldx, float *y, size_t ldy,
                            kb_stream stream);
/* Host buffers: x [count, K] and y [count, M], contiguous; copies, launches and synchronisation inside
 * the call.  Groups of 32 or more members run as a pipeline over chunks of members on the group's own
 * streams — upload, grouped launch and download of neighbouring chunks overlap when the host buffers are
 * pinned (pageable buffers make the copies synchronous).  Calls on one group are serialised. */
int kb_linear_group_forward_host(const kb_linear_group *g, const float *x, float *y);

/* ---- kernel-shaped one-shots (host pointers), signatures of
 * ternary_matmul (crates/kore-kernels/src/cpu_ternary_matmul.rs:29-36) and
 * quat_matmul (crates/kore-kernels/src/cpu_quat_matmul.rs:22-29):
 * a_packed wire format, b [K,N] f32, c [M,N] f32.  Buffer-length checks and their
 * messages follow :44-57 / :37-50. */
int kb_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                      size_t scales_len, const float *b, float *c, size_t m, size_t n, size_t k);
int kb_quat_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales, size_t scales_len,
                   const float *b, float *c, size_t m, size_t n, size_t k);

/* cuda_dequant_quat_matmul_bias_relu_f32 (crates/kore-kernels/src/cuda/ops.rs:828-878), host
 * pointers: c[m,n] = max(0, dequant(a)[m,:] . b[:,n] * a_scales[m] + bias[m]), c [M,N] f32.
 * bias has one value per weight row (output feature): the reference kernel reads bias[col]
 * with col running over N (dequant_matmul.cu:259), which indexes tokens in the layer's
 * orientation; the per-feature form is the one a linear layer needs and the one built here. */
int kb_quat_matmul_bias_relu(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                             size_t scales_len, const float *b, const float *bias, size_t bias_len,
                             float *c, size_t m, size_t n, size_t k);

/* ternary_ternary_matmul (cpu_ternary_matmul.rs:131-193): both operands base-243 rows,
 * a [M, ceil(K/5)] with a_scales [M], b [N, ceil(K/5)] with b_scales [N], integer dot product,
 * c[m,n] = float(dot) * a_scale[m] * b_scale[n], c [M,N] f32 (host pointers).  Too-short inputs
 * return the storage error "packed arrays too small" (:142-146). */
int kb_ternary_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales,
                              const uint8_t *b_packed, size_t b_len, const float *b_scales, float *c,
                              size_t m, size_t n, size_t k);

/* pack_weights_ternary (cpu_ternary_matmul.rs:198-240) and pack_weights_quaternary
 * (cpu_quat_matmul.rs:174-214), computed on the device: f32 [M,K] host in,
 * wire-format bytes and per-row scales out (host). */
int kb_pack_weights_ternary(const float *w, size_t m, size_t k, float threshold, uint8_t *packed,
                            size_t packed_len, float *scales, size_t scales_len, int device);
int kb_pack_weights_quaternary(const float *w, size_t m, size_t k, uint8_t *packed,
                               size_t packed_len, float *scales, size_t scales_len, int device);

/* ---- column-sharded forward across the GPUs of one box (one process per GPU) ----
 * No counterpart in the reference, which has no multi-device execution (its only
 * cross-device code is a host-staged copy, crates/kore-kernels/src/cuda/memory.rs:93-100).
 *
 * Rank r holds the weight rows (= output features) [col_offset, col_offset + M_shard) of a
 * layer with m_total output features.  y_bases[q] is rank q's full output buffer
 * [N, m_total] f32 as seen from this process: y_bases[rank] is local, the others are
 * peer mappings obtained with kb_ipc_open.  The kernel epilogue stores this rank's
 * slice into all of them (peer stores over NVLink).  When flag_arrays_dev and
 * sync_words_dev (three local int32, zero-initialised: epoch, CTA counter, status) are
 * given, completion is published to the peers and theirs awaited (bounded, about a
 * second): inside the tail of the GEMV kernel, or by kb_peer_barrier after the GEMM.
 * With both NULL the caller runs kb_peer_barrier (or any other barrier) itself. */
int kb_linear_forward_sharded(const kb_linear *h, const float *x, size_t n, size_t in_dim,
                              float *const *y_bases, int world, int rank, size_t m_total,
                              size_t col_offset, int path, void *workspace,
                              size_t workspace_bytes, int *const *flag_arrays_dev,
                              int *sync_words_dev, kb_stream stream);
/* The same for activations that are already quantised (kb_quantize_act_i8, kb_rmsnorm_quant,
 * ...): no per-launch quantiser, so a decode step shares one quantisation among its ranks' kernels. */
int kb_linear_forward_sharded_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx,
                                 const int32_t *sumq, size_t n, float *const *y_bases, int world, int rank,
                                 size_t m_total, size_t col_offset, int path, int *const *flag_arrays_dev,
                                 int *sync_words_dev, kb_stream stream);
/* Chain form for a sequence of sharded layers (up to 32 tokens, pre-quantised activations): the launch first
 * streams its weights, then waits (bounded) until every peer has published the PREVIOUS forward of the chain —
 * so the cross-GPU latency hides behind the weight stream and launches keep programmatic dependent launch —
 * and publishes its own slice at its end WITHOUT waiting.  Every rank must issue the same sequence of chain
 * forwards on the same exchange state; call kb_peer_wait after the last one before reading its output.  Where
 * the streaming kernel does not take the shape, the call behaves like kb_linear_forward_sharded_q8 (full
 * barrier), which is stronger. */
int kb_linear_forward_sharded_chain_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx,
                                       const int32_t *sumq, size_t n, float *const *y_bases, int world,
                                       int rank, size_t m_total, size_t col_offset,
                                       int *const *flag_arrays_dev, int *sync_words_dev, kb_stream stream);
/* Flagged exchange for chains of dependent sharded layers of up to 128 tokens (streaming kernel up to 8 tokens, 32
 * pre-quantised; medium-batch GEMM beyond): every
 * output value travels as an 8-byte word (f32 bits in the low half, an epoch in the high half) written with a
 * single 8-byte store into every rank's buffer, so a reader that finds the expected epoch has the value too — no
 * fence, no flag array, no barrier, and nothing waits in the producer.  y_bases[q] = rank q's buffer of
 * [n][m_total] such words (16-byte aligned, m_total even; local or peer mapping).
 *   A chain is forwards seq = 1, 2, ... (at most 255), each consuming the previous one's words, ended by ONE
 * kb_flagged_unpack of the last result; every rank issues the same chain.  seq = 1 takes plain f32 x [n][in_dim]
 * (x_is_flagged = 0, ldx 0 or in_dim) or pre-quantised activations; seq >= 2 takes x_is_flagged = 1: x is this
 * rank's buffer of forward seq - 1, ldx its leading dimension in words, K a multiple of 4.  The consumer waits,
 * bounded, per word: either in the forward kernel's own quantiser prologue (fuse = 1; every CTA reads the whole
 * row, good for short rows) or in a cluster kernel that quantises the row once for all CTAs (fuse = 2; needs
 * `workspace`, 256-byte aligned, twice (n * kb_act_ld(K) rounded up to 256 + 2 * (4 n rounded up to 256))
 * bytes, or NULL to allocate on the stream); fuse = 0 chooses.  Either way the forward kernel has issued its first
 * weight copies before it waits.  Epoch = (round << 8) | seq with the round in sync_words_dev[3], advanced by the
 * unpack, so chains are graph-replayable.  sync_words_dev: 8 int32, zero-initialised ({0,1}: the fence protocol
 * of the other sharded entry points, [2] status, [3] round, [4] counter of the unpack).
 *   Buffer rule: consecutive flagged forwards — across chains too — alternate between two buffers.  Then a rank
 * cannot overwrite words a peer still has to read, because it needs that peer's next words first.
 *   A word that never arrives ends the wait after about a second with status 110 (sync_words_dev[2], or
 * kb_linear_last_device_status for the fused prologue). */
int kb_linear_forward_sharded_flagged(const kb_linear *h, const void *x, int x_is_flagged, size_t ldx, size_t n,
                                      size_t in_dim, unsigned long long *const *y_bases, int world, int rank,
                                      size_t m_total, size_t col_offset, int seq, int fuse, void *workspace,
                                      size_t workspace_bytes, int *sync_words_dev, kb_stream stream);
int kb_linear_forward_sharded_flagged_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx,
                                         const int32_t *sumq, size_t n, unsigned long long *const *y_bases,
                                         int world, int rank, size_t m_total, size_t col_offset, int seq,
                                         int *sync_words_dev, kb_stream stream);
/* end of a chain: flagged words [n][ld_src] of forward `seq` -> plain f32 [n][ld_dst], first m columns; waits
 * (bounded) until every word has arrived, then advances the round */
int kb_flagged_unpack(const unsigned long long *src, size_t ld_src, size_t n, size_t m, float *dst, size_t ld_dst,
                      int seq, int *sync_words_dev, kb_stream stream);
/* waits (bounded) until every rank has published as many forwards as this rank (epoch_counter_dev = the first
 * of the three sync words) */
int kb_peer_wait(int *const *flag_arrays_dev, int world, int rank, const int *epoch_counter_dev,
                 int *status_dev, kb_stream stream);
/* flag_arrays_dev: device array of `world` pointers, entry q = rank q's int32[world]
 * flag array (local or peer mapping); epoch_counter_dev: one local int32, starts at 0 and
 * is bumped by every barrier (all ranks must issue the same sequence of barriers);
 * status_dev: one int32, set to 100+q if rank q never arrived. */
int kb_peer_barrier(int *const *flag_arrays_dev, int world, int rank, int *epoch_counter_dev,
                    int *status_dev, kb_stream stream);
/* zero-filled device allocation that can be shared with peer processes, and its sharing */
int kb_symm_alloc(size_t bytes, void **out);
int kb_symm_free(void *p);
int kb_ipc_export(const void *p, uint8_t *handle64);
int kb_ipc_open(const uint8_t *handle64, void **out);
int kb_ipc_close(void *p);

/* ---- plumbing used by the host layers ---- */

/* Raw device pointers of a handle (read-only views; valid until destroy). */
int kb_linear_device_ptrs(const kb_linear *h, const void **w2, size_t *row_bytes,
                          const float **scales, const float **bias);
/* Device-side status word of the last tcgen05 GEMM launched by the calling thread
 * on this handle: 0 = clean, otherwise a code saying which bounded wait gave up. */
int kb_linear_last_device_status(const kb_linear *h, kb_stream stream, int *status);

#ifdef __cplusplus
}
#endif
#endif /* KORE_B200_H */
