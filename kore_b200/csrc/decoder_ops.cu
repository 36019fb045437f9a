// Glue kernels of the decoder step around the quantized-linear path (sm_100a).
//
// Each of them ends in the per-token int8 quantiser, so the following projection reads
// codes instead of f32 activations and no separate quantiser launch is needed:
//   rmsnorm_quant   y = (x * (1 / sqrt(mean(x^2) + eps))) * gamma            -> int8
//                   (KORE: crates/kore-kernels/src/cpu_fused.rs:160-190,
//                    cuda/kernels/rms_norm.cu:17)
//   swiglu_quant    h = (g / (1 + exp(-g))) * u, g|u = the two halves of a row -> int8
//                   (crates/kore-edge/src/ops/activation.rs:21-26, runtime.rs:232-265)
//   rope_kv         half-split rotary embedding of q and k from a [q|k|v] row with
//                   host-supplied cos/sin tables, k and v appended to the head-major cache
//                   (crates/kore-edge/src/ops/rope.rs:9-36)
//   attn_decode     one query token per sequence against its KV cache, softmax in f32
//                   (crates/kore-edge/src/ops/attention.rs:74-135, causal rule of
//                    crates/kore-serve/src/layered/engine.rs:734-751)
// All are HBM/latency-bound elementwise or row-reduction work, one CTA per token (or per
// sequence-head); none is reshaped into a GEMM.
//
// Every kernel is launched with programmatic stream serialization: it lets its successor
// start at once (griddepcontrol.launch_dependents — the following GEMV streams its first
// weights meanwhile) and reads its own inputs only after griddepcontrol.wait, which returns
// when the predecessor grid has completed and its writes are visible.
#include <stdlib.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

// Every kernel here is launched with programmatic stream serialization, so its CTAs may be resident while the
// producer of its inputs still runs.  Inputs that an earlier kernel of the step writes (activations, positions,
// lengths, caches) are therefore plain pointers, read after the wait below: a `const __restrict__` pointer would let
// the compiler use the non-coherent path and hoist the loads above the wait (a head kernel did exactly that and read
// the previous step's row).  Only true constants (weights, gamma, the RoPE tables) keep the qualifier.
__device__ __forceinline__ void pdl_release_and_wait() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    static const bool pdl = [] {
        const char *v = getenv("KB_GEMV_PDL");
        return !(v && *v == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

__device__ __forceinline__ float block_reduce_sum_f(float v, float *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = lane < nwarps ? scratch[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// quantise `vals` (this thread's elements idx = threadIdx.x + i*blockDim.x, i < CNT) of one row
template <int CNT>
__device__ __forceinline__ void quantise_row_from_regs(const float (&vals)[CNT], int d, int ldq, int8_t *qrow,
                                                       float *sx_out, int32_t *sum_out, float *red_f, int *red_i) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < CNT; ++i) amax = fmaxf(amax, fabsf(vals[i]));
    amax = block_reduce_max(amax, red_f);
    const float s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float rs = __frcp_rn(s);
    int local = 0;
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < ldq) {
            const int q = idx < d ? quantise_one_fast(vals[i], s, rs) : 0;
            local += q;
            qrow[idx] = (int8_t)q;
        }
    }
    local = block_reduce_sum(local, red_i);
    if (threadIdx.x == 0) {
        *sx_out = s;
        if (sum_out) *sum_out = local;
    }
}

constexpr int ROW_REGS = 36;  // elements per thread held in registers: rows up to 36 * 256 = 9216

__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const float *x, const float *__restrict__ gamma,
                                                            int d, float eps, float *__restrict__ xn,
                                                            int8_t *__restrict__ xq, int ldq, float *__restrict__ sx,
                                                            int32_t *__restrict__ sumq) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const size_t t = blockIdx.x;
    const float *row = x + t * (size_t)d;
    // every global load of the row (and of gamma) is issued before the first use, so the
    // single CTA pays one memory round trip instead of one per element
    float v[ROW_REGS], gm[ROW_REGS];
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) {  // gamma is a constant of the layer: fetched before the wait
        const int idx = threadIdx.x + i * blockDim.x;
        gm[i] = idx < d ? gamma[idx] : 0.0f;
    }
    pdl_release_and_wait();
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        v[i] = idx < d ? row[idx] : 0.0f;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) ss = __fadd_rn(ss, __fmul_rn(v[i], v[i]));
    ss = block_reduce_sum_f(ss, red_f);
    const float rms = sqrtf(__fadd_rn(__fdiv_rn(ss, (float)d), eps));
    const float inv = __fdiv_rn(1.0f, rms);
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], inv), gm[i]);
    if (xn) {
#pragma unroll
        for (int i = 0; i < ROW_REGS; ++i) {
            const int idx = threadIdx.x + i * blockDim.x;
            if (idx < d) xn[t * (size_t)d + idx] = v[i];
        }
    }
    if (xq) quantise_row_from_regs<ROW_REGS>(v, d, ldq, xq + t * (size_t)ldq, sx + t, sumq ? sumq + t : nullptr, red_f, red_i);
}

// PAIRS: the row alternates gate_i, up_i instead of holding the two halves one after the other
template <bool PAIRS>
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const float *gu, int f, size_t ld,
                                                           float *__restrict__ h_out, int8_t *__restrict__ xq, int ldq,
                                                           float *__restrict__ sx, int32_t *__restrict__ sumq) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const size_t t = blockIdx.x;
    const float *g = gu + t * ld, *u = g + f;
    float v[ROW_REGS], uv[ROW_REGS];
    pdl_release_and_wait();
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) {  // all loads first: one memory round trip for the row
        const int idx = threadIdx.x + i * blockDim.x;
        if (PAIRS) {
            const float2 gu2 = idx < f ? reinterpret_cast<const float2 *>(g)[idx] : make_float2(0.0f, 0.0f);
            v[i] = gu2.x;
            uv[i] = gu2.y;
        } else {
            v[i] = idx < f ? g[idx] : 0.0f;
            uv[i] = idx < f ? u[idx] : 0.0f;
        }
    }
#pragma unroll
    for (int i = 0; i < ROW_REGS; ++i) {
        const float silu = __fdiv_rn(v[i], __fadd_rn(1.0f, expf(-v[i])));
        v[i] = __fmul_rn(silu, uv[i]);
    }
    if (h_out) {
#pragma unroll
        for (int i = 0; i < ROW_REGS; ++i) {
            const int idx = threadIdx.x + i * blockDim.x;
            if (idx < f) h_out[t * (size_t)f + idx] = v[i];
        }
    }
    if (xq) quantise_row_from_regs<ROW_REGS>(v, f, ldq, xq + t * (size_t)ldq, sx + t, sumq ? sumq + t : nullptr, red_f, red_i);
}

// grid (token, chunk): thread handles one (head, i) pair of q and k and one or two elements of
// v, so every load of a token is in flight at once.  Rotation pairs are (i, i + hd/2) inside
// each head; k and v go to row cache_rows[t] of the caches; cos/sin tables are [max_pos][hd/2].
__global__ void __launch_bounds__(256) rope_kv_kernel(const float *qkv, const int *positions, const long long *cache_rows,
                                                      const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                                      int n_heads, int hd, int lmax, float *__restrict__ q_out,
                                                      float *__restrict__ k_cache, float *__restrict__ v_cache) {
    const size_t t = blockIdx.x;
    const int d = n_heads * hd, half = hd / 2;
    const float *q = qkv + t * (size_t)(3 * d), *k = q + d, *v = k + d;
    pdl_release_and_wait();
    const int pos = positions[t];
    // caches are head-major, [sequence][head][lmax][hd]: a head's keys are contiguous, so decode attention streams
    // them at full DRAM page efficiency; cache_rows[t] = sequence * lmax + position
    const long long crow_flat = cache_rows[t];
    const size_t seq = (size_t)(crow_flat / lmax), cpos = (size_t)(crow_flat % lmax);
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;  // pair index, 0 .. n_heads*half-1
    if (idx < n_heads * half) {
        const int h = idx / half, i = idx - h * half;
        const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
        const int a = h * hd + i, b = a + half;
        const float q0 = q[a], q1 = q[b], k0 = k[a], k1 = k[b], va = v[a], vb2 = v[b];
        q_out[t * (size_t)d + a] = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, s));
        q_out[t * (size_t)d + b] = __fadd_rn(__fmul_rn(q0, s), __fmul_rn(q1, c));
        const size_t crow = ((seq * n_heads + h) * lmax + cpos) * hd;
        k_cache[crow + i] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, s));
        k_cache[crow + i + half] = __fadd_rn(__fmul_rn(k0, s), __fmul_rn(k1, c));
        v_cache[crow + i] = va;
        v_cache[crow + i + half] = vb2;
    }
}

// Decode attention, split over the cache length (flash-decoding style): CTA (b, h, s) handles
// key positions [s*chunk, (s+1)*chunk) of sequence b / head h.  A warp owns one position at a
// time: its lanes read the key row coalesced (dims lane, lane+32, ...) and reduce the dot with
// shuffles, keep a running (max, sum) and a running V accumulator with the usual rescaling.
// Per-warp partials are merged in shared memory, per-CTA partials in `scratch`
// ([b*h][splits][2 + hd]); the last CTA of a (b, h) — found with a self-resetting counter —
// merges them and writes the output.
constexpr int ATT_WARPS = 8;
constexpr int ATT_MAX_HD = 128;
constexpr int ATT_UNROLL = 4;
constexpr int ATT_MAX_SPLITS = 32;

// VEC4 (head_dim a multiple of 4, 16-byte aligned rows): lane l owns dims 4l .. 4l+3 and reads them
// with one 128-bit load per row; otherwise lane l owns dims l, l + 32, ...
template <bool VEC4>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_kernel(
    const float *q, const float *k_cache, const float *v_cache, const int *lens, int n_heads, int hd, int lmax, int splits, float *__restrict__ scratch,
    int *__restrict__ counters, float *__restrict__ out) {
    __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS], s_acc[ATT_WARPS][ATT_MAX_HD];
    __shared__ int s_last;
    const int bh = blockIdx.x / splits, sp = blockIdx.x % splits;
    const int b = bh / n_heads, h = bh % n_heads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_release_and_wait();
    const int d = n_heads * hd, len = lens[b];
    const int chunk = (len + splits - 1) / splits;
    const int j0 = sp * chunk, j1 = min(len, j0 + chunk);
    constexpr int DPL = ATT_MAX_HD / 32;  // dims per lane
    static_assert(DPL == 4, "the vector path reads one float4 per lane");
    auto dim_of = [&](int i) { return VEC4 ? 4 * lane + i : lane + 32 * i; };
    auto load_row = [&](const float *row, bool ok, float (&dst)[DPL]) {
        if (VEC4) {
            const float4 f = (ok && 4 * lane < hd) ? *reinterpret_cast<const float4 *>(row + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            dst[0] = f.x; dst[1] = f.y; dst[2] = f.z; dst[3] = f.w;
        } else {
#pragma unroll
            for (int i = 0; i < DPL; ++i) dst[i] = (ok && lane + 32 * i < hd) ? row[lane + 32 * i] : 0.0f;
        }
    };
    float qv[DPL], acc[DPL];
    load_row(q + (size_t)b * d + h * hd, true, qv);
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
    const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
    const float *kb_ = k_cache + ((size_t)b * n_heads + h) * lmax * hd;  // head-major cache: rows of hd floats
    const float *vb = v_cache + ((size_t)b * n_heads + h) * lmax * hd;
    float m = -INFINITY, l = 0.0f;
    // ATT_UNROLL positions per warp iteration: all their key and value loads are issued before
    // the first use, so a warp pays one memory round trip per ATT_UNROLL positions
    for (int jb = j0 + warp; jb < j1; jb += ATT_WARPS * ATT_UNROLL) {
        float kk[ATT_UNROLL][DPL], vv[ATT_UNROLL][DPL];
#pragma unroll
        for (int u = 0; u < ATT_UNROLL; ++u) {
            const int j = jb + u * ATT_WARPS;
            const bool ok = j < j1;
            load_row(kb_ + (size_t)(ok ? j : j0) * hd, ok, kk[u]);
            load_row(vb + (size_t)(ok ? j : j0) * hd, ok, vv[u]);
        }
#pragma unroll
        for (int u = 0; u < ATT_UNROLL; ++u) {
            if (jb + u * ATT_WARPS >= j1) break;  // uniform over the warp
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) dot = fmaf(qv[i], kk[u][i], dot);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            dot *= scale;
            const float m_new = fmaxf(m, dot);
            const float corr = expf(m - m_new), pj = expf(dot - m_new);
            l = l * corr + pj;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pj, vv[u][i], acc[i] * corr);
            m = m_new;
        }
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < DPL; ++i)
        if (dim_of(i) < ATT_MAX_HD) s_acc[warp][dim_of(i)] = acc[i];
    __syncthreads();
    // merge the warps of this CTA (threads 0..hd-1 each own one output dim)
    float cm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) cm = fmaxf(cm, s_m[w]);
    float cl = 0.0f, ca = 0.0f;
    if ((int)threadIdx.x < hd) {
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float f = s_m[w] == -INFINITY ? 0.0f : expf(s_m[w] - cm);
            cl += s_l[w] * f;
            ca += s_acc[w][threadIdx.x] * f;
        }
    }
    if (splits == 1) {
        if ((int)threadIdx.x < hd) out[(size_t)b * d + h * hd + threadIdx.x] = ca * __fdiv_rn(1.0f, cl);
        return;
    }
    float *part = scratch + ((size_t)bh * splits + sp) * (2 + ATT_MAX_HD);
    if (threadIdx.x == 0) { part[0] = cm; part[1] = cl; }
    if ((int)threadIdx.x < hd) part[2 + threadIdx.x] = ca;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(counters + bh, 1);
        s_last = (ticket == splits - 1);
        if (s_last) counters[bh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float *base = scratch + (size_t)bh * splits * (2 + ATT_MAX_HD);
    float gm = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) gm = fmaxf(gm, base[s2 * (2 + ATT_MAX_HD)]);
    if ((int)threadIdx.x < hd) {
        float gl = 0.0f, ga = 0.0f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float *ps = base + s2 * (2 + ATT_MAX_HD);
            const float f = ps[0] == -INFINITY ? 0.0f : expf(ps[0] - gm);
            gl += ps[1] * f;
            ga += ps[2 + threadIdx.x] * f;
        }
        out[(size_t)b * d + h * hd + threadIdx.x] = ga * __fdiv_rn(1.0f, gl);
    }
}

// ---- dense f32 head of a greedy decode step for a few sequences: logits = x W^T, argmax per token ----
// The weights [vocab][d] are the stream (410 MB for 32000 x 3200).  A CTA of 512 threads keeps up to 8 tokens' rows of x
// in registers (thread t owns the float4s t and t + 512 of every row: 64 registers for 8 tokens) and walks the
// vocabulary two rows per step.  The weights travel global -> shared memory as 16-byte asynchronous copies in a ring
// of HEAD_DEPTH steps; every thread copies exactly the float4s it later multiplies, so its own copy groups are all the
// synchronisation the ring needs (192 KB in flight per SM).  The 16 partial dot products of a thread are reduced over
// the warp with a transposing shuffle reduction and over the 16 warps through shared memory (one barrier per row pair,
// two buffers).  blockIdx.y selects the group of 8 tokens; both groups walk the same rows at the same pace, so the
// second read of a row is an L2 hit.  Thread (row of the pair, token) keeps the running maximum and folds it into
// keys[token] at the end: key = (order-preserving bits of the logit << 32) | ~row, so the largest key is the largest
// logit and, among equals, the lowest row — torch.argmax's answer.
constexpr int HEAD_THREADS = 512;
constexpr int HEAD_TOK = 8;
constexpr int HEAD_ROWS = 2;
constexpr int HEAD_V4 = 2;     // float4s of a row per thread: d <= 4 * 512 * 2
constexpr int HEAD_DEPTH = 6;  // steps of the weight ring
constexpr int HEAD_STEP_BYTES = HEAD_ROWS * HEAD_V4 * HEAD_THREADS * 16;

__device__ __forceinline__ unsigned long long argmax_key(float v, int row) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // unsigned order == float order (NaN aside)
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (uint32_t)row);
}

// TOK = tokens per CTA (8, 4 or 2: fewer tokens, fewer multiply-adds per weight)
template <int TOK>
__global__ void __launch_bounds__(HEAD_THREADS, 1) lm_head_argmax_kernel(const float *x, int n, int d,
                                                                          const float *__restrict__ w, int vocab,
                                                                          float *__restrict__ logits,
                                                                          unsigned long long *__restrict__ keys) {
    extern __shared__ __align__(128) uint8_t head_ring[];  // [HEAD_DEPTH][HEAD_ROWS][HEAD_V4][HEAD_THREADS] float4
    constexpr int NVAL = HEAD_ROWS * TOK;  // dot products a thread carries per step: 16, 8 or 4
    __shared__ float part[2][HEAD_THREADS / 32][NVAL];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tok0 = blockIdx.y * TOK;
    const int nv4 = d >> 2;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(head_ring) + threadIdx.x * 16u;
    const int stride = gridDim.x * HEAD_ROWS;
    // the weights do not depend on the previous kernel: the ring fills before the wait
    auto issue = [&](int step) {  // rows r0 = (blockIdx.x + step * gridDim.x) * HEAD_ROWS
        const int r0 = blockIdx.x * HEAD_ROWS + step * stride;
        const uint32_t dst = ring + (uint32_t)(step % HEAD_DEPTH) * HEAD_STEP_BYTES;
#pragma unroll
        for (int r = 0; r < HEAD_ROWS; ++r)
#pragma unroll
            for (int i = 0; i < HEAD_V4; ++i) {
                const int c = threadIdx.x + i * HEAD_THREADS;
                const bool live = r0 + r < vocab && c < nv4;
                const float *src = live ? w + (size_t)(r0 + r) * d + 4 * c : w;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (uint32_t)((r * HEAD_V4 + i) * HEAD_THREADS * 16)),
                             "l"(src), "r"(live ? 16 : 0)
                             : "memory");
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int steps = blockIdx.x * HEAD_ROWS < vocab ? (vocab - blockIdx.x * HEAD_ROWS + stride - 1) / stride : 0;
    for (int sft = 0; sft < HEAD_DEPTH - 1; ++sft) {
        if (sft < steps) issue(sft);
        else asm volatile("cp.async.commit_group;" ::: "memory");  // keeps the group count in step
    }
    // starts behind the final norm by programmatic dependent launch, but releases no dependent of its own early: the
    // launch that ends the step must see this kernel's keys, and it is the last word on the step's state
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float4 xr[TOK][HEAD_V4];
#pragma unroll
    for (int t = 0; t < TOK; ++t)
#pragma unroll
        for (int i = 0; i < HEAD_V4; ++i) {
            const int c = threadIdx.x + i * HEAD_THREADS;
            // read through L2 (the producer of x may still have been running when this CTA became resident)
            xr[t][i] = (tok0 + t < n && c < nv4) ? __ldcg(reinterpret_cast<const float4 *>(x + (size_t)(tok0 + t) * d) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    // reducer threads: thread r * TOK + t (< NVAL) owns (row r of the pair, token t)
    const int red_r = threadIdx.x / TOK, red_t = threadIdx.x % TOK;
    float best = -INFINITY;
    int best_row = 0;
    for (int it = 0; it < steps; ++it) {
        if (it + HEAD_DEPTH - 1 < steps) issue(it + HEAD_DEPTH - 1);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(HEAD_DEPTH - 1) : "memory");  // this thread's copies of step `it` have landed
        const int r0 = blockIdx.x * HEAD_ROWS + it * stride;
        const uint8_t *src = head_ring + (size_t)(it % HEAD_DEPTH) * HEAD_STEP_BYTES + threadIdx.x * 16;
        float4 wv[HEAD_ROWS][HEAD_V4];
#pragma unroll
        for (int r = 0; r < HEAD_ROWS; ++r)
#pragma unroll
            for (int i = 0; i < HEAD_V4; ++i) wv[r][i] = *reinterpret_cast<const float4 *>(src + (size_t)((r * HEAD_V4 + i) * HEAD_THREADS * 16));
        float acc[NVAL];
#pragma unroll
        for (int r = 0; r < HEAD_ROWS; ++r)
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                float a = 0.0f;
#pragma unroll
                for (int i = 0; i < HEAD_V4; ++i) {
                    a = fmaf(wv[r][i].x, xr[t][i].x, a);
                    a = fmaf(wv[r][i].y, xr[t][i].y, a);
                    a = fmaf(wv[r][i].z, xr[t][i].z, a);
                    a = fmaf(wv[r][i].w, xr[t][i].w, a);
                }
                acc[r * TOK + t] = a;
            }
        // NVAL values over 32 lanes: while more than one value is left, a lane keeps half of its values and receives the
        // partner's share of them (lane bit 16, 8, ... decides which half); the remaining steps sum the lanes that hold the
        // same value.  Value index = the kept-half bits in order, most significant first.
        int idx = 0;
        {
            int cnt = NVAL;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                if (cnt > 1) {
                    const bool hi = (lane & off) != 0;
                    cnt >>= 1;
#pragma unroll
                    for (int j = 0; j < NVAL / 2; ++j)
                        if (j < cnt) acc[j] = (hi ? acc[cnt + j] : acc[j]) + __shfl_xor_sync(0xffffffffu, hi ? acc[j] : acc[cnt + j], off);
                    idx = idx * 2 + (hi ? 1 : 0);
                } else {
                    acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], off);
                }
            }
        }
        // lanes whose low bits (those of the summing steps) are zero publish
        constexpr int SUM_MASK = NVAL == 16 ? 1 : (NVAL == 8 ? 3 : 7);
        if ((lane & SUM_MASK) == 0) part[it & 1][warp][idx] = acc[0];
        __syncthreads();
        if (threadIdx.x < NVAL) {
            float sum = 0.0f;
#pragma unroll
            for (int wp = 0; wp < HEAD_THREADS / 32; ++wp) sum += part[it & 1][wp][threadIdx.x];
            const int row = r0 + red_r, tok = tok0 + red_t;
            if (row < vocab && tok < n) {
                if (logits) logits[(size_t)tok * vocab + row] = sum;
                if (sum > best) { best = sum; best_row = row; }  // rows ascend: the first maximum stays
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (threadIdx.x < NVAL && tok0 + red_t < n && best > -INFINITY) atomicMax(keys + tok0 + red_t, argmax_key(best, best_row));
}

// End of a greedy step: token = the row in the key, positions / lens / cache rows advance by one, keys are cleared.
__global__ void decode_advance_kernel(unsigned long long *keys, int n, long long *tokens, int *positions, int *lens,
                                      long long *cache_rows) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) {
        const unsigned long long key = keys[t];
        tokens[t] = key ? (long long)(0xffffffffu - (uint32_t)(key & 0xffffffffull)) : 0;  // no finite logit: token 0
        keys[t] = 0ull;
        if (positions) positions[t] += 1;
        if (lens) lens[t] += 1;
        if (cache_rows) cache_rows[t] += 1;
    }
}

}  // namespace kb

using namespace kb;

extern "C" {

int kb_lm_head_argmax(const float *x, size_t n, size_t d, const float *w, size_t vocab, float *logits, unsigned long long *keys,
                      kb_stream stream) {
    if (!x || !w || !keys) return fail(KB_ERR_INVALID, "null pointer");
    if (n == 0) return KB_OK;
    if (n > 16) return fail(KB_ERR_UNSUPPORTED, "lm_head: %zu tokens (at most 16)", n);
    if (d == 0 || d % 4 || d > (size_t)4 * HEAD_THREADS * HEAD_V4 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15))
        return fail(KB_ERR_UNSUPPORTED, "lm_head: width %zu must be a multiple of 4 up to %d, with 16-byte aligned rows", d,
                    4 * HEAD_THREADS * HEAD_V4);
    if (vocab == 0 || vocab > ((size_t)1 << 31)) return fail(KB_ERR_INVALID, "lm_head: vocabulary size %zu", vocab);
    int dev = 0;
    KB_CUDA(cudaGetDevice(&dev));
    const int tok = n <= 2 ? 2 : (n <= 4 ? 4 : HEAD_TOK);
    const unsigned groups = (unsigned)((n + tok - 1) / tok);
    size_t gx = (size_t)sm_count(dev) / groups;
    const size_t pairs = (vocab + HEAD_ROWS - 1) / HEAD_ROWS;
    if (gx > pairs) gx = pairs;
    if (gx < 1) gx = 1;
    const size_t smem = (size_t)HEAD_DEPTH * HEAD_STEP_BYTES;
    void (*kern)(const float *, int, int, const float *, int, float *, unsigned long long *) =
        tok == 2 ? lm_head_argmax_kernel<2> : (tok == 4 ? lm_head_argmax_kernel<4> : lm_head_argmax_kernel<HEAD_TOK>);
    if (int rc = set_dyn_smem_once(reinterpret_cast<const void *>(kern), dev, (int)smem, "lm_head smem attribute")) return rc;
    static const bool pdl = [] { const char *v = getenv("KB_GEMV_PDL"); return !(v && *v == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, groups);
    cfg.blockDim = dim3(HEAD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, x, (int)n, (int)d, w, (int)vocab, logits, keys);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "lm_head launch");
}

int kb_decode_advance(unsigned long long *keys, size_t n, long long *tokens, int *positions, int *lens, long long *cache_rows,
                      kb_stream stream) {
    if (!keys || !tokens) return fail(KB_ERR_INVALID, "null pointer");
    if (n == 0) return KB_OK;
    decode_advance_kernel<<<(unsigned)((n + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(keys, (int)n, tokens, positions, lens,
                                                                                                    cache_rows);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "decode advance launch");
}

int kb_rmsnorm_quant(const float *x, const float *gamma, size_t n, size_t d, float eps, float *xn, int8_t *xq, size_t ldq,
                     float *sx, int32_t *sumq, kb_stream stream) {
    if (!x || !gamma || (!xn && !xq) || (xq && !sx)) return fail(KB_ERR_INVALID, "null pointer");
    if (d == 0 || d > (size_t)ROW_REGS * 256) return fail(KB_ERR_UNSUPPORTED, "rmsnorm: dim %zu outside 1..%d", d, ROW_REGS * 256);
    if (xq && (ldq < d || ldq > (size_t)ROW_REGS * 256 || ldq % 16)) return fail(KB_ERR_INVALID, "rmsnorm: bad ldq %zu", ldq);
    if (n == 0) return KB_OK;
    cudaError_t e = launch_pdl(rmsnorm_quant_kernel, dim3((unsigned)n), dim3(256), static_cast<cudaStream_t>(stream), x, gamma,
                               (int)d, eps, xn, xq, (int)ldq, sx, sumq);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "rmsnorm launch");
}

static int swiglu_quant(bool pairs, const float *gate_up, size_t n, size_t f, size_t ld, float *h, int8_t *xq, size_t ldq,
                        float *sx, int32_t *sumq, kb_stream stream) {
    if (!gate_up || (!h && !xq) || (xq && !sx)) return fail(KB_ERR_INVALID, "null pointer");
    if (pairs && ((reinterpret_cast<uintptr_t>(gate_up) & 7) || (ld & 1)))
        return fail(KB_ERR_INVALID, "swiglu: interleaved rows must be 8-byte aligned");
    if (f == 0 || f > (size_t)ROW_REGS * 256 || ld < 2 * f) return fail(KB_ERR_UNSUPPORTED, "swiglu: width %zu outside 1..%d", f, ROW_REGS * 256);
    if (xq && (ldq < f || ldq > (size_t)ROW_REGS * 256 || ldq % 16)) return fail(KB_ERR_INVALID, "swiglu: bad ldq %zu", ldq);
    if (n == 0) return KB_OK;
    cudaError_t e = pairs ? launch_pdl(swiglu_quant_kernel<true>, dim3((unsigned)n), dim3(256), static_cast<cudaStream_t>(stream),
                                       gate_up, (int)f, ld, h, xq, (int)ldq, sx, sumq)
                          : launch_pdl(swiglu_quant_kernel<false>, dim3((unsigned)n), dim3(256), static_cast<cudaStream_t>(stream),
                                       gate_up, (int)f, ld, h, xq, (int)ldq, sx, sumq);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "swiglu launch");
}

int kb_swiglu_quant(const float *gate_up, size_t n, size_t f, size_t ld, float *h, int8_t *xq, size_t ldq, float *sx,
                    int32_t *sumq, kb_stream stream) {
    return swiglu_quant(false, gate_up, n, f, ld, h, xq, ldq, sx, sumq, stream);
}

int kb_swiglu_quant_pairs(const float *gate_up, size_t n, size_t f, size_t ld, float *h, int8_t *xq, size_t ldq, float *sx,
                          int32_t *sumq, kb_stream stream) {
    return swiglu_quant(true, gate_up, n, f, ld, h, xq, ldq, sx, sumq, stream);
}

int kb_rope_kv(const float *qkv, const int *positions, const long long *cache_rows, const float *cos_table,
               const float *sin_table, size_t n, int n_heads, int head_dim, int lmax, float *q_out, float *k_cache,
               float *v_cache, kb_stream stream) {
    if (!qkv || !positions || !cache_rows || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
        return fail(KB_ERR_INVALID, "null pointer");
    if (n_heads < 1 || head_dim < 2 || head_dim % 2) return fail(KB_ERR_INVALID, "rope: head_dim must be even");
    if (lmax < 1) return fail(KB_ERR_INVALID, "rope: cache length %d", lmax);
    if (n == 0) return KB_OK;
    const unsigned chunks = (unsigned)((n_heads * (head_dim / 2) + 255) / 256);
    cudaError_t e = launch_pdl(rope_kv_kernel, dim3((unsigned)n, chunks), dim3(256), static_cast<cudaStream_t>(stream), qkv,
                               positions, cache_rows, cos_table, sin_table, n_heads, head_dim, lmax, q_out, k_cache, v_cache);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "rope launch");
}

int kb_attn_decode(const float *q, const float *k_cache, const float *v_cache, const int *lens, size_t batch, int n_heads,
                   int head_dim, int lmax, float *out, float *scratch, size_t scratch_bytes, kb_stream stream) {
    if (!q || !k_cache || !v_cache || !lens || !out) return fail(KB_ERR_INVALID, "null pointer");
    if (head_dim < 1 || head_dim > ATT_MAX_HD) return fail(KB_ERR_UNSUPPORTED, "attention: head_dim %d outside 1..%d", head_dim, ATT_MAX_HD);
    if (batch == 0) return KB_OK;
    // about one wave of CTAs (four are resident per SM): a CTA's start and its split merge are dead time for its
    // warps, so for many sequences few long CTAs beat many short ones (16 sequences x 32 heads x 576 positions:
    // 45.6 us with one CTA per head against 52.9 us with three); a split is at least 32 positions (8 warps x 4)
    const size_t bh = batch * (size_t)n_heads;
    int dev = 0;
    KB_CUDA(cudaGetDevice(&dev));
    const size_t wave = (size_t)sm_count(dev) * 4 * 85 / 100;
    int splits = (int)((wave + bh - 1) / bh);
    const int max_splits = (lmax + 31) / 32 < ATT_MAX_SPLITS ? (lmax + 31) / 32 : ATT_MAX_SPLITS;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    const size_t need = bh * sizeof(int) + 256 + bh * (size_t)splits * (2 + ATT_MAX_HD) * sizeof(float);
    if (splits > 1 && (!scratch || scratch_bytes < need)) splits = 1;
    int *counters = reinterpret_cast<int *>(scratch);
    float *parts = scratch ? reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + (bh * sizeof(int) + 255) / 256 * 256) : nullptr;
    const bool vec4 = head_dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
                                             reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
    cudaError_t e = vec4 ? launch_pdl(attn_decode_kernel<true>, dim3((unsigned)(bh * splits)), dim3(ATT_WARPS * 32),
                                      static_cast<cudaStream_t>(stream), q, k_cache, v_cache, lens, n_heads, head_dim, lmax,
                                      splits, parts, counters, out)
                         : launch_pdl(attn_decode_kernel<false>, dim3((unsigned)(bh * splits)), dim3(ATT_WARPS * 32),
                                      static_cast<cudaStream_t>(stream), q, k_cache, v_cache, lens, n_heads, head_dim, lmax,
                                      splits, parts, counters, out);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "attention launch");
}

size_t kb_attn_decode_scratch_bytes(size_t batch, int n_heads) {
    const size_t bh = batch * (size_t)n_heads;
    return bh * sizeof(int) + 256 + bh * ATT_MAX_SPLITS * (2 + ATT_MAX_HD) * sizeof(float);
}

}  // extern "C"
