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

__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
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
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const float *__restrict__ gu, int f, size_t ld,
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
__global__ void __launch_bounds__(256) rope_kv_kernel(const float *__restrict__ qkv, const int *__restrict__ positions,
                                                      const long long *__restrict__ cache_rows,
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
    const float *__restrict__ q, const float *__restrict__ k_cache, const float *__restrict__ v_cache,
    const int *__restrict__ lens, int n_heads, int hd, int lmax, int splits, float *__restrict__ scratch,
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

}  // namespace kb

using namespace kb;

extern "C" {

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
