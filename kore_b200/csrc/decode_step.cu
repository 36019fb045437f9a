// Persistent decode step (sm_100a): one greedy decode step of a LLaMA-style decoder whose
// projections are BitLinear layers, for one or two sequences, as ONE cooperative kernel.
//
// Why: at batch 1 every projection of the step is a GEMV that streams a few megabytes — less
// time than a kernel launch, its ramp-up and its tail.  Launched one by one (even with
// programmatic dependent launch) the ~160 kernels of a step cost 5-14 us each and the step runs
// at a tenth of the HBM roofline.  Here the whole step is one grid of one CTA per SM that walks
// the phases of every layer, separated by a device-side grid barrier:
//
//   A  x = quantise(rmsnorm(hidden) * g1) (every CTA, from L2)      qkv = W_qkv . x
//   B  RoPE on q and k, k / v appended to the cache, attention of the new token over the cache
//      (work item = (sequence, head, cache split); last item of a head merges the splits)
//   C  x = quantise(attn)                                           hidden += W_o . x
//   D  x = quantise(rmsnorm(hidden) * g2)                           h = silu(gate) * up, max|h|
//   E  x = quantise(h) with the known max|h|                        hidden += W_down . x
//   ... after the last layer: final RMSNorm, dense f32 lm_head GEMV, argmax, position update.
//
// The structure follows the reference's decoder loop (crates/kore-edge/src/runtime.rs:106-294);
// the arithmetic of every operator is that of the separate kernels (decoder_ops.cu, the
// streaming GEMV of gemv_stream.cu): per-token absmax int8 activations, int32 accumulation,
// y = (float(acc) * w_scale) * s_x with separately rounded multiplies, f32 everywhere else.
//
// Weights never depend on activations, so a warp issues the first copies of its NEXT phase's
// weight rows before it enters the barrier: the HBM stream runs through barrier and prologue.
// Almost all of an SM's memory is configured as shared memory here (stage rings), which leaves an
// L1 of a few KB: bulk reads therefore go global -> shared with cp.async (weights, and the keys and
// values of the attention phase, staged in the rings while they are empty), never through
// register loads — those were measured at ~10 GB/s per SM in this configuration.
// A GEMV phase is the streaming kernel's dp4a form: unit = 16 weight rows x a K slice per warp,
// private cp.async ring per warp, KS warps of a CTA share a row block and meet in shared memory.
//
// Every wait is bounded (about a second): a stage wait or the grid barrier that gives up sets
// the status word; every later wait of every CTA then returns at once, so the grid drains and
// the host reads the status.
#include <cooperative_groups.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace kb {

namespace {

using namespace ptx;

constexpr int DW = 12;               // warps per CTA
constexpr int DTHREADS = DW * 32;
constexpr int CH = 256;              // bytes of one weight row per stage
constexpr int RS = CH + 64;          // row stride inside a stage
constexpr int STAGE_BYTES = 16 * RS;
constexpr int NST = 3;               // stages per warp
constexpr int BAR_BYTES = 512;       // DW * NST barriers
constexpr int ATT_MAX_HD = 128;
constexpr int ATT_MAX_SPLITS = 16;
constexpr long long WAIT_CYCLES = 2000000000ll;
constexpr uint32_t DECODER_MAGIC = 0x4b423244u;  // "KB2D"

struct DecLayer {
    LayerRef qkv, o, gu, down;  // packed rows: q|k|v concatenated; gate_i, up_i interleaved
    const float *g1, *g2;       // RMSNorm weights
    float *kc, *vc;             // KV cache, head-major: [batch][heads][max_len][hd]
};

struct DecodeParams {
    const DecLayer *layers;
    int n_layers, batch, d, f, n_heads, hd, vocab, max_len;
    float eps;
    const float *embed, *lm_head, *norm_f, *cos_t, *sin_t;
    long long *tokens;       // [batch] in: tokens of this step, out: tokens chosen by it
    int *positions, *lens;   // [batch] advanced by one at the end of the step
    long long *cache_rows;   // [batch] row of the flattened cache the new k / v go to; advanced too
    float *hidden, *qkv, *attn, *h, *absmax, *logits;
    float *att_scratch;      // [batch * heads][splits][2 + ATT_MAX_HD]
    int *att_counters;       // [batch * heads], zero between steps
    unsigned *barrier;       // arrival counter, zero at launch
    unsigned long long *best;  // [batch] argmax keys, zero at launch
    int *status;
    int ks_qkv, ks_o, ks_gu, ks_down, att_splits;
    int xs_stride;
};

// ---- small PTX helpers (same as the streaming GEMV) ----
template <int DST_OFF>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1], 16;" ::"r"(dst), "l"(src), "n"(DST_OFF) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}
__device__ __forceinline__ int xs_offset(int o) { return (o & ~255) | ((o & 0x30) << 2) | ((o & 0xc0) >> 2); }

__device__ __forceinline__ bool aborted(const int *status) { return *reinterpret_cast<const volatile int *>(status) != 0; }

__device__ __forceinline__ bool wait_stage(uint32_t bar, uint32_t parity, int *status) {
    long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u) {
            if (aborted(status)) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_CYCLES) { atomicCAS(status, 0, 30); return false; }
        }
    }
}

// All CTAs of the (cooperative) grid meet: arrival counter in global memory, `target` grows by the
// grid size per barrier.  Bounded; on expiry (or when another wait already gave up) it returns false.
__device__ __forceinline__ bool grid_barrier(const DecodeParams &p, unsigned &target) {
    __syncthreads();
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        target += gridDim.x;
        // release: this CTA's writes of the finished phase (ordered before by the CTA barrier) become visible
        // to whoever acquires the counter
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.barrier) : "memory");
        bool ok = true;
        long long t0 = 0;
        for (uint32_t i = 0;; ++i) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.barrier) : "memory");
            if ((int)(v - target) >= 0) break;
            if ((i & 255u) == 255u) {
                if (aborted(p.status)) { ok = false; break; }
                const long long now = clock64();
                if (t0 == 0) t0 = now;
                else if (now - t0 > WAIT_CYCLES) { atomicCAS(p.status, 0, 31); ok = false; break; }
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    return s_ok != 0;
}

// ---- block-wide reductions: one CTA barrier each; every thread combines the per-warp partials itself in
// a fixed order.  `red` must not be rewritten before the next CTA barrier (callers alternate two arrays). ----
__device__ __forceinline__ float block_sum_f(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < DW; ++w) r += red[w];
    return r;
}
__device__ __forceinline__ float block_max_f(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < DW; ++w) r = fmaxf(r, red[w]);
    return r;
}
// the row's code sum is only needed by the projection's epilogue: one shared-memory atomic per warp, completed
// by the CTA barrier that ends the prologue
__device__ __forceinline__ void warp_add_to(int v, int *dst) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(dst, v);
}

// ---- activation prologues: one f32 row -> int8 codes in the staged (transposed-cell) layout ----
// MODE 0: x;  MODE 1: rmsnorm(x) * gamma;  MODE 2: x with a known max|x| (no reduction).
// cells = 16-byte cells to write (codes beyond k are zero).  Rows up to 12 * DTHREADS elements.
constexpr int PRO_V4 = 3;  // float4 per thread held in registers (rows up to 4608 elements) for MODE 0 / 1
template <int MODE>
__device__ __forceinline__ void stage_row(const float *row, const float *gamma, float eps, float known_absmax, int k,
                                          uint8_t *dst, int cells, float *sx_out, int *sum_out, float *red_f) {
    const int nv4 = k >> 2;  // k % 4 == 0 (checked by the host)
    float s;
    int local = 0;
    if (threadIdx.x == 0) *sum_out = 0;
    if (MODE == 2) __syncthreads();  // no reduction follows in this mode: order the zeroing before the adds
    if (MODE == 2 || nv4 > PRO_V4 * DTHREADS) {
        // streaming form: the scale is known (MODE 2), or two passes over the row
        float amax = known_absmax;
        float inv = 1.0f;
        if (MODE == 1) {
            float ss = 0.0f;
            for (int i = threadIdx.x; i < nv4; i += DTHREADS) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + i);
                ss += __fmul_rn(v.x, v.x) + __fmul_rn(v.y, v.y) + __fmul_rn(v.z, v.z) + __fmul_rn(v.w, v.w);
            }
            ss = block_sum_f(ss, red_f);
            inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)k), eps)));
        }
        auto value = [&](int i) {
            float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + i);
            if (MODE == 1) {
                const float4 gm = reinterpret_cast<const float4 *>(gamma)[i];
                v.x = __fmul_rn(__fmul_rn(v.x, inv), gm.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), gm.y);
                v.z = __fmul_rn(__fmul_rn(v.z, inv), gm.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), gm.w);
            }
            return v;
        };
        if (MODE != 2) {
            amax = 0.0f;
            for (int i = threadIdx.x; i < nv4; i += DTHREADS) {
                const float4 v = value(i);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
            amax = block_max_f(amax, red_f + 16);
        }
        s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
        const float rs = __frcp_rn(s);
        for (int i = threadIdx.x; i < cells * 4; i += DTHREADS) {  // word i = codes 4i .. 4i + 3
            uint32_t word = 0;
            if (i < nv4) {
                const float4 v = value(i);
                const int q0 = quantise_one_fast(v.x, s, rs), q1 = quantise_one_fast(v.y, s, rs);
                const int q2 = quantise_one_fast(v.z, s, rs), q3 = quantise_one_fast(v.w, s, rs);
                local += q0 + q1 + q2 + q3;
                word = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
            }
            *reinterpret_cast<uint32_t *>(dst + xs_offset((i >> 2) << 4) + ((i & 3) << 2)) = word;
        }
    } else {
        // single pass: the row sits in registers between the reductions
        float4 v[PRO_V4], gm[PRO_V4];
#pragma unroll
        for (int j = 0; j < PRO_V4; ++j) {
            const int i = threadIdx.x + j * DTHREADS;
            v[j] = i < nv4 ? __ldcg(reinterpret_cast<const float4 *>(row) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            // the norm weights travel with the row: one memory round trip instead of a second one after the reduction
            if (MODE == 1) gm[j] = i < nv4 ? reinterpret_cast<const float4 *>(gamma)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (MODE == 1) {
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < PRO_V4; ++j)
                ss += __fmul_rn(v[j].x, v[j].x) + __fmul_rn(v[j].y, v[j].y) + __fmul_rn(v[j].z, v[j].z) + __fmul_rn(v[j].w, v[j].w);
            ss = block_sum_f(ss, red_f);
            const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)k), eps)));
#pragma unroll
            for (int j = 0; j < PRO_V4; ++j) {
                const int i = threadIdx.x + j * DTHREADS;
                if (i < nv4) {
                    v[j].x = __fmul_rn(__fmul_rn(v[j].x, inv), gm[j].x); v[j].y = __fmul_rn(__fmul_rn(v[j].y, inv), gm[j].y);
                    v[j].z = __fmul_rn(__fmul_rn(v[j].z, inv), gm[j].z); v[j].w = __fmul_rn(__fmul_rn(v[j].w, inv), gm[j].w);
                }
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < PRO_V4; ++j)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
        amax = block_max_f(amax, red_f + 16);
        s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
        const float rs = __frcp_rn(s);
#pragma unroll
        for (int j = 0; j < PRO_V4; ++j) {
            const int i = threadIdx.x + j * DTHREADS;
            if (i < cells * 4) {
                uint32_t word = 0;
                if (i < nv4) {
                    const int q0 = quantise_one_fast(v[j].x, s, rs), q1 = quantise_one_fast(v[j].y, s, rs);
                    const int q2 = quantise_one_fast(v[j].z, s, rs), q3 = quantise_one_fast(v[j].w, s, rs);
                    local += q0 + q1 + q2 + q3;
                    word = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                }
                *reinterpret_cast<uint32_t *>(dst + xs_offset((i >> 2) << 4) + ((i & 3) << 2)) = word;
            }
        }
        // cells beyond what the registers cover (padding up to the last chunk): zero
        for (int i = threadIdx.x + PRO_V4 * DTHREADS; i < cells * 4; i += DTHREADS)
            *reinterpret_cast<uint32_t *>(dst + xs_offset((i >> 2) << 4) + ((i & 3) << 2)) = 0u;
    }
    warp_add_to(local, sum_out);  // *sum_out was zeroed before the reductions above
    if (threadIdx.x == 0) *sx_out = s;
}

// ---- one GEMV phase ----
// EPI 0: y[t][row] = v;  EPI 1: y[t][row] = v + resid[t][row];  EPI 2: rows alternate gate_i, up_i ->
// y[t][row / 2] = silu(gate) * up and max|.| into absmax[t] (atomic max on the float bits).
struct Gemv {
    LayerRef L;
    int m, kp, ks;
    size_t row_bytes;
    // cursor state of the producer, kept across the barrier that precedes the phase
    int p_rb, p_c;
    bool p_valid;
    const uint8_t *p_src;
    uint32_t fs;  // stage the next fill goes to (the ring continues across phases)
};

struct Ctx {
    int lane, warp;
    uint32_t bar0, stage0, lane_dst, xs_addr;
    uint8_t *xs;
    int *part;
    float *s_sx;
    int *s_sum;
    float *red_f;
    uint32_t cs, cph;  // consumer's next stage and its barrier phase (continue across phases)
};

__device__ __forceinline__ void gemv_setup(Gemv &g, const LayerRef &L, int m, int kp, int ks, const Ctx &c) {
    g.L = L; g.m = m; g.kp = kp; g.ks = ks; g.row_bytes = (size_t)kp / 4;
    const int gp = DW / ks, gi = c.warp / ks;
    g.p_rb = (int)blockIdx.x * gp + gi;
    const int nchunks = (int)((g.row_bytes + CH - 1) / CH), slice = c.warp % ks;
    g.p_c = slice * nchunks / ks;
    g.p_valid = g.p_rb < (m + 15) / 16;
    g.p_src = L.w2 + (size_t)(g.p_rb * 16 + (c.lane >> 4)) * g.row_bytes + (c.lane & 15) * 16;
}

// one stage of the current unit; advances the producer cursor
__device__ __forceinline__ void gemv_fill(Gemv &g, const Ctx &c) {
    if (!g.p_valid) return;
    const int nchunks = (int)((g.row_bytes + CH - 1) / CH), slice = c.warp % g.ks;
    const int c_first = slice * nchunks / g.ks, c_last = (slice + 1) * nchunks / g.ks;
    const uint32_t dst = c.lane_dst + g.fs * STAGE_BYTES, bar = c.bar0 + 8 * g.fs;
    g.fs = g.fs + 1 == NST ? 0 : g.fs + 1;
    const int off = g.p_c * CH;
    if ((c.lane & 15) * 16 < (int)g.row_bytes - off) {
        const uint8_t *src = g.p_src + off;
        const size_t two_rows = 2 * g.row_bytes;
        cp_async16<0 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<1 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<2 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<3 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<4 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<5 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<6 * 2 * RS>(dst, src); src += two_rows;
        cp_async16<7 * 2 * RS>(dst, src);
    }
    cp_async_arrive(bar);
    if (++g.p_c == c_last) {
        g.p_c = c_first;
        const int step = (int)gridDim.x * (DW / g.ks);
        g.p_rb += step;
        g.p_valid = g.p_rb < (g.m + 15) / 16;
        g.p_src += (size_t)step * 16 * g.row_bytes;
    }
}

// y[tk] / resid[tk]: token tk's output row and residual row (EPI 1)
template <int NT, int EPI>
__device__ __forceinline__ void gemv_run(Gemv &g, Ctx &c, const DecodeParams &p, float *const (&y)[NT],
                                         const float *const (&resid)[NT], unsigned int *absmax_smem) {
    const int lane = c.lane, warp = c.warp, ks = g.ks;
    const int gp = DW / ks, gi = warp / ks, slice = warp % ks;
    const int nchunks = (int)((g.row_bytes + CH - 1) / CH);
    const int c_first = slice * nchunks / ks, c_last = (slice + 1) * nchunks / ks;
    const int row_blocks = (g.m + 15) / 16;
    const int my_row = (lane >> 4) + 2 * ((lane >> 1) & 7);
    int acc[8 * NT * 4];
#pragma unroll
    for (int i = 0; i < 8 * NT * 4; ++i) acc[i] = 0;
    int parity = 0;
    bool ok = !aborted(p.status);
    for (int rb = (int)blockIdx.x * gp + gi; rb < row_blocks; rb += (int)gridDim.x * gp) {
        const int row = rb * 16 + my_row;  // rows up to m_alloc - 1 are allocated
        const float sw = g.L.sw[row];
        for (int ch = c_first; ch < c_last; ++ch) {
            if (ok && !(ok = wait_stage(c.bar0 + 8 * c.cs, c.cph, p.status))) g.p_valid = false;
            if (ok) {
                const int cc = lane & 15;
                const uint32_t xcol = (uint32_t)(ch * CH * 4) + 256 * (cc >> 2) + 16 * (cc & 3);
                uint32_t xr[NT][16];
#pragma unroll
                for (int tk = 0; tk < NT; ++tk) {
                    const uint32_t xb = c.xs_addr + (uint32_t)(tk * p.xs_stride) + xcol;
                    const uint4 v0 = lds128<0>(xb), v1 = lds128<64>(xb), v2 = lds128<128>(xb), v3 = lds128<192>(xb);
                    xr[tk][0] = v0.x; xr[tk][1] = v0.y; xr[tk][2] = v0.z; xr[tk][3] = v0.w;
                    xr[tk][4] = v1.x; xr[tk][5] = v1.y; xr[tk][6] = v1.z; xr[tk][7] = v1.w;
                    xr[tk][8] = v2.x; xr[tk][9] = v2.y; xr[tk][10] = v2.z; xr[tk][11] = v2.w;
                    xr[tk][12] = v3.x; xr[tk][13] = v3.y; xr[tk][14] = v3.z; xr[tk][15] = v3.w;
                }
                const uint32_t wb = c.lane_dst + c.cs * STAGE_BYTES;
                uint4 wrow[8];
                wrow[0] = lds128<0 * 2 * RS>(wb); wrow[1] = lds128<1 * 2 * RS>(wb); wrow[2] = lds128<2 * 2 * RS>(wb);
                wrow[3] = lds128<3 * 2 * RS>(wb); wrow[4] = lds128<4 * 2 * RS>(wb); wrow[5] = lds128<5 * 2 * RS>(wb);
                wrow[6] = lds128<6 * 2 * RS>(wb); wrow[7] = lds128<7 * 2 * RS>(wb);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t ww[4] = {wrow[i].x, wrow[i].y, wrow[i].z, wrow[i].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t a = ww[q] & (0x03030303u << (2 * j));
#pragma unroll
                            for (int tk = 0; tk < NT; ++tk)
                                acc[(i * NT + tk) * 4 + j] = dp4a_u8s8(a, xr[tk][4 * q + j], acc[(i * NT + tk) * 4 + j]);
                        }
                }
            }
            __syncwarp();
            gemv_fill(g, c);
            if (ok && ++c.cs == NST) { c.cs = 0; c.cph ^= 1u; }
        }
        // ---- unit finished: combine the scaled accumulators, transposing reduction over the 16 lanes of a row ----
        int v[NT];
#pragma unroll
        for (int tk = 0; tk < NT; ++tk) {
            int sres[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int b = (i * NT + tk) * 4;
                sres[i] = acc[b] + (acc[b + 1] >> 2) + (acc[b + 2] >> 4) + (acc[b + 3] >> 6);
                acc[b] = acc[b + 1] = acc[b + 2] = acc[b + 3] = 0;
            }
            const bool h8 = (lane & 8) != 0, h4 = (lane & 4) != 0, h2 = (lane & 2) != 0;
            int a4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) a4[j] = (h8 ? sres[4 + j] : sres[j]) + __shfl_xor_sync(0xffffffffu, h8 ? sres[j] : sres[4 + j], 8);
            int b2[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) b2[j] = (h4 ? a4[2 + j] : a4[j]) + __shfl_xor_sync(0xffffffffu, h4 ? a4[j] : a4[2 + j], 4);
            int dd = (h2 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, h2 ? b2[0] : b2[1], 2);
            dd += __shfl_xor_sync(0xffffffffu, dd, 1);
            v[tk] = dd;
        }
        bool finisher = true;
        if (ks > 1) {
            int *mine = c.part + (size_t)((gi * 2 + parity) * ks + slice) * (NT * 32);
#pragma unroll
            for (int tk = 0; tk < NT; ++tk) mine[tk * 32 + lane] = v[tk];
            asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
            finisher = slice == 0;
            if (finisher) {
                const int *base = c.part + (size_t)((gi * 2 + parity) * ks) * (NT * 32);
#pragma unroll
                for (int tk = 0; tk < NT; ++tk) {
                    int sum = 0;
                    for (int q = 0; q < ks; ++q) sum += base[q * (NT * 32) + tk * 32 + lane];
                    v[tk] = sum;
                }
            }
            parity ^= 1;
        }
        if (finisher) {
#pragma unroll
            for (int tk = 0; tk < NT; ++tk) {
                // ternary codes: value = code - 1 -> acc = S - sum(xq)
                const int a = v[tk] - c.s_sum[tk];
                float out = __fmul_rn(__fmul_rn(__int2float_rn(a), sw), c.s_sx[tk]);
                if (EPI == 2) {
                    // lanes h = 0 hold gate rows (even), h = 1 the matching up rows: partner = lane ^ 16
                    const float up = __shfl_xor_sync(0xffffffffu, out, 16);
                    if ((lane & 17) == 0 && row + 1 < g.m && tk < p.batch) {
                        const float silu = __fdiv_rn(out, __fadd_rn(1.0f, expf(-out)));
                        const float hv = __fmul_rn(silu, up);
                        y[tk][row >> 1] = hv;
                        atomicMax(absmax_smem + tk, __float_as_uint(fabsf(hv)));  // CTA-local; one global atomic per CTA later
                    }
                } else if ((lane & 1) == 0 && row < g.m && tk < p.batch) {
                    if (EPI == 1) out = __fadd_rn(out, __ldcg(resid[tk] + row));
                    y[tk][row] = out;
                }
            }
        }
    }
}

// ---- phase B: RoPE + cache append + attention of the new token, work item = (sequence, head, split) ----
// The item's keys and values (a contiguous block of the head-major cache) are staged in shared memory with
// 16-byte asynchronous copies, all in flight at once: with almost all of the SM's memory configured as shared
// memory the L1 is a few KB, and register loads (which allocate there) were throttled to ~10 GB/s per SM.
// The staging area is the warps' stage rings, which are empty between two GEMV phases.
// Each warp then takes positions in turn (lanes over the head's dims) with a running (max, sum) and a rescaled
// value accumulator; per-warp partials meet in shared memory, per-item partials in att_scratch, and the last
// item of a head to finish — found with a self-resetting counter — merges them and writes the output.
__device__ void attention_phase(const DecodeParams &p, const DecLayer &L, float *smem_f, float *kv_stage, int kv_floats,
                                const int *s_pos, const float *s_cs, int *s_flag) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int d = p.d, hd = p.hd, half = hd / 2, splits = p.att_splits;
    float *s_q = smem_f, *s_k = smem_f + ATT_MAX_HD;                 // rotated q and k of the new token
    float *s_m = smem_f + 2 * ATT_MAX_HD, *s_l = s_m + DW, *s_acc = s_l + DW;  // per-warp partials [DW][ATT_MAX_HD]
    const int items = p.batch * p.n_heads * splits;
    const int cap = kv_floats / (2 * hd);  // positions that fit in the staging area (keys then values)
    constexpr int DPL = ATT_MAX_HD / 32;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int bh = item / splits, sp = item - bh * splits;
        const int b = bh / p.n_heads, h = bh - b * p.n_heads;
        const int pos = s_pos[b], len = pos + 1;
        const float *qkv = p.qkv + (size_t)b * 3 * d;
        const int chunk = (len + splits - 1) / splits;
        const int j0 = sp * chunk, j1 = min(len, j0 + chunk);
        float *kc = L.kc + ((size_t)b * p.n_heads + h) * p.max_len * hd, *vc = L.vc + ((size_t)b * p.n_heads + h) * p.max_len * hd;
        __syncthreads();  // the previous item's shared values are no longer read
        float qv[DPL], acc[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        const float scale = __fdiv_rn(1.0f, sqrtf((float)hd));
        for (int c0 = j0; c0 < j1; c0 += cap) {
            const int c1 = min(j1, c0 + cap), np = c1 - c0;
            float *sk = kv_stage, *sv = kv_stage + (size_t)cap * hd;
            // stage positions [c0, c1): the block is contiguous in the cache (rows of hd floats, hd % 4 == 0)
            const int cells = np * hd / 4;
            const uint32_t sk_addr = smem_u32(sk), sv_addr = smem_u32(sv);
            for (int i = threadIdx.x; i < cells; i += DTHREADS) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sk_addr + 16 * i), "l"(kc + (size_t)c0 * hd + 4 * i) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sv_addr + 16 * i), "l"(vc + (size_t)c0 * hd + 4 * i) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (c0 == j0 && (int)threadIdx.x < half) {  // meanwhile: rotate the new token's q and k
                const int i = threadIdx.x;
                const float cs = s_cs[b * ATT_MAX_HD + i], sn = s_cs[b * ATT_MAX_HD + half + i];
                const int a = h * hd + i, bb = a + half;
                const float q0 = __ldcg(qkv + a), q1 = __ldcg(qkv + bb), k0 = __ldcg(qkv + d + a), k1 = __ldcg(qkv + d + bb);
                s_q[i] = __fsub_rn(__fmul_rn(q0, cs), __fmul_rn(q1, sn));
                s_q[i + half] = __fadd_rn(__fmul_rn(q0, sn), __fmul_rn(q1, cs));
                s_k[i] = __fsub_rn(__fmul_rn(k0, cs), __fmul_rn(k1, sn));
                s_k[i + half] = __fadd_rn(__fmul_rn(k0, sn), __fmul_rn(k1, cs));
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            if (pos >= c0 && pos < c1 && (int)threadIdx.x < hd) {
                // the new position: its key / value are not in the cache yet — take them from this step, and store them
                const float kn = s_k[threadIdx.x], vn = __ldcg(qkv + 2 * d + h * hd + threadIdx.x);
                sk[(size_t)(pos - c0) * hd + threadIdx.x] = kn;
                sv[(size_t)(pos - c0) * hd + threadIdx.x] = vn;
                kc[(size_t)pos * hd + threadIdx.x] = kn;
                vc[(size_t)pos * hd + threadIdx.x] = vn;
            }
            __syncthreads();
            if (c0 == j0) {
#pragma unroll
                for (int i = 0; i < DPL; ++i) qv[i] = 4 * lane + i < hd ? s_q[4 * lane + i] : 0.0f;
            }
            for (int j = warp; j < np; j += DW) {
                float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
                if (4 * lane < hd) {
                    k4 = *reinterpret_cast<const float4 *>(sk + (size_t)j * hd + 4 * lane);
                    v4 = *reinterpret_cast<const float4 *>(sv + (size_t)j * hd + 4 * lane);
                }
                float dot = fmaf(qv[3], k4.w, fmaf(qv[2], k4.z, fmaf(qv[1], k4.y, fmaf(qv[0], k4.x, 0.0f))));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                dot *= scale;
                const float m_new = fmaxf(m, dot);
                const float corr = expf(m - m_new), pj = expf(dot - m_new);
                l = l * corr + pj;
                acc[0] = fmaf(pj, v4.x, acc[0] * corr); acc[1] = fmaf(pj, v4.y, acc[1] * corr);
                acc[2] = fmaf(pj, v4.z, acc[2] * corr); acc[3] = fmaf(pj, v4.w, acc[3] * corr);
                m = m_new;
            }
            if (c1 < j1) __syncthreads();  // the staging area is rewritten by the next chunk
        }
        if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
        for (int i = 0; i < DPL; ++i)
            if (4 * lane + i < ATT_MAX_HD) s_acc[warp * ATT_MAX_HD + 4 * lane + i] = acc[i];
        __syncthreads();
        float cm = -INFINITY;
        for (int w = 0; w < DW; ++w) cm = fmaxf(cm, s_m[w]);
        float cl = 0.0f, ca = 0.0f;
        if ((int)threadIdx.x < hd) {
            for (int w = 0; w < DW; ++w) {
                const float f = s_m[w] == -INFINITY ? 0.0f : expf(s_m[w] - cm);
                cl += s_l[w] * f;
                ca += s_acc[w * ATT_MAX_HD + threadIdx.x] * f;
            }
        }
        float *out = p.attn + (size_t)b * d + h * hd;
        if (splits == 1) {
            if ((int)threadIdx.x < hd) out[threadIdx.x] = ca * __fdiv_rn(1.0f, cl);
            continue;
        }
        float *part = p.att_scratch + ((size_t)bh * splits + sp) * (2 + ATT_MAX_HD);
        if (threadIdx.x == 0) { part[0] = cm; part[1] = cl; }
        if ((int)threadIdx.x < hd) part[2 + threadIdx.x] = ca;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();  // cumulative: the CTA's partial (ordered before by the barrier) is visible before the ticket
            const int ticket = atomicAdd(p.att_counters + bh, 1);
            *s_flag = (ticket == splits - 1);
            if (*s_flag) p.att_counters[bh] = 0;
        }
        __syncthreads();
        if (!*s_flag) continue;
        __threadfence();
        const float *base = p.att_scratch + (size_t)bh * splits * (2 + ATT_MAX_HD);
        float gm = -INFINITY;
        for (int s2 = 0; s2 < splits; ++s2) gm = fmaxf(gm, __ldcg(base + s2 * (2 + ATT_MAX_HD)));
        if ((int)threadIdx.x < hd) {
            float gl = 0.0f, ga = 0.0f;
            for (int s2 = 0; s2 < splits; ++s2) {
                const float *ps = base + s2 * (2 + ATT_MAX_HD);
                const float pm = __ldcg(ps);
                const float f = pm == -INFINITY ? 0.0f : expf(pm - gm);
                gl += __ldcg(ps + 1) * f;
                ga += __ldcg(ps + 2 + threadIdx.x) * f;
            }
            out[threadIdx.x] = ga * __fdiv_rn(1.0f, gl);
        }
    }
}

// ---- final phase: RMSNorm, dense f32 lm_head (one warp per vocabulary row at a time), argmax ----
// key = (order-preserving bits of the logit) << 32 | ~index: the maximum key is the largest logit, lowest index on ties
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned)idx);
}

template <int NT>
__device__ void head_phase(const DecodeParams &p, float *xn /* smem [NT][d] */, float *red_f) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int d = p.d, nv4 = d >> 2;
    for (int tk = 0; tk < NT; ++tk) {
        const float *row = p.hidden + (size_t)min(tk, p.batch - 1) * d;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < nv4; i += DTHREADS) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + i);
            ss += __fmul_rn(v.x, v.x) + __fmul_rn(v.y, v.y) + __fmul_rn(v.z, v.z) + __fmul_rn(v.w, v.w);
        }
        ss = block_sum_f(ss, red_f + 16 * (tk & 1));
        const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)d), p.eps)));
        for (int i = threadIdx.x; i < nv4; i += DTHREADS) {
            float4 v = __ldcg(reinterpret_cast<const float4 *>(row) + i);
            const float4 gm = reinterpret_cast<const float4 *>(p.norm_f)[i];
            v.x = __fmul_rn(__fmul_rn(v.x, inv), gm.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), gm.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv), gm.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), gm.w);
            reinterpret_cast<float4 *>(xn + (size_t)tk * d)[i] = v;
        }
    }
    __syncthreads();
    unsigned long long best[NT];
#pragma unroll
    for (int tk = 0; tk < NT; ++tk) best[tk] = 0ull;
    const int gw = blockIdx.x * DW + warp, nw = gridDim.x * DW;
    constexpr int UN = 8;  // float4 loads of a weight row in flight per lane
    for (int v0 = gw; v0 < p.vocab; v0 += nw) {
        const float4 *wrow = reinterpret_cast<const float4 *>(p.lm_head + (size_t)v0 * d);
        float sum[NT];
#pragma unroll
        for (int tk = 0; tk < NT; ++tk) sum[tk] = 0.0f;
        for (int i0 = lane; i0 < nv4; i0 += 32 * UN) {
            float4 w[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int i = i0 + 32 * u;
                w[u] = i < nv4 ? __ldcs(wrow + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int i = i0 + 32 * u;
                if (i < nv4) {
#pragma unroll
                    for (int tk = 0; tk < NT; ++tk) {
                        const float4 x = reinterpret_cast<const float4 *>(xn + (size_t)tk * d)[i];
                        sum[tk] = fmaf(w[u].x, x.x, sum[tk]); sum[tk] = fmaf(w[u].y, x.y, sum[tk]);
                        sum[tk] = fmaf(w[u].z, x.z, sum[tk]); sum[tk] = fmaf(w[u].w, x.w, sum[tk]);
                    }
                }
            }
        }
#pragma unroll
        for (int tk = 0; tk < NT; ++tk) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum[tk] += __shfl_xor_sync(0xffffffffu, sum[tk], o);
            if (tk < p.batch) {
                if (lane == 0 && p.logits) p.logits[(size_t)tk * p.vocab + v0] = sum[tk];
                const unsigned long long key = argmax_key(sum[tk], v0);
                best[tk] = key > best[tk] ? key : best[tk];
            }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int tk = 0; tk < NT; ++tk)
            if (tk < p.batch && best[tk]) atomicMax(p.best + tk, best[tk]);
    }
}

template <int NT>
__global__ void __launch_bounds__(DTHREADS, 1) decode_step_kernel(const DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ float s_sx[2];
    __shared__ int s_sum[2];
    __shared__ float red_f[32];
    __shared__ int s_pos[2];
    __shared__ int s_flag;
    __shared__ unsigned int s_amax[2];
    __shared__ float s_cs[2 * ATT_MAX_HD];  // cos | sin of each sequence's position

    Ctx c;
    c.lane = threadIdx.x & 31; c.warp = threadIdx.x >> 5;
    const uint32_t smem_base = smem_u32(smem);
    c.bar0 = smem_base + (uint32_t)(c.warp * NST * 8);
    c.stage0 = smem_base + BAR_BYTES + (uint32_t)(c.warp * NST * STAGE_BYTES);
    c.lane_dst = c.stage0 + (c.lane >> 4) * RS + (c.lane & 15) * 16;
    c.xs = smem + BAR_BYTES + (size_t)DW * NST * STAGE_BYTES;
    c.xs_addr = smem_base + BAR_BYTES + (uint32_t)(DW * NST * STAGE_BYTES);
    c.part = reinterpret_cast<int *>(c.xs + (size_t)NT * p.xs_stride);
    c.s_sx = s_sx; c.s_sum = s_sum; c.red_f = red_f;
    c.cs = 0; c.cph = 0;
    float *scratch_f = reinterpret_cast<float *>(c.xs);  // attention / lm_head phases reuse the activation rows' space

    if (c.lane == 0) {
        for (int s = 0; s < NST; ++s) mbar_init(c.bar0 + 8 * s, 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const int d = p.d, f = p.f;
    const int kp_d = (d + 127) / 128 * 128, kp_f = (f + 127) / 128 * 128;
    unsigned target = 0;
    Gemv g;
    g.fs = 0;
    bool alive = true;
    auto prefetch = [&](const LayerRef &L, int m, int kp, int ks) {
        gemv_setup(g, L, m, kp, ks, c);
        for (int s = 0; s < NST; ++s) gemv_fill(g, c);
    };
    auto cells_for = [&](int kp) { return (int)(((size_t)kp / 4 + CH - 1) / CH) * 64; };

    if (blockIdx.x == 0 && threadIdx.x < 2) p.absmax[threadIdx.x] = 0.0f;  // layer 0's slots (used after three barriers)
    if (threadIdx.x < 2) { s_pos[threadIdx.x] = p.positions[min((int)threadIdx.x, p.batch - 1)]; s_amax[threadIdx.x] = 0u; }
    for (int i = threadIdx.x; i < NT * p.hd; i += DTHREADS) {
        const int b = min(i / p.hd, p.batch - 1), r = i % p.hd, half = p.hd / 2;
        const size_t row = (size_t)p.positions[b] * half;
        s_cs[(i / p.hd) * ATT_MAX_HD + r] = r < half ? p.cos_t[row + r] : p.sin_t[row + r - half];
    }
    __syncthreads();
    prefetch(p.layers[0].qkv, 3 * d, kp_d, p.ks_qkv);
    for (int li = 0; li < p.n_layers && alive; ++li) {
        const DecLayer &L = p.layers[li];
        const bool first = li == 0;
        // ---- A: qkv = W_qkv . quantise(rmsnorm(hidden) * g1) ----
        for (int tk = 0; tk < NT; ++tk) {
            const int b = min(tk, p.batch - 1);
            const float *row = first ? p.embed + (size_t)p.tokens[b] * d : p.hidden + (size_t)b * d;
            stage_row<1>(row, L.g1, p.eps, 0.0f, d, c.xs + (size_t)tk * p.xs_stride, cells_for(kp_d), s_sx + tk, s_sum + tk, red_f);
        }
        __syncthreads();
        float *y_rows[NT];
        const float *r_rows[NT];
        for (int tk = 0; tk < NT; ++tk) { y_rows[tk] = p.qkv + (size_t)tk * 3 * d; r_rows[tk] = nullptr; }
        gemv_run<NT, 0>(g, c, p, y_rows, r_rows, nullptr);
        if (!(alive = grid_barrier(p, target))) break;
        // ---- B: attention (stages keys and values in the empty stage rings; the next phase's weights follow) ----
        attention_phase(p, L, scratch_f, reinterpret_cast<float *>(smem + BAR_BYTES), DW * NST * STAGE_BYTES / 4, s_pos, s_cs, &s_flag);
        __syncthreads();
        prefetch(L.o, d, kp_d, p.ks_o);
        if (!(alive = grid_barrier(p, target))) break;
        // ---- C: hidden (+)= W_o . quantise(attn) ----
        for (int tk = 0; tk < NT; ++tk)
            stage_row<0>(p.attn + (size_t)min(tk, p.batch - 1) * d, nullptr, 0.0f, 0.0f, d, c.xs + (size_t)tk * p.xs_stride,
                         cells_for(kp_d), s_sx + tk, s_sum + tk, red_f);
        __syncthreads();
        // the residual stream starts at the embedding rows: the first layer adds to them and materialises hidden
        for (int tk = 0; tk < NT; ++tk) {
            const int b = min(tk, p.batch - 1);
            y_rows[tk] = p.hidden + (size_t)tk * d;
            r_rows[tk] = first ? p.embed + (size_t)p.tokens[b] * d : p.hidden + (size_t)tk * d;
        }
        gemv_run<NT, 1>(g, c, p, y_rows, r_rows, nullptr);
        prefetch(L.gu, 2 * f, kp_d, p.ks_gu);
        if (!(alive = grid_barrier(p, target))) break;
        // ---- D: h = silu(gate) * up of W_gu . quantise(rmsnorm(hidden) * g2), max|h| ----
        float *am = p.absmax + (size_t)(li & 1) * 2, *am_other = p.absmax + (size_t)((li + 1) & 1) * 2;
        for (int tk = 0; tk < NT; ++tk)
            stage_row<1>(p.hidden + (size_t)min(tk, p.batch - 1) * d, L.g2, p.eps, 0.0f, d, c.xs + (size_t)tk * p.xs_stride,
                         cells_for(kp_d), s_sx + tk, s_sum + tk, red_f);
        __syncthreads();
        for (int tk = 0; tk < NT; ++tk) { y_rows[tk] = p.h + (size_t)tk * f; r_rows[tk] = nullptr; }
        gemv_run<NT, 2>(g, c, p, y_rows, r_rows, s_amax);
        __syncthreads();
        if ((int)threadIdx.x < NT && threadIdx.x < (unsigned)p.batch) {
            if (s_amax[threadIdx.x]) atomicMax(reinterpret_cast<unsigned int *>(am) + threadIdx.x, s_amax[threadIdx.x]);
            s_amax[threadIdx.x] = 0u;
        }
        prefetch(L.down, d, kp_f, p.ks_down);
        if (!(alive = grid_barrier(p, target))) break;
        // ---- E: hidden += W_down . quantise(h) with the known max|h| ----
        if (blockIdx.x == 0 && threadIdx.x < 2) am_other[threadIdx.x] = 0.0f;  // the next layer's slots
        for (int tk = 0; tk < NT; ++tk)
            stage_row<2>(p.h + (size_t)min(tk, p.batch - 1) * f, nullptr, 0.0f, __ldcg(am + min(tk, p.batch - 1)), f,
                         c.xs + (size_t)tk * p.xs_stride, cells_for(kp_f), s_sx + tk, s_sum + tk, red_f);
        __syncthreads();
        for (int tk = 0; tk < NT; ++tk) { y_rows[tk] = p.hidden + (size_t)tk * d; r_rows[tk] = y_rows[tk]; }
        gemv_run<NT, 1>(g, c, p, y_rows, r_rows, nullptr);
        if (li + 1 < p.n_layers) prefetch(p.layers[li + 1].qkv, 3 * d, kp_d, p.ks_qkv);
        if (!(alive = grid_barrier(p, target))) break;
    }
    if (!alive) return;
    // ---- head ----
    head_phase<NT>(p, scratch_f, red_f);
    if (!grid_barrier(p, target)) return;
    if (blockIdx.x == 0 && (int)threadIdx.x < p.batch) {
        const int b = threadIdx.x;
        const unsigned long long key = *reinterpret_cast<volatile unsigned long long *>(p.best + b);
        p.tokens[b] = (long long)(0xffffffffu - (unsigned)(key & 0xffffffffull));
        p.best[b] = 0ull;
        p.positions[b] += 1;
        p.lens[b] += 1;
        p.cache_rows[b] += 1;
    }
}

struct Decoder {
    uint32_t magic;
    int device, batch, sms;
    DecodeParams p;
    DecLayer *layers_dev;
    void *misc;  // one allocation: qkv, attn, h, absmax, att scratch, counters, barrier, best, status
    size_t smem;
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int pick_ks(int row_blocks, int nchunks, int sms) {
    // slices per row block: a divisor of the warps per CTA, at most the chunks per row; prefer the smallest
    // number of rounds over the CTA's warp groups, then the fewest chunks per warp
    const int cand[6] = {1, 2, 3, 4, 6, 12};
    int best = 1;
    long long best_cost = -1;
    for (int i = 0; i < 6; ++i) {
        const int ks = cand[i];
        if (ks > nchunks) break;
        const long long groups = (long long)sms * (DW / ks);
        const long long rounds = (row_blocks + groups - 1) / groups;
        // per round: the stages a warp computes one after the other + the unit's reduction, exchange and epilogue
        // (about three stage computations)
        const long long cost = rounds * ((nchunks + ks - 1) / ks + 3);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
}

}  // namespace

}  // namespace kb

using namespace kb;

extern "C" {

int kb_decoder_create(const kb_linear *const *qkv, const kb_linear *const *o, const kb_linear *const *gate_up,
                      const kb_linear *const *down, const float *const *norm1, const float *const *norm2,
                      float *const *k_cache, float *const *v_cache, size_t n_layers, size_t batch, size_t n_heads,
                      size_t max_len, size_t vocab, float eps, const float *embed, const float *lm_head,
                      const float *norm_f, const float *cos_table, const float *sin_table, kb_decoder **out) {
    if (out) *out = nullptr;
    if (!qkv || !o || !gate_up || !down || !norm1 || !norm2 || !k_cache || !v_cache || !embed || !lm_head || !norm_f ||
        !cos_table || !sin_table || !out)
        return fail(KB_ERR_INVALID, "null pointer");
    if (n_layers == 0 || batch == 0 || n_heads == 0) return fail(KB_ERR_INVALID, "zero dimension");
    if (batch > 2) return fail(KB_ERR_UNSUPPORTED, "the persistent decode step takes one or two sequences, got %zu", batch);
    std::vector<DecLayer> host(n_layers);
    const Linear *q0 = reinterpret_cast<const Linear *>(qkv[0]);
    if (!q0 || q0->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    const size_t d = q0->k, device = (size_t)q0->device;
    size_t f = 0;
    for (size_t i = 0; i < n_layers; ++i) {
        const Linear *Ls[4] = {reinterpret_cast<const Linear *>(qkv[i]), reinterpret_cast<const Linear *>(o[i]),
                               reinterpret_cast<const Linear *>(gate_up[i]), reinterpret_cast<const Linear *>(down[i])};
        for (int j = 0; j < 4; ++j)
            if (!Ls[j] || Ls[j]->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle (layer %zu)", i);
        if (i == 0) f = Ls[2]->m / 2;
        const bool shapes = Ls[0]->m == 3 * d && Ls[0]->k == d && Ls[1]->m == d && Ls[1]->k == d && Ls[2]->m == 2 * f &&
                            Ls[2]->k == d && Ls[3]->m == d && Ls[3]->k == f;
        if (!shapes) return fail(KB_ERR_SHAPE, "shape mismatch: layer %zu is not [3d,d], [d,d], [2f,d], [d,f] with d=%zu f=%zu", i, d, f);
        for (int j = 0; j < 4; ++j) {
            if (Ls[j]->kind != KB_TERNARY || Ls[j]->bias || (size_t)Ls[j]->device != device)
                return fail(KB_ERR_UNSUPPORTED, "the persistent decode step takes ternary layers without bias on one device");
        }
        host[i].qkv = LayerRef{Ls[0]->w2, Ls[0]->scales, nullptr};
        host[i].o = LayerRef{Ls[1]->w2, Ls[1]->scales, nullptr};
        host[i].gu = LayerRef{Ls[2]->w2, Ls[2]->scales, nullptr};
        host[i].down = LayerRef{Ls[3]->w2, Ls[3]->scales, nullptr};
        host[i].g1 = norm1[i]; host[i].g2 = norm2[i];
        host[i].kc = k_cache[i]; host[i].vc = v_cache[i];
        if (!norm1[i] || !norm2[i] || !k_cache[i] || !v_cache[i]) return fail(KB_ERR_INVALID, "null pointer (layer %zu)", i);
    }
    if (d % n_heads || d % 4 || f % 4 || (d / n_heads) % 4 || d / n_heads > (size_t)ATT_MAX_HD)
        return fail(KB_ERR_UNSUPPORTED, "the persistent decode step needs d %% 4 == 0, f %% 4 == 0, head_dim %% 4 == 0, head_dim <= %d", ATT_MAX_HD);
    cudaError_t e;
    int prev = -1;
    if ((e = cudaGetDevice(&prev)) != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != (int)device && (e = cudaSetDevice((int)device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    Decoder *D = new Decoder{};
    D->device = (int)device; D->batch = (int)batch; D->sms = sm_count((int)device);
    DecodeParams &p = D->p;
    p.n_layers = (int)n_layers; p.batch = (int)batch; p.d = (int)d; p.f = (int)f; p.n_heads = (int)n_heads;
    p.hd = (int)(d / n_heads); p.vocab = (int)vocab; p.max_len = (int)max_len; p.eps = eps;
    p.embed = embed; p.lm_head = lm_head; p.norm_f = norm_f; p.cos_t = cos_table; p.sin_t = sin_table;
    const size_t kp_d = round_up(d, 128), kp_f = round_up(f, 128);
    p.xs_stride = (int)(round_up(kp_f > kp_d ? kp_f : kp_d, 1024) + 64);
    const int nch_d = (int)((kp_d / 4 + CH - 1) / CH), nch_f = (int)((kp_f / 4 + CH - 1) / CH);
    p.ks_qkv = pick_ks((int)((3 * d + 15) / 16), nch_d, D->sms);
    p.ks_o = pick_ks((int)((d + 15) / 16), nch_d, D->sms);
    p.ks_gu = pick_ks((int)((2 * f + 15) / 16), nch_d, D->sms);
    p.ks_down = pick_ks((int)((d + 15) / 16), nch_f, D->sms);
    int splits = D->sms / (int)(batch * n_heads);
    if (splits < 1) splits = 1;
    if (splits > ATT_MAX_SPLITS) splits = ATT_MAX_SPLITS;
    p.att_splits = splits;
    // device memory: layer table + one block for the buffers
    const size_t off_qkv = 0, off_attn = off_qkv + round_up(batch * 3 * d * 4, 256), off_h = off_attn + round_up(batch * d * 4, 256);
    const size_t off_am = off_h + round_up(batch * f * 4, 256), off_sc = off_am + 256;
    const size_t off_cnt = off_sc + round_up(batch * n_heads * splits * (2 + ATT_MAX_HD) * 4, 256);
    const size_t off_bar = off_cnt + round_up(batch * n_heads * 4, 256), off_best = off_bar + 256, off_status = off_best + 256;
    const size_t total = off_status + 256;
    uint8_t *misc = nullptr;
    if ((e = cudaMalloc(&D->layers_dev, n_layers * sizeof(DecLayer))) != cudaSuccess ||
        (e = cudaMemcpy(D->layers_dev, host.data(), n_layers * sizeof(DecLayer), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMalloc(&misc, total)) != cudaSuccess || (e = cudaMemset(misc, 0, total)) != cudaSuccess) {
        if (D->layers_dev) cudaFree(D->layers_dev);
        if (misc) cudaFree(misc);
        delete D;
        if (prev != (int)device) cudaSetDevice(prev);
        return cuda_fail(e, "decoder buffers");
    }
    D->misc = misc;
    p.layers = D->layers_dev;
    p.qkv = reinterpret_cast<float *>(misc + off_qkv); p.attn = reinterpret_cast<float *>(misc + off_attn);
    p.h = reinterpret_cast<float *>(misc + off_h); p.absmax = reinterpret_cast<float *>(misc + off_am);
    p.att_scratch = reinterpret_cast<float *>(misc + off_sc); p.att_counters = reinterpret_cast<int *>(misc + off_cnt);
    p.barrier = reinterpret_cast<unsigned *>(misc + off_bar); p.best = reinterpret_cast<unsigned long long *>(misc + off_best);
    p.status = reinterpret_cast<int *>(misc + off_status);
    // shared memory: barriers, stage rings, activation rows, K-split scratch; the attention and lm_head phases reuse the rows
    const size_t part_bytes = (size_t)DW * 2 * batch * 32 * 4;
    size_t rows = batch * (size_t)p.xs_stride + part_bytes;
    const size_t att_need = (2 * ATT_MAX_HD + 2 * DW + DW * ATT_MAX_HD) * 4;
    const size_t head_need = batch * d * 4;
    if (att_need > rows) rows = att_need;
    if (head_need > rows) rows = head_need;
    D->smem = BAR_BYTES + (size_t)DW * NST * STAGE_BYTES + rows;
    if (D->smem > 224 * 1024) {
        cudaFree(D->layers_dev); cudaFree(misc); delete D;
        if (prev != (int)device) cudaSetDevice(prev);
        return fail(KB_ERR_UNSUPPORTED, "the persistent decode step needs %zu bytes of shared memory (d=%zu, f=%zu)", D->smem, d, f);
    }
    if (prev != (int)device) cudaSetDevice(prev);
    D->magic = DECODER_MAGIC;
    *out = reinterpret_cast<kb_decoder *>(D);
    return KB_OK;
}

void kb_decoder_destroy(kb_decoder *h) {
    Decoder *D = reinterpret_cast<Decoder *>(h);
    if (!D || D->magic != DECODER_MAGIC) return;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != D->device) cudaSetDevice(D->device);
    D->magic = 0;
    cudaFree(D->layers_dev);
    cudaFree(D->misc);
    if (prev != D->device) cudaSetDevice(prev);
    delete D;
}

int kb_decoder_step(kb_decoder *h, long long *tokens, int *positions, int *lens, long long *cache_rows, float *hidden,
                    float *logits, kb_stream stream) {
    Decoder *D = reinterpret_cast<Decoder *>(h);
    if (!D || D->magic != DECODER_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_decoder handle");
    if (!tokens || !positions || !lens || !cache_rows || !hidden) return fail(KB_ERR_INVALID, "null pointer");
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != D->device && (e = cudaSetDevice(D->device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    DecodeParams p = D->p;
    p.tokens = tokens; p.positions = positions; p.lens = lens; p.cache_rows = cache_rows; p.hidden = hidden; p.logits = logits;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = KB_OK;
    void (*kern)(const DecodeParams) = D->batch == 1 ? decode_step_kernel<1> : decode_step_kernel<2>;
    rc = set_dyn_smem_once(reinterpret_cast<const void *>(kern), D->device, (int)D->smem, "decode step smem attribute");
    if (rc == KB_OK && (e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), st)) != cudaSuccess) rc = cuda_fail(e, "barrier reset");
    if (rc == KB_OK) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)D->sms, 1, 1);
        cfg.blockDim = dim3(DTHREADS, 1, 1);
        cfg.dynamicSmemBytes = D->smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: the grid barrier needs it
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e != cudaSuccess) rc = cuda_fail(e, "decode step launch");
    }
    if (prev != D->device) cudaSetDevice(prev);
    return rc;
}

int kb_decoder_status(kb_decoder *h, kb_stream stream, int *status) {
    Decoder *D = reinterpret_cast<Decoder *>(h);
    if (!D || D->magic != DECODER_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_decoder handle");
    if (!status) return fail(KB_ERR_INVALID, "null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KB_CUDA(cudaMemcpyAsync(status, D->p.status, sizeof(int), cudaMemcpyDeviceToHost, st));
    KB_CUDA(cudaStreamSynchronize(st));
    if (*status != 0) {
        KB_CUDA(cudaMemsetAsync(D->p.status, 0, sizeof(int), st));
        KB_CUDA(cudaStreamSynchronize(st));
        return fail(KB_ERR_TIMEOUT, "persistent decode step gave up on a bounded wait (device code %d)", *status);
    }
    return KB_OK;
}

}  // extern "C"
