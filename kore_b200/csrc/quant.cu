// Activation quantiser and load-time weight kernels (sm_100a).
//
//  * act_quant_kernel      per-token absmax -> int8, scale and code sum, one CTA per token
//  * repack_*              reference wire format (base-243 / 2-bit LSB-first) -> device layout
//  * quantise_*            f32 weights -> device layout + per-row scales, on the device
//  * export_wire / dequantize   device layout -> wire format / f32
//
// Everything here is HBM-bound byte work: one thread produces one aligned 32-bit word
// of the destination so stores coalesce; nothing is reshaped into a GEMM.
#include <cooperative_groups.h>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

// status of the launch just issued: the error is read once (reading it clears it)
static int launch_status(const char *what) {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, what);
}

// ------------------------------------------------------------------ activations

// One CTA per token row.  Pass 1 reduces max|x|, pass 2 (re-reading the row from L1/L2)
// emits 16 codes per thread-iteration as one 16-byte store.  Codes equal the CPU
// definition clamp(rne(x / s)) bit for bit: the quotient is formed as x * (1/s) and the
// exact IEEE division is evaluated only for the rare element that lands next to a
// rounding tie (see quantise_one_fast).
template <bool VEC4>
__global__ void __launch_bounds__(256) act_quant_kernel(const float *__restrict__ x, int k,
                                                        int8_t *__restrict__ xq, int ldq,
                                                        float *__restrict__ sx,
                                                        int32_t *__restrict__ sumq) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const size_t t = blockIdx.x;
    const float *row = x + t * (size_t)k;
    float amax = 0.0f;
    if (VEC4) {
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
        for (int i = threadIdx.x; i < k / 4; i += blockDim.x) {
            float4 v = row4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    }
    amax = block_reduce_max(amax, red_f);
    const float s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float rs = __frcp_rn(s);

    int local_sum = 0;
    int8_t *qrow = xq + t * (size_t)ldq;
    for (int g = threadIdx.x; g < ldq / 16; g += blockDim.x) {
        uint32_t out[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int base = g * 16 + w * 4;
            float v[4];
            if (VEC4 && base + 3 < k) {
                float4 f = *reinterpret_cast<const float4 *>(row + base);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = (base + e < k) ? row[base + e] : 0.0f;
            }
            uint32_t word = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int q = quantise_one_fast(v[e], s, rs);
                local_sum += q;
                word |= (uint32_t)(q & 0xff) << (8 * e);
            }
            out[w] = word;
        }
        *reinterpret_cast<uint4 *>(qrow + g * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
    local_sum = block_reduce_sum(local_sum, red_i);
    if (threadIdx.x == 0) {
        sx[t] = s;
        if (sumq) sumq[t] = local_sum;
    }
}

// Single-pass form for 16-byte aligned rows of up to G * 4096 elements: a thread keeps its G groups of 16
// elements in registers between the maximum and the quantisation, so the row is read from memory once
// (the two-pass form reads it twice; at 2048 x 11008 that second read is a third of the kernel).
template <int G>
__global__ void __launch_bounds__(256) act_quant_regs_kernel(const float *__restrict__ x, int k, int8_t *__restrict__ xq,
                                                             int ldq, float *__restrict__ sx, int32_t *__restrict__ sumq) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const size_t t = blockIdx.x;
    const float4 *row4 = reinterpret_cast<const float4 *>(x + t * (size_t)k);
    const int nv4 = k >> 2;
    float4 v[G][4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int g = threadIdx.x + i * 256;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int j = g * 4 + w;
            v[i][w] = j < nv4 ? row4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i][w].x), fabsf(v[i][w].y)), fmaxf(fabsf(v[i][w].z), fabsf(v[i][w].w))));
        }
    }
    amax = block_reduce_max(amax, red_f);
    const float s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float rs = __frcp_rn(s);
    int local_sum = 0;
    int8_t *qrow = xq + t * (size_t)ldq;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int g = threadIdx.x + i * 256;
        if (g < ldq / 16) {
            uint32_t out[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int q0 = quantise_one_fast(v[i][w].x, s, rs), q1 = quantise_one_fast(v[i][w].y, s, rs);
                const int q2 = quantise_one_fast(v[i][w].z, s, rs), q3 = quantise_one_fast(v[i][w].w, s, rs);
                local_sum += q0 + q1 + q2 + q3;
                out[w] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
            }
            *reinterpret_cast<uint4 *>(qrow + g * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
    local_sum = block_reduce_sum(local_sum, red_i);
    if (threadIdx.x == 0) {
        sx[t] = s;
        if (sumq) sumq[t] = local_sum;
    }
}

// The quantiser for a few tokens of a long row, plain f32 or flagged words ((f32 value, epoch) pairs written by the
// ranks of a column-sharded layer): a cluster of FQ_CLUSTER CTAs per token, each owning a contiguous part of the row,
// so that the row is pulled through eight SMs' load paths instead of one.  A thread holds G cells of 16 values in
// registers; flagged: it waits, bounded, until both pairs of every 16-byte load carry the expected epoch.  The
// cluster agrees on max|x| and on the code sum through distributed shared memory; the codes equal those of
// act_quant_kernel bit for bit.  Dependent launches may start at once (they wait for this grid before they read).
constexpr int FQ_CLUSTER = 8;
template <int G, bool FLAGGED>
__global__ void __cluster_dims__(FQ_CLUSTER, 1, 1) __launch_bounds__(256)
    act_quant_cluster_kernel(const void *__restrict__ xin, size_t ldx, int k, const int *round, int seq, int8_t *__restrict__ xq,
                             int ldq, float *__restrict__ sx, int32_t *__restrict__ sumq, int *status, long long max_cycles) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    __shared__ float part_max;
    __shared__ int part_sum;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");  // flagged: the round word is final, the producer's own stores are done
    const int t = blockIdx.x / FQ_CLUSTER, part = (int)cluster.block_rank();
    const int cells = ldq / 16, per_cta = (cells + FQ_CLUSTER - 1) / FQ_CLUSTER;
    float v[G][16];
    float amax = 0.0f;
    if (FLAGGED) {
        const uint32_t epoch = ((uint32_t)(*reinterpret_cast<const volatile int *>(round)) << 8) | (uint32_t)seq;
        const uint2 *row = static_cast<const uint2 *>(xin) + (size_t)t * ldx;
        long long t0 = 0;
        bool ok = true;
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const int local = threadIdx.x + i * 256;
            const int c = part * per_cta + local;
            const bool mine = local < per_cta && c < cells;
            uint4 raw[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const int e = c * 16 + 2 * w;
                raw[w] = make_uint4(0u, epoch, 0u, epoch);
                if (mine && e < k)
                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(raw[w].x), "=r"(raw[w].y), "=r"(raw[w].z), "=r"(raw[w].w)
                                 : "l"(row + e)
                                 : "memory");
            }
            for (;;) {
                bool all = true;
#pragma unroll
                for (int w = 0; w < 8; ++w)
                    if (raw[w].y != epoch || raw[w].w != epoch) {
                        all = false;
                        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(raw[w].x), "=r"(raw[w].y), "=r"(raw[w].z), "=r"(raw[w].w)
                                     : "l"(row + c * 16 + 2 * w)
                                     : "memory");
                    }
                if (all) break;
                const long long now = clock64();
                if (t0 == 0) t0 = now;
                else if (now - t0 > max_cycles) { ok = false; break; }
            }
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                v[i][2 * w] = __uint_as_float(raw[w].x);
                v[i][2 * w + 1] = __uint_as_float(raw[w].z);
            }
        }
        if (!ok) atomicCAS(status, 0, 110);
    } else {
        const float *row = static_cast<const float *>(xin) + (size_t)t * ldx;
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const int local = threadIdx.x + i * 256;
            const int c = part * per_cta + local;
            const bool mine = local < per_cta && c < cells;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int e = c * 16 + 4 * w;
                const float4 f = (mine && e < k) ? *reinterpret_cast<const float4 *>(row + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[i][4 * w] = f.x; v[i][4 * w + 1] = f.y; v[i][4 * w + 2] = f.z; v[i][4 * w + 3] = f.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[i][e]));
    amax = block_reduce_max(amax, red_f);
    if (threadIdx.x == 0) part_max = amax;
    cluster.sync();
    amax = 0.0f;
#pragma unroll
    for (int r = 0; r < FQ_CLUSTER; ++r) amax = fmaxf(amax, *cluster.map_shared_rank(&part_max, r));
    const float s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float rs = __frcp_rn(s);
    int local_sum = 0;
    int8_t *qrow = xq + (size_t)t * ldq;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int local = threadIdx.x + i * 256;
        const int c = part * per_cta + local;
        if (local < per_cta && c < cells) {
            uint32_t out[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int q0 = quantise_one_fast(v[i][4 * w], s, rs), q1 = quantise_one_fast(v[i][4 * w + 1], s, rs);
                const int q2 = quantise_one_fast(v[i][4 * w + 2], s, rs), q3 = quantise_one_fast(v[i][4 * w + 3], s, rs);
                local_sum += q0 + q1 + q2 + q3;
                out[w] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
            }
            *reinterpret_cast<uint4 *>(qrow + c * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
    local_sum = block_reduce_sum(local_sum, red_i);
    if (threadIdx.x == 0) part_sum = local_sum;
    cluster.sync();
    if (part == 0 && threadIdx.x == 0) {
        int total = 0;
#pragma unroll
        for (int r = 0; r < FQ_CLUSTER; ++r) total += *cluster.map_shared_rank(&part_sum, r);
        sx[t] = s;
        if (sumq) sumq[t] = total;
    }
    cluster.sync();  // no CTA leaves while its shared memory may still be read
}

template <bool FLAGGED>
static int launch_act_quant_cluster(const void *x, size_t ldx, size_t n, size_t k, const int *round, int seq, int8_t *xq, size_t ldq,
                                    float *sx, int32_t *sumq, int *status, cudaStream_t stream) {
    const size_t per_cta = (ldq / 16 + FQ_CLUSTER - 1) / FQ_CLUSTER;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n * FQ_CLUSTER), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = FLAGGED ? 1 : 0;  // the flagged form may start behind its producer; the plain form reads finished data
    const int ki = (int)k, ldqi = (int)ldq;
    const long long cycles = 2000000000ll;
    cudaError_t e;
    if (per_cta <= 256)
        e = cudaLaunchKernelEx(&cfg, act_quant_cluster_kernel<1, FLAGGED>, x, ldx, ki, round, seq, xq, ldqi, sx, sumq, status, cycles);
    else if (per_cta <= 512)
        e = cudaLaunchKernelEx(&cfg, act_quant_cluster_kernel<2, FLAGGED>, x, ldx, ki, round, seq, xq, ldqi, sx, sumq, status, cycles);
    else
        e = cudaLaunchKernelEx(&cfg, act_quant_cluster_kernel<4, FLAGGED>, x, ldx, ki, round, seq, xq, ldqi, sx, sumq, status, cycles);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "cluster quantiser launch");
}

int launch_act_quant_flagged(const unsigned long long *x, size_t ldx, size_t n, size_t k, const int *round, int seq, int8_t *xq,
                             size_t ldq, float *sx, int32_t *sumq, int *status, cudaStream_t stream) {
    if (n == 0) return KB_OK;
    if ((k % 4) || (ldx % 2) || ldx < k || (reinterpret_cast<uintptr_t>(x) & 15) || (ldq % 16) || ldq < k)
        return fail(KB_ERR_UNSUPPORTED, "flagged quantiser: K %% 4 == 0, 16-byte aligned rows and ld >= K are required");
    if ((ldq / 16 + FQ_CLUSTER - 1) / FQ_CLUSTER > 4 * 256) return fail(KB_ERR_UNSUPPORTED, "flagged quantiser: K=%zu too large", k);
    return launch_act_quant_cluster<true>(x, ldx, n, k, round, seq, xq, ldq, sx, sumq, status, stream);
}

int launch_act_quant(const float *x, size_t n, size_t k, int8_t *xq, size_t ldq, float *sx,
                     int32_t *sumq, cudaStream_t stream) {
    if (n == 0) return KB_OK;
    const bool vec4 = (k % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    // a few tokens of a long row: one CTA per token would pull the row through a single SM (a cluster launch costs
    // more than a plain one, so rows of 4096 values stay with one CTA: 16 streams of 4096 x 4096 layers, each with its
    // own quantiser launch, ran at 1.14 instead of 0.92 us per layer with the cluster form)
    if (vec4 && n <= 16 && k >= 8192 && (ldq % 16) == 0 && (ldq / 16 + FQ_CLUSTER - 1) / FQ_CLUSTER <= 4 * 256)
        return launch_act_quant_cluster<false>(x, k, n, k, nullptr, 0, xq, ldq, sx, sumq, nullptr, stream);
    if (vec4 && ldq <= 4 * 4096) {
        const unsigned grid = (unsigned)n;
        if (ldq <= 4096) act_quant_regs_kernel<1><<<grid, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
        else if (ldq <= 2 * 4096) act_quant_regs_kernel<2><<<grid, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
        else if (ldq <= 3 * 4096) act_quant_regs_kernel<3><<<grid, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
        else act_quant_regs_kernel<4><<<grid, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
        return launch_status("act_quant launch");
    }
    if (vec4)
        act_quant_kernel<true><<<(unsigned)n, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
    else
        act_quant_kernel<false><<<(unsigned)n, 256, 0, stream>>>(x, (int)k, xq, (int)ldq, sx, sumq);
    return launch_status("act_quant launch");
}

// ------------------------------------------------------------------ weights

// position of element i (0..15) of a 32-bit word: byte i%4, bit pair i/4
__device__ __forceinline__ uint32_t place_code(uint32_t code, int i) {
    return code << (8 * (i & 3) + 2 * (i >> 2));
}
__device__ __forceinline__ uint32_t take_code(uint32_t word, int i) {
    return (word >> (8 * (i & 3) + 2 * (i >> 2))) & 3u;
}

// base-243 digit i of a wire byte as a device code (digit 0/1/2 = trit -1/0/+1 = code);
// bytes >= 243 decode to five zero trits (code 1)
__device__ __forceinline__ uint32_t trit_code_of_byte(uint32_t byte, int i) {
    if (byte >= 243u) return 1u;
    const uint32_t p3[5] = {1u, 3u, 9u, 27u, 81u};
    return (byte / p3[i]) % 3u;
}

// one thread per destination word; rows >= m and k >= K are filled with the pad code
template <int KIND>
__global__ void repack_wire_kernel(const uint8_t *__restrict__ wire, int m, int k, int kpw,
                                   uint32_t *__restrict__ w2, int row_words, size_t total_words) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int row = (int)(idx / row_words);
    const int k0 = (int)(idx % row_words) * 16;
    const uint32_t pad = KIND == KB_TERNARY ? 1u : 0u;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int kk = k0 + i;
        uint32_t code = pad;
        if (row < m && kk < k) {
            if (KIND == KB_TERNARY)
                code = trit_code_of_byte(wire[(size_t)row * kpw + kk / 5], kk % 5);
            else
                code = (wire[(size_t)row * kpw + kk / 4] >> (2 * (kk % 4))) & 3u;
        }
        word |= place_code(code, i);
    }
    w2[idx] = word;
}

int launch_repack_wire(int kind, const uint8_t *wire, size_t m, size_t k, uint8_t *w2,
                       size_t row_bytes, size_t m_alloc, cudaStream_t stream) {
    const int row_words = (int)(row_bytes / 4);
    const size_t total = m_alloc * (size_t)row_words;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (kind == KB_TERNARY)
        repack_wire_kernel<KB_TERNARY><<<blocks, 256, 0, stream>>>(
            wire, (int)m, (int)k, (int)((k + 4) / 5), reinterpret_cast<uint32_t *>(w2), row_words, total);
    else
        repack_wire_kernel<KB_QUATERNARY><<<blocks, 256, 0, stream>>>(
            wire, (int)m, (int)k, (int)((k + 3) / 4), reinterpret_cast<uint32_t *>(w2), row_words, total);
    return launch_status("repack launch");
}

// base-243 rows -> int8 trits [n][ldq] (tail zero) and their per-row sums: a ternary operand in
// the role of the quantised activations (both-operands-ternary product).  One CTA per row.
__global__ void __launch_bounds__(256) decode_trits_i8_kernel(const uint8_t *__restrict__ wire, int k, int kpw,
                                                              int8_t *__restrict__ xq, int ldq,
                                                              int32_t *__restrict__ sumq) {
    __shared__ int red[32];
    const uint8_t *row = wire + blockIdx.x * (size_t)kpw;
    int8_t *dst = xq + blockIdx.x * (size_t)ldq;
    int local = 0;
    for (int kk = threadIdx.x; kk < ldq; kk += blockDim.x) {
        const int t = kk < k ? (int)trit_code_of_byte(row[kk / 5], kk % 5) - 1 : 0;
        dst[kk] = (int8_t)t;
        local += t;
    }
    local = block_reduce_sum(local, red);
    if (threadIdx.x == 0) sumq[blockIdx.x] = local;
}

int launch_decode_trits_i8(const uint8_t *wire, size_t n, size_t k, int8_t *xq, size_t ldq, int32_t *sumq,
                           cudaStream_t stream) {
    if (n == 0) return KB_OK;
    decode_trits_i8_kernel<<<(unsigned)n, 256, 0, stream>>>(wire, (int)k, (int)((k + 4) / 5), xq, (int)ldq, sumq);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "trit decode launch");
}

// per-row max|w| -> scale (mode 0: absmax, mode 1: absmax/3), 1.0 below 1e-8
__global__ void __launch_bounds__(256) row_scale_kernel(const float *__restrict__ w, int k, int mode,
                                                        float *__restrict__ scales) {
    __shared__ float red[32];
    const float *row = w + blockIdx.x * (size_t)k;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_reduce_max(amax, red);
    if (threadIdx.x == 0)
        scales[blockIdx.x] = amax < 1e-8f ? 1.0f : (mode == 0 ? amax : __fdiv_rn(amax, 3.0f));
}

// absmean: each row summed in ascending k in f64 by one thread, then the row sums are
// added in ascending m by a single thread — the exact order the CPU definition uses,
// so the f32 scale is reproducible bit for bit.  Load-time only.
__global__ void abs_rowsum_f64_kernel(const float *__restrict__ w, int m, int k,
                                      double *__restrict__ rowsum) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= m) return;
    const float *p = w + (size_t)row * k;
    double s = 0.0;
    for (int i = 0; i < k; ++i) s += (double)fabsf(p[i]);
    rowsum[row] = s;
}
__global__ void absmean_finish_kernel(const double *__restrict__ rowsum, int m, int k, int m_alloc,
                                      float *__restrict__ scales) {
    __shared__ float s_sh;
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int r = 0; r < m; ++r) total += rowsum[r];
        float s = (float)(total / ((double)m * (double)k));
        s_sh = s < 1e-8f ? 1.0f : s;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < m_alloc; r += blockDim.x) scales[r] = r < m ? s_sh : 1.0f;
}

// MODE 0: ternary, reference rule (sign beyond threshold); 1: ternary absmean (rne, clamp);
// 2: quaternary reference rule
template <int MODE>
__global__ void quantise_f32_kernel(const float *__restrict__ w, int m, int k, float thr,
                                    const float *__restrict__ scales, uint32_t *__restrict__ w2,
                                    int row_words, size_t total_words) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int row = (int)(idx / row_words);
    const int k0 = (int)(idx % row_words) * 16;
    const uint32_t pad = MODE == 2 ? 0u : 1u;
    const float scale = row < m ? scales[row] : 1.0f;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int kk = k0 + i;
        uint32_t code = pad;
        if (row < m && kk < k) {
            const float nrm = __fdiv_rn(w[(size_t)row * k + kk], scale);
            if (MODE == 0) {
                code = nrm > thr ? 2u : (nrm < -thr ? 0u : 1u);
            } else if (MODE == 1) {
                const float q = rintf(nrm);
                code = q > 1.0f ? 2u : (q < -1.0f ? 0u : (uint32_t)((int)q + 1));
            } else {
                code = nrm < -2.0f ? 0u : (nrm < 0.0f ? 1u : (nrm < 2.0f ? 2u : 3u));
            }
        }
        word |= place_code(code, i);
    }
    w2[idx] = word;
}

__global__ void fill_f32_kernel(float *p, size_t from, size_t to, float v) {
    const size_t i = from + blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < to) p[i] = v;
}

int launch_quantise_f32(int kind, int quantiser, const float *w, size_t m, size_t k, float threshold,
                        uint8_t *w2, size_t row_bytes, size_t m_alloc, float *scales,
                        cudaStream_t stream) {
    const int row_words = (int)(row_bytes / 4);
    const size_t total = m_alloc * (size_t)row_words;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    uint32_t *dst = reinterpret_cast<uint32_t *>(w2);
    if (kind == KB_TERNARY && quantiser == KB_QUANT_ABSMEAN) {
        double *rowsum = nullptr;
        KB_CUDA(cudaMallocAsync(&rowsum, m * sizeof(double), stream));
        abs_rowsum_f64_kernel<<<(unsigned)((m + 63) / 64), 64, 0, stream>>>(w, (int)m, (int)k, rowsum);
        absmean_finish_kernel<<<1, 256, 0, stream>>>(rowsum, (int)m, (int)k, (int)m_alloc, scales);
        quantise_f32_kernel<1><<<blocks, 256, 0, stream>>>(w, (int)m, (int)k, threshold, scales, dst,
                                                           row_words, total);
        KB_CUDA(cudaFreeAsync(rowsum, stream));
    } else {
        row_scale_kernel<<<(unsigned)m, 256, 0, stream>>>(w, (int)k, kind == KB_TERNARY ? 0 : 1, scales);
        if (m_alloc > m)
            fill_f32_kernel<<<(unsigned)((m_alloc - m + 255) / 256), 256, 0, stream>>>(scales, m, m_alloc, 1.0f);
        if (kind == KB_TERNARY)
            quantise_f32_kernel<0><<<blocks, 256, 0, stream>>>(w, (int)m, (int)k, threshold, scales, dst,
                                                               row_words, total);
        else
            quantise_f32_kernel<2><<<blocks, 256, 0, stream>>>(w, (int)m, (int)k, threshold, scales, dst,
                                                               row_words, total);
    }
    return launch_status("quantise launch");
}

// device layout -> wire format, one thread per wire byte.  Pad slots follow the
// reference packers: Zero trits for ternary, code 0 for quaternary.
template <int KIND>
__global__ void export_wire_kernel(const uint32_t *__restrict__ w2, int row_words, int m, int k,
                                   int kpw, uint8_t *__restrict__ wire) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)m * kpw) return;
    const int row = (int)(idx / kpw);
    const int kb_ = (int)(idx % kpw);
    const uint32_t *wrow = w2 + (size_t)row * row_words;
    uint32_t byte = 0;
    if (KIND == KB_TERNARY) {
        uint32_t mult = 1;
        for (int i = 0; i < 5; ++i) {
            const int kk = kb_ * 5 + i;
            const uint32_t code = kk < k ? take_code(wrow[kk / 16], kk % 16) : 1u;
            byte += code * mult;
            mult *= 3;
        }
    } else {
        for (int i = 0; i < 4; ++i) {
            const int kk = kb_ * 4 + i;
            const uint32_t code = kk < k ? take_code(wrow[kk / 16], kk % 16) : 0u;
            byte |= code << (2 * i);
        }
    }
    wire[idx] = (uint8_t)byte;
}

int launch_export_wire(int kind, const uint8_t *w2, size_t row_bytes, size_t m, size_t k,
                       uint8_t *wire, cudaStream_t stream) {
    const int kpw = (int)(kind == KB_TERNARY ? (k + 4) / 5 : (k + 3) / 4);
    const size_t total = m * (size_t)kpw;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    const uint32_t *src = reinterpret_cast<const uint32_t *>(w2);
    if (kind == KB_TERNARY)
        export_wire_kernel<KB_TERNARY><<<blocks, 256, 0, stream>>>(src, (int)(row_bytes / 4), (int)m, (int)k, kpw, wire);
    else
        export_wire_kernel<KB_QUATERNARY><<<blocks, 256, 0, stream>>>(src, (int)(row_bytes / 4), (int)m, (int)k, kpw, wire);
    return launch_status("export launch");
}

__global__ void dequantize_kernel(const uint32_t *__restrict__ w2, int row_words, int kind,
                                  const float *__restrict__ scales, int m, int k,
                                  float *__restrict__ w) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)m * k) return;
    const int row = (int)(idx / k), kk = (int)(idx % k);
    const int code = (int)take_code(w2[(size_t)row * row_words + kk / 16], kk % 16);
    const float v = kind == KB_TERNARY ? (float)(code - 1) : (float)(2 * code - 3);
    w[idx] = __fmul_rn(v, scales[row]);
}

int launch_dequantize(int kind, const uint8_t *w2, size_t row_bytes, const float *scales, size_t m,
                      size_t k, float *w, cudaStream_t stream) {
    const size_t total = m * k;
    dequantize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const uint32_t *>(w2), (int)(row_bytes / 4), kind, scales, (int)m, (int)k, w);
    return launch_status("dequantize launch");
}

// [rows, cols] -> [cols, rows] through a padded shared-memory tile (coalesced both ways)
__global__ void transpose_f32_kernel(const float *__restrict__ src, int rows, int cols,
                                     float *__restrict__ dst) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = src[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][j];
    }
}

int launch_transpose_f32(const float *src, size_t rows, size_t cols, float *dst, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return KB_OK;
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    transpose_f32_kernel<<<grid, dim3(32, 8), 0, stream>>>(src, (int)rows, (int)cols, dst);
    return launch_status("transpose launch");
}

}  // namespace kb
