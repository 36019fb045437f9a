// Decode GEMV for 2-bit weights (sm_100a): y[n, m] for a handful of tokens.
//
// HBM-bound: every weight byte is read exactly once with 128-bit streaming loads
// (one warp instruction = 512 contiguous bytes of one weight row), unpacked in
// registers and accumulated in int32 with dp4a; lanes are combined with warp
// shuffles.  Algorithmic bytes per launch: M*Kp/4 (weights) + 4*M (scales)
// + 4*K*N (activations) + 4*M*N (outputs).
//
// Unpack trick: a 32-bit word holds 16 codes, element 4j+b in byte b at bits 2j.
// dp4a(word & (0x03030303 << 2j), x_j) equals 4^j times the partial sum of the four
// products of group j, so four AND-masks replace all shifts; the four partial
// accumulators are exact multiples of 1, 4, 16, 64 and are divided out once per row.
// Codes are unsigned (0..3); the signed value is recovered in the epilogue as
// mul * S - off * sum(xq).
//
// Latency structure (what matters for a 4 MiB layer that streams in under a
// microsecond): each warp keeps PF weight chunks x R rows in flight in registers and
// issues the first PF of them before anything else — before the activation prologue
// and before griddepcontrol.wait — so with programmatic dependent launch a layer's
// weights arrive while the previous kernel of the stream is still finishing.
//
// Activations sit in shared memory, permuted so that for a fixed 16-byte sub-chunk
// the 32 lanes of a warp read 32 consecutive 16-byte slots (conflict-free).  When the
// caller passes f32 activations the per-token absmax quantiser runs in the prologue of
// every CTA from registers (one global read of the row, L2-resident), which removes a
// launch and a global round trip per linear layer in decode.
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

struct GemvParams {
    const uint8_t *w2;
    size_t row_bytes;
    int m, k, kp;
    const float *sw;
    const float *bias;
    const float *x;  // f32 [n,k] (fused quantiser) or nullptr
    const int8_t *xq;
    size_t ldq;
    const float *sx;
    const int32_t *sumq;
    int n;
    float *y;
    int32_t *acc;
    size_t ldy;
    int mul, off;
    int x_vec4;
    float *y_more[MAX_PEERS - 1];  // further copies of y (peer GPUs), same offsets
    int n_more;
    PeerSync sync;  // sync.world == 0: no fused barrier
    const float *resid;
    // decoder fusions (fused-quantiser launches only):
    const float *gamma;     // RMSNorm weight: the prologue normalises the row before quantising it
    float eps;
    const float *x_absmax;  // per-token max|x| already known: the prologue skips its reduction
    float *absmax_out;      // SwiGLU epilogue: per-token max|h| (atomic max on the float bits)
    float *clear_word;      // n floats the launch sets to zero (the other parity's absmax slots)
    int relu;               // max(y, 0) after the bias
};

// 16-element group g (k = 16*g .. 16*g+15) <-> shared-memory slot: inside each
// 2048-element block, lane l = (g%128)/4 and sub-chunk i = g%4 live at slot i*32 + l
__device__ __forceinline__ int xs_group_of_slot(int d) {
    const int blk = d >> 7, within = d & 127;
    return (blk << 7) + ((within & 31) << 2) + (within >> 5);
}


constexpr int XR = 8;  // float4 registers per thread for the single-pass fused quantiser

__device__ __forceinline__ float block_reduce_sum_float(float v, float *scratch) {
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

// EPI 0: y = dequantised output (+ residual).  EPI 1 (SwiGLU): weight rows alternate gate_i,
// up_i; the output is h_i = silu(gate_i) * up_i, M / 2 values per token.
template <int NT, int R, int PF, bool FUSED, int EPI = 0>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);  // [NT][slots] permuted 16-byte slots
    __shared__ float s_sx[NT];
    __shared__ int s_sum[NT];
    __shared__ float red_f[32];
    __shared__ int red_i[32];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int tok0 = blockIdx.y * NT;
    const int groups16 = p.kp >> 4;
    const int slots = (groups16 + 127) & ~127;  // row stride in slots (whole 2048-element blocks)
    const int nch = (p.kp + 2047) >> 11;        // 2048-element chunks per row (uniform over lanes)
    const int row_groups = (p.m + R - 1) / R;
    const int first_group = blockIdx.x * nwarps + warp;
    const int stride_groups = gridDim.x * nwarps;
    const int kc0 = lane * 64;
    // ---- weight pipeline: PF chunks x R rows in registers ----
    uint4 buf[PF][R];
    int lg = first_group, lci = 0;  // load cursor (row group, chunk)
    auto issue = [&](uint4(&dst)[R]) {
        const int kc = kc0 + (lci << 11);
        const bool ok = lg < row_groups && kc < p.kp;
        const uint8_t *src = p.w2 + (size_t)(lg * R) * p.row_bytes + (kc >> 2);
#pragma unroll
        for (int r = 0; r < R; ++r)
            dst[r] = ok ? ld_stream_v4(src + (size_t)r * p.row_bytes) : make_uint4(0, 0, 0, 0);
        if (++lci == nch) { lci = 0; lg += stride_groups; }
    };
#pragma unroll
    for (int s = 0; s < PF; ++s) issue(buf[s]);
    // per-row constants of the group a lane will finish (lane r*NT+t <-> row r): loaded at the
    // start of a group so their latency is hidden behind the group's weight stream
    float my_sw = 0.0f, my_bias = 0.0f;
    auto load_row_consts = [&](int g) {
        if (lane < R * NT && g < row_groups) {
            const int row = g * R + lane / NT;  // rows up to m_alloc-1 are allocated
            my_sw = p.sw[row];
            my_bias = p.bias ? p.bias[row] : 0.0f;
        }
    };
    load_row_consts(first_group);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (FUSED && p.clear_word && blockIdx.x == 0 && blockIdx.y == 0 && (int)threadIdx.x < p.n) p.clear_word[threadIdx.x] = 0.0f;

    // ---- prologue: activations -> shared memory (int8, permuted) ----
    if (FUSED) {
        const bool single_pass = p.x_vec4 && slots * 4 <= XR * (int)blockDim.x;
#pragma unroll 1
        for (int t = 0; t < NT; ++t) {
            const int tok = tok0 + t;
            uint4 *dst = xs + (size_t)t * slots;
            if (tok >= p.n) {
                for (int d = threadIdx.x; d < slots; d += blockDim.x) dst[d] = make_uint4(0, 0, 0, 0);
                if (threadIdx.x == 0) { s_sx[t] = 1.0f; s_sum[t] = 0; }
                continue;
            }
            const float *row = p.x + (size_t)tok * p.k;
            int local_sum = 0;
            float s, rs;
            if (single_pass) {
                // thread owns destination words widx = tid + i*blockDim (conflict-free stores);
                // word w of slot d holds elements 16*g + 4*w .. +3 of group g = group_of_slot(d)
                float4 v[XR];
                float amax = 0.0f;
                const int nv4 = p.k >> 2;
#pragma unroll
                for (int i = 0; i < XR; ++i) {
                    const int widx = threadIdx.x + i * blockDim.x;
                    const int src = xs_group_of_slot(widx >> 2) * 4 + (widx & 3);
                    v[i] = (widx < slots * 4 && src < nv4) ? reinterpret_cast<const float4 *>(row)[src]
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (p.gamma) {
                    // RMSNorm of the row: (x * (1 / sqrt(mean(x^2) + eps))) * gamma
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < XR; ++i)
                        ss += __fmul_rn(v[i].x, v[i].x) + __fmul_rn(v[i].y, v[i].y) + __fmul_rn(v[i].z, v[i].z) + __fmul_rn(v[i].w, v[i].w);
                    ss = block_reduce_sum_float(ss, red_f);
                    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)p.k), p.eps)));
#pragma unroll
                    for (int i = 0; i < XR; ++i) {
                        const int widx = threadIdx.x + i * blockDim.x;
                        const int src = xs_group_of_slot(widx >> 2) * 4 + (widx & 3);
                        if (widx < slots * 4 && src < nv4) {
                            const float4 gm = reinterpret_cast<const float4 *>(p.gamma)[src];
                            v[i].x = __fmul_rn(__fmul_rn(v[i].x, inv), gm.x);
                            v[i].y = __fmul_rn(__fmul_rn(v[i].y, inv), gm.y);
                            v[i].z = __fmul_rn(__fmul_rn(v[i].z, inv), gm.z);
                            v[i].w = __fmul_rn(__fmul_rn(v[i].w, inv), gm.w);
                        }
                    }
                }
                if (p.x_absmax) {
                    amax = p.x_absmax[tok];
                } else {
#pragma unroll
                    for (int i = 0; i < XR; ++i)
                        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
                    amax = block_reduce_max(amax, red_f);
                }
                s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
                rs = __frcp_rn(s);
                uint32_t *dstw = reinterpret_cast<uint32_t *>(dst);
#pragma unroll
                for (int i = 0; i < XR; ++i) {
                    const int widx = threadIdx.x + i * blockDim.x;
                    if (widx < slots * 4) {
                        const int q0 = quantise_one_fast(v[i].x, s, rs), q1 = quantise_one_fast(v[i].y, s, rs);
                        const int q2 = quantise_one_fast(v[i].z, s, rs), q3 = quantise_one_fast(v[i].w, s, rs);
                        local_sum += q0 + q1 + q2 + q3;
                        dstw[widx] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                                     ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                    }
                }
            } else {
                float amax = 0.0f;
                if (p.x_absmax) {
                    amax = p.x_absmax[tok];
                } else if (p.x_vec4) {
                    const float4 *row4 = reinterpret_cast<const float4 *>(row);
                    for (int i = threadIdx.x; i < (p.k >> 2); i += blockDim.x) {
                        float4 v = row4[i];
                        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
                } else {
                    for (int i = threadIdx.x; i < p.k; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
                }
                if (!p.x_absmax) amax = block_reduce_max(amax, red_f);
                s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
                rs = __frcp_rn(s);
                for (int d = threadIdx.x; d < slots; d += blockDim.x) {
                    const int g = xs_group_of_slot(d);
                    if (g >= groups16) continue;  // slot of a lane that lies beyond Kp in the last block
                    uint32_t out[4];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const int base = g * 16 + w * 4;
                        float v[4];
                        if (p.x_vec4 && base + 3 < p.k) {
                            float4 f = *reinterpret_cast<const float4 *>(row + base);
                            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[e] = (base + e < p.k) ? row[base + e] : 0.0f;
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
                    dst[d] = make_uint4(out[0], out[1], out[2], out[3]);
                }
            }
            local_sum = block_reduce_sum(local_sum, red_i);
            if (threadIdx.x == 0) { s_sx[t] = s; s_sum[t] = local_sum; }
        }
    } else {
        for (int idx = threadIdx.x; idx < NT * slots; idx += blockDim.x) {
            const int t = idx / slots, d = idx - t * slots;
            const int tok = tok0 + t;
            const int g = xs_group_of_slot(d);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < p.n && g < groups16)
                v = *reinterpret_cast<const uint4 *>(p.xq + (size_t)tok * p.ldq + (size_t)g * 16);
            xs[idx] = v;
        }
        if (threadIdx.x < NT) {
            const int tok = tok0 + threadIdx.x;
            s_sx[threadIdx.x] = tok < p.n ? p.sx[tok] : 1.0f;
            s_sum[threadIdx.x] = tok < p.n ? p.sumq[tok] : 0;
        }
    }
    __syncthreads();

    // ---- main loop: consume chunk, refill its registers, finish a row group when its
    //      last chunk has been consumed (control flow is uniform across the warp) ----
    int acc[R][NT][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][t][j] = 0;

    int cg = first_group, cci = 0;  // consume cursor
    while (cg < row_groups) {
#pragma unroll
        for (int s = 0; s < PF; ++s) {
            if (cg < row_groups) {
                // lanes beyond Kp hold zero weights, so their (unwritten) activation slots contribute 0
                const int slot0 = (cci << 7) + lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 xv[NT];
#pragma unroll
                    for (int t = 0; t < NT; ++t) xv[t] = xs[(size_t)t * slots + slot0 + 32 * i];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t w = i == 0 ? buf[s][r].x : (i == 1 ? buf[s][r].y : (i == 2 ? buf[s][r].z : buf[s][r].w));
                        const uint32_t w0 = w & 0x03030303u, w1 = w & 0x0c0c0c0cu;
                        const uint32_t w2_ = w & 0x30303030u, w3 = w & 0xc0c0c0c0u;
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            acc[r][t][0] = dp4a_u8s8(w0, xv[t].x, acc[r][t][0]);
                            acc[r][t][1] = dp4a_u8s8(w1, xv[t].y, acc[r][t][1]);
                            acc[r][t][2] = dp4a_u8s8(w2_, xv[t].z, acc[r][t][2]);
                            acc[r][t][3] = dp4a_u8s8(w3, xv[t].w, acc[r][t][3]);
                        }
                    }
                }
                issue(buf[s]);
                if (++cci == nch) {
                    // combine the four scaled partials (exact), reduce over lanes, and let lane
                    // r*NT+t finish output (row cg*R+r, token tok0+t)
                    int mine = 0;
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            int v = acc[r][t][0] + (acc[r][t][1] >> 2) + (acc[r][t][2] >> 4) + (acc[r][t][3] >> 6);
                            v = warp_reduce_sum(v);
                            if (lane == r * NT + t) mine = v;
                            acc[r][t][0] = acc[r][t][1] = acc[r][t][2] = acc[r][t][3] = 0;
                        }
                    if (EPI == 1) {
                        // lanes r*NT+t hold rows gate (r even) / up (r odd) of token t: the gate lane
                        // fetches its partner's value and writes h = silu(g) * u
                        const int r = lane / NT, t = lane - r * NT;
                        const int row = cg * R + r, tok = tok0 + t;
                        float v = 0.0f;
                        if (lane < R * NT && row < p.m && tok < p.n)
                            v = dequant_out(p.mul * mine - p.off * s_sum[t], my_sw, s_sx[t], my_bias, p.bias != nullptr);
                        const float u = __shfl_down_sync(0xffffffffu, v, NT);
                        if (lane < R * NT && (r & 1) == 0 && row + 1 < p.m && tok < p.n) {
                            const float silu = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
                            const float h = __fmul_rn(silu, u);
                            p.y[(size_t)tok * p.ldy + (row >> 1)] = h;
                            if (p.absmax_out) atomicMax(reinterpret_cast<unsigned int *>(p.absmax_out) + tok, __float_as_uint(fabsf(h)));
                        }
                    } else if (lane < R * NT) {
                        const int r = lane / NT, t = lane - r * NT;
                        const int row = cg * R + r, tok = tok0 + t;
                        if (row < p.m && tok < p.n) {
                            const int a = p.mul * mine - p.off * s_sum[t];
                            const size_t o = (size_t)tok * p.ldy + row;
                            if (p.acc) p.acc[o] = a;
                            if (p.y) {
                                float v = dequant_out(a, my_sw, s_sx[t], my_bias, p.bias != nullptr);
                                if (p.resid) v = __fadd_rn(v, p.resid[o]);
                                if (p.relu) v = fmaxf(v, 0.0f);
                                p.y[o] = v;
                                for (int q = 0; q < p.n_more; ++q) p.y_more[q][o] = v;  // peer copies over NVLink
                            }
                        }
                    }
                    cci = 0;
                    cg += stride_groups;
                    load_row_consts(cg);
                }
            }
        }
    }

    // ---- sharded layers: publish this rank's slice and wait for the peers' ----
    // Every CTA orders its peer stores at system scope; the last CTA of the launch to get
    // here bumps the epoch, writes it into slot [rank] of every rank's flag array and waits,
    // bounded (about a second), until all slots of the local array have reached it.
    if (p.sync.world > 0) {
        __shared__ int s_last, s_epoch;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();  // this CTA's peer stores are performed before it is counted
            const int total = gridDim.x * gridDim.y;
            const int ticket = atomicAdd(p.sync.done_counter, 1);
            s_last = (ticket == total - 1);
            if (s_last) {
                __threadfence_system();  // cumulative: orders every counted CTA's stores before the flags
                *p.sync.done_counter = 0;
                s_epoch = ++(*p.sync.epoch_counter);
            }
        }
        __syncthreads();
        if (s_last && (int)threadIdx.x < p.sync.world) {
            const int j = threadIdx.x, epoch = s_epoch;
            volatile int *remote = p.sync.flag_arrays[j] + p.sync.rank;
            *remote = epoch;
            const volatile int *mine = p.sync.flag_arrays[p.sync.rank] + j;
            const long long t0 = clock64();
            bool ok = false;
            for (;;) {
                if (*mine - epoch >= 0) { ok = true; break; }
                if (clock64() - t0 > 2000000000ll) break;
            }
            __threadfence_system();  // acquire side: later reads of the peers' slices see their data
            if (!ok) atomicCAS(p.sync.status, 0, 100 + j);
        }
    }
}


static size_t gemv_smem_bytes(size_t kp, size_t nt) { return nt * ((kp + 2047) / 2048 * 2048); }

bool gemv_supports(const Linear *lin, size_t n) {
    // the activations of up to 8 tokens must fit in shared memory
    const size_t nt = n >= 8 ? 8 : (n > 2 ? (n > 4 ? 8 : 4) : n);
    return gemv_smem_bytes(lin->kp, nt) <= 200 * 1024;
}

// tuning overrides, read once: KB_GEMV_THREADS (64..256, multiple of 32), KB_GEMV_PDL (0|1), KB_GEMV_PF (2|4),
// KB_GEMV_MAXCTAS (cap on the grid's x extent; rows are grid-strided)
static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

template <int NT, int R, int PF, bool FUSED, int EPI = 0>
static int launch_one(const GemvParams &p, int tok_groups, bool shared_grid, cudaStream_t stream) {
    static const int env_threads = env_int("KB_GEMV_THREADS", 0);
    static const int env_pdl = env_int("KB_GEMV_PDL", 1);
    static const int env_maxctas = env_int("KB_GEMV_MAXCTAS", 0);
    const int row_groups = (p.m + R - 1) / R;
    int threads = 256;
    if (env_threads >= 64 && env_threads <= 256 && env_threads % 32 == 0) threads = env_threads;
    if (p.gamma) threads = 256;  // the normalising prologue holds the row in the registers of 256 threads
    const int nwarps = threads / 32;
    const size_t smem = gemv_smem_bytes((size_t)p.kp, NT);
    auto kern = gemv_kernel<NT, R, PF, FUSED, EPI>;
    if (smem > 40 * 1024) {  // the static arrays count toward the 48 KB default limit too
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv smem attribute");
    }
    // persistent grid: at most one resident wave (SMs x CTAs per SM), rows are grid-strided,
    // so there is no partial last wave and activations are staged once per CTA
    // (occupancy and SM count are looked up once per kernel instance, CTA size and smem size)
    static thread_local int c_threads = 0, c_occ = 0, c_sms = 0;
    static thread_local size_t c_smem = ~(size_t)0;
    if (c_threads != threads || c_smem != smem) {
        int occ_q = 0, dev = 0, sms_q = 148;
        cudaGetDevice(&dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ_q, kern, threads, smem) != cudaSuccess || occ_q < 1) occ_q = 1;
        if (cudaDeviceGetAttribute(&sms_q, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms_q < 1) sms_q = 148;
        c_threads = threads; c_smem = smem; c_occ = occ_q; c_sms = sms_q;
    }
    const int occ = c_occ, sms = c_sms;
    // shared_grid: two row groups per warp, so a launch leaves room for other streams' launches
    // and each CTA stages the activations once for twice the weight bytes
    // (four when the launch ends in the cross-GPU barrier: every CTA then also pays a system-scope
    // fence for its peer stores, and fewer, longer CTAs measured faster)
    const int groups_per_cta = shared_grid ? (p.sync.world > 0 ? 4 : 2) * nwarps : nwarps;
    int ctas = (row_groups + groups_per_cta - 1) / groups_per_cta;
    if (ctas > sms * occ) ctas = sms * occ;
    if (env_maxctas > 0 && ctas > env_maxctas) ctas = env_maxctas;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, (unsigned)tok_groups, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // no early launch for kernels that end in a cross-GPU wait: a dependent grid parked at its
    // dependency wait would hold its CTAs resident for the whole exchange latency
    cfg.numAttrs = (env_pdl && p.sync.world == 0) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "gemv launch");
}

template <bool FUSED>
static int dispatch_swiglu(const GemvParams &p, bool sg, cudaStream_t stream) {
    return p.n == 1 ? launch_one<1, 4, 2, FUSED, 1>(p, 1, sg, stream) : launch_one<2, 4, 2, FUSED, 1>(p, 1, sg, stream);
}

template <bool FUSED>
static int dispatch(const GemvParams &p, bool sg, cudaStream_t stream) {
    const int n = p.n;
    static const int env_pf = env_int("KB_GEMV_PF", 0);
    if (n == 1) {
        // two chunks in flight per warp at two CTAs per SM measured faster than four chunks at
        // one CTA per SM (register pressure) on 8192-wide rows; the deep variant stays selectable
        const bool deep = env_pf == 4;
        return deep ? launch_one<1, 4, 4, FUSED>(p, 1, sg, stream) : launch_one<1, 4, 2, FUSED>(p, 1, sg, stream);
    }
    if (n == 2) return launch_one<2, 4, 2, FUSED>(p, 1, sg, stream);
    if (n <= 4) return launch_one<4, 2, 2, FUSED>(p, 1, sg, stream);
    return launch_one<8, 1, 2, FUSED>(p, (n + 7) / 8, sg, stream);
}

int launch_gemv(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!gemv_supports(L, a.n))
        return fail(KB_ERR_UNSUPPORTED, "gemv: K=%zu too large for the shared-memory activation stage", L->k);
    GemvParams p;
    p.w2 = L->w2; p.row_bytes = L->row_bytes;
    p.m = (int)L->m; p.k = (int)L->k; p.kp = (int)L->kp;
    p.sw = L->scales; p.bias = L->bias;
    p.x = a.x; p.xq = a.xq; p.ldq = a.ldq; p.sx = a.sx; p.sumq = a.sumq;
    p.n = (int)a.n; p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.mul = L->mul; p.off = L->off;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    p.sync = PeerSync{};
    if (a.sync && a.y) p.sync = *a.sync;
    p.n_more = a.y ? a.n_more : 0;
    for (int q = 0; q < MAX_PEERS - 1; ++q) p.y_more[q] = q < p.n_more ? a.y_more[q] : nullptr;
    p.x_vec4 = a.x && (L->k % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    p.gamma = a.x ? a.gamma : nullptr;
    p.eps = a.eps;
    p.x_absmax = a.x ? a.x_absmax : nullptr;
    p.absmax_out = a.swiglu ? a.absmax_out : nullptr;
    p.clear_word = a.x ? a.clear_word : nullptr;
    if ((a.gamma || a.x_absmax || a.clear_word) && !a.x)
        return fail(KB_ERR_INVALID, "gemv: the normalising / pre-scaled prologues take f32 activations");
    if (p.gamma) {
        // the normalised row is held in registers: 8 float4 per thread of a 256-thread CTA
        const int slots = (((int)L->kp >> 4) + 127) & ~127;
        if (!p.x_vec4 || (reinterpret_cast<uintptr_t>(a.gamma) & 15) || slots * 4 > XR * 256)
            return fail(KB_ERR_UNSUPPORTED, "gemv: RMSNorm prologue needs K %% 4 == 0, K <= 8192 and 16-byte aligned x and gamma");
    }
    if (a.swiglu) {
        if (a.n > 2 || !a.y || a.acc || a.resid || p.n_more || p.sync.world || (L->m & 1))
            return fail(KB_ERR_UNSUPPORTED, "gemv: the SwiGLU epilogue takes 1 or 2 tokens, an even number of rows and a plain output");
        p.ldy = a.ldy ? a.ldy : L->m / 2;
        return a.x ? dispatch_swiglu<true>(p, a.shared_grid, stream) : dispatch_swiglu<false>(p, a.shared_grid, stream);
    }
    if (a.x) return dispatch<true>(p, a.shared_grid, stream);
    if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
        return fail(KB_ERR_INVALID, "gemv: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    return dispatch<false>(p, a.shared_grid, stream);
}

}  // namespace kb
