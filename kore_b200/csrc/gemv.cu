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
// Activations sit in shared memory, permuted so that for a fixed 16-byte sub-chunk
// the 32 lanes of a warp read 32 consecutive 16-byte slots (conflict-free).  When
// the caller passes f32 activations the per-token absmax quantiser runs in the
// prologue of every CTA (the row is a few KB and L2-resident), which removes one
// launch and one global round trip per linear layer in decode.
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
};

// shared-memory slot of the 16-element group g (k = 16*g .. 16*g+15) of one token row:
// inside each 2048-element block, lane l = (g%128)/4 and sub-chunk i = g%4 land at i*32 + l
__device__ __forceinline__ int xs_slot(int g) {
    const int blk = g >> 7, within = g & 127;
    return (blk << 7) + ((within & 3) << 5) + (within >> 2);
}
__device__ __forceinline__ int xs_group_of_slot(int d) {
    const int blk = d >> 7, within = d & 127;
    return (blk << 7) + ((within & 31) << 2) + (within >> 5);
}

template <int NT, int R, bool FUSED>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);  // [NT][kp/16] permuted slots
    __shared__ float s_sx[NT];
    __shared__ int s_sum[NT];
    __shared__ float red_f[32];
    __shared__ int red_i[32];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int tok0 = blockIdx.y * NT;
    const int groups16 = p.kp >> 4;
    const int slots = (groups16 + 127) & ~127;  // row stride in 16-byte slots (whole 2048-element blocks)
    const int row_groups = (p.m + R - 1) / R;
    const int first_group = blockIdx.x * nwarps + warp;

    // Weight loads do not depend on the activations: issue the first chunk before the
    // prologue (and before waiting on the previous kernel of the stream).
    uint4 wpre[R];
    {
        const int g0 = first_group < row_groups ? first_group : 0;
        const int kc = lane * 64;
#pragma unroll
        for (int r = 0; r < R; ++r)
            wpre[r] = kc < p.kp ? ld_stream_v4(p.w2 + (size_t)(g0 * R + r) * p.row_bytes + (kc >> 2))
                                : make_uint4(0, 0, 0, 0);
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- prologue: activations -> shared memory (int8, permuted) ----
    if (FUSED) {
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
            float amax = 0.0f;
            if (p.x_vec4) {
                const float4 *row4 = reinterpret_cast<const float4 *>(row);
                for (int i = threadIdx.x; i < (p.k >> 2); i += blockDim.x) {
                    float4 v = row4[i];
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            } else {
                for (int i = threadIdx.x; i < p.k; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
            }
            amax = block_reduce_max(amax, red_f);
            const float s = amax < 1e-8f ? 1.0f : __fdiv_rn(amax, 127.0f);
            int local_sum = 0;
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
                        int q = quantise_one(v[e], s);
                        local_sum += q;
                        word |= (uint32_t)(q & 0xff) << (8 * e);
                    }
                    out[w] = word;
                }
                dst[d] = make_uint4(out[0], out[1], out[2], out[3]);
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

    // ---- main loop: one warp owns R weight rows at a time ----
    const int stride_groups = gridDim.x * nwarps;
    for (int g = first_group; g < row_groups; g += stride_groups) {
        int acc[R][NT][4];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[r][t][j] = 0;

        const uint8_t *wbase = p.w2 + (size_t)(g * R) * p.row_bytes;
        const bool first = (g == first_group);
        for (int kc = lane * 64; kc < p.kp; kc += 2048) {
            uint4 wv[R];
            if (first && kc == lane * 64) {
#pragma unroll
                for (int r = 0; r < R; ++r) wv[r] = wpre[r];
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) wv[r] = ld_stream_v4(wbase + (size_t)r * p.row_bytes + (kc >> 2));
            }
            const int slot0 = ((kc >> 11) << 7) + lane;  // block*128 + lane, sub-chunk i adds 32*i
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 xv[NT];
#pragma unroll
                for (int t = 0; t < NT; ++t) xv[t] = xs[(size_t)t * slots + slot0 + 32 * i];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t w = i == 0 ? wv[r].x : (i == 1 ? wv[r].y : (i == 2 ? wv[r].z : wv[r].w));
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
        }

        // combine the four scaled partials (exact), reduce over lanes, and let lane
        // r*NT+t finish output (row g*R+r, token tok0+t)
        int mine = 0;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                int s = acc[r][t][0] + (acc[r][t][1] >> 2) + (acc[r][t][2] >> 4) + (acc[r][t][3] >> 6);
                s = warp_reduce_sum(s);
                if (lane == r * NT + t) mine = s;
            }
        if (lane < R * NT) {
            const int r = lane / NT, t = lane - r * NT;
            const int row = g * R + r, tok = tok0 + t;
            if (row < p.m && tok < p.n) {
                const int a = p.mul * mine - p.off * s_sum[t];
                const size_t o = (size_t)tok * p.ldy + row;
                if (p.acc) p.acc[o] = a;
                if (p.y) p.y[o] = dequant_out(a, p.sw[row], s_sx[t], p.bias ? p.bias[row] : 0.0f, p.bias != nullptr);
            }
        }
    }
}

bool gemv_supports(const Linear *lin, size_t n) {
    // the activations of up to 8 tokens must fit in shared memory
    const size_t nt = n >= 8 ? 8 : (n > 2 ? (n > 4 ? 8 : 4) : n);
    return nt * ((lin->kp + 2047) / 2048 * 2048) <= 200 * 1024;
}

template <int NT, int R, bool FUSED>
static int launch_one(const GemvParams &p, int tok_groups, cudaStream_t stream) {
    const int row_groups = (p.m + R - 1) / R;
    // few rows: smaller CTAs so that every SM gets work
    const int threads = row_groups <= 148 * 16 ? 128 : 256;
    const int nwarps = threads / 32;
    int ctas = (row_groups + nwarps - 1) / nwarps;
    const int cap = 148 * 8;
    if (ctas > cap) ctas = cap;
    const size_t smem = (size_t)NT * (((size_t)p.kp + 2047) / 2048 * 2048);
    auto kern = gemv_kernel<NT, R, FUSED>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv smem attribute");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, (unsigned)tok_groups, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "gemv launch");
}

template <bool FUSED>
static int dispatch(const GemvParams &p, cudaStream_t stream) {
    const int n = p.n;
    if (n == 1) return launch_one<1, 4, FUSED>(p, 1, stream);
    if (n == 2) return launch_one<2, 4, FUSED>(p, 1, stream);
    if (n <= 4) return launch_one<4, 2, FUSED>(p, 1, stream);
    return launch_one<8, 1, FUSED>(p, (n + 7) / 8, stream);
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
    p.x_vec4 = a.x && (L->k % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    if (a.x) return dispatch<true>(p, stream);
    if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
        return fail(KB_ERR_INVALID, "gemv: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    return dispatch<false>(p, stream);
}

}  // namespace kb
