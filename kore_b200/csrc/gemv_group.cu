// Grouped decode GEMV (sm_100a): one token through each of L independent layers of the same
// shape in ONE launch — y[l, :] = layer_l(x[l, :]).
//
// A 4 MiB layer streams in well under a microsecond, less than the launch, ramp-up and tail of
// any kernel, so launching such layers one by one (even on many streams) leaves a quarter of the
// HBM bandwidth unused.  Here the L layers form one virtual matrix of L * M rows: every CTA owns a
// contiguous range of row groups (R rows each), its warps take the groups of the range in turn,
// and the register pipeline of weight loads (PF chunks x R rows per warp, 512 contiguous bytes
// per warp instruction) runs across layer boundaries without draining.  The arithmetic per row is
// that of the single-layer GEMV: (word & (0x03030303 << 2j)) dp4a x, four partial accumulators
// that are exact multiples of 1, 4, 16, 64, mul * S - off * sum(xq), then (acc * w_scale) * s + bias.
//
// Activations: layer l reads token row l of the quantised matrix (int8 codes, scale, code sum),
// i.e. one quantiser launch over an [L, K] matrix feeds the whole group.  A CTA stages the rows
// of the layers its range touches (two for ranges shorter than a layer) in shared memory in the
// GEMV's permuted order; the host grows the grid until they fit.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

namespace {

constexpr uint32_t GROUP_MAGIC = 0x4b423247u;  // "KB2G"
constexpr int MAX_STAGED = 32;                 // layers whose activations one CTA may hold

struct Group {
    uint32_t magic;
    int device;
    int kind, mul, off;
    size_t count, m, k, kp, row_bytes;
    LayerRef *table;  // device, [count]
    // host entry point: device copies of x [count, k] and y [count, m]; one call at a time
    float *dx, *dy;
    std::mutex host_mutex;
};

struct GroupParams {
    const LayerRef *table;
    int count, m, kp;
    size_t row_bytes;
    const float *x;  // f32 [count, ldx]: the per-token quantiser runs in the prologue (then xq, sx, sumq are unused)
    size_t ldx;
    int k, x_vec4;
    const int8_t *xq;
    size_t ldq;
    const float *sx;
    const int32_t *sumq;
    float *y;
    size_t ldy;
    int mul, off;
    int groups_per_cta;  // row groups per CTA (a multiple of the warps per CTA)
    int staged;          // activation rows a CTA stages (layers its range can touch)
};

// same permutation as the single-layer GEMV: inside each 2048-element block, 16-element group g
// of lane (g % 128) / 4, sub-chunk g % 4 lives at slot (g % 4) * 32 + lane
__device__ __forceinline__ int group_of_slot(int d) {
    const int blk = d >> 7, within = d & 127;
    return (blk << 7) + ((within & 31) << 2) + (within >> 5);
}

// Sum over the warp of four per-lane values at once: after the call lanes 8r .. 8r+7 hold the
// total of value r.  Halving the number of live values at each of the first two steps takes
// 6 shuffles instead of the 20 of four separate butterflies — at K = 4096 a row is only two
// 512-byte warp loads, so what is spent per row decides whether the kernel is issue-bound.
__device__ __forceinline__ int warp_reduce4(int v0, int v1, int v2, int v3, int lane) {
    const bool hi = (lane & 16) != 0, h8 = (lane & 8) != 0;
    int a = hi ? v2 : v0, b = hi ? v3 : v1;
    a += __shfl_xor_sync(0xffffffffu, hi ? v0 : v2, 16);
    b += __shfl_xor_sync(0xffffffffu, hi ? v1 : v3, 16);
    int c = h8 ? b : a;
    c += __shfl_xor_sync(0xffffffffu, h8 ? a : b, 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

// block-wide reductions of two values at once (one barrier pair for both rows of a prologue pass)
__device__ __forceinline__ void block_max2(float &a, float &b, float *scratch /* [64] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
    __syncthreads();
    a = lane < nwarps ? scratch[lane] : 0.0f;
    b = lane < nwarps ? scratch[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
    }
}
__device__ __forceinline__ void block_sum2(int &a, int &b, int *scratch /* [64] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
    __syncthreads();
    a = lane < nwarps ? scratch[lane] : 0;
    b = lane < nwarps ? scratch[32 + lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
}

// a cursor over the virtual row groups a warp owns: v, v + nwarps, ... ; (layer, g) follow without divisions
struct Cursor {
    int v, layer, g;
    __device__ __forceinline__ void init(int v0, int row_groups) { v = v0; layer = v0 / row_groups; g = v0 - layer * row_groups; }
    __device__ __forceinline__ void advance(int step, int row_groups) {
        v += step; g += step;
        while (g >= row_groups) { g -= row_groups; ++layer; }
    }
};

// FULLK: Kp is a multiple of 2048, so every lane of every chunk lies inside the row.
// FUSED: the activations arrive as f32 and each CTA quantises the rows of the layers it touches
// itself (per-token absmax -> int8, the quantiser kernel's arithmetic), which costs a CTA that
// streams for a hundred microseconds a few microseconds once and removes the quantiser launch.
// TPB threads per CTA, MINB CTAs per SM (bounds the registers: more resident warps hide more of
// the load latency than a third chunk in flight per warp)
template <int PF, bool FULLK, bool FUSED, int TPB, int MINB>
__global__ void __launch_bounds__(TPB, MINB) gemv_group_kernel(const GroupParams p) {
    constexpr int R = 4;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);  // [staged][slots]
    __shared__ float s_sx[MAX_STAGED];
    __shared__ int s_sum[MAX_STAGED];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int groups16 = p.kp >> 4;
    const int slots = (groups16 + 127) & ~127;
    const int nch = (p.kp + 2047) >> 11;
    const int row_groups = (p.m + R - 1) / R;  // per layer
    const int total = p.count * row_groups;    // the host checks that this fits
    const int begin = min(blockIdx.x * p.groups_per_cta, total);
    const int end = min(begin + p.groups_per_cta, total);
    const int layer0 = begin / row_groups;
    const int kc0 = lane * 64;

    // ---- weight pipeline: PF chunks x R rows in registers, cursor over (virtual group, chunk) ----
    uint4 buf[PF][R];
#pragma unroll
    for (int s = 0; s < PF; ++s)
#pragma unroll
        for (int r = 0; r < R; ++r) buf[s][r] = make_uint4(0, 0, 0, 0);
    Cursor lc;
    lc.init(begin + warp, row_groups);
    int lci = 0, l_layer = -1;
    const uint8_t *l_w2 = nullptr;
    auto issue = [&](uint4(&dst)[R]) {
        const int kc = kc0 + (lci << 11);
        if (lc.v < end && (FULLK || kc < p.kp)) {  // registers of a skipped load keep zeros or stale codes nobody consumes
            if (lc.layer != l_layer) { l_layer = lc.layer; l_w2 = p.table[l_layer].w2; }
            const uint8_t *src = l_w2 + (size_t)(lc.g * R) * p.row_bytes + (kc >> 2);
#pragma unroll
            for (int r = 0; r < R; ++r) dst[r] = ld_stream_v4(src + (size_t)r * p.row_bytes);
        } else if (!FULLK) {
#pragma unroll
            for (int r = 0; r < R; ++r) dst[r] = make_uint4(0, 0, 0, 0);
        }
        if (++lci == nch) { lci = 0; lc.advance(nwarps, row_groups); }
    };
#pragma unroll
    for (int s = 0; s < PF; ++s) issue(buf[s]);

    // consume cursor; lane 8r finishes row r of a group and fetches that row's scale and bias one
    // group ahead, so the epilogue of a group never waits on them
    Cursor cc, nc;
    cc.init(begin + warp, row_groups);
    nc = cc;
    int cci = 0, ref_layer = -1;
    const float *ref_sw = nullptr, *ref_bias = nullptr;
    float my_sw = 0.0f, my_bias = 0.0f, nx_sw = 0.0f, nx_bias = 0.0f;
    bool my_hb = false, nx_hb = false;
    const bool finisher = (lane & 7) == 0;
    const int my_r = lane >> 3;
    auto fetch_consts = [&](const Cursor &c, float &sw, float &bias, bool &hb) {
        if (c.v < end && finisher) {
            if (c.layer != ref_layer) {
                const LayerRef ref = p.table[c.layer];
                ref_layer = c.layer; ref_sw = ref.sw; ref_bias = ref.bias;
            }
            const int row = c.g * R + my_r;  // rows up to m_alloc - 1 are allocated
            sw = ref_sw[row];
            hb = ref_bias != nullptr;
            bias = hb ? ref_bias[row] : 0.0f;
        }
    };
    fetch_consts(nc, my_sw, my_bias, my_hb);
    nc.advance(nwarps, row_groups);
    fetch_consts(nc, nx_sw, nx_bias, nx_hb);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations of the layers this range touches -> shared memory (int8, permuted) ----
    if (FUSED) {
        // two rows per pass: their loads are in flight together and share the block reductions
        __shared__ float red_f[64];
        __shared__ int red_i[64];
#pragma unroll 1
        for (int t0 = 0; t0 < p.staged; t0 += 2) {
            const float *row[2];
            bool live[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int layer = layer0 + t0 + u;
                live[u] = t0 + u < p.staged && layer < p.count;
                row[u] = p.x + (size_t)(live[u] ? layer : 0) * p.ldx;
            }
            float amax[2] = {0.0f, 0.0f};
            if (p.x_vec4) {
                // eight independent 16-byte loads per thread in flight: one L2 round trip for K = 4096
                const int nv4 = p.k >> 2;
                for (int i0 = threadIdx.x; i0 < nv4; i0 += 4 * blockDim.x) {
                    float4 v[2][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = i0 + j * blockDim.x;
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            v[u][j] = (live[u] && i < nv4) ? reinterpret_cast<const float4 *>(row[u])[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            amax[u] = fmaxf(amax[u], fmaxf(fmaxf(fabsf(v[u][j].x), fabsf(v[u][j].y)), fmaxf(fabsf(v[u][j].z), fabsf(v[u][j].w))));
                }
            } else {
                for (int i = threadIdx.x; i < p.k; i += blockDim.x) {
#pragma unroll
                    for (int u = 0; u < 2; ++u)
                        if (live[u]) amax[u] = fmaxf(amax[u], fabsf(row[u][i]));
                }
            }
            block_max2(amax[0], amax[1], red_f);
            float sc[2], rs[2];
            int local_sum[2] = {0, 0};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                sc[u] = amax[u] < 1e-8f ? 1.0f : __fdiv_rn(amax[u], 127.0f);
                rs[u] = __frcp_rn(sc[u]);
            }
            for (int d = threadIdx.x; d < slots; d += blockDim.x) {
                const int g = group_of_slot(d);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (t0 + u >= p.staged) continue;
                    uint32_t out[4] = {0u, 0u, 0u, 0u};
                    if (live[u] && g < groups16) {
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            const int base = g * 16 + w * 4;
                            float v[4];
                            if (p.x_vec4 && base + 3 < p.k) {
                                const float4 f = *reinterpret_cast<const float4 *>(row[u] + base);
                                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e) v[e] = (base + e < p.k) ? row[u][base + e] : 0.0f;
                            }
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int q = quantise_one_fast(v[e], sc[u], rs[u]);
                                local_sum[u] += q;
                                out[w] |= (uint32_t)(q & 0xff) << (8 * e);
                            }
                        }
                    }
                    xs[(size_t)(t0 + u) * slots + d] = make_uint4(out[0], out[1], out[2], out[3]);
                }
            }
            block_sum2(local_sum[0], local_sum[1], red_i);
            if (threadIdx.x == 0) {
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    if (t0 + u < p.staged) { s_sx[t0 + u] = live[u] ? sc[u] : 1.0f; s_sum[t0 + u] = live[u] ? local_sum[u] : 0; }
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < p.staged * slots; idx += blockDim.x) {
            const int t = idx / slots, d = idx - t * slots;
            const int layer = layer0 + t;
            const int g = group_of_slot(d);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (layer < p.count && g < groups16)
                v = *reinterpret_cast<const uint4 *>(p.xq + (size_t)layer * p.ldq + (size_t)g * 16);
            xs[idx] = v;
        }
        if ((int)threadIdx.x < p.staged) {
            const int layer = layer0 + threadIdx.x;
            s_sx[threadIdx.x] = layer < p.count ? p.sx[layer] : 1.0f;
            s_sum[threadIdx.x] = layer < p.count ? p.sumq[layer] : 0;
        }
    }
    __syncthreads();

    int acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0;

    while (cc.v < end) {
#pragma unroll
        for (int s = 0; s < PF; ++s) {
            if (cc.v < end) {
                const uint4 *xrow = xs + (size_t)(cc.layer - layer0) * slots + (cci << 7) + lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 xv = xrow[32 * i];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t w = i == 0 ? buf[s][r].x : (i == 1 ? buf[s][r].y : (i == 2 ? buf[s][r].z : buf[s][r].w));
                        acc[r][0] = dp4a_u8s8(w & 0x03030303u, xv.x, acc[r][0]);
                        acc[r][1] = dp4a_u8s8(w & 0x0c0c0c0cu, xv.y, acc[r][1]);
                        acc[r][2] = dp4a_u8s8(w & 0x30303030u, xv.z, acc[r][2]);
                        acc[r][3] = dp4a_u8s8(w & 0xc0c0c0c0u, xv.w, acc[r][3]);
                    }
                }
                issue(buf[s]);
                if (++cci == nch) {
                    int v[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {  // the four partials are exact multiples of 1, 4, 16, 64
                        v[r] = acc[r][0] + (acc[r][1] >> 2) + (acc[r][2] >> 4) + (acc[r][3] >> 6);
                        acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0;
                    }
                    const int mine = warp_reduce4(v[0], v[1], v[2], v[3], lane);
                    const int row = cc.g * R + my_r;
                    if (finisher && row < p.m) {
                        const int t = cc.layer - layer0;
                        const int a = p.mul * mine - p.off * s_sum[t];
                        p.y[(size_t)cc.layer * p.ldy + row] = dequant_out(a, my_sw, s_sx[t], my_bias, my_hb);
                    }
                    cci = 0;
                    cc.advance(nwarps, row_groups);
                    my_sw = nx_sw; my_bias = nx_bias; my_hb = nx_hb;
                    nc.advance(nwarps, row_groups);
                    fetch_consts(nc, nx_sw, nx_bias, nx_hb);
                }
            }
        }
    }
}

}  // namespace

namespace {

constexpr int GROUP_R = 4, GROUP_THREADS = 256;

struct ScopedDevice {
    int prev = -1;
    bool switched = false;
    explicit ScopedDevice(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~ScopedDevice() {
        if (switched) cudaSetDevice(prev);
    }
};

const Group *check_group(const kb_linear_group *g) {
    const Group *G = reinterpret_cast<const Group *>(g);
    if (!G || G->magic != GROUP_MAGIC) {
        fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear_group handle");
        return nullptr;
    }
    return G;
}

int env_int(const char *name, int dflt) {
    const char *e = getenv(name);
    return e ? atoi(e) : dflt;
}

int group_forward(const Group *G, const float *x, size_t ldx, const int8_t *xq, size_t ldq, const float *sx,
                  const int32_t *sumq, float *y, size_t ldy, cudaStream_t stream) {
    if (ldy == 0) ldy = G->m;
    if (ldy < G->m) return fail(KB_ERR_SHAPE, "shape mismatch: ldy %zu is smaller than out_features %zu", ldy, G->m);
    ScopedDevice dev(G->device);
    static const int impl = env_int("KB_GROUP_IMPL", 1);  // 1: streaming MMA kernel, 0: dp4a kernel
    if (impl == 1) {
        GroupArgs ga = {};
        ga.table = G->table; ga.device = G->device; ga.kind = G->kind; ga.mul = G->mul; ga.off = G->off;
        ga.count = G->count; ga.m = G->m; ga.k = G->k; ga.kp = G->kp; ga.row_bytes = G->row_bytes;
        ga.x = x; ga.ldx = ldx; ga.xq = xq; ga.ldq = ldq; ga.sx = sx; ga.sumq = sumq;
        ga.y = y; ga.ldy = ldy; ga.status = nullptr;
        return launch_group_stream(ga, stream);
    }
    // launch shapes: {chunks in flight per warp, threads per CTA, CTAs per SM}
    static const int cfg_id = env_int("KB_GROUP_CFG", 1);
    const int shape = (cfg_id >= 0 && cfg_id <= 4) ? cfg_id : 1;
    static const int cfg_threads[5] = {256, 128, 128, 256, 128}, cfg_minb[5] = {2, 5, 6, 3, 4};
    const int threads = cfg_threads[shape];
    const int nwarps = threads / 32;
    const long long row_groups = (long long)((G->m + GROUP_R - 1) / GROUP_R);
    const long long total = (long long)G->count * row_groups;
    const size_t row_smem = (G->kp + 2047) / 2048 * 2048;  // bytes of one staged activation row
    // persistent-size grid; grown (smaller ranges touch fewer layers) until a CTA's activation rows fit
    long long grid = (long long)sm_count(G->device) * cfg_minb[shape];
    if (grid < 1) grid = 1;
    long long per_cta = 0, staged = 0;
    for (;;) {
        per_cta = (total + grid - 1) / grid;
        per_cta = (per_cta + nwarps - 1) / nwarps * nwarps;
        staged = (per_cta + row_groups - 2) / row_groups + 1;
        if (staged > (long long)G->count) staged = (long long)G->count;
        if ((staged <= MAX_STAGED && (size_t)staged * row_smem <= 200 * 1024) || per_cta <= nwarps) break;
        grid *= 2;
    }
    if (staged > MAX_STAGED || (size_t)staged * row_smem > 200 * 1024)
        return fail(KB_ERR_UNSUPPORTED, "group: %lld activation rows of %zu bytes per CTA do not fit in shared memory", staged, row_smem);
    grid = (total + per_cta - 1) / per_cta;
    GroupParams p;
    p.table = G->table;
    p.count = (int)G->count; p.m = (int)G->m; p.kp = (int)G->kp;
    p.row_bytes = G->row_bytes;
    p.x = x; p.ldx = ldx; p.k = (int)G->k;
    p.x_vec4 = x && (G->k % 4 == 0) && (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    p.xq = xq; p.ldq = ldq; p.sx = sx; p.sumq = sumq;
    p.y = y; p.ldy = ldy;
    p.mul = G->mul; p.off = G->off;
    p.groups_per_cta = (int)per_cta;
    p.staged = (int)staged;
    const bool fullk = G->kp % 2048 == 0;
    void (*kern)(const GroupParams) = nullptr;
#define KB_GROUP_PICK(PF_, TPB_, MINB_)                                                                              \
    kern = x ? (fullk ? gemv_group_kernel<PF_, true, true, TPB_, MINB_> : gemv_group_kernel<PF_, false, true, TPB_, MINB_>) \
             : (fullk ? gemv_group_kernel<PF_, true, false, TPB_, MINB_> : gemv_group_kernel<PF_, false, false, TPB_, MINB_>)
    switch (shape) {
        case 0: KB_GROUP_PICK(3, 256, 2); break;
        case 2: KB_GROUP_PICK(2, 128, 6); break;
        case 3: KB_GROUP_PICK(2, 256, 3); break;
        case 4: KB_GROUP_PICK(3, 128, 4); break;
        default: KB_GROUP_PICK(2, 128, 5); break;
    }
#undef KB_GROUP_PICK
    const size_t smem = (size_t)staged * row_smem;
    if (smem > 40 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "group smem attribute");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "group launch");
}

}  // namespace

}  // namespace kb

using namespace kb;

extern "C" {

int kb_linear_group_create(const kb_linear *const *handles, size_t count, kb_linear_group **out) {
    if (!handles || !out) return fail(KB_ERR_INVALID, "null pointer");
    if (count == 0) return fail(KB_ERR_INVALID, "empty group");
    std::vector<LayerRef> host(count);
    const Linear *first = nullptr;
    for (size_t i = 0; i < count; ++i) {
        const Linear *L = reinterpret_cast<const Linear *>(handles[i]);
        if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle (group member %zu)", i);
        if (!first) first = L;
        if (L->kind != first->kind || L->m != first->m || L->k != first->k || L->device != first->device)
            return fail(KB_ERR_SHAPE, "shape mismatch: group member %zu is [%zu, %zu] kind %d on device %d, member 0 is [%zu, %zu] kind %d on device %d",
                        i, L->m, L->k, L->kind, L->device, first->m, first->k, first->kind, first->device);
        host[i] = LayerRef{L->w2, L->scales, L->bias};
    }
    const size_t row_groups = (first->m + GROUP_R - 1) / GROUP_R;
    if (count * row_groups > (size_t)1 << 30) return fail(KB_ERR_UNSUPPORTED, "group too large: %zu layers of %zu rows", count, first->m);
    ScopedDevice dev(first->device);
    Group *G = new Group{};
    G->device = first->device;
    G->kind = first->kind; G->mul = first->mul; G->off = first->off;
    G->count = count; G->m = first->m; G->k = first->k; G->kp = first->kp; G->row_bytes = first->row_bytes;
    cudaError_t e = cudaMalloc(&G->table, count * sizeof(LayerRef));
    if (e == cudaSuccess) e = cudaMemcpy(G->table, host.data(), count * sizeof(LayerRef), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&G->dx, count * first->k * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&G->dy, count * first->m * sizeof(float));
    if (e != cudaSuccess) {
        if (G->table) cudaFree(G->table);
        if (G->dx) cudaFree(G->dx);
        if (G->dy) cudaFree(G->dy);
        delete G;
        return cuda_fail(e, "group table");
    }
    G->magic = GROUP_MAGIC;
    *out = reinterpret_cast<kb_linear_group *>(G);
    return KB_OK;
}

void kb_linear_group_destroy(kb_linear_group *g) {
    Group *G = reinterpret_cast<Group *>(g);
    if (!G || G->magic != GROUP_MAGIC) return;
    ScopedDevice dev(G->device);
    G->magic = 0;
    cudaFree(G->table);
    cudaFree(G->dx);
    cudaFree(G->dy);
    delete G;
}

size_t kb_linear_group_count(const kb_linear_group *g) {
    const Group *G = check_group(g);
    return G ? G->count : 0;
}

int kb_linear_group_forward_q8(const kb_linear_group *g, const int8_t *xq, size_t ldq, const float *sx, const int32_t *sumq,
                               float *y, size_t ldy, kb_stream stream) {
    const Group *G = check_group(g);
    if (!G) return KB_ERR_BAD_HANDLE;
    if (!xq || !sx || !sumq || !y) return fail(KB_ERR_INVALID, "null activation or output pointer");
    if ((reinterpret_cast<uintptr_t>(xq) & 15) || (ldq % 16) || ldq < G->kp)
        return fail(KB_ERR_INVALID, "group: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", G->kp);
    return group_forward(G, nullptr, 0, xq, ldq, sx, sumq, y, ldy, static_cast<cudaStream_t>(stream));
}

int kb_linear_group_forward(const kb_linear_group *g, const float *x, size_t ldx, float *y, size_t ldy, kb_stream stream) {
    const Group *G = check_group(g);
    if (!G) return KB_ERR_BAD_HANDLE;
    if (!x || !y) return fail(KB_ERR_INVALID, "null activation or output pointer");
    if (ldx == 0) ldx = G->k;
    if (ldx < G->k) return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got row stride %zu", G->k, ldx);
    return group_forward(G, x, ldx, nullptr, 0, nullptr, nullptr, y, ldy, static_cast<cudaStream_t>(stream));
}

int kb_linear_group_forward_host(const kb_linear_group *g, const float *x, float *y) {
    const Group *Gc = check_group(g);
    if (!Gc) return KB_ERR_BAD_HANDLE;
    if (!x || !y) return fail(KB_ERR_INVALID, "null activation or output pointer");
    Group *G = const_cast<Group *>(Gc);  // the staging buffers are the only state a call touches
    std::lock_guard<std::mutex> lock(G->host_mutex);
    ScopedDevice dev(G->device);
    cudaStream_t st = cudaStreamPerThread;
    int rc = KB_OK;
    cudaError_t e;
    if ((e = cudaMemcpyAsync(G->dx, x, G->count * G->k * sizeof(float), cudaMemcpyHostToDevice, st)) != cudaSuccess)
        rc = cuda_fail(e, "activation upload");
    if (rc == KB_OK) rc = group_forward(G, G->dx, G->k, nullptr, 0, nullptr, nullptr, G->dy, G->m, st);
    if (rc == KB_OK && (e = cudaMemcpyAsync(y, G->dy, G->count * G->m * sizeof(float), cudaMemcpyDeviceToHost, st)) != cudaSuccess)
        rc = cuda_fail(e, "output download");
    e = cudaStreamSynchronize(st);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "stream synchronize");
    return rc;
}

}  // extern "C"
