// Streaming decode kernel for 2-bit weights (sm_100a): 1..32 tokens, or one token through each
// of many same-shaped layers in one launch.
//
// HBM-bound byte work: every packed weight byte is read once.  What decides how close a kernel
// gets to the HBM roofline is (a) how many bytes it keeps in flight and (b) how many
// instructions it spends per byte.  Both are addressed by the structure below.
//
//  * Work unit = 16 weight rows x a contiguous slice of K, owned by ONE warp.  Each warp runs a
//    private ring of NST stages in shared memory; a stage holds CH = 256 bytes (1024 codes) of
//    each of the 16 rows.  A stage is filled by 16 one-dimensional bulk copies
//    (cp.async.bulk.shared::cluster.global, one row each, issued by lanes 0..15 as a single warp
//    instruction) that complete on the stage's mbarrier.  Copies run NST stages ahead of the
//    arithmetic and across unit boundaries, they are first issued before the activation prologue
//    and before griddepcontrol.wait, and no CTA-wide barrier exists in the main loop.  With 8
//    warps x 4 stages an SM keeps 128 KB of weight bytes in flight.
//  * Arithmetic = mma.sync.m16n8k32 (u8 x s8 -> s32): rows g / g + 8 of the unit are the A rows,
//    tokens the B columns.  A 32-bit packed word holds 16 codes, element 4j + b in byte b at bits
//    2j, so word & (0x03030303 << 2j) is one A-fragment register whose bytes are 4^j x the codes:
//    one AND per register, no shifts; the four j planes accumulate into four separate
//    accumulators that are exact multiples of 1, 4, 16, 64 and are divided out once per unit.
//    The MMA sums over k inside the instruction, so no shuffle reduction exists, and any k
//    permutation applied to both operands is legal: lane (g, t) takes the 16-byte chunk 4i + t of
//    rows g and g + 8 at step i, and the activation fragment it needs is the matching 64 bytes
//    of token g.  Per 512 bytes of weights a warp issues 16 ANDs, 4 MMAs, 1 + 2 shared-memory
//    loads and a few bookkeeping instructions (the dp4a form needed 72).
//  * Shared-memory layouts are chosen so that every fragment read is conflict-free: stage rows
//    are CH + 64 bytes apart; activation rows are round_up(Kp, 1024) + 64 bytes apart and every
//    256-byte block of a row is stored with its 4 x 4 grid of 16-byte cells transposed.
//  * Codes are unsigned (0..3); the signed value is recovered per output as
//    mul * S - off * sum(xq), then y = (float(acc) * w_scale) * s_x (+ bias) (+ resid), each
//    operation separately rounded.
//  * K split: for a single small layer (few row blocks) KS warps of a CTA share a row block,
//    each streaming 1/KS of K; partial sums meet in shared memory behind a named barrier of
//    those KS warps only.
//
// Every mbarrier wait is bounded (about a second of clock64); on expiry the warp records a
// code in the status word, stops consuming, gives its copies in flight a second bounded wait
// and leaves.
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace kb {

namespace {

using namespace ptx;

constexpr int SW = 8;                // warps per CTA
constexpr int CH = 256;              // bytes of one weight row per stage
constexpr int RS = CH + 64;          // row stride inside a stage
constexpr int STAGE_BYTES = 16 * RS;
constexpr int NST_MAX = 6;
constexpr int BAR_BYTES = 1024;      // SW * NST_MAX barriers, padded so that the stages stay 1 KB aligned
constexpr int MAX_ROWS = 32;         // activation rows a CTA may stage (tokens, or layers of a group)
constexpr long long WAIT_CYCLES = 2000000000ll;
constexpr int DEV_TIMEOUT_STREAM = 20;  // status code of a stage wait that gave up

struct StreamParams {
    // weights: one layer (table == nullptr) or `count` layers
    const LayerRef *table;
    LayerRef one;
    int count;
    int m, k, kp;
    size_t row_bytes;
    int row_blocks;  // ceil(m / 16), per layer
    int nchunks;     // ceil(row_bytes / CH)
    int ks;          // warps sharing a row block (K split), 1 for groups
    int nst;         // stages per warp
    // activations: f32 (quantised in the prologue) or pre-quantised
    const float *x;
    size_t ldx;
    int x_vec4;
    const int8_t *xq;
    size_t ldq;
    const float *sx;
    const int32_t *sumq;
    int n;           // tokens (single layer); groups: one token per layer
    int x_rows;      // activation rows staged per CTA
    int xs_stride;   // bytes between staged rows
    // outputs
    float *y;
    int32_t *acc;
    size_t ldy;
    const float *resid;
    int relu;
    float *y_more[MAX_PEERS - 1];
    int n_more;
    int mul, off;
    int units_per_cta;  // groups: virtual row blocks per CTA (a multiple of SW)
    int *status;
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ bool wait_stage(uint32_t bar, uint32_t parity) {
    long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u) {
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_CYCLES) return false;
        }
    }
}

// byte offset of logical code position o (a multiple of 16) inside a staged activation row: every
// 256-byte block keeps its 4 x 4 grid of 16-byte cells transposed, so that the four fragment reads of
// a lane (cells u = 0..3 of block column t) are 64 bytes apart and the lanes t = 0..3 sit side by side
__device__ __forceinline__ int xs_offset(int o) {
    return (o & ~255) | ((o & 0x30) << 2) | ((o & 0xc0) >> 2);
}

// Block-wide: quantise up to two f32 rows (per-token absmax -> int8, the arithmetic of the quantiser
// kernel) into staged rows d0 / d1 of `cells` 16-byte cells each; codes beyond k are zero.
__device__ __forceinline__ void quantise_rows2(const float *r0, const float *r1, bool live0, bool live1, bool have1, int k,
                                               bool vec4, uint8_t *d0, uint8_t *d1, int cells, float *sc_out, int *sum_out,
                                               float *red_f, int *red_i) {
    const float *row[2] = {r0, r1};
    const bool live[2] = {live0, live1};
    float amax[2] = {0.0f, 0.0f};
    if (vec4) {
        const int nv4 = k >> 2;
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
        for (int i = threadIdx.x; i < k; i += blockDim.x) {
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (live[u]) amax[u] = fmaxf(amax[u], fabsf(row[u][i]));
        }
    }
    // both maxima through one pair of barriers
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax[0] = fmaxf(amax[0], __shfl_xor_sync(0xffffffffu, amax[0], o));
        amax[1] = fmaxf(amax[1], __shfl_xor_sync(0xffffffffu, amax[1], o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { red_f[warp] = amax[0]; red_f[32 + warp] = amax[1]; }
    __syncthreads();
    amax[0] = lane < nwarps ? red_f[lane] : 0.0f;
    amax[1] = lane < nwarps ? red_f[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax[0] = fmaxf(amax[0], __shfl_xor_sync(0xffffffffu, amax[0], o));
        amax[1] = fmaxf(amax[1], __shfl_xor_sync(0xffffffffu, amax[1], o));
    }
    float sc[2], rs[2];
    int local_sum[2] = {0, 0};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        sc[u] = amax[u] < 1e-8f ? 1.0f : __fdiv_rn(amax[u], 127.0f);
        rs[u] = __frcp_rn(sc[u]);
    }
    uint8_t *dst[2] = {d0, d1};
    for (int c = threadIdx.x; c < cells; c += blockDim.x) {
        const int o = c * 16, phys = xs_offset(o);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (u == 1 && !have1) continue;
            uint32_t out[4] = {0u, 0u, 0u, 0u};
            if (live[u] && o < k) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int base = o + w * 4;
                    float v[4];
                    if (vec4 && base + 3 < k) {
                        const float4 f = *reinterpret_cast<const float4 *>(row[u] + base);
                        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = (base + e < k) ? row[u][base + e] : 0.0f;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int q = quantise_one_fast(v[e], sc[u], rs[u]);
                        local_sum[u] += q;
                        out[w] |= (uint32_t)(q & 0xff) << (8 * e);
                    }
                }
            }
            *reinterpret_cast<uint4 *>(dst[u] + phys) = make_uint4(out[0], out[1], out[2], out[3]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        local_sum[0] += __shfl_xor_sync(0xffffffffu, local_sum[0], o);
        local_sum[1] += __shfl_xor_sync(0xffffffffu, local_sum[1], o);
    }
    __syncthreads();
    if (lane == 0) { red_i[warp] = local_sum[0]; red_i[32 + warp] = local_sum[1]; }
    __syncthreads();
    if (warp == 0) {
        int a = lane < nwarps ? red_i[lane] : 0, b = lane < nwarps ? red_i[32 + lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            b += __shfl_xor_sync(0xffffffffu, b, o);
        }
        if (lane == 0) {
            sc_out[0] = live[0] ? sc[0] : 1.0f; sum_out[0] = live[0] ? a : 0;
            if (have1) { sc_out[1] = live[1] ? sc[1] : 1.0f; sum_out[1] = live[1] ? b : 0; }
        }
    }
}

// a position in a warp's sequence of (unit, chunk)
struct Cursor {
    int j;         // ordinal of the unit among this warp's units
    int c, c_end;  // chunk inside the row, end of this unit's K slice
    int rb;        // row block inside the layer
    int layer;     // groups: which layer
    bool valid;
};

// NB = blocks of 8 tokens (single layer); GROUPED: one token per layer, NB = 1
template <int NB, bool GROUPED>
__global__ void __launch_bounds__(SW * 32, 1) gemv_stream_kernel(const StreamParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ float s_sx[MAX_ROWS];
    __shared__ int s_sum[MAX_ROWS];
    __shared__ float red_f[64];
    __shared__ int red_i[64];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nst = p.nst;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar0 = smem_base + (uint32_t)(warp * NST_MAX * 8);
    const uint32_t stage0 = smem_base + BAR_BYTES + (uint32_t)(warp * nst * STAGE_BYTES);
    uint8_t *xs = smem + BAR_BYTES + (size_t)SW * nst * STAGE_BYTES;
    const uint32_t xs_addr = smem_base + BAR_BYTES + (uint32_t)(SW * nst * STAGE_BYTES);
    int *part = reinterpret_cast<int *>(xs + (size_t)p.x_rows * p.xs_stride);  // K split only

    // ---- this warp's units ----
    const int ks = p.ks, slice = GROUPED ? 0 : warp % ks, gi = GROUPED ? 0 : warp / ks, gp = SW / ks;
    int begin = 0, end = 0, layer0 = 0;
    if (GROUPED) {
        const int total = p.count * p.row_blocks;
        begin = min((int)blockIdx.x * p.units_per_cta, total);
        end = min(begin + p.units_per_cta, total);
        layer0 = begin / p.row_blocks;
    }
    auto load_unit = [&](Cursor &u, int j) {
        u.j = j;
        if (GROUPED) {
            const int v = begin + warp + j * SW;
            u.valid = v < end;
            u.layer = v / p.row_blocks;
            u.rb = v - u.layer * p.row_blocks;
            u.c = 0;
            u.c_end = p.nchunks;
        } else {
            u.rb = ((int)blockIdx.x * gp + gi) + j * ((int)gridDim.x * gp);
            u.valid = u.rb < p.row_blocks;
            u.layer = 0;
            u.c = slice * p.nchunks / ks;          // every slice is non-empty: ks <= nchunks
            u.c_end = (slice + 1) * p.nchunks / ks;
        }
    };

    // ---- producer: 16 bulk copies fill one stage ----
    if (lane == 0) {
        for (int s = 0; s < nst; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    Cursor pc;
    load_unit(pc, 0);
    const uint8_t *p_w2 = GROUPED ? nullptr : p.one.w2;
    int p_layer = -1;
    uint32_t fills = 0;
    auto fill = [&]() {
        if (!pc.valid) return;
        const uint32_t s = fills % (uint32_t)nst;
        if (GROUPED && pc.layer != p_layer) { p_layer = pc.layer; p_w2 = p.table[p_layer].w2; }
        const int off = pc.c * CH;
        const uint32_t bytes = (uint32_t)min(CH, (int)p.row_bytes - off);
        if (lane == 0) mbar_expect_tx(bar0 + 8 * s, 16u * bytes);
        __syncwarp();
        if (lane < 16)
            bulk_g2s(stage0 + s * STAGE_BYTES + lane * RS, p_w2 + (size_t)(pc.rb * 16 + lane) * p.row_bytes + off, bytes,
                     bar0 + 8 * s);
        ++fills;
        if (++pc.c == pc.c_end) load_unit(pc, pc.j + 1);
    };
    for (int s = 0; s < nst; ++s) fill();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations -> shared memory (int8, transposed cells) ----
    const int cells = (p.xs_stride - 64) >> 4;
    if (p.x) {
        for (int r0 = 0; r0 < p.x_rows; r0 += 2) {
            const int i0 = GROUPED ? layer0 + r0 : r0, i1 = i0 + 1;
            const int lim = GROUPED ? p.count : p.n;
            const bool have1 = r0 + 1 < p.x_rows;
            if (i0 >= lim) {  // no token / layer behind either row (uniform over the CTA): zero codes, unit scale
                for (int c = threadIdx.x; c < cells * (have1 ? 2 : 1); c += blockDim.x) {
                    const int rr = c >= cells ? 1 : 0, cc_ = c - rr * cells;
                    *reinterpret_cast<uint4 *>(xs + (size_t)(r0 + rr) * p.xs_stride + cc_ * 16) = make_uint4(0, 0, 0, 0);
                }
                if (threadIdx.x < 2 && r0 + (int)threadIdx.x < p.x_rows) { s_sx[r0 + threadIdx.x] = 1.0f; s_sum[r0 + threadIdx.x] = 0; }
                continue;
            }
            quantise_rows2(p.x + (size_t)(i0 < lim ? i0 : 0) * p.ldx, p.x + (size_t)(i1 < lim ? i1 : 0) * p.ldx, i0 < lim,
                           have1 && i1 < lim, have1, p.k, p.x_vec4 != 0, xs + (size_t)r0 * p.xs_stride,
                           xs + (size_t)(r0 + 1) * p.xs_stride, cells, s_sx + r0, s_sum + r0, red_f, red_i);
        }
    } else {
        const int lim = GROUPED ? p.count : p.n;
        for (int idx = threadIdx.x; idx < p.x_rows * cells; idx += blockDim.x) {
            const int r = idx / cells, c = idx - r * cells;
            const int src_row = GROUPED ? layer0 + r : r;
            const int o = c * 16;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src_row < lim && o < p.kp) v = *reinterpret_cast<const uint4 *>(p.xq + (size_t)src_row * p.ldq + o);
            *reinterpret_cast<uint4 *>(xs + (size_t)r * p.xs_stride + xs_offset(o)) = v;
        }
        if ((int)threadIdx.x < p.x_rows) {
            const int src_row = GROUPED ? layer0 + threadIdx.x : threadIdx.x;
            s_sx[threadIdx.x] = src_row < lim ? p.sx[src_row] : 1.0f;
            s_sum[threadIdx.x] = src_row < lim ? p.sumq[src_row] : 0;
        }
    }
    __syncthreads();

    // ---- consumer ----
    int acc[NB][4][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[nb][j][0] = acc[nb][j][1] = acc[nb][j][2] = acc[nb][j][3] = 0;

    Cursor cc;
    load_unit(cc, 0);
    // per-unit epilogue constants of rows g and g + 8, fetched when the unit starts
    const LayerRef *ref_tab = p.table;
    LayerRef ref = p.one;
    int ref_layer = GROUPED ? -1 : 0;
    float sw0 = 0.f, sw1 = 0.f, bi0 = 0.f, bi1 = 0.f;
    bool has_bias = false;
    auto fetch_consts = [&](const Cursor &u) {
        if (!u.valid) return;
        if (GROUPED && u.layer != ref_layer) { ref_layer = u.layer; ref = ref_tab[ref_layer]; }
        const int row = u.rb * 16 + g;  // rows up to m_alloc - 1 are allocated
        sw0 = ref.sw[row]; sw1 = ref.sw[row + 8];
        has_bias = ref.bias != nullptr;
        if (has_bias) { bi0 = ref.bias[row]; bi1 = ref.bias[row + 8]; }
    };
    fetch_consts(cc);

    uint32_t cons = 0;
    int parity = 0;
    bool ok = true;
    while (cc.valid) {
        const uint32_t s = cons % (uint32_t)nst, ph = (cons / (uint32_t)nst) & 1u;
        if (ok && !(ok = wait_stage(bar0 + 8 * s, ph))) pc.valid = false;  // gave up: no more copies, no more waits
        if (ok) {
            const int off = cc.c * CH;
            const int bytes = min(CH, (int)p.row_bytes - off);
            const int ni = (bytes + 63) >> 6;
            const uint32_t sg = stage0 + s * STAGE_BYTES + g * RS + t * 16, sh = sg + 8 * RS;
            const int xrow = GROUPED ? cc.layer - layer0 : g;
            const uint32_t xa = xs_addr + (uint32_t)(xrow * p.xs_stride) + (uint32_t)(off * 4) + t * 16;
#pragma unroll
            for (int i = 0; i < CH / 64; ++i) {
                if (i < ni) {
                    const uint4 wa = lds128(sg + 64 * i), wb = lds128(sh + 64 * i);
                    const uint32_t a[4] = {wa.x, wa.y, wa.z, wa.w}, b[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const uint32_t xb = xa + (uint32_t)(nb * 8 * p.xs_stride) + 256 * i;
                        uint4 xv[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) xv[u] = lds128(xb + 64 * u);
#pragma unroll
                        for (int pp = 0; pp < 2; ++pp) {
                            const uint4 x0 = xv[2 * pp], x1 = xv[2 * pp + 1];
                            const uint32_t xb0[4] = {x0.x, x0.y, x0.z, x0.w}, xb1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t mk = 0x03030303u << (2 * j);
                                mma_u8s8(acc[nb][j], a[2 * pp] & mk, b[2 * pp] & mk, a[2 * pp + 1] & mk, b[2 * pp + 1] & mk,
                                         xb0[j], xb1[j]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();  // every lane has read the stage: it can be refilled
        fill();
        if (ok) ++cons;
        if (++cc.c == cc.c_end) {
            // ---- unit finished: combine the four scaled accumulators (exact), K-split partials, epilogue ----
            int v[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    v[nb][r] = acc[nb][0][r] + (acc[nb][1][r] >> 2) + (acc[nb][2][r] >> 4) + (acc[nb][3][r] >> 6);
                    acc[nb][0][r] = acc[nb][1][r] = acc[nb][2][r] = acc[nb][3][r] = 0;
                }
            bool finisher = true;
            if (!GROUPED && ks > 1) {
                int *mine = part + (size_t)((gi * 2 + parity) * ks + slice) * (NB * 4 * 32);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int r = 0; r < 4; ++r) mine[(nb * 4 + r) * 32 + lane] = v[nb][r];
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
                finisher = slice == 0;
                if (finisher) {
                    const int *base = part + (size_t)((gi * 2 + parity) * ks) * (NB * 4 * 32);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            int sum = 0;
                            for (int q = 0; q < ks; ++q) sum += base[q * (NB * 4 * 32) + (nb * 4 + r) * 32 + lane];
                            v[nb][r] = sum;
                        }
                }
                parity ^= 1;
            }
            if (finisher) {
                // lane (g, t) holds rows g (r = 0, 1) and g + 8 (r = 2, 3) x tokens 8 nb + 2t (r even), + 1 (r odd)
                const int row0 = cc.rb * 16 + g;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int row = row0 + (r >> 1) * 8;
                        const int col = 2 * t + (r & 1);
                        const int tok = GROUPED ? cc.layer : nb * 8 + col;
                        const int xr = GROUPED ? cc.layer - layer0 : nb * 8 + col;
                        const bool live = GROUPED ? col == 0 : tok < p.n;
                        if (live && row < p.m) {
                            const int a = p.mul * v[nb][r] - p.off * s_sum[xr];
                            const size_t o = (size_t)tok * p.ldy + row;
                            if (p.acc) p.acc[o] = a;
                            if (p.y) {
                                float out = dequant_out(a, (r >> 1) ? sw1 : sw0, s_sx[xr], (r >> 1) ? bi1 : bi0, has_bias);
                                if (p.resid) out = __fadd_rn(out, p.resid[o]);
                                if (p.relu) out = fmaxf(out, 0.0f);
                                p.y[o] = out;
                                for (int q = 0; q < p.n_more; ++q) p.y_more[q][o] = out;  // peer copies over NVLink
                            }
                        }
                    }
            }
            load_unit(cc, cc.j + 1);
            fetch_consts(cc);
        }
    }
    if (!ok) {
        // a wait gave up (the warp then walked its remaining units without computing, so that the warps
        // it shares row blocks with still met it at their barriers): report, and give the copies that
        // are still in flight towards this CTA's shared memory a second bounded wait before leaving
        if (lane == 0 && p.status) atomicCAS(p.status, 0, DEV_TIMEOUT_STREAM);
        for (uint32_t f = cons; f < fills; ++f)
            if (!wait_stage(bar0 + 8 * (f % (uint32_t)nst), (f / (uint32_t)nst) & 1u)) break;
    }
    if (p.n_more) __threadfence_system();
}

size_t xs_stride_for(size_t kp) { return (kp + 1023) / 1024 * 1024 + 64; }

// stages per warp that fit beside `x_rows` staged activation rows and the K-split scratch (0: does not fit)
int stages_that_fit(size_t kp, int x_rows, size_t part_bytes) {
    const size_t budget = 224 * 1024;  // leaves room for the static arrays
    const size_t fixed = BAR_BYTES + (size_t)x_rows * xs_stride_for(kp) + part_bytes;
    if (fixed + (size_t)SW * 2 * STAGE_BYTES > budget) return 0;
    size_t nst = (budget - fixed) / ((size_t)SW * STAGE_BYTES);
    static const int env_nst = [] { const char *v = getenv("KB_STREAM_NST"); return v && *v ? atoi(v) : 0; }();
    size_t cap = 4;
    if (env_nst >= 2 && env_nst <= NST_MAX) cap = (size_t)env_nst;
    return (int)(nst > cap ? cap : nst);
}

template <int NB, bool GROUPED>
int launch_stream(const StreamParams &p, int device, int grid, size_t smem, cudaStream_t stream) {
    auto kern = gemv_stream_kernel<NB, GROUPED>;
    if (int rc = set_dyn_smem_once(reinterpret_cast<const void *>(kern), device, 227 * 1024 - 2048, "stream smem attribute")) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(SW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool pdl = [] { const char *v = getenv("KB_GEMV_PDL"); return !(v && *v == '0'); }();
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "stream launch");
}

}  // namespace

bool gemv_stream_supports(const Linear *lin, size_t n) {
    if (n < 1 || n > 32 || lin->kp > 80000) return false;  // 64 * 3 * 127 * K must stay below 2^31
    const int nb = n <= 8 ? 1 : (n <= 16 ? 2 : 4);
    return stages_that_fit(lin->kp, nb * 8, (size_t)SW * 2 * nb * 512) >= 2;
}

int launch_gemv_stream(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!gemv_stream_supports(L, a.n))
        return fail(KB_ERR_UNSUPPORTED, "streaming kernel: %zu tokens x K=%zu do not fit in shared memory", a.n, L->k);
    if (a.x && a.n > 8) return fail(KB_ERR_UNSUPPORTED, "streaming kernel: the fused quantiser takes up to 8 tokens");
    if (!a.x) {
        if (!a.xq || !a.sx || !a.sumq) return fail(KB_ERR_INVALID, "streaming kernel: needs activations");
        if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
            return fail(KB_ERR_INVALID, "gemv: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    }
    const int nb = a.n <= 8 ? 1 : (a.n <= 16 ? 2 : 4);
    StreamParams p = {};
    p.table = nullptr;
    p.one = LayerRef{L->w2, L->scales, L->bias};
    p.count = 1;
    p.m = (int)L->m; p.k = (int)L->k; p.kp = (int)L->kp;
    p.row_bytes = L->row_bytes;
    p.row_blocks = (int)((L->m + 15) / 16);
    p.nchunks = (int)((L->row_bytes + CH - 1) / CH);
    const int sms = sm_count(L->device);
    // K split: enough (row block, slice) units to give every warp of every SM one
    int ks = 1;
    static const int env_ks = [] { const char *v = getenv("KB_STREAM_KS"); return v && *v ? atoi(v) : 0; }();
    while (ks < SW && ks * 2 <= p.nchunks && (long long)p.row_blocks * ks < (long long)sms * SW) ks *= 2;
    if (env_ks == 1 || env_ks == 2 || env_ks == 4 || env_ks == 8) ks = env_ks <= p.nchunks ? env_ks : ks;
    p.ks = ks;
    const size_t part_bytes = ks > 1 ? (size_t)SW * 2 * nb * 512 : 0;
    p.x_rows = nb * 8;
    p.xs_stride = (int)xs_stride_for(L->kp);
    p.nst = stages_that_fit(L->kp, p.x_rows, part_bytes);
    p.x = a.x; p.ldx = L->k;
    p.x_vec4 = a.x && (L->k % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    p.xq = a.xq; p.ldq = a.ldq; p.sx = a.sx; p.sumq = a.sumq;
    p.n = (int)a.n;
    p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    p.n_more = a.y ? a.n_more : 0;
    for (int q = 0; q < MAX_PEERS - 1; ++q) p.y_more[q] = q < p.n_more ? a.y_more[q] : nullptr;
    p.mul = L->mul; p.off = L->off;
    p.units_per_cta = 0;
    p.status = L->dev_status;
    const int gp = SW / ks;
    int grid = (p.row_blocks + gp - 1) / gp;
    if (grid > sms) grid = sms;
    const size_t smem = BAR_BYTES + (size_t)SW * p.nst * STAGE_BYTES + (size_t)p.x_rows * p.xs_stride + part_bytes;
    if (nb == 1) return launch_stream<1, false>(p, L->device, grid, smem, stream);
    if (nb == 2) return launch_stream<2, false>(p, L->device, grid, smem, stream);
    return launch_stream<4, false>(p, L->device, grid, smem, stream);
}

int launch_group_stream(const GroupArgs &a, cudaStream_t stream) {
    if (a.kp > 80000) return fail(KB_ERR_UNSUPPORTED, "group: K=%zu too large for the int32 partial sums", a.k);
    StreamParams p = {};
    p.table = a.table;
    p.count = (int)a.count;
    p.m = (int)a.m; p.k = (int)a.k; p.kp = (int)a.kp;
    p.row_bytes = a.row_bytes;
    p.row_blocks = (int)((a.m + 15) / 16);
    p.nchunks = (int)((a.row_bytes + CH - 1) / CH);
    p.ks = 1;
    const long long total = (long long)a.count * p.row_blocks;
    if (total > (1ll << 30)) return fail(KB_ERR_UNSUPPORTED, "group too large: %zu layers of %zu rows", a.count, a.m);
    // one CTA per SM; grown (shorter ranges touch fewer layers) until a CTA's activation rows fit
    long long grid = sm_count(a.device);
    long long per_cta = 0, staged = 0;
    int nst = 0;
    for (;;) {
        per_cta = (total + grid - 1) / grid;
        per_cta = (per_cta + SW - 1) / SW * SW;
        staged = (per_cta + p.row_blocks - 2) / p.row_blocks + 1;
        if (staged > (long long)a.count) staged = (long long)a.count;
        nst = staged <= MAX_ROWS ? stages_that_fit(a.kp, (int)staged, 0) : 0;
        if (nst >= 2 || per_cta <= SW) break;
        grid *= 2;
    }
    if (nst < 2)
        return fail(KB_ERR_UNSUPPORTED, "group: %lld activation rows of %zu bytes per CTA do not fit in shared memory", staged,
                    xs_stride_for(a.kp));
    grid = (total + per_cta - 1) / per_cta;
    p.nst = nst;
    p.x = a.x; p.ldx = a.ldx;
    p.x_vec4 = a.x && (a.k % 4 == 0) && (a.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    p.xq = a.xq; p.ldq = a.ldq; p.sx = a.sx; p.sumq = a.sumq;
    p.n = 1;
    p.x_rows = (int)staged;
    p.xs_stride = (int)xs_stride_for(a.kp);
    p.y = a.y; p.acc = nullptr; p.ldy = a.ldy;
    p.mul = a.mul; p.off = a.off;
    p.units_per_cta = (int)per_cta;
    p.status = a.status;
    const size_t smem = BAR_BYTES + (size_t)SW * p.nst * STAGE_BYTES + (size_t)p.x_rows * p.xs_stride;
    return launch_stream<1, true>(p, a.device, (int)grid, smem, stream);
}

}  // namespace kb
