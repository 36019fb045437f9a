// Streaming decode kernel for 2-bit weights (sm_100a): 1..32 tokens, or one token through each
// of many same-shaped layers in one launch.
//
// HBM-bound byte work: every packed weight byte is read once.  What decides how close a kernel
// gets to the HBM roofline is (a) how many bytes it keeps in flight and (b) how many
// instructions it spends per byte.  Both are addressed by the structure below.
//
//  * Work unit = 16 weight rows x a contiguous slice of K, owned by ONE warp.  Each warp runs a
//    private ring of NST stages in shared memory; a stage holds CH = 256 bytes (1024 codes) of
//    each of the 16 rows.  A stage is filled by 16-byte asynchronous copies (cp.async.cg, global ->
//    shared without passing through registers or L1; one warp instruction moves 256 contiguous
//    bytes of two rows) whose completion arrives on the stage's mbarrier
//    (cp.async.mbarrier.arrive.noinc).  One-dimensional bulk copies (cp.async.bulk, one 256-byte
//    row piece per request) were measured first and delivered only 2.8 TB/s: the copy engine's
//    request rate, not HBM, was the limit at that size.  Copies run NST stages ahead of the
//    arithmetic and across unit boundaries, they are first issued before the activation prologue
//    and before griddepcontrol.wait, and no CTA-wide barrier exists in the main loop.  With 8
//    warps x 4 stages an SM keeps 128 KB of weight bytes in flight.
//  * Arithmetic, 3..32 tokens = mma.sync.m16n8k32 (u8 x s8 -> s32): rows g / g + 8 of the unit are the A
//    rows, tokens the B columns.  A 32-bit packed word holds 16 codes, element 4j + b in byte b at bits
//    2j, so word & (0x03030303 << 2j) is one A-fragment register whose bytes are 4^j x the codes:
//    one AND per register, no shifts; the four j planes accumulate into four separate
//    accumulators that are exact multiples of 1, 4, 16, 64 and are divided out once per unit.
//    The MMA sums over k inside the instruction, so no shuffle reduction exists, and any k
//    permutation applied to both operands is legal: lane (g, t) takes the 16-byte chunk 4i + t of
//    rows g and g + 8 at step i, and the activation fragment it needs is the matching 64 bytes
//    of token g.  Per 512 bytes of weights a warp issues 16 ANDs, 4 MMAs and 1 + 4 shared-memory loads.
//  * Arithmetic, 1..2 tokens = dp4a.  The warp-level int8 MMA of this GPU retires one m16n8k32 per
//    ~4.5 cycles per SM (measured: 8 useful columns or 1, the cost is the same), which for a single
//    token is slower than HBM delivers the weights.  Here lane (c = lane % 16, h = lane / 16) owns
//    16-byte cell c of the stage's rows h, h + 2, ..., h + 14: its 64 activation codes are read
//    once per stage and stay in registers for the eight rows, the same AND masks feed
//    dp4a.u32.s32 into four scaled accumulators per row, and the sixteen lanes of a row meet once
//    per unit in a transposing shuffle reduction (8 shuffles for 8 rows).  Per 512 bytes of weights:
//    16 ANDs, 16 dp4a, 1.5 shared-memory loads, 1 copy instruction (the register-pipelined
//    dp4a kernel this replaces needed 72 instructions and was issue-bound).
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

constexpr int CH = 256;              // bytes of one weight row per stage
constexpr int RS = CH + 64;          // row stride inside a stage
constexpr int STAGE_BYTES = 16 * RS;
constexpr int NST_MAX = 6;
constexpr int BAR_BYTES = 1024;      // 16 warps x NST_MAX barriers, padded so that the stages stay 1 KB aligned
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
    int units_per_cta;  // groups: virtual row blocks per CTA
    int *status;
    // column-sharded layers in a chain (sync.world > 0): before it touches its activations the launch waits,
    // bounded, until every peer has published the PREVIOUS forward of the chain (the wait hides behind the weight
    // stream that is already in flight); after its last store it publishes this one without waiting
    PeerSync sync;
    // flagged words (see FwdArgs): activations as (value, epoch) pairs, outputs stored as such pairs;
    // epoch = (*flag_round << 8) | position in the chain (x: flag_seq - 1, y: flag_seq)
    const uint2 *xf;
    size_t ldxf;
    int y_flagged;
    const int *flag_round;
    int flag_seq;
};

// 16-byte asynchronous copy global -> shared that bypasses L1 and the register file
template <int DST_OFF>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1], 16;" ::"r"(dst), "l"(src), "n"(DST_OFF) : "memory");
}
// the barrier receives one arrival from this thread once all its earlier cp.async have landed
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// 16-byte shared-memory read at base + a compile-time offset (the offset folds into the instruction)
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
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

// The same for 16-byte aligned rows of at most CPT cells per thread: the rows stay in registers between the maximum
// and the quantisation, so a launch pays one memory round trip for its activations instead of two.
template <int CPT>
__device__ __forceinline__ void quantise_rows2_regs(const float *r0, const float *r1, bool live0, bool live1, bool have1, int k,
                                                    uint8_t *d0, uint8_t *d1, int cells, float *sc_out, int *sum_out, float *red_f,
                                                    int *red_i) {
    const float *row[2] = {r0, r1};
    const bool live[2] = {live0, live1};
    const int nv4 = k >> 2;
    float4 v[2][CPT][4];
    float amax[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int j = c * 4 + w;
                v[u][i][w] = (live[u] && j < nv4) ? reinterpret_cast<const float4 *>(row[u])[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i)
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int w = 0; w < 4; ++w)
                amax[u] = fmaxf(amax[u], fmaxf(fmaxf(fabsf(v[u][i][w].x), fabsf(v[u][i][w].y)), fmaxf(fabsf(v[u][i][w].z), fabsf(v[u][i][w].w))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax[0] = fmaxf(amax[0], __shfl_xor_sync(0xffffffffu, amax[0], o));
        amax[1] = fmaxf(amax[1], __shfl_xor_sync(0xffffffffu, amax[1], o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { red_f[warp] = amax[0]; red_f[32 + warp] = amax[1]; }
    __syncthreads();
    amax[0] = amax[1] = 0.0f;
    for (int w = 0; w < nwarps; ++w) { amax[0] = fmaxf(amax[0], red_f[w]); amax[1] = fmaxf(amax[1], red_f[32 + w]); }
    float sc[2], rs[2];
    int local_sum[2] = {0, 0};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        sc[u] = amax[u] < 1e-8f ? 1.0f : __fdiv_rn(amax[u], 127.0f);
        rs[u] = __frcp_rn(sc[u]);
    }
    uint8_t *dst[2] = {d0, d1};
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < cells) {
            const int phys = xs_offset(c * 16);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u == 1 && !have1) continue;
                uint32_t out[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int q0 = quantise_one_fast(v[u][i][w].x, sc[u], rs[u]), q1 = quantise_one_fast(v[u][i][w].y, sc[u], rs[u]);
                    const int q2 = quantise_one_fast(v[u][i][w].z, sc[u], rs[u]), q3 = quantise_one_fast(v[u][i][w].w, sc[u], rs[u]);
                    local_sum[u] += q0 + q1 + q2 + q3;
                    out[w] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                }
                *reinterpret_cast<uint4 *>(dst[u] + phys) = make_uint4(out[0], out[1], out[2], out[3]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        local_sum[0] += __shfl_xor_sync(0xffffffffu, local_sum[0], o);
        local_sum[1] += __shfl_xor_sync(0xffffffffu, local_sum[1], o);
    }
    if (lane == 0) { red_i[warp] = local_sum[0]; red_i[32 + warp] = local_sum[1]; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, b = 0;
        for (int w = 0; w < nwarps; ++w) { a += red_i[w]; b += red_i[32 + w]; }
        sc_out[0] = live[0] ? sc[0] : 1.0f; sum_out[0] = live[0] ? a : 0;
        if (have1) { sc_out[1] = live[1] ? sc[1] : 1.0f; sum_out[1] = live[1] ? b : 0; }
    }
}

constexpr int DEV_TIMEOUT_FLAGGED = 110;  // status code: a flagged activation pair never showed its epoch

// two (value, epoch) pairs with one 16-byte load that is neither cached in L1 nor reordered by the compiler
__device__ __forceinline__ uint4 ld_pairs(const uint2 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// 16 consecutive values of a flagged row from element e0 (k is a multiple of 4, rows are 16-byte aligned, so the
// 16-byte loads never straddle the row's end): waits, bounded, until every pair carries `epoch`.  Elements from k on are 0.
__device__ __forceinline__ bool load_cell_flagged(const uint2 *row, bool live, int e0, int k, uint32_t epoch, float (&v)[16],
                                                  long long &t0) {
    uint4 raw[8];
    bool need[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        need[w] = live && e0 + 2 * w < k;
        raw[w] = need[w] ? ld_pairs(row + e0 + 2 * w) : make_uint4(0u, epoch, 0u, epoch);
    }
    bool ok = true;
    for (;;) {
        bool all = true;
#pragma unroll
        for (int w = 0; w < 8; ++w)
            if (raw[w].y != epoch || raw[w].w != epoch) {
                all = false;
                raw[w] = ld_pairs(row + e0 + 2 * w);
            }
        if (all) break;
        const long long now = clock64();
        if (t0 == 0) t0 = now;
        else if (now - t0 > WAIT_CYCLES) { ok = false; break; }
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        v[2 * w] = __uint_as_float(raw[w].x);
        v[2 * w + 1] = __uint_as_float(raw[w].z);
    }
    return ok;
}

// Block-wide: the quantiser of quantise_rows2 on up to two rows of flagged words.  CPT > 0: a thread owns at most CPT
// cells of 16 values per row and keeps them in registers between the maximum and the quantisation; CPT == 0: any
// number of cells, read twice (the second read finds the pairs it has already seen).  A pair that never shows its
// epoch ends the wait after about a second with a status code; the launch then runs on with whatever it read.
template <int CPT>
__device__ __forceinline__ void quantise_rows2_flagged(const uint2 *r0, const uint2 *r1, bool live0, bool live1, bool have1, int k,
                                                       uint32_t epoch, int *status, uint8_t *d0, uint8_t *d1, int cells,
                                                       float *sc_out, int *sum_out, float *red_f, int *red_i) {
    constexpr int HOLD = CPT > 0 ? CPT : 1;
    const uint2 *row[2] = {r0, r1};
    const bool live[2] = {live0, live1};
    float v[2][HOLD][16];
    float amax[2] = {0.0f, 0.0f};
    long long t0 = 0;
    bool ok = true;
    if (CPT > 0) {
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                ok &= load_cell_flagged(row[u], live[u] && c < cells, c * 16, k, epoch, v[u][i], t0);
#pragma unroll
                for (int e = 0; e < 16; ++e) amax[u] = fmaxf(amax[u], fabsf(v[u][i][e]));
            }
        }
    } else {
        for (int c = threadIdx.x; c < cells; c += blockDim.x)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                ok &= load_cell_flagged(row[u], live[u], c * 16, k, epoch, v[u][0], t0);
#pragma unroll
                for (int e = 0; e < 16; ++e) amax[u] = fmaxf(amax[u], fabsf(v[u][0][e]));
            }
    }
    if (!ok && status) atomicCAS(status, 0, DEV_TIMEOUT_FLAGGED);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax[0] = fmaxf(amax[0], __shfl_xor_sync(0xffffffffu, amax[0], o));
        amax[1] = fmaxf(amax[1], __shfl_xor_sync(0xffffffffu, amax[1], o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { red_f[warp] = amax[0]; red_f[32 + warp] = amax[1]; }
    __syncthreads();
    amax[0] = amax[1] = 0.0f;
    for (int w = 0; w < nwarps; ++w) { amax[0] = fmaxf(amax[0], red_f[w]); amax[1] = fmaxf(amax[1], red_f[32 + w]); }
    float sc[2], rs[2];
    int local_sum[2] = {0, 0};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        sc[u] = amax[u] < 1e-8f ? 1.0f : __fdiv_rn(amax[u], 127.0f);
        rs[u] = __frcp_rn(sc[u]);
    }
    uint8_t *dst[2] = {d0, d1};
    auto emit = [&](int c, int u, const float (&val)[16]) {
        uint32_t out[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int q0 = quantise_one_fast(val[4 * w], sc[u], rs[u]), q1 = quantise_one_fast(val[4 * w + 1], sc[u], rs[u]);
            const int q2 = quantise_one_fast(val[4 * w + 2], sc[u], rs[u]), q3 = quantise_one_fast(val[4 * w + 3], sc[u], rs[u]);
            local_sum[u] += q0 + q1 + q2 + q3;
            out[w] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        }
        *reinterpret_cast<uint4 *>(dst[u] + xs_offset(c * 16)) = make_uint4(out[0], out[1], out[2], out[3]);
    };
    if (CPT > 0) {
#pragma unroll
        for (int i = 0; i < HOLD; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < cells) {
                emit(c, 0, v[0][i]);
                if (have1) emit(c, 1, v[1][i]);
            }
        }
    } else {
        for (int c = threadIdx.x; c < cells; c += blockDim.x)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u == 1 && !have1) continue;
                load_cell_flagged(row[u], live[u], c * 16, k, epoch, v[u][0], t0);
                emit(c, u, v[u][0]);
            }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        local_sum[0] += __shfl_xor_sync(0xffffffffu, local_sum[0], o);
        local_sum[1] += __shfl_xor_sync(0xffffffffu, local_sum[1], o);
    }
    if (lane == 0) { red_i[warp] = local_sum[0]; red_i[32 + warp] = local_sum[1]; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, b = 0;
        for (int w = 0; w < nwarps; ++w) { a += red_i[w]; b += red_i[32 + w]; }
        sc_out[0] = live[0] ? sc[0] : 1.0f; sum_out[0] = live[0] ? a : 0;
        if (have1) { sc_out[1] = live[1] ? sc[1] : 1.0f; sum_out[1] = live[1] ? b : 0; }
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

// NT > 0: dp4a form for NT tokens (1 or 2; GROUPED: one token per layer, NT = 1).
// NT == 0: MMA form for NB blocks of 8 tokens.  W = most warps per CTA (bounds the registers).
template <int NB, bool GROUPED, int NT, int W>
__global__ void __launch_bounds__(W * 32, 1) gemv_stream_kernel(const StreamParams p) {
    constexpr bool DP = NT > 0;
    constexpr int NV = DP ? NT : NB * 4;  // values a lane holds when a unit ends
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ float s_sx[MAX_ROWS];
    __shared__ int s_sum[MAX_ROWS];
    __shared__ float red_f[64];
    __shared__ int red_i[64];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sw = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nst = p.nst;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar0 = smem_base + (uint32_t)(warp * NST_MAX * 8);
    const uint32_t stage0 = smem_base + BAR_BYTES + (uint32_t)(warp * nst * STAGE_BYTES);
    uint8_t *xs = smem + BAR_BYTES + (size_t)sw * nst * STAGE_BYTES;
    const uint32_t xs_addr = smem_base + BAR_BYTES + (uint32_t)(sw * nst * STAGE_BYTES);
    int *part = reinterpret_cast<int *>(xs + (size_t)p.x_rows * p.xs_stride);  // K split only

    // ---- this warp's units ----
    const int ks = p.ks, slice = GROUPED ? 0 : warp % ks, gi = GROUPED ? 0 : warp / ks, gp = sw / ks;
    int begin = 0, end = 0, layer0 = 0;
    if (GROUPED) {
        const int total = p.count * p.row_blocks;
        begin = min((int)blockIdx.x * p.units_per_cta, total);
        end = min(begin + p.units_per_cta, total);
        layer0 = begin / p.row_blocks;
    }
    // a warp's units are visited in order; (layer, rb) follow without divisions
    const int c_first = GROUPED ? 0 : slice * p.nchunks / ks;  // every slice is non-empty: ks <= nchunks
    const int c_last = GROUPED ? p.nchunks : (slice + 1) * p.nchunks / ks;
    auto first_unit = [&](Cursor &u) {
        u.j = 0;
        if (GROUPED) {
            const int v = begin + warp;
            u.valid = v < end;
            u.layer = v / p.row_blocks;
            u.rb = v - u.layer * p.row_blocks;
        } else {
            u.rb = (int)blockIdx.x * gp + gi;
            u.valid = u.rb < p.row_blocks;
            u.layer = 0;
        }
        u.c = c_first;
        u.c_end = c_last;
    };
    auto next_unit = [&](Cursor &u) {
        ++u.j;
        if (GROUPED) {
            u.rb += sw;
            while (u.rb >= p.row_blocks) { u.rb -= p.row_blocks; ++u.layer; }
            u.valid = begin + warp + u.j * sw < end;
        } else {
            u.rb += (int)gridDim.x * gp;
            u.valid = u.rb < p.row_blocks;
        }
        u.c = c_first;
    };

    // ---- producer: eight 16-byte asynchronous copies per lane fill one stage ----
    if (lane == 0) {
        for (int s = 0; s < nst; ++s) mbar_init(bar0 + 8 * s, 32);  // one arrival per lane and fill
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    Cursor pc;
    first_unit(pc);
    const uint8_t *p_w2 = GROUPED ? nullptr : p.one.w2;
    int p_layer = -1;
    uint32_t fills = 0, fs = 0;  // fills issued, and the stage the next one goes to
    // 256 cells of 16 bytes per stage (16 rows x CH): cell e = 32 q + lane -> row e / 16, column e % 16, so one
    // warp instruction copies two rows' 256 contiguous bytes.  p_src = this lane's first cell of the current unit
    const uint32_t lane_dst = stage0 + (lane >> 4) * RS + (lane & 15) * 16;
    const int lane_col = (lane & 15) * 16;
    const size_t two_rows = 2 * p.row_bytes;
    const uint8_t *p_src = nullptr;
    auto unit_src = [&]() {
        if (!pc.valid) return;
        if (GROUPED && pc.layer != p_layer) { p_layer = pc.layer; p_w2 = p.table[p_layer].w2; }
        p_src = p_w2 + (size_t)(pc.rb * 16 + (lane >> 4)) * p.row_bytes + lane_col;
    };
    unit_src();
    auto fill = [&]() {
        if (!pc.valid) return;
        const uint32_t dst = lane_dst + fs * STAGE_BYTES, bar = bar0 + 8 * fs;
        fs = fs + 1 == (uint32_t)nst ? 0 : fs + 1;
        const int off = pc.c * CH;
        if (lane_col < (int)p.row_bytes - off) {  // cells beyond the row's end are not copied (they meet zero codes)
            const uint8_t *src = p_src + off;
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
        ++fills;
        if (++pc.c == pc.c_end) { next_unit(pc); unit_src(); }
    };
    for (int s = 0; s < nst; ++s) fill();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    __shared__ uint32_t s_epoch;
    const bool flagged = p.xf != nullptr || p.y_flagged != 0;
    if (flagged) {
        // the round changes only in the unpack that ends a chain, which is complete once the wait above returns
        if (threadIdx.x == 0) s_epoch = (uint32_t)(*reinterpret_cast<const volatile int *>(p.flag_round)) << 8;
        __syncthreads();
    }
    const uint32_t x_epoch = flagged ? (s_epoch | (uint32_t)(p.flag_seq - 1)) : 0u, y_epoch = flagged ? (s_epoch | (uint32_t)p.flag_seq) : 0u;

    if (p.sync.world > 0) {
        // every peer's previous forward has landed in this rank's buffers (and, by the same token, every peer
        // has finished reading the buffer this forward is about to overwrite)
        if ((int)threadIdx.x < p.sync.world) {
            const int j = threadIdx.x;
            const int want = *reinterpret_cast<volatile int *>(p.sync.epoch_counter);  // forwards published so far by this rank
            const volatile int *mine = p.sync.flag_arrays[p.sync.rank] + j;
            const long long t0 = clock64();
            bool ok = false;
            for (;;) {
                if (*mine - want >= 0) { ok = true; break; }
                if (clock64() - t0 > WAIT_CYCLES) break;
            }
            __threadfence_system();  // acquire side: later reads of the peers' slices see their data
            if (!ok) atomicCAS(p.sync.status, 0, 100 + j);  // peer j never arrived
        }
        __syncthreads();
    }

    // ---- activations -> shared memory (int8, transposed cells) ----
    const int cells = (p.xs_stride - 64) >> 4;
    if (p.xf) {
        for (int r0 = 0; r0 < p.x_rows; r0 += 2) {
            const bool have1 = r0 + 1 < p.x_rows;
            const uint2 *ra = p.xf + (size_t)r0 * p.ldxf, *rb_ = p.xf + (size_t)(have1 ? r0 + 1 : r0) * p.ldxf;
            uint8_t *da = xs + (size_t)r0 * p.xs_stride, *db = xs + (size_t)(r0 + 1) * p.xs_stride;
            const int cpt = (cells + (int)blockDim.x - 1) / (int)blockDim.x;
            if (r0 > 0) __syncthreads();
            if (cpt == 1)
                quantise_rows2_flagged<1>(ra, rb_, true, have1, have1, p.k, x_epoch, p.status, da, db, cells, s_sx + r0, s_sum + r0, red_f, red_i);
            else
                quantise_rows2_flagged<0>(ra, rb_, true, have1, have1, p.k, x_epoch, p.status, da, db, cells, s_sx + r0, s_sum + r0, red_f, red_i);
        }
    } else if (p.x) {
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
            const float *ra = p.x + (size_t)(i0 < lim ? i0 : 0) * p.ldx, *rb_ = p.x + (size_t)(i1 < lim ? i1 : 0) * p.ldx;
            uint8_t *da = xs + (size_t)r0 * p.xs_stride, *db = xs + (size_t)(r0 + 1) * p.xs_stride;
            const int cpt = p.x_vec4 ? (cells + (int)blockDim.x - 1) / (int)blockDim.x : 99;
            if (r0 > 0) __syncthreads();  // the reduction scratch of the previous pair is no longer read
            if (cpt == 1)
                quantise_rows2_regs<1>(ra, rb_, i0 < lim, have1 && i1 < lim, have1, p.k, da, db, cells, s_sx + r0, s_sum + r0, red_f, red_i);
            else if (cpt == 2)
                quantise_rows2_regs<2>(ra, rb_, i0 < lim, have1 && i1 < lim, have1, p.k, da, db, cells, s_sx + r0, s_sum + r0, red_f, red_i);
            else
                quantise_rows2(ra, rb_, i0 < lim, have1 && i1 < lim, have1, p.k, p.x_vec4 != 0, da, db, cells, s_sx + r0, s_sum + r0,
                               red_f, red_i);
        }
    } else {
        const int lim = GROUPED ? p.count : p.n;
        // eight 16-byte loads in flight per thread before the first store (a load-then-store loop pays one L2 round trip
        // per iteration; asynchronous copies cannot be used here: their completion is tracked per thread in issue order,
        // so waiting for them would also wait for every weight stage this thread has in flight)
        constexpr int U = 8;
        const int total = p.x_rows * cells;
        for (int base = threadIdx.x; base < total; base += U * (int)blockDim.x) {
            uint4 v[U];
            int dst[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * (int)blockDim.x;
                v[u] = make_uint4(0, 0, 0, 0);
                dst[u] = -1;
                if (idx < total) {
                    const int r = idx / cells, c = idx - r * cells;
                    const int src_row = GROUPED ? layer0 + r : r;
                    const int o = c * 16;
                    dst[u] = r * p.xs_stride + xs_offset(o);
                    if (src_row < lim && o < p.kp) v[u] = *reinterpret_cast<const uint4 *>(p.xq + (size_t)src_row * p.ldq + o);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (dst[u] >= 0) *reinterpret_cast<uint4 *>(xs + dst[u]) = v[u];
        }
        if ((int)threadIdx.x < p.x_rows) {
            const int src_row = GROUPED ? layer0 + threadIdx.x : threadIdx.x;
            s_sx[threadIdx.x] = src_row < lim ? p.sx[src_row] : 1.0f;
            s_sum[threadIdx.x] = src_row < lim ? p.sumq[src_row] : 0;
        }
    }
    __syncthreads();

    // ---- consumer ----
    constexpr int NACC = DP ? 8 * NT * 4 : NB * 16;
    int acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0;

    Cursor cc;
    first_unit(cc);
    // epilogue constants of the rows this lane finishes (MMA: rows g and g + 8; dp4a: row h + 2 * ((lane >> 1) & 7)),
    // fetched when the unit starts
    const LayerRef *ref_tab = p.table;
    LayerRef ref = p.one;
    int ref_layer = GROUPED ? -1 : 0;
    float sw0 = 0.f, sw1 = 0.f, bi0 = 0.f, bi1 = 0.f;
    bool has_bias = false;
    const int my_row = DP ? (lane >> 4) + 2 * ((lane >> 1) & 7) : g;
    auto fetch_consts = [&](const Cursor &u) {
        if (!u.valid) return;
        if (GROUPED && u.layer != ref_layer) { ref_layer = u.layer; ref = ref_tab[ref_layer]; }
        const int row = u.rb * 16 + my_row;  // rows up to m_alloc - 1 are allocated
        sw0 = ref.sw[row];
        if (!DP) sw1 = ref.sw[row + 8];
        has_bias = ref.bias != nullptr;
        if (has_bias) {
            bi0 = ref.bias[row];
            if (!DP) bi1 = ref.bias[row + 8];
        }
    };
    fetch_consts(cc);

    uint32_t cons = 0, cs = 0, cph = 0;  // stages consumed, the next one's index and barrier phase
    int parity = 0;
    bool ok = true;
    while (cc.valid) {
        const uint32_t s = cs, ph = cph;
        if (ok && !(ok = wait_stage(bar0 + 8 * s, ph))) pc.valid = false;  // gave up: no more copies, no more waits
        if (ok) {
            const int off = cc.c * CH;
            if constexpr (DP) {
                // cell c of rows h, h + 2, ...: stale bytes beyond the row's end meet zero activation codes
                const int c = lane & 15;
                const uint32_t xcol = (uint32_t)(off * 4) + 256 * (c >> 2) + 16 * (c & 3);
                uint32_t xr[NT][16];
#pragma unroll
                for (int tk = 0; tk < NT; ++tk) {
                    const int xrow = GROUPED ? cc.layer - layer0 : min(tk, p.x_rows - 1);
                    const uint32_t xb = xs_addr + (uint32_t)(xrow * p.xs_stride) + xcol;
                    const uint4 v0 = lds128<0>(xb), v1 = lds128<64>(xb), v2 = lds128<128>(xb), v3 = lds128<192>(xb);
                    xr[tk][0] = v0.x; xr[tk][1] = v0.y; xr[tk][2] = v0.z; xr[tk][3] = v0.w;
                    xr[tk][4] = v1.x; xr[tk][5] = v1.y; xr[tk][6] = v1.z; xr[tk][7] = v1.w;
                    xr[tk][8] = v2.x; xr[tk][9] = v2.y; xr[tk][10] = v2.z; xr[tk][11] = v2.w;
                    xr[tk][12] = v3.x; xr[tk][13] = v3.y; xr[tk][14] = v3.z; xr[tk][15] = v3.w;
                }
                const uint32_t wb = lane_dst + s * STAGE_BYTES;  // this lane's copy cell is also its first read cell
                uint4 wrow[8];
                wrow[0] = lds128<0 * 2 * RS>(wb); wrow[1] = lds128<1 * 2 * RS>(wb); wrow[2] = lds128<2 * 2 * RS>(wb);
                wrow[3] = lds128<3 * 2 * RS>(wb); wrow[4] = lds128<4 * 2 * RS>(wb); wrow[5] = lds128<5 * 2 * RS>(wb);
                wrow[6] = lds128<6 * 2 * RS>(wb); wrow[7] = lds128<7 * 2 * RS>(wb);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 w4 = wrow[i];
                    const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
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
            } else {
                const int bytes = min(CH, (int)p.row_bytes - off);
                const int ni = (bytes + 63) >> 6;
                const uint32_t sg = stage0 + s * STAGE_BYTES + g * RS + t * 16, sh = sg + 8 * RS;
                // byte offset of this lane's activation cells inside a staged row; the row is token 8 nb + g's
                // (columns of absent tokens repeat the last staged row: never stored)
                const uint32_t xcol = (uint32_t)(off * 4) + t * 16;
#pragma unroll
                for (int i = 0; i < CH / 64; ++i) {
                    if (i < ni) {
                        const uint4 wa = lds128<0>(sg + 64 * i), wb = lds128<0>(sh + 64 * i);
                        const uint32_t a[4] = {wa.x, wa.y, wa.z, wa.w}, b[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const int xrow = min(nb * 8 + g, p.x_rows - 1);
                            const uint32_t xb = xs_addr + (uint32_t)(xrow * p.xs_stride) + xcol + 256 * i;
                            uint4 xv[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) xv[u] = lds128<0>(xb + 64 * u);
#pragma unroll
                            for (int pp = 0; pp < 2; ++pp) {
                                const uint4 x0 = xv[2 * pp], x1 = xv[2 * pp + 1];
                                const uint32_t xb0[4] = {x0.x, x0.y, x0.z, x0.w}, xb1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t mk = 0x03030303u << (2 * j);
                                    mma_u8s8(*reinterpret_cast<int(*)[4]>(&acc[(nb * 4 + j) * 4]), a[2 * pp] & mk, b[2 * pp] & mk,
                                             a[2 * pp + 1] & mk, b[2 * pp + 1] & mk, xb0[j], xb1[j]);
                                }
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();  // every lane has read the stage: it can be refilled
        fill();
        if (ok) {
            ++cons;
            if (++cs == (uint32_t)nst) { cs = 0; cph ^= 1u; }
        }
        if (++cc.c == cc.c_end) {
            // ---- unit finished: combine the four scaled accumulators (exact), reduce, K-split partials, epilogue ----
            int v[NV];
            if constexpr (DP) {
                // s[i] = this lane's share of row h + 2 i; the 16 lanes of a half-warp hold the 16 cells of a row.
                // Transposing reduction: at each step a lane keeps half of its values and receives the partner's
                // share of them, so 8 values need 4 + 2 + 1 + 1 shuffles; the lane ends with row h + 2 ((lane >> 1) & 7)
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
                    for (int j = 0; j < 4; ++j)
                        a4[j] = (h8 ? sres[4 + j] : sres[j]) + __shfl_xor_sync(0xffffffffu, h8 ? sres[j] : sres[4 + j], 8);
                    int b2[2];
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        b2[j] = (h4 ? a4[2 + j] : a4[j]) + __shfl_xor_sync(0xffffffffu, h4 ? a4[j] : a4[2 + j], 4);
                    int d = (h2 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, h2 ? b2[0] : b2[1], 2);
                    d += __shfl_xor_sync(0xffffffffu, d, 1);
                    v[tk] = d;
                }
            } else {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int b = nb * 16 + r;
                        v[nb * 4 + r] = acc[b] + (acc[b + 4] >> 2) + (acc[b + 8] >> 4) + (acc[b + 12] >> 6);
                        acc[b] = acc[b + 4] = acc[b + 8] = acc[b + 12] = 0;
                    }
            }
            bool finisher = true;
            if (!GROUPED && ks > 1) {
                int *mine = part + (size_t)((gi * 2 + parity) * ks + slice) * (NV * 32);
#pragma unroll
                for (int i = 0; i < NV; ++i) mine[i * 32 + lane] = v[i];
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(ks * 32) : "memory");
                finisher = slice == 0;
                if (finisher) {
                    const int *base = part + (size_t)((gi * 2 + parity) * ks) * (NV * 32);
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        int sum = 0;
                        for (int q = 0; q < ks; ++q) sum += base[q * (NV * 32) + i * 32 + lane];
                        v[i] = sum;
                    }
                }
                parity ^= 1;
            }
            if (finisher) {
                auto store = [&](int value, int row, int tok, int xr_, float sw_, float bi_) {
                    const int a = p.mul * value - p.off * s_sum[xr_];
                    const size_t o = (size_t)tok * p.ldy + row;
                    if (p.acc) p.acc[o] = a;
                    if (p.y) {
                        float out = dequant_out(a, sw_, s_sx[xr_], bi_, has_bias);
                        if (p.resid) out = __fadd_rn(out, p.resid[o]);
                        if (p.relu) out = fmaxf(out, 0.0f);
                        if (p.y_flagged) {  // (value, epoch) pairs, locally and into the peers' buffers over NVLink
                            st_pair(p.y, o, out, y_epoch);
                            for (int q = 0; q < p.n_more; ++q) st_pair(p.y_more[q], o, out, y_epoch);
                        } else {
                            p.y[o] = out;
                            for (int q = 0; q < p.n_more; ++q) p.y_more[q][o] = out;  // peer copies over NVLink
                        }
                    }
                };
                if constexpr (DP) {
                    const int row = cc.rb * 16 + my_row;
                    if ((lane & 1) == 0 && row < p.m) {
#pragma unroll
                        for (int tk = 0; tk < NT; ++tk) {
                            const int tok = GROUPED ? cc.layer : tk;
                            const int xr_ = GROUPED ? cc.layer - layer0 : tk;
                            if (GROUPED || tk < p.n) store(v[tk], row, tok, xr_, sw0, bi0);
                        }
                    }
                } else {
                    // lane (g, t) holds rows g (r = 0, 1) and g + 8 (r = 2, 3) x tokens 8 nb + 2t (r even), + 1 (r odd)
                    const int row0 = cc.rb * 16 + g;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int row = row0 + (r >> 1) * 8;
                            const int tok = nb * 8 + 2 * t + (r & 1);
                            if (tok < p.n && row < p.m) store(v[nb * 4 + r], row, tok, tok, (r >> 1) ? sw1 : sw0, (r >> 1) ? bi1 : bi0);
                        }
                }
            }
            next_unit(cc);
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
    if (p.sync.world > 0) {
        // publish this rank's slice: every CTA orders its peer stores at system scope before it is counted; the
        // last CTA of the launch bumps the epoch and writes it into slot [rank] of every rank's flag array
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            const int ticket = atomicAdd(p.sync.done_counter, 1);
            if (ticket == (int)gridDim.x - 1) {
                __threadfence_system();  // cumulative: every counted CTA's stores are ordered before the flags
                *p.sync.done_counter = 0;
                const int epoch = *p.sync.epoch_counter + 1;
                for (int j = 0; j < p.sync.world; ++j) *reinterpret_cast<volatile int *>(p.sync.flag_arrays[j] + p.sync.rank) = epoch;
                __threadfence_system();
                *reinterpret_cast<volatile int *>(p.sync.epoch_counter) = epoch;
            }
        }
    } else if (p.n_more && !flagged) {
        __threadfence_system();
    }
}

size_t xs_stride_for(size_t kp) { return (kp + 1023) / 1024 * 1024 + 64; }

int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

// launch shape: warps per CTA and stages per warp that fit beside `x_rows` staged activation rows and the
// K-split scratch.  Prefers many warps (the arithmetic of a warp is serial; more warps overlap more of it with
// the copies) with at least two stages each.  warps == 0: does not fit.
struct Shape { int warps, nst; };
Shape pick_shape(size_t kp, int x_rows, size_t part_per_warp, int max_warps) {
    static const int env_w = env_int("KB_STREAM_WARPS", 0), env_nst = env_int("KB_STREAM_NST", 0);
    const size_t budget = 224 * 1024;  // leaves room for the static arrays
    const size_t fixed = BAR_BYTES + (size_t)x_rows * xs_stride_for(kp);
    int w = max_warps;
    if (env_w >= 4 && env_w <= max_warps) w = env_w;
    for (; w >= 4; w -= (w % 2 ? 1 : 2)) {  // even counts: 14 warps where 16 do not fit run 14 % faster than 12 (8 tokens of 8192 -> 28672)
        const size_t need2 = fixed + (size_t)w * (part_per_warp + 2 * STAGE_BYTES);
        if (need2 > budget) continue;
        size_t nst = (budget - fixed - (size_t)w * part_per_warp) / ((size_t)w * STAGE_BYTES);
        size_t cap = (env_nst >= 2 && env_nst <= NST_MAX) ? (size_t)env_nst : 4;
        return Shape{w, (int)(nst > cap ? cap : nst)};
    }
    return Shape{0, 0};
}

template <int NB, bool GROUPED, int NT, int W>
int launch_stream(const StreamParams &p, int device, int grid, int warps, size_t smem, cudaStream_t stream) {
    auto kern = gemv_stream_kernel<NB, GROUPED, NT, W>;
    if (int rc = set_dyn_smem_once(reinterpret_cast<const void *>(kern), device, 227 * 1024 - 2048, "stream smem attribute")) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)(warps * 32), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool pdl = env_int("KB_GEMV_PDL", 1) != 0;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "stream launch");
}

// two tokens: the dp4a form (NT = 2) for layers of up to 16 MB, where the launch is latency-bound; above, its
// doubled dp4a work no longer hides behind the copies and the MMA form is faster (17.1 against 24.7 us for
// 8192 -> 28672, 5.9 against 6.3 us for its eighth)
bool two_tokens_dp4a(const Linear *lin) { return lin->m_alloc * lin->row_bytes <= ((size_t)16 << 20); }
// the instance that serves n tokens: 1 / 2 = dp4a form for that many tokens, 0 = MMA form
int dp4a_tokens(const Linear *lin, size_t n) { return n == 1 ? 1 : (n == 2 && two_tokens_dp4a(lin) ? 2 : 0); }
// values a lane parks in shared memory per unit when K is split
int nv_for(const Linear *lin, size_t n) { return dp4a_tokens(lin, n) ? (int)n : (n <= 8 ? 4 : (n <= 16 ? 8 : 16)); }
// most warps per CTA of that instance (register bound)
int max_warps_for(const Linear *lin, size_t n) { return dp4a_tokens(lin, n) == 2 ? 12 : (n <= 8 ? 16 : (n <= 16 ? 12 : 8)); }

struct SinglePlan { int ks, warps, nst; size_t part_bytes; };
// launch shape of a single layer (warps == 0: does not fit)
SinglePlan plan_single(const Linear *lin, size_t n) {
    const int nchunks = (int)((lin->row_bytes + CH - 1) / CH);
    const int row_blocks = (int)((lin->m + 15) / 16);
    const int sms = sm_count(lin->device);
    static const int env_ks = env_int("KB_STREAM_KS", 0);
    const int maxw = max_warps_for(lin, n);
    // K split: enough (row block, slice) units to give every warp of every SM one
    int ks = 1;
    while (ks < 16 && ks * 2 <= nchunks && ks * 2 <= maxw && (long long)row_blocks * ks < (long long)sms * maxw) ks *= 2;
    if ((env_ks == 1 || env_ks == 2 || env_ks == 4 || env_ks == 8 || env_ks == 16) && env_ks <= nchunks && env_ks <= maxw) ks = env_ks;
    // a layer of a few tens of KB per SM is over before a second launch could start behind it: take half an SM's
    // shared memory (8 warps x 2 stages), so that the next launch of a chain is resident early (programmatic
    // dependent launch) and streams its first weights while this one finishes
    const bool small = lin->m_alloc * lin->row_bytes / (size_t)sms < ((size_t)64 << 10);
    for (;; ks /= 2) {  // a smaller K split needs less scratch
        const size_t part_per_warp = ks > 1 ? (size_t)2 * nv_for(lin, n) * 32 * 4 : 0;
        Shape sh = pick_shape(lin->kp, (int)n, part_per_warp, maxw);
        if (small && sh.warps > 8 && (size_t)n * xs_stride_for(lin->kp) <= ((size_t)24 << 10)) { sh.warps = 8; sh.nst = 2; }
        while (sh.warps > 0 && sh.warps % ks) sh.warps -= 2;  // whole groups of ks warps
        if (sh.warps >= ks && sh.warps > 0 && sh.nst >= 2) return SinglePlan{ks, sh.warps, sh.nst, (size_t)sh.warps * part_per_warp};
        if (ks == 1) return SinglePlan{1, 0, 0, 0};
    }
}

}  // namespace

bool gemv_stream_supports(const Linear *lin, size_t n) {
    if (n < 1 || n > 32 || lin->kp > 80000) return false;  // 64 * 3 * 127 * K must stay below 2^31
    return plan_single(lin, n).warps > 0;
}

int launch_gemv_stream(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!gemv_stream_supports(L, a.n))
        return fail(KB_ERR_UNSUPPORTED, "streaming kernel: %zu tokens x K=%zu do not fit in shared memory", a.n, L->k);
    if ((a.x || a.xf) && a.n > 8) return fail(KB_ERR_UNSUPPORTED, "streaming kernel: the fused quantiser takes up to 8 tokens");
    const bool flagged = a.xf || a.y_flagged;
    if (flagged) {
        if (!a.flag_round || a.flag_seq < 1 || a.flag_seq > 255 || (a.xf && a.flag_seq < 2))
            return fail(KB_ERR_INVALID, "streaming kernel: flagged words need the round word and a chain position in 1..255 "
                                        "(2.. for flagged activations)");
        if (a.y_flagged && (!a.y || a.acc || (reinterpret_cast<uintptr_t>(a.y) & 7)))
            return fail(KB_ERR_INVALID, "streaming kernel: flagged outputs need an 8-byte aligned y and no accumulator output");
        if (a.xf && ((L->k % 4) || (a.ldxf % 2) || a.ldxf < L->k || (reinterpret_cast<uintptr_t>(a.xf) & 15)))
            return fail(KB_ERR_UNSUPPORTED, "streaming kernel: flagged activations need K %% 4 == 0, 16-byte aligned rows, ld >= K");
    }
    if (!a.x && !a.xf) {
        if (!a.xq || !a.sx || !a.sumq) return fail(KB_ERR_INVALID, "streaming kernel: needs activations");
        if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
            return fail(KB_ERR_INVALID, "gemv: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    }
    const SinglePlan plan = plan_single(L, a.n);
    StreamParams p = {};
    p.table = nullptr;
    p.one = LayerRef{L->w2, L->scales, L->bias};
    p.count = 1;
    p.m = (int)L->m; p.k = (int)L->k; p.kp = (int)L->kp;
    p.row_bytes = L->row_bytes;
    p.row_blocks = (int)((L->m + 15) / 16);
    p.nchunks = (int)((L->row_bytes + CH - 1) / CH);
    p.ks = plan.ks;
    p.x_rows = (int)a.n;
    p.xs_stride = (int)xs_stride_for(L->kp);
    p.nst = plan.nst;
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
    p.sync = PeerSync{};
    if (a.sync && a.y) p.sync = *a.sync;
    p.xf = reinterpret_cast<const uint2 *>(a.xf);
    p.ldxf = a.ldxf;
    p.y_flagged = a.y_flagged ? 1 : 0;
    p.flag_round = a.flag_round;
    p.flag_seq = a.flag_seq;
    if (flagged) p.sync = PeerSync{};  // the pairs replace the flag arrays: no fence-and-flag wait or publication
    const int gp = plan.warps / plan.ks;
    int grid = (p.row_blocks + gp - 1) / gp;
    const int sms = sm_count(L->device);
    if (grid > sms) grid = sms;
    const size_t smem = BAR_BYTES + (size_t)plan.warps * p.nst * STAGE_BYTES + (size_t)p.x_rows * p.xs_stride + plan.part_bytes;
    if (a.n == 1) return launch_stream<1, false, 1, 16>(p, L->device, grid, plan.warps, smem, stream);
    if (a.n == 2 && two_tokens_dp4a(L)) return launch_stream<1, false, 2, 12>(p, L->device, grid, plan.warps, smem, stream);
    if (a.n <= 8) return launch_stream<1, false, 0, 16>(p, L->device, grid, plan.warps, smem, stream);
    if (a.n <= 16) return launch_stream<2, false, 0, 12>(p, L->device, grid, plan.warps, smem, stream);
    return launch_stream<4, false, 0, 8>(p, L->device, grid, plan.warps, smem, stream);
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
    Shape sh = {0, 0};
    for (;;) {
        per_cta = (total + grid - 1) / grid;
        staged = (per_cta + p.row_blocks - 2) / p.row_blocks + 1;  // layers a range of per_cta row blocks can touch
        if (staged > (long long)a.count) staged = (long long)a.count;
        // 12 warps x 3 stages measured 4 % faster under sustained load than 16 x 2 (and than 10, 11, 13, 14 warps)
        sh = staged <= MAX_ROWS ? pick_shape(a.kp, (int)staged, 0, 12) : Shape{0, 0};
        if ((sh.warps > 0 && sh.nst >= 2) || per_cta <= 12) break;
        grid *= 2;
    }
    if (sh.warps == 0 || sh.nst < 2)
        return fail(KB_ERR_UNSUPPORTED, "group: %lld activation rows of %zu bytes per CTA do not fit in shared memory", staged,
                    xs_stride_for(a.kp));
    grid = (total + per_cta - 1) / per_cta;
    p.nst = sh.nst;
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
    p.sync = PeerSync{};
    const size_t smem = BAR_BYTES + (size_t)sh.warps * p.nst * STAGE_BYTES + (size_t)p.x_rows * p.xs_stride;
    return launch_stream<1, true, 1, 12>(p, a.device, (int)grid, sh.warps, smem, stream);
}

}  // namespace kb
