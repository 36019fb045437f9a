// Medium-batch GEMM (33..128 tokens) on tcgen05 with the weight operand in tensor memory (sm_100a).
//
// With up to 128 tokens the work is still dominated by streaming and unpacking the weights, so
// the tile is 128 weight rows x BN tokens (BN = 64 or 128) per CTA, one CTA per SM, and the
// pipeline is built around the unpack:
//   * a pipeline stage is two "slabs" of 128 bytes of K.  Warp 0 TMA-loads the stage's int8
//     activations (2 x BN x 128 B, 128-byte swizzle) into a ring of shared-memory stages; warp 3
//     TMA-loads the packed weights of the tile's 128 rows as 128-byte-wide swizzled tiles (16 KB =
//     four slabs = two stages) into a ring of their own — the wide tile is one copy instead of four;
//   * warps 4-11 unpack: two groups of four warps take the two slabs of a stage; a thread owns one
//     row, turns its 32 packed bytes of the slab into 32 words of four u8 codes and writes them with
//     one tcgen05.st into its own lane of tensor memory (lane = weight row, column = 4 codes along
//     K).  The unpacked weights never touch shared memory;
//   * warp 1 issues tcgen05.mma.cta_group::1.kind::i8 with A from tensor memory and B from
//     shared memory, accumulating 128 x BN int32 in tensor memory; one tcgen05.commit per stage
//     releases the stage's activations and its weight slots together;
//   * warps 12-15 run the epilogue of tile i (tcgen05.ld, integer correction, dequantisation,
//     residual, stores coalesced along the output features) while the main loop of tile i+1 fills
//     the second accumulator.
// Tensor memory (512 columns): two BN-column accumulators and (512 - 2 BN) / 64 stages of weight
// slots — 6 stages at BN = 64, 4 at BN = 128; stage s of shared memory and stage s of tensor memory
// are filled and freed together, so the MMA thread waits on one barrier and commits once per eight
// MMAs.  Layers of few row tiles split K over CTAs (work item = (tile, split); the splits' raw int32 sums meet in a
// scratch buffer and a second launch adds them and runs the epilogue).  All barriers are local to the CTA.  Every wait is bounded; a wait that gives up records a
// code in the status word and raises the CTA's abort flag, and the CTA drains its copies, frees its
// tensor memory and returns.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace kb {

namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 128;
constexpr int NUM_THREADS = 512;
// Packed weights arrive as 128-byte-wide, 128-byte-swizzled tiles of 128 rows (16 KB = four slabs).
constexpr int PKT_SLABS = 4;
constexpr int PKT_BYTES = BM * 128;
constexpr int PKS = 4;                   // packed tiles in flight
constexpr int SLAB_COLS = BK / 4;        // 32 columns of tensor memory per slab
constexpr int TMEM_COLS = 512;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr long long WAIT_CYCLES = 2000000000ll;

// A pipeline stage is two slabs: their activations in shared memory and their unpacked weights in
// tensor memory travel together, so the MMA thread pays one barrier wait and one tcgen05.commit per
// eight MMAs — with a stage per slab and separate rings that thread's waits and commits alone took
// longer than the MMAs they ordered.
constexpr int ST_SLABS = 2;

template <int BN>
struct Cfg {
    static constexpr int ACT_SLAB = BN * BK;
    static constexpr int STAGE_BYTES = ST_SLABS * ACT_SLAB;
    static constexpr int A_COL0 = 2 * BN;                                             // after the two accumulators
    static constexpr int NS = (TMEM_COLS - A_COL0) / (ST_SLABS * SLAB_COLS);          // stages: 6 at BN = 64, 4 at 128
    static constexpr int NUM_BARS = 2 * NS + 2 * PKS + 5;
    static constexpr int SMEM_BYTES = 1024 + NS * STAGE_BYTES + PKS * PKT_BYTES + 8 * NUM_BARS + 16;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct TcsParams {
    int m, n, kp;
    const float *sw, *bias, *sx;
    const int32_t *sumq;
    float *y;
    int32_t *acc;
    size_t ldy;
    int mul, off;
    int *status;
    float *y_more[MAX_PEERS - 1];
    int n_more;
    const float *resid;
    int relu;  // max(y, 0) after the bias
    // K split over CTAs (layers of few row tiles): work item = (tile, split), a split covers `split_slabs` slabs of K
    // (a multiple of PKT_SLABS) and stores its raw int32 sums to part[split][n][m]; a second kernel adds them up
    int splits, split_slabs;
    int32_t *part;
    // flagged words (see FwdArgs): y and y_more are buffers of (value, epoch) pairs, epoch = (*flag_round << 8) | flag_seq
    int y_flagged;
    const int *flag_round;
    int flag_seq;
};

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    long long t0 = 0;
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcs_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const TcsParams p) {
    using C = Cfg<BN>;
    constexpr int NS = C::NS;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_dyn + (base - smem_u32(smem_dyn));

    auto act_addr = [&](int s, int j) { return base + (uint32_t)s * C::STAGE_BYTES + (uint32_t)j * C::ACT_SLAB; };
    auto pkt_addr = [&](int q) { return base + (uint32_t)(NS * C::STAGE_BYTES) + (uint32_t)q * PKT_BYTES; };
    const uint32_t tail = base + NS * C::STAGE_BYTES + PKS * PKT_BYTES;
    // full: the stage's activations landed (1 arrival with the byte count) and its weight codes are
    // in tensor memory (8 unpack warps); empty: the stage's MMAs completed (tcgen05.commit)
    auto full = [&](int s) { return tail + 8u * s; };
    auto empty = [&](int s) { return tail + 8u * (NS + s); };
    auto pk_full = [&](int q) { return tail + 8u * (2 * NS + q); };         // the packed tile landed
    auto pk_empty = [&](int q) { return tail + 8u * (2 * NS + PKS + q); };  // every unpack warp is done with it
    auto tfull = [&](int b) { return tail + 8u * (2 * NS + 2 * PKS + b); };
    auto tempty = [&](int b) { return tail + 8u * (2 * NS + 2 * PKS + 2 + b); };
    const uint32_t drain_bar = tail + 8u * (2 * NS + 2 * PKS + 4);
    uint8_t *tail_ptr = base_ptr + NS * C::STAGE_BYTES + PKS * PKT_BYTES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail_ptr + 8 * C::NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb_all = p.kp / BK;
    const int tiles_n = (p.n + BN - 1) / BN;
    const int tiles_m = (p.m + BM - 1) / BM;
    const int num_tiles = tiles_m * tiles_n;
    const int num_work = num_tiles * p.splits;  // work item w = tile * splits + split
    // slabs, stages and packed tiles of split sp (the last split may be shorter; every role derives the same numbers)
    auto slabs_of = [&](int sp) { return min(p.split_slabs, num_kb_all - sp * p.split_slabs); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full(s), 9);
            mbar_init(empty(s), 1);
        }
        for (int q = 0; q < PKS; ++q) {
            mbar_init(pk_full(q), 1);
            mbar_init(pk_empty(q), 8);  // one arrival per unpack warp
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull(b), 1);
            mbar_init(tempty(b), 4);   // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == 3) {
        // ---------------- TMA producers: warp 0 the activations, warp 3 the packed weights ----------------
        // (one thread issues a tensor copy every couple of hundred nanoseconds; two issue in parallel)
        if (lane == 0 && warp == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
                const int tile = w / p.splits, sp = w - tile * p.splits;
                const int n0 = (tile % tiles_n) * BN;
                const int num_kb = slabs_of(sp), slab0 = sp * p.split_slabs;
                const int num_st = (num_kb + ST_SLABS - 1) / ST_SLABS;
                for (int st = 0; st < num_st; ++st, ++it) {
                    const int s = it % NS;
                    if (!(ok = wait_bar(empty(s), ((it / NS) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_TMA_EMPTY))) break;
                    const int nsl = min(ST_SLABS, num_kb - st * ST_SLABS);
                    mbar_expect_tx(full(s), (uint32_t)(nsl * C::ACT_SLAB));
                    for (int j = 0; j < nsl; ++j) tma_load_2d(act_addr(s, j), &tmap_x, full(s), (slab0 + st * ST_SLABS + j) * BK, n0);
                }
            }
            // every copy this thread issued must have landed before the CTA exits
            const uint32_t issued = it;
            for (uint32_t j = (issued > (uint32_t)NS ? issued - NS : 0); j < issued; ++j) {
                bool landed = false;
                for (uint32_t i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(full(j % NS), (j / NS) & 1u);
                if (!landed) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
            }
        } else if (lane == 0) {
            uint32_t pt = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
                const int tile = w / p.splits, sp = w - tile * p.splits;
                const int m0 = (tile / tiles_n) * BM;
                const int num_pkt = (slabs_of(sp) + PKT_SLABS - 1) / PKT_SLABS, pkt0 = sp * p.split_slabs / PKT_SLABS;
                for (int k = 0; k < num_pkt; ++k, ++pt) {
                    const int q = pt % PKS;
                    if (!(ok = wait_bar(pk_empty(q), ((pt / PKS) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_TMA_EMPTY))) break;
                    mbar_expect_tx(pk_full(q), PKT_BYTES);  // columns past the row's end arrive as zeros and count
                    tma_load_2d(pkt_addr(q), &tmap_w, pk_full(q), (pkt0 + k) * 128, m0);
                }
            }
            const uint32_t issued = pt;
            for (uint32_t j = (issued > (uint32_t)PKS ? issued - PKS : 0); j < issued; ++j) {
                bool landed = false;
                for (uint32_t i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(pk_full(j % PKS), (j / PKS) & 1u);
                if (!landed) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D = s32, A (weight codes) = u8 from tensor memory, B (activations) = s8 K-major, M = 128, N = BN
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++ti) {
                const int b = ti & 1;
                const int num_kb = slabs_of(w % p.splits);
                const int num_st = (num_kb + ST_SLABS - 1) / ST_SLABS;
                if (!(ok = wait_bar(tempty(b), ((ti >> 1) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM_EMPTY))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                for (int st = 0; st < num_st; ++st, ++it) {
                    const int s = it % NS;
                    if (!(ok = wait_bar(full(s), (it / NS) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL))) break;
                    tc_fence_after();
                    const int nsl = min(ST_SLABS, num_kb - st * ST_SLABS);
                    for (int j = 0; j < nsl; ++j) {
                        const uint32_t a_tmem = tmem_base + (uint32_t)(C::A_COL0 + (s * ST_SLABS + j) * SLAB_COLS);
                        const uint64_t bdesc = umma_desc_sw128(act_addr(s, j));
#pragma unroll
                        for (int k4 = 0; k4 < BK / 32; ++k4)  // 32 bytes of K = 8 columns of A, 32 bytes of a B row
                            umma_i8_ta(tmem_d, a_tmem + (uint32_t)(k4 * 8), bdesc + (uint64_t)(k4 * 2), idesc, (st | j | k4) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty(s));  // frees the stage's activations and its weight slots
                }
                if (ok) umma_commit(tfull(b));
            }
            // all MMAs issued by this thread must retire before shared and tensor memory are released
            umma_commit(drain_bar);
            bool done = false;
            for (uint32_t i = 0; i < WAIT_LIMIT && !done; ++i) done = mbar_try_wait(drain_bar, 0);
            if (!done) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
        }
    } else if (warp >= 4 && warp < 12) {
        // ---------------- unpack: packed 2-bit -> code bytes in tensor memory ----------------
        // group 0 (warps 4-7) takes the even slabs, group 1 (warps 8-11) the odd ones; thread = row;
        // warp w writes the lane quarter w % 4, which is the row quarter it unpacks
        const int grp = (warp - 4) >> 2;
        const int r = (threadIdx.x - 128) & 127;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t swz = (uint32_t)(r & 7);
        uint32_t it = 0, pt = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
            const int num_kb = slabs_of(w % p.splits);
            const int num_st = (num_kb + ST_SLABS - 1) / ST_SLABS;
            for (int st = 0; st < num_st; ++st, ++it) {
                const int s = it % NS, q = pt % PKS;
                // a packed tile covers two stages; every unpack warp waits for it, also one that owns
                // none of its slabs: its arrival below must belong to this use of the barrier
                if ((st & 1) == 0 && !(ok = wait_bar(pk_full(q), (pt / PKS) & 1u, abort_flag, p.status, DEV_TIMEOUT_UNPACK_FULL))) break;
                const bool work = st * ST_SLABS + grp < num_kb;
                const int j = (st & 1) * ST_SLABS + grp;  // the slab's place in the packed tile
                uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
                if (work) {
                    const uint8_t *row = base_ptr + (pkt_addr(q) - base) + r * 128;
                    lo = *reinterpret_cast<const uint4 *>(row + (((uint32_t)(2 * j) ^ swz) << 4));
                    hi = *reinterpret_cast<const uint4 *>(row + (((uint32_t)(2 * j + 1) ^ swz) << 4));
                }
                // the weight slots are free once the MMAs of the stage's previous use have completed
                if (!(ok = wait_bar(empty(s), ((it / NS) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_UNPACK_FULL))) break;
                tc_fence_after();
                if (work) {
                    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    uint32_t codes[32];  // word 4c+j = codes of elements 16c+4j .. 16c+4j+3
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        codes[4 * c + 0] = w[c] & 0x03030303u;
                        codes[4 * c + 1] = (w[c] >> 2) & 0x03030303u;
                        codes[4 * c + 2] = (w[c] >> 4) & 0x03030303u;
                        codes[4 * c + 3] = (w[c] >> 6) & 0x03030303u;
                    }
                    tmem_st32(tmem_base + lane_base + (uint32_t)(C::A_COL0 + (s * ST_SLABS + grp) * SLAB_COLS), codes);
                    tmem_wait_st();
                    tc_fence_before();
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full(s));
                    if ((st & 1) || st == num_st - 1) mbar_arrive(pk_empty(q));  // all lanes have read their rows
                }
                if ((st & 1) || st == num_st - 1) ++pt;
            }
        }
    } else if (warp >= 12) {
        // ---------------- epilogue ----------------
        // Lane l of warp e owns output feature m0 + 32e + l (one lane of tensor memory); a chunk is
        // 32 token columns whose scale and code sum sit one per lane and are broadcast by shuffles.
        const int e = warp - 12;
        constexpr int NCH = BN / 32;
        const bool has_bias = p.bias != nullptr;
        const uint32_t epoch = p.y_flagged ? (((uint32_t)(*reinterpret_cast<const volatile int *>(p.flag_round)) << 8) | (uint32_t)p.flag_seq) : 0u;
        uint32_t ti = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++ti) {
            const int b = ti & 1;
            const int tile = w / p.splits, sp = w - tile * p.splits;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            const int row = m0 + e * 32 + lane;
            const bool row_ok = row < p.m;
            if (p.splits > 1) {
                // K split: this item's raw sums go to its slice of the partial buffer ([split][token][row], rows
                // contiguous: a warp stores 128 bytes per token)
                ok = wait_bar(tfull(b), (ti >> 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_EPI_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                int32_t *prow = p.part + ((size_t)sp * p.n + n0) * p.m + row;
#pragma unroll 1
                for (int c = 0; c < NCH; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + (uint32_t)(b * BN + c * 32) + ((uint32_t)(e * 32) << 16), v);
                    if (c == NCH - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty(b));
                    }
                    const int valid = p.n - (n0 + c * 32);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) prow[(size_t)(c * 32 + i) * p.m] = (int)v[i];
                    }
                }
                continue;
            }
            const float sw = row_ok ? p.sw[row] : 0.0f;
            const float bias = (row_ok && has_bias) ? p.bias[row] : 0.0f;
            const size_t yoff = (size_t)n0 * p.ldy + row;
            float *yrow = p.y ? p.y + yoff : nullptr;
            int32_t *arow = p.acc ? p.acc + yoff : nullptr;
            ok = wait_bar(tfull(b), (ti >> 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_EPI_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < NCH; ++c) {
                const int tok_l = n0 + 32 * c + lane;
                const float sx_cur = tok_l < p.n ? __ldg(p.sx + tok_l) : 1.0f;
                const int sm_cur = tok_l < p.n ? __ldg(p.sumq + tok_l) : 0;
                uint32_t v[32];
                tmem_ld32(tmem_base + (uint32_t)(b * BN + c * 32) + ((uint32_t)(e * 32) << 16), v);
                if (c == NCH - 1) {  // the whole accumulator has been read: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty(b));
                }
                const int valid = p.n - (n0 + c * 32);
                const size_t cbase = (size_t)(c * 32) * p.ldy;
                const bool add_resid = p.resid != nullptr && row_ok;
                float outv[32];
                if (add_resid) {
                    const float *rrow = p.resid + yoff + cbase;
#pragma unroll
                    for (int i = 0; i < 32; ++i) outv[i] = i < valid ? rrow[(size_t)i * p.ldy] : 0.0f;
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) outv[i] = 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float r_i = outv[i];
                    const float sx_i = __shfl_sync(0xffffffffu, sx_cur, i);
                    const int sm_i = __shfl_sync(0xffffffffu, sm_cur, i);
                    const int a = p.mul * (int)v[i] - p.off * sm_i;
                    outv[i] = dequant_out(a, sw, sx_i, bias, has_bias);
                    if (add_resid) outv[i] = __fadd_rn(outv[i], r_i);
                    if (p.relu) outv[i] = fmaxf(outv[i], 0.0f);
                    v[i] = (uint32_t)a;
                }
                if (row_ok) {
                    if (arow) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) arow[cbase + (size_t)i * p.ldy] = (int)v[i];
                    }
                    if (yrow && p.y_flagged) {  // (value, epoch) pairs, locally and into the peers' buffers
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) st_pair(p.y, yoff + cbase + (size_t)i * p.ldy, outv[i], epoch);
                        for (int q = 0; q < p.n_more; ++q) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < valid) st_pair(p.y_more[q], yoff + cbase + (size_t)i * p.ldy, outv[i], epoch);
                        }
                    } else if (yrow) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) yrow[cbase + (size_t)i * p.ldy] = outv[i];
                        for (int q = 0; q < p.n_more; ++q) {  // column-sharded layers: peer copies over NVLink
                            float *peer = p.y_more[q] + yoff + cbase;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < valid) peer[(size_t)i * p.ldy] = outv[i];
                        }
                    }
                }
            }
        }
        if (p.n_more && !p.y_flagged) __threadfence_system();  // once per launch: the peer copies are performed before the exit
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// Scratch of the K split: one buffer per (device, stream), created at the largest size a split launch can need
// (8 splits x 128 tokens x 74 row tiles of int32: 38.8 MB) and never moved or freed, so a captured graph that holds
// its address stays valid.  Launches on one stream use the buffer one after the other; other streams have their own,
// so concurrent forwards never share one.  (A stream-ordered allocation per launch costs more than the split saves
// on short layers and puts allocation nodes into captured graphs.)  A buffer cannot be created during stream capture
// (cudaMalloc is not capturable) and at most SPLIT_SCRATCH_MAX exist: otherwise the launch falls back to a
// stream-ordered allocation.
constexpr size_t SPLIT_SCRATCH_BYTES = (size_t)8 * 128 * 74 * 128 * sizeof(int32_t);
constexpr size_t SPLIT_SCRATCH_MAX = 64;
struct SplitScratch {
    struct Entry { int device; cudaStream_t stream; void *ptr; };
    std::mutex mu;
    std::vector<Entry> entries;
    void *get(int device, cudaStream_t stream, size_t bytes) {
        if (bytes > SPLIT_SCRATCH_BYTES) return nullptr;
        std::lock_guard<std::mutex> lock(mu);
        for (auto &e : entries)
            if (e.device == device && e.stream == stream) return e.ptr;
        if (entries.size() >= SPLIT_SCRATCH_MAX) return nullptr;
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) { cudaGetLastError(); return nullptr; }
        void *ptr = nullptr;
        if (cudaMalloc(&ptr, SPLIT_SCRATCH_BYTES) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        entries.push_back(Entry{device, stream, ptr});
        return ptr;
    }
};
SplitScratch g_split_scratch;

// second step of the K split: adds the splits' raw sums (int32, exact in any order) and runs the epilogue of the
// unsplit kernel on them; thread = one output, rows fastest
struct CombineParams {
    const int32_t *part;
    int splits, n, m;
    const float *sw, *bias, *sx;
    const int32_t *sumq;
    int mul, off;
    float *y;
    int32_t *acc;
    size_t ldy;
    const float *resid;
    int relu;
    float *y_more[MAX_PEERS - 1];
    int n_more;
    int y_flagged;
    const int *flag_round;
    int flag_seq;
};
__global__ void __launch_bounds__(256) splitk_combine_kernel(const CombineParams p) {
    const size_t total = (size_t)p.n * p.m;
    // a few CTAs per SM walk the outputs: the system-scope fence behind the peer stores is then paid once per
    // CTA at the end of the launch, not once per wave of short-lived CTAs
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int tok = (int)(idx / p.m), row = (int)(idx - (size_t)tok * p.m);
        int sum = 0;
        for (int sp = 0; sp < p.splits; ++sp) sum += p.part[(size_t)sp * total + idx];
        const int a = p.mul * sum - p.off * p.sumq[tok];
        const size_t o = (size_t)tok * p.ldy + row;
        if (p.acc) p.acc[o] = a;
        if (p.y) {
            const bool has_bias = p.bias != nullptr;
            float out = dequant_out(a, p.sw[row], p.sx[tok], has_bias ? p.bias[row] : 0.0f, has_bias);
            if (p.resid) out = __fadd_rn(out, p.resid[o]);
            if (p.relu) out = fmaxf(out, 0.0f);
            if (p.y_flagged) {
                const uint32_t epoch = ((uint32_t)(*reinterpret_cast<const volatile int *>(p.flag_round)) << 8) | (uint32_t)p.flag_seq;
                st_pair(p.y, o, out, epoch);
                for (int q = 0; q < p.n_more; ++q) st_pair(p.y_more[q], o, out, epoch);
            } else {
                p.y[o] = out;
                for (int q = 0; q < p.n_more; ++q) p.y_more[q][o] = out;  // column-sharded layers: peer copies over NVLink
            }
        }
    }
    if (p.n_more && !p.y_flagged) __threadfence_system();
}

template <int BN>
int launch_bn(const FwdArgs &a, cudaStream_t stream) {
    using C = Cfg<BN>;
    const Linear *L = a.lin;
    CUtensorMap tmap_x;
    int rc = encode_2d(&tmap_x, a.xq, L->kp, a.n, a.ldq, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    TcsParams p;
    p.m = (int)L->m; p.n = (int)a.n; p.kp = (int)L->kp;
    p.sw = L->scales; p.bias = L->bias; p.sx = a.sx; p.sumq = a.sumq;
    p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.n_more = a.y ? a.n_more : 0;
    for (int q = 0; q < MAX_PEERS - 1; ++q) p.y_more[q] = q < p.n_more ? a.y_more[q] : nullptr;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    p.mul = L->mul; p.off = L->off; p.status = L->dev_status;
    p.y_flagged = a.y_flagged ? 1 : 0; p.flag_round = a.flag_round; p.flag_seq = a.flag_seq;
    if (a.y_flagged && (!a.y || a.acc || a.resid || !a.flag_round || a.flag_seq < 1 || a.flag_seq > 255))
        return fail(KB_ERR_INVALID, "gemm: flagged outputs need y, the round word and a chain position, and take no accumulator or residual");
    auto kern = gemm_tcs_kernel<BN>;
    const int dev = L->device;
    if (int rc_attr = set_dyn_smem_once(reinterpret_cast<const void *>(kern), dev, C::SMEM_BYTES, "gemm smem attribute")) return rc_attr;
    const int tiles = (int)(((L->m + BM - 1) / BM) * ((a.n + BN - 1) / BN));
    const int sms = sm_count(L->device);
    // A tile walks all of K on one SM, so a layer of few tiles leaves most SMs idle for the whole walk (25 tiles of
    // 3200 x 8640: 21.5 us whatever the token count).  Then K is split over CTAs: at least 8 slabs per split, splits
    // on packed-tile boundaries, raw sums through a scratch buffer (small: such layers have few rows) and a second
    // launch that adds them up.  The two launches and the scratch traffic cost about 4 us, so short rows (K < 6144)
    // and two-way splits of 128-token tiles stay unsplit (measured, 64 / 128 tokens: 8192 -> 3584 20.6 / 22.5 ->
    // 14.0 / 17.7 us, 8640 -> 3200 21.6 / 23.4 -> 14.3 / 18.2 us, 8192 -> 7168 21.1 / 22.8 -> 19.3 / 25.0 us,
    // 3200 -> 3200 11.7 / 13.4 -> 12.8 / 16.9 us).
    const int num_kb = (int)(L->kp / BK);
    static const int env_splits = []() { const char *e = getenv("KB_GEMM_SPLITS"); return e ? atoi(e) : 0; }();
    int splits = 1;
    if (tiles * 2 <= sms && num_kb >= 48 && !a.no_alloc) {
        splits = sms / tiles;
        if (splits > 8) splits = 8;
        if (splits > num_kb / 8) splits = num_kb / 8;
        if (splits < (BN > 64 ? 3 : 2)) splits = 1;
    }
    if (env_splits >= 1 && !a.no_alloc) splits = env_splits;
    if (splits < 1) splits = 1;
    int split_slabs = ((num_kb + splits - 1) / splits + PKT_SLABS - 1) / PKT_SLABS * PKT_SLABS;
    splits = (num_kb + split_slabs - 1) / split_slabs;
    p.splits = splits; p.split_slabs = splits > 1 ? split_slabs : num_kb; p.part = nullptr;
    bool part_async = false;
    if (splits > 1) {
        const size_t bytes = (size_t)splits * a.n * L->m * sizeof(int32_t);
        p.part = static_cast<int32_t *>(g_split_scratch.get(dev, stream, bytes));
        if (!p.part) {
            cudaError_t ea = cudaMallocAsync(reinterpret_cast<void **>(&p.part), bytes, stream);
            if (ea != cudaSuccess) return cuda_fail(ea, "split scratch allocation");
            part_async = true;
        }
    }
    const int work = tiles * splits;
    const int grid = work < sms ? work : sms;
    kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmap_x, L->tmap_w128, p);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && splits > 1) {
        CombineParams c;
        c.part = p.part; c.splits = splits; c.n = p.n; c.m = p.m;
        c.sw = p.sw; c.bias = p.bias; c.sx = p.sx; c.sumq = p.sumq; c.mul = p.mul; c.off = p.off;
        c.y = p.y; c.acc = p.acc; c.ldy = p.ldy; c.resid = p.resid; c.relu = p.relu;
        c.n_more = p.n_more;
        c.y_flagged = p.y_flagged; c.flag_round = p.flag_round; c.flag_seq = p.flag_seq;
        for (int q = 0; q < MAX_PEERS - 1; ++q) c.y_more[q] = p.y_more[q];
        const size_t total = (size_t)p.n * p.m;
        size_t blocks = (total + 255) / 256;
        if (blocks > (size_t)sms * 4) blocks = (size_t)sms * 4;
        splitk_combine_kernel<<<(unsigned)blocks, 256, 0, stream>>>(c);
        e = cudaGetLastError();
    }
    if (part_async) {
        cudaError_t ef = cudaFreeAsync(p.part, stream);
        if (e == cudaSuccess) e = ef;
    }
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "gemm launch");
}

}  // namespace

// up to 128 tokens: tile of 64 or 128 tokens, weights unpacked into tensor memory
int launch_gemm_tcs(const FwdArgs &a, cudaStream_t stream) { return a.n <= 64 ? launch_bn<64>(a, stream) : launch_bn<128>(a, stream); }

}  // namespace kb
