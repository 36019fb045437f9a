// Prefill GEMM, CTA-pair version (sm_100a): tcgen05.mma.cta_group::2, kind::i8.
//
// Two CTAs of a cluster (two SMs) share one 256-row x 256-token tile:
//   * each CTA TMA-loads and unpacks ITS 128 weight rows (A operand half) and TMA-loads HALF
//     of the activation tile (128 tokens, B operand half); the MMA, issued by the pair's
//     leader CTA only, reads A rows and B columns from both CTAs' shared memory and writes
//     each CTA's 128 x 256 int32 accumulator into that CTA's own TMEM;
//   * per k-block (128 bytes of K) a CTA therefore moves 16 KB of activations + 4 KB of
//     packed weights through TMA instead of 32 + 4 KB in the single-CTA kernel, which
//     shortens the copy pipeline's latency per unit of MMA time; a stage (activations and
//     unpacked weights) is released by one tcgen05.commit multicast to both CTAs;
//   * the packed weights do not ride in the stage: they arrive as 128-byte-wide, 128-byte-
//     swizzled tiles (128 rows x 512 codes, four k-blocks) in a ring of their own: one copy
//     of 128-byte rows instead of four copies of 32-byte rows for the same bytes measured 7 %
//     faster end to end, and the unpack warps can turn a tile into codes in registers before
//     the stage they will store into is free.  They release a packed tile themselves when its
//     last k-block has been read.
// Barriers the leader's MMA thread waits on live in the leader; the peer's TMA completes its
// activation bytes on the leader's barrier (cta_group::2 form) and the peer's unpack /
// epilogue warps arrive there through shared::cluster addresses.  No multicast loads.
//
// A pipeline stage covers 256 bytes of K (two 128-byte swizzle slabs), so every barrier
// handshake and tcgen05.commit is paid once per eight MMAs.  Warp roles per CTA: 0 TMA,
// 1 MMA (leader only), 2 TMEM owner, 4-11 unpack (one thread per row and slab), 12-15
// epilogue.  Every wait is bounded; a wait that gives up records a code in the status word
// and raises the CTA's abort flag.
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace kb {

namespace {

using namespace ptx;

constexpr int BM = 128;   // weight rows per CTA (256 per pair)
constexpr int BN = 256;   // tokens per pair tile (MMA N)
constexpr int BNH = 128;  // tokens loaded by each CTA
constexpr int BK = 128;   // one 128-byte swizzle row of K (a "slab")
constexpr int SLABS = 2;  // slabs per pipeline stage: barrier traffic is paid once per 256 bytes of K
constexpr int RS = 3;     // pipeline stages: raw (activations + packed weights) + unpacked weights
constexpr int ACT_SLAB = BNH * BK;                 // 16 KB
constexpr int ACT_BYTES = SLABS * ACT_SLAB;        // 32 KB
constexpr int RAW_BYTES = ACT_BYTES;               // 32 KB
constexpr int UNP_SLAB = BM * BK;                  // 16 KB
constexpr int UNP_BYTES = SLABS * UNP_SLAB;        // 32 KB
constexpr int STAGE_BYTES = RAW_BYTES + UNP_BYTES;  // 64 KB
// Packed weights travel in their own ring of 128-byte-wide tiles (128 rows x 128 B = 16 KB = four
// slabs = two stages).
constexpr int PKS = 2;                              // packed-weight tiles in flight
constexpr int PKT_STAGES = 2;                       // stages covered by one packed tile
constexpr int PKT_BYTES = BM * 128;                 // 16 KB, 128-byte swizzle
constexpr int NUM_BARS = 2 * RS + 2 * PKS + 5;
constexpr int SMEM_BYTES = 1024 + RS * STAGE_BYTES + PKS * PKT_BYTES + 8 * NUM_BARS + 16;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
constexpr int NUM_THREADS = 512;  // warps: 0 TMA, 1 MMA, 2 TMEM, 3 idle, 4-11 unpack, 12-15 epilogue
constexpr int TMEM_COLS = 2 * BN;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr long long WAIT_CYCLES = 2000000000ll;

struct Gemm2Params {
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
};

template <bool CLUSTER_ACQUIRE>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    long long t0 = 0;
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (CLUSTER_ACQUIRE ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
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

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                const Gemm2Params p) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_dyn + (base - smem_u32(smem_dyn));

    auto act_addr = [&](int s) { return base + (uint32_t)s * STAGE_BYTES; };
    auto unp_addr = [&](int s) { return act_addr(s) + RAW_BYTES; };
    auto pkt_addr = [&](int q) { return base + (uint32_t)(RS * STAGE_BYTES) + (uint32_t)q * PKT_BYTES; };
    const uint32_t tail = base + RS * STAGE_BYTES + PKS * PKT_BYTES;
    auto ready = [&](int s) { return tail + 8u * s; };                 // leader: activations landed + weights unpacked
    auto empty = [&](int s) { return tail + 8u * (RS + s); };          // local: the stage's MMAs completed
    auto pk_full = [&](int q) { return tail + 8u * (2 * RS + q); };    // local: a packed-weight tile landed
    auto pk_empty = [&](int q) { return tail + 8u * (2 * RS + PKS + q); };  // local: the tile has been unpacked
    auto tfull = [&](int b) { return tail + 8u * (2 * RS + 2 * PKS + b); };
    auto tempty = [&](int b) { return tail + 8u * (2 * RS + 2 * PKS + 2 + b); };
    const uint32_t drain_bar = tail + 8u * (2 * RS + 2 * PKS + 4);
    uint8_t *tail_ptr = base_ptr + RS * STAGE_BYTES + PKS * PKT_BYTES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail_ptr + 8 * NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader of the pair
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (p.kp + SLABS * BK - 1) / (SLABS * BK);  // stages per tile; a missing last slab is zero-filled by TMA
    const int tiles_n = (p.n + BN - 1) / BN;
    const int tiles_m = (p.m + 2 * BM - 1) / (2 * BM);
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; ++s) {
            // leader's producer arrives once carrying the pair's 64 KB of activation tx;
            // the 8 unpack warps of each CTA arrive once each
            mbar_init(ready(s), 17);
            mbar_init(empty(s), 1);  // tcgen05.commit (multicast)
        }
        for (int q = 0; q < PKS; ++q) {
            mbar_init(pk_full(q), 1);
            mbar_init(pk_empty(q), 8);  // the CTA's 8 unpack warps, after their last read of the tile
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull(b), 1);      // tcgen05.commit (multicast)
            mbar_init(tempty(b), 8);     // 4 epilogue warps of each CTA (used in the leader)
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before any remote arrival or TMA completion
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0, pit = 0;  // stage counter, packed-tile counter
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile / tiles_n) * (2 * BM) + (int)rank * BM;
                const int nh0 = (tile % tiles_n) * BN + (int)rank * BNH;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if ((kb % PKT_STAGES) == 0) {  // the packed weights of this and the next stage: one 128-byte-wide tile
                        const int q = pit % PKS;
                        if (!(ok = wait_bar<false>(pk_empty(q), ((pit / PKS) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_TMA_EMPTY))) break;
                        mbar_expect_tx(pk_full(q), PKT_BYTES);
                        tma_load_2d(pkt_addr(q), &tmap_w, pk_full(q), kb * (SLABS * BK / 4), m0);
                        ++pit;
                    }
                    const int s = it % RS;
                    const uint32_t ph = (it / RS) & 1u;
                    if (!(ok = wait_bar<false>(empty(s), ph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_TMA_EMPTY))) break;
                    if (leader) mbar_expect_tx(ready(s), 2 * ACT_BYTES);
                    const uint32_t lead_bar = mapa(ready(s), 0);
#pragma unroll
                    for (int sl = 0; sl < SLABS; ++sl)
                        tma_load_2d_pair(act_addr(s) + sl * ACT_SLAB, &tmap_x, lead_bar, (kb * SLABS + sl) * BK, nh0);
                }
            }
            // drain the packed-weight copies (their barriers are local); the activation copies
            // are accounted on the leader's barrier, which the leader's MMA thread drains
            const uint32_t issued = pit;
            for (uint32_t j = (issued > (uint32_t)PKS ? issued - PKS : 0); j < issued; ++j) {
                bool landed = false;
                for (uint32_t i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(pk_full(j % PKS), (j / PKS) & 1u);
                if (!landed) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && leader) {
            // D = s32, A (weight codes) = u8, B (activations) = s8, K-major, M = 256 (pair), N = 256
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++ti) {
                const int b = ti & 1;
                if (!(ok = wait_bar<false>(tempty(b), ((ti >> 1) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM_EMPTY))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % RS;
                    if (!(ok = wait_bar<false>(ready(s), (it / RS) & 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL))) break;
                    tc_fence_after();
#pragma unroll
                    for (int sl = 0; sl < SLABS; ++sl) {
                        const uint64_t adesc = umma_desc_sw128(unp_addr(s) + sl * UNP_SLAB);
                        const uint64_t bdesc = umma_desc_sw128(act_addr(s) + sl * ACT_SLAB);
#pragma unroll
                        for (int k4 = 0; k4 < BK / 32; ++k4)
                            umma_i8_pair(tmem_d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc,
                                         (kb | sl | k4) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair_multicast(empty(s), 3);
                }
                if (ok) umma_commit_pair_multicast(tfull(b), 3);
            }
            umma_commit_pair_multicast(drain_bar, 1);
            bool done = false;
            for (uint32_t i = 0; i < WAIT_LIMIT && !done; ++i) done = mbar_try_wait(drain_bar, 0);
            if (!done) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
        }
    } else if (warp >= 4 && warp < 12) {
        // ---------------- unpack: packed 2-bit -> swizzled code bytes (both CTAs) ----------------
        // thread = (row r, slab sl): 32 packed bytes -> one 128-byte swizzled row of that slab
        const int r = (threadIdx.x - 128) & 127, sl = (threadIdx.x - 128) >> 7;
        uint32_t it = 0, pit = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % RS;
                const int half = kb % PKT_STAGES;  // which stage of the packed tile
                if (half == 0) ++pit;
                const uint32_t pt = pit - 1;
                const int q = pt % PKS;
                if (!(ok = wait_bar<false>(pk_full(q), (pt / PKS) & 1u, abort_flag, p.status, DEV_TIMEOUT_UNPACK_FULL))) break;
                const bool last_use = half == PKT_STAGES - 1 || kb == num_kb - 1;
                // packed tile: 128-byte rows, 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)),
                // so the eight rows of a quarter-warp read eight different bank groups
                const uint8_t *prow = base_ptr + (pkt_addr(q) - base) + r * 128;
                const int c0 = half * 4 + sl * 2;
                uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
                {
                    lo = *reinterpret_cast<const uint4 *>(prow + (((c0) ^ (r & 7)) << 4));
                    hi = *reinterpret_cast<const uint4 *>(prow + (((c0 + 1) ^ (r & 7)) << 4));
                }
                // the codes are ready in registers before the stage's buffer is asked for: only the
                // stores sit between the stage being freed and its being ready again
                const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                uint4 o[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    o[c].x = w[c] & 0x03030303u;
                    o[c].y = (w[c] >> 2) & 0x03030303u;
                    o[c].z = (w[c] >> 4) & 0x03030303u;
                    o[c].w = (w[c] >> 6) & 0x03030303u;
                }
                if (last_use) {  // this warp has read all it needs from the tile
                    __syncwarp();
                    if (lane == 0) mbar_arrive(pk_empty(q));
                }
                // the code buffer of this stage is free once the MMAs of iteration it - RS have completed
                if (it >= (uint32_t)RS) {
                    if (!(ok = wait_bar<false>(empty(s), ((it / RS) - 1u) & 1u, abort_flag, p.status, DEV_TIMEOUT_UNPACK_FULL))) break;
                }
                uint8_t *dst = base_ptr + (unp_addr(s) - base) + sl * UNP_SLAB + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4 *>(dst + ((c ^ (r & 7)) << 4)) = o[c];
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa(ready(s), 0));
            }
        }
    } else if (warp >= 12) {
        // ---------------- epilogue (both CTAs, own 128 rows x 256 tokens) ----------------
        const int e = warp - 12;  // TMEM lane quarter (warp index % 4)
        constexpr int NCH = BN / 32;
        const bool has_bias = p.bias != nullptr;
        uint32_t ti = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++ti) {
            const int b = ti & 1;
            const int m0 = (tile / tiles_n) * (2 * BM) + (int)rank * BM, n0 = (tile % tiles_n) * BN;
            const int row = m0 + e * 32 + lane;
            const bool row_ok = row < p.m;
            const float sw = row_ok ? p.sw[row] : 0.0f;
            const float bias = (row_ok && has_bias) ? p.bias[row] : 0.0f;
            auto load_cols = [&](int c, float &sxv, int &smv) {
                const int tok = n0 + 32 * c + lane;
                const bool in = c < NCH && tok < p.n;
                sxv = in ? __ldg(p.sx + tok) : 1.0f;
                smv = in ? __ldg(p.sumq + tok) : 0;
            };
            float sx_cur, sx_next;
            int sm_cur, sm_next;
            load_cols(0, sx_next, sm_next);
            const size_t yoff = (size_t)n0 * p.ldy + row;
            float *yrow = p.y ? p.y + yoff : nullptr;
            int32_t *arow = p.acc ? p.acc + yoff : nullptr;
            ok = wait_bar<false>(tfull(b), (ti >> 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_EPI_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            // 16 half-chunks of 16 token columns; the TMEM load of the next half-chunk is in
            // flight while the current one is converted and stored
            constexpr int N16 = BN / 16;
            auto taddr = [&](int h16) { return tmem_base + (uint32_t)(b * BN + h16 * 16) + ((uint32_t)(e * 32) << 16); };
            auto process = [&](uint32_t(&v)[16], int h16) {
                const int hh = h16 & 1;
                const int valid = p.n - (n0 + h16 * 16);
                const size_t cbase = (size_t)(h16 * 16) * p.ldy;
                float outv[16];
                const bool add_resid = p.resid != nullptr && row_ok;
                if (add_resid) {
                    const float *rrow = p.resid + yoff + cbase;
#pragma unroll
                    for (int i = 0; i < 16; ++i) outv[i] = i < valid ? rrow[(size_t)i * p.ldy] : 0.0f;
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) outv[i] = 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float r_i = outv[i];
                    const float sx_i = __shfl_sync(0xffffffffu, sx_cur, hh * 16 + i);
                    const int sm_i = __shfl_sync(0xffffffffu, sm_cur, hh * 16 + i);
                    const int a = p.mul * (int)v[i] - p.off * sm_i;
                    outv[i] = dequant_out(a, sw, sx_i, bias, has_bias);
                    if (add_resid) outv[i] = __fadd_rn(outv[i], r_i);
                    if (p.relu) outv[i] = fmaxf(outv[i], 0.0f);
                    v[i] = (uint32_t)a;
                }
                if (row_ok) {
                    if (arow) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i < valid) arow[cbase + (size_t)i * p.ldy] = (int)v[i];
                    }
                    if (yrow) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i < valid) yrow[cbase + (size_t)i * p.ldy] = outv[i];
                        for (int q = 0; q < p.n_more; ++q) {
                            float *peer = p.y_more[q] + yoff + cbase;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < valid) peer[(size_t)i * p.ldy] = outv[i];
                        }
                    }
                }
            };
            uint32_t va[16], vb[16];
            tmem_ld16_async(taddr(0), va);
#pragma unroll 1
            for (int c = 0; c < NCH; ++c) {  // one pass = 32 columns = two half-chunks
                sx_cur = sx_next;
                sm_cur = sm_next;
                load_cols(c + 1, sx_next, sm_next);
                tmem_wait16(va);
                tmem_ld16_async(taddr(2 * c + 1), vb);
                process(va, 2 * c);
                tmem_wait16(vb);
                if (c + 1 < NCH) {
                    tmem_ld16_async(taddr(2 * c + 2), va);
                } else {
                    // the whole accumulator is in registers: hand the TMEM buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa(tempty(b), 0));
                }
                process(vb, 2 * c + 1);
            }
            (void)N16;
        }
        if (p.n_more) __threadfence_system();  // once per launch: the peer copies are performed before the exit
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the pair leaves together: no multicast arrival or MMA read targets an exited CTA
    tc_fence_after();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_act_map(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t rows, uint64_t row_stride) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    if (!fn) return fail(KB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {row_stride};
    cuuint32_t box[2] = {BK, BNH};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return KB_OK;
}

}  // namespace


// CTA-pair GEMM: used for token counts above 128 (a full 256-token MMA N)
int launch_gemm_tc2(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!L->has_tmap128) return fail(KB_ERR_UNSUPPORTED, "gemm: weight tensor map missing");
    if (!a.xq || !a.sx || !a.sumq) return fail(KB_ERR_INVALID, "gemm: needs pre-quantised activations");
    if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
        return fail(KB_ERR_INVALID, "gemm: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    CUtensorMap tmap_x;
    int rc = encode_act_map(&tmap_x, a.xq, L->kp, a.n, a.ldq);
    if (rc) return rc;
    Gemm2Params p;
    p.m = (int)L->m; p.n = (int)a.n; p.kp = (int)L->kp;
    p.sw = L->scales; p.bias = L->bias; p.sx = a.sx; p.sumq = a.sumq;
    p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.mul = L->mul; p.off = L->off; p.status = L->dev_status;
    p.n_more = a.y ? a.n_more : 0;
    for (int q = 0; q < MAX_PEERS - 1; ++q) p.y_more[q] = q < p.n_more ? a.y_more[q] : nullptr;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    const int dev = L->device;
    if (int rc_attr = set_dyn_smem_once(reinterpret_cast<const void *>(gemm_tc2_kernel), dev, SMEM_BYTES, "gemm2 smem attribute")) return rc_attr;
    int sms = 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) sms = 148;
    const int tiles = (int)(((L->m + 2 * BM - 1) / (2 * BM)) * ((a.n + BN - 1) / BN));
    int pairs = sms / 2;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel, tmap_x, L->tmap_w128, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "gemm2 launch");
}

}  // namespace kb
