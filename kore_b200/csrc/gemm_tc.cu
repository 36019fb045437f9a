// Prefill GEMM for 2-bit weights on the 5th-generation tensor cores (sm_100a only).
//
//   acc[tok, row] = sum_k code(W[row, k]) * xq[tok, k]      (u8 x s8 -> s32, tcgen05 kind::i8)
//
// Tile: 128 weight rows (MMA M, one TMEM lane each) x BN tokens (MMA N, TMEM columns),
// K consumed 128 bytes per pipeline stage (= one 128-byte swizzle row, four K=32 MMAs).
// One persistent CTA per SM, 12 warps with fixed roles:
//   warp 0      TMA producer: int8 activation tile [BN x 128 B] (128-byte swizzle) and the
//               PACKED weight tile [128 rows x 32 B] into the stage, completing on `full`
//   warps 4-7   unpack: thread r expands row r's 32 packed bytes into 128 code bytes
//               (word >> 2j) & 0x03030303 and stores them with the same 128-byte swizzle
//               the MMA descriptor expects, then fence.proxy.async + arrive on `unpacked`
//   warp 1      one lane issues tcgen05.mma (A = codes from smem, B = activations from
//               smem, D = int32 in TMEM), tcgen05.commit frees the stage / publishes the tile
//   warp 2      owns the TMEM allocation (2 accumulator buffers of BN columns)
//   warps 8-11  epilogue: tcgen05.ld 32 lanes x 32 columns, integer correction
//               mul*S - off*sum(xq), dequantise, coalesced stores (lanes = consecutive rows
//               of y[tok, :]); overlaps with the next tile's main loop
// Tensor-pipe bound: 2*128*BN*128 ops per stage.  No multicast anywhere.
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in a
// device status word, raises a CTA-wide abort flag that all other waits observe, and
// the CTA drains its copies, frees its TMEM and returns.
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

namespace {

constexpr int BM = 128;
constexpr int BK = 128;
constexpr int NUM_THREADS = 384;
constexpr uint32_t WAIT_LIMIT = 1u << 22;          // try_wait polls before a wait gives up ...
constexpr long long WAIT_CYCLES = 2000000000ll;    // ... or about one second of SM clocks, whichever is first

template <int BN>
struct Cfg {
    static constexpr int ACT_BYTES = BN * BK;        // int8 activations
    static constexpr int UNP_BYTES = BM * BK;        // unpacked codes
    static constexpr int PK_BYTES = BM * (BK / 4);   // packed codes
    static constexpr int STAGE_BYTES = ACT_BYTES + UNP_BYTES + PK_BYTES;
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 5 : 6);
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int TAIL_BYTES = 8 * (3 * STAGES + 5) + 16;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + TAIL_BYTES;
};

struct GemmParams {
    int m, n, kp;
    const float *sw, *bias, *sx;
    const int32_t *sumq;
    float *y;
    int32_t *acc;
    size_t ldy;
    int mul, off;
    int *status;
    float *y_more[MAX_PEERS - 1];  // further copies of y (peer GPUs), same offsets
    int n_more;
    const float *resid;
    int relu;  // max(y, 0) after the bias
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it gave up or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, int code) {
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// K-major operand tile, 128-byte rows, 128-byte swizzle: 8-row groups are 1024 B apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const GemmParams p) {
    using C = Cfg<BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_dyn + (base - smem_u32(smem_dyn));

    auto act_addr = [&](int s) { return base + (uint32_t)s * C::STAGE_BYTES; };
    auto unp_addr = [&](int s) { return act_addr(s) + C::ACT_BYTES; };
    auto pk_addr = [&](int s) { return unp_addr(s) + C::UNP_BYTES; };
    const uint32_t tail = base + STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return tail + 8u * s; };
    auto unp_bar = [&](int s) { return tail + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return tail + 8u * (2 * STAGES + s); };
    auto tfull_bar = [&](int b) { return tail + 8u * (3 * STAGES + b); };
    auto tempty_bar = [&](int b) { return tail + 8u * (3 * STAGES + 2 + b); };
    const uint32_t drain_bar = tail + 8u * (3 * STAGES + 4);
    uint8_t *tail_ptr = base_ptr + STAGES * C::STAGE_BYTES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail_ptr + 8 * (3 * STAGES + 5));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = p.kp / BK;
    const int tiles_n = (p.n + BN - 1) / BN;
    const int tiles_m = (p.m + BM - 1) / BM;
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(unp_bar(s), 4);     // one arrival per unpack warp
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 4);  // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)C::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, DEV_TIMEOUT_TMA_EMPTY))) break;
                    mbar_expect_tx(full_bar(s), C::ACT_BYTES + C::PK_BYTES);
                    tma_load_2d(act_addr(s), &tmap_x, full_bar(s), kb * BK, n0);
                    tma_load_2d(pk_addr(s), &tmap_w, full_bar(s), kb * (BK / 4), m0);
                }
            }
            // drain: every copy this thread issued must have landed before the CTA exits
            const uint32_t issued = it;
            for (uint32_t j = (issued > (uint32_t)STAGES ? issued - STAGES : 0); j < issued; ++j) {
                const int s = j % STAGES;
                const uint32_t ph = (j / STAGES) & 1u;
                bool landed = false;
                for (uint32_t i = 0; i < WAIT_LIMIT && !landed; ++i) landed = mbar_try_wait(full_bar(s), ph);
                if (!landed) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D = s32, A (weight codes) = u8, B (activations) = s8, both K-major, M = 128, N = BN
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++ti) {
                const int b = ti & 1;
                if (!(ok = mbar_wait(tempty_bar(b), ((ti >> 1) & 1u) ^ 1u, abort_flag, p.status, DEV_TIMEOUT_MMA_TMEM_EMPTY))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_MMA_FULL))) break;
                    if (!(ok = mbar_wait(unp_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_MMA_UNPACKED))) break;
                    tc_fence_after();
                    const uint64_t adesc = umma_desc_sw128(unp_addr(s));
                    const uint64_t bdesc = umma_desc_sw128(act_addr(s));
#pragma unroll
                    for (int k4 = 0; k4 < BK / 32; ++k4)
                        umma_i8(tmem_d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc,
                                (kb | k4) != 0 ? 1u : 0u);
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(tfull_bar(b));
            }
            // all MMAs issued by this thread must retire before smem/TMEM are released
            umma_commit(drain_bar);
            bool done = false;
            for (uint32_t i = 0; i < WAIT_LIMIT && !done; ++i) done = mbar_try_wait(drain_bar, 0);
            if (!done) atomicCAS(p.status, 0, DEV_TIMEOUT_DRAIN);
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------- unpack: packed 2-bit -> swizzled code bytes ----------------
        const int r = threadIdx.x - 128;  // weight row inside the tile
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1u;
                if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, DEV_TIMEOUT_UNPACK_FULL))) break;
                const uint8_t *pk = base_ptr + (pk_addr(s) - base) + r * 32;
                uint8_t *dst = base_ptr + (unp_addr(s) - base) + r * 128;
                const uint4 lo = *reinterpret_cast<const uint4 *>(pk);
                const uint4 hi = *reinterpret_cast<const uint4 *>(pk + 16);
                const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 o;
                    o.x = w[c] & 0x03030303u;
                    o.y = (w[c] >> 2) & 0x03030303u;
                    o.z = (w[c] >> 4) & 0x03030303u;
                    o.w = (w[c] >> 6) & 0x03030303u;
                    *reinterpret_cast<uint4 *>(dst + ((c ^ (r & 7)) << 4)) = o;
                }
                // every thread publishes its own generic-proxy stores to the async proxy, then
                // one lane per warp arrives (128 arrivals on one mbarrier would serialise)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(unp_bar(s));
            }
        }
    } else if (warp >= 8) {
        // ---------------- epilogue ----------------
        // Lane l of warp e owns output feature m0 + 32e + l (one TMEM lane); a chunk is 32
        // token columns.  Per-token scale and code sum are held one column per lane in
        // registers and broadcast with shuffles, so the loop touches no memory besides the
        // output stores (32 lanes x 4 B = one 128-byte row segment per instruction).
        const int e = warp - 8;            // TMEM lane quarter (warp index % 4)
        const int et = threadIdx.x - 256;  // 0..127
        constexpr int NCH = BN / 32;
        const bool has_bias = p.bias != nullptr;
        uint32_t ti = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++ti) {
            const int b = ti & 1;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            const int row = m0 + e * 32 + lane;
            const bool row_ok = row < p.m;
            const float sw = row_ok ? p.sw[row] : 0.0f;
            const float bias = (row_ok && has_bias) ? p.bias[row] : 0.0f;
            // per-token scale and code sum of chunk c, one column per lane (next chunk prefetched)
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
            int32_t *arow = p.acc ? p.acc + (size_t)n0 * p.ldy + row : nullptr;
            ok = mbar_wait(tfull_bar(b), (ti >> 1) & 1u, abort_flag, p.status, DEV_TIMEOUT_EPI_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < NCH; ++c) {
                sx_cur = sx_next;
                sm_cur = sm_next;
                load_cols(c + 1, sx_next, sm_next);
                uint32_t v[32];
                tmem_ld32(tmem_base + (uint32_t)(b * BN + c * 32) + ((uint32_t)(e * 32) << 16), v);
                if (c == NCH - 1) {
                    // this thread has read its whole accumulator: hand the TMEM buffer back
                    // before the last stores go out
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(b));
                }
                const int valid = p.n - (n0 + c * 32);  // columns of this chunk that are real tokens
                const size_t cbase = (size_t)(c * 32) * p.ldy;
                float outv[32];
                const bool add_resid = p.resid != nullptr && row_ok;
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
                    if (yrow) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) yrow[cbase + (size_t)i * p.ldy] = outv[i];
                        // column-sharded layers: the same values into every peer's copy (NVLink stores)
                        for (int q = 0; q < p.n_more; ++q) {
                            float *peer = p.y_more[q] + yoff + cbase;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < valid) peer[(size_t)i * p.ldy] = outv[i];
                        }
                    }
                }
            }
        }
        if (p.n_more) __threadfence_system();  // once per launch: the peer copies are performed before the exit
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::TMEM_COLS)
                     : "memory");
    }
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

// 2-D byte tensor [rows][row_stride bytes], box [box_inner bytes x box_rows]
int encode_2d(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t rows, uint64_t row_stride,
              uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(KB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {row_stride};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return KB_OK;
}

int sm_count(int device) {
    static int cached[64] = {0};
    if (device < 0 || device >= 64) return 148;
    if (!cached[device]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        cached[device] = v;
    }
    return cached[device];
}

namespace {

template <int BN>
int launch_bn(const FwdArgs &a, cudaStream_t stream) {
    using C = Cfg<BN>;
    const Linear *L = a.lin;
    CUtensorMap tmap_x;
    int rc = encode_2d(&tmap_x, a.xq, L->kp, a.n, a.ldq, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    GemmParams p;
    p.m = (int)L->m; p.n = (int)a.n; p.kp = (int)L->kp;
    p.sw = L->scales; p.bias = L->bias; p.sx = a.sx; p.sumq = a.sumq;
    p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.n_more = a.y ? a.n_more : 0;
    for (int q = 0; q < MAX_PEERS - 1; ++q) p.y_more[q] = q < p.n_more ? a.y_more[q] : nullptr;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    p.mul = L->mul; p.off = L->off; p.status = L->dev_status;
    auto kern = gemm_tc_kernel<BN>;
    const int dev = L->device;
    if (int rc_attr = set_dyn_smem_once(reinterpret_cast<const void *>(kern), dev, C::SMEM_BYTES, "gemm smem attribute")) return rc_attr;
    const int tiles = (int)(((L->m + BM - 1) / BM) * ((a.n + BN - 1) / BN));
    const int sms = sm_count(L->device);
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmap_x, L->tmap_w, p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "gemm launch");
}

}  // namespace

int encode_weight_tmap(Linear *lin) {
    int rc = encode_2d(&lin->tmap_w, lin->w2, lin->row_bytes, lin->m_alloc, lin->row_bytes, BK / 4, BM,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    lin->has_tmap = (rc == KB_OK);
    // the CTA-pair kernel's map is optional: without it the single-CTA kernel serves every size
    lin->has_tmap64 = rc == KB_OK && encode_2d(&lin->tmap_w64, lin->w2, lin->row_bytes, lin->m_alloc, lin->row_bytes,
                                               BK / 2, BM, CU_TENSOR_MAP_SWIZZLE_NONE) == KB_OK;
    // 128-byte-wide, swizzled tiles for the CTA-pair kernel (rows shorter than 128 bytes keep the single-CTA kernel)
    lin->has_tmap128 = rc == KB_OK && lin->row_bytes >= 128 &&
                       encode_2d(&lin->tmap_w128, lin->w2, lin->row_bytes, lin->m_alloc, lin->row_bytes, BK, BM,
                                 CU_TENSOR_MAP_SWIZZLE_128B) == KB_OK;
    return rc;
}

bool gemm_tc_supports(const Linear *lin, size_t n) {
    return lin->has_tmap && n >= 1 && n < (1u << 30);
}

int launch_gemm_tc(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!L->has_tmap) return fail(KB_ERR_UNSUPPORTED, "gemm: weight tensor map missing");
    if (!a.xq || !a.sx || !a.sumq) return fail(KB_ERR_INVALID, "gemm: needs pre-quantised activations");
    if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
        return fail(KB_ERR_INVALID, "gemm: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    // up to 128 tokens: weights unpacked into tensor memory (KB_GEMM_TMEM_A=0 keeps the shared-memory tiles)
    static const int use_tmem_a = []() { const char *e = getenv("KB_GEMM_TMEM_A"); return e ? atoi(e) : 1; }();
    if (a.n <= 128 && use_tmem_a && L->has_tmap128) return launch_gemm_tcs(a, stream);
    if (a.n <= 64) return launch_bn<64>(a, stream);
    if (a.n <= 128) return launch_bn<128>(a, stream);
    // full 256-token tiles go to the CTA-pair kernel (KB_GEMM_PAIR=0 keeps the single-CTA one)
    static const int use_pair = []() { const char *e = getenv("KB_GEMM_PAIR"); return e ? atoi(e) : 1; }();
    if (use_pair && L->has_tmap128) return launch_gemm_tc2(a, stream);
    return launch_bn<256>(a, stream);
}

}  // namespace kb
