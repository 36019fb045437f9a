// Small-batch forward for 2-bit weights (sm_100a): up to 32 tokens, weight streaming on the
// warp-level int8 MMA.
//
// For a handful of tokens the layer is still HBM-bound (every weight byte is read once, the
// activations fit in shared memory), but the dp4a GEMV spends one instruction per 4 products
// per token and becomes issue-bound from about 8 tokens on, while the tcgen05 GEMM has to push
// every unpacked weight through shared memory for a 64-token tile that is mostly padding.
// Here the weights go global -> registers -> MMA operand directly:
//   * a warp owns 16 weight rows x 256 k per step; lane (g = lane / 4, q = lane % 4) loads
//     16 packed bytes (64 codes, k = 64q .. 64q+63 of the step) of row g and of row g + 8;
//   * (word >> 2j) & 0x03030303 is four u8 codes in k order — exactly one 32-bit A-fragment
//     register of mma.sync.m16n8k32 (u8 x s8 -> s32).  The MMA sums over k, so any k
//     permutation applied to both operands is legal: MMA number 2w + h of a step takes, in lane
//     (g, q), the codes j = 2h, 2h + 1 of word w, i.e. k = 64q + 16w + 8h + {0..7}, and the
//     activation fragment of lane (token g, q) is bytes 8h .. 8h+7 of that token's 16-byte
//     chunk 4q + w — one 128-bit shared-memory read feeds both MMAs of a word;
//   * the 16 warps of a CTA split K (steps w, w + 16, ...), so a CTA works on one 16-row block at
//     a time and even a 3200-row layer spreads over 200 CTAs; partial accumulators meet in
//     shared memory (double-buffered, one barrier per block) and all 512 threads share
//     the epilogue: mul * S - off * sum(xq), dequantise, optional residual, coalesced stores.
// Weight loads run PF steps ahead across block boundaries and are first issued before
// griddepcontrol.wait, as in the GEMV.  Activations are staged once per CTA as int8, 16-byte
// chunk c of token n at slot c * NTOK + (n ^ 2 * ((c >> 2) & 3)): the XOR makes the fragment
// reads of every quarter-warp hit eight different bank groups.
#include <cstdlib>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

namespace {

struct MmaGemvParams {
    const uint8_t *w2;
    size_t row_bytes;
    int m, kp;
    const float *sw, *bias;
    const int8_t *xq;
    size_t ldq;
    const float *sx;
    const int32_t *sumq;
    int n;
    float *y;
    int32_t *acc;
    size_t ldy;
    int mul, off;
    float *y_more[MAX_PEERS - 1];
    int n_more;
    const float *resid;
    int relu;  // max(y, 0) after the bias
};

constexpr int WARPS = 16;
constexpr int PF = 4;  // steps in flight per warp (2 x 16 bytes per lane each)

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the 16 warps of a group; reached once per row block by every warp of the group, from
// whichever unrolled copy of the loop body the warp happens to be in
__device__ __forceinline__ void group_barrier(int grp) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(WARPS * 32) : "memory");
}

// NB = blocks of 8 tokens; G = groups of 16 warps per CTA.  The groups work on different row
// blocks and share one staged copy of the activations, which halves the activation traffic
// from L2 per weight byte compared with two separate CTAs on the SM.
template <int NB, int G>
__global__ void __launch_bounds__(G * WARPS * 32, 1) gemv_mma_kernel(const MmaGemvParams p) {
    constexpr int NTOK = NB * 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ float s_sx[NTOK];
    __shared__ int s_sum[NTOK];
    const int lane = threadIdx.x & 31, grp = threadIdx.x / (WARPS * 32), warp = (threadIdx.x >> 5) % WARPS;
    const int gtid = threadIdx.x % (WARPS * 32);  // thread index inside the group
    const int vblock = blockIdx.x * G + grp, vgrid = gridDim.x * G;  // the group's place in the row-block rotation
    const int g = lane >> 2, q = lane & 3;
    const int nsteps = (p.kp + 255) >> 8;
    const int chunks = nsteps * 16;
    uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);                               // [chunks][NTOK]
    int4 *part = reinterpret_cast<int4 *>(smem_raw + (size_t)chunks * NTOK * 16) + (size_t)grp * 2 * WARPS * NB * 32;  // [G][2][WARPS][16 * NTOK ints]
    const int row_blocks = (p.m + 15) >> 4;
    const bool has_steps = warp < nsteps;  // this warp's steps of a block: warp, warp + WARPS, ...

    // ---- weight pipeline: PF steps x (row g, row g + 8) in registers ----
    uint4 buf[PF][2];
    int lrb = vblock, lks = warp;  // load cursor over (row block, step)
    auto issue = [&](uint4(&dst)[2]) {
        const int kbyte = lks * 64 + q * 16;  // byte offset inside the packed row
        const bool ok = has_steps && lrb < row_blocks && kbyte * 4 < p.kp;
        const uint8_t *src = p.w2 + (size_t)(lrb * 16 + g) * p.row_bytes + kbyte;
        dst[0] = ok ? ld_stream_v4(src) : make_uint4(0, 0, 0, 0);
        dst[1] = ok ? ld_stream_v4(src + 8 * p.row_bytes) : make_uint4(0, 0, 0, 0);
        lks += WARPS;
        if (lks >= nsteps) { lks = warp; lrb += vgrid; }
    };
#pragma unroll
    for (int s = 0; s < PF; ++s) issue(buf[s]);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- activations -> shared memory: 16-byte asynchronous copies (global -> shared without a register stop; with
    // most of the SM configured as shared memory the L1 that register loads pass through is a few KB and they crawl),
    // all of a thread's copies in flight at once; absent tokens and the row tail are zero-filled ----
    {
        const int total = chunks * NTOK;
        const unsigned rot = total > 0 ? (unsigned)((blockIdx.x * 2654435761u) % (unsigned)total) & ~7u : 0u;
        const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);
        for (int lin = threadIdx.x; lin < total; lin += G * WARPS * 32) {
            // every CTA copies the same bytes: each starts at a different offset, so that at any
            // moment the SMs ask different L2 lines instead of queueing on one
            const int idx = (int)(((unsigned)lin + rot) % (unsigned)total);
            const int n_lo = idx & 7, rest = idx >> 3;
            const int c = rest % chunks, nb = rest / chunks;
            const int n = nb * 8 + n_lo;
            const int slot = c * NTOK + (n ^ (2 * ((c >> 2) & 3)));
            const bool live = n < p.n && c * 16 < p.kp;
            const int8_t *src = live ? p.xq + (size_t)n * p.ldq + (size_t)c * 16 : p.xq;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(xs_addr + (uint32_t)slot * 16u), "l"(src), "r"(live ? 16 : 0)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    if (threadIdx.x < NTOK) {
        s_sx[threadIdx.x] = (int)threadIdx.x < p.n ? p.sx[threadIdx.x] : 1.0f;
        s_sum[threadIdx.x] = (int)threadIdx.x < p.n ? p.sumq[threadIdx.x] : 0;
    }
    __syncthreads();

    int acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0;

    // the partial sums of a finished block meet in shared memory (buffer = block parity, one
    // barrier per block), and the threads share the epilogue: thread o < 16 * NTOK owns output
    // (row o % 16, token o / 16) of every block.  Its row scale, bias and residual are fetched
    // when the block starts, so the epilogue itself waits on no global load.
    const int row_l = gtid & 15, tok = gtid >> 4;
    const bool owner = gtid < 16 * NTOK && tok < p.n;
    // partials are stored [warp][token][row ^ 8 * ((token >> 1) & 1)]: the fragment stores are
    // two-way conflicted at worst and the epilogue reads are conflict-free
    const int src_word = tok * 16 + (row_l ^ (8 * ((tok >> 1) & 1)));
    const float my_sx = owner ? s_sx[tok] : 1.0f;
    const int my_sum = owner ? s_sum[tok] : 0;
    float e_sw = 0.0f, e_bias = 0.0f, e_res = 0.0f;
    auto prefetch_epilogue = [&](int rb) {
        const int row = rb * 16 + row_l;
        if (owner && rb < row_blocks && row < p.m) {
            e_sw = p.sw[row];
            if (p.bias) e_bias = p.bias[row];
            if (p.resid && p.y) e_res = p.resid[(size_t)tok * p.ldy + row];
        }
    };
    int parity = 0;
    auto finish_block = [&](int rb) {
        int *mine = reinterpret_cast<int *>(part) + (size_t)(parity * WARPS + warp) * (16 * NTOK);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            // lane (g, q) holds rows g, g + 8 x tokens nb * 8 + 2q, + 1
            int *dst = mine + (nb * 8 + 2 * q) * 16;
            const int r0 = g ^ (8 * (q & 1)), r1 = (g + 8) ^ (8 * (q & 1));
            dst[r0] = acc[nb][0];
            dst[16 + r0] = acc[nb][1];
            dst[r1] = acc[nb][2];
            dst[16 + r1] = acc[nb][3];
            acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0;
        }
        group_barrier(grp);
        const int row = rb * 16 + row_l;
        if (owner && row < p.m) {
            const int *pi = reinterpret_cast<const int *>(part) + (size_t)parity * WARPS * (16 * NTOK) + src_word;
            int sum = 0;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) sum += pi[w * (16 * NTOK)];
            const int a = p.mul * sum - p.off * my_sum;
            const size_t off = (size_t)tok * p.ldy + row;
            if (p.acc) p.acc[off] = a;
            if (p.y) {
                float v = dequant_out(a, e_sw, my_sx, e_bias, p.bias != nullptr);
                if (p.resid) v = __fadd_rn(v, e_res);
                if (p.relu) v = fmaxf(v, 0.0f);
                p.y[off] = v;
                for (int r = 0; r < p.n_more; ++r) p.y_more[r][off] = v;  // peer copies over NVLink
            }
        }
        parity ^= 1;
        prefetch_epilogue(rb + vgrid);
    };
    prefetch_epilogue(vblock);

    int crb = vblock, cks = warp;  // consume cursor
    while (crb < row_blocks) {
#pragma unroll
        for (int s = 0; s < PF; ++s) {
            if (crb < row_blocks) {  // uniform over the warp
                if (has_steps) {
                    const uint32_t wa[4] = {buf[s][0].x, buf[s][0].y, buf[s][0].z, buf[s][0].w};
                    const uint32_t wb[4] = {buf[s][1].x, buf[s][1].y, buf[s][1].z, buf[s][1].w};
                    const int c0 = cks * 16 + 4 * q;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const uint32_t g_lo0 = wa[w] & 0x03030303u, g_lo1 = (wa[w] >> 2) & 0x03030303u;  // row g
                        const uint32_t g_hi0 = (wa[w] >> 4) & 0x03030303u, g_hi1 = (wa[w] >> 6) & 0x03030303u;
                        const uint32_t h_lo0 = wb[w] & 0x03030303u, h_lo1 = (wb[w] >> 2) & 0x03030303u;  // row g + 8
                        const uint32_t h_hi0 = (wb[w] >> 4) & 0x03030303u, h_hi1 = (wb[w] >> 6) & 0x03030303u;
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint4 xv = xs[(c0 + w) * NTOK + ((nb * 8 + g) ^ (2 * q))];
                            mma_u8s8(acc[nb], g_lo0, h_lo0, g_lo1, h_lo1, xv.x, xv.y);
                            mma_u8s8(acc[nb], g_hi0, h_hi0, g_hi1, h_hi1, xv.z, xv.w);
                        }
                    }
                    issue(buf[s]);
                    cks += WARPS;
                }
                if (!has_steps || cks >= nsteps) {
                    finish_block(crb);
                    cks = warp;
                    crb += vgrid;
                }
            }
        }
    }
    if (p.n_more) __threadfence_system();
}

constexpr int groups_for(int nb) { return nb == 1 ? 2 : 1; }  // 16 tokens and more need the registers

size_t mma_smem_bytes(size_t kp, int nb) {
    const size_t nsteps = (kp + 255) / 256;
    return nsteps * 256 * (size_t)(nb * 8) + (size_t)groups_for(nb) * nb * 2 * WARPS * 512;
}

template <int NB>
int launch_nb(const MmaGemvParams &p, cudaStream_t stream) {
    constexpr int G = groups_for(NB);
    auto kern = gemv_mma_kernel<NB, G>;
    const size_t smem = mma_smem_bytes((size_t)p.kp, NB);
    if (smem > 40 * 1024) {  // the static arrays count toward the 48 KB default limit too
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "small-batch smem attribute");
    }
    static thread_local size_t c_smem = ~(size_t)0;
    static thread_local int c_occ = 0, c_sms = 0;
    if (c_smem != smem) {
        int occ = 0, dev = 0, sms = 148;
        cudaGetDevice(&dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, G * WARPS * 32, smem) != cudaSuccess || occ < 1) occ = 1;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
        c_smem = smem; c_occ = occ; c_sms = sms;
    }
    const int row_blocks = (p.m + 15) / 16;
    const int want = (row_blocks + G - 1) / G;
    int ctas = want < c_sms * c_occ ? want : c_sms * c_occ;
    static const int env_maxctas = [] { const char *v = getenv("KB_MMA_MAXCTAS"); return v && *v ? atoi(v) : 0; }();
    if (env_maxctas > 0 && ctas > env_maxctas) ctas = env_maxctas;  // tuning override
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
    cfg.blockDim = dim3(G * WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool pdl = [] { const char *v = getenv("KB_GEMV_PDL"); return !(v && *v == '0'); }();
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "small-batch launch");
}

}  // namespace

// up to 32 tokens, as long as their int8 activations fit in shared memory
bool gemv_mma_supports(const Linear *lin, size_t n) {
    if (n < 1 || n > 32) return false;
    const int nb = n <= 8 ? 1 : (n <= 16 ? 2 : 4);
    return mma_smem_bytes(lin->kp, nb) <= 200 * 1024;
}

int auto_path(const Linear *lin, size_t n, bool prequantised) {
    const size_t gemv_max = prequantised ? 2 : 4;
    // one or two pre-quantised tokens: the streaming kernel (3.1 us per dependent 4096 x 4096 layer against 3.7),
    // except for the largest layers with short rows (one token) or long rows (two), where the register-pipelined
    // GEMV's shorter ramp wins
    // (measured, one / two tokens, streaming kernel against the GEMV: 14336 x 8192 8.6 / 11.2 against 8.9 / 11.8 us,
    // 4096 x 28672 9.3 / 14.1 against 12.6 / 17.4, 8192 x 28672 14.8 / 22.0 against 16.9 / 19.6, 28672 x 8192
    // 13.9 / 17.1 against 13.4 / 17.9)
    // and many short rows (9600 x 3200: 5.2 / 7.3 against 4.1 / 5.5 us; 17280 x 3200: 6.4 / 9.4 against 5.8 / 7.3)
    const bool big = lin->m_alloc * lin->row_bytes > ((size_t)32 << 20), wide = lin->kp >= 16384;
    const bool many_short_rows = lin->kp < 4096 && lin->m >= 8192;
    if (prequantised && !many_short_rows && ((n == 1 && (!big || wide)) || (n == 2 && !(big && wide))) && gemv_stream_supports(lin, n))
        return KB_PATH_GEMV_STREAM;
    if (n <= gemv_max && gemv_supports(lin, n)) return KB_PATH_GEMV;
    // 3..8 tokens of a large layer: the streaming kernel's MMA form (19 us against 23 for 4 tokens of 8192 -> 28672);
    // small layers are latency-bound and the kernel below has the shorter prologue
    if (prequantised && n <= 8 && lin->m * lin->kp >= ((size_t)64 << 20) && gemv_stream_supports(lin, n)) return KB_PATH_GEMV_STREAM;
    // 17..32 tokens of a mid-sized or large layer: the tensor-memory GEMM's 64-token tile is already ahead
    // (32 tokens: 9600 x 3200 12.0 against 13.5 us, 17280 x 3200 12.7 against 18.7; 3200 x 3200 11.4 against 9.7)
    if (n > 16 && n <= 32 && lin->m * lin->kp >= ((size_t)24 << 20)) return KB_PATH_GEMM_TC;
    if (n <= 32 && gemv_mma_supports(lin, n)) return KB_PATH_GEMV_MMA;
    if (n <= 8 && gemv_supports(lin, n)) return KB_PATH_GEMV;
    return KB_PATH_GEMM_TC;
}

int launch_gemv_mma(const FwdArgs &a, cudaStream_t stream) {
    const Linear *L = a.lin;
    if (a.n == 0) return KB_OK;
    if (!gemv_mma_supports(L, a.n))
        return fail(KB_ERR_UNSUPPORTED, "small-batch kernel: %zu tokens x K=%zu do not fit in shared memory", a.n, L->k);
    if (!a.xq || !a.sx || !a.sumq) return fail(KB_ERR_INVALID, "small-batch kernel: needs pre-quantised activations");
    if ((reinterpret_cast<uintptr_t>(a.xq) & 15) || (a.ldq % 16) || a.ldq < L->kp)
        return fail(KB_ERR_INVALID, "small-batch kernel: xq must be 16-byte aligned with ldq >= %zu and ldq %% 16 == 0", L->kp);
    MmaGemvParams p;
    p.w2 = L->w2; p.row_bytes = L->row_bytes; p.m = (int)L->m; p.kp = (int)L->kp;
    p.sw = L->scales; p.bias = L->bias;
    p.xq = a.xq; p.ldq = a.ldq; p.sx = a.sx; p.sumq = a.sumq; p.n = (int)a.n;
    p.y = a.y; p.acc = a.acc; p.ldy = a.ldy ? a.ldy : L->m;
    p.mul = L->mul; p.off = L->off;
    p.n_more = a.y ? a.n_more : 0;
    for (int r = 0; r < MAX_PEERS - 1; ++r) p.y_more[r] = r < p.n_more ? a.y_more[r] : nullptr;
    p.resid = a.y ? a.resid : nullptr;
    p.relu = a.relu ? 1 : 0;
    if (a.n <= 8) return launch_nb<1>(p, stream);
    if (a.n <= 16) return launch_nb<2>(p, stream);
    return launch_nb<4>(p, stream);
}

}  // namespace kb
