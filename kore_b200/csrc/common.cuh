// Shared declarations of the kore_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/kore_b200.h"

namespace kb {

// ---- device weight layout -------------------------------------------------------
// Weights live in HBM as 2-bit codes, row-major [M_alloc][Kp/4] bytes with
// Kp = K rounded up to 128 (row stride is a multiple of 32 bytes) and M_alloc = M
// rounded up to 128 (pad rows are zero).  Inside every aligned 32-bit word, which
// covers 16 consecutive k, element k0 + 4*j + b sits in byte b at bits [2j+1:2j].
// (word >> 2j) & 0x03030303 therefore yields the four codes of k0+4j .. k0+4j+3 as
// four bytes in memory order — the operand order of dp4a and of an int8 MMA tile.
//   ternary   : code = trit + 1      value = code - 1       (pad code 1)
//   quaternary: code = KORE's index  value = 2*code - 3     (pad code 0)
// Kernels accumulate S = sum(code * xq) and correct in the epilogue:
//   acc = mul * S - off * sum(xq),  (mul, off) = (1,1) ternary, (2,3) quaternary.
constexpr int MAX_PEERS = 8;  // GPUs of one NVSwitch box
constexpr int K_ALIGN = 128;
constexpr int M_ALIGN = 128;

constexpr uint32_t HANDLE_MAGIC = 0x4b42324cu;  // "KB2L"

// status word written by the tcgen05 GEMM when a bounded wait gives up
enum DevStatus : int {
    DEV_OK = 0,
    DEV_TIMEOUT_TMA_EMPTY = 1,
    DEV_TIMEOUT_UNPACK_FULL = 2,
    DEV_TIMEOUT_MMA_FULL = 3,
    DEV_TIMEOUT_MMA_UNPACKED = 4,
    DEV_TIMEOUT_MMA_TMEM_EMPTY = 5,
    DEV_TIMEOUT_EPI_TMEM_FULL = 6,
    DEV_TIMEOUT_DRAIN = 7
};

struct Linear {
    uint32_t magic;
    int kind;
    int device;
    size_t m, k, kp, m_alloc, row_bytes;
    uint8_t *w2;    // [m_alloc][row_bytes]
    float *scales;  // [m_alloc]
    float *bias;    // [m_alloc] or nullptr
    int mul, off;
    CUtensorMap tmap_w;    // 2-D map over w2 for the GEMM (box 32 B x 128 rows)
    CUtensorMap tmap_w64;  // same tensor, box 64 B x 128 rows
    CUtensorMap tmap_w128;  // same tensor, box 128 B x 128 rows, 128-byte swizzle (CTA-pair GEMM: four K slabs per tile)
    bool has_tmap;
    bool has_tmap64, has_tmap128;
    int *dev_status;  // one int in device memory
};

// one member of a grouped launch (device pointers of its handle)
struct LayerRef {
    const uint8_t *w2;
    const float *sw;
    const float *bias;  // nullptr: no bias
};

// ---- error plumbing (api.cu) -----------------------------------------------------
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
#define KB_CUDA(expr)                                      \
    do {                                                   \
        cudaError_t _e = (expr);                           \
        if (_e != cudaSuccess) return kb::cuda_fail(_e, #expr); \
    } while (0)

// Raises a kernel's dynamic shared-memory limit once per (kernel, device).  The device is made
// current for the call, and concurrent callers are serialised, so the forward entry points may
// be used from many host threads and on several devices.
int set_dyn_smem_once(const void *kernel, int device, int bytes, const char *what);

// ---- launchers (each returns a KB_* status; all work is enqueued on `stream`) ----
// the same quantiser on rows of flagged words (see FwdArgs::xf): waits, bounded, for epoch (*round << 8) | seq
int launch_act_quant_flagged(const unsigned long long *x, size_t ldx, size_t n, size_t k, const int *round, int seq, int8_t *xq,
                             size_t ldq, float *sx, int32_t *sumq, int *status, cudaStream_t stream);
int launch_act_quant(const float *x, size_t n, size_t k, int8_t *xq, size_t ldq, float *sx,
                     int32_t *sumq, cudaStream_t stream);

int launch_repack_wire(int kind, const uint8_t *wire, size_t m, size_t k, uint8_t *w2,
                       size_t row_bytes, size_t m_alloc, cudaStream_t stream);
int launch_quantise_f32(int kind, int quantiser, const float *w, size_t m, size_t k, float threshold,
                        uint8_t *w2, size_t row_bytes, size_t m_alloc, float *scales,
                        cudaStream_t stream);
int launch_export_wire(int kind, const uint8_t *w2, size_t row_bytes, size_t m, size_t k,
                       uint8_t *wire, cudaStream_t stream);
int launch_dequantize(int kind, const uint8_t *w2, size_t row_bytes, const float *scales, size_t m,
                      size_t k, float *w, cudaStream_t stream);
int launch_transpose_f32(const float *src, size_t rows, size_t cols, float *dst, cudaStream_t stream);
// base-243 rows [n][ceil(k/5)] -> int8 trits [n][ldq] (tail zero) + per-row sums
int launch_decode_trits_i8(const uint8_t *wire, size_t n, size_t k, int8_t *xq, size_t ldq, int32_t *sumq,
                           cudaStream_t stream);

// State of the flag barrier between the ranks of a sharded layer (all device pointers).
struct PeerSync {
    int *const *flag_arrays;  // [world] -> each rank's int32[world] flag array (local or peer mapping)
    int *epoch_counter;       // local, bumped once per barrier
    int *done_counter;        // local, CTAs finished in the current launch (returns to 0)
    int *status;              // local, 100+q if rank q never arrived
    int world, rank;
};

struct FwdArgs {
    const Linear *lin;
    // exactly one of (x) or (xq, sx, sumq) is set
    const float *x;
    const int8_t *xq;
    size_t ldq;
    const float *sx;
    const int32_t *sumq;
    size_t n;
    float *y;      // nullable
    int32_t *acc;  // nullable
    size_t ldy;
    // column-sharded layers: the same y values are also stored into these buffers (peer GPUs'
    // copies of the full output, mapped into this process) at the same offsets as in y
    float *y_more[MAX_PEERS - 1];
    int n_more;
    // optional cross-GPU completion barrier fused into the tail of the kernel (GEMV only)
    const struct PeerSync *sync;
    // optional residual, same [N][ldy] layout as y (may be y itself): y = dequant(...) + resid
    const float *resid;
    // ReLU on the dequantised output (after the bias): y = max(dequant(...) + bias, 0); not combined with resid
    bool relu;
    // GEMV only: size the grid for launches that overlap with other streams' GEMVs
    bool shared_grid;
    // GEMV with f32 input only (decoder fusions): RMSNorm in the prologue (gamma, eps), a known
    // per-token max|x| instead of the prologue's reduction, SiLU(gate) * up in the epilogue for
    // weights whose rows alternate gate_i, up_i (y is then [N][M / 2]) with the per-token max|h|
    // collected by atomic max, and N floats the launch zeroes
    const float *gamma;
    float eps;
    const float *x_absmax;
    bool swiglu;
    float *absmax_out;
    float *clear_word;
    // streaming kernel only, column-sharded layers exchanging "flagged" words: every f32 value travels as an
    // 8-byte pair (value bits, epoch), stored with one 8-byte store, so a reader that finds the epoch it expects
    // has the value as well and no fence, flag array or barrier is needed.  xf: activations [n][ldxf] in that
    // form (produced by the previous flagged forward; the prologue waits, bounded, per pair); y_flagged: y and
    // y_more point at such buffers (ldy in pairs).  epoch = (*flag_round << 8) | position in the chain of
    // dependent forwards: flag_seq for y, flag_seq - 1 for xf; the unpack that ends a chain advances the round.
    const unsigned long long *xf;
    size_t ldxf;
    bool y_flagged;
    const int *flag_round;
    int flag_seq;
    // the launch must not allocate: the medium-batch GEMM then never splits K (its scratch is created on first use)
    bool no_alloc;
};
// kernel choice for `n` tokens when the caller passes KB_PATH_AUTO: the dp4a GEMV for one or two
// tokens (up to four when it also has to quantise, which it does in its prologue), the
// small-batch MMA kernel up to 32 tokens while their activations fit in shared memory, the
// tensor-core GEMM above
int auto_path(const Linear *lin, size_t n, bool prequantised);
// small-batch kernel on the warp-level MMA (pre-quantised activations, up to 32 tokens)
bool gemv_mma_supports(const Linear *lin, size_t n);
int launch_gemv_mma(const FwdArgs &a, cudaStream_t stream);
// decode GEMV; when args.x is set the activation quantiser is fused into its prologue
int launch_gemv(const FwdArgs &a, cudaStream_t stream);
// streaming decode kernel (bulk-copy row pipeline + warp-level int8 MMA), up to 32 tokens;
// activations f32 (quantised in the prologue, up to 8 tokens) or pre-quantised
bool gemv_stream_supports(const Linear *lin, size_t n);
int launch_gemv_stream(const FwdArgs &a, cudaStream_t stream);
// the same kernel over `count` same-shaped layers, one token each (layer i reads row i of the inputs)
struct GroupArgs {
    const LayerRef *table;  // device, [count]
    int device, kind, mul, off;
    size_t count, m, k, kp, row_bytes;
    const float *x; size_t ldx;                                               // f32 inputs, or
    const int8_t *xq; size_t ldq; const float *sx; const int32_t *sumq;        // pre-quantised inputs
    float *y; size_t ldy;
    int *status;  // device word for a bounded wait that gave up (nullable)
};
int launch_group_stream(const GroupArgs &a, cudaStream_t stream);
// tcgen05 int8 GEMM; needs pre-quantised activations
int launch_gemm_tc(const FwdArgs &a, cudaStream_t stream);
// same contract, CTA-pair kernel (tcgen05 cta_group::2); chosen by launch_gemm_tc for large token counts
int launch_gemm_tc2(const FwdArgs &a, cudaStream_t stream);
// tcgen05 GEMM for up to 128 tokens with the unpacked weights in tensor memory
int launch_gemm_tcs(const FwdArgs &a, cudaStream_t stream);
// 2-D byte tensor map [rows][row_stride bytes] with box [box_inner bytes x box_rows]; SM count of a device
int encode_2d(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t rows, uint64_t row_stride, uint32_t box_inner,
              uint32_t box_rows, CUtensorMapSwizzle swz);
int sm_count(int device);
bool gemv_supports(const Linear *lin, size_t n);
bool gemm_tc_supports(const Linear *lin, size_t n);
int encode_weight_tmap(Linear *lin);

}  // namespace kb
