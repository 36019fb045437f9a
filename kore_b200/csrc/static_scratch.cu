// kb_linear_forward_static: the forward pass for callers that must not allocate.
//
// Who needs it: code that runs where device-memory allocation is forbidden or
// unaffordable — a real-time inference loop that promised a fixed memory footprint, a
// plugin loaded into a host process whose allocator owns the whole GPU, a section of a
// serving engine that runs after its memory pool has been frozen.  The regular forward
// quantises the activations into a scratch buffer it obtains from the stream-ordered
// allocator (or from the caller); this variant keeps that scratch in a fixed array that
// is part of the library image, so the call itself never allocates or frees anything.
//
// Cost and limits: every GPU that loads the library carries the array
// (KB_STATIC_SCRATCH_BYTES, 1 MiB) until the process exits.  A call whose quantised
// activations do not fit is rejected with KB_ERR_UNSUPPORTED.  All calls on one device
// share the array, which still holds whatever the previous call left there: each call
// rewrites every byte it later reads (codes, zero padding, scales, sums), so nothing
// needs clearing, but two calls that overlap in time on the GPU (different streams, or
// different host threads) corrupt each other — serialise them.
//
// The array's name is only a host-side stand-in for the device object, not an address a
// kernel can use.  The first call on each device therefore looks the address up with
// cudaGetSymbolAddress (device made current first, return code checked) and caches it;
// later calls reuse the cached pointer.  The first launch of each kernel the call can pick
// (by token count: 1, 2, 3..4, 5..8, 9..128, 129..256, above 256) additionally loads that kernel and
// sets its shared-memory limit.  Make one warm-up call per token-count class in use during
// set-up, before any stream capture begins and before the memory budget is frozen.
#include <mutex>

#include "common.cuh"

namespace kb {

constexpr size_t STATIC_SCRATCH_BYTES = 1u << 20;
static __device__ __align__(256) uint8_t g_static_scratch[STATIC_SCRATCH_BYTES];

static std::mutex g_scratch_mutex;
static uint8_t *g_scratch_ptr[64] = {nullptr};

// device address of g_static_scratch on `device` (which must be current)
static int static_scratch_address(int device, uint8_t **out) {
    if (device < 0 || device >= 64) return fail(KB_ERR_UNSUPPORTED, "device index %d outside 0..63", device);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255))
            return fail(KB_ERR_CUDA, "static scratch address %p is null or not 256-byte aligned", p);
        g_scratch_ptr[device] = static_cast<uint8_t *>(p);
    }
    *out = g_scratch_ptr[device];
    return KB_OK;
}

static size_t round_up_256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace kb

using namespace kb;

extern "C" size_t kb_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int kb_linear_forward_static(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y,
                                        kb_stream stream) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (in_dim != L->k)
        return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got last dimension %zu", L->k, in_dim);
    if (!x || !y) return fail(KB_ERR_INVALID, "null activation or output pointer");
    if (n == 0) return KB_OK;
    const size_t xq_bytes = round_up_256(n * L->kp), vec_bytes = round_up_256(n * 4);
    const size_t need = xq_bytes + 2 * vec_bytes;
    if (need > STATIC_SCRATCH_BYTES)
        return fail(KB_ERR_UNSUPPORTED,
                    "static scratch too small: %zu tokens x %zu padded features need %zu bytes, the fixed array holds %zu",
                    n, L->kp, need, STATIC_SCRATCH_BYTES);
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != L->device && (e = cudaSetDevice(L->device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    uint8_t *ws = nullptr;
    int rc = static_scratch_address(L->device, &ws);
    if (rc == KB_OK) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        int8_t *xq = reinterpret_cast<int8_t *>(ws);
        float *sx = reinterpret_cast<float *>(ws + xq_bytes);
        int32_t *sumq = reinterpret_cast<int32_t *>(ws + xq_bytes + vec_bytes);
        rc = launch_act_quant(x, n, L->k, xq, L->kp, sx, sumq, st);
        if (rc == KB_OK) {
            FwdArgs a = {};
            a.lin = L; a.xq = xq; a.ldq = L->kp; a.sx = sx; a.sumq = sumq; a.n = n; a.y = y; a.ldy = 0;
            a.no_alloc = true;  // no K split in the medium-batch GEMM: its scratch buffer would be an allocation
            rc = (n <= 8 && gemv_supports(L, n)) ? launch_gemv(a, st) : launch_gemm_tc(a, st);
        }
    }
    if (prev != L->device) cudaSetDevice(prev);
    return rc;
}
