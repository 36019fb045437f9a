// extern "C" boundary of kore_b200 (see include/kore_b200.h).  Host logic only:
// argument checks in the wording of the KoreError they mirror, handle lifetime,
// workspace, kernel choice.  No arithmetic happens on the host.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <set>
#include <utility>

#include "common.cuh"

namespace kb {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(KB_ERR_CUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int dev) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != dev) {
            err = cudaSetDevice(dev);
            switched = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

int set_dyn_smem_once(const void *kernel, int device, int bytes, const char *what) {
    static std::mutex mu;
    static std::set<std::pair<const void *, int>> done;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair(kernel, device);
    if (done.count(key)) return KB_OK;
    DeviceGuard g(device);
    if (g.err != cudaSuccess) return cuda_fail(g.err, "cudaSetDevice");
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return cuda_fail(e, what);
    done.insert(key);
    return KB_OK;
}

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t wire_row_bytes(int kind, size_t k) { return kind == KB_TERNARY ? (k + 4) / 5 : (k + 3) / 4; }

static const Linear *check(const kb_linear *h) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) {
        fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
        return nullptr;
    }
    return L;
}

static void free_linear(Linear *L) {
    if (!L) return;
    DeviceGuard g(L->device);
    if (L->w2) cudaFree(L->w2);
    if (L->scales) cudaFree(L->scales);
    if (L->bias) cudaFree(L->bias);
    if (L->dev_status) cudaFree(L->dev_status);
    L->magic = 0;
    delete L;
}

// allocate the device-side containers of a layer (weights zeroed, scales unset)
static int alloc_linear(int kind, size_t m, size_t k, const float *bias, int device, Linear **out) {
    if (kind != KB_TERNARY && kind != KB_QUATERNARY) return fail(KB_ERR_INVALID, "unknown kind %d", kind);
    if (m == 0 || k == 0) return fail(KB_ERR_INVALID, "zero dimension: m=%zu k=%zu", m, k);
    if (m >= (1u << 30) || k >= (1u << 30)) return fail(KB_ERR_UNSUPPORTED, "dimension too large: m=%zu k=%zu", m, k);
    Linear *L = new (std::nothrow) Linear();
    if (!L) return fail(KB_ERR_CUDA, "host allocation failed");
    memset(L, 0, sizeof(*L));
    L->magic = HANDLE_MAGIC;
    L->kind = kind;
    L->device = device;
    L->m = m;
    L->k = k;
    L->kp = round_up(k, K_ALIGN);
    L->m_alloc = round_up(m, M_ALIGN);
    L->row_bytes = L->kp / 4;
    L->mul = kind == KB_TERNARY ? 1 : 2;
    L->off = kind == KB_TERNARY ? 1 : 3;
    cudaError_t e;
    if ((e = cudaMalloc(&L->w2, L->m_alloc * L->row_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&L->scales, L->m_alloc * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&L->dev_status, sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(L->dev_status, 0, sizeof(int))) != cudaSuccess) {
        free_linear(L);
        return cuda_fail(e, "weight allocation");
    }
    if (bias) {
        if ((e = cudaMalloc(&L->bias, L->m_alloc * sizeof(float))) != cudaSuccess ||
            (e = cudaMemset(L->bias, 0, L->m_alloc * sizeof(float))) != cudaSuccess ||
            (e = cudaMemcpy(L->bias, bias, m * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) {
            free_linear(L);
            return cuda_fail(e, "bias upload");
        }
    }
    *out = L;
    return KB_OK;
}

static size_t workspace_bytes(const Linear *L, size_t n) {
    return round_up(n * L->kp, 256) + 2 * round_up(n * 4, 256);
}

static int forward_impl(const Linear *L, const float *x, size_t n, size_t in_dim, float *y, size_t ldy,
                        int32_t *acc, int path, void *workspace, size_t ws_bytes, cudaStream_t stream,
                        int act = KB_ACT_NONE) {
    if (in_dim != L->k)
        return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got last dimension %zu", L->k, in_dim);
    if (!x || (!y && !acc)) return fail(KB_ERR_INVALID, "null activation or output pointer");
    if (ldy != 0 && ldy < L->m) return fail(KB_ERR_INVALID, "ldy %zu smaller than out_features %zu", ldy, L->m);
    if (act != KB_ACT_NONE && act != KB_ACT_RELU) return fail(KB_ERR_INVALID, "unknown activation %d", act);
    if (n == 0) return KB_OK;
    bool separate = false;  // quantise in a kernel of its own even where the forward kernel could do it
    if (path == KB_PATH_AUTO) {
        path = auto_path(L, n, false);
        // long rows, or several tokens of a large layer: every CTA of a fused launch would read and quantise all
        // the rows again in its prologue (8192 -> 28672, 2 / 4 tokens: 25.9 / 37.0 us fused against 20.2 / 20.9 us;
        // 28672 -> 8192, one token: 23.1 against 18.0 us); short rows of small layers stay fused (8192 -> 3584,
        // one / two tokens: 7.0 / 9.5 against 8.0 / 9.9 us)
        if (path == KB_PATH_GEMV && (L->kp >= 16384 || n * L->kp >= 32768 || (n >= 2 && L->m_alloc * L->row_bytes > ((size_t)16 << 20)))) {
            path = auto_path(L, n, true);
            separate = true;
        }
    }
    FwdArgs a = {};
    a.lin = L; a.n = n; a.y = y; a.acc = acc; a.ldy = ldy;
    a.relu = act == KB_ACT_RELU;
    if (path == KB_PATH_GEMV_SHARED) { a.shared_grid = true; path = KB_PATH_GEMV; }
    if (path == KB_PATH_GEMV && !separate) {
        a.x = x;
        return launch_gemv(a, stream);
    }
    if (path == KB_PATH_GEMV_STREAM && n <= 8 && !separate) {  // the quantiser runs in the kernel's prologue
        a.x = x;
        return launch_gemv_stream(a, stream);
    }
    if (path != KB_PATH_GEMM_TC && path != KB_PATH_GEMV_MMA && path != KB_PATH_GEMV_STREAM && path != KB_PATH_GEMV)
        return fail(KB_ERR_INVALID, "unknown path %d", path);
    const size_t need = workspace_bytes(L, n);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    bool own = false;
    if (!ws) {
        KB_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&ws), need, stream));
        own = true;
    } else if (ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255)) {
        return fail(KB_ERR_STORAGE, "workspace too small or misaligned: need %zu bytes (256-byte aligned), got %zu", need, ws_bytes);
    }
    int8_t *xq = reinterpret_cast<int8_t *>(ws);
    float *sx = reinterpret_cast<float *>(ws + round_up(n * L->kp, 256));
    int32_t *sumq = reinterpret_cast<int32_t *>(ws + round_up(n * L->kp, 256) + round_up(n * 4, 256));
    int rc = launch_act_quant(x, n, L->k, xq, L->kp, sx, sumq, stream);
    if (rc == KB_OK) {
        a.xq = xq; a.ldq = L->kp; a.sx = sx; a.sumq = sumq;
        rc = path == KB_PATH_GEMV_MMA ? launch_gemv_mma(a, stream)
             : (path == KB_PATH_GEMV_STREAM ? launch_gemv_stream(a, stream)
                : (path == KB_PATH_GEMV ? launch_gemv(a, stream) : launch_gemm_tc(a, stream)));
    }
    if (own) {
        cudaError_t e = cudaFreeAsync(ws, stream);
        if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "workspace free");
    }
    return rc;
}

// Per-thread device staging for the host-pointer entry point: grown on demand, reused by
// later calls of the same thread, released when the thread ends.
struct HostStaging {
    int device = -1;
    void *dx = nullptr, *dy = nullptr, *ws = nullptr;
    void *hy = nullptr;  // pinned twin of dy: a device -> pageable copy would be staged by the driver anyway
    size_t dx_cap = 0, dy_cap = 0, ws_cap = 0;
    ~HostStaging() { release(); }
    void release() {
        if (dx) cudaFree(dx);
        if (dy) cudaFree(dy);
        if (ws) cudaFree(ws);
        if (hy) cudaFreeHost(hy);
        dx = dy = hy = ws = nullptr;
        dx_cap = dy_cap = ws_cap = 0;
    }
    int ensure(int dev, size_t xb, size_t yb, size_t wsb) {
        if (dev != device) { release(); device = dev; }
        if (wsb > ws_cap) {  // quantised activations of the multi-token kernels
            if (ws) cudaFree(ws);
            ws = nullptr; ws_cap = 0;
            cudaError_t e = cudaMalloc(&ws, wsb);
            if (e != cudaSuccess) return cuda_fail(e, "workspace staging");
            ws_cap = wsb;
        }
        if (xb > dx_cap) {
            if (dx) cudaFree(dx);
            dx = nullptr; dx_cap = 0;
            cudaError_t e = cudaMalloc(&dx, xb);
            if (e != cudaSuccess) return cuda_fail(e, "activation staging");
            dx_cap = xb;
        }
        if (yb > dy_cap) {
            if (dy) cudaFree(dy);
            if (hy) cudaFreeHost(hy);
            dy = hy = nullptr; dy_cap = 0;
            cudaError_t e = cudaMalloc(&dy, yb);
            if (e != cudaSuccess) return cuda_fail(e, "output staging");
            // small results come back through pinned memory; large ones go straight to the caller
            if (yb <= (4u << 20) && cudaHostAlloc(&hy, yb, cudaHostAllocDefault) != cudaSuccess) { hy = nullptr; cudaGetLastError(); }
            dy_cap = yb;
        }
        return KB_OK;
    }
};
static thread_local HostStaging g_staging;

// x [n,k] host -> y [n,m] host, on this thread's private stream
static int forward_host_impl(const Linear *L, const float *x, size_t n, size_t in_dim, float *y) {
    if (in_dim != L->k)
        return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got last dimension %zu", L->k, in_dim);
    if (!x || !y) return fail(KB_ERR_INVALID, "null activation or output pointer");
    if (n == 0) return KB_OK;
    cudaStream_t st = cudaStreamPerThread;
    int rc = g_staging.ensure(L->device, n * L->k * sizeof(float), n * L->m * sizeof(float), workspace_bytes(L, n));
    if (rc) return rc;
    float *dx = static_cast<float *>(g_staging.dx), *dy = static_cast<float *>(g_staging.dy);
    cudaError_t e;
    if ((e = cudaMemcpyAsync(dx, x, n * L->k * sizeof(float), cudaMemcpyHostToDevice, st)) != cudaSuccess)
        rc = cuda_fail(e, "activation upload");
    if (rc == KB_OK) rc = forward_impl(L, dx, n, in_dim, dy, 0, nullptr, KB_PATH_AUTO, g_staging.ws, g_staging.ws_cap, st);
    const size_t yb = n * L->m * sizeof(float);
    void *landing = (g_staging.hy && yb <= (4u << 20)) ? g_staging.hy : static_cast<void *>(y);
    if (rc == KB_OK && (e = cudaMemcpyAsync(landing, dy, yb, cudaMemcpyDeviceToHost, st)) != cudaSuccess)
        rc = cuda_fail(e, "output download");
    e = cudaStreamSynchronize(st);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "stream synchronize");
    if (rc == KB_OK && landing != y) memcpy(y, landing, yb);
    return rc;
}

static int create_from_wire(int kind, const uint8_t *packed, size_t packed_len, const float *scales,
                            size_t scales_len, const float *bias, size_t m, size_t k, int device,
                            Linear **out) {
    if (!packed || !scales || !out) return fail(KB_ERR_INVALID, "null pointer");
    if (kind != KB_TERNARY && kind != KB_QUATERNARY) return fail(KB_ERR_INVALID, "unknown kind %d", kind);
    const size_t need = m * wire_row_bytes(kind, k);
    if (packed_len < need)
        return fail(KB_ERR_STORAGE, "a_packed too small: need %zu bytes, got %zu", need, packed_len);
    if (scales_len < m) return fail(KB_ERR_STORAGE, "a_scales too small: need %zu, got %zu", m, scales_len);
    DeviceGuard g(device);
    if (g.err != cudaSuccess) return cuda_fail(g.err, "cudaSetDevice");
    Linear *L = nullptr;
    int rc = alloc_linear(kind, m, k, bias, device, &L);
    if (rc) return rc;
    uint8_t *dwire = nullptr;
    cudaError_t e;
    if ((e = cudaMalloc(&dwire, need)) != cudaSuccess) { free_linear(L); return cuda_fail(e, "wire staging"); }
    if ((e = cudaMemcpy(dwire, packed, need, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemset(L->scales, 0, L->m_alloc * sizeof(float))) != cudaSuccess ||
        (e = cudaMemcpy(L->scales, scales, m * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) {
        cudaFree(dwire); free_linear(L);
        return cuda_fail(e, "weight upload");
    }
    rc = launch_repack_wire(kind, dwire, m, k, L->w2, L->row_bytes, L->m_alloc, 0);
    e = cudaDeviceSynchronize();
    cudaFree(dwire);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "repack");
    if (rc == KB_OK) rc = encode_weight_tmap(L);
    if (rc) { free_linear(L); return rc; }
    *out = L;
    return KB_OK;
}

static int create_from_f32(int kind, int quantiser, const float *w, const float *bias, size_t m, size_t k,
                           float threshold, int device, Linear **out) {
    if (!w || !out) return fail(KB_ERR_INVALID, "null pointer");
    if (kind != KB_TERNARY && kind != KB_QUATERNARY) return fail(KB_ERR_INVALID, "unknown kind %d", kind);
    if (quantiser != KB_QUANT_REFERENCE && !(quantiser == KB_QUANT_ABSMEAN && kind == KB_TERNARY))
        return fail(KB_ERR_INVALID, "quantiser %d not defined for kind %d", quantiser, kind);
    DeviceGuard g(device);
    if (g.err != cudaSuccess) return cuda_fail(g.err, "cudaSetDevice");
    Linear *L = nullptr;
    int rc = alloc_linear(kind, m, k, bias, device, &L);
    if (rc) return rc;
    float *dw = nullptr;
    cudaError_t e;
    if ((e = cudaMalloc(&dw, m * k * sizeof(float))) != cudaSuccess) { free_linear(L); return cuda_fail(e, "f32 weight staging"); }
    if ((e = cudaMemcpy(dw, w, m * k * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) {
        cudaFree(dw); free_linear(L);
        return cuda_fail(e, "weight upload");
    }
    rc = launch_quantise_f32(kind, quantiser, dw, m, k, threshold, L->w2, L->row_bytes, L->m_alloc, L->scales, 0);
    e = cudaDeviceSynchronize();
    cudaFree(dw);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "quantise");
    if (rc == KB_OK) rc = encode_weight_tmap(L);
    if (rc) { free_linear(L); return rc; }
    *out = L;
    return KB_OK;
}

// reference-shaped one-shot: b [K,N] host -> c [M,N] host
static int one_shot(int kind, const uint8_t *a_packed, size_t a_len, const float *a_scales, size_t scales_len,
                    const float *b, float *c, size_t m, size_t n, size_t k, const float *bias = nullptr,
                    int act = KB_ACT_NONE) {
    if (!b || !c) return fail(KB_ERR_INVALID, "null pointer");
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    Linear *L = nullptr;
    int rc = create_from_wire(kind, a_packed, a_len, a_scales, scales_len, bias, m, k, device, &L);
    if (rc) return rc;
    if (n == 0) { free_linear(L); return KB_OK; }
    cudaStream_t st = cudaStreamPerThread;
    float *db = nullptr, *dx = nullptr, *dy = nullptr, *dc = nullptr;
    const size_t xb = n * k * sizeof(float), yb = n * m * sizeof(float);
    if ((e = cudaMalloc(&db, xb)) != cudaSuccess || (e = cudaMalloc(&dx, xb)) != cudaSuccess ||
        (e = cudaMalloc(&dy, yb)) != cudaSuccess || (e = cudaMalloc(&dc, yb)) != cudaSuccess) {
        rc = cuda_fail(e, "one-shot allocation");
    }
    if (rc == KB_OK && (e = cudaMemcpyAsync(db, b, xb, cudaMemcpyHostToDevice, st)) != cudaSuccess) rc = cuda_fail(e, "b upload");
    if (rc == KB_OK) rc = launch_transpose_f32(db, k, n, dx, st);  // [K,N] -> [N,K]
    if (rc == KB_OK) rc = forward_impl(L, dx, n, k, dy, 0, nullptr, KB_PATH_AUTO, nullptr, 0, st, act);
    if (rc == KB_OK) rc = launch_transpose_f32(dy, n, m, dc, st);  // [N,M] -> [M,N]
    if (rc == KB_OK && (e = cudaMemcpyAsync(c, dc, yb, cudaMemcpyDeviceToHost, st)) != cudaSuccess) rc = cuda_fail(e, "c download");
    e = cudaStreamSynchronize(st);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "stream synchronize");
    cudaFree(db); cudaFree(dx); cudaFree(dy); cudaFree(dc);
    free_linear(L);
    return rc;
}

// C[M,N] = (sum_k a[m,k] * b[n,k]) * a_scale[m] * b_scale[n], both operands base-243 rows: B's
// trits take the place of the int8 activations (scale b_scale[n], code sum = sum of trits), so
// the integer accumulation and the two separately rounded multiplies are the forward path's own.
static int ternary_ternary(const uint8_t *a_packed, size_t a_len, const float *a_scales, const uint8_t *b_packed,
                           size_t b_len, const float *b_scales, float *c, size_t m, size_t n, size_t k) {
    if (!a_packed || !a_scales || !b_packed || !b_scales || !c) return fail(KB_ERR_INVALID, "null pointer");
    const size_t kpw = (k + 4) / 5;
    if (a_len < m * kpw || b_len < n * kpw) return fail(KB_ERR_STORAGE, "packed arrays too small");
    if (m == 0 || n == 0) return KB_OK;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    Linear *L = nullptr;
    int rc = create_from_wire(KB_TERNARY, a_packed, a_len, a_scales, m, nullptr, m, k, device, &L);
    if (rc) return rc;
    cudaStream_t st = cudaStreamPerThread;
    uint8_t *dwire = nullptr;
    int8_t *xq = nullptr;
    float *sx = nullptr, *dy = nullptr, *dc = nullptr;
    int32_t *sumq = nullptr;
    const size_t yb = n * m * sizeof(float);
    if ((e = cudaMalloc(&dwire, n * kpw)) != cudaSuccess || (e = cudaMalloc(&xq, n * L->kp)) != cudaSuccess ||
        (e = cudaMalloc(&sx, n * sizeof(float))) != cudaSuccess || (e = cudaMalloc(&sumq, n * sizeof(int32_t))) != cudaSuccess ||
        (e = cudaMalloc(&dy, yb)) != cudaSuccess || (e = cudaMalloc(&dc, yb)) != cudaSuccess)
        rc = cuda_fail(e, "one-shot allocation");
    if (rc == KB_OK && (e = cudaMemcpyAsync(dwire, b_packed, n * kpw, cudaMemcpyHostToDevice, st)) != cudaSuccess) rc = cuda_fail(e, "b upload");
    if (rc == KB_OK && (e = cudaMemcpyAsync(sx, b_scales, n * sizeof(float), cudaMemcpyHostToDevice, st)) != cudaSuccess) rc = cuda_fail(e, "scale upload");
    if (rc == KB_OK) rc = launch_decode_trits_i8(dwire, n, k, xq, L->kp, sumq, st);
    if (rc == KB_OK) {
        FwdArgs a = {};
        a.lin = L; a.xq = xq; a.ldq = L->kp; a.sx = sx; a.sumq = sumq; a.n = n; a.y = dy; a.ldy = 0;
        const int path = auto_path(L, n, true);
        rc = path == KB_PATH_GEMV ? launch_gemv(a, st)
             : (path == KB_PATH_GEMV_MMA ? launch_gemv_mma(a, st)
                : (path == KB_PATH_GEMV_STREAM ? launch_gemv_stream(a, st) : launch_gemm_tc(a, st)));
    }
    if (rc == KB_OK) rc = launch_transpose_f32(dy, n, m, dc, st);  // [N,M] -> [M,N]
    if (rc == KB_OK && (e = cudaMemcpyAsync(c, dc, yb, cudaMemcpyDeviceToHost, st)) != cudaSuccess) rc = cuda_fail(e, "c download");
    e = cudaStreamSynchronize(st);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "stream synchronize");
    cudaFree(dwire); cudaFree(xq); cudaFree(sx); cudaFree(sumq); cudaFree(dy); cudaFree(dc);
    free_linear(L);
    return rc;
}

static int pack_weights(int kind, const float *w, size_t m, size_t k, float threshold, uint8_t *packed,
                        size_t packed_len, float *scales, size_t scales_len, int device) {
    if (!w || !packed || !scales) return fail(KB_ERR_INVALID, "null pointer");
    const size_t need = m * wire_row_bytes(kind, k);
    if (packed_len < need) return fail(KB_ERR_STORAGE, "packed too small: need %zu bytes, got %zu", need, packed_len);
    if (scales_len < m) return fail(KB_ERR_STORAGE, "scales too small: need %zu, got %zu", m, scales_len);
    Linear *L = nullptr;
    int rc = create_from_f32(kind, KB_QUANT_REFERENCE, w, nullptr, m, k, threshold, device, &L);
    if (rc) return rc;
    rc = kb_linear_packed_weights(reinterpret_cast<kb_linear *>(L), packed, packed_len);
    if (rc == KB_OK) rc = kb_linear_scales(reinterpret_cast<kb_linear *>(L), scales, scales_len);
    free_linear(L);
    return rc;
}

}  // namespace kb

using namespace kb;

extern "C" {

const char *kb_version(void) { return "kore_b200 0.1.0 (sm_100a)"; }
const char *kb_last_error(void) { return g_err; }

int kb_device_count(int *count) {
    if (!count) return fail(KB_ERR_INVALID, "null pointer");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) { *count = 0; return cuda_fail(e, "cudaGetDeviceCount"); }
    return KB_OK;
}

int kb_linear_create_from_ref_packed(int kind, const uint8_t *packed, size_t packed_len, const float *scales,
                                     size_t scales_len, const float *bias, size_t m, size_t k, int device,
                                     kb_linear **out) {
    if (out) *out = nullptr;
    Linear *L = nullptr;
    int rc = create_from_wire(kind, packed, packed_len, scales, scales_len, bias, m, k, device, &L);
    if (rc == KB_OK) *out = reinterpret_cast<kb_linear *>(L);
    return rc;
}

int kb_linear_create_from_f32(int kind, int quantiser, const float *w, const float *bias, size_t m, size_t k,
                              float threshold, int device, kb_linear **out) {
    if (out) *out = nullptr;
    Linear *L = nullptr;
    int rc = create_from_f32(kind, quantiser, w, bias, m, k, threshold, device, &L);
    if (rc == KB_OK) *out = reinterpret_cast<kb_linear *>(L);
    return rc;
}

void kb_linear_destroy(kb_linear *h) {
    Linear *L = reinterpret_cast<Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return;
    free_linear(L);
}

int kb_linear_info(const kb_linear *h, size_t *m, size_t *k, int *kind, int *device, size_t *weight_bytes) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (m) *m = L->m;
    if (k) *k = L->k;
    if (kind) *kind = L->kind;
    if (device) *device = L->device;
    if (weight_bytes) *weight_bytes = L->m * wire_row_bytes(L->kind, L->k) + 4 * L->m;
    return KB_OK;
}

int kb_linear_scales(const kb_linear *h, float *scales, size_t scales_len) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!scales) return fail(KB_ERR_INVALID, "null pointer");
    if (scales_len < L->m) return fail(KB_ERR_STORAGE, "scales too small: need %zu, got %zu", L->m, scales_len);
    DeviceGuard g(L->device);
    KB_CUDA(cudaMemcpy(scales, L->scales, L->m * sizeof(float), cudaMemcpyDeviceToHost));
    return KB_OK;
}

int kb_linear_packed_weights(const kb_linear *h, uint8_t *packed, size_t packed_len) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!packed) return fail(KB_ERR_INVALID, "null pointer");
    const size_t need = L->m * wire_row_bytes(L->kind, L->k);
    if (packed_len < need) return fail(KB_ERR_STORAGE, "packed too small: need %zu bytes, got %zu", need, packed_len);
    DeviceGuard g(L->device);
    uint8_t *d = nullptr;
    KB_CUDA(cudaMalloc(&d, need));
    int rc = launch_export_wire(L->kind, L->w2, L->row_bytes, L->m, L->k, d, 0);
    cudaError_t e = cudaMemcpy(packed, d, need, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "wire download");
    return rc;
}

int kb_linear_dequantize_weights(const kb_linear *h, float *w, size_t w_len) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!w) return fail(KB_ERR_INVALID, "null pointer");
    if (w_len < L->m * L->k) return fail(KB_ERR_STORAGE, "w too small: need %zu, got %zu", L->m * L->k, w_len);
    DeviceGuard g(L->device);
    float *d = nullptr;
    KB_CUDA(cudaMalloc(&d, L->m * L->k * sizeof(float)));
    int rc = launch_dequantize(L->kind, L->w2, L->row_bytes, L->scales, L->m, L->k, d, 0);
    cudaError_t e = cudaMemcpy(w, d, L->m * L->k * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "weight download");
    return rc;
}

size_t kb_act_ld(size_t k) { return round_up(k, K_ALIGN); }

int kb_quantize_act_i8(const float *x, size_t n, size_t k, int8_t *xq, size_t ldq, float *sx, int32_t *sumq,
                       kb_stream stream) {
    if (!x || !xq || !sx) return fail(KB_ERR_INVALID, "null pointer");
    if (k == 0) return fail(KB_ERR_INVALID, "zero dimension: k=0");
    if (ldq < k || ldq % 16 || (reinterpret_cast<uintptr_t>(xq) & 15))
        return fail(KB_ERR_INVALID, "xq must be 16-byte aligned with ldq >= k and ldq %% 16 == 0 (ldq=%zu, k=%zu)", ldq, k);
    return launch_act_quant(x, n, k, xq, ldq, sx, sumq, static_cast<cudaStream_t>(stream));
}

int kb_linear_forward(const kb_linear *h, const float *x, size_t n, float *y, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    DeviceGuard g(L->device);
    return forward_impl(L, x, n, L->k, y, 0, nullptr, KB_PATH_AUTO, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int kb_linear_forward_ex(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y, size_t ldy,
                         int32_t *acc, int path, void *workspace, size_t workspace_bytes_, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    DeviceGuard g(L->device);
    return forward_impl(L, x, n, in_dim, y, ldy, acc, path, workspace, workspace_bytes_,
                        static_cast<cudaStream_t>(stream));
}

int kb_linear_forward_act(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y, size_t ldy, int act,
                          int path, void *workspace, size_t workspace_bytes_, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    DeviceGuard g(L->device);
    return forward_impl(L, x, n, in_dim, y, ldy, nullptr, path, workspace, workspace_bytes_,
                        static_cast<cudaStream_t>(stream), act);
}

size_t kb_linear_workspace_bytes(const kb_linear *h, size_t n) {
    const Linear *L = check(h);
    return L ? workspace_bytes(L, n) : 0;
}

int kb_linear_forward_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx, const int32_t *sumq,
                         size_t n, float *y, size_t ldy, int32_t *acc, int path, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!xq || !sx || !sumq || (!y && !acc)) return fail(KB_ERR_INVALID, "null pointer");
    if (ldy != 0 && ldy < L->m) return fail(KB_ERR_INVALID, "ldy %zu smaller than out_features %zu", ldy, L->m);
    if (n == 0) return KB_OK;
    DeviceGuard g(L->device);
    if (path == KB_PATH_AUTO) path = auto_path(L, n, true);
    FwdArgs a = {};
    a.lin = L; a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq; a.n = n; a.y = y; a.acc = acc; a.ldy = ldy;
    if (path == KB_PATH_GEMV_SHARED) { a.shared_grid = true; path = KB_PATH_GEMV; }
    if (path == KB_PATH_GEMV) return launch_gemv(a, static_cast<cudaStream_t>(stream));
    if (path == KB_PATH_GEMV_MMA) return launch_gemv_mma(a, static_cast<cudaStream_t>(stream));
    if (path == KB_PATH_GEMV_STREAM) return launch_gemv_stream(a, static_cast<cudaStream_t>(stream));
    if (path == KB_PATH_GEMM_TC) return launch_gemm_tc(a, static_cast<cudaStream_t>(stream));
    return fail(KB_ERR_INVALID, "unknown path %d", path);
}

int kb_linear_forward_fused(const kb_linear *h, const float *x, const int8_t *xq, size_t ldq, const float *sx,
                            const int32_t *sumq, size_t n, const float *resid, float *y, size_t ldy, int path,
                            void *workspace, size_t workspace_bytes_, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!y || (!x && !(xq && sx && sumq))) return fail(KB_ERR_INVALID, "null pointer");
    if (ldy != 0 && ldy < L->m) return fail(KB_ERR_INVALID, "ldy %zu smaller than out_features %zu", ldy, L->m);
    if (n == 0) return KB_OK;
    DeviceGuard g(L->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (path == KB_PATH_AUTO) path = auto_path(L, n, xq != nullptr);
    FwdArgs a = {};
    a.lin = L; a.n = n; a.y = y; a.ldy = ldy; a.resid = resid;
    if (path == KB_PATH_GEMV_SHARED) { a.shared_grid = true; path = KB_PATH_GEMV; }
    if (xq) {
        a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq;
        if (path == KB_PATH_GEMV) return launch_gemv(a, st);
        if (path == KB_PATH_GEMV_MMA) return launch_gemv_mma(a, st);
        if (path == KB_PATH_GEMV_STREAM) return launch_gemv_stream(a, st);
        if (path == KB_PATH_GEMM_TC) return launch_gemm_tc(a, st);
        return fail(KB_ERR_INVALID, "unknown path %d", path);
    }
    if (path == KB_PATH_GEMV) {
        a.x = x;
        return launch_gemv(a, st);
    }
    if (path == KB_PATH_GEMV_STREAM && n <= 8) {
        a.x = x;
        return launch_gemv_stream(a, st);
    }
    if (path != KB_PATH_GEMM_TC && path != KB_PATH_GEMV_MMA && path != KB_PATH_GEMV_STREAM)
        return fail(KB_ERR_INVALID, "unknown path %d", path);
    const size_t need = workspace_bytes(L, n);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    if (!ws || workspace_bytes_ < need || (reinterpret_cast<uintptr_t>(ws) & 255))
        return fail(KB_ERR_STORAGE, "workspace too small or misaligned: need %zu bytes (256-byte aligned), got %zu", need,
                    workspace_bytes_);
    int8_t *wq = reinterpret_cast<int8_t *>(ws);
    float *wsx = reinterpret_cast<float *>(ws + round_up(n * L->kp, 256));
    int32_t *wsum = reinterpret_cast<int32_t *>(ws + round_up(n * L->kp, 256) + round_up(n * 4, 256));
    int rc = launch_act_quant(x, n, L->k, wq, L->kp, wsx, wsum, st);
    if (rc) return rc;
    a.xq = wq; a.ldq = L->kp; a.sx = wsx; a.sumq = wsum;
    return path == KB_PATH_GEMV_MMA ? launch_gemv_mma(a, st)
           : (path == KB_PATH_GEMV_STREAM ? launch_gemv_stream(a, st) : launch_gemm_tc(a, st));
}

int kb_linear_forward_rmsnorm(const kb_linear *h, const float *x, const float *gamma, float eps, size_t n, float *y,
                              size_t ldy, int swiglu, float *absmax_out, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!x || !gamma || !y) return fail(KB_ERR_INVALID, "null pointer");
    if (n == 0) return KB_OK;
    const size_t width = swiglu ? L->m / 2 : L->m;
    if (ldy != 0 && ldy < width) return fail(KB_ERR_INVALID, "ldy %zu smaller than the output width %zu", ldy, width);
    if (n > (swiglu ? 2u : 8u) || !gemv_supports(L, n))
        return fail(KB_ERR_UNSUPPORTED, "the fused RMSNorm projection takes up to %d tokens", swiglu ? 2 : 8);
    DeviceGuard g(L->device);
    FwdArgs a = {};
    a.lin = L; a.x = x; a.n = n; a.y = y; a.ldy = ldy;
    a.gamma = gamma; a.eps = eps; a.swiglu = swiglu != 0; a.absmax_out = absmax_out;
    return launch_gemv(a, static_cast<cudaStream_t>(stream));
}

int kb_linear_forward_scaled(const kb_linear *h, const float *x, const float *x_absmax, size_t n, const float *resid,
                             float *y, size_t ldy, float *clear_word, kb_stream stream) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!x || !x_absmax || !y) return fail(KB_ERR_INVALID, "null pointer");
    if (n == 0) return KB_OK;
    if (ldy != 0 && ldy < L->m) return fail(KB_ERR_INVALID, "ldy %zu smaller than out_features %zu", ldy, L->m);
    if (n > 8 || !gemv_supports(L, n)) return fail(KB_ERR_UNSUPPORTED, "the pre-scaled projection takes up to 8 tokens");
    DeviceGuard g(L->device);
    FwdArgs a = {};
    a.lin = L; a.x = x; a.n = n; a.y = y; a.ldy = ldy; a.resid = resid;
    a.x_absmax = x_absmax; a.clear_word = clear_word;
    return launch_gemv(a, static_cast<cudaStream_t>(stream));
}

int kb_linear_forward_host(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *y) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    DeviceGuard g(L->device);
    return forward_host_impl(L, x, n, in_dim, y);
}

int kb_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales, size_t scales_len,
                      const float *b, float *c, size_t m, size_t n, size_t k) {
    return one_shot(KB_TERNARY, a_packed, a_len, a_scales, scales_len, b, c, m, n, k);
}

int kb_ternary_ternary_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales, const uint8_t *b_packed,
                              size_t b_len, const float *b_scales, float *c, size_t m, size_t n, size_t k) {
    return ternary_ternary(a_packed, a_len, a_scales, b_packed, b_len, b_scales, c, m, n, k);
}

int kb_quat_matmul(const uint8_t *a_packed, size_t a_len, const float *a_scales, size_t scales_len, const float *b,
                   float *c, size_t m, size_t n, size_t k) {
    return one_shot(KB_QUATERNARY, a_packed, a_len, a_scales, scales_len, b, c, m, n, k);
}

int kb_quat_matmul_bias_relu(const uint8_t *a_packed, size_t a_len, const float *a_scales, size_t scales_len,
                             const float *b, const float *bias, size_t bias_len, float *c, size_t m, size_t n, size_t k) {
    if (!bias) return fail(KB_ERR_INVALID, "null pointer");
    if (bias_len < m) return fail(KB_ERR_STORAGE, "bias too small: need %zu, got %zu", m, bias_len);
    return one_shot(KB_QUATERNARY, a_packed, a_len, a_scales, scales_len, b, c, m, n, k, bias, KB_ACT_RELU);
}

int kb_pack_weights_ternary(const float *w, size_t m, size_t k, float threshold, uint8_t *packed, size_t packed_len,
                            float *scales, size_t scales_len, int device) {
    return pack_weights(KB_TERNARY, w, m, k, threshold, packed, packed_len, scales, scales_len, device);
}

int kb_pack_weights_quaternary(const float *w, size_t m, size_t k, uint8_t *packed, size_t packed_len,
                               float *scales, size_t scales_len, int device) {
    return pack_weights(KB_QUATERNARY, w, m, k, 0.0f, packed, packed_len, scales, scales_len, device);
}

int kb_linear_device_ptrs(const kb_linear *h, const void **w2, size_t *row_bytes, const float **scales,
                          const float **bias) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (w2) *w2 = L->w2;
    if (row_bytes) *row_bytes = L->row_bytes;
    if (scales) *scales = L->scales;
    if (bias) *bias = L->bias;
    return KB_OK;
}

int kb_linear_last_device_status(const kb_linear *h, kb_stream stream, int *status) {
    const Linear *L = check(h);
    if (!L) return KB_ERR_BAD_HANDLE;
    if (!status) return fail(KB_ERR_INVALID, "null pointer");
    DeviceGuard g(L->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KB_CUDA(cudaMemcpyAsync(status, L->dev_status, sizeof(int), cudaMemcpyDeviceToHost, st));
    KB_CUDA(cudaStreamSynchronize(st));
    if (*status != 0) {
        KB_CUDA(cudaMemsetAsync(L->dev_status, 0, sizeof(int), st));
        KB_CUDA(cudaStreamSynchronize(st));
        return fail(KB_ERR_TIMEOUT, "tcgen05 GEMM gave up on a bounded wait (device code %d)", *status);
    }
    return KB_OK;
}

}  // extern "C"
