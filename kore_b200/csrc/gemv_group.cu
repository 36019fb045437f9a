// Grouped decode (sm_100a): one token through each of L independent layers of the same shape in
// ONE launch — y[l, :] = layer_l(x[l, :]).
//
// A 4 MiB layer streams in well under a microsecond, less than the launch, ramp-up and tail of
// any kernel, so launching such layers one by one (even on many streams) leaves a quarter of the
// HBM bandwidth unused.  Here the L layers form one virtual matrix of L * M rows that the streaming
// kernel (gemv_stream.cu) walks in 16-row blocks: every CTA owns a contiguous range of row blocks,
// its warps take them in turn, and each warp's copy pipeline runs across layer boundaries without
// draining.  Layer l reads token row l of the inputs — f32 rows that the kernel quantises in its
// prologue (per-token absmax -> int8, the quantiser kernel's arithmetic), or rows quantised
// beforehand by one kb_quantize_act_i8 call over the [L, K] matrix.
//
// This file holds the group object (a device table of its members' pointers, staging buffers of
// the host entry point) and the C entry points.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "device_utils.cuh"

namespace kb {

namespace {

constexpr uint32_t GROUP_MAGIC = 0x4b423247u;  // "KB2G"

struct Group {
    uint32_t magic;
    int device;
    int kind, mul, off;
    size_t count, m, k, kp, row_bytes;
    LayerRef *table;  // device, [count]
    // host entry point: device copies of x [count, k] and y [count, m]; one call at a time
    float *dx, *dy;
    int *status;  // device word: set when a bounded wait inside the launch gave up
    std::mutex host_mutex;
    // host entry point: streams of its pipeline (created on first use)
    static constexpr int HOST_STREAMS = 5;
    cudaStream_t hs[HOST_STREAMS] = {};
    cudaEvent_t launched[HOST_STREAMS] = {};  // a chunk's launch has finished
    int *h_status = nullptr;                  // pinned
    bool hs_ready = false;
};

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

// members [first, first + count) of the group: row i of x / y belongs to member first + i
int group_forward_range(const Group *G, size_t first, size_t count, const float *x, size_t ldx, const int8_t *xq, size_t ldq,
                        const float *sx, const int32_t *sumq, float *y, size_t ldy, cudaStream_t stream) {
    if (ldy == 0) ldy = G->m;
    if (ldy < G->m) return fail(KB_ERR_SHAPE, "shape mismatch: ldy %zu is smaller than out_features %zu", ldy, G->m);
    ScopedDevice dev(G->device);
    GroupArgs ga = {};
    ga.table = G->table + first; ga.device = G->device; ga.kind = G->kind; ga.mul = G->mul; ga.off = G->off;
    ga.count = count; ga.m = G->m; ga.k = G->k; ga.kp = G->kp; ga.row_bytes = G->row_bytes;
    ga.x = x; ga.ldx = ldx; ga.xq = xq; ga.ldq = ldq; ga.sx = sx; ga.sumq = sumq;
    ga.y = y; ga.ldy = ldy; ga.status = G->status;
    return launch_group_stream(ga, stream);
}

int group_forward(const Group *G, const float *x, size_t ldx, const int8_t *xq, size_t ldq, const float *sx,
                  const int32_t *sumq, float *y, size_t ldy, cudaStream_t stream) {
    return group_forward_range(G, 0, G->count, x, ldx, xq, ldq, sx, sumq, y, ldy, stream);
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
    const size_t row_blocks = (first->m + 15) / 16;
    if (count * row_blocks > (size_t)1 << 30) return fail(KB_ERR_UNSUPPORTED, "group too large: %zu layers of %zu rows", count, first->m);
    ScopedDevice dev(first->device);
    Group *G = new Group{};
    G->device = first->device;
    G->kind = first->kind; G->mul = first->mul; G->off = first->off;
    G->count = count; G->m = first->m; G->k = first->k; G->kp = first->kp; G->row_bytes = first->row_bytes;
    cudaError_t e = cudaMalloc(&G->table, count * sizeof(LayerRef));
    if (e == cudaSuccess) e = cudaMemcpy(G->table, host.data(), count * sizeof(LayerRef), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&G->dx, count * first->k * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&G->dy, count * first->m * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&G->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(G->status, 0, sizeof(int));
    if (e != cudaSuccess) {
        if (G->status) cudaFree(G->status);
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
    cudaFree(G->status);
    for (cudaStream_t st : G->hs)
        if (st) cudaStreamDestroy(st);
    for (cudaEvent_t ev : G->launched)
        if (ev) cudaEventDestroy(ev);
    if (G->h_status) cudaFreeHost(G->h_status);
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
    Group *G = const_cast<Group *>(Gc);  // the staging buffers and streams are the only state a call touches
    std::lock_guard<std::mutex> lock(G->host_mutex);
    ScopedDevice dev(G->device);
    cudaError_t e;
    if (!G->hs_ready) {
        for (int i = 0; i < Group::HOST_STREAMS; ++i) {
            if ((e = cudaStreamCreateWithFlags(&G->hs[i], cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e, "host pipeline stream");
            if ((e = cudaEventCreateWithFlags(&G->launched[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "host pipeline event");
        }
        if ((e = cudaHostAlloc(reinterpret_cast<void **>(&G->h_status), sizeof(int), cudaHostAllocDefault)) != cudaSuccess)
            return cuda_fail(e, "host pipeline status word");
        G->hs_ready = true;
    }
    // The members are independent, so the call is a pipeline over chunks of members, each on its own stream: upload,
    // grouped launch, download.  The launches keep the SMs busy back to back while the copy engines move the
    // neighbouring chunks (with pinned host buffers; pageable ones make the copies synchronous and the call
    // degenerates to the plain sequence).  A short first and last chunk keep the exposed upload and download short.
    size_t bounds[Group::HOST_STREAMS + 1];
    int chunks = 1;
    bounds[0] = 0;
    static const int env_chunks = [] { const char *v = getenv("KB_GROUP_HOST_CHUNKS"); return v && *v ? atoi(v) : 0; }();
    if (G->count >= 32 && env_chunks != 1) {
        // short chunks at both ends, the rest in equal parts (160 layers of 4096 x 4096, plain sequence / 3 / 4 / 5
        // chunks: 422 / 378 / 345 / 338 us on a host whose copies run at 17 GB/s, 294 / 237 / 266 / - us on one
        // with 30 GB/s; every further chunk adds host calls and copy set-ups)
        chunks = env_chunks >= 2 && env_chunks <= Group::HOST_STREAMS ? env_chunks : 4;
        const size_t edge = G->count / 10 < 8 ? 8 : G->count / 10;
        if (chunks == 2) {
            bounds[1] = G->count / 2;
        } else {
            bounds[1] = edge;
            const size_t mid = G->count - 2 * edge;
            for (int c = 2; c < chunks; ++c) bounds[c] = edge + mid * (size_t)(c - 1) / (size_t)(chunks - 2);
        }
    }
    bounds[chunks] = G->count;
    int rc = KB_OK;
    for (int c = 0; c < chunks && rc == KB_OK; ++c) {
        const size_t first = bounds[c], cnt = bounds[c + 1] - bounds[c];
        cudaStream_t st = G->hs[c];
        if ((e = cudaMemcpyAsync(G->dx + first * G->k, x + first * G->k, cnt * G->k * sizeof(float), cudaMemcpyHostToDevice, st)) != cudaSuccess)
            rc = cuda_fail(e, "activation upload");
        if (rc == KB_OK) rc = group_forward_range(G, first, cnt, G->dx + first * G->k, G->k, nullptr, 0, nullptr, nullptr, G->dy + first * G->m, G->m, st);
        if (rc == KB_OK && c + 1 < chunks && (e = cudaEventRecord(G->launched[c], st)) != cudaSuccess) rc = cuda_fail(e, "event record");
        if (rc == KB_OK && (e = cudaMemcpyAsync(y + first * G->m, G->dy + first * G->m, cnt * G->m * sizeof(float), cudaMemcpyDeviceToHost, st)) != cudaSuccess)
            rc = cuda_fail(e, "output download");
    }
    // the device status word, once, behind every chunk's launch
    *G->h_status = 0;
    if (rc == KB_OK) {
        cudaStream_t last = G->hs[chunks - 1];
        for (int c = 0; c + 1 < chunks && rc == KB_OK; ++c)
            if ((e = cudaStreamWaitEvent(last, G->launched[c], 0)) != cudaSuccess) rc = cuda_fail(e, "event wait");
        if (rc == KB_OK && (e = cudaMemcpyAsync(G->h_status, G->status, sizeof(int), cudaMemcpyDeviceToHost, last)) != cudaSuccess)
            rc = cuda_fail(e, "status download");
    }
    for (int c = 0; c < chunks; ++c) {
        e = cudaStreamSynchronize(G->hs[c]);
        if (rc == KB_OK && e != cudaSuccess) rc = cuda_fail(e, "stream synchronize");
    }
    const int status = *G->h_status;
    if (rc == KB_OK && status != 0) {
        cudaMemset(G->status, 0, sizeof(int));
        rc = fail(KB_ERR_TIMEOUT, "grouped launch gave up on a bounded wait (device code %d)", status);
    }
    return rc;
}

}  // extern "C"
