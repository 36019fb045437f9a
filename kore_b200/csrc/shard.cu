// Column-sharded forward across the GPUs of one NVSwitch box (one process per GPU).
//
// Output features are independent, so rank r owns weight rows [r*M/g, (r+1)*M/g) and
// every rank needs the full y[N, M].  Instead of computing a slice and then calling a
// collective, the GEMV / GEMM epilogue stores each output value into every rank's copy
// of y (local store + peer stores over NVLink, plain st.global to peer-mapped memory),
// so the exchange overlaps the kernel tile by tile.  A small barrier kernel then tells
// the peers that this rank's slice has landed and waits until theirs have.
//
// Peer buffers are cudaMalloc allocations exchanged as CUDA IPC handles (the host layer
// moves the 64-byte handles with torch.distributed).  No cluster multicast, no multimem:
// ordinary peer loads and stores only.
#include <cstring>

#include "common.cuh"

namespace kb {

// Every rank runs one CTA.  The epoch is a device-side counter bumped by each barrier, so
// the same captured launch can be replayed from a CUDA graph (all ranks run the same
// sequence of barriers, hence agree on the epoch).  Thread j < world publishes the epoch
// into slot [rank] of rank j's flag array (after a system-scope fence; the slice stores of the
// preceding kernel on this stream are complete before this kernel starts), then waits,
// bounded, until slot [j] of the local flag array has reached it.
__global__ void peer_barrier_kernel(int *const *flag_arrays, int world, int rank, int *epoch_counter,
                                    int *status, long long max_cycles) {
    __shared__ int s_epoch;
    if (threadIdx.x == 0) s_epoch = ++(*epoch_counter);
    __syncthreads();
    const int epoch = s_epoch;
    const int j = threadIdx.x;
    if (j < world) {
        __threadfence_system();  // release: everything this stream wrote before is performed first
        volatile int *remote = flag_arrays[j] + rank;
        *remote = epoch;
        const volatile int *mine = flag_arrays[rank] + j;
        const long long t0 = clock64();
        bool ok = false;
        for (;;) {
            if (*mine - epoch >= 0) { ok = true; break; }
            if (clock64() - t0 > max_cycles) break;
        }
        __threadfence_system();  // acquire: later reads of the peers' slices see their data
        if (!ok) atomicCAS(status, 0, 100 + j);  // peer j never arrived
    }
}

// Wait-only counterpart for chains of sharded forwards that publish without waiting: thread j waits, bounded,
// until rank j has published as many forwards as this rank has.
__global__ void peer_wait_kernel(int *const *flag_arrays, int world, int rank, const int *epoch_counter, int *status,
                                 long long max_cycles) {
    const int j = threadIdx.x;
    if (j < world) {
        const int want = *reinterpret_cast<const volatile int *>(epoch_counter);
        const volatile int *mine = flag_arrays[rank] + j;
        const long long t0 = clock64();
        bool ok = false;
        for (;;) {
            if (*mine - want >= 0) { ok = true; break; }
            if (clock64() - t0 > max_cycles) break;
        }
        __threadfence_system();
        if (!ok) atomicCAS(status, 0, 100 + j);
    }
}

// Flagged words -> plain f32, the end of a chain of flagged forwards: every thread waits, bounded, until its two
// (value, epoch) pairs carry epoch (*round << 8) | seq and stores the two values; the last CTA to finish advances
// the round (every CTA has read it by then), so the next chain's words differ from everything still in the buffers.
__global__ void flagged_unpack_kernel(const uint2 *src, size_t ld_src, float *dst, size_t ld_dst, int n, int m, int seq,
                                      int *round, int *done_counter, int *status, long long max_cycles) {
    // the next launch may start (it waits for this grid before it reads anything); this one waits for the forward
    // before it, and with it for the previous chain's unpack, whose update of the round is then visible
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r_now = *reinterpret_cast<const volatile int *>(round);
    const uint32_t epoch = ((uint32_t)r_now << 8) | (uint32_t)seq;
    const int pairs = (m + 1) / 2;
    const long long total = (long long)n * pairs;
    bool ok = true;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / pairs), c = (int)(i - (long long)r * pairs) * 2;
        const uint2 *s = src + (size_t)r * ld_src + c;
        const bool two = c + 1 < m;
        uint32_t v0, f0, v1 = 0, f1 = epoch;
        long long t0 = 0;
        for (;;) {
            if (two) {
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v0), "=r"(f0), "=r"(v1), "=r"(f1) : "l"(s) : "memory");
            } else {
                asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v0), "=r"(f0) : "l"(s) : "memory");
            }
            if (f0 == epoch && f1 == epoch) break;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > max_cycles) { ok = false; break; }
        }
        float *d = dst + (size_t)r * ld_dst + c;
        d[0] = __uint_as_float(v0);
        if (two) d[1] = __uint_as_float(v1);
    }
    if (!ok) atomicCAS(status, 0, 110);
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(done_counter, 1);
        if (ticket == (int)gridDim.x - 1) {
            *done_counter = 0;
            __threadfence();
            *reinterpret_cast<volatile int *>(round) = (r_now + 1) & 0xffffff;
        }
    }
}

}  // namespace kb

using namespace kb;

extern "C" {

int kb_symm_alloc(size_t bytes, void **out) {
    if (!out || bytes == 0) return fail(KB_ERR_INVALID, "null pointer or zero size");
    void *p = nullptr;
    KB_CUDA(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "cudaMemset"); }
    *out = p;
    return KB_OK;
}

int kb_symm_free(void *p) {
    if (!p) return KB_OK;
    KB_CUDA(cudaFree(p));
    return KB_OK;
}

int kb_ipc_export(const void *p, uint8_t *handle64) {
    if (!p || !handle64) return fail(KB_ERR_INVALID, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    cudaIpcMemHandle_t h;
    KB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(p)));
    memcpy(handle64, &h, 64);
    return KB_OK;
}

int kb_ipc_open(const uint8_t *handle64, void **out) {
    if (!handle64 || !out) return fail(KB_ERR_INVALID, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    KB_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
    return KB_OK;
}

int kb_ipc_close(void *p) {
    if (!p) return KB_OK;
    KB_CUDA(cudaIpcCloseMemHandle(p));
    return KB_OK;
}

int kb_peer_barrier(int *const *flag_arrays_dev, int world, int rank, int *epoch_counter_dev, int *status_dev,
                    kb_stream stream) {
    if (!flag_arrays_dev || !status_dev || !epoch_counter_dev) return fail(KB_ERR_INVALID, "null pointer");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(KB_ERR_INVALID, "world %d / rank %d outside 1..%d", world, rank, MAX_PEERS);
    // about one second of SM clocks: a peer that never arrives ends the wait with a status code
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag_arrays_dev, world, rank, epoch_counter_dev,
                                                                         status_dev, 2000000000ll);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "peer barrier launch");
}

int kb_peer_wait(int *const *flag_arrays_dev, int world, int rank, const int *epoch_counter_dev, int *status_dev,
                 kb_stream stream) {
    if (!flag_arrays_dev || !status_dev || !epoch_counter_dev) return fail(KB_ERR_INVALID, "null pointer");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(KB_ERR_INVALID, "world %d / rank %d outside 1..%d", world, rank, MAX_PEERS);
    peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag_arrays_dev, world, rank, epoch_counter_dev, status_dev,
                                                                      2000000000ll);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "peer wait launch");
}

// x (f32) or xq/sx/sumq (already quantised) -> this rank's slice of y in every rank's buffer
static int sharded_forward(const kb_linear *h, const float *x, const int8_t *xq, size_t ldq, const float *sx,
                           const int32_t *sumq, size_t n, size_t in_dim, float *const *y_bases, int world, int rank,
                           size_t m_total, size_t col_offset, int path, void *workspace, size_t workspace_bytes,
                           int *const *flag_arrays_dev, int *sync_words_dev, kb_stream stream, bool chain = false) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (!y_bases || (!x && !(xq && sx && sumq))) return fail(KB_ERR_INVALID, "null pointer");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(KB_ERR_INVALID, "world %d / rank %d outside 1..%d", world, rank, MAX_PEERS);
    if (in_dim != L->k)
        return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got last dimension %zu", L->k, in_dim);
    if (col_offset + L->m > m_total)
        return fail(KB_ERR_SHAPE, "slice [%zu, %zu) does not fit in %zu output features", col_offset,
                    col_offset + L->m, m_total);
    if (n == 0) return KB_OK;
    for (int q = 0; q < world; ++q)
        if (!y_bases[q]) return fail(KB_ERR_INVALID, "null output base for rank %d", q);
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != L->device && (e = cudaSetDevice(L->device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdArgs a = {};
    a.lin = L; a.n = n; a.ldy = m_total;
    a.y = y_bases[rank] + col_offset;
    a.n_more = 0;
    for (int q = 0; q < world; ++q)
        if (q != rank) a.y_more[a.n_more++] = y_bases[q] + col_offset;
    // the GEMV (a few tokens) ends in the fused barrier; the small-batch kernel and the GEMM store
    // to the peers and a barrier kernel follows
    if (path == KB_PATH_AUTO) path = auto_path(L, n, xq != nullptr);
    if (path == KB_PATH_GEMV_SHARED) { a.shared_grid = true; path = KB_PATH_GEMV; }
    int rc;
    // sync_words_dev = {epoch counter, CTA-done counter, status}
    PeerSync sync = {flag_arrays_dev, sync_words_dev, sync_words_dev ? sync_words_dev + 1 : nullptr,
                     sync_words_dev ? sync_words_dev + 2 : nullptr, world, rank};
    const bool want_sync = flag_arrays_dev && sync_words_dev;
    if (chain && want_sync && xq && gemv_stream_supports(L, n)) {
        // chain form: the streaming kernel waits for the peers' previous publication in its prologue and
        // publishes its own at its end, without waiting
        a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq;
        a.sync = &sync;
        rc = launch_gemv_stream(a, st);
        if (prev != L->device) cudaSetDevice(prev);
        return rc;
    }
    if (path == KB_PATH_GEMV) {
        if (xq) { a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq; } else { a.x = x; }
        a.sync = want_sync ? &sync : nullptr;  // barrier fused into the kernel's tail
        rc = launch_gemv(a, st);
    } else {
        rc = KB_OK;
        uint8_t *ws = nullptr;
        bool own = false;
        if (xq) {
            a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq;
        } else {
            const size_t xq_bytes = (n * L->kp + 255) / 256 * 256, vec_bytes = (n * 4 + 255) / 256 * 256;
            const size_t need = xq_bytes + 2 * vec_bytes;
            ws = static_cast<uint8_t *>(workspace);
            if (!ws) {
                e = cudaMallocAsync(reinterpret_cast<void **>(&ws), need, st);
                if (e != cudaSuccess) rc = cuda_fail(e, "workspace allocation");
                own = true;
            } else if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255)) {
                rc = fail(KB_ERR_STORAGE, "workspace too small or misaligned: need %zu bytes, got %zu", need, workspace_bytes);
            }
            if (rc == KB_OK) {
                int8_t *wq = reinterpret_cast<int8_t *>(ws);
                float *wsx = reinterpret_cast<float *>(ws + xq_bytes);
                int32_t *wsum = reinterpret_cast<int32_t *>(ws + xq_bytes + vec_bytes);
                rc = launch_act_quant(x, n, L->k, wq, L->kp, wsx, wsum, st);
                a.xq = wq; a.ldq = L->kp; a.sx = wsx; a.sumq = wsum;
            }
        }
        if (rc == KB_OK)
            rc = path == KB_PATH_GEMV_MMA ? launch_gemv_mma(a, st)
                 : (path == KB_PATH_GEMV_STREAM ? launch_gemv_stream(a, st) : launch_gemm_tc(a, st));
        if (own && ws) cudaFreeAsync(ws, st);
        if (rc == KB_OK && want_sync)
            rc = kb_peer_barrier(flag_arrays_dev, world, rank, sync_words_dev, sync_words_dev + 2, stream);
    }
    if (prev != L->device) cudaSetDevice(prev);
    return rc;
}

int kb_linear_forward_sharded(const kb_linear *h, const float *x, size_t n, size_t in_dim, float *const *y_bases,
                              int world, int rank, size_t m_total, size_t col_offset, int path, void *workspace,
                              size_t workspace_bytes, int *const *flag_arrays_dev, int *sync_words_dev,
                              kb_stream stream) {
    if (!x) return fail(KB_ERR_INVALID, "null pointer");
    return sharded_forward(h, x, nullptr, 0, nullptr, nullptr, n, in_dim, y_bases, world, rank, m_total, col_offset, path,
                           workspace, workspace_bytes, flag_arrays_dev, sync_words_dev, stream);
}

int kb_linear_forward_sharded_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx, const int32_t *sumq,
                                 size_t n, float *const *y_bases, int world, int rank, size_t m_total, size_t col_offset,
                                 int path, int *const *flag_arrays_dev, int *sync_words_dev, kb_stream stream) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (!xq || !sx || !sumq) return fail(KB_ERR_INVALID, "null pointer");
    return sharded_forward(h, nullptr, xq, ldq, sx, sumq, n, L->k, y_bases, world, rank, m_total, col_offset, path, nullptr, 0,
                           flag_arrays_dev, sync_words_dev, stream);
}

int kb_linear_forward_sharded_chain_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx, const int32_t *sumq,
                                       size_t n, float *const *y_bases, int world, int rank, size_t m_total,
                                       size_t col_offset, int *const *flag_arrays_dev, int *sync_words_dev, kb_stream stream) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (!xq || !sx || !sumq || !flag_arrays_dev || !sync_words_dev) return fail(KB_ERR_INVALID, "null pointer");
    return sharded_forward(h, nullptr, xq, ldq, sx, sumq, n, L->k, y_bases, world, rank, m_total, col_offset, KB_PATH_AUTO,
                           nullptr, 0, flag_arrays_dev, sync_words_dev, stream, true);
}

// Flagged exchange: the slice goes into every rank's buffer as (value, epoch) pairs; nothing waits in the producer
// and nothing is fenced.  x is plain f32, the flagged output of the previous forward of the chain, or pre-quantised.
// sync words: [2] status, [3] round of the flagged chains, [4] CTA counter of the unpack.
static int sharded_flagged(const kb_linear *h, const void *x, int x_is_flagged, size_t ldx, const int8_t *xq, size_t ldq,
                           const float *sx, const int32_t *sumq, size_t n, unsigned long long *const *y_bases, int world,
                           int rank, size_t m_total, size_t col_offset, int seq, int fuse, void *workspace,
                           size_t workspace_bytes, int *sync_words_dev, kb_stream stream) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (!y_bases || !sync_words_dev || (!x && !(xq && sx && sumq))) return fail(KB_ERR_INVALID, "null pointer");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return fail(KB_ERR_INVALID, "world %d / rank %d outside 1..%d", world, rank, MAX_PEERS);
    if (seq < 1 || seq > 255 || (x_is_flagged && seq < 2))
        return fail(KB_ERR_INVALID, "chain position %d outside 1..255 (a forward on flagged activations is at least the second)", seq);
    if (col_offset + L->m > m_total)
        return fail(KB_ERR_SHAPE, "slice [%zu, %zu) does not fit in %zu output features", col_offset, col_offset + L->m, m_total);
    if (n == 0) return KB_OK;
    for (int q = 0; q < world; ++q)
        if (!y_bases[q]) return fail(KB_ERR_INVALID, "null output base for rank %d", q);
    // up to 8 tokens (32 pre-quantised) the streaming kernel, beyond it the medium-batch GEMM (up to 128 tokens)
    const bool use_stream = gemv_stream_supports(L, n) && n <= (size_t)(xq ? 32 : 8);
    if (!use_stream && (n > 128 || !L->has_tmap128))
        return fail(KB_ERR_UNSUPPORTED, "flagged exchange: %zu tokens x K=%zu fit neither the streaming kernel nor the medium-batch GEMM", n,
                    L->k);
    if (!xq && !x_is_flagged && ldx && ldx != L->k)
        return fail(KB_ERR_UNSUPPORTED, "flagged exchange: plain f32 activations must be dense rows");
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != L->device && (e = cudaSetDevice(L->device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdArgs a = {};
    a.lin = L; a.n = n; a.ldy = m_total;
    a.y = reinterpret_cast<float *>(y_bases[rank] + col_offset);
    a.n_more = 0;
    for (int q = 0; q < world; ++q)
        if (q != rank) a.y_more[a.n_more++] = reinterpret_cast<float *>(y_bases[q] + col_offset);
    a.y_flagged = true;
    a.flag_round = sync_words_dev + 3;
    a.flag_seq = seq;
    int rc = KB_OK;
    uint8_t *ws = nullptr;
    bool own = false;
    // flagged activations: the kernel's own prologue waits for them and quantises (every CTA reads the whole row:
    // short rows only), or a cluster kernel does it once for all CTAs
    const bool separate = !use_stream || (x_is_flagged && (fuse == 2 || (fuse == 0 && (L->kp > 4096 || n > 2))));
    if (xq) {
        a.xq = xq; a.ldq = ldq; a.sx = sx; a.sumq = sumq;
    } else if (separate) {
        const size_t xq_bytes = (n * L->kp + 255) / 256 * 256, vec_bytes = (n * 4 + 255) / 256 * 256;
        const size_t need = xq_bytes + 2 * vec_bytes;
        ws = static_cast<uint8_t *>(workspace);
        if (!ws) {
            e = cudaMallocAsync(reinterpret_cast<void **>(&ws), need, st);
            if (e != cudaSuccess) rc = cuda_fail(e, "workspace allocation");
            own = true;
        } else if (workspace_bytes < 2 * need || (reinterpret_cast<uintptr_t>(ws) & 255)) {
            rc = fail(KB_ERR_STORAGE, "workspace too small or misaligned: need %zu bytes (two halves), got %zu", 2 * need, workspace_bytes);
        } else {
            ws += (size_t)(seq & 1) * need;  // consecutive links never share a half
        }
        if (rc == KB_OK) {
            int8_t *wq = reinterpret_cast<int8_t *>(ws);
            float *wsx = reinterpret_cast<float *>(ws + xq_bytes);
            int32_t *wsum = reinterpret_cast<int32_t *>(ws + xq_bytes + vec_bytes);
            rc = x_is_flagged ? launch_act_quant_flagged(static_cast<const unsigned long long *>(x), ldx ? ldx : L->k, n, L->k,
                                                         sync_words_dev + 3, seq - 1, wq, L->kp, wsx, wsum, sync_words_dev + 2, st)
                              : launch_act_quant(static_cast<const float *>(x), n, L->k, wq, L->kp, wsx, wsum, st);
            a.xq = wq; a.ldq = L->kp; a.sx = wsx; a.sumq = wsum;
        }
    } else if (x_is_flagged) {
        a.xf = static_cast<const unsigned long long *>(x);
        a.ldxf = ldx ? ldx : L->k;
    } else {
        a.x = static_cast<const float *>(x);
    }
    if (rc == KB_OK) rc = use_stream ? launch_gemv_stream(a, st) : launch_gemm_tcs(a, st);
    if (own && ws) cudaFreeAsync(ws, st);
    if (prev != L->device) cudaSetDevice(prev);
    return rc;
}

int kb_linear_forward_sharded_flagged(const kb_linear *h, const void *x, int x_is_flagged, size_t ldx, size_t n, size_t in_dim,
                                      unsigned long long *const *y_bases, int world, int rank, size_t m_total, size_t col_offset,
                                      int seq, int fuse, void *workspace, size_t workspace_bytes, int *sync_words_dev,
                                      kb_stream stream) {
    const Linear *L = reinterpret_cast<const Linear *>(h);
    if (!L || L->magic != HANDLE_MAGIC) return fail(KB_ERR_BAD_HANDLE, "null or destroyed kb_linear handle");
    if (!x) return fail(KB_ERR_INVALID, "null pointer");
    if (in_dim != L->k) return fail(KB_ERR_SHAPE, "shape mismatch: expected [%zu], got last dimension %zu", L->k, in_dim);
    if (fuse < 0 || fuse > 2) return fail(KB_ERR_INVALID, "fuse must be 0 (automatic), 1 (prologue) or 2 (separate quantiser)");
    return sharded_flagged(h, x, x_is_flagged, ldx, nullptr, 0, nullptr, nullptr, n, y_bases, world, rank, m_total, col_offset, seq,
                           fuse, workspace, workspace_bytes, sync_words_dev, stream);
}

int kb_linear_forward_sharded_flagged_q8(const kb_linear *h, const int8_t *xq, size_t ldq, const float *sx, const int32_t *sumq,
                                         size_t n, unsigned long long *const *y_bases, int world, int rank, size_t m_total,
                                         size_t col_offset, int seq, int *sync_words_dev, kb_stream stream) {
    if (!xq || !sx || !sumq) return fail(KB_ERR_INVALID, "null pointer");
    return sharded_flagged(h, nullptr, 0, 0, xq, ldq, sx, sumq, n, y_bases, world, rank, m_total, col_offset, seq, 0, nullptr, 0,
                           sync_words_dev, stream);
}

int kb_flagged_unpack(const unsigned long long *src, size_t ld_src, size_t n, size_t m, float *dst, size_t ld_dst, int seq,
                      int *sync_words_dev, kb_stream stream) {
    if (!src || !dst || !sync_words_dev) return fail(KB_ERR_INVALID, "null pointer");
    if (seq < 1 || seq > 255) return fail(KB_ERR_INVALID, "chain position %d outside 1..255", seq);
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (ld_src % 2) || ld_src < m || ld_dst < m)
        return fail(KB_ERR_INVALID, "flagged rows must be 16-byte aligned with an even leading dimension >= %zu", m);
    if (n == 0 || m == 0) return KB_OK;
    if (n > (size_t)1 << 20 || m > (size_t)1 << 30) return fail(KB_ERR_UNSUPPORTED, "flagged unpack: %zu x %zu too large", n, m);
    const long long work = (long long)n * (long long)((m + 1) / 2);
    const int threads = 256;
    long long blocks = (work + threads - 1) / threads;
    if (blocks > 1184) blocks = 1184;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, flagged_unpack_kernel, reinterpret_cast<const uint2 *>(src), ld_src, dst, ld_dst, (int)n,
                                       (int)m, seq, sync_words_dev + 3, sync_words_dev + 4, sync_words_dev + 2, 2000000000ll);
    return e == cudaSuccess ? KB_OK : cuda_fail(e, "flagged unpack launch");
}

}  // extern "C"
