// Exchange + combine of split-KV partial states across the GPUs of one box, in ONE kernel over peer memory.
//
// Used when a very long stream's keys are split over several GPUs: every rank has the partial softmax state
// (m, l, o[128]) of each (stream, query head) row over its own slice.  Instead of a library all-gather followed by
// a combine kernel, each rank's kernel, one CTA per row,
//   1. takes the row's next sequence number from a counter in its OWN buffer (device state, so the host passes no
//      call number and a captured launch can be replayed),
//   2. stores its row straight into slot (sequence parity, this rank, row) of every rank's buffer - plain
//      peer-to-peer stores over NVLink - and then publishes it by storing the sequence number into the slot's
//      arrival word with a system-scope release,
//   3. waits (bounded) until the arrival words of ALL ranks for this row in its own buffer carry that number,
//   4. folds the world's partials of the row in rank order and writes the bf16 context.
// A row's CTA waits only for that same row of the other ranks, so rows do not depend on one another.  Slots are
// double-buffered by sequence parity: a peer can be at most one call ahead (it cannot finish call n + 1 without
// this rank's row of call n + 1), so it never overwrites a slot that is still being read.  No multicast, no TMA:
// ordinary global stores and loads on peer addresses.  The reference has no multi-GPU path; this is new.
//
// Also here: the exchange object that owns such a buffer and maps the peers' buffers through CUDA IPC handles (for
// hosts with one process per GPU) or takes peer pointers directly (one process driving several GPUs).
#include <cstring>
#include <new>

#include "qm_exchange_layout.cuh"

namespace {

constexpr int kPartialWidth = kExchangeWidth;      // m, l, o[128]
constexpr int kExchangeThreads = 128;              // one thread per output dimension of the row
constexpr int kMaxWorld = kExchangeMaxWorld;

struct ExchangeArgs {
    const float* local;              // [rows][130] this rank's partials (m in natural-log domain)
    ExchangeView view;
    uint16_t* out;                   // [rows][128]
    uint32_t* status;
};

__host__ __device__ __forceinline__ size_t payload_bytes(int world, int rows_capacity) {
    return exchange_payload_bytes(world, rows_capacity);
}

__global__ void __launch_bounds__(kExchangeThreads) qm_exchange_combine_kernel(const ExchangeArgs a) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int t = threadIdx.x;
    __shared__ uint32_t shared2[2];
    __shared__ unsigned char* peer_cache[kExchangeMaxWorld];
    const ExchangeView view = exchange_cache_peers(a.view, peer_cache, t);
    const float* mine = a.local + (size_t)row * kPartialWidth;
    const float m = mine[0], l = mine[1], o = mine[2 + t];
    __syncthreads();
    exchange_row(view, row, t, m, l, o, true, a.out + (size_t)row * kHeadDim, a.status, shared2, [] { __syncthreads(); });
}

// Rows one launch may carry: every row's CTA must be able to be resident at once.  A CTA spins until the same row
// of every other rank has arrived; if the ranks' hardware handed out CTAs in different orders and only some fit,
// two ranks could each hold rows the other has not started.  With all CTAs resident that cannot happen.
int32_t exchange_row_limit(qm_kv_pool* pool, int* limit_out) {
    static thread_local int known_device = -1, known_limit = 0;
    if (known_device != pool->device) {
        int per_sm = 0;
        QM_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qm_exchange_combine_kernel, kExchangeThreads, 0),
                    "query exchange kernel occupancy");
        known_limit = per_sm * pool->sm_count;
        known_device = pool->device;
    }
    *limit_out = known_limit;
    return QM_OK;
}

}  // namespace

struct qm_exchange {
    int device;
    int world, rank, rows_capacity;
    size_t bytes;
    unsigned char* own;                 // this rank's buffer (cudaMalloc)
    unsigned char* mapped[kMaxWorld];   // every rank's buffer as seen from this process; [rank] == own
    bool opened_by_ipc[kMaxWorld];
    unsigned char** table_dev;          // device copy of mapped[0..world)
    bool peers_known;
};

extern "C" {

int64_t qm_exchange_buffer_bytes(int32_t world, int32_t rows_capacity) {
    if (world < 1 || rows_capacity < 1) return 0;
    return (int64_t)payload_bytes(world, rows_capacity) + (int64_t)2 * world * rows_capacity * 4 + (int64_t)rows_capacity * 4 + 64;
}

int32_t qm_attention_exchange_combine(qm_kv_pool* pool, const float* local_partials, void* const* peer_buffers_dev,
                                      int32_t world, int32_t rank, int32_t rows, int32_t rows_capacity, uint16_t* out,
                                      void* stream) {
    if (!pool || !local_partials || !peer_buffers_dev || !out) return qm_fail(QM_EINVAL, "null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || rows < 0 || rows > rows_capacity)
        return qm_fail(QM_EINVAL, "invalid exchange geometry");
    if (rows == 0) return QM_OK;
    int limit = 0;
    const int32_t rc = exchange_row_limit(pool, &limit);
    if (rc != QM_OK) return rc;
    if (rows > limit)
        return qm_fail(QM_ECAPACITY, "more rows than can be resident on the GPU at once; exchange them in several calls");
    ExchangeArgs a{};
    a.local = local_partials;
    a.view.peers = reinterpret_cast<unsigned char* const*>(peer_buffers_dev);
    a.view.world = world;
    a.view.rank = rank;
    a.view.rows_capacity = rows_capacity;
    a.out = out;
    a.status = pool->status_dev;
    QM_CUDA_TRY(qm_launch(qm_exchange_combine_kernel, dim3(rows), dim3(kExchangeThreads), 0, static_cast<cudaStream_t>(stream), a),
                "partial exchange + combine launch");
    return QM_OK;
}

// ---- the exchange object: owns this rank's buffer, maps the peers'

int32_t qm_exchange_create(int32_t world, int32_t rank, int32_t rows_capacity, qm_exchange** exchange_out) {
    if (!exchange_out) return qm_fail(QM_EINVAL, "exchange_out is null");
    *exchange_out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || rows_capacity < 1)
        return qm_fail(QM_EINVAL, "invalid exchange geometry");
    qm_exchange* ex = new (std::nothrow) qm_exchange();
    if (!ex) return qm_fail(QM_ENOMEM, "host allocation of exchange object failed");
    std::memset(ex, 0, sizeof(*ex));
    ex->world = world;
    ex->rank = rank;
    ex->rows_capacity = rows_capacity;
    ex->bytes = (size_t)qm_exchange_buffer_bytes(world, rows_capacity);
    cudaError_t status = cudaGetDevice(&ex->device);
    if (status == cudaSuccess) status = cudaMalloc(&ex->own, ex->bytes);
    if (status == cudaSuccess) status = cudaMalloc(&ex->table_dev, sizeof(unsigned char*) * kMaxWorld);
    if (status == cudaSuccess) status = cudaMemset(ex->own, 0, ex->bytes);
    if (status == cudaSuccess) status = cudaDeviceSynchronize();
    if (status != cudaSuccess) {
        const int32_t code = qm_fail_cuda(status, "allocate exchange buffer");
        qm_exchange_destroy(ex);
        return code;
    }
    ex->mapped[rank] = ex->own;
    *exchange_out = ex;
    return QM_OK;
}

int32_t qm_exchange_destroy(qm_exchange* ex) {
    if (!ex) return QM_OK;
    for (int r = 0; r < ex->world; ++r)
        if (ex->opened_by_ipc[r] && ex->mapped[r]) cudaIpcCloseMemHandle(ex->mapped[r]);
    if (ex->table_dev) cudaFree(ex->table_dev);
    if (ex->own) cudaFree(ex->own);
    delete ex;
    return QM_OK;
}

void* qm_exchange_local_buffer(qm_exchange* ex) { return ex ? ex->own : nullptr; }

int32_t qm_exchange_ipc_handle(qm_exchange* ex, void* handle_out) {
    if (!ex || !handle_out) return qm_fail(QM_EINVAL, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == QM_IPC_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t handle;
    QM_CUDA_TRY(cudaIpcGetMemHandle(&handle, ex->own), "export exchange buffer");
    std::memcpy(handle_out, &handle, sizeof(handle));
    return QM_OK;
}

static int32_t upload_peer_table(qm_exchange* ex) {
    QM_CUDA_TRY(cudaMemcpy(ex->table_dev, ex->mapped, sizeof(unsigned char*) * ex->world, cudaMemcpyHostToDevice),
                "upload peer pointer table");
    ex->peers_known = true;
    return QM_OK;
}

int32_t qm_exchange_open_peers(qm_exchange* ex, const void* handles) {
    if (!ex || !handles) return qm_fail(QM_EINVAL, "null pointer");
    const unsigned char* bytes = static_cast<const unsigned char*>(handles);
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank || ex->mapped[r]) continue;
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, bytes + (size_t)r * QM_IPC_HANDLE_BYTES, sizeof(handle));
        void* mapped = nullptr;
        QM_CUDA_TRY(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess), "map a peer's exchange buffer");
        ex->mapped[r] = static_cast<unsigned char*>(mapped);
        ex->opened_by_ipc[r] = true;
    }
    return upload_peer_table(ex);
}

int32_t qm_exchange_set_peers(qm_exchange* ex, void* const* peer_buffers) {
    if (!ex || !peer_buffers) return qm_fail(QM_EINVAL, "null pointer");
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank) continue;
        if (!peer_buffers[r]) return qm_fail(QM_EINVAL, "a peer buffer pointer is null");
        ex->mapped[r] = static_cast<unsigned char*>(peer_buffers[r]);
        ex->opened_by_ipc[r] = false;
    }
    return upload_peer_table(ex);
}

int32_t qm_exchange_reset(qm_exchange* ex, void* stream) {
    if (!ex) return qm_fail(QM_EINVAL, "exchange is null");
    QM_CUDA_TRY(cudaMemsetAsync(ex->own, 0, ex->bytes, static_cast<cudaStream_t>(stream)), "clear exchange buffer");
    return QM_OK;
}

int32_t qm_exchange_combine(qm_kv_pool* pool, qm_exchange* ex, const float* local_partials, int32_t rows, uint16_t* out,
                            void* stream) {
    if (!ex) return qm_fail(QM_EINVAL, "exchange is null");
    if (!ex->peers_known && ex->world > 1)
        return qm_fail(QM_EINVAL, "peer buffers are not mapped yet: call qm_exchange_open_peers or qm_exchange_set_peers first");
    if (!ex->peers_known) {
        const int32_t rc = upload_peer_table(ex);
        if (rc != QM_OK) return rc;
    }
    return qm_attention_exchange_combine(pool, local_partials, reinterpret_cast<void* const*>(ex->table_dev), ex->world, ex->rank,
                                         rows, ex->rows_capacity, out, stream);
}

int32_t qm_exchange_decode_attention(qm_kv_pool* pool, qm_exchange* ex, int32_t layer, const uint16_t* q_rot,
                                     const int32_t* local_seq_lens, const int32_t* page_table, int32_t max_pages,
                                     int32_t batch, int32_t q_heads, uint16_t* out, void* workspace, int64_t workspace_bytes,
                                     void* stream) {
    if (!ex) return qm_fail(QM_EINVAL, "exchange is null");
    if (!ex->peers_known && ex->world > 1)
        return qm_fail(QM_EINVAL, "peer buffers are not mapped yet: call qm_exchange_open_peers or qm_exchange_set_peers first");
    if (!ex->peers_known) {
        const int32_t rc = upload_peer_table(ex);
        if (rc != QM_OK) return rc;
    }
    return qm_decode_attention_exchange(pool, layer, q_rot, local_seq_lens, page_table, max_pages, batch, q_heads, out,
                                        reinterpret_cast<void* const*>(ex->table_dev), ex->world, ex->rank, ex->rows_capacity,
                                        workspace, workspace_bytes, stream);
}

}  // extern "C"
