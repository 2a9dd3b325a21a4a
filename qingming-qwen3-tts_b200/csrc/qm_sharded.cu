// Decode attention for streams whose keys are split across the GPUs of one box, with the partials exchanged by
// NCCL: split-KV kernel on this rank's slice -> ncclAllGather of the [batch][q_heads][130] fp32 partials ->
// rank-order combine.  The reference is single-GPU (its launch_attention, 17.cu:17895, sees the whole cache); this
// entry point is what a C++ host with one process (or thread) per GPU calls in its place for very long contexts.
//
// NCCL is not linked: its five functions are resolved at first use from libnccl.so.2 (or the file named by
// QM_NCCL_LIBRARY), or supplied by the host through qm_nccl_set_api - which is also how the CPU tests drive the
// failure handling with a fake.  Failure handling follows NCCL's own recipe for a hung or broken collective: a
// host loop polls the stream and ncclCommGetAsyncError until the work is done, an error shows up, or a deadline
// passes; in the last two cases it calls ncclCommAbort, which ends the collective's kernel, and reports
// QM_ENCCL / QM_ETIMEOUT.  Nothing on the GPU waits without a limit.
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <thread>

#include "qm_common.cuh"

namespace {

constexpr int kNcclSuccess = 0;
constexpr int kNcclInProgress = 7;
constexpr int kNcclFloat32 = 7;
constexpr int kPartialWidth = kHeadDim + 2;

struct NcclUniqueId {
    char internal[128];
};

int default_stream_query(void* stream) {
    const cudaError_t status = cudaStreamQuery(static_cast<cudaStream_t>(stream));
    if (status == cudaSuccess) return 0;
    if (status == cudaErrorNotReady) return 1;
    return -1;
}

struct Resolved {
    qm_nccl_api api{};
    int (*get_unique_id)(NcclUniqueId*) = nullptr;
    int (*comm_init_rank)(void**, int, NcclUniqueId, int) = nullptr;
    int (*comm_destroy)(void*) = nullptr;
    bool from_host = false;
    bool loaded = false;
    char error[256] = "";
};

std::mutex g_guard;
Resolved g_nccl;

template <class F>
bool resolve(void* library, const char* name, F* slot) {
    *slot = reinterpret_cast<F>(dlsym(library, name));
    if (!*slot) std::snprintf(g_nccl.error, sizeof(g_nccl.error), "NCCL symbol %s not found", name);
    return *slot != nullptr;
}

// Fills g_nccl from the NCCL shared library unless the host supplied a table.  Call with g_guard held.
bool ensure_nccl() {
    if (g_nccl.from_host || g_nccl.loaded) return true;
    const char* path = std::getenv("QM_NCCL_LIBRARY");
    void* library = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!library) {
        std::snprintf(g_nccl.error, sizeof(g_nccl.error), "cannot load NCCL: %s", dlerror());
        return false;
    }
    bool ok = resolve(library, "ncclAllGather", &g_nccl.api.all_gather);
    ok = ok && resolve(library, "ncclCommGetAsyncError", &g_nccl.api.comm_get_async_error);
    ok = ok && resolve(library, "ncclCommAbort", &g_nccl.api.comm_abort);
    ok = ok && resolve(library, "ncclCommCount", &g_nccl.api.comm_count);
    ok = ok && resolve(library, "ncclGetErrorString", &g_nccl.api.get_error_string);
    ok = ok && resolve(library, "ncclGetUniqueId", &g_nccl.get_unique_id);
    ok = ok && resolve(library, "ncclCommInitRank", &g_nccl.comm_init_rank);
    ok = ok && resolve(library, "ncclCommDestroy", &g_nccl.comm_destroy);
    if (!ok) return false;
    g_nccl.api.stream_query = default_stream_query;
    g_nccl.loaded = true;
    return true;
}

int32_t fail_nccl(const char* operation, int result) {
    char text[384];
    const char* detail = (g_nccl.api.get_error_string && result >= 0) ? g_nccl.api.get_error_string(result) : "";
    std::snprintf(text, sizeof(text), "%s: NCCL result %d %s", operation, result, detail ? detail : "");
    return qm_fail(QM_ENCCL, text);
}

}  // namespace

extern "C" {

int32_t qm_nccl_set_api(const qm_nccl_api* api) {
    std::lock_guard<std::mutex> lock(g_guard);
    if (!api) {                       // back to the shared library
        g_nccl.from_host = false;
        if (!g_nccl.loaded) g_nccl.api = qm_nccl_api{};
        return QM_OK;
    }
    if (!api->all_gather || !api->comm_get_async_error || !api->comm_abort || !api->comm_count)
        return qm_fail(QM_EINVAL, "qm_nccl_set_api: all_gather, comm_get_async_error, comm_abort and comm_count are required");
    g_nccl.api = *api;
    if (!g_nccl.api.stream_query) g_nccl.api.stream_query = default_stream_query;
    g_nccl.from_host = true;
    g_nccl.loaded = false;
    return QM_OK;
}

int32_t qm_nccl_unique_id(void* id_out) {
    if (!id_out) return qm_fail(QM_EINVAL, "id_out is null");
    std::lock_guard<std::mutex> lock(g_guard);
    if (!ensure_nccl()) return qm_fail(QM_ENCCL, g_nccl.error);
    if (!g_nccl.get_unique_id) return qm_fail(QM_ENCCL, "communicator helpers need the NCCL shared library, not a host-supplied table");
    const int result = g_nccl.get_unique_id(static_cast<NcclUniqueId*>(id_out));
    return result == kNcclSuccess ? QM_OK : fail_nccl("ncclGetUniqueId", result);
}

int32_t qm_nccl_comm_init_rank(void** comm_out, int32_t world, const void* id, int32_t rank) {
    if (!comm_out || !id) return qm_fail(QM_EINVAL, "null pointer");
    std::lock_guard<std::mutex> lock(g_guard);
    if (!ensure_nccl()) return qm_fail(QM_ENCCL, g_nccl.error);
    if (!g_nccl.comm_init_rank) return qm_fail(QM_ENCCL, "communicator helpers need the NCCL shared library, not a host-supplied table");
    NcclUniqueId copy;
    std::memcpy(&copy, id, sizeof(copy));
    const int result = g_nccl.comm_init_rank(comm_out, world, copy, rank);
    return result == kNcclSuccess ? QM_OK : fail_nccl("ncclCommInitRank", result);
}

int32_t qm_nccl_comm_destroy(void* comm) {
    if (!comm) return QM_OK;
    std::lock_guard<std::mutex> lock(g_guard);
    if (!ensure_nccl()) return qm_fail(QM_ENCCL, g_nccl.error);
    if (!g_nccl.comm_destroy) return qm_fail(QM_ENCCL, "communicator helpers need the NCCL shared library, not a host-supplied table");
    const int result = g_nccl.comm_destroy(comm);
    return result == kNcclSuccess ? QM_OK : fail_nccl("ncclCommDestroy", result);
}

int32_t qm_nccl_wait(void* nccl_comm, void* stream, int32_t deadline_ms) {
    if (!nccl_comm) return qm_fail(QM_EINVAL, "communicator is null");
    if (deadline_ms < 0) return qm_fail(QM_EINVAL, "deadline must not be negative");
    qm_nccl_api api;
    {
        std::lock_guard<std::mutex> lock(g_guard);
        if (!ensure_nccl()) return qm_fail(QM_ENCCL, g_nccl.error);
        api = g_nccl.api;
    }
    const auto begin = std::chrono::steady_clock::now();
    unsigned polls = 0;
    for (;;) {
        const int done = api.stream_query(stream);
        if (done == 0) return QM_OK;
        if (done < 0) {
            api.comm_abort(nccl_comm);
            return qm_fail(QM_ECUDA, "the stream reported an error while a collective was in flight; communicator aborted");
        }
        int async_error = kNcclSuccess;
        const int result = api.comm_get_async_error(nccl_comm, &async_error);
        if (result != kNcclSuccess || (async_error != kNcclSuccess && async_error != kNcclInProgress)) {
            api.comm_abort(nccl_comm);
            return fail_nccl("collective failed (communicator aborted)", result != kNcclSuccess ? result : async_error);
        }
        const auto elapsed = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - begin);
        if (elapsed.count() >= deadline_ms) {
            api.comm_abort(nccl_comm);
            return qm_fail(QM_ETIMEOUT, "collective did not finish before the deadline (a rank is missing?); communicator aborted");
        }
        if (++polls > 64) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int32_t qm_decode_attention_sharded(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* local_seq_lens,
                                    const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                                    uint16_t* out, float* partial_send, float* partial_recv, int32_t world,
                                    void* workspace, int64_t workspace_bytes, void* nccl_comm, void* stream) {
    if (!nccl_comm || !partial_send || !partial_recv) return qm_fail(QM_EINVAL, "null pointer");
    if (world < 1) return qm_fail(QM_EINVAL, "world must be >= 1");
    qm_nccl_api api;
    {
        std::lock_guard<std::mutex> lock(g_guard);
        if (!ensure_nccl()) return qm_fail(QM_ENCCL, g_nccl.error);
        api = g_nccl.api;
    }
    int count = 0;
    int result = api.comm_count(nccl_comm, &count);
    if (result != kNcclSuccess) return fail_nccl("ncclCommCount", result);
    if (count != world) return qm_fail(QM_EINVAL, "world does not match the communicator's rank count");
    int32_t rc = qm_decode_attention_partial(pool, layer, q_rot, local_seq_lens, page_table, max_pages, batch, q_heads,
                                             partial_send, workspace, workspace_bytes, stream);
    if (rc != QM_OK) return rc;
    if (batch == 0) return QM_OK;
    const size_t elements = (size_t)batch * q_heads * kPartialWidth;
    result = api.all_gather(partial_send, partial_recv, elements, kNcclFloat32, nccl_comm, stream);
    if (result != kNcclSuccess) return fail_nccl("ncclAllGather of the attention partials", result);
    return qm_attention_combine(partial_recv, world, batch * q_heads, out, stream);
}

}  // extern "C"
