// Exchange + combine of split-KV partial states across the GPUs of one box, in ONE kernel over peer memory.
//
// Used when a very long stream's keys are split over several GPUs: every rank has the partial softmax state
// (m, l, o[128]) of each (stream, query head) row over its own slice.  Instead of a library all-gather followed by
// a combine kernel, each rank's kernel
//   1. stores its rows straight into the exchange buffer of every peer (plain peer-to-peer stores over NVLink),
//   2. publishes them with a system-scope release on a per-source counter in the peer's buffer,
//   3. waits (bounded) until the counters of all sources in its OWN buffer have reached this call's value,
//   4. folds the world's partials of each row in rank order and writes the bf16 context.
// Every rank runs the same kernel at the same time on its own GPU.  Counters only grow (call number * rows), the
// payload is double-buffered by call parity, so nothing has to be cleared between calls.  No multicast, no TMA:
// ordinary global stores and loads on peer addresses.  The reference has no multi-GPU path; this is new.
#include <math_constants.h>

#include "qm_common.cuh"

namespace {

constexpr int kPartialWidth = kHeadDim + 2;        // m, l, o[128]
constexpr int kExchangeThreads = 160;              // 130 payload lanes, rounded up to warps
constexpr uint32_t kExchangeSpinLimit = 1u << 20;

struct ExchangeArgs {
    const float* local;              // [rows][130] this rank's partials (m in natural-log domain)
    unsigned char* const* peers;     // [world] device pointers to every rank's exchange buffer (own included)
    uint16_t* out;                   // [rows][128]
    uint32_t* status;
    unsigned long long epoch;        // 1, 2, 3, ... : number of this call
    int world, rank, rows, rows_capacity;
};

// buffer layout: float payload[2][world][rows_capacity][130]; then unsigned long long arrived[world]
__device__ __forceinline__ size_t payload_offset(const ExchangeArgs& a, int slot, int source, int row) {
    return ((((size_t)slot * a.world + source) * a.rows_capacity + row) * kPartialWidth) * sizeof(float);
}
__device__ __forceinline__ size_t counter_offset(const ExchangeArgs& a, int source) {
    return (size_t)2 * a.world * a.rows_capacity * kPartialWidth * sizeof(float) + (size_t)source * sizeof(unsigned long long);
}

__global__ void __launch_bounds__(kExchangeThreads) qm_exchange_combine_kernel(const ExchangeArgs a) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int t = threadIdx.x;
    const int slot = (int)(a.epoch & 1ull);
    __shared__ int timed_out;
    if (t == 0) timed_out = 0;

    // 1. my row to every rank's buffer
    if (t < kPartialWidth) {
        const float v = a.local[(size_t)row * kPartialWidth + t];
        for (int p = 0; p < a.world; ++p)
            *reinterpret_cast<float*>(a.peers[p] + payload_offset(a, slot, a.rank, row) + (size_t)t * sizeof(float)) = v;
    }
    __threadfence_system();
    __syncthreads();
    // 2. one arrival per row on every rank's counter for this source
    if (t < a.world) {
        unsigned long long* counter = reinterpret_cast<unsigned long long*>(a.peers[t] + counter_offset(a, a.rank));
        asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(counter), "l"(1ull) : "memory");
    }
    // 3. wait for every source's rows of this call
    if (t < a.world) {
        const unsigned long long* counter =
            reinterpret_cast<const unsigned long long*>(a.peers[a.rank] + counter_offset(a, t));
        const unsigned long long want = a.epoch * (unsigned long long)a.rows;
        bool ok = false;
        for (uint32_t spin = 0; spin < kExchangeSpinLimit; ++spin) {
            unsigned long long seen;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(counter) : "memory");
            if (seen >= want) {
                ok = true;
                break;
            }
            if (spin > 64) __nanosleep(200);
        }
        if (!ok) {
            atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
            timed_out = 1;
        }
    }
    __syncthreads();
    // 4. fold in rank order
    if (t < kHeadDim) {
        const unsigned char* mine = a.peers[a.rank];
        float big = -CUDART_INF_F;
        for (int g = 0; g < a.world; ++g)
            big = fmaxf(big, *reinterpret_cast<const volatile float*>(mine + payload_offset(a, slot, g, row)));
        float acc = 0.0f, denom = 0.0f;
        for (int g = 0; g < a.world; ++g) {
            const volatile float* src = reinterpret_cast<const volatile float*>(mine + payload_offset(a, slot, g, row));
            const float l = src[1];
            if (!(l > 0.0f)) continue;
            const float w = __expf(src[0] - big);
            denom = fmaf(w, l, denom);
            acc = fmaf(w, src[2 + t], acc);
        }
        a.out[(size_t)row * kHeadDim + t] = (denom > 0.0f && !timed_out) ? (uint16_t)f32_to_bf16_bits(acc / denom) : (uint16_t)0;
    }
}

}  // namespace

extern "C" {

int64_t qm_exchange_buffer_bytes(int32_t world, int32_t rows_capacity) {
    if (world < 1 || rows_capacity < 1) return 0;
    return (int64_t)2 * world * rows_capacity * kPartialWidth * (int64_t)sizeof(float) + (int64_t)world * 8 + 64;
}

int32_t qm_attention_exchange_combine(qm_kv_pool* pool, const float* local_partials, void* const* peer_buffers_dev,
                                      int32_t world, int32_t rank, int32_t rows, int32_t rows_capacity, uint64_t epoch,
                                      uint16_t* out, void* stream) {
    if (!pool || !local_partials || !peer_buffers_dev || !out) return qm_fail(QM_EINVAL, "null pointer");
    if (world < 1 || world > 32 || rank < 0 || rank >= world || rows < 0 || rows > rows_capacity || epoch == 0)
        return qm_fail(QM_EINVAL, "invalid exchange geometry");
    if (rows == 0) return QM_OK;
    ExchangeArgs a{};
    a.local = local_partials;
    a.peers = reinterpret_cast<unsigned char* const*>(peer_buffers_dev);
    a.out = out;
    a.status = pool->status_dev;
    a.epoch = epoch;
    a.world = world;
    a.rank = rank;
    a.rows = rows;
    a.rows_capacity = rows_capacity;
    QM_CUDA_TRY(qm_launch(qm_exchange_combine_kernel, dim3(rows), dim3(kExchangeThreads), 0, static_cast<cudaStream_t>(stream), a),
                "partial exchange + combine launch");
    return QM_OK;
}

}  // extern "C"
