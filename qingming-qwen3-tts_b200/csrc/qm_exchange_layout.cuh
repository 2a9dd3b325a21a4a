// Layout of one rank's exchange buffer for split-KV partial states, shared by the stand-alone exchange kernel
// (qm_exchange.cu) and the decode kernel's fused exchange (qm_decode.cu), and the per-row exchange step itself.
//
//   float    payload[2][world][rows_capacity][130]   (m in natural-log domain, l, o[128]) by call parity, source rank, row
//   uint32_t arrived[2][world][rows_capacity]        sequence number of the payload in that slot
//   uint32_t calls[rows_capacity]                    how often THIS rank has exchanged that row
#pragma once

#include <math_constants.h>

#include "qm_common.cuh"

constexpr int kExchangeWidth = kHeadDim + 2;
constexpr uint32_t kExchangeSpinLimit = 1u << 20;
constexpr int kExchangeMaxWorld = 32;

struct ExchangeView {
    unsigned char* const* peers;     // [world] pointers to every rank's buffer (own included).  The kernels copy the
                                     // array into shared memory first: it is read several times per row, and a
                                     // pointer fetched from global memory costs an L2 round trip before each use.
    int world, rank, rows_capacity;
};

// Copies the peer pointer array into `cache` (shared memory, kExchangeMaxWorld entries) and returns a view on it.
// Call from all threads of the CTA, then synchronise before the first exchange_row.
__device__ __forceinline__ ExchangeView exchange_cache_peers(const ExchangeView& x, unsigned char** cache, int tid) {
    if (tid < x.world && tid < kExchangeMaxWorld) cache[tid] = x.peers[tid];
    ExchangeView cached = x;
    cached.peers = cache;
    return cached;
}

__host__ __device__ __forceinline__ size_t exchange_payload_bytes(int world, int rows_capacity) {
    return (size_t)2 * world * rows_capacity * kExchangeWidth * sizeof(float);
}
__device__ __forceinline__ size_t exchange_payload_offset(const ExchangeView& x, int slot, int source, int row) {
    return ((((size_t)slot * x.world + source) * x.rows_capacity + row) * kExchangeWidth) * sizeof(float);
}
__device__ __forceinline__ size_t exchange_arrived_offset(const ExchangeView& x, int slot, int source, int row) {
    return exchange_payload_bytes(x.world, x.rows_capacity) + (((size_t)slot * x.world + source) * x.rows_capacity + row) * sizeof(uint32_t);
}
__device__ __forceinline__ size_t exchange_calls_offset(const ExchangeView& x, int row) {
    return exchange_payload_bytes(x.world, x.rows_capacity) + (size_t)2 * x.world * x.rows_capacity * sizeof(uint32_t) +
           (size_t)row * sizeof(uint32_t);
}

// One row's exchange + rank-order fold, executed by a group of 128 threads (t = 0 .. 127 within the group) that all
// call it together; `sync` is a barrier over exactly those threads.  Thread t holds o[t] of this rank's partial
// row, every thread holds its m (natural-log domain) and l.  `live` = false makes the thread keep step with the
// barriers without touching memory (a thread whose earlier wait gave up).  `shared2` is two words of shared memory
// owned by the group.  Steps: next sequence number of the row from this rank's own counter; the row into slot
// (sequence parity, this rank) of every rank's buffer by plain peer stores; the sequence number into the slot's
// arrival word with a system-scope release; a bounded wait until every rank's copy of the row of this call has
// arrived here; the fold in rank order - the arithmetic of qm_combine_partials_kernel - and the bf16 context.
template <class Sync>
__device__ __forceinline__ void exchange_row(const ExchangeView& x, int row, int t, float m, float l, float o, bool live,
                                             uint16_t* out_row, uint32_t* status, volatile uint32_t* shared2, Sync sync) {
    if (t == 0) {
        uint32_t sequence = 0;
        if (live) {
            uint32_t* calls = reinterpret_cast<uint32_t*>(x.peers[x.rank] + exchange_calls_offset(x, row));
            sequence = *calls + 1u;          // only this row's group of this rank ever touches the word
            *calls = sequence;
        }
        shared2[0] = sequence;
        shared2[1] = 0u;                     // set when a wait gives up
    }
    sync();
    const uint32_t sequence = shared2[0];
    const int slot = (int)(sequence & 1u);
    if (live) {
        for (int p = 0; p < x.world; ++p) {
            float* dst = reinterpret_cast<float*>(x.peers[p] + exchange_payload_offset(x, slot, x.rank, row));
            dst[2 + t] = o;
            if (t == 0) {
                dst[0] = m;
                dst[1] = l;
            }
        }
    }
    // The group's barrier orders every thread's payload stores before the stores below; the release at system scope
    // is cumulative over what the storing thread has observed through that barrier, so one fence per arrival word
    // (not one per payload thread) publishes the whole row.
    sync();
    if (t < x.world && live) {
        uint32_t* word = reinterpret_cast<uint32_t*>(x.peers[t] + exchange_arrived_offset(x, slot, x.rank, row));
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(word), "r"(sequence) : "memory");
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(x.peers[x.rank] + exchange_arrived_offset(x, slot, t, row));
        bool ok = false;
        for (uint32_t spin = 0; spin < kExchangeSpinLimit; ++spin) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int32_t)(seen - sequence) >= 0) {
                ok = true;
                break;
            }
            if (spin > 64) __nanosleep(200);
        }
        if (!ok) {
            atomicOr(status, QM_DEVSTAT_TIMEOUT);
            shared2[1] = 1u;
        }
    }
    sync();
    if (live) {
        const bool timed_out = shared2[1] != 0u;
        const unsigned char* own = x.peers[x.rank];
        float big = -CUDART_INF_F;
        for (int g = 0; g < x.world; ++g)
            big = fmaxf(big, *reinterpret_cast<const volatile float*>(own + exchange_payload_offset(x, slot, g, row)));
        float acc = 0.0f, denom = 0.0f;
        for (int g = 0; g < x.world; ++g) {
            const volatile float* src = reinterpret_cast<const volatile float*>(own + exchange_payload_offset(x, slot, g, row));
            const float lg = src[1];
            if (!(lg > 0.0f)) continue;
            const float w = __expf(src[0] - big);
            denom = fmaf(w, lg, denom);
            acc = fmaf(w, src[2 + t], acc);
        }
        out_row[t] = (denom > 0.0f && !timed_out) ? (uint16_t)f32_to_bf16_bits(acc / denom) : (uint16_t)0;
    }
    sync();      // shared2 may be reused by the group's next row
}
