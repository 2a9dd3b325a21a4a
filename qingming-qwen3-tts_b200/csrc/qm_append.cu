// Fused per-head RMSNorm + RoPE + paged KV append, for decode (one token per
// stream) and packed varlen prefill.
//
// Stands in for talker_qk_norm_rope_cache_fused_kernel (17.cu:15412-15574) and
// for the prefill sequence rmsnorm_kernel x2 (17.cu:8295-8357), talker_rope_rows_kernel
// x2 (:15578-15673), talker_scatter_prefill_kv_kernel (:15677-15735).
//
// One warp owns one (token, head) row of 128 values: lane l holds dimensions
// 4l..4l+3 (one 8-byte load/store per row, 256 B per warp).  The arithmetic
// (qm_norm_rope.cuh) keeps the reference's five bf16 roundings per element,
// its rsqrtf and its sum-of-squares reduction order, so the output bits equal
// the reference kernel's.
#include "qm_norm_rope.cuh"

namespace {

constexpr int kAppendWarps = 8;

struct AppendArgs {
    const uint16_t* q;
    const uint16_t* k;
    const uint16_t* v;
    const uint16_t* q_norm_weight;
    const uint16_t* k_norm_weight;
    const uint16_t* rope_cos;
    const uint16_t* rope_sin;
    const int32_t* positions;     // decode: [batch]; prefill: start_positions or null
    const int32_t* cu_seqlens;    // null for decode
    const int32_t* cache_positions;   // decode only, optional: slot index in this pool (-1: do not append here)
    const int32_t* page_table;
    uint16_t* q_rot;
    uint16_t* key_pool;
    uint16_t* value_pool;
    uint32_t* status;
    long long rows_total;         // tokens * (q_heads + kv_heads)
    int rope_rows;
    int max_pages;
    int num_pages;
    int batch;
    int q_heads;
    int kv_heads;
    float epsilon;
};

// R consecutive head rows of the same token per warp (R divides q_heads + kv_heads): one stream / position
// lookup and R independent 256-byte loads in flight per warp.  With R = 8 the sums of squares of the eight rows
// are reduced together (reference_order_sum_of_squares_rows8), which takes a quarter of the shuffles.
template <int R>
__global__ void __launch_bounds__(kAppendWarps * 32, R == 8 ? 4 : 1) qm_norm_rope_append_kernel(const AppendArgs a) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long row0 = ((long long)blockIdx.x * kAppendWarps + (threadIdx.x >> 5)) * R;
    if (row0 >= a.rows_total) return;
    const int heads = a.q_heads + a.kv_heads;
    const int token = (int)(row0 / heads);
    const int slot0 = (int)(row0 % heads);

    // Which stream and position this packed token belongs to.
    int stream, position;
    if (a.cu_seqlens == nullptr) {
        stream = token;
        position = a.positions[token];
    } else {
        if (token >= a.cu_seqlens[a.batch]) return;   // padding rows past the last sequence
        int lo = 0, hi = a.batch;          // largest s with cu_seqlens[s] <= token
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (a.cu_seqlens[mid] <= token) lo = mid; else hi = mid;
        }
        stream = lo;
        position = (a.positions ? a.positions[stream] : 0) + (token - a.cu_seqlens[stream]);
    }
    if (position < 0 || position >= a.rope_rows) {
        if (lane == 0) atomicOr(a.status, QM_DEVSTAT_BAD_POS);
        return;
    }

    uint2 raw[R], vraw[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int slot = slot0 + r;
        const bool is_query = slot < a.q_heads;
        const int head = is_query ? slot : slot - a.q_heads;
        const uint16_t* source = is_query ? a.q + ((size_t)token * a.q_heads + head) * kHeadDim
                                          : a.k + ((size_t)token * a.kv_heads + head) * kHeadDim;
        raw[r] = *reinterpret_cast<const uint2*>(source + 4 * lane);
        // eight rows: the V rows are copied after the K rows are done, which keeps them out of the registers
        // while the sums of squares are reduced
        if constexpr (R != 8)
            vraw[r] = is_query ? make_uint2(0u, 0u)
                               : *reinterpret_cast<const uint2*>(a.v + ((size_t)token * a.kv_heads + head) * kHeadDim + 4 * lane);
    }
    const uint2 qwraw = *reinterpret_cast<const uint2*>(a.q_norm_weight + 4 * lane);
    const uint2 kwraw = *reinterpret_cast<const uint2*>(a.k_norm_weight + 4 * lane);
    const uint2 craw = *reinterpret_cast<const uint2*>(a.rope_cos + (size_t)position * kHeadDim + 4 * lane);
    const uint2 sraw = *reinterpret_cast<const uint2*>(a.rope_sin + (size_t)position * kHeadDim + 4 * lane);

    // Where this token's K/V rows go (same page and slot for every KV head).
    long long kv_row = -1;          // ((page * kv_heads) * 64 + slot) in rows of 128, head added below
    if (slot0 + R > a.q_heads) {
        // The RoPE row is the absolute position; the cache slot may be given separately when this pool
        // holds only a slice of the stream.
        const int cache_pos = a.cache_positions ? a.cache_positions[stream] : position;
        if (cache_pos < 0) {
            // this rank does not own the new token
        } else if (cache_pos >= a.max_pages * kPageTokens) {
            if (lane == 0) atomicOr(a.status, QM_DEVSTAT_BAD_POS);
        } else {
            const int page = a.page_table[(size_t)stream * a.max_pages + (cache_pos >> 6)];
            if (page < 0 || page >= a.num_pages) {
                if (lane == 0) atomicOr(a.status, QM_DEVSTAT_BAD_PAGE);
            } else {
                kv_row = (long long)page * a.kv_heads * kPageTokens + (cache_pos & 63);
            }
        }
    }

    // R == 8: lane l works out the inverse RMS of row (l & 7) once and the rows fetch it with one shuffle each
    float row_inverse = 0.0f;
    unsigned exact_rows = 0u;        // bit r: row r's sum of squares is not finite
    if constexpr (R == 8) {
        const float row_sum = reference_order_sum_of_squares_rows8(raw, lane);
        row_inverse = inverse_rms_of(row_sum, a.epsilon);
        exact_rows = __ballot_sync(0xffffffffu, !(row_sum < CUDART_INF_F)) & 0xffu;
    }

#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int slot = slot0 + r;
        const bool is_query = slot < a.q_heads;
        const int head = is_query ? slot : slot - a.q_heads;
        uint2 packed;
        if constexpr (R == 8)
            packed = norm_rope_row_with_inverse(raw[r], is_query ? qwraw : kwraw, craw, sraw, lane,
                                                __shfl_sync(0xffffffffu, row_inverse, r), (exact_rows >> r) & 1u);
        else
            packed = norm_rope_row(raw[r], is_query ? qwraw : kwraw, craw, sraw, lane, a.epsilon);

        if (is_query) {
            *reinterpret_cast<uint2*>(a.q_rot + ((size_t)token * a.q_heads + head) * kHeadDim + 4 * lane) = packed;
        } else if (kv_row >= 0) {
            const size_t dst = ((size_t)kv_row + (size_t)head * kPageTokens) * kHeadDim + 4 * lane;
            *reinterpret_cast<uint2*>(a.key_pool + dst) = packed;
            if constexpr (R != 8) *reinterpret_cast<uint2*>(a.value_pool + dst) = vraw[r];
        }
    }
    if constexpr (R == 8) {
        if (kv_row < 0) return;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int head = slot0 + r - a.q_heads;
            if (head >= 0) vraw[r] = *reinterpret_cast<const uint2*>(a.v + ((size_t)token * a.kv_heads + head) * kHeadDim + 4 * lane);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int head = slot0 + r - a.q_heads;
            if (head >= 0)
                *reinterpret_cast<uint2*>(a.value_pool + ((size_t)kv_row + (size_t)head * kPageTokens) * kHeadDim + 4 * lane) = vraw[r];
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Prefill form: persistent CTAs over a ring of bulk copies.
//
// The one-shot kernel above loads a warp's rows, then computes on them for several hundred instructions with
// nothing in flight; over thousands of prompt tokens neither the memory system nor the issue slots stay busy.
// Here a producer warp keeps a ring of stages filled with bulk copies (the q, k and v rows of a few consecutive
// tokens are three contiguous ranges), works out each token's stream, position and cache row while the copies
// fly, and twelve consumer warps take eight head rows of one token at a time out of shared memory.  The
// arithmetic is the same functions as above, so the bits are the same.
constexpr int kRingConsumerWarps = 12;
constexpr int kRingThreads = (kRingConsumerWarps + 1) * 32;
constexpr int kRingStages = 3;
constexpr int kRingStageBytes = 32 * 1024;
constexpr int kRingMaxTokens = 8;          // tokens per stage at most

struct RingSmem {
    static constexpr int kMetaOff = kRingStages * kRingStageBytes;                    // int4[kRingStages][kRingMaxTokens]
    static constexpr int kBarOff = kMetaOff + kRingStages * kRingMaxTokens * 16;      // full[kRingStages], empty[kRingStages]
    static constexpr int kTotal = kBarOff + 2 * kRingStages * 8;
};

__global__ void __launch_bounds__(kRingThreads, 2) qm_prefill_append_ring_kernel(const AppendArgs a, const int tokens,
                                                                                  const int group_tokens) {
    extern __shared__ __align__(128) unsigned char smem[];
    int4* meta = reinterpret_cast<int4*>(smem + RingSmem::kMetaOff);
    const uint32_t bar_base = smem_addr(smem + RingSmem::kBarOff);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kRingStages + s); };
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kRingStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kRingConsumerWarps);
        }
        fence_mbar_init();
    }
    pdl_trigger();
    __syncthreads();
    pdl_wait();

    const int groups = (tokens + group_tokens - 1) / group_tokens;
    const uint32_t q_token_bytes = (uint32_t)a.q_heads * kHeadDim * 2;
    const uint32_t kv_token_bytes = (uint32_t)a.kv_heads * kHeadDim * 2;
    const uint32_t k_region = (uint32_t)group_tokens * q_token_bytes;       // stage: [q rows][k rows][v rows]
    const uint32_t v_region = k_region + (uint32_t)group_tokens * kv_token_bytes;
    bool dead = false;

    if (warp == kRingConsumerWarps) {
        // ------------------------------------------------------------------------------------------ producer
        const int packed_tokens = a.cu_seqlens[a.batch];
        int issued = 0;
        for (int g = blockIdx.x; g < groups; g += gridDim.x, ++issued) {
            const int stage = issued % kRingStages;
            const int token0 = g * group_tokens;
            const int n = tokens - token0 < group_tokens ? tokens - token0 : group_tokens;
            // lane t: where token (token0 + t) goes.  x = RoPE row or -1 (skip the token), (y, z) = cache row of KV
            // head 0 in rows of 128 values, or -1
            int4 m = make_int4(-1, -1, -1, 0);
            if (lane < n && token0 + lane < packed_tokens) {
                const int token = token0 + lane;
                int lo = 0, hi = a.batch;          // largest s with cu_seqlens[s] <= token
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (a.cu_seqlens[mid] <= token) lo = mid; else hi = mid;
                }
                const int position = (a.positions ? a.positions[lo] : 0) + (token - a.cu_seqlens[lo]);
                if (position < 0 || position >= a.rope_rows) {
                    atomicOr(a.status, QM_DEVSTAT_BAD_POS);
                } else {
                    m.x = position;
                    if (position >= a.max_pages * kPageTokens) {
                        atomicOr(a.status, QM_DEVSTAT_BAD_POS);
                    } else {
                        const int page = a.page_table[(size_t)lo * a.max_pages + (position >> 6)];
                        if (page < 0 || page >= a.num_pages) {
                            atomicOr(a.status, QM_DEVSTAT_BAD_PAGE);
                        } else {
                            const long long kv_row = (long long)page * a.kv_heads * kPageTokens + (position & 63);
                            m.y = (int)(kv_row & 0xffffffffLL);
                            m.z = (int)(kv_row >> 32);
                            m.w = 1;
                        }
                    }
                }
            }
            int ok = 1;
            if (lane == 0) {
                const uint32_t parity = ((issued / kRingStages) & 1) ^ 1;
                if (!mbar_wait_bounded(empty_bar(stage), parity, dead)) {
                    atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                    ok = 0;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;                            // the consumers run into their own bounded waits
            if (lane < kRingMaxTokens) meta[stage * kRingMaxTokens + lane] = m;
            __syncwarp();
            if (lane == 0) {
                const uint32_t dst = smem_addr(smem + stage * kRingStageBytes);
                mbar_arrive_expect_tx(full_bar(stage), (uint32_t)n * (q_token_bytes + 2 * kv_token_bytes));
                bulk_copy_g2s(dst, a.q + (size_t)token0 * a.q_heads * kHeadDim, (uint32_t)n * q_token_bytes, full_bar(stage));
                bulk_copy_g2s(dst + k_region, a.k + (size_t)token0 * a.kv_heads * kHeadDim, (uint32_t)n * kv_token_bytes,
                              full_bar(stage));
                bulk_copy_g2s(dst + v_region, a.v + (size_t)token0 * a.kv_heads * kHeadDim, (uint32_t)n * kv_token_bytes,
                              full_bar(stage));
            }
        }
        // No copy may be in flight when the CTA retires: the consumers wait for every stage unless one of their
        // waits gave up, so wait (bounded) for the last stages issued.
        if (lane == 0) {
            bool ignore = false;
            const int first = issued > kRingStages ? issued - kRingStages : 0;
            for (int i = first; i < issued; ++i) mbar_wait_bounded(full_bar(i % kRingStages), (i / kRingStages) & 1, ignore);
        }
        return;
    }

    // --------------------------------------------------------------------------------------------- consumers
    const uint2 qwraw = *reinterpret_cast<const uint2*>(a.q_norm_weight + 4 * lane);
    const uint2 kwraw = *reinterpret_cast<const uint2*>(a.k_norm_weight + 4 * lane);
    const int octets_per_token = (a.q_heads + a.kv_heads) >> 3;
    int taken = 0;
    for (int g = blockIdx.x; g < groups; g += gridDim.x, ++taken) {
        const int stage = taken % kRingStages;
        const int token0 = g * group_tokens;
        const int n = tokens - token0 < group_tokens ? tokens - token0 : group_tokens;
        if (!mbar_wait_bounded(full_bar(stage), (taken / kRingStages) & 1, dead) && lane == 0)
            atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
        const unsigned char* base = smem + stage * kRingStageBytes;
        for (int o = warp; o < n * octets_per_token && !dead; o += kRingConsumerWarps) {
            const int t = o / octets_per_token;
            const int slot0 = (o - t * octets_per_token) * 8;
            const int4 m = meta[stage * kRingMaxTokens + t];
            if (m.x < 0) continue;
            const int token = token0 + t;
            const bool is_query = slot0 < a.q_heads;         // q_heads is a multiple of 8: the same for all eight rows
            const int head0 = is_query ? slot0 : slot0 - a.q_heads;
            const unsigned char* rows = is_query ? base + ((size_t)t * a.q_heads + head0) * (kHeadDim * 2)
                                                 : base + k_region + ((size_t)t * a.kv_heads + head0) * (kHeadDim * 2);
            uint2 raw[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) raw[r] = *reinterpret_cast<const uint2*>(rows + r * (kHeadDim * 2) + 8 * lane);
            const uint2 craw = *reinterpret_cast<const uint2*>(a.rope_cos + (size_t)m.x * kHeadDim + 4 * lane);
            const uint2 sraw = *reinterpret_cast<const uint2*>(a.rope_sin + (size_t)m.x * kHeadDim + 4 * lane);
            const float row_sum = reference_order_sum_of_squares_rows8(raw, lane);      // of row (lane & 7)
            const float row_inverse = inverse_rms_of(row_sum, a.epsilon);
            const unsigned exact_rows = __ballot_sync(0xffffffffu, !(row_sum < CUDART_INF_F)) & 0xffu;
            const long long kv_row = m.w ? (((long long)m.z << 32) | (uint32_t)m.y) : -1;
            if (is_query) {
                uint16_t* dst = a.q_rot + ((size_t)token * a.q_heads + head0) * kHeadDim + 4 * lane;
#pragma unroll
                for (int r = 0; r < 8; ++r)
                    *reinterpret_cast<uint2*>(dst + r * kHeadDim) =
                        norm_rope_row_with_inverse(raw[r], qwraw, craw, sraw, lane, __shfl_sync(0xffffffffu, row_inverse, r),
                                                   (exact_rows >> r) & 1u);
            } else {
                const size_t dst0 = ((size_t)(kv_row < 0 ? 0 : kv_row) + (size_t)head0 * kPageTokens) * kHeadDim + 4 * lane;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const uint2 packed =
                        norm_rope_row_with_inverse(raw[r], kwraw, craw, sraw, lane, __shfl_sync(0xffffffffu, row_inverse, r),
                                                   (exact_rows >> r) & 1u);
                    if (kv_row >= 0) *reinterpret_cast<uint2*>(a.key_pool + dst0 + (size_t)r * kPageTokens * kHeadDim) = packed;
                }
                if (kv_row >= 0) {
                    const unsigned char* vrows = base + v_region + ((size_t)t * a.kv_heads + head0) * (kHeadDim * 2);
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        *reinterpret_cast<uint2*>(a.value_pool + dst0 + (size_t)r * kPageTokens * kHeadDim) =
                            *reinterpret_cast<const uint2*>(vrows + r * (kHeadDim * 2) + 8 * lane);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
    }
}

bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

int32_t launch_append(qm_kv_pool* pool, int32_t layer, const AppendArgs& proto, long long tokens, cudaStream_t stream) {
    AppendArgs a = proto;
    a.key_pool = qm_kv_pool_key_ptr(pool, layer);
    a.value_pool = qm_kv_pool_value_ptr(pool, layer);
    a.status = pool->status_dev;
    a.num_pages = pool->num_pages;
    a.kv_heads = pool->kv_heads;
    a.rows_total = tokens * (a.q_heads + a.kv_heads);
    if (a.rows_total == 0) return QM_OK;
    const int heads = a.q_heads + a.kv_heads;
    // Packed prompts whose rows come in eights and whose inputs a bulk copy can read take the ring kernel.
    const size_t token_bytes = (size_t)(a.q_heads + 2 * a.kv_heads) * kHeadDim * 2;
    if (a.cu_seqlens != nullptr && a.cache_positions == nullptr && a.q_heads % 8 == 0 && a.kv_heads % 8 == 0 &&
        token_bytes <= (size_t)kRingStageBytes && !misaligned16(a.q) && !misaligned16(a.k) && !misaligned16(a.v) &&
        tokens <= 0x7fffffffLL) {
        int group_tokens = (int)((size_t)kRingStageBytes / token_bytes);
        if (group_tokens > kRingMaxTokens) group_tokens = kRingMaxTokens;
        static thread_local int attr_device = -1;
        if (attr_device != pool->device) {
            QM_CUDA_TRY(cudaFuncSetAttribute(qm_prefill_append_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             RingSmem::kTotal),
                        "raise prefill append shared memory");
            attr_device = pool->device;
        }
        const long long groups = (tokens + group_tokens - 1) / group_tokens;
        const long long resident = 2LL * pool->sm_count;
        const dim3 grid((unsigned)(groups < resident ? groups : resident));
        QM_CUDA_TRY(qm_launch(qm_prefill_append_ring_kernel, grid, dim3(kRingThreads), RingSmem::kTotal, stream, a, (int)tokens,
                              group_tokens),
                    "prefill QK norm/RoPE/cache launch");
        QM_CUDA_TRY(cudaGetLastError(), "prefill QK norm/RoPE/cache launch");
        return QM_OK;
    }
    const int rows_per_warp = heads % 8 == 0 ? 8 : (heads % 4 == 0 ? 4 : (heads % 2 == 0 ? 2 : 1));
    const long long warps = (a.rows_total + rows_per_warp - 1) / rows_per_warp;
    const long long blocks = (warps + kAppendWarps - 1) / kAppendWarps;
    if (blocks > 0x7fffffffLL) return qm_fail(QM_ECAPACITY, "too many rows for one append launch");
    const dim3 grid((unsigned)blocks), block(kAppendWarps * 32);
    if (rows_per_warp == 8)
        QM_CUDA_TRY(qm_launch(qm_norm_rope_append_kernel<8>, grid, block, 0, stream, a), "QK norm/RoPE/cache launch");
    else if (rows_per_warp == 4)
        QM_CUDA_TRY(qm_launch(qm_norm_rope_append_kernel<4>, grid, block, 0, stream, a), "QK norm/RoPE/cache launch");
    else if (rows_per_warp == 2)
        QM_CUDA_TRY(qm_launch(qm_norm_rope_append_kernel<2>, grid, block, 0, stream, a), "QK norm/RoPE/cache launch");
    else
        QM_CUDA_TRY(qm_launch(qm_norm_rope_append_kernel<1>, grid, block, 0, stream, a), "QK norm/RoPE/cache launch");
    QM_CUDA_TRY(cudaGetLastError(), "QK norm/RoPE/cache launch");
    return QM_OK;
}

bool misaligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) != 0; }

int32_t decode_append(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                      const uint16_t* q_norm_weight, const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                      const uint16_t* rope_sin, int32_t rope_rows, const int32_t* positions,
                      const int32_t* cache_positions, const int32_t* page_table, int32_t max_pages, int32_t batch,
                      int32_t q_heads, float epsilon, uint16_t* q_rot, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (layer < 0 || layer >= pool->layers) return qm_fail(QM_EINVAL, "layer out of range");
    if (!q || !k || !v || !q_norm_weight || !k_norm_weight || !rope_cos || !rope_sin || !positions || !page_table ||
        !q_rot)
        return qm_fail(QM_EINVAL, "null tensor pointer");
    if (misaligned8(q) || misaligned8(k) || misaligned8(v) || misaligned8(q_norm_weight) || misaligned8(k_norm_weight) ||
        misaligned8(rope_cos) || misaligned8(rope_sin) || misaligned8(q_rot))
        return qm_fail(QM_EINVAL, "bf16 tensors must be 8-byte aligned");
    if (batch < 0 || q_heads < 1 || max_pages < 1 || rope_rows < 1) return qm_fail(QM_EINVAL, "invalid geometry");
    AppendArgs a{};
    a.q = q; a.k = k; a.v = v;
    a.q_norm_weight = q_norm_weight; a.k_norm_weight = k_norm_weight;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.positions = positions; a.cu_seqlens = nullptr; a.page_table = page_table;
    a.cache_positions = cache_positions;
    a.q_rot = q_rot;
    a.rope_rows = rope_rows; a.max_pages = max_pages; a.batch = batch; a.q_heads = q_heads; a.epsilon = epsilon;
    return launch_append(pool, layer, a, batch, static_cast<cudaStream_t>(stream));
}

}  // namespace

extern "C" {

int32_t qm_decode_append_rope(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                              const uint16_t* v, const uint16_t* q_norm_weight, const uint16_t* k_norm_weight,
                              const uint16_t* rope_cos, const uint16_t* rope_sin, int32_t rope_rows,
                              const int32_t* positions, const int32_t* page_table, int32_t max_pages,
                              int32_t batch, int32_t q_heads, float epsilon, uint16_t* q_rot, void* stream) {
    return decode_append(pool, layer, q, k, v, q_norm_weight, k_norm_weight, rope_cos, rope_sin, rope_rows, positions,
                         nullptr, page_table, max_pages, batch, q_heads, epsilon, q_rot, stream);
}

int32_t qm_decode_append_rope_sliced(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                                     const uint16_t* v, const uint16_t* q_norm_weight,
                                     const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                                     const uint16_t* rope_sin, int32_t rope_rows, const int32_t* positions,
                                     const int32_t* cache_positions, const int32_t* page_table,
                                     int32_t max_pages, int32_t batch, int32_t q_heads, float epsilon,
                                     uint16_t* q_rot, void* stream) {
    if (!cache_positions) return qm_fail(QM_EINVAL, "cache_positions is null");
    return decode_append(pool, layer, q, k, v, q_norm_weight, k_norm_weight, rope_cos, rope_sin, rope_rows, positions,
                         cache_positions, page_table, max_pages, batch, q_heads, epsilon, q_rot, stream);
}

int32_t qm_prefill_append_rope_varlen(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                                      const uint16_t* v, const uint16_t* q_norm_weight,
                                      const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                                      const uint16_t* rope_sin, int32_t rope_rows, const int32_t* cu_seqlens,
                                      const int32_t* start_positions, const int32_t* page_table,
                                      int32_t max_pages, int32_t batch, int32_t total_tokens, int32_t q_heads,
                                      float epsilon, uint16_t* q_rot, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (layer < 0 || layer >= pool->layers) return qm_fail(QM_EINVAL, "layer out of range");
    if (!q || !k || !v || !q_norm_weight || !k_norm_weight || !rope_cos || !rope_sin || !cu_seqlens || !page_table ||
        !q_rot)
        return qm_fail(QM_EINVAL, "null tensor pointer");
    if (misaligned8(q) || misaligned8(k) || misaligned8(v) || misaligned8(q_norm_weight) || misaligned8(k_norm_weight) ||
        misaligned8(rope_cos) || misaligned8(rope_sin) || misaligned8(q_rot))
        return qm_fail(QM_EINVAL, "bf16 tensors must be 8-byte aligned");
    if (batch < 1 || total_tokens < 0 || q_heads < 1 || max_pages < 1 || rope_rows < 1)
        return qm_fail(QM_EINVAL, "invalid geometry");
    AppendArgs a{};
    a.q = q; a.k = k; a.v = v;
    a.q_norm_weight = q_norm_weight; a.k_norm_weight = k_norm_weight;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.positions = start_positions; a.cu_seqlens = cu_seqlens; a.page_table = page_table;
    a.q_rot = q_rot;
    a.rope_rows = rope_rows; a.max_pages = max_pages; a.batch = batch; a.q_heads = q_heads; a.epsilon = epsilon;
    return launch_append(pool, layer, a, total_tokens, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
