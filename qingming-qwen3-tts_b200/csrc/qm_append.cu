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
// lookup and R independent 256-byte loads in flight per warp.
template <int R>
__global__ void __launch_bounds__(kAppendWarps * 32) qm_norm_rope_append_kernel(const AppendArgs a) {
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
        vraw[r] = is_query ? make_uint2(0u, 0u)
                           : *reinterpret_cast<const uint2*>(a.v + ((size_t)token * a.kv_heads + head) * kHeadDim + 4 * lane);
    }
    const uint2 qwraw = *reinterpret_cast<const uint2*>(a.q_norm_weight + 4 * lane);
    const uint2 kwraw = *reinterpret_cast<const uint2*>(a.k_norm_weight + 4 * lane);
    const uint2 craw = *reinterpret_cast<const uint2*>(a.rope_cos + (size_t)position * kHeadDim + 4 * lane);
    const uint2 sraw = *reinterpret_cast<const uint2*>(a.rope_sin + (size_t)position * kHeadDim + 4 * lane);
    const float c[4] = {bf16_lo(craw.x), bf16_hi(craw.x), bf16_lo(craw.y), bf16_hi(craw.y)};
    const float s[4] = {bf16_lo(sraw.x), bf16_hi(sraw.x), bf16_lo(sraw.y), bf16_hi(sraw.y)};

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

#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int slot = slot0 + r;
        const bool is_query = slot < a.q_heads;
        const int head = is_query ? slot : slot - a.q_heads;
        const uint2 packed = norm_rope_row(raw[r], is_query ? qwraw : kwraw, c, s, lane, a.epsilon);

        if (is_query) {
            *reinterpret_cast<uint2*>(a.q_rot + ((size_t)token * a.q_heads + head) * kHeadDim + 4 * lane) = packed;
        } else if (kv_row >= 0) {
            const size_t dst = ((size_t)kv_row + (size_t)head * kPageTokens) * kHeadDim + 4 * lane;
            *reinterpret_cast<uint2*>(a.key_pool + dst) = packed;
            *reinterpret_cast<uint2*>(a.value_pool + dst) = vraw[r];
        }
    }
}

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
    const int rows_per_warp = heads % 4 == 0 ? 4 : (heads % 2 == 0 ? 2 : 1);
    const long long warps = (a.rows_total + rows_per_warp - 1) / rows_per_warp;
    const long long blocks = (warps + kAppendWarps - 1) / kAppendWarps;
    if (blocks > 0x7fffffffLL) return qm_fail(QM_ECAPACITY, "too many rows for one append launch");
    const dim3 grid((unsigned)blocks), block(kAppendWarps * 32);
    if (rows_per_warp == 4)
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
