// Header-only C++ mirror of the reference engine's launcher surface for the
// talker attention path, on top of the C ABI (include/qm_attention.h).
//
// The reference reaches this path through private methods of
// NativeTalkerEngine (devices/rtx4090-24g/qwen3_tts_1_7b.cu, "17.cu"):
//     launch_qk_norm_rope_cache_m1   17.cu:17741
//     launch_attention               17.cu:17895
//     launch_rmsnorm x2, launch_rope_rows x2, scatter_prefill_cache   17.cu:16763-16798
//     reset_request                  17.cu:16607
//     max_cache                      17.cu:16650
// The methods below keep those names, argument meaning and error behaviour
// (a failed launch throws std::runtime_error carrying the operation name and
// the CUDA error text, as cuda_check does at 17.cu:17440-17453), so that
// decode_device() / prefill() read as before.  Differences that the batching
// and paging bring: scalars cache_position / cache_before become device
// arrays positions[] / seq_lens[], and the per-layer LayerCache objects become
// one pool addressed through a page table.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "qm_attention.h"

namespace qm {

inline void check(int32_t rc, const char* operation) {
    if (rc != QM_OK) throw std::runtime_error(std::string(operation) + ": " + qm_last_error_string());
}

// Move-only device allocation, the counterpart of the reference's DeviceBuffer (17.cu:8008-8060).
struct DeviceBuffer {
    void* pointer = nullptr;
    std::size_t bytes = 0;
    DeviceBuffer() = default;
    explicit DeviceBuffer(std::size_t n) : bytes(n) {
        if (cudaMalloc(&pointer, n ? n : 1) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : pointer(o.pointer), bytes(o.bytes) { o.pointer = nullptr; o.bytes = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) {
            if (pointer) cudaFree(pointer);
            pointer = o.pointer; bytes = o.bytes; o.pointer = nullptr; o.bytes = 0;
        }
        return *this;
    }
    ~DeviceBuffer() { if (pointer) cudaFree(pointer); }
    template <class T> T* as() const { return static_cast<T*>(pointer); }
};

class TalkerAttentionB200 {
public:
    // layers x num_pages pages of 64 tokens; rope_rows positions of RoPE table (theta 1e6 as the talker uses).
    TalkerAttentionB200(int layers, int num_pages, int q_heads, int kv_heads, int max_batch, int rope_rows,
                        cudaStream_t stream, double theta = 1000000.0)
        : q_heads_(q_heads), kv_heads_(kv_heads), rope_rows_(rope_rows), stream_(stream),
          rope_cos_(static_cast<std::size_t>(rope_rows) * QM_HEAD_DIM * 2),
          rope_sin_(static_cast<std::size_t>(rope_rows) * QM_HEAD_DIM * 2),
          workspace_(static_cast<std::size_t>(qm_decode_workspace_bytes(max_batch, kv_heads))) {
        int sm_count = 0, device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) throw std::runtime_error("cudaGetDevice failed");
        check(qm_validate_b200_device(device, &sm_count), "B200 device validation");
        check(qm_kv_pool_create(layers, num_pages, kv_heads, &pool_), "Talker KV pool allocation");
        check(qm_rope_table_fill(rope_cos_.as<uint16_t>(), rope_sin_.as<uint16_t>(), rope_rows, 0, theta, stream_),
              "Talker RoPE table");
        check(qm_decode_workspace_init(workspace_.pointer, static_cast<int64_t>(workspace_.bytes), stream_),
              "Talker decode workspace");
    }
    TalkerAttentionB200(const TalkerAttentionB200&) = delete;
    TalkerAttentionB200& operator=(const TalkerAttentionB200&) = delete;
    ~TalkerAttentionB200() { qm_kv_pool_destroy(pool_); }

    cudaStream_t stream() const { return stream_; }
    // Tokens one stream can hold with `max_pages` page-table entries.
    static int max_cache(int max_pages) { return max_pages * QM_PAGE_TOKENS; }

    void reset_request() { check(qm_kv_pool_reset(pool_, stream_), "Talker reset request"); }

    // Decode: per-head RMSNorm + RoPE of q and k, append of K (roped) and V (raw) at positions[s].
    void launch_qk_norm_rope_cache_m1(int layer, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                      const uint16_t* q_norm, const uint16_t* k_norm, const int32_t* positions,
                                      const int32_t* page_table, int max_pages, int batch, uint16_t* q_rotated) {
        check(qm_decode_append_rope(pool_, layer, q, k, v, q_norm, k_norm, rope_cos_.as<uint16_t>(),
                                    rope_sin_.as<uint16_t>(), rope_rows_, positions, page_table, max_pages, batch,
                                    q_heads_, 1.0e-6f, q_rotated, stream_),
              "Qingming QK norm/RoPE/cache launch");
    }

    // Decode attention (query_length == 1): seq_lens[s] = cache_before + 1 keys of stream s.
    void launch_attention(int layer, const uint16_t* query, const int32_t* seq_lens, const int32_t* page_table,
                          int max_pages, int batch, uint16_t* context) {
        check(qm_decode_attention(pool_, layer, query, seq_lens, page_table, max_pages, batch, q_heads_, context,
                                  workspace_.pointer, static_cast<int64_t>(workspace_.bytes), stream_),
              "Talker GQA2 M1 attention launch");
    }

    // launch_qk_norm_rope_cache_m1 + launch_attention of one layer in a single launch (same bits).
    void decode_step(int layer, const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* q_norm,
                     const uint16_t* k_norm, const int32_t* positions, const int32_t* page_table, int max_pages,
                     int batch, uint16_t* context) {
        check(qm_decode_step(pool_, layer, q, k, v, q_norm, k_norm, rope_cos_.as<uint16_t>(), rope_sin_.as<uint16_t>(),
                             rope_rows_, positions, page_table, max_pages, batch, q_heads_, 1.0e-6f, context,
                             workspace_.pointer, static_cast<int64_t>(workspace_.bytes), stream_),
              "Talker fused decode step launch");
    }

    // Prefill: launch_rmsnorm(q), launch_rmsnorm(k), launch_rope_rows(q), launch_rope_rows(k),
    // scatter_prefill_cache in one launch over packed varlen rows.
    void scatter_prefill_cache(int layer, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                               const uint16_t* q_norm, const uint16_t* k_norm, const int32_t* cu_seqlens,
                               const int32_t* page_table, int max_pages, int batch, int total_tokens,
                               uint16_t* q_rotated) {
        check(qm_prefill_append_rope_varlen(pool_, layer, q, k, v, q_norm, k_norm, rope_cos_.as<uint16_t>(),
                                            rope_sin_.as<uint16_t>(), rope_rows_, cu_seqlens, nullptr, page_table,
                                            max_pages, batch, total_tokens, q_heads_, 1.0e-6f, q_rotated, stream_),
              "Qingming prefill norm/RoPE/KV scatter launch");
    }

    // Prefill attention (query_length > 1), causal over the cache just written.
    void launch_attention(int layer, const uint16_t* query, const int32_t* cu_seqlens, const int32_t* page_table,
                          int max_pages, int batch, int total_tokens, int max_seqlen, uint16_t* context) {
        check(qm_prefill_attention_varlen(pool_, layer, query, cu_seqlens, nullptr, page_table, max_pages, batch,
                                          total_tokens, max_seqlen, q_heads_, context, stream_),
              "Talker generic fused attention launch");
    }

    // ---- the rest of the decoder layer at decode time (17.cu:17259-17386), `batch` token rows per launch
    void launch_rmsnorm(const uint16_t* x, const uint16_t* weight, uint16_t* out, int batch, int hidden) {
        check(qm_rmsnorm(x, weight, out, batch, hidden, 1.0e-6f, stream_), "Talker RMSNorm launch");
    }
    void launch_qkv_m1(const uint16_t* normed, const uint16_t* q_w, const uint16_t* q_b, const uint16_t* k_w,
                       const uint16_t* k_b, const uint16_t* v_w, const uint16_t* v_b, uint16_t* q, uint16_t* k,
                       uint16_t* v, int batch, int hidden) {
        check(qm_qkv_linear(pool_, normed, q_w, q_b, k_w, k_b, v_w, v_b, q, k, v, batch, hidden, q_heads_ * QM_HEAD_DIM,
                            kv_heads_ * QM_HEAD_DIM, stream_),
              "Qingming fused QKV launch");
    }
    void launch_linear_m1(const uint16_t* input, const uint16_t* weight, const uint16_t* bias, const uint16_t* residual,
                          uint16_t* output, int batch, int output_columns, int reduction_columns) {
        check(qm_linear(pool_, input, weight, bias, residual, output, batch, output_columns, reduction_columns, stream_),
              "Qingming M1 linear launch");
    }
    void launch_add_postnorm_m1(const uint16_t* hidden_rows, const uint16_t* attention, const uint16_t* norm_weight,
                                uint16_t* residual, uint16_t* normalized, int batch, int hidden) {
        check(qm_add_postnorm(hidden_rows, attention, norm_weight, residual, normalized, batch, hidden, 1.0e-6f, stream_),
              "Qingming add/postnorm launch");
    }
    void launch_gate_up_swiglu_m1(const uint16_t* input, const uint16_t* gate_w, const uint16_t* up_w, uint16_t* output,
                                  int batch, int hidden, int intermediate) {
        check(qm_gate_up_swiglu(pool_, input, gate_w, up_w, output, batch, hidden, intermediate, stream_),
              "Qingming fused gate/up/SwiGLU launch");
    }

    // linear_generic of the prefill loop (17.cu:16730-16860) for `rows` token rows; `residual` folds the loop's
    // launch_add into the same launch.
    void linear_generic(const uint16_t* input, const uint16_t* weight, const uint16_t* bias, const uint16_t* residual,
                        uint16_t* output, int rows, int output_columns, int reduction_columns) {
        check(qm_linear_rows(pool_, input, weight, bias, residual, output, rows, output_columns, reduction_columns, stream_),
              "Qingming generic linear launch");
    }
    // The prefill loop's gate and up projections plus launch_swiglu (17.cu:16833-16860) in one launch.
    void gate_up_swiglu_rows(const uint16_t* input, const uint16_t* gate_w, const uint16_t* up_w, uint16_t* output, int rows,
                             int hidden, int intermediate) {
        check(qm_gate_up_swiglu_rows(pool_, input, gate_w, up_w, output, rows, hidden, intermediate, stream_),
              "Qingming prefill gate/up/SwiGLU launch");
    }

    // NativeFinalHead::run_fast_device after the head projection (17.cu:14475-14560) for every stream at once:
    // cast, repetition penalty, token suppression, greedy argmax (top_k = 0) or top-k sampling, history record.
    void final_head_sample(const uint16_t* logits, int batch, int vocab, int32_t* history, int history_capacity,
                           const int32_t* generation_index, int flags, int top_k, float temperature, uint64_t* rng_state,
                           int32_t* codes, int eos_token = 2150) {
        check(qm_final_head_sample(pool_, logits, batch, vocab, history, history_capacity, generation_index, flags,
                                   eos_token, vocab - 1024, top_k, temperature, rng_state, codes, nullptr, stream_),
              "FinalHead sampling launch");
    }
    // gather_embedding_kernel (17.cu:8875) for a batch of rows.
    void gather_embeddings(const uint16_t* table, const int32_t* token_ids, int rows, int vocab, int hidden, uint16_t* out) {
        check(qm_embedding_gather(pool_, table, token_ids, rows, vocab, hidden, out, stream_), "embedding gather launch");
    }

    // QM_DEVSTAT_* bits raised by kernels since the last call (synchronises the stream).
    uint32_t device_status() {
        uint32_t bits = 0;
        check(qm_kv_pool_status(pool_, stream_, &bits), "Talker status read");
        return bits;
    }

    qm_kv_pool* pool() const { return pool_; }

private:
    int q_heads_, kv_heads_, rope_rows_;
    cudaStream_t stream_;
    qm_kv_pool* pool_ = nullptr;
    DeviceBuffer rope_cos_, rope_sin_, workspace_;
};

}  // namespace qm
