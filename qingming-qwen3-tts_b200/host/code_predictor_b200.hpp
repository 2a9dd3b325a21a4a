// Header-only C++ driver of the code predictor's frame for a batch of streams, on the launcher mirror.
//
// Mirrors PersistentPredictor::capture_step / capture_graph of the reference
// (devices/rtx4090-24g/qwen3_tts_1_7b.cu "17.cu":13616-13935): per audio frame 15 steps of a 5-layer decoder (hidden
// 1024, 16 query / 8 KV heads of 128, SwiGLU 3072, vocabulary 2048, at most 16 cached positions).  Step 0 feeds TWO
// rows per stream - the talker's last hidden state and the embedding of the frame's first code - every later step
// one row, the embedding of the code just drawn; each step ends with the final norm, that step's own head, a draw
// (argmax_bf16_kernel or gpu_sample_topk_bf16_kernel) and that step's own embedding table
// (gather_predictor_embedding_kernel).  The decoder layer has the talker layer's structure, so a one-row step is
// the same seven launches per layer as a talker decode step.
//
// The reference runs the two rows of step 0 through its staged many-row kernels (linear, rmsnorm, rope,
// update_cache, attention; "the exact staged 2-row anchor", 17.cu:13661) and the later steps through its one-row
// kernels.  Both spellings are here: FirstStep::kStagedRows sends the two rows of every stream through this
// library's many-row path (packed varlen prefill with two tokens per stream), FirstStep::kTwoPositions through the
// one-row path twice (positions 0 and 1) - the same causal attention, fewer and smaller launches.
// Nothing synchronises with the host, so a frame can be captured as one CUDA graph as the reference does.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <vector>

#include "talker_engine_b200.hpp"

namespace qm {

// Device pointers of the predictor's weights, named as the reference's PredictorWeights.
struct CodePredictorWeights {
    int outer_hidden = 2048;      // kOuterHidden: width of the talker's hidden state and of the code embeddings
    int hidden = 1024;            // kHidden
    int intermediate = 3072;      // kIntermediate
    int vocab = 2048;             // kVocab
    int steps = 15;               // kSteps
    int q_heads = 16, kv_heads = 8;
    const uint16_t* projection_weight = nullptr;     // [hidden][outer_hidden]
    const uint16_t* projection_bias = nullptr;       // [hidden]
    std::vector<TalkerLayerWeights> layers;          // kLayers = 5
    const uint16_t* final_norm = nullptr;            // [hidden]
    std::vector<const uint16_t*> lm_heads;           // per step [vocab][hidden]
    std::vector<const uint16_t*> embeddings;         // per step [vocab][outer_hidden]
};

class CodePredictorB200 {
public:
    enum class FirstStep { kTwoPositions, kStagedRows };
    static constexpr int kMaxCache = 16;             // positions a frame uses: 2 + 14

    CodePredictorB200(const CodePredictorWeights& weights, int streams, cudaStream_t stream)
        : w_(weights), streams_(streams), stream_(stream),
          // 16 positions fit one 64-token page per stream; the step inputs are at most two rows per stream
          attention_((int)weights.layers.size(), streams, weights.q_heads, weights.kv_heads, streams, 64, stream) {
        if (streams < 1 || w_.layers.empty() || (int)w_.lm_heads.size() < w_.steps || (int)w_.embeddings.size() < w_.steps ||
            w_.steps + 1 > kMaxCache)
            throw std::runtime_error("code predictor weights are incomplete");
        const std::size_t rows = 2 * (std::size_t)streams;
        const std::size_t h = (std::size_t)w_.hidden * 2, qd = (std::size_t)w_.q_heads * QM_HEAD_DIM * 2,
                          kd = (std::size_t)w_.kv_heads * QM_HEAD_DIM * 2;
        free_input_ = DeviceBuffer(rows * (std::size_t)w_.outer_hidden * 2);
        hidden_a_ = DeviceBuffer(rows * h); hidden_b_ = DeviceBuffer(rows * h); norm_ = DeviceBuffer(rows * h);
        q_ = DeviceBuffer(rows * qd); k_ = DeviceBuffer(rows * kd); v_ = DeviceBuffer(rows * kd);
        q_rotated_ = DeviceBuffer(rows * qd); context_ = DeviceBuffer(rows * qd);
        attention_output_ = DeviceBuffer(rows * h); residual_ = DeviceBuffer(rows * h); post_norm_ = DeviceBuffer(rows * h);
        swiglu_ = DeviceBuffer(rows * (std::size_t)w_.intermediate * 2); final_norm_ = DeviceBuffer(rows * h);
        last_rows_ = DeviceBuffer((std::size_t)streams * h);
        logits_ = DeviceBuffer((std::size_t)streams * (std::size_t)w_.vocab * 2);
        next_input_ = DeviceBuffer((std::size_t)streams * (std::size_t)w_.outer_hidden * 2);
        codes_ = DeviceBuffer((std::size_t)w_.steps * (std::size_t)streams * sizeof(int32_t));
        // constant index arrays: positions[p][s] = p, one page per stream, two-row packing of the staged first step
        std::vector<int32_t> positions((std::size_t)kMaxCache * streams), table((std::size_t)streams), cu((std::size_t)streams + 1),
            last((std::size_t)streams);
        for (int p = 0; p < kMaxCache; ++p)
            for (int s = 0; s < streams; ++s) positions[(std::size_t)p * streams + s] = p;
        for (int s = 0; s < streams; ++s) {
            table[(std::size_t)s] = s;
            cu[(std::size_t)s] = 2 * s;
            last[(std::size_t)s] = 2 * s + 1;
        }
        cu[(std::size_t)streams] = 2 * streams;
        positions_ = upload(positions);
        page_table_ = upload(table);
        cu_seqlens_ = upload(cu);
        last_row_index_ = upload(last);
    }

    // One frame: talker_hidden and first_code_embedding are [streams][outer_hidden] bf16 device rows.  Greedy when
    // top_k is 0, else top-k sampling from rng_state[stream] (device SplitMix64 states).  Returns the device
    // pointer of codes [steps][streams] int32; nothing is synchronised.  logits_trace, when not null, receives every
    // step's logits [steps][streams][vocab] (what the reference's validation mode keeps).
    const int32_t* frame(const uint16_t* talker_hidden, const uint16_t* first_code_embedding, uint64_t* rng_state = nullptr,
                         int top_k = 0, float temperature = 0.9f, FirstStep first = FirstStep::kTwoPositions,
                         uint16_t* logits_trace = nullptr) {
        if (!talker_hidden || !first_code_embedding) throw std::runtime_error("code predictor input is null");
        const uint16_t* last_hidden;
        if (first == FirstStep::kStagedRows) {
            last_hidden = staged_first_step(talker_hidden, first_code_embedding);
        } else {
            token_step(talker_hidden, 0);                        // first row of step 0: only fills the cache
            const uint16_t* cur = token_step(first_code_embedding, 1);
            attention_.launch_rmsnorm(cur, w_.final_norm, final_norm_.as<uint16_t>(), streams_, w_.hidden);
            last_hidden = final_norm_.as<uint16_t>();
        }
        for (int step = 0; step < w_.steps; ++step) {
            if (step > 0) {
                const uint16_t* cur = token_step(next_input_.as<uint16_t>(), step + 1);
                attention_.launch_rmsnorm(cur, w_.final_norm, final_norm_.as<uint16_t>(), streams_, w_.hidden);
                last_hidden = final_norm_.as<uint16_t>();
            }
            attention_.launch_linear_m1(last_hidden, w_.lm_heads[(std::size_t)step], nullptr, nullptr, logits_.as<uint16_t>(), streams_,
                                        w_.vocab, w_.hidden);
            if (logits_trace &&
                cudaMemcpyAsync(logits_trace + (std::size_t)step * streams_ * w_.vocab, logits_.pointer,
                                (std::size_t)streams_ * w_.vocab * 2, cudaMemcpyDeviceToDevice, stream_) != cudaSuccess)
                throw std::runtime_error("code predictor logits trace copy failed");
            int32_t* step_codes = codes_.as<int32_t>() + (std::size_t)step * streams_;
            check(qm_final_head_sample(attention_.pool(), logits_.as<uint16_t>(), streams_, w_.vocab, nullptr, 0, nullptr, 0, 0, 0,
                                       top_k, temperature, rng_state, step_codes, nullptr, stream_),
                  "Predictor sampling launch");
            attention_.gather_embeddings(w_.embeddings[(std::size_t)step], step_codes, streams_, w_.vocab, w_.outer_hidden,
                                         next_input_.as<uint16_t>());
        }
        return codes_.as<int32_t>();
    }

    const int32_t* codes() const { return codes_.as<int32_t>(); }
    const uint16_t* logits() const { return logits_.as<uint16_t>(); }      // of the last step
    TalkerAttentionB200& attention() { return attention_; }

private:
    template <class T>
    DeviceBuffer upload(const std::vector<T>& host) {
        DeviceBuffer d(host.size() * sizeof(T));
        if (cudaMemcpy(d.pointer, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess)
            throw std::runtime_error("code predictor upload failed");
        return d;
    }

    // One row per stream at `position` through the projection and the layers (capture_step with rows == 1).
    const uint16_t* token_step(const uint16_t* row_input, int position) {
        const int b = streams_, hidden = w_.hidden;
        const int32_t* positions = positions_.as<int32_t>() + (std::size_t)position * b;
        uint16_t* cur = hidden_a_.as<uint16_t>();
        uint16_t* nxt = hidden_b_.as<uint16_t>();
        attention_.launch_linear_m1(row_input, w_.projection_weight, w_.projection_bias, nullptr, cur, b, hidden, w_.outer_hidden);
        for (std::size_t li = 0; li < w_.layers.size(); ++li) {
            const TalkerLayerWeights& layer = w_.layers[li];
            attention_.launch_rmsnorm(cur, layer.input_norm, norm_.as<uint16_t>(), b, hidden);
            attention_.launch_qkv_m1(norm_.as<uint16_t>(), layer.q_weight, layer.q_bias, layer.k_weight, layer.k_bias, layer.v_weight,
                                     layer.v_bias, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(), b, hidden);
            attention_.decode_step((int)li, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(), layer.q_norm, layer.k_norm, positions,
                                   page_table_.as<int32_t>(), 1, b, context_.as<uint16_t>());
            attention_.launch_linear_m1(context_.as<uint16_t>(), layer.o_weight, layer.o_bias, nullptr, attention_output_.as<uint16_t>(), b,
                                        hidden, w_.q_heads * QM_HEAD_DIM);
            attention_.launch_add_postnorm_m1(cur, attention_output_.as<uint16_t>(), layer.post_norm, residual_.as<uint16_t>(),
                                              post_norm_.as<uint16_t>(), b, hidden);
            attention_.launch_gate_up_swiglu_m1(post_norm_.as<uint16_t>(), layer.gate_weight, layer.up_weight, swiglu_.as<uint16_t>(), b,
                                                hidden, w_.intermediate);
            attention_.launch_linear_m1(swiglu_.as<uint16_t>(), layer.down_weight, nullptr, residual_.as<uint16_t>(), nxt, b, hidden,
                                        w_.intermediate);
            std::swap(cur, nxt);
        }
        return cur;
    }

    // Step 0 with both rows of every stream at once, through the many-row kernels (capture_step with rows == 2).
    // Returns the normalised last row of every stream, [streams][hidden].
    const uint16_t* staged_first_step(const uint16_t* talker_hidden, const uint16_t* first_code_embedding) {
        const int b = streams_, rows = 2 * streams_, hidden = w_.hidden;
        const std::size_t row_bytes = (std::size_t)w_.outer_hidden * 2;
        // free_input_: rows 2s = talker hidden of stream s, 2s + 1 = embedding of its first code (17.cu:11980-12010)
        if (cudaMemcpy2DAsync(free_input_.pointer, 2 * row_bytes, talker_hidden, row_bytes, row_bytes, (std::size_t)b,
                              cudaMemcpyDeviceToDevice, stream_) != cudaSuccess ||
            cudaMemcpy2DAsync(free_input_.as<unsigned char>() + row_bytes, 2 * row_bytes, first_code_embedding, row_bytes, row_bytes,
                              (std::size_t)b, cudaMemcpyDeviceToDevice, stream_) != cudaSuccess)
            throw std::runtime_error("code predictor input interleave failed");
        uint16_t* cur = hidden_a_.as<uint16_t>();
        uint16_t* nxt = hidden_b_.as<uint16_t>();
        attention_.linear_generic(free_input_.as<uint16_t>(), w_.projection_weight, w_.projection_bias, nullptr, cur, rows, hidden,
                                  w_.outer_hidden);
        const int qd = w_.q_heads * QM_HEAD_DIM, kd = w_.kv_heads * QM_HEAD_DIM;
        for (std::size_t li = 0; li < w_.layers.size(); ++li) {
            const TalkerLayerWeights& layer = w_.layers[li];
            attention_.launch_rmsnorm(cur, layer.input_norm, norm_.as<uint16_t>(), rows, hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.q_weight, layer.q_bias, nullptr, q_.as<uint16_t>(), rows, qd, hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.k_weight, layer.k_bias, nullptr, k_.as<uint16_t>(), rows, kd, hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.v_weight, layer.v_bias, nullptr, v_.as<uint16_t>(), rows, kd, hidden);
            attention_.scatter_prefill_cache((int)li, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(), layer.q_norm, layer.k_norm,
                                             cu_seqlens_.as<int32_t>(), page_table_.as<int32_t>(), 1, b, rows, q_rotated_.as<uint16_t>());
            attention_.launch_attention((int)li, q_rotated_.as<uint16_t>(), cu_seqlens_.as<int32_t>(), page_table_.as<int32_t>(), 1, b, rows,
                                        2, context_.as<uint16_t>());
            attention_.linear_generic(context_.as<uint16_t>(), layer.o_weight, layer.o_bias, cur, residual_.as<uint16_t>(), rows, hidden, qd);
            attention_.launch_rmsnorm(residual_.as<uint16_t>(), layer.post_norm, post_norm_.as<uint16_t>(), rows, hidden);
            attention_.gate_up_swiglu_rows(post_norm_.as<uint16_t>(), layer.gate_weight, layer.up_weight, swiglu_.as<uint16_t>(), rows,
                                           hidden, w_.intermediate);
            attention_.linear_generic(swiglu_.as<uint16_t>(), layer.down_weight, nullptr, residual_.as<uint16_t>(), nxt, rows, hidden,
                                      w_.intermediate);
            std::swap(cur, nxt);
        }
        attention_.launch_rmsnorm(cur, w_.final_norm, final_norm_.as<uint16_t>(), rows, hidden);
        // the head reads the LAST of the two rows ((rows - 1) * kVocab in the reference's sampler call, 17.cu:13880)
        attention_.gather_embeddings(final_norm_.as<uint16_t>(), last_row_index_.as<int32_t>(), b, rows, hidden, last_rows_.as<uint16_t>());
        return last_rows_.as<uint16_t>();
    }

    CodePredictorWeights w_;
    int streams_;
    cudaStream_t stream_;
    TalkerAttentionB200 attention_;
    DeviceBuffer free_input_, hidden_a_, hidden_b_, norm_, q_, k_, v_, q_rotated_, context_, attention_output_, residual_, post_norm_,
        swiglu_, final_norm_, last_rows_, logits_, next_input_, codes_, positions_, page_table_, cu_seqlens_, last_row_index_;
};

}  // namespace qm
