// Header-only C++ drivers of the talker decoder on top of the launcher mirror (talker_attention_b200.hpp):
// the loops that order a layer's launches over all layers, with the reference's optional cudaEvent profile.
//
// Mirrors, in devices/rtx4090-24g/qwen3_tts_1_7b.cu ("17.cu") of the reference:
//     NativeTalkerEngine::prefill           17.cu:16654-16912
//     NativeTalkerEngine::decode_device     17.cu:17189-17435
//     GenerationProfileEventSpan            17.cu:7184-7270
//     TalkerDecodeGpuProfile / TalkerLayerProfileSpans   17.cu:16447-16471
//     the profile report lines              17.cu:21950-21972, JSON keys devices/rtx4090-24g/main.cu:1268-1277
// Same call order, same live buffers (hidden_a_/hidden_b_, norm_, q_, k_, v_, q_rotated_, context_,
// attention_output_, residual_, post_norm_, swiglu_, final_norm_; 17.cu:17485-17531), same bucket names.  What
// changes with batching and paging: one call serves `batch` streams (decode) or a packed varlen batch of prompts
// (prefill); cache_position becomes the device array positions[], the per-layer LayerCache objects one pool
// addressed through a page table; the RoPE rows come from a table built once instead of a per-step upload.
// Without profiling a layer's decode attention is ONE launch (qm_decode_step); with profiling the two launches the
// reference times separately (qk_norm_rope_cache, attention) are issued, so that both buckets can be filled - the
// bits are the same either way.
#pragma once

#include <cstdint>
#include <iomanip>
#include <ostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "talker_attention_b200.hpp"

namespace qm {

// cudaEvent pair around a span of launches on one stream (GenerationProfileEventSpan, 17.cu:7184).  A span built
// with enabled = false owns no events and every method is a no-op, as in the reference when profiling is off.
class GenerationProfileEventSpan {
public:
    explicit GenerationProfileEventSpan(bool enabled = false) {
        if (!enabled) return;
        if (cudaEventCreateWithFlags(&begin_, cudaEventDefault) != cudaSuccess)
            throw std::runtime_error("generation profile event create");
        if (cudaEventCreateWithFlags(&end_, cudaEventDefault) != cudaSuccess) {
            cudaEventDestroy(begin_);
            begin_ = nullptr;
            throw std::runtime_error("generation profile event create");
        }
    }
    ~GenerationProfileEventSpan() {
        if (begin_) cudaEventDestroy(begin_);
        if (end_) cudaEventDestroy(end_);
    }
    GenerationProfileEventSpan(const GenerationProfileEventSpan&) = delete;
    GenerationProfileEventSpan& operator=(const GenerationProfileEventSpan&) = delete;
    GenerationProfileEventSpan(GenerationProfileEventSpan&& o) noexcept : begin_(o.begin_), end_(o.end_) {
        o.begin_ = nullptr;
        o.end_ = nullptr;
    }
    GenerationProfileEventSpan& operator=(GenerationProfileEventSpan&& o) noexcept {
        if (this != &o) {
            if (begin_) cudaEventDestroy(begin_);
            if (end_) cudaEventDestroy(end_);
            begin_ = o.begin_;
            end_ = o.end_;
            o.begin_ = nullptr;
            o.end_ = nullptr;
        }
        return *this;
    }
    bool enabled() const { return begin_ != nullptr && end_ != nullptr; }
    void begin(cudaStream_t stream) {
        if (enabled() && cudaEventRecord(begin_, stream) != cudaSuccess) throw std::runtime_error("generation profile begin");
    }
    void end(cudaStream_t stream) {
        if (enabled() && cudaEventRecord(end_, stream) != cudaSuccess) throw std::runtime_error("generation profile end");
    }
    // Milliseconds between begin and end; the stream must have been synchronised.
    double elapsed_ms() const {
        if (!enabled()) return 0.0;
        float value = 0.0f;
        if (cudaEventElapsedTime(&value, begin_, end_) != cudaSuccess) throw std::runtime_error("generation profile elapsed");
        return (double)value;
    }

private:
    cudaEvent_t begin_ = nullptr, end_ = nullptr;
};

// One decode step's GPU time per bucket, summed over the layers (TalkerDecodeGpuProfile, 17.cu:16447-16458).
struct TalkerDecodeGpuProfile {
    double total_ms = 0.0;
    double input_norm_ms = 0.0;
    double qkv_ms = 0.0;
    double qk_norm_rope_cache_ms = 0.0;
    double attention_ms = 0.0;
    double o_projection_ms = 0.0;
    double residual_postnorm_ms = 0.0;
    double gate_up_swiglu_ms = 0.0;
    double down_residual_ms = 0.0;
    double final_norm_ms = 0.0;
};

// TalkerLayerProfileSpans, 17.cu:16460-16471.
struct TalkerLayerProfileSpans {
    GenerationProfileEventSpan input_norm, qkv, qk_norm_rope_cache, attention, o_projection, residual_postnorm,
        gate_up_swiglu, down_residual;
    explicit TalkerLayerProfileSpans(bool enabled)
        : input_norm(enabled), qkv(enabled), qk_norm_rope_cache(enabled), attention(enabled), o_projection(enabled),
          residual_postnorm(enabled), gate_up_swiglu(enabled), down_residual(enabled) {}
};

// Mean of every bucket over the recorded steps.
inline TalkerDecodeGpuProfile mean_profile(const std::vector<TalkerDecodeGpuProfile>& steps) {
    TalkerDecodeGpuProfile m;
    if (steps.empty()) return m;
    for (const TalkerDecodeGpuProfile& p : steps) {
        m.total_ms += p.total_ms; m.input_norm_ms += p.input_norm_ms; m.qkv_ms += p.qkv_ms;
        m.qk_norm_rope_cache_ms += p.qk_norm_rope_cache_ms; m.attention_ms += p.attention_ms;
        m.o_projection_ms += p.o_projection_ms; m.residual_postnorm_ms += p.residual_postnorm_ms;
        m.gate_up_swiglu_ms += p.gate_up_swiglu_ms; m.down_residual_ms += p.down_residual_ms;
        m.final_norm_ms += p.final_norm_ms;
    }
    const double n = (double)steps.size();
    m.total_ms /= n; m.input_norm_ms /= n; m.qkv_ms /= n; m.qk_norm_rope_cache_ms /= n; m.attention_ms /= n;
    m.o_projection_ms /= n; m.residual_postnorm_ms /= n; m.gate_up_swiglu_ms /= n; m.down_residual_ms /= n;
    m.final_norm_ms /= n;
    return m;
}

// The report lines the reference prints after a profiled generation (17.cu:21950-21972).
inline void print_generation_profile(std::ostream& out, const TalkerDecodeGpuProfile& mean) {
    out << std::fixed << std::setprecision(6)
        << "generation_profile_talker_decode_mean_ms: " << mean.total_ms << "\n"
        << "generation_profile_talker_input_norm_mean_ms: " << mean.input_norm_ms << "\n"
        << "generation_profile_talker_qkv_mean_ms: " << mean.qkv_ms << "\n"
        << "generation_profile_talker_qk_norm_rope_cache_mean_ms: " << mean.qk_norm_rope_cache_ms << "\n"
        << "generation_profile_talker_attention_mean_ms: " << mean.attention_ms << "\n"
        << "generation_profile_talker_o_projection_mean_ms: " << mean.o_projection_ms << "\n"
        << "generation_profile_talker_residual_postnorm_mean_ms: " << mean.residual_postnorm_ms << "\n"
        << "generation_profile_talker_gate_up_swiglu_mean_ms: " << mean.gate_up_swiglu_ms << "\n"
        << "generation_profile_talker_down_residual_mean_ms: " << mean.down_residual_ms << "\n"
        << "generation_profile_talker_final_norm_mean_ms: " << mean.final_norm_ms << "\n";
}

// The same numbers under the keys of the reference's result JSON (devices/rtx4090-24g/main.cu:1268-1277), as the
// inside of an object: "profile_talker_decode_ms":..., ..., "profile_talker_final_norm_ms":...
inline std::string generation_profile_json_fields(const TalkerDecodeGpuProfile& mean) {
    std::ostringstream out;
    out << std::fixed << std::setprecision(6)
        << "\"profile_talker_decode_ms\":" << mean.total_ms << ","
        << "\"profile_talker_input_norm_ms\":" << mean.input_norm_ms << ","
        << "\"profile_talker_qkv_ms\":" << mean.qkv_ms << ","
        << "\"profile_talker_qk_norm_rope_cache_ms\":" << mean.qk_norm_rope_cache_ms << ","
        << "\"profile_talker_attention_ms\":" << mean.attention_ms << ","
        << "\"profile_talker_o_projection_ms\":" << mean.o_projection_ms << ","
        << "\"profile_talker_residual_postnorm_ms\":" << mean.residual_postnorm_ms << ","
        << "\"profile_talker_gate_up_swiglu_ms\":" << mean.gate_up_swiglu_ms << ","
        << "\"profile_talker_down_residual_ms\":" << mean.down_residual_ms << ","
        << "\"profile_talker_final_norm_ms\":" << mean.final_norm_ms;
    return out.str();
}

// Device pointers of one decoder layer's weights, named as the reference's LayerWeights (17.cu:14880-14930):
// projection weights [out][in] row-major bf16, biases may be null (the talker has none), norm weights [hidden] and
// q_norm / k_norm [128].
struct TalkerLayerWeights {
    const uint16_t* input_norm = nullptr;
    const uint16_t* post_norm = nullptr;
    const uint16_t* q_weight = nullptr;
    const uint16_t* q_bias = nullptr;
    const uint16_t* k_weight = nullptr;
    const uint16_t* k_bias = nullptr;
    const uint16_t* v_weight = nullptr;
    const uint16_t* v_bias = nullptr;
    const uint16_t* q_norm = nullptr;
    const uint16_t* k_norm = nullptr;
    const uint16_t* o_weight = nullptr;
    const uint16_t* o_bias = nullptr;
    const uint16_t* gate_weight = nullptr;
    const uint16_t* up_weight = nullptr;
    const uint16_t* down_weight = nullptr;
};

struct TalkerWeights {
    int hidden = 2048;          // kHidden
    int intermediate = 6144;
    int q_heads = 16;
    int kv_heads = 8;
    std::vector<TalkerLayerWeights> layers;
    const uint16_t* final_norm = nullptr;
    int layer_count() const { return (int)layers.size(); }
    int q_dim() const { return q_heads * QM_HEAD_DIM; }
    int kv_dim() const { return kv_heads * QM_HEAD_DIM; }
};

class NativeTalkerEngineB200 {
public:
    // num_pages pages of 64 tokens shared by all streams; max_rows = the most token rows one call carries (the
    // longest packed prefill, and at least max_batch); rope_rows = positions the RoPE table covers.
    NativeTalkerEngineB200(const TalkerWeights& weights, int num_pages, int max_batch, int max_rows, int rope_rows,
                           cudaStream_t stream, bool generation_profile = false)
        : weights_(weights), max_batch_(max_batch), max_rows_(max_rows < max_batch ? max_batch : max_rows), stream_(stream),
          generation_profile_(generation_profile),
          attention_(weights.layer_count(), num_pages, weights.q_heads, weights.kv_heads, max_batch, rope_rows, stream),
          profile_decode_total_(generation_profile), profile_final_norm_(generation_profile) {
        if (weights_.layers.empty() || !weights_.final_norm) throw std::runtime_error("Talker weights are incomplete");
        const std::size_t rows = (std::size_t)max_rows_;
        const std::size_t h = (std::size_t)weights_.hidden * 2, qd = (std::size_t)weights_.q_dim() * 2,
                          kd = (std::size_t)weights_.kv_dim() * 2, im = (std::size_t)weights_.intermediate * 2;
        hidden_a_ = DeviceBuffer(rows * h); hidden_b_ = DeviceBuffer(rows * h); norm_ = DeviceBuffer(rows * h);
        q_ = DeviceBuffer(rows * qd); k_ = DeviceBuffer(rows * kd); v_ = DeviceBuffer(rows * kd);
        q_rotated_ = DeviceBuffer(rows * qd); context_ = DeviceBuffer(rows * qd);
        attention_output_ = DeviceBuffer(rows * h); residual_ = DeviceBuffer(rows * h); post_norm_ = DeviceBuffer(rows * h);
        swiglu_ = DeviceBuffer(rows * im); final_norm_ = DeviceBuffer(rows * h);
        last_rows_ = DeviceBuffer((std::size_t)max_batch_ * h);
        profile_layers_.reserve(weights_.layers.size());
        for (std::size_t i = 0; i < weights_.layers.size(); ++i) profile_layers_.emplace_back(generation_profile);
    }

    TalkerAttentionB200& attention() { return attention_; }
    cudaStream_t stream() const { return stream_; }
    int max_batch() const { return max_batch_; }
    void reset_request() { attention_.reset_request(); }

    // prefill (17.cu:16654-16912) for a packed varlen batch: input_device [total_tokens][hidden] bf16, sequence s
    // owning rows cu_seqlens[s] .. cu_seqlens[s+1]-1 and starting an empty cache.  After the call final_norm()
    // holds the normalised last layer's rows [total_tokens][hidden]; with last_row_index (device int32[batch], the
    // packed index of each sequence's last row) the rows the first decode step continues from are also gathered
    // into last_rows() [batch][hidden] - what the reference downloads as StepResult::hidden.
    void prefill(const uint16_t* input_device, const int32_t* cu_seqlens, const int32_t* page_table, int max_pages,
                 int batch, int total_tokens, int max_seqlen, const int32_t* last_row_index = nullptr) {
        if (input_device == nullptr) throw std::runtime_error("Talker prefill input is null");
        if (total_tokens < 1 || total_tokens > max_rows_ || batch < 1 || batch > max_batch_)
            throw std::runtime_error("native Talker prefill input/RoPE size mismatch.");
        const int hidden = weights_.hidden;
        const uint16_t* current = input_device;
        uint16_t* next = hidden_a_.as<uint16_t>();
        uint16_t* other = hidden_b_.as<uint16_t>();
        for (int layer_index = 0; layer_index < weights_.layer_count(); ++layer_index) {
            const TalkerLayerWeights& layer = weights_.layers[(std::size_t)layer_index];
            attention_.launch_rmsnorm(current, layer.input_norm, norm_.as<uint16_t>(), total_tokens, hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.q_weight, layer.q_bias, nullptr, q_.as<uint16_t>(),
                                      total_tokens, weights_.q_dim(), hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.k_weight, layer.k_bias, nullptr, k_.as<uint16_t>(),
                                      total_tokens, weights_.kv_dim(), hidden);
            attention_.linear_generic(norm_.as<uint16_t>(), layer.v_weight, layer.v_bias, nullptr, v_.as<uint16_t>(),
                                      total_tokens, weights_.kv_dim(), hidden);
            // launch_rmsnorm(q), launch_rmsnorm(k), launch_rope_rows(q), launch_rope_rows(k), scatter_prefill_cache
            attention_.scatter_prefill_cache(layer_index, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(), layer.q_norm,
                                             layer.k_norm, cu_seqlens, page_table, max_pages, batch, total_tokens,
                                             q_rotated_.as<uint16_t>());
            attention_.launch_attention(layer_index, q_rotated_.as<uint16_t>(), cu_seqlens, page_table, max_pages, batch,
                                        total_tokens, max_seqlen, context_.as<uint16_t>());
            // o-projection, with launch_add(current, attention_output_, residual_) folded in
            attention_.linear_generic(context_.as<uint16_t>(), layer.o_weight, layer.o_bias, current, residual_.as<uint16_t>(),
                                      total_tokens, hidden, weights_.q_dim());
            attention_.launch_rmsnorm(residual_.as<uint16_t>(), layer.post_norm, post_norm_.as<uint16_t>(), total_tokens, hidden);
            attention_.gate_up_swiglu_rows(post_norm_.as<uint16_t>(), layer.gate_weight, layer.up_weight, swiglu_.as<uint16_t>(),
                                           total_tokens, hidden, weights_.intermediate);
            // down-projection, with launch_add(residual_, down_, next) folded in
            attention_.linear_generic(swiglu_.as<uint16_t>(), layer.down_weight, nullptr, residual_.as<uint16_t>(), next,
                                      total_tokens, hidden, weights_.intermediate);
            current = next;
            std::swap(next, other);
        }
        attention_.launch_rmsnorm(current, weights_.final_norm, final_norm_.as<uint16_t>(), total_tokens, hidden);
        if (last_row_index)
            attention_.gather_embeddings(final_norm_.as<uint16_t>(), last_row_index, batch, total_tokens, hidden,
                                         last_rows_.as<uint16_t>());
        final_rows_ = total_tokens;
    }

    // decode_device (17.cu:17189-17435) for `batch` streams: input_device [batch][hidden] bf16 (the embedded
    // previous code of each stream), positions[s] = the reference's cache_position of stream s, seq_lens[s] =
    // positions[s] + 1 (only read when profiling splits the attention into its two launches).  max_position is the
    // largest position as the host knows it, for the reference's overflow check; pass -1 to skip it.  Afterwards
    // final_norm() holds [batch][hidden].
    void decode_device(const uint16_t* input_device, const int32_t* positions, const int32_t* seq_lens,
                       const int32_t* page_table, int max_pages, int batch, int max_position = -1) {
        if (input_device == nullptr) throw std::runtime_error("Talker device decode input is null");
        if (batch < 1 || batch > max_batch_) throw std::runtime_error("Talker device decode batch out of range");
        if (max_position >= TalkerAttentionB200::max_cache(max_pages))
            throw std::runtime_error("Talker device decode cache overflow");
        const int hidden = weights_.hidden;
        profile_decode_total_.begin(stream_);
        const uint16_t* current = input_device;
        uint16_t* next = hidden_a_.as<uint16_t>();
        uint16_t* other = hidden_b_.as<uint16_t>();
        for (int layer_index = 0; layer_index < weights_.layer_count(); ++layer_index) {
            const TalkerLayerWeights& layer = weights_.layers[(std::size_t)layer_index];
            TalkerLayerProfileSpans* profile_layer = generation_profile_ ? &profile_layers_[(std::size_t)layer_index] : nullptr;
            if (profile_layer) profile_layer->input_norm.begin(stream_);
            attention_.launch_rmsnorm(current, layer.input_norm, norm_.as<uint16_t>(), batch, hidden);
            if (profile_layer) {
                profile_layer->input_norm.end(stream_);
                profile_layer->qkv.begin(stream_);
            }
            attention_.launch_qkv_m1(norm_.as<uint16_t>(), layer.q_weight, layer.q_bias, layer.k_weight, layer.k_bias,
                                     layer.v_weight, layer.v_bias, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(),
                                     batch, hidden);
            if (profile_layer) {
                profile_layer->qkv.end(stream_);
                profile_layer->qk_norm_rope_cache.begin(stream_);
                attention_.launch_qk_norm_rope_cache_m1(layer_index, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(),
                                                        layer.q_norm, layer.k_norm, positions, page_table, max_pages, batch,
                                                        q_rotated_.as<uint16_t>());
                profile_layer->qk_norm_rope_cache.end(stream_);
                profile_layer->attention.begin(stream_);
                attention_.launch_attention(layer_index, q_rotated_.as<uint16_t>(), seq_lens, page_table, max_pages, batch,
                                            context_.as<uint16_t>());
                profile_layer->attention.end(stream_);
                profile_layer->o_projection.begin(stream_);
            } else {
                attention_.decode_step(layer_index, q_.as<uint16_t>(), k_.as<uint16_t>(), v_.as<uint16_t>(), layer.q_norm,
                                       layer.k_norm, positions, page_table, max_pages, batch, context_.as<uint16_t>());
            }
            attention_.launch_linear_m1(context_.as<uint16_t>(), layer.o_weight, layer.o_bias, nullptr,
                                        attention_output_.as<uint16_t>(), batch, hidden, weights_.q_dim());
            if (profile_layer) {
                profile_layer->o_projection.end(stream_);
                profile_layer->residual_postnorm.begin(stream_);
            }
            attention_.launch_add_postnorm_m1(current, attention_output_.as<uint16_t>(), layer.post_norm,
                                              residual_.as<uint16_t>(), post_norm_.as<uint16_t>(), batch, hidden);
            if (profile_layer) {
                profile_layer->residual_postnorm.end(stream_);
                profile_layer->gate_up_swiglu.begin(stream_);
            }
            attention_.launch_gate_up_swiglu_m1(post_norm_.as<uint16_t>(), layer.gate_weight, layer.up_weight,
                                                swiglu_.as<uint16_t>(), batch, hidden, weights_.intermediate);
            if (profile_layer) {
                profile_layer->gate_up_swiglu.end(stream_);
                profile_layer->down_residual.begin(stream_);
            }
            attention_.launch_linear_m1(swiglu_.as<uint16_t>(), layer.down_weight, nullptr, residual_.as<uint16_t>(), next, batch,
                                        hidden, weights_.intermediate);
            if (profile_layer) profile_layer->down_residual.end(stream_);
            current = next;
            std::swap(next, other);
        }
        profile_final_norm_.begin(stream_);
        attention_.launch_rmsnorm(current, weights_.final_norm, final_norm_.as<uint16_t>(), batch, hidden);
        profile_final_norm_.end(stream_);
        profile_decode_total_.end(stream_);
        if (generation_profile_) {
            if (cudaStreamSynchronize(stream_) != cudaSuccess) throw std::runtime_error("Talker generation profile synchronize");
            TalkerDecodeGpuProfile profile;
            profile.total_ms = profile_decode_total_.elapsed_ms();
            profile.final_norm_ms = profile_final_norm_.elapsed_ms();
            for (const TalkerLayerProfileSpans& lp : profile_layers_) {
                profile.input_norm_ms += lp.input_norm.elapsed_ms();
                profile.qkv_ms += lp.qkv.elapsed_ms();
                profile.qk_norm_rope_cache_ms += lp.qk_norm_rope_cache.elapsed_ms();
                profile.attention_ms += lp.attention.elapsed_ms();
                profile.o_projection_ms += lp.o_projection.elapsed_ms();
                profile.residual_postnorm_ms += lp.residual_postnorm.elapsed_ms();
                profile.gate_up_swiglu_ms += lp.gate_up_swiglu.elapsed_ms();
                profile.down_residual_ms += lp.down_residual.elapsed_ms();
            }
            last_decode_gpu_profile_ = profile;
        } else {
            last_decode_gpu_profile_ = TalkerDecodeGpuProfile{};
        }
        // No device-wide synchronisation here (17.cu:17431): whatever is queued next on the same stream follows.
        final_rows_ = batch;
    }

    // [rows of the last call][hidden] bf16: the final RMSNorm of the last layer's output.
    const uint16_t* final_norm() const { return final_norm_.as<uint16_t>(); }
    int final_rows() const { return final_rows_; }
    // After prefill with last_row_index: the last row of every sequence, [batch][hidden].
    const uint16_t* last_rows() const { return last_rows_.as<uint16_t>(); }
    const TalkerDecodeGpuProfile& last_decode_gpu_profile() const { return last_decode_gpu_profile_; }
    bool generation_profile() const { return generation_profile_; }

private:
    TalkerWeights weights_;
    int max_batch_, max_rows_;
    cudaStream_t stream_;
    bool generation_profile_;
    TalkerAttentionB200 attention_;
    DeviceBuffer hidden_a_, hidden_b_, norm_, q_, k_, v_, q_rotated_, context_, attention_output_, residual_, post_norm_,
        swiglu_, final_norm_, last_rows_;
    GenerationProfileEventSpan profile_decode_total_, profile_final_norm_;
    std::vector<TalkerLayerProfileSpans> profile_layers_;
    TalkerDecodeGpuProfile last_decode_gpu_profile_;
    int final_rows_ = 0;
};

}  // namespace qm
