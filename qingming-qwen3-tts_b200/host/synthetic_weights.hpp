// Seeded random bf16 tensors on the host, and a talker decoder's worth of them uploaded to the device: stands in
// for the reference's checkpoint loader (TalkerWeights, devices/rtx4090-24g/qwen3_tts_1_7b.cu:14880-15060), which
// reads safetensors files that are not part of this path.  Shapes are the reference's; values follow the recipe
// the parity tests use (SplitMix64 -> Box-Muller on two 53-bit uniforms -> bf16, then scaled and rounded again), so
// a tensor drawn here equals the one the test oracle draws from the same seed.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "talker_engine_b200.hpp"

namespace qm {

inline uint16_t host_f32_to_bf16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}
inline float host_bf16_to_f32(uint16_t v) {
    const uint32_t bits = (uint32_t)v << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// Elements [begin, end) (begin even) of the N(0,1) stream of `seed`; SplitMix64 is a counter, so any range can be
// produced on its own: the k-th 64-bit draw comes from state seed + (k + 1) * 0x9E3779B97F4A7C15.
inline void fill_normal_range(uint64_t seed, float scale, uint16_t* out, std::size_t begin, std::size_t end) {
    auto draw = [&](std::size_t k) {
        uint64_t z = seed + (uint64_t)(k + 1) * 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        return (double)(z >> 11) * (1.0 / 9007199254740992.0);
    };
    auto store = [&](std::size_t i, double v) {
        uint16_t bits = host_f32_to_bf16((float)v);
        if (scale != 1.0f) bits = host_f32_to_bf16(host_bf16_to_f32(bits) * scale);
        out[i] = bits;
    };
    for (std::size_t i = begin; i < end; i += 2) {
        double u1 = draw(i), u2 = draw(i + 1);
        if (u1 < 1e-300) u1 = 1e-300;
        const double radius = std::sqrt(-2.0 * std::log(u1));
        const double angle = 6.283185307179586476925286766559 * u2;
        store(i, radius * std::cos(angle));
        if (i + 1 < end) store(i + 1, radius * std::sin(angle));
    }
}

// n values ~ N(0, scale^2) as bf16, on all host threads.
inline std::vector<uint16_t> scaled_normal_bf16(uint64_t seed, std::size_t n, float scale) {
    std::vector<uint16_t> out(n);
    unsigned workers = std::thread::hardware_concurrency();
    if (workers == 0) workers = 1;
    if (n < (1u << 16)) workers = 1;
    std::size_t chunk = (n + workers - 1) / workers;
    chunk += chunk & 1;
    std::vector<std::thread> pool;
    for (std::size_t begin = 0; begin < n; begin += chunk) {
        const std::size_t end = begin + chunk < n ? begin + chunk : n;
        pool.emplace_back(fill_normal_range, seed, scale, out.data(), begin, end);
    }
    for (std::thread& t : pool) t.join();
    return out;
}

// A whole random-init talker decoder on the device.  Keeps the allocations alive; view() hands the pointers to
// the engine.  Tensor t of layer l is drawn from seed * 1000003 + l * 64 + t; projections ~ N(0, 0.02), norm
// weights 1 + N(0, 0.1) (so that a missing norm weight would show), codec head ~ N(0, 0.02), embedding ~ N(0, 1).
class SyntheticTalker {
public:
    SyntheticTalker(uint64_t seed, int layers, int hidden, int intermediate, int vocab, int q_heads = 16, int kv_heads = 8,
                    float projection_scale = 0.02f) {
        weights_.hidden = hidden;
        weights_.intermediate = intermediate;
        weights_.q_heads = q_heads;
        weights_.kv_heads = kv_heads;
        const std::size_t h = (std::size_t)hidden, im = (std::size_t)intermediate, qd = (std::size_t)q_heads * QM_HEAD_DIM,
                          kd = (std::size_t)kv_heads * QM_HEAD_DIM;
        auto norm_like = [&](uint64_t s, std::size_t n) {
            std::vector<uint16_t> v = scaled_normal_bf16(s, n, 0.1f);
            for (uint16_t& x : v) x = host_f32_to_bf16(1.0f + host_bf16_to_f32(x));
            return upload(v);
        };
        for (int l = 0; l < layers; ++l) {
            const uint64_t base = seed * 1000003ull + (uint64_t)l * 64ull;
            TalkerLayerWeights w;
            w.input_norm = norm_like(base + 0, h);
            w.post_norm = norm_like(base + 1, h);
            w.q_weight = upload(scaled_normal_bf16(base + 2, qd * h, projection_scale));
            w.k_weight = upload(scaled_normal_bf16(base + 3, kd * h, projection_scale));
            w.v_weight = upload(scaled_normal_bf16(base + 4, kd * h, projection_scale));
            w.o_weight = upload(scaled_normal_bf16(base + 5, h * qd, projection_scale));
            w.gate_weight = upload(scaled_normal_bf16(base + 6, im * h, projection_scale));
            w.up_weight = upload(scaled_normal_bf16(base + 7, im * h, projection_scale));
            w.down_weight = upload(scaled_normal_bf16(base + 8, h * im, projection_scale));
            w.q_norm = norm_like(base + 9, QM_HEAD_DIM);
            w.k_norm = norm_like(base + 10, QM_HEAD_DIM);
            weights_.layers.push_back(w);
        }
        const uint64_t tail = seed * 1000003ull + (uint64_t)layers * 64ull;
        weights_.final_norm = norm_like(tail + 0, h);
        codec_head_ = upload(scaled_normal_bf16(tail + 1, (std::size_t)vocab * h, projection_scale));
        embedding_ = upload(scaled_normal_bf16(tail + 2, (std::size_t)vocab * h, 1.0f));
    }
    const TalkerWeights& view() const { return weights_; }
    const uint16_t* codec_head() const { return codec_head_; }
    const uint16_t* embedding() const { return embedding_; }

private:
    const uint16_t* upload(const std::vector<uint16_t>& host) {
        buffers_.emplace_back(host.size() * sizeof(uint16_t));
        if (cudaMemcpy(buffers_.back().pointer, host.data(), host.size() * sizeof(uint16_t), cudaMemcpyHostToDevice) != cudaSuccess)
            throw std::runtime_error("weight upload failed");
        return buffers_.back().as<uint16_t>();
    }
    TalkerWeights weights_;
    std::vector<DeviceBuffer> buffers_;
    const uint16_t* codec_head_ = nullptr;
    const uint16_t* embedding_ = nullptr;
};

}  // namespace qm
