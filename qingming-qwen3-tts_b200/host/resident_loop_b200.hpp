// Header-only C++ resident serving loop for the talker on the batched, paged path: JSONL requests in, prefill and
// decode steps for every active request at once, one JSON result line per request out.
//
// The reference's resident lifecycle (ResidentEngine, devices/rtx4090-24g/qwen3_tts_1_7b.cu:26555-27369; request
// parsing parse_resident_request :26356-26450; wire loop main.cpp:609-837; result fields CONTRACT.md "Output")
// serves ONE request at a time through a NativeTalkerEngine sized for it.  Here many requests share one
// NativeTalkerEngineB200: StreamBatcher admits a request when the page pool can promise its worst case, newly
// admitted prompts are prefilled together as one packed varlen batch, and every decode step runs all active
// streams in one batch.  Only what touches the attention path is here.  The reference's tokenizer, front-end and
// codec decoder are not: a request says how many prefill rows its prompt has ("prompt_rows"; the reference derives
// that from "text"), the rows fed to the talker are embedding rows of seeded pseudo-random tokens, and "output"
// receives the generated codec-0 codes as raw little-endian int32 instead of a WAV file.
//
// Request line (keys of the reference's format that concern this path, same validation messages):
//     {"prompt_rows": 120, "seed": 7, "max_new_tokens": 200, "output": "codes.bin"}
//   "text" may stand in for "prompt_rows" (rows = 9 + UTF-8 bytes, a stand-in for the tokenizer's count).
// Result line (stable fields of CONTRACT.md that this path can fill):
//     {"status":"ok","device":"b200-sxm","family":"1.7b","lifecycle":"resident","request_index":0,"seed":7,
//      "max_new_tokens":200,"max_new_tokens_capacity":256,"frames":57,"codec_fnv1a64":"...","eos":true,
//      "eos_frame":57,"ttft_ms":...,"generation_ms":...,"e2e_ms":...,"output":"codes.bin"}
//
// Step structure.  Row r of every batched array IS slot r of the batcher, for all max_streams slots, every step:
// a slot without a running request points its page table at a spare page nobody reads and writes position 0
// there.  Membership therefore never moves rows, the per-slot history / sampler state stay where they are, and
// the host touches the device only at interval boundaries: every `eos_check_interval` steps it reads the codes
// back (the reference reads 4 bytes per step, 17.cu:14560), retires streams that produced EOS or reached their
// limit, admits and prefills waiting requests, and uploads the next interval's positions.
#pragma once

#include <poll.h>
#include <unistd.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <deque>
#include <fstream>
#include <optional>
#include <ostream>
#include <sstream>
#include <string>
#include <vector>

#include "stream_batcher.hpp"
#include "talker_engine_b200.hpp"

namespace qm {

// fnv1a64 (17.cu:869-878), including the reference's own starting value, so that hashes are comparable with its
// "codec_fnv1a64" field.
inline uint64_t fnv1a64(const void* data, std::size_t bytes) {
    const auto* p = static_cast<const uint8_t*>(data);
    uint64_t value = 1469598103934665603ull;
    for (std::size_t i = 0; i < bytes; ++i) {
        value ^= p[i];
        value *= 1099511628211ull;
    }
    return value;
}

// SplitMix64 (the generator the reference's sampler uses, 17.cu:7154-7161).
inline uint64_t splitmix64_next(uint64_t& state) {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct ResidentRequest {
    std::size_t index = 0;
    int prompt_rows = 0;
    uint64_t seed = 0;
    std::size_t max_new_tokens = 0;
    std::string output;
};

// "key": "value" of a flat JSON object line; escapes \" \\ \n \t are undone, anything else is kept as written.
inline std::optional<std::string> resident_json_string_field(const std::string& line, const std::string& key) {
    const std::string needle = "\"" + key + "\"";
    std::size_t at = line.find(needle);
    if (at == std::string::npos) return std::nullopt;
    at = line.find(':', at + needle.size());
    if (at == std::string::npos) return std::nullopt;
    at = line.find_first_not_of(" \t", at + 1);
    if (at == std::string::npos || line[at] != '"') return std::nullopt;
    std::string value;
    for (std::size_t i = at + 1; i < line.size(); ++i) {
        const char c = line[i];
        if (c == '"') return value;
        if (c == '\\' && i + 1 < line.size()) {
            const char e = line[++i];
            value.push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
        } else {
            value.push_back(c);
        }
    }
    throw std::runtime_error("resident JSON string is not terminated: " + key);
}

inline std::optional<uint64_t> resident_json_u64_field(const std::string& line, const std::string& key) {
    const std::string needle = "\"" + key + "\"";
    std::size_t at = line.find(needle);
    if (at == std::string::npos) return std::nullopt;
    at = line.find(':', at + needle.size());
    if (at == std::string::npos) return std::nullopt;
    at = line.find_first_not_of(" \t", at + 1);
    if (at == std::string::npos || line[at] < '0' || line[at] > '9')
        throw std::runtime_error("resident JSON field is not an unsigned integer: " + key);
    uint64_t value = 0;
    while (at < line.size() && line[at] >= '0' && line[at] <= '9') {
        const uint64_t digit = (uint64_t)(line[at] - '0');
        if (value > (UINT64_MAX - digit) / 10u) throw std::runtime_error("resident JSON integer overflow: " + key);
        value = value * 10u + digit;
        ++at;
    }
    return value;
}

// parse_resident_request (17.cu:26356-26450), for the keys this path uses.
inline ResidentRequest parse_resident_request(const std::string& line, std::size_t index) {
    ResidentRequest request;
    request.index = index;
    const auto output = resident_json_string_field(line, "output");
    if (!output || output->empty()) throw std::runtime_error("resident request requires \"output\"");
    request.output = *output;
    if (const auto rows = resident_json_u64_field(line, "prompt_rows")) {
        if (*rows == 0 || *rows > 1000000) throw std::runtime_error("resident prefill rows must be positive");
        request.prompt_rows = (int)*rows;
    } else {
        const auto text = resident_json_string_field(line, "text");
        if (!text || text->empty()) throw std::runtime_error("resident request requires non-empty \"text\"");
        request.prompt_rows = 9 + (int)text->size();
    }
    if (const auto seed = resident_json_u64_field(line, "seed")) request.seed = *seed;
    const auto maximum = resident_json_u64_field(line, "max_new_tokens");
    if (!maximum) throw std::runtime_error("resident request requires max_new_tokens");
    if (*maximum == 0 || *maximum > 8192) throw std::runtime_error("resident request max_new_tokens must be in [1,8192]");
    request.max_new_tokens = (std::size_t)*maximum;
    return request;
}

inline std::string json_escape(const std::string& text) {
    std::string out;
    for (const char c : text) {
        if (c == '"' || c == '\\') { out.push_back('\\'); out.push_back(c); }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else out.push_back(c);
    }
    return out;
}

// Lines from a file descriptor without blocking the serving loop: next(false) returns a line only if one is
// already there; next(true) waits for one.  A regular file is always readable, so a request file is consumed in
// order at the first opportunity, which makes a run over a file reproducible.
class LineSource {
public:
    explicit LineSource(int fd) : fd_(fd) {}
    bool exhausted() const { return eof_ && buffer_.empty(); }
    std::optional<std::string> next(bool block) {
        for (;;) {
            const std::size_t nl = buffer_.find('\n');
            if (nl != std::string::npos) {
                std::string line = buffer_.substr(0, nl);
                buffer_.erase(0, nl + 1);
                return line;
            }
            if (eof_) {
                if (buffer_.empty()) return std::nullopt;
                std::string line;
                line.swap(buffer_);
                return line;
            }
            pollfd p{fd_, POLLIN, 0};
            const int ready = ::poll(&p, 1, block ? -1 : 0);
            if (ready <= 0) return std::nullopt;
            char chunk[4096];
            const ssize_t n = ::read(fd_, chunk, sizeof(chunk));
            if (n <= 0) eof_ = true;
            else buffer_.append(chunk, (std::size_t)n);
        }
    }

private:
    int fd_;
    bool eof_ = false;
    std::string buffer_;
};

struct ResidentConfig {
    int max_streams = 32;
    int max_pages_per_stream = 136;     // 8 704 positions: the longest prompt plus the largest capacity class
    int num_pages = 2048;               // pages the batcher hands out; the engine's pool holds one more (the spare page)
    int vocab = 3072;                   // codec vocabulary (17.cu final head)
    int eos_token = 2150;
    int top_k = 50;                     // 0 = greedy argmax
    float temperature = 0.9f;
    int eos_check_interval = 4;         // decode steps between two read-backs of the codes
    std::string device = "b200-sxm";
    std::string family = "1.7b";
};

class ResidentTalkerLoopB200 {
public:
    // codec_head [vocab][hidden] and embedding [vocab][hidden] are device pointers (bf16); `engine` must have been
    // built with num_pages = config.num_pages + 1 and max_batch >= config.max_streams.
    ResidentTalkerLoopB200(NativeTalkerEngineB200& engine, const TalkerWeights& weights, const uint16_t* codec_head,
                           const uint16_t* embedding, const ResidentConfig& config)
        : engine_(engine), hidden_(weights.hidden), config_(config), codec_head_(codec_head), embedding_(embedding),
          batcher_(config.num_pages, config.max_streams, config.max_pages_per_stream), slots_((std::size_t)config.max_streams) {
        if (config.max_streams > engine.max_batch()) throw std::runtime_error("resident loop: more streams than the engine's batch");
        if (config.eos_check_interval < 1 || config.eos_check_interval > 64) throw std::runtime_error("resident loop: bad interval");
        const std::size_t s = (std::size_t)config.max_streams, k = (std::size_t)config.eos_check_interval;
        step_input_ = DeviceBuffer(s * (std::size_t)hidden_ * 2);
        logits_ = DeviceBuffer(s * (std::size_t)config.vocab * 2);
        history_ = DeviceBuffer(s * kHistoryCapacity * sizeof(int32_t));
        generation_index_ = DeviceBuffer(k * s * sizeof(int32_t));
        positions_ = DeviceBuffer(k * s * sizeof(int32_t));
        seq_lens_ = DeviceBuffer(k * s * sizeof(int32_t));
        page_table_ = DeviceBuffer(s * (std::size_t)config.max_pages_per_stream * sizeof(int32_t));
        rng_state_ = DeviceBuffer(s * sizeof(uint64_t));
        codes_ = DeviceBuffer((k + 1) * s * sizeof(int32_t));
        if (cudaMemsetAsync(history_.pointer, 0, history_.bytes, engine_.stream()) != cudaSuccess ||
            cudaMemsetAsync(codes_.pointer, 0, codes_.bytes, engine_.stream()) != cudaSuccess)
            throw std::runtime_error("resident loop: clearing device state failed");
        host_codes_.assign((k + 1) * s, 0);
    }

    // Serves requests from `source` until it is exhausted and every admitted request has finished.  One result line
    // per request goes to `out`.  Returns the number of requests served.
    std::size_t serve(LineSource& source, std::ostream& out) {
        std::size_t served = 0, next_index = 0;
        for (;;) {
            // ---- boundary: take in whatever requests have arrived (wait for one when there is nothing to do)
            const bool idle = batcher_.active_streams() == 0 && waiting_.empty();
            if (idle && source.exhausted()) break;
            bool block = idle;
            while (auto line = source.next(block)) {
                block = false;
                if (line->find_first_not_of(" \t\r") == std::string::npos) continue;
                const std::size_t index = next_index++;
                try {
                    Waiting w;
                    w.request = parse_resident_request(*line, index);
                    w.arrived = Clock::now();
                    waiting_.push_back(w);
                } catch (const std::exception& e) {
                    emit_error(out, index, e.what());
                    ++served;
                }
            }
            admit_and_prefill(out, served);
            if (batcher_.active_streams() == 0) {
                // Nothing runs and the head of the queue still was not admitted: the whole pool cannot hold it.
                if (!waiting_.empty()) {
                    emit_error(out, waiting_.front().request.index, "resident request exceeds resident capacity");
                    waiting_.pop_front();
                    ++served;
                }
                continue;
            }
            run_interval();
            served += harvest(out);
        }
        return served;
    }

    const std::vector<TalkerDecodeGpuProfile>& decode_profiles() const { return decode_profiles_; }
    std::size_t decode_steps() const { return decode_steps_; }

private:
    using Clock = std::chrono::steady_clock;
    static constexpr std::size_t kHistoryCapacity = 8192;      // the reference's history buffer (17.cu final head)

    struct Waiting {
        ResidentRequest request;
        Clock::time_point arrived;
    };
    struct Slot {
        bool running = false;
        ResidentRequest request;
        Clock::time_point arrived, admitted, first_code;
        std::vector<int32_t> codes;
        bool eos = false;
    };

    static double ms_between(Clock::time_point a, Clock::time_point b) {
        return std::chrono::duration<double, std::milli>(b - a).count();
    }

    void check_cuda(cudaError_t status, const char* what) {
        if (status != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
    }

    template <class T>
    void upload(DeviceBuffer& dst, const std::vector<T>& src, std::size_t offset_elems = 0) {
        check_cuda(cudaMemcpyAsync(dst.as<T>() + offset_elems, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice,
                                   engine_.stream()),
                   "resident loop upload");
    }

    // Admits waiting requests in arrival order while the pool can promise their worst case, prefills the newly
    // admitted prompts as one packed batch and draws each one's first code.
    void admit_and_prefill(std::ostream& out, std::size_t& served) {
        std::vector<int> fresh;
        while (!waiting_.empty()) {
            const Waiting& w = waiting_.front();
            const int worst = w.request.prompt_rows + (int)generation_capacity_for(w.request.max_new_tokens);
            if ((worst + kBatcherPageTokens - 1) / kBatcherPageTokens > config_.max_pages_per_stream) {
                emit_error(out, w.request.index, "resident request does not fit one stream's page table");
                ++served;
                waiting_.pop_front();
                continue;
            }
            const int slot = batcher_.admit((int64_t)w.request.index, w.request.prompt_rows, (int)w.request.max_new_tokens);
            if (slot < 0) break;        // keep it (and everything behind it) queued until a stream retires
            Slot& s = slots_[(std::size_t)slot];
            s = Slot{};
            s.running = true;
            s.request = w.request;
            s.arrived = w.arrived;
            s.admitted = Clock::now();
            fresh.push_back(slot);
            waiting_.pop_front();
        }
        if (fresh.empty()) return;
        const PrefillPlan plan = batcher_.plan_prefill(fresh);
        // the prompt rows: embedding rows of seeded pseudo-random codes (stand-in for the front-end's embeddings)
        std::vector<int32_t> prompt_ids((std::size_t)plan.total_tokens), last_rows((std::size_t)plan.batch);
        for (int row = 0; row < plan.batch; ++row) {
            uint64_t state = slots_[(std::size_t)fresh[(std::size_t)row]].request.seed ^ 0x5157454E33545453ull;
            for (int t = plan.cu_seqlens[(std::size_t)row]; t < plan.cu_seqlens[(std::size_t)row + 1]; ++t)
                prompt_ids[(std::size_t)t] = (int32_t)(splitmix64_next(state) % (uint64_t)config_.vocab);
            last_rows[(std::size_t)row] = plan.cu_seqlens[(std::size_t)row + 1] - 1;
        }
        DeviceBuffer ids_dev(prompt_ids.size() * sizeof(int32_t)), rows_dev((std::size_t)plan.total_tokens * (std::size_t)hidden_ * 2),
            cu_dev(plan.cu_seqlens.size() * sizeof(int32_t)), table_dev(plan.page_table.size() * sizeof(int32_t)),
            last_dev(last_rows.size() * sizeof(int32_t));
        upload(ids_dev, prompt_ids);
        upload(cu_dev, plan.cu_seqlens);
        upload(table_dev, plan.page_table);
        upload(last_dev, last_rows);
        engine_.attention().gather_embeddings(embedding_, ids_dev.as<int32_t>(), plan.total_tokens, config_.vocab, hidden_,
                                              rows_dev.as<uint16_t>());
        engine_.prefill(rows_dev.as<uint16_t>(), cu_dev.as<int32_t>(), table_dev.as<int32_t>(), plan.max_pages, plan.batch,
                        plan.total_tokens, plan.max_seqlen, last_dev.as<int32_t>());
        batcher_.commit_prefill(plan);
        // first code of each new stream: head + sampler on its last prompt row, then that code's embedding goes to
        // the stream's row of the step input
        DeviceBuffer first_logits((std::size_t)plan.batch * (std::size_t)config_.vocab * 2), first_codes((std::size_t)plan.batch * 4),
            zeros((std::size_t)plan.batch * 4), first_rng((std::size_t)plan.batch * 8), first_hist((std::size_t)plan.batch * kHistoryCapacity * 4),
            first_rows((std::size_t)plan.batch * (std::size_t)hidden_ * 2);
        check_cuda(cudaMemsetAsync(zeros.pointer, 0, zeros.bytes, engine_.stream()), "resident loop clear");
        check_cuda(cudaMemsetAsync(first_hist.pointer, 0, first_hist.bytes, engine_.stream()), "resident loop clear");
        std::vector<uint64_t> seeds((std::size_t)plan.batch);
        for (int row = 0; row < plan.batch; ++row) seeds[(std::size_t)row] = slots_[(std::size_t)fresh[(std::size_t)row]].request.seed;
        upload(first_rng, seeds);
        engine_.attention().launch_linear_m1(engine_.last_rows(), codec_head_, nullptr, nullptr, first_logits.as<uint16_t>(), plan.batch,
                                             config_.vocab, hidden_);
        engine_.attention().final_head_sample(first_logits.as<uint16_t>(), plan.batch, config_.vocab, first_hist.as<int32_t>(),
                                              (int)kHistoryCapacity, zeros.as<int32_t>(),
                                              QM_SAMPLE_REPETITION | QM_SAMPLE_SUPPRESS | QM_SAMPLE_RECORD, config_.top_k,
                                              config_.temperature, first_rng.as<uint64_t>(), first_codes.as<int32_t>(), config_.eos_token);
        engine_.attention().gather_embeddings(embedding_, first_codes.as<int32_t>(), plan.batch, config_.vocab, hidden_,
                                              first_rows.as<uint16_t>());
        // scatter the per-request state into the slots' rows
        for (int row = 0; row < plan.batch; ++row) {
            const std::size_t slot = (std::size_t)fresh[(std::size_t)row];
            check_cuda(cudaMemcpyAsync(step_input_.as<uint16_t>() + slot * (std::size_t)hidden_, first_rows.as<uint16_t>() + (std::size_t)row * hidden_,
                                       (std::size_t)hidden_ * 2, cudaMemcpyDeviceToDevice, engine_.stream()), "resident loop scatter");
            check_cuda(cudaMemcpyAsync(history_.as<int32_t>() + slot * kHistoryCapacity, first_hist.as<int32_t>() + (std::size_t)row * kHistoryCapacity,
                                       kHistoryCapacity * 4, cudaMemcpyDeviceToDevice, engine_.stream()), "resident loop scatter");
            check_cuda(cudaMemcpyAsync(rng_state_.as<uint64_t>() + slot, first_rng.as<uint64_t>() + row, 8, cudaMemcpyDeviceToDevice,
                                       engine_.stream()), "resident loop scatter");
        }
        std::vector<int32_t> codes((std::size_t)plan.batch);
        check_cuda(cudaMemcpyAsync(codes.data(), first_codes.pointer, codes.size() * 4, cudaMemcpyDeviceToHost, engine_.stream()),
                   "resident loop first codes");
        check_cuda(cudaStreamSynchronize(engine_.stream()), "resident loop prefill synchronize");
        const Clock::time_point now = Clock::now();
        for (int row = 0; row < plan.batch; ++row) {
            Slot& s = slots_[(std::size_t)fresh[(std::size_t)row]];
            s.first_code = now;
            s.codes.push_back(codes[(std::size_t)row]);
            if (codes[(std::size_t)row] == config_.eos_token) s.eos = true;
        }
    }

    // One interval: up to eos_check_interval decode steps for all slots, queued without touching the host.
    void run_interval() {
        const int S = config_.max_streams, P = config_.max_pages_per_stream;
        const int spare_page = config_.num_pages;           // the engine's pool has num_pages + 1 pages
        // how many steps every running stream can still take inside this interval
        int steps = config_.eos_check_interval;
        std::vector<int32_t> positions((std::size_t)steps * S, 0), seq_lens((std::size_t)steps * S, 1),
            generation((std::size_t)steps * S, 0), table((std::size_t)S * P, spare_page);
        std::vector<int> budget((std::size_t)S, 0);
        int max_position = 0;
        for (int j = 0; j < steps; ++j) {
            // a stream that has produced all its tokens (or EOS) idles on the spare page for the rest of the interval
            std::vector<char> takes((std::size_t)S, 0);
            for (int slot = 0; slot < S; ++slot) {
                const Slot& s = slots_[(std::size_t)slot];
                takes[(std::size_t)slot] = s.running && !s.eos && (int)s.codes.size() + budget[(std::size_t)slot] < (int)s.request.max_new_tokens;
            }
            const DecodePlan plan = batcher_.plan_decode_step();
            DecodePlan committed = plan;
            committed.slots.clear();
            for (int row = 0; row < plan.batch; ++row) {
                const int slot = plan.slots[(std::size_t)row];
                if (!takes[(std::size_t)slot]) continue;
                committed.slots.push_back(slot);
                positions[(std::size_t)j * S + slot] = plan.positions[(std::size_t)row];
                seq_lens[(std::size_t)j * S + slot] = plan.seq_lens[(std::size_t)row];
                generation[(std::size_t)j * S + slot] = (int32_t)slots_[(std::size_t)slot].codes.size() + budget[(std::size_t)slot];
                max_position = plan.positions[(std::size_t)row] > max_position ? plan.positions[(std::size_t)row] : max_position;
                budget[(std::size_t)slot] += 1;
            }
            batcher_.commit_decode_step(committed);
        }
        for (int slot = 0; slot < S; ++slot) {
            if (!slots_[(std::size_t)slot].running || budget[(std::size_t)slot] == 0) continue;
            const std::vector<int>& pages = batcher_.pages(slot);
            for (std::size_t p = 0; p < pages.size(); ++p) table[(std::size_t)slot * P + p] = pages[p];
        }
        // rows that idle: position 0 on the spare page, every step
        upload(positions_, positions);
        upload(seq_lens_, seq_lens);
        upload(generation_index_, generation);
        upload(page_table_, table);
        interval_budget_ = budget;
        interval_steps_ = steps;
        for (int j = 0; j < steps; ++j) {
            engine_.decode_device(step_input_.as<uint16_t>(), positions_.as<int32_t>() + (std::size_t)j * S,
                                  seq_lens_.as<int32_t>() + (std::size_t)j * S, page_table_.as<int32_t>(), P, S, max_position);
            if (engine_.generation_profile()) decode_profiles_.push_back(engine_.last_decode_gpu_profile());
            engine_.attention().launch_linear_m1(engine_.final_norm(), codec_head_, nullptr, nullptr, logits_.as<uint16_t>(), S,
                                                 config_.vocab, hidden_);
            int32_t* step_codes = codes_.as<int32_t>() + (std::size_t)j * S;
            engine_.attention().final_head_sample(logits_.as<uint16_t>(), S, config_.vocab, history_.as<int32_t>(), (int)kHistoryCapacity,
                                                  generation_index_.as<int32_t>() + (std::size_t)j * S,
                                                  QM_SAMPLE_REPETITION | QM_SAMPLE_SUPPRESS | QM_SAMPLE_RECORD, config_.top_k,
                                                  config_.temperature, rng_state_.as<uint64_t>(), step_codes, config_.eos_token);
            engine_.attention().gather_embeddings(embedding_, step_codes, S, config_.vocab, hidden_, step_input_.as<uint16_t>());
            ++decode_steps_;
        }
        check_cuda(cudaMemcpyAsync(host_codes_.data(), codes_.pointer, (std::size_t)steps * S * sizeof(int32_t), cudaMemcpyDeviceToHost,
                                   engine_.stream()), "resident loop code read-back");
        check_cuda(cudaStreamSynchronize(engine_.stream()), "resident loop interval synchronize");
        if (const uint32_t bits = engine_.attention().device_status())
            throw std::runtime_error("resident loop: device status " + std::to_string(bits));
    }

    // After an interval: append the codes each stream produced, stop at EOS or its limit, emit results, retire.
    std::size_t harvest(std::ostream& out) {
        const int S = config_.max_streams;
        std::size_t finished = 0;
        const Clock::time_point now = Clock::now();
        for (int slot = 0; slot < S; ++slot) {
            Slot& s = slots_[(std::size_t)slot];
            if (!s.running) continue;
            for (int j = 0; j < interval_budget_[(std::size_t)slot] && !s.eos; ++j) {
                const int32_t code = host_codes_[(std::size_t)j * S + slot];
                s.codes.push_back(code);
                if (code == config_.eos_token) s.eos = true;
            }
            if (!s.eos && s.codes.size() < s.request.max_new_tokens) continue;
            emit_result(out, s, now);
            batcher_.retire(slot);
            s = Slot{};
            ++finished;
        }
        return finished;
    }

    void emit_result(std::ostream& out, const Slot& s, Clock::time_point now) {
        // frames: codes before EOS (the EOS code itself is not a frame), as the reference counts them
        std::size_t frames = s.codes.size();
        long eos_frame = -1;
        if (s.eos) {
            frames = s.codes.size() - 1;
            eos_frame = (long)frames;
        }
        const uint64_t hash = fnv1a64(s.codes.data(), frames * sizeof(int32_t));
        if (s.request.output != "-") {
            std::ofstream file(s.request.output, std::ios::binary);
            if (!file) throw std::runtime_error("failed to open: " + s.request.output);
            file.write(reinterpret_cast<const char*>(s.codes.data()), (std::streamsize)(frames * sizeof(int32_t)));
        }
        std::ostringstream line;
        line << std::fixed << std::setprecision(3) << "{\"status\":\"ok\",\"device\":\"" << config_.device << "\",\"family\":\""
             << config_.family << "\",\"lifecycle\":\"resident\",\"request_index\":" << s.request.index << ",\"error\":\"\",\"seed\":"
             << s.request.seed << ",\"prompt_rows\":" << s.request.prompt_rows << ",\"max_new_tokens\":" << s.request.max_new_tokens
             << ",\"max_new_tokens_capacity\":" << generation_capacity_for(s.request.max_new_tokens) << ",\"frames\":" << frames
             << ",\"codec_fnv1a64\":\"" << hash << "\",\"eos\":" << (s.eos ? "true" : "false") << ",\"eos_frame\":" << eos_frame
             << ",\"queue_ms\":" << ms_between(s.arrived, s.admitted) << ",\"ttft_ms\":" << ms_between(s.admitted, s.first_code)
             << ",\"generation_ms\":" << ms_between(s.admitted, now) << ",\"e2e_ms\":" << ms_between(s.arrived, now)
             << ",\"output\":\"" << json_escape(s.request.output) << "\"}\n";
        out << line.str() << std::flush;
    }

    void emit_error(std::ostream& out, std::size_t index, const std::string& message) {
        out << "{\"status\":\"error\",\"device\":\"" << config_.device << "\",\"family\":\"" << config_.family
            << "\",\"lifecycle\":\"resident\",\"request_index\":" << index << ",\"error\":\"" << json_escape(message) << "\"}\n"
            << std::flush;
    }

    NativeTalkerEngineB200& engine_;
    int hidden_;
    ResidentConfig config_;
    const uint16_t* codec_head_;
    const uint16_t* embedding_;
    StreamBatcher batcher_;
    std::vector<Slot> slots_;
    std::deque<Waiting> waiting_;
    DeviceBuffer step_input_, logits_, history_, generation_index_, positions_, seq_lens_, page_table_, rng_state_, codes_;
    std::vector<int32_t> host_codes_;
    std::vector<int> interval_budget_;
    int interval_steps_ = 0;
    std::vector<TalkerDecodeGpuProfile> decode_profiles_;
    std::size_t decode_steps_ = 0;
};

}  // namespace qm
