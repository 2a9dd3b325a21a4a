// Streams that join and leave between decode steps, driven by host/stream_batcher.hpp through the C++ mirror of
// the reference's launchers: two prompts are prefilled together, decode steps run for whoever is active, a third
// request is admitted and prefilled in the middle, one stream retires and a fourth request takes over its pages.
// After every decode step each active stream's context is compared with the CPU oracle run on that stream alone
// (contiguous cache, fp32 attention), so a wrong page, position or length in a plan shows as a mismatch.
// Exit code 0 = pass.  Links libqm_attention_b200.so and (test-only) libqm_oracle.so.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>

#include "stream_batcher.hpp"
#include "talker_attention_b200.hpp"

extern "C" {
void qmo_fill_normal_bf16(uint64_t seed, uint16_t* out, int64_t n);
void qmo_make_rope(int rows, int start, double theta, uint16_t* cosine, uint16_t* sine);
void qmo_append(const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*,
                const uint16_t*, float, int, int, int, int, int, uint16_t*, uint16_t*, uint16_t*);
int qmo_decode_attention_batch(const uint16_t*, const uint16_t* const*, const uint16_t* const*, const int32_t*,
                               const int32_t*, int, int, int, int, uint16_t*, float*);
float qmo_bf16_to_f32(uint16_t);
}

namespace {

constexpr int Hq = 16, Hkv = 8, D = 128, kMaxPages = 8, kMaxCache = kMaxPages * 64, kRopeRows = 512;

template <class T>
T* upload(const std::vector<T>& h, qm::DeviceBuffer& d) {
    d = qm::DeviceBuffer(h.size() * sizeof(T));
    cudaMemcpy(d.pointer, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d.as<T>();
}

// What one request feeds the attention path: its projections for every position, and the oracle's view of it.
struct Request {
    int64_t id;
    int prompt;
    std::vector<uint16_t> q, k, v;                 // [positions][heads][128], enough for prompt + all steps
    std::vector<uint16_t> key_cache, value_cache;  // oracle, reference layout [Hkv][kMaxCache][128]
    int oracle_length = 0;
    Request(int64_t id_, int prompt_, int positions) : id(id_), prompt(prompt_) {
        q.resize((size_t)positions * Hq * D);
        k.resize((size_t)positions * Hkv * D);
        v.resize((size_t)positions * Hkv * D);
        qmo_fill_normal_bf16((uint64_t)id * 10 + 1, q.data(), (int64_t)q.size());
        qmo_fill_normal_bf16((uint64_t)id * 10 + 2, k.data(), (int64_t)k.size());
        qmo_fill_normal_bf16((uint64_t)id * 10 + 3, v.data(), (int64_t)v.size());
        key_cache.assign((size_t)Hkv * kMaxCache * D, 0);
        value_cache.assign(key_cache.size(), 0);
    }
};

}  // namespace

int main() {
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    try {
        const int num_pages = 20, max_streams = 3;
        qm::TalkerAttentionB200 engine(/*layers=*/1, num_pages, Hq, Hkv, /*max_batch=*/max_streams, kRopeRows, stream);
        qm::StreamBatcher batcher(num_pages, max_streams, kMaxPages);
        std::vector<uint16_t> norm_w(D), cosv((size_t)kRopeRows * D), sinv(cosv.size());
        qmo_fill_normal_bf16(5, norm_w.data(), D);
        for (auto& w : norm_w) w = (uint16_t)(0x3f80 + (w & 0x1f));      // weights between 1 and 1.25
        qmo_make_rope(kRopeRows, 0, 1.0e6, cosv.data(), sinv.data());
        qm::DeviceBuffer dw;
        upload(norm_w, dw);
        engine.reset_request();

        std::map<int, Request*> by_slot;
        double worst_abs = 0.0, worst_rel = 0.0;
        int checked = 0;

        auto prefill = [&](const std::vector<int>& slots) {
            qm::PrefillPlan plan = batcher.plan_prefill(slots);
            std::vector<uint16_t> q, k, v;
            for (int slot : slots) {
                Request& r = *by_slot[slot];
                q.insert(q.end(), r.q.begin(), r.q.begin() + (size_t)r.prompt * Hq * D);
                k.insert(k.end(), r.k.begin(), r.k.begin() + (size_t)r.prompt * Hkv * D);
                v.insert(v.end(), r.v.begin(), r.v.begin() + (size_t)r.prompt * Hkv * D);
                std::vector<uint16_t> unused((size_t)r.prompt * Hq * D);
                qmo_append(r.q.data(), r.k.data(), r.v.data(), norm_w.data(), norm_w.data(), cosv.data(), sinv.data(), 1.0e-6f,
                           r.prompt, 0, Hq, Hkv, kMaxCache, unused.data(), r.key_cache.data(), r.value_cache.data());
                r.oracle_length = r.prompt;
            }
            qm::DeviceBuffer dq, dk, dv, dcu, dt, dqr(q.size() * 2);
            upload(q, dq); upload(k, dk); upload(v, dv); upload(plan.cu_seqlens, dcu); upload(plan.page_table, dt);
            engine.scatter_prefill_cache(0, dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dw.as<uint16_t>(),
                                         dw.as<uint16_t>(), dcu.as<int32_t>(), dt.as<int32_t>(), plan.max_pages, plan.batch,
                                         plan.total_tokens, dqr.as<uint16_t>());
            cudaStreamSynchronize(stream);
            batcher.commit_prefill(plan);
        };

        auto decode_step = [&]() -> int {
            qm::DecodePlan plan = batcher.plan_decode_step();
            if (plan.batch == 0) return 0;
            std::vector<uint16_t> q, k, v;
            for (int row = 0; row < plan.batch; ++row) {
                Request& r = *by_slot[plan.slots[(size_t)row]];
                const size_t pos = (size_t)plan.positions[(size_t)row];
                q.insert(q.end(), r.q.begin() + pos * Hq * D, r.q.begin() + (pos + 1) * Hq * D);
                k.insert(k.end(), r.k.begin() + pos * Hkv * D, r.k.begin() + (pos + 1) * Hkv * D);
                v.insert(v.end(), r.v.begin() + pos * Hkv * D, r.v.begin() + (pos + 1) * Hkv * D);
            }
            qm::DeviceBuffer dq, dk, dv, dpos, dlens, dt, dqr(q.size() * 2), dctx(q.size() * 2);
            upload(q, dq); upload(k, dk); upload(v, dv); upload(plan.positions, dpos); upload(plan.seq_lens, dlens);
            upload(plan.page_table, dt);
            engine.launch_qk_norm_rope_cache_m1(0, dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dw.as<uint16_t>(),
                                                dw.as<uint16_t>(), dpos.as<int32_t>(), dt.as<int32_t>(), plan.max_pages,
                                                plan.batch, dqr.as<uint16_t>());
            engine.launch_attention(0, dqr.as<uint16_t>(), dlens.as<int32_t>(), dt.as<int32_t>(), plan.max_pages, plan.batch,
                                    dctx.as<uint16_t>());
            cudaStreamSynchronize(stream);
            if (engine.device_status() != 0) { std::printf("device status set\n"); return -1; }
            std::vector<uint16_t> ctx(q.size());
            cudaMemcpy(ctx.data(), dctx.pointer, ctx.size() * 2, cudaMemcpyDeviceToHost);
            batcher.commit_decode_step(plan);
            // the oracle, one stream at a time
            for (int row = 0; row < plan.batch; ++row) {
                Request& r = *by_slot[plan.slots[(size_t)row]];
                const int pos = plan.positions[(size_t)row];
                if (pos != r.oracle_length) { std::printf("plan position %d, stream holds %d tokens\n", pos, r.oracle_length); return -1; }
                std::vector<uint16_t> qrot((size_t)Hq * D);
                qmo_append(r.q.data() + (size_t)pos * Hq * D, r.k.data() + (size_t)pos * Hkv * D, r.v.data() + (size_t)pos * Hkv * D,
                           norm_w.data(), norm_w.data(), cosv.data() + (size_t)pos * D, sinv.data() + (size_t)pos * D, 1.0e-6f, 1, pos,
                           Hq, Hkv, kMaxCache, qrot.data(), r.key_cache.data(), r.value_cache.data());
                r.oracle_length = pos + 1;
                const uint16_t* kcp = r.key_cache.data();
                const uint16_t* vcp = r.value_cache.data();
                int32_t mc = kMaxCache, len = pos + 1;
                std::vector<float> want((size_t)Hq * D);
                qmo_decode_attention_batch(qrot.data(), &kcp, &vcp, &mc, &len, 1, Hq, Hkv, 1, nullptr, want.data());
                double max_abs = 0, num = 0, den = 0;
                for (size_t i = 0; i < want.size(); ++i) {
                    const double d = std::fabs((double)qmo_bf16_to_f32(ctx[(size_t)row * Hq * D + i]) - want[i]);
                    max_abs = d > max_abs ? d : max_abs;
                    num += d;
                    den += std::fabs(want[i]);
                }
                worst_abs = max_abs > worst_abs ? max_abs : worst_abs;
                worst_rel = num / den > worst_rel ? num / den : worst_rel;
                ++checked;
            }
            return plan.batch;
        };

        // two requests arrive together
        Request a(1, 70, 70 + 40), b(2, 130, 130 + 40);
        const int sa = batcher.admit(a.id, a.prompt, 40), sb = batcher.admit(b.id, b.prompt, 3);
        if (sa < 0 || sb < 0) { std::printf("admission refused\n"); return 2; }
        by_slot[sa] = &a; by_slot[sb] = &b;
        prefill({sa, sb});
        if (decode_step() != 2 || decode_step() != 2) return 3;
        // a third one joins: prefilled alone, then it decodes with the others
        Request c(3, 5, 5 + 40);
        const int sc = batcher.admit(c.id, c.prompt, 40);
        if (sc < 0) { std::printf("third admission refused\n"); return 2; }
        by_slot[sc] = &c;
        prefill({sc});
        if (decode_step() != 3) return 3;
        // request 2 has produced its 3 tokens: it drops out of the plans by itself and is retired
        if (!batcher.finished(sb) || decode_step() != 2) return 3;
        const std::vector<int> released = batcher.pages(sb);
        batcher.retire(sb);
        by_slot.erase(sb);
        // the next request takes the slot and the pages that were just released
        Request d(4, 64, 64 + 40);
        const int sd = batcher.admit(d.id, d.prompt, 40);
        if (sd != sb) { std::printf("freed slot not reused\n"); return 2; }
        by_slot[sd] = &d;
        prefill({sd});
        if (batcher.pages(sd)[0] != released.back()) { std::printf("freed page not reused\n"); return 2; }
        for (int step = 0; step < 4; ++step)
            if (decode_step() != 3) return 3;
        std::printf("stream batcher: %d stream-steps checked, worst max_abs %.3g mean_rel %.3g\n", checked, worst_abs, worst_rel);
        if (!(worst_abs <= 2e-2 && worst_rel <= 1e-2)) return 4;      // bf16 tolerance against the fp32 oracle
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 1;
    }
    std::printf("STREAM_BATCHER_GPU_OK\n");
    return 0;
}
