// Drives the C++ host mirror the way NativeTalkerEngine::prefill / decode_device drive the reference launchers
// (17.cu:16763-16807, :17284-17309): prefill a short prompt, then one decode step, single stream, identity page
// table - the reference's own operating point - and checks the decode context against the CPU oracle (fp32 mode).
// Exit code 0 = pass.  Links libqm_attention_b200.so and (test-only) libqm_oracle.so.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "talker_attention_b200.hpp"

extern "C" {
void qmo_fill_normal_bf16(uint64_t seed, uint16_t* out, int64_t n);
void qmo_make_rope(int rows, int start, double theta, uint16_t* cosine, uint16_t* sine);
void qmo_append(const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*,
                const uint16_t*, float, int, int, int, int, int, uint16_t*, uint16_t*, uint16_t*);
int qmo_decode_attention_batch(const uint16_t*, const uint16_t* const*, const uint16_t* const*, const int32_t*,
                               const int32_t*, int, int, int, int, uint16_t*, float*);
float qmo_bf16_to_f32(uint16_t);
void qmo_linear(const uint16_t*, const uint16_t*, const uint16_t*, const uint16_t*, int, int, int, int, uint16_t*);
int qmo_final_head_sample(const uint16_t*, int, int32_t*, int, int, int, int, int, int, float, uint64_t*, float*);
}

template <class T>
static T* upload(const std::vector<T>& h, qm::DeviceBuffer& d) {
    d = qm::DeviceBuffer(h.size() * sizeof(T));
    cudaMemcpy(d.pointer, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d.as<T>();
}

int main() {
    const int Hq = 16, Hkv = 8, D = 128, prompt = 70, max_pages = 2, rope_rows = 128;
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    try {
        qm::TalkerAttentionB200 engine(/*layers=*/1, /*num_pages=*/max_pages, Hq, Hkv, /*max_batch=*/1, rope_rows, stream);
        std::vector<uint16_t> q((prompt + 1) * Hq * D), k((prompt + 1) * Hkv * D), v((prompt + 1) * Hkv * D), w(D, 0x3f80);
        qmo_fill_normal_bf16(11, q.data(), (int64_t)q.size());
        qmo_fill_normal_bf16(12, k.data(), (int64_t)k.size());
        qmo_fill_normal_bf16(13, v.data(), (int64_t)v.size());
        std::vector<int32_t> table = {0, 1}, cu = {0, prompt}, pos = {prompt}, lens = {prompt + 1};
        qm::DeviceBuffer dq, dk, dv, dw, dt, dcu, dpos, dlens, dqr((prompt + 1) * Hq * D * 2), dctx(Hq * D * 2);
        upload(q, dq); upload(k, dk); upload(v, dv); upload(w, dw); upload(table, dt); upload(cu, dcu); upload(pos, dpos);
        upload(lens, dlens);
        engine.reset_request();
        // prefill: norm + RoPE + scatter of the prompt (its attention output is not needed for this check)
        engine.scatter_prefill_cache(0, dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dw.as<uint16_t>(),
                                     dw.as<uint16_t>(), dcu.as<int32_t>(), dt.as<int32_t>(), max_pages, 1, prompt,
                                     dqr.as<uint16_t>());
        // decode step at position `prompt`
        const size_t qo = (size_t)prompt * Hq * D, ko = (size_t)prompt * Hkv * D;
        engine.launch_qk_norm_rope_cache_m1(0, dq.as<uint16_t>() + qo, dk.as<uint16_t>() + ko, dv.as<uint16_t>() + ko,
                                            dw.as<uint16_t>(), dw.as<uint16_t>(), dpos.as<int32_t>(), dt.as<int32_t>(),
                                            max_pages, 1, dqr.as<uint16_t>() + qo);
        engine.launch_attention(0, dqr.as<uint16_t>() + qo, dlens.as<int32_t>(), dt.as<int32_t>(), max_pages, 1,
                                dctx.as<uint16_t>());
        if (engine.device_status() != 0) { std::printf("device status set\n"); return 2; }
        std::vector<uint16_t> ctx(Hq * D);
        cudaMemcpy(ctx.data(), dctx.pointer, ctx.size() * 2, cudaMemcpyDeviceToHost);

        // oracle: append all prompt + 1 tokens, attend prompt + 1 keys
        const int max_cache = max_pages * 64;
        std::vector<uint16_t> cosv(rope_rows * D), sinv(rope_rows * D), qrot(q.size()), kc(Hkv * max_cache * D), vc(kc.size());
        qmo_make_rope(rope_rows, 0, 1.0e6, cosv.data(), sinv.data());
        qmo_append(q.data(), k.data(), v.data(), w.data(), w.data(), cosv.data(), sinv.data(), 1.0e-6f, prompt + 1, 0, Hq,
                   Hkv, max_cache, qrot.data(), kc.data(), vc.data());
        const uint16_t* kcp = kc.data();
        const uint16_t* vcp = vc.data();
        std::vector<float> want(Hq * D);
        int32_t mc = max_cache, len = prompt + 1;
        qmo_decode_attention_batch(qrot.data() + qo, &kcp, &vcp, &mc, &len, 1, Hq, Hkv, 1, nullptr, want.data());
        double max_abs = 0, num = 0, den = 0;
        for (size_t i = 0; i < want.size(); ++i) {
            const double d = std::fabs((double)qmo_bf16_to_f32(ctx[i]) - want[i]);
            max_abs = d > max_abs ? d : max_abs;
            num += d;
            den += std::fabs(want[i]);
        }
        std::printf("host mirror decode: max_abs %.3g mean_rel %.3g\n", max_abs, num / den);
        if (!(max_abs <= 2e-2 && num / den <= 1e-2)) return 3;   // bf16 tolerance against the fp32 oracle

        // error behaviour: an out-of-range layer throws before anything is launched
        bool threw = false;
        try {
            engine.launch_attention(7, dqr.as<uint16_t>(), dlens.as<int32_t>(), dt.as<int32_t>(), max_pages, 1, dctx.as<uint16_t>());
        } catch (const std::runtime_error& e) {
            threw = std::string(e.what()).find("attention launch") != std::string::npos;
        }
        if (!threw) { std::printf("invalid layer did not throw\n"); return 4; }

        // the end of a step: logits -> code (greedy, with the reference's processors) -> embedding row
        const int vocab = 3072, hidden = 256;
        std::vector<uint16_t> logits(vocab), table_rows((size_t)vocab * hidden);
        qmo_fill_normal_bf16(21, logits.data(), vocab);
        qmo_fill_normal_bf16(22, table_rows.data(), (int64_t)table_rows.size());
        std::vector<int32_t> history(8192, 0), generation = {3};
        history[0] = 5; history[1] = 6; history[2] = 7;
        uint64_t state = 99;
        std::vector<int32_t> history_copy = history;
        const int want_code = qmo_final_head_sample(logits.data(), vocab, history_copy.data(), 8192, 3, 7, 2150, vocab - 1024, 0,
                                                    0.9f, &state, nullptr);
        qm::DeviceBuffer dlogits, dtable, dhist, dgen, dcode(sizeof(int32_t)), drow(hidden * 2);
        upload(logits, dlogits); upload(table_rows, dtable); upload(history, dhist); upload(generation, dgen);
        engine.final_head_sample(dlogits.as<uint16_t>(), 1, vocab, dhist.as<int32_t>(), 8192, dgen.as<int32_t>(),
                                 QM_SAMPLE_REPETITION | QM_SAMPLE_SUPPRESS | QM_SAMPLE_RECORD, 0, 0.9f, nullptr, dcode.as<int32_t>());
        engine.gather_embeddings(dtable.as<uint16_t>(), dcode.as<int32_t>(), 1, vocab, hidden, drow.as<uint16_t>());
        cudaStreamSynchronize(stream);
        int32_t code = -1, recorded = -1;
        std::vector<uint16_t> row(hidden);
        cudaMemcpy(&code, dcode.pointer, sizeof(code), cudaMemcpyDeviceToHost);
        cudaMemcpy(&recorded, dhist.as<int32_t>() + 3, sizeof(recorded), cudaMemcpyDeviceToHost);
        cudaMemcpy(row.data(), drow.pointer, hidden * 2, cudaMemcpyDeviceToHost);
        if (code != want_code || recorded != want_code) { std::printf("final head: code %d, oracle %d, recorded %d\n", code, want_code, recorded); return 5; }
        for (int i = 0; i < hidden; ++i)
            if (row[i] != table_rows[(size_t)code * hidden + i]) { std::printf("embedding row differs at %d\n", i); return 6; }

        // the prefill loop's generic linear with its residual add, for more rows than one tile holds
        const int prows = 200, pin = 128, pout = 192;
        std::vector<uint16_t> px((size_t)prows * pin), pw((size_t)pout * pin), pb(pout), pres((size_t)prows * pout), pwant((size_t)prows * pout),
            pgot((size_t)prows * pout);
        qmo_fill_normal_bf16(31, px.data(), (int64_t)px.size());
        qmo_fill_normal_bf16(32, pw.data(), (int64_t)pw.size());
        qmo_fill_normal_bf16(33, pb.data(), (int64_t)pb.size());
        qmo_fill_normal_bf16(34, pres.data(), (int64_t)pres.size());
        qmo_linear(px.data(), pw.data(), pb.data(), pres.data(), prows, pout, pin, 1, pwant.data());
        qm::DeviceBuffer dpx, dpw, dpb, dpres, dpout(pgot.size() * 2);
        upload(px, dpx); upload(pw, dpw); upload(pb, dpb); upload(pres, dpres);
        engine.linear_generic(dpx.as<uint16_t>(), dpw.as<uint16_t>(), dpb.as<uint16_t>(), dpres.as<uint16_t>(), dpout.as<uint16_t>(),
                              prows, pout, pin);
        cudaStreamSynchronize(stream);
        cudaMemcpy(pgot.data(), dpout.pointer, pgot.size() * 2, cudaMemcpyDeviceToHost);
        double worst = 0.0;
        for (size_t i = 0; i < pgot.size(); ++i)
            worst = std::fmax(worst, std::fabs((double)qmo_bf16_to_f32(pgot[i]) - (double)qmo_bf16_to_f32(pwant[i])));
        // unit-variance operands: outputs of magnitude up to ~50, one bf16 ulp there is 0.25
        if (!(worst <= 0.26)) { std::printf("generic linear: worst difference %g\n", worst); return 7; }
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 1;
    }
    std::printf("HOST_MIRROR_OK\n");
    return 0;
}
