// Host-only checks of the resident loop's protocol helpers (host/resident_loop_b200.hpp): request parsing with the
// reference's validation messages (parse_resident_request, 17.cu:26356-26450), fnv1a64 (17.cu:869), the
// non-blocking line source, JSON escaping and the profile report keys (main.cu:1268-1277).  Touches no GPU.
#include <unistd.h>

#include <cstdio>
#include <iostream>
#include <sstream>
#include <string>

#include "resident_loop_b200.hpp"

static int failures = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("line %d: %s\n", __LINE__, #cond);                  \
            ++failures;                                                     \
        }                                                                   \
    } while (0)

static std::string error_of(const std::string& line) {
    try {
        qm::parse_resident_request(line, 0);
    } catch (const std::exception& e) {
        return e.what();
    }
    return "";
}

int main() {
    // ---- requests
    const qm::ResidentRequest r = qm::parse_resident_request(
        "{\"prompt_rows\": 120, \"seed\": 18446744073709551615, \"max_new_tokens\": 200, \"output\": \"a \\\"b\\\".bin\"}", 7);
    EXPECT(r.index == 7 && r.prompt_rows == 120 && r.seed == 18446744073709551615ull && r.max_new_tokens == 200);
    EXPECT(r.output == "a \"b\".bin");
    const qm::ResidentRequest t = qm::parse_resident_request("{\"text\":\"abc\",\"max_new_tokens\":1,\"output\":\"-\"}", 0);
    EXPECT(t.prompt_rows == 12 && t.seed == 0);
    EXPECT(error_of("{\"prompt_rows\": 5, \"max_new_tokens\": 3}") == "resident request requires \"output\"");
    EXPECT(error_of("{\"prompt_rows\": 5, \"output\": \"x\"}") == "resident request requires max_new_tokens");
    EXPECT(error_of("{\"prompt_rows\": 5, \"output\": \"x\", \"max_new_tokens\": 0}") == "resident request max_new_tokens must be in [1,8192]");
    EXPECT(error_of("{\"prompt_rows\": 5, \"output\": \"x\", \"max_new_tokens\": 8193}") == "resident request max_new_tokens must be in [1,8192]");
    EXPECT(error_of("{\"output\": \"x\", \"max_new_tokens\": 4}") == "resident request requires non-empty \"text\"");
    EXPECT(error_of("{\"prompt_rows\": 0, \"output\": \"x\", \"max_new_tokens\": 4}") == "resident prefill rows must be positive");
    EXPECT(error_of("{\"prompt_rows\": 5, \"output\": \"x\", \"max_new_tokens\": 99999999999999999999}").find("overflow") != std::string::npos);
    EXPECT(error_of("{\"prompt_rows\": 5, \"output\": \"x\", \"seed\": -3, \"max_new_tokens\": 4}").find("unsigned") != std::string::npos);
    EXPECT(qm::generation_capacity_for(200) == 256 && qm::generation_capacity_for(257) == 512 && qm::generation_capacity_for(8192) == 8192);

    // ---- hash and generator.  The reference starts its FNV-1a from 1469598103934665603 (17.cu:872), which is not
    // the usual 64-bit offset basis; results must be comparable with its "codec_fnv1a64", so that start is kept:
    // ("a" -> (start ^ 0x61) * 1099511628211 mod 2^64).  Then the first SplitMix64 outputs of seed 0.
    EXPECT(qm::fnv1a64("a", 1) == 0x44bd8ad473cd9906ull);
    EXPECT(qm::fnv1a64("", 0) == 1469598103934665603ull);
    uint64_t state = 0;
    EXPECT(qm::splitmix64_next(state) == 0xe220a8397b1dcdafull);
    EXPECT(qm::splitmix64_next(state) == 0x6e789e6aa1b965f4ull);

    // ---- line source over a pipe: nothing yet, then lines, then a last line without newline, then exhausted
    int fds[2];
    EXPECT(pipe(fds) == 0);
    qm::LineSource source(fds[0]);
    EXPECT(!source.next(false).has_value() && !source.exhausted());
    const std::string text = "one\n\ntwo\nlast";
    EXPECT(write(fds[1], text.data(), text.size()) == (ssize_t)text.size());
    auto line = source.next(false);
    EXPECT(line && *line == "one");
    line = source.next(false);
    EXPECT(line && line->empty());
    line = source.next(true);
    EXPECT(line && *line == "two");
    EXPECT(!source.next(false).has_value());     // "last" is not a line until the writer closes or sends a newline
    close(fds[1]);
    line = source.next(true);
    EXPECT(line && *line == "last");
    EXPECT(!source.next(true).has_value() && source.exhausted());
    close(fds[0]);

    // ---- result plumbing
    EXPECT(qm::json_escape("a\"b\\c\n") == "a\\\"b\\\\c\\n");
    qm::TalkerDecodeGpuProfile a, b;
    a.total_ms = 2.0; a.attention_ms = 1.0; a.qk_norm_rope_cache_ms = 0.25;
    b.total_ms = 4.0; b.attention_ms = 3.0; b.qk_norm_rope_cache_ms = 0.75;
    const qm::TalkerDecodeGpuProfile mean = qm::mean_profile({a, b});
    EXPECT(mean.total_ms == 3.0 && mean.attention_ms == 2.0 && mean.qk_norm_rope_cache_ms == 0.5);
    const std::string fields = qm::generation_profile_json_fields(mean);
    for (const char* key : {"profile_talker_decode_ms", "profile_talker_input_norm_ms", "profile_talker_qkv_ms",
                            "profile_talker_qk_norm_rope_cache_ms", "profile_talker_attention_ms", "profile_talker_o_projection_ms",
                            "profile_talker_residual_postnorm_ms", "profile_talker_gate_up_swiglu_ms",
                            "profile_talker_down_residual_ms", "profile_talker_final_norm_ms"})
        EXPECT(fields.find(std::string("\"") + key + "\":") != std::string::npos);
    EXPECT(fields.find("\"profile_talker_attention_ms\":2.000000") != std::string::npos);
    std::ostringstream report;
    qm::print_generation_profile(report, mean);
    EXPECT(report.str().find("generation_profile_talker_qk_norm_rope_cache_mean_ms: 0.500000") != std::string::npos);
    // a span that is switched off owns nothing and measures nothing
    qm::GenerationProfileEventSpan off(false);
    EXPECT(!off.enabled() && off.elapsed_ms() == 0.0);

    if (failures) return 1;
    std::printf("RESIDENT_PROTOCOL_OK\n");
    return 0;
}
