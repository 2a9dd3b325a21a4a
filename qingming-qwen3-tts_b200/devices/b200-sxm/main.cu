// Production entry of the b200-sxm device directory: the talker serving binary
//     qingming-qwen3-tts_b200-sxm_<family>
// It takes the place devices/rtx4090-24g/main.cu has in the reference tree (a thin main around the family's
// engine), for the part of the engine this device directory provides: the talker decoder on the batched, paged
// attention path.  The family is chosen at compile time exactly as there (-DQINGMING_MODEL_FAMILY_1_7B=1 or
// _0_6B=1).  The reference's checkpoint loader, tokenizer, front-end and codec decoder are outside this path:
// weights are random-init in the family's shapes, a request names its prompt length, and the output file
// receives codec codes.
//
//   --lifecycle resident   JSON request lines on stdin (or --requests FILE), one JSON result line each on stdout
//   --lifecycle once       one request from --prompt-rows / --seed / --max-new-tokens / --output
//   --generation-profile   cudaEvent spans per decode step; the reference's report lines go to stderr and a
//                          final {"status":"profile", "profile_talker_*_ms": ...} line to stdout
//   --layers / --hidden / --intermediate / --max-streams / --num-pages / --max-pages / --top-k /
//   --eos-check-interval / --weight-seed   override the defaults (small shapes for tests)
#include <fcntl.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <string>

#include "device.h"
#include "resident_loop_b200.hpp"
#include "synthetic_weights.hpp"

namespace {

using Options = std::map<std::string, std::string>;

Options parse_options(int argc, char** argv) {
    Options o;
    for (int i = 1; i < argc; ++i) {
        std::string key = argv[i];
        if (key.rfind("--", 0) != 0) throw std::runtime_error("unexpected argument: " + key);
        key = key.substr(2);
        if (key == "generation-profile") {
            o[key] = "1";
        } else {
            if (i + 1 >= argc) throw std::runtime_error("missing value for --" + key);
            o[key] = argv[++i];
        }
    }
    return o;
}

long number(const Options& o, const std::string& key, long fallback) {
    const auto it = o.find(key);
    if (it == o.end()) return fallback;
    char* end = nullptr;
    const long v = std::strtol(it->second.c_str(), &end, 10);
    if (end == it->second.c_str() || *end != '\0') throw std::runtime_error("--" + key + " needs an integer");
    return v;
}

}  // namespace

int main(int argc, char** argv) {
    namespace dev = qingming::b200_sxm;
    try {
        const Options options = parse_options(argc, argv);
        const std::string lifecycle = options.count("lifecycle") ? options.at("lifecycle") : "resident";
        if (lifecycle != "once" && lifecycle != "resident") throw std::runtime_error("--lifecycle once|resident");
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) throw std::runtime_error("cudaGetDevice failed");
        const int sm_count = dev::validate_b200_device(device);

        const int layers = (int)number(options, "layers", dev::kLayers);
        const int hidden = (int)number(options, "hidden", dev::kHidden);
        const int intermediate = (int)number(options, "intermediate", dev::kIntermediate);
        qm::ResidentConfig config;
        config.device = dev::kDevice;
        config.family = dev::kFamily;
        config.vocab = dev::kCodecVocab;
        config.max_streams = (int)number(options, "max-streams", config.max_streams);
        config.num_pages = (int)number(options, "num-pages", config.num_pages);
        config.max_pages_per_stream = (int)number(options, "max-pages", config.max_pages_per_stream);
        config.top_k = (int)number(options, "top-k", config.top_k);
        config.eos_check_interval = (int)number(options, "eos-check-interval", config.eos_check_interval);
        const bool profile = options.count("generation-profile") != 0;
        const int max_prefill_rows = (int)number(options, "max-prefill-rows", 16384);

        cudaStream_t stream = nullptr;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess)
            throw std::runtime_error("Talker generation stream");
        std::cerr << "device: " << dev::kDevice << "\nfamily: " << dev::kFamily << "\nsm_count: " << sm_count
                  << "\ntalker_generation_stream: cuda_nonblocking\n";
        qm::SyntheticTalker model((uint64_t)number(options, "weight-seed", 4), layers, hidden, intermediate, config.vocab,
                                  dev::kQueryHeads, dev::kKvHeads);
        qm::NativeTalkerEngineB200 engine(model.view(), config.num_pages + 1, config.max_streams, max_prefill_rows,
                                          config.max_pages_per_stream * QM_PAGE_TOKENS, stream, profile);
        qm::ResidentTalkerLoopB200 loop(engine, model.view(), model.codec_head(), model.embedding(), config);
        std::cerr << "resident_ready: True\n";

        std::size_t served = 0;
        if (lifecycle == "once") {
            const std::string line = "{\"prompt_rows\": " + std::to_string(number(options, "prompt-rows", 64)) +
                                     ", \"seed\": " + std::to_string(number(options, "seed", 0)) +
                                     ", \"max_new_tokens\": " + std::to_string(number(options, "max-new-tokens", 64)) +
                                     ", \"output\": \"" + (options.count("output") ? options.at("output") : std::string("-")) + "\"}\n";
            int fds[2];
            if (pipe(fds) != 0) throw std::runtime_error("pipe failed");
            if (write(fds[1], line.data(), line.size()) != (ssize_t)line.size()) throw std::runtime_error("pipe write failed");
            close(fds[1]);
            qm::LineSource source(fds[0]);
            served = loop.serve(source, std::cout);
            close(fds[0]);
        } else {
            int fd = 0;
            if (options.count("requests")) {
                fd = open(options.at("requests").c_str(), O_RDONLY);
                if (fd < 0) throw std::runtime_error("failed to open: " + options.at("requests"));
            }
            qm::LineSource source(fd);
            served = loop.serve(source, std::cout);
            if (fd != 0) close(fd);
        }
        if (profile) {
            const qm::TalkerDecodeGpuProfile mean = qm::mean_profile(loop.decode_profiles());
            qm::print_generation_profile(std::cerr, mean);
            std::cout << "{\"status\":\"profile\",\"generation_profile\":true,\"decode_steps\":" << loop.decode_steps() << ","
                      << qm::generation_profile_json_fields(mean) << "}\n";
        }
        std::cerr << "requests_served: " << served << "\ndecode_steps: " << loop.decode_steps() << "\n";
        cudaStreamDestroy(stream);
        return 0;
    } catch (const std::exception& e) {
        std::string text = e.what();
        std::cout << "{\"status\":\"error\",\"device\":\"b200-sxm\",\"error\":\"" << qm::json_escape(text) << "\"}\n";
        return 1;
    }
}
