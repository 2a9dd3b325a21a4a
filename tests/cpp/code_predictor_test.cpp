// Runs one frame of the C++ code predictor driver (host/code_predictor_b200.hpp, the counterpart of the reference's
// capture_step, 17.cu:13616-13905) on weights and inputs a test wrote as raw files, once with the two rows of step 0
// as two one-row positions and once through the staged many-row path, and writes codes and per-step logits back.
//
//   code_predictor_test.bin DIR streams=S outer=O hidden=H intermediate=I layers=L vocab=V steps=T top_k=K
// Inputs in DIR (bf16 as uint16): projection.bin [H][O], projection_bias.bin [H], final_norm.bin [H],
//   l<i>_{input_norm,post_norm,q,k,v,o,gate,up,down,q_norm,k_norm}.bin, head<t>.bin [V][H], embedding<t>.bin [V][O],
//   talker_hidden.bin [S][O], first_embedding.bin [S][O], rng.bin (uint64 [S])
// Outputs: codes_<mode>.bin int32 [T][S], logits_<mode>.bin [T][S][V], rng_<mode>.bin, mode = positions | staged.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "code_predictor_b200.hpp"

static std::string g_dir;

template <class T>
static std::vector<T> read_file(const std::string& name, std::size_t expect) {
    std::ifstream f(g_dir + "/" + name, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + name);
    const std::size_t bytes = (std::size_t)f.tellg();
    f.seekg(0);
    std::vector<T> v(bytes / sizeof(T));
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)bytes);
    if (v.size() != expect) throw std::runtime_error(name + ": unexpected size");
    return v;
}

static void write_device(const std::string& name, const void* device, std::size_t bytes) {
    std::vector<char> host(bytes);
    if (cudaMemcpy(host.data(), device, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) throw std::runtime_error("download failed");
    std::ofstream f(g_dir + "/" + name, std::ios::binary);
    f.write(host.data(), (std::streamsize)bytes);
}

struct Uploads {
    std::vector<qm::DeviceBuffer> buffers;
    template <class T>
    T* put(const std::vector<T>& host) {
        buffers.emplace_back(host.size() * sizeof(T));
        if (cudaMemcpy(buffers.back().pointer, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess)
            throw std::runtime_error("upload failed");
        return buffers.back().as<T>();
    }
};

int main(int argc, char** argv) {
    try {
        if (argc < 3) throw std::runtime_error("usage: code_predictor_test.bin DIR key=value ...");
        g_dir = argv[1];
        std::map<std::string, int> kv;
        for (int i = 2; i < argc; ++i) {
            const std::string a = argv[i];
            const std::size_t eq = a.find('=');
            if (eq == std::string::npos) throw std::runtime_error("expected key=value: " + a);
            kv[a.substr(0, eq)] = std::atoi(a.substr(eq + 1).c_str());
        }
        const int S = kv.at("streams"), O = kv.at("outer"), H = kv.at("hidden"), I = kv.at("intermediate"), L = kv.at("layers"),
                  V = kv.at("vocab"), T = kv.at("steps"), top_k = kv.at("top_k");
        const int qd = 16 * QM_HEAD_DIM, kd = 8 * QM_HEAD_DIM;
        cudaStream_t stream;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("stream");
        Uploads up;
        qm::CodePredictorWeights w;
        w.outer_hidden = O; w.hidden = H; w.intermediate = I; w.vocab = V; w.steps = T;
        w.projection_weight = up.put(read_file<uint16_t>("projection.bin", (std::size_t)H * O));
        w.projection_bias = up.put(read_file<uint16_t>("projection_bias.bin", (std::size_t)H));
        w.final_norm = up.put(read_file<uint16_t>("final_norm.bin", (std::size_t)H));
        for (int l = 0; l < L; ++l) {
            const std::string p = "l" + std::to_string(l) + "_";
            qm::TalkerLayerWeights lw;
            lw.input_norm = up.put(read_file<uint16_t>(p + "input_norm.bin", (std::size_t)H));
            lw.post_norm = up.put(read_file<uint16_t>(p + "post_norm.bin", (std::size_t)H));
            lw.q_weight = up.put(read_file<uint16_t>(p + "q.bin", (std::size_t)qd * H));
            lw.k_weight = up.put(read_file<uint16_t>(p + "k.bin", (std::size_t)kd * H));
            lw.v_weight = up.put(read_file<uint16_t>(p + "v.bin", (std::size_t)kd * H));
            lw.o_weight = up.put(read_file<uint16_t>(p + "o.bin", (std::size_t)H * qd));
            lw.gate_weight = up.put(read_file<uint16_t>(p + "gate.bin", (std::size_t)I * H));
            lw.up_weight = up.put(read_file<uint16_t>(p + "up.bin", (std::size_t)I * H));
            lw.down_weight = up.put(read_file<uint16_t>(p + "down.bin", (std::size_t)H * I));
            lw.q_norm = up.put(read_file<uint16_t>(p + "q_norm.bin", (std::size_t)QM_HEAD_DIM));
            lw.k_norm = up.put(read_file<uint16_t>(p + "k_norm.bin", (std::size_t)QM_HEAD_DIM));
            w.layers.push_back(lw);
        }
        for (int t = 0; t < T; ++t) {
            w.lm_heads.push_back(up.put(read_file<uint16_t>("head" + std::to_string(t) + ".bin", (std::size_t)V * H)));
            w.embeddings.push_back(up.put(read_file<uint16_t>("embedding" + std::to_string(t) + ".bin", (std::size_t)V * O)));
        }
        const uint16_t* talker_hidden = up.put(read_file<uint16_t>("talker_hidden.bin", (std::size_t)S * O));
        const uint16_t* first_embedding = up.put(read_file<uint16_t>("first_embedding.bin", (std::size_t)S * O));
        const std::vector<uint64_t> rng_host = read_file<uint64_t>("rng.bin", (std::size_t)S);
        qm::DeviceBuffer trace((std::size_t)T * S * V * 2);

        qm::CodePredictorB200 predictor(w, S, stream);
        const struct { const char* name; qm::CodePredictorB200::FirstStep mode; } runs[] = {
            {"positions", qm::CodePredictorB200::FirstStep::kTwoPositions}, {"staged", qm::CodePredictorB200::FirstStep::kStagedRows}};
        for (const auto& run : runs) {
            predictor.attention().reset_request();
            uint64_t* rng = up.put(rng_host);
            const int32_t* codes = predictor.frame(talker_hidden, first_embedding, top_k > 0 ? rng : nullptr, top_k, 0.9f, run.mode,
                                                   trace.as<uint16_t>());
            if (cudaStreamSynchronize(stream) != cudaSuccess) throw std::runtime_error("synchronize failed");
            const uint32_t status = predictor.attention().device_status();
            if (status != 0) throw std::runtime_error("device status " + std::to_string(status));
            write_device(std::string("codes_") + run.name + ".bin", codes, (std::size_t)T * S * sizeof(int32_t));
            write_device(std::string("logits_") + run.name + ".bin", trace.pointer, trace.bytes);
            write_device(std::string("rng_") + run.name + ".bin", rng, (std::size_t)S * sizeof(uint64_t));
        }
        std::cout << "CODE_PREDICTOR_OK\n";
        return 0;
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 1;
    }
}
