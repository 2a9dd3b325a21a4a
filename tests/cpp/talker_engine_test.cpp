// Runs the C++ talker drivers (host/talker_engine_b200.hpp: NativeTalkerEngineB200::decode_device / prefill, the
// counterparts of the reference's 17.cu:17189-17435 and :16654-16912) on inputs a test wrote as raw files, and
// writes what they produce back as raw files for the test to compare with the CPU oracle's chain.
//
//   talker_engine_test.bin DIR mode=decode|prefill layers=L hidden=H intermediate=I num_pages=P max_pages=M
//                          batch=B rope_rows=R [total=T max_seqlen=S] [profile=0|1]
// Inputs in DIR (bf16 as uint16, ints as int32, row-major):
//   l<i>_{input_norm,post_norm,q,k,v,o,gate,up,down,q_norm,k_norm}.bin, final_norm.bin
//   decode:  x.bin [B][H], positions.bin [B], page_table.bin [B][M], kpool<i>.bin / vpool<i>.bin [P][8][64][128]
//   prefill: x.bin [T][H], cu_seqlens.bin [B+1], page_table.bin [B][M], last_rows.bin [B]
// Outputs in DIR: out_final.bin (final norm rows), out_kpool<i>.bin / out_vpool<i>.bin, prefill: out_last.bin;
// with profile=1 the reference's report lines and JSON keys are printed.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "talker_engine_b200.hpp"

static std::string g_dir;

template <class T>
static std::vector<T> read_file(const std::string& name, std::size_t expect_elems = 0) {
    std::ifstream f(g_dir + "/" + name, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + name);
    const std::size_t bytes = (std::size_t)f.tellg();
    f.seekg(0);
    std::vector<T> v(bytes / sizeof(T));
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)bytes);
    if (expect_elems && v.size() != expect_elems)
        throw std::runtime_error(name + ": expected " + std::to_string(expect_elems) + " elements, found " + std::to_string(v.size()));
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
    const T* put(const std::vector<T>& host) {
        buffers.emplace_back(host.size() * sizeof(T));
        if (cudaMemcpy(buffers.back().pointer, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess)
            throw std::runtime_error("upload failed");
        return buffers.back().as<T>();
    }
};

int main(int argc, char** argv) {
    try {
        if (argc < 3) throw std::runtime_error("usage: talker_engine_test.bin DIR key=value ...");
        g_dir = argv[1];
        std::map<std::string, std::string> kv;
        for (int i = 2; i < argc; ++i) {
            const std::string a = argv[i];
            const std::size_t eq = a.find('=');
            if (eq == std::string::npos) throw std::runtime_error("expected key=value: " + a);
            kv[a.substr(0, eq)] = a.substr(eq + 1);
        }
        auto num = [&](const char* key, int fallback = -1) {
            const auto it = kv.find(key);
            if (it == kv.end()) {
                if (fallback < 0) throw std::runtime_error(std::string("missing ") + key);
                return fallback;
            }
            return std::atoi(it->second.c_str());
        };
        const std::string mode = kv.count("mode") ? kv["mode"] : "decode";
        const int layers = num("layers"), hidden = num("hidden"), inter = num("intermediate"), num_pages = num("num_pages"),
                  max_pages = num("max_pages"), batch = num("batch"), rope_rows = num("rope_rows"), profile = num("profile", 0);
        const int hq = 16, hkv = 8, d = QM_HEAD_DIM, qd = hq * d, kd = hkv * d;

        cudaStream_t stream;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) throw std::runtime_error("stream");
        Uploads up;
        qm::TalkerWeights w;
        w.hidden = hidden;
        w.intermediate = inter;
        w.q_heads = hq;
        w.kv_heads = hkv;
        for (int l = 0; l < layers; ++l) {
            const std::string p = "l" + std::to_string(l) + "_";
            qm::TalkerLayerWeights lw;
            lw.input_norm = up.put(read_file<uint16_t>(p + "input_norm.bin", (std::size_t)hidden));
            lw.post_norm = up.put(read_file<uint16_t>(p + "post_norm.bin", (std::size_t)hidden));
            lw.q_weight = up.put(read_file<uint16_t>(p + "q.bin", (std::size_t)qd * hidden));
            lw.k_weight = up.put(read_file<uint16_t>(p + "k.bin", (std::size_t)kd * hidden));
            lw.v_weight = up.put(read_file<uint16_t>(p + "v.bin", (std::size_t)kd * hidden));
            lw.o_weight = up.put(read_file<uint16_t>(p + "o.bin", (std::size_t)hidden * qd));
            lw.gate_weight = up.put(read_file<uint16_t>(p + "gate.bin", (std::size_t)inter * hidden));
            lw.up_weight = up.put(read_file<uint16_t>(p + "up.bin", (std::size_t)inter * hidden));
            lw.down_weight = up.put(read_file<uint16_t>(p + "down.bin", (std::size_t)hidden * inter));
            lw.q_norm = up.put(read_file<uint16_t>(p + "q_norm.bin", (std::size_t)d));
            lw.k_norm = up.put(read_file<uint16_t>(p + "k_norm.bin", (std::size_t)d));
            w.layers.push_back(lw);
        }
        w.final_norm = up.put(read_file<uint16_t>("final_norm.bin", (std::size_t)hidden));

        const int total = mode == "prefill" ? num("total") : batch;
        qm::NativeTalkerEngineB200 engine(w, num_pages, batch, total, rope_rows, stream, profile != 0);
        qm_kv_pool* pool = engine.attention().pool();
        const std::size_t pool_elems = (std::size_t)num_pages * hkv * QM_PAGE_TOKENS * d;
        const int32_t* table = up.put(read_file<int32_t>("page_table.bin", (std::size_t)batch * max_pages));
        const uint16_t* x = up.put(read_file<uint16_t>("x.bin", (std::size_t)total * hidden));

        if (mode == "decode") {
            for (int l = 0; l < layers; ++l) {
                const auto kp = read_file<uint16_t>("kpool" + std::to_string(l) + ".bin", pool_elems);
                const auto vp = read_file<uint16_t>("vpool" + std::to_string(l) + ".bin", pool_elems);
                cudaMemcpy(qm_kv_pool_key_ptr(pool, l), kp.data(), pool_elems * 2, cudaMemcpyHostToDevice);
                cudaMemcpy(qm_kv_pool_value_ptr(pool, l), vp.data(), pool_elems * 2, cudaMemcpyHostToDevice);
            }
            const auto positions_host = read_file<int32_t>("positions.bin", (std::size_t)batch);
            std::vector<int32_t> lens_host(positions_host);
            int max_position = 0;
            for (int32_t& v : lens_host) {
                max_position = v > max_position ? v : max_position;
                v += 1;
            }
            const int32_t* positions = up.put(positions_host);
            const int32_t* seq_lens = up.put(lens_host);
            engine.decode_device(x, positions, seq_lens, table, max_pages, batch, max_position);
            // the reference's overflow check: a position beyond the page table's reach throws before any launch
            bool threw = false;
            try {
                engine.decode_device(x, positions, seq_lens, table, max_pages, batch, max_pages * QM_PAGE_TOKENS);
            } catch (const std::runtime_error& e) {
                threw = std::string(e.what()) == "Talker device decode cache overflow";
            }
            if (!threw) throw std::runtime_error("cache overflow was not reported");
        } else {
            const int32_t* cu = up.put(read_file<int32_t>("cu_seqlens.bin", (std::size_t)batch + 1));
            const int32_t* last = up.put(read_file<int32_t>("last_rows.bin", (std::size_t)batch));
            engine.reset_request();
            engine.prefill(x, cu, table, max_pages, batch, total, num("max_seqlen"), last);
        }
        if (cudaStreamSynchronize(stream) != cudaSuccess) throw std::runtime_error("synchronize failed");
        const uint32_t status = engine.attention().device_status();
        if (status != 0) throw std::runtime_error("device status " + std::to_string(status));
        write_device("out_final.bin", engine.final_norm(), (std::size_t)engine.final_rows() * hidden * 2);
        if (mode == "prefill") write_device("out_last.bin", engine.last_rows(), (std::size_t)batch * hidden * 2);
        for (int l = 0; l < layers; ++l) {
            write_device("out_kpool" + std::to_string(l) + ".bin", qm_kv_pool_key_ptr(pool, l), pool_elems * 2);
            write_device("out_vpool" + std::to_string(l) + ".bin", qm_kv_pool_value_ptr(pool, l), pool_elems * 2);
        }
        if (profile && mode == "decode") {
            const qm::TalkerDecodeGpuProfile p = engine.last_decode_gpu_profile();
            qm::print_generation_profile(std::cout, p);
            std::cout << "{" << qm::generation_profile_json_fields(p) << "}\n";
        }
        std::cout << "TALKER_ENGINE_OK\n";
        return 0;
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 1;
    }
}
