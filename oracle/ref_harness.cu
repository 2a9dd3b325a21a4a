// Include-only harness around the reference engine's own device kernels.
//
// TEST INFRASTRUCTURE ONLY: nothing in the shipped library links or loads it.
// It compiles the reference's 1.7B translation unit unmodified, from where it
// lies in the reference checkout (REFERENCE_DIR on the nvcc command line), and
// exposes plain C entry points that launch the reference's talker kernels with
// host buffers.  No reference source is copied: the only reference text here
// is the names of the symbols being called.
//
// Built by oracle/Makefile into oracle/_ref/libqm_refkernels.so.  Used to
//   * pin the C restatement (oracle/qm_oracle.c) against the reference's real
//     output bits on the same inputs,
//   * produce the golden fixtures under tests/golden/,
//   * time the reference's kernels on the same GPU for the report.
//
// Kernels launched (devices/rtx4090-24g/qwen3_tts_1_7b.cu):
//   talker_qk_norm_rope_cache_fused_kernel    :15412   launcher :17741
//   talker_attention_gqa2_m1_locality_kernel  :16061   dispatch :17916
//   talker_attention_kernel                   :15791   dispatch :17954
//   talker_rope_rows_kernel                   :15578   launcher :17780
//   talker_scatter_prefill_kv_kernel          :15677   launcher :17818
//   code_predictor::rmsnorm_kernel            :8295    launcher :8927
//   talker_linear_fused_kernel                :15250   launcher :17646
//   talker_add_postnorm_fused_kernel          :16258   launcher :17989
//   talker_gate_up_swiglu_fused_kernel        :16348   launcher :18020
// and the code predictor's one-row kernels (namespace code_predictor; launchers :13395-13575):
//   predictor_qkv_m1_fused_kernel             :12063   launcher qkv_m1
//   predictor_qk_norm_rope_cache_m1_kernel    :12150   launcher qk_norm_rope_cache_m1
//   predictor_attention_gqa2_m1_kernel        :12331   launcher attention_m1
//   predictor_linear_m1_fused_kernel          :12596   launcher linear_m1
//   predictor_add_postnorm_m1_kernel          :12675   launcher add_postnorm_m1
//   predictor_gate_up_swiglu_m1_kernel        :12753   launcher gate_up_swiglu_m1
// Launch shapes and shared-memory sizes follow the cited launchers.

#define main qm_refharness_unused_reference_main
#include "devices/rtx4090-24g/qwen3_tts_1_7b.cu"
#undef main

#include <cstdint>
#include <cstring>

namespace {

namespace rt = qwen3_tts::baseline::talker;
namespace rp = qwen3_tts::baseline::code_predictor;

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    cudaError_t alloc(size_t n) {
        bytes = n;
        return cudaMalloc(&p, n ? n : 1);
    }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    template <class T>
    T* as() {
        return static_cast<T*>(p);
    }
};

#define RH_CHECK(expr)                                   \
    do {                                                 \
        cudaError_t rh_status = (expr);                  \
        if (rh_status != cudaSuccess) return (int)rh_status; \
    } while (0)

constexpr int kD = 128;

}  // namespace

extern "C" {

// Decode: fused per-head RMSNorm + RoPE; K heads also append K (roped) and V
// (raw) at cache_position.  Caches are host arrays [kv_heads][max_cache][128],
// updated in place.  cosine/sine: the 128-entry row of that position.
int qmref_decode_append(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* q_norm_w,
                        const uint16_t* k_norm_w, const uint16_t* cosine, const uint16_t* sine, uint16_t* q_rot,
                        uint16_t* key_cache, uint16_t* value_cache, int q_heads, int kv_heads, int max_cache,
                        int cache_position) {
    const size_t qb = (size_t)q_heads * kD * 2, kb = (size_t)kv_heads * kD * 2;
    const size_t cb = (size_t)kv_heads * max_cache * kD * 2;
    DevBuf dq, dk, dv, dqw, dkw, dc, ds, dqr, dkc, dvc;
    RH_CHECK(dq.alloc(qb)); RH_CHECK(dk.alloc(kb)); RH_CHECK(dv.alloc(kb));
    RH_CHECK(dqw.alloc(kD * 2)); RH_CHECK(dkw.alloc(kD * 2)); RH_CHECK(dc.alloc(kD * 2)); RH_CHECK(ds.alloc(kD * 2));
    RH_CHECK(dqr.alloc(qb)); RH_CHECK(dkc.alloc(cb)); RH_CHECK(dvc.alloc(cb));
    RH_CHECK(cudaMemcpy(dq.p, q, qb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dk.p, k, kb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dv.p, v, kb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dqw.p, q_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkw.p, k_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dc.p, cosine, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(ds.p, sine, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkc.p, key_cache, cb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvc.p, value_cache, cb, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rt::talker_qk_norm_rope_cache_fused_kernel, dim3((unsigned)(q_heads + kv_heads)), dim3(128), 0,
                         (cudaStream_t) nullptr, dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(),
                         dqw.as<uint16_t>(), dkw.as<uint16_t>(), dc.as<uint16_t>(), ds.as<uint16_t>(),
                         dqr.as<uint16_t>(), dkc.as<uint16_t>(), dvc.as<uint16_t>(), q_heads, kv_heads, kD, max_cache,
                         cache_position, 1.0e-6f);
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(q_rot, dqr.p, qb, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(key_cache, dkc.p, cb, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(value_cache, dvc.p, cb, cudaMemcpyDeviceToHost));
    return 0;
}

// Prefill spelling of the same math: rmsnorm(q), rmsnorm(k), rope(q), rope(k),
// scatter into the cache rows 0..seq-1.  cosine/sine [seq][128].
int qmref_prefill_append(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* q_norm_w,
                         const uint16_t* k_norm_w, const uint16_t* cosine, const uint16_t* sine, uint16_t* q_rot,
                         uint16_t* key_cache, uint16_t* value_cache, int seq, int q_heads, int kv_heads,
                         int max_cache) {
    const size_t qb = (size_t)seq * q_heads * kD * 2, kb = (size_t)seq * kv_heads * kD * 2;
    const size_t cb = (size_t)kv_heads * max_cache * kD * 2, rb = (size_t)seq * kD * 2;
    DevBuf dq, dk, dv, dqw, dkw, dc, ds, dqn, dkn, dqr, dkr, dkc, dvc;
    RH_CHECK(dq.alloc(qb)); RH_CHECK(dk.alloc(kb)); RH_CHECK(dv.alloc(kb));
    RH_CHECK(dqw.alloc(kD * 2)); RH_CHECK(dkw.alloc(kD * 2)); RH_CHECK(dc.alloc(rb)); RH_CHECK(ds.alloc(rb));
    RH_CHECK(dqn.alloc(qb)); RH_CHECK(dkn.alloc(kb)); RH_CHECK(dqr.alloc(qb)); RH_CHECK(dkr.alloc(kb));
    RH_CHECK(dkc.alloc(cb)); RH_CHECK(dvc.alloc(cb));
    RH_CHECK(cudaMemcpy(dq.p, q, qb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dk.p, k, kb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dv.p, v, kb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dqw.p, q_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkw.p, k_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dc.p, cosine, rb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(ds.p, sine, rb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkc.p, key_cache, cb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvc.p, value_cache, cb, cudaMemcpyHostToDevice));
    rp::launch_rmsnorm(dq.as<uint16_t>(), dqw.as<uint16_t>(), dqn.as<uint16_t>(), seq * q_heads, kD, nullptr);
    rp::launch_rmsnorm(dk.as<uint16_t>(), dkw.as<uint16_t>(), dkn.as<uint16_t>(), seq * kv_heads, kD, nullptr);
    {
        const uint64_t count = (uint64_t)seq * q_heads * kD;
        QINGMING_CUDA_LAUNCH(rt::talker_rope_rows_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0,
                             (cudaStream_t) nullptr, dqn.as<uint16_t>(), dc.as<uint16_t>(), ds.as<uint16_t>(),
                             dqr.as<uint16_t>(), seq, q_heads, kD);
        RH_CHECK(cudaGetLastError());
    }
    {
        const uint64_t count = (uint64_t)seq * kv_heads * kD;
        QINGMING_CUDA_LAUNCH(rt::talker_rope_rows_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0,
                             (cudaStream_t) nullptr, dkn.as<uint16_t>(), dc.as<uint16_t>(), ds.as<uint16_t>(),
                             dkr.as<uint16_t>(), seq, kv_heads, kD);
        RH_CHECK(cudaGetLastError());
        QINGMING_CUDA_LAUNCH(rt::talker_scatter_prefill_kv_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0,
                             (cudaStream_t) nullptr, dkr.as<uint16_t>(), dv.as<uint16_t>(), dkc.as<uint16_t>(),
                             dvc.as<uint16_t>(), seq, kv_heads, kD, max_cache);
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(q_rot, dqr.p, qb, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(key_cache, dkc.p, cb, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(value_cache, dvc.p, cb, cudaMemcpyDeviceToHost));
    return 0;
}

// Attention over a cache that already holds keys 0..cache_before+query_length-1.
// query_length == 1 with q_heads == 2*kv_heads takes the GQA-2 M=1 kernel,
// anything else the generic one, exactly as the reference dispatcher does.
// iterations > 1 repeats the launch and reports the mean milliseconds per
// launch through *mean_ms (device time, CUDA events).  Returns a cudaError_t
// value, or -2 when the dynamic shared memory the launcher would request
// exceeds the 48 KB the reference never raises.
int qmref_attention(const uint16_t* q_rot, const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* context,
                    int query_length, int cache_before, int q_heads, int kv_heads, int max_cache, int iterations,
                    float* mean_ms) {
    const size_t qb = (size_t)query_length * q_heads * kD * 2;
    const size_t cb = (size_t)kv_heads * max_cache * kD * 2;
    const int max_key_len = cache_before + query_length;
    const float scale = 1.0f / std::sqrt((float)kD);
    const bool gqa2 = query_length == 1 && q_heads == 2 * kv_heads;
    const size_t shared = gqa2 ? (size_t)(2 * kD + 2 * max_key_len) * 2 : (size_t)(kD + max_key_len) * 2;
    if (shared > 48 * 1024) return -2;
    DevBuf dq, dkc, dvc, dctx;
    RH_CHECK(dq.alloc(qb)); RH_CHECK(dkc.alloc(cb)); RH_CHECK(dvc.alloc(cb)); RH_CHECK(dctx.alloc(qb));
    RH_CHECK(cudaMemcpy(dq.p, q_rot, qb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkc.p, key_cache, cb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvc.p, value_cache, cb, cudaMemcpyHostToDevice));
    cudaEvent_t e0, e1;
    RH_CHECK(cudaEventCreate(&e0));
    RH_CHECK(cudaEventCreate(&e1));
    if (iterations < 1) iterations = 1;
    for (int it = -1; it < iterations; ++it) {
        if (it == 0) RH_CHECK(cudaEventRecord(e0, nullptr));
        if (gqa2) {
            QINGMING_CUDA_LAUNCH(rt::talker_attention_gqa2_m1_locality_kernel, dim3((unsigned)kv_heads), dim3(256),
                                 shared, (cudaStream_t) nullptr, dq.as<uint16_t>(), dkc.as<uint16_t>(),
                                 dvc.as<uint16_t>(), dctx.as<uint16_t>(), cache_before, q_heads, kv_heads, kD,
                                 max_cache, -1, scale);
        } else {
            QINGMING_CUDA_LAUNCH(rt::talker_attention_kernel, dim3((unsigned)(q_heads * query_length)), dim3(256),
                                 shared, (cudaStream_t) nullptr, dq.as<uint16_t>(), dkc.as<uint16_t>(),
                                 dvc.as<uint16_t>(), dctx.as<uint16_t>(), query_length, cache_before, q_heads,
                                 kv_heads, kD, max_cache, -1, scale);
        }
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaEventRecord(e1, nullptr));
    RH_CHECK(cudaDeviceSynchronize());
    float ms = 0.0f;
    RH_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    if (mean_ms) *mean_ms = ms / (float)iterations;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    RH_CHECK(cudaMemcpy(context, dctx.p, qb, cudaMemcpyDeviceToHost));
    return 0;
}

// ---- the non-attention operators of the talker layer, one row at a time (the reference is M = 1) ----
// Launch shapes follow launch_linear_m1 (:17646), launch_add_postnorm_m1 (:17989),
// launch_gate_up_swiglu_m1 (:18020) and code_predictor::launch_rmsnorm (:8927).

// out[r] = linear(x[r]) (+bias) (+residual[r]); weight [n_dim][k_dim].
int qmref_linear_rows(const uint16_t* x, const uint16_t* weight, const uint16_t* bias, const uint16_t* residual,
                      uint16_t* out, int rows, int n_dim, int k_dim) {
    DevBuf dx, dw, db, dr, dout;
    RH_CHECK(dx.alloc((size_t)rows * k_dim * 2)); RH_CHECK(dw.alloc((size_t)n_dim * k_dim * 2));
    RH_CHECK(db.alloc((size_t)n_dim * 2)); RH_CHECK(dr.alloc((size_t)rows * n_dim * 2)); RH_CHECK(dout.alloc((size_t)rows * n_dim * 2));
    RH_CHECK(cudaMemcpy(dx.p, x, dx.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, weight, dw.bytes, cudaMemcpyHostToDevice));
    if (bias) RH_CHECK(cudaMemcpy(db.p, bias, db.bytes, cudaMemcpyHostToDevice));
    if (residual) RH_CHECK(cudaMemcpy(dr.p, residual, dr.bytes, cudaMemcpyHostToDevice));
    for (int r = 0; r < rows; ++r) {
        QINGMING_CUDA_LAUNCH(rt::talker_linear_fused_kernel, dim3((unsigned)((n_dim + 15) / 16)), dim3(256), (size_t)k_dim * 2,
                             (cudaStream_t) nullptr, dx.as<uint16_t>() + (size_t)r * k_dim, dw.as<uint16_t>(),
                             bias ? db.as<uint16_t>() : (uint16_t*)nullptr,
                             residual ? dr.as<uint16_t>() + (size_t)r * n_dim : (uint16_t*)nullptr,
                             dout.as<uint16_t>() + (size_t)r * n_dim, n_dim, k_dim);
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_rmsnorm_rows(const uint16_t* x, const uint16_t* weight, uint16_t* out, int rows, int dim) {
    DevBuf dx, dw, dout;
    RH_CHECK(dx.alloc((size_t)rows * dim * 2)); RH_CHECK(dw.alloc((size_t)dim * 2)); RH_CHECK(dout.alloc((size_t)rows * dim * 2));
    RH_CHECK(cudaMemcpy(dx.p, x, dx.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, weight, dw.bytes, cudaMemcpyHostToDevice));
    rp::launch_rmsnorm(dx.as<uint16_t>(), dw.as<uint16_t>(), dout.as<uint16_t>(), rows, dim, nullptr);
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_add_postnorm_rows(const uint16_t* hidden, const uint16_t* attention, const uint16_t* weight, uint16_t* residual,
                            uint16_t* normalized, int rows, int dim) {
    DevBuf dh, da, dw, dr, dn;
    const size_t bytes = (size_t)rows * dim * 2;
    RH_CHECK(dh.alloc(bytes)); RH_CHECK(da.alloc(bytes)); RH_CHECK(dw.alloc((size_t)dim * 2)); RH_CHECK(dr.alloc(bytes)); RH_CHECK(dn.alloc(bytes));
    RH_CHECK(cudaMemcpy(dh.p, hidden, bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(da.p, attention, bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, weight, (size_t)dim * 2, cudaMemcpyHostToDevice));
    for (int r = 0; r < rows; ++r) {
        const size_t off = (size_t)r * dim;
        QINGMING_CUDA_LAUNCH(rt::talker_add_postnorm_fused_kernel, dim3(1), dim3(256), (size_t)dim * 2, (cudaStream_t) nullptr,
                             dh.as<uint16_t>() + off, da.as<uint16_t>() + off, dw.as<uint16_t>(), dr.as<uint16_t>() + off,
                             dn.as<uint16_t>() + off, dim, 1.0e-6f);
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(residual, dr.p, bytes, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(normalized, dn.p, bytes, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_gate_up_swiglu_rows(const uint16_t* x, const uint16_t* gate_w, const uint16_t* up_w, uint16_t* out, int rows,
                              int hidden, int intermediate) {
    DevBuf dx, dg, du, dout;
    RH_CHECK(dx.alloc((size_t)rows * hidden * 2)); RH_CHECK(dg.alloc((size_t)intermediate * hidden * 2));
    RH_CHECK(du.alloc((size_t)intermediate * hidden * 2)); RH_CHECK(dout.alloc((size_t)rows * intermediate * 2));
    RH_CHECK(cudaMemcpy(dx.p, x, dx.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dg.p, gate_w, dg.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(du.p, up_w, du.bytes, cudaMemcpyHostToDevice));
    for (int r = 0; r < rows; ++r) {
        QINGMING_CUDA_LAUNCH(rt::talker_gate_up_swiglu_fused_kernel, dim3((unsigned)((intermediate + 15) / 16)), dim3(256),
                             (size_t)hidden * 2, (cudaStream_t) nullptr, dx.as<uint16_t>() + (size_t)r * hidden, dg.as<uint16_t>(),
                             du.as<uint16_t>(), dout.as<uint16_t>() + (size_t)r * intermediate, hidden, intermediate);
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// The prefill loop's projections (17.cu:16730-16880): native_ops::linear_bf16 for `rows` token rows at once, and
// code_predictor::launch_add for the residual sum that follows the o- and down-projections.
int qmref_linear_generic(const uint16_t* x, const uint16_t* weight, const uint16_t* bias, const uint16_t* residual,
                         uint16_t* out, int rows, int n_dim, int k_dim) {
    DevBuf dx, dw, db, dr, dout;
    RH_CHECK(dx.alloc((size_t)rows * k_dim * 2)); RH_CHECK(dw.alloc((size_t)n_dim * k_dim * 2));
    RH_CHECK(db.alloc((size_t)n_dim * 2)); RH_CHECK(dr.alloc((size_t)rows * n_dim * 2)); RH_CHECK(dout.alloc((size_t)rows * n_dim * 2));
    RH_CHECK(cudaMemcpy(dx.p, x, dx.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, weight, dw.bytes, cudaMemcpyHostToDevice));
    if (bias) RH_CHECK(cudaMemcpy(db.p, bias, db.bytes, cudaMemcpyHostToDevice));
    if (residual) RH_CHECK(cudaMemcpy(dr.p, residual, dr.bytes, cudaMemcpyHostToDevice));
    try {
        qwen3_tts::native_ops::linear_bf16(dx.as<uint16_t>(), dw.as<uint16_t>(), bias ? db.as<uint16_t>() : (uint16_t*)nullptr,
                                           dout.as<uint16_t>(), rows, n_dim, k_dim, nullptr);
        if (residual) rp::launch_add(dr.as<uint16_t>(), dout.as<uint16_t>(), dout.as<uint16_t>(), (uint64_t)rows * n_dim, nullptr);
    } catch (const std::exception&) {
        return 1;
    }
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// The prefill loop's gate and up projections (linear_bf16 twice) followed by code_predictor::launch_swiglu.
int qmref_gate_up_swiglu_generic(const uint16_t* x, const uint16_t* gate_w, const uint16_t* up_w, uint16_t* out, int rows,
                                 int hidden, int intermediate) {
    DevBuf dx, dg, du, dgate, dup, dout;
    const size_t out_bytes = (size_t)rows * intermediate * 2;
    RH_CHECK(dx.alloc((size_t)rows * hidden * 2)); RH_CHECK(dg.alloc((size_t)intermediate * hidden * 2));
    RH_CHECK(du.alloc((size_t)intermediate * hidden * 2)); RH_CHECK(dgate.alloc(out_bytes)); RH_CHECK(dup.alloc(out_bytes));
    RH_CHECK(dout.alloc(out_bytes));
    RH_CHECK(cudaMemcpy(dx.p, x, dx.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dg.p, gate_w, dg.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(du.p, up_w, du.bytes, cudaMemcpyHostToDevice));
    try {
        qwen3_tts::native_ops::linear_bf16(dx.as<uint16_t>(), dg.as<uint16_t>(), nullptr, dgate.as<uint16_t>(), rows, intermediate, hidden, nullptr);
        qwen3_tts::native_ops::linear_bf16(dx.as<uint16_t>(), du.as<uint16_t>(), nullptr, dup.as<uint16_t>(), rows, intermediate, hidden, nullptr);
        rp::launch_swiglu(dgate.as<uint16_t>(), dup.as<uint16_t>(), dout.as<uint16_t>(), (uint64_t)rows * intermediate, nullptr);
    } catch (const std::exception&) {
        return 1;
    }
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// The reference's final-head chain for one stream, as NativeFinalHead::run_fast strings it together:
// cast_final_head_logits, repetition_penalty (flag 1), suppress_tokens (flag 2), then argmax_final_head
// (top_k <= 0) or gpu_sample_topk_f32_kernel, then record_sampled_code_kernel (flag 4).  The vocabulary is the
// reference's fixed 3072.  processed: 3072 floats out; history updated in place when recording; rng_state in/out.
int qmref_final_head(const uint16_t* logits, int32_t* history, int history_count, int generation_index, int flags,
                     int top_k, float temperature, uint64_t* rng_state, float* processed, int32_t* code_out) {
    namespace rb = qwen3_tts::baseline;
    constexpr int kVocab = 3072;
    DevBuf dl, dp, dh, dseen, dcode, drng;
    RH_CHECK(dl.alloc(kVocab * 2)); RH_CHECK(dp.alloc(kVocab * sizeof(float)));
    RH_CHECK(dh.alloc(8192 * sizeof(int32_t))); RH_CHECK(dseen.alloc(kVocab)); RH_CHECK(dcode.alloc(sizeof(int32_t)));
    RH_CHECK(drng.alloc(sizeof(uint64_t)));
    RH_CHECK(cudaMemcpy(dl.p, logits, kVocab * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemset(dseen.p, 0, kVocab));
    if (history_count > 0) RH_CHECK(cudaMemcpy(dh.p, history, (size_t)history_count * sizeof(int32_t), cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(drng.p, rng_state, sizeof(uint64_t), cudaMemcpyHostToDevice));
    const dim3 grid((kVocab + 255) / 256), block(256);
    QINGMING_CUDA_LAUNCH(rb::cast_final_head_logits, grid, block, 0, (cudaStream_t) nullptr, dl.as<uint16_t>(), dp.as<float>());
    RH_CHECK(cudaGetLastError());
    if (flags & 1) {
        QINGMING_CUDA_LAUNCH(rb::repetition_penalty, grid, block, 0, (cudaStream_t) nullptr, dp.as<float>(),
                             dh.as<int32_t>(), history_count);
        RH_CHECK(cudaGetLastError());
    }
    if (flags & 2) {
        QINGMING_CUDA_LAUNCH(rb::suppress_tokens, grid, block, 0, (cudaStream_t) nullptr, dp.as<float>(), generation_index);
        RH_CHECK(cudaGetLastError());
    }
    if (top_k > 0) {
        QINGMING_CUDA_LAUNCH(rb::gpu_sample_topk_f32_kernel, dim3(1), dim3(rb::kGpuSamplerThreads),
                             rb::gpu_sampler_shared_bytes(), (cudaStream_t) nullptr, dp.as<float>(), kVocab, top_k,
                             temperature, drng.as<std::uint64_t>(), dcode.as<int32_t>());
    } else {
        QINGMING_CUDA_LAUNCH(rb::argmax_final_head, dim3(1), dim3(256), 0, (cudaStream_t) nullptr, dp.as<float>(),
                             dcode.as<int32_t>());
    }
    RH_CHECK(cudaGetLastError());
    if (flags & 4) {
        QINGMING_CUDA_LAUNCH(rb::record_sampled_code_kernel, dim3(1), dim3(1), 0, (cudaStream_t) nullptr, dcode.as<int32_t>(),
                             dh.as<int32_t>(), dseen.as<std::uint8_t>(), generation_index);
        RH_CHECK(cudaGetLastError());
    }
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(processed, dp.p, kVocab * sizeof(float), cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(code_out, dcode.p, sizeof(int32_t), cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(rng_state, drng.p, sizeof(uint64_t), cudaMemcpyDeviceToHost));
    if (flags & 4) RH_CHECK(cudaMemcpy(history + generation_index, dh.as<int32_t>() + generation_index, sizeof(int32_t),
                                       cudaMemcpyDeviceToHost));
    return 0;
}

// ---- the code predictor's one-row kernels (fixed shapes: hidden 1024, SwiGLU 3072, 16 / 8 heads of 128,
// caches [8][16][128]).  One call = one launch with the launcher's grid, block and shared-memory size.

int qmref_predictor_qkv_m1(const uint16_t* input, const uint16_t* q_w, const uint16_t* k_w, const uint16_t* v_w, uint16_t* q_out,
                           uint16_t* k_out, uint16_t* v_out) {
    constexpr int H = rp::kHidden, QD = rp::kQueryDim, KD = rp::kKvDim;
    DevBuf di, dqw, dkw, dvw, dq, dk, dv;
    RH_CHECK(di.alloc(H * 2)); RH_CHECK(dqw.alloc((size_t)QD * H * 2)); RH_CHECK(dkw.alloc((size_t)KD * H * 2));
    RH_CHECK(dvw.alloc((size_t)KD * H * 2)); RH_CHECK(dq.alloc(QD * 2)); RH_CHECK(dk.alloc(KD * 2)); RH_CHECK(dv.alloc(KD * 2));
    RH_CHECK(cudaMemcpy(di.p, input, di.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dqw.p, q_w, dqw.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkw.p, k_w, dkw.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvw.p, v_w, dvw.bytes, cudaMemcpyHostToDevice));
    const int total = QD + 2 * KD;
    QINGMING_CUDA_LAUNCH(rp::predictor_qkv_m1_fused_kernel, dim3((unsigned)((total + 15) / 16)), dim3(rp::kThreads), (size_t)H * 2,
                         (cudaStream_t) nullptr, di.as<uint16_t>(), dqw.as<uint16_t>(), dkw.as<uint16_t>(), dvw.as<uint16_t>(),
                         dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>());
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(q_out, dq.p, dq.bytes, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(k_out, dk.p, dk.bytes, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(v_out, dv.p, dv.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// caches are host arrays [8][16][128], updated in place at cache_position; cosine / sine: that position's 128-entry row.
int qmref_predictor_qk_norm_rope_cache_m1(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* q_norm_w,
                                          const uint16_t* k_norm_w, const uint16_t* cosine, const uint16_t* sine, uint16_t* q_rot,
                                          uint16_t* key_cache, uint16_t* value_cache, int cache_position) {
    constexpr int QD = rp::kQueryDim, KD = rp::kKvDim;
    const size_t cb = (size_t)rp::kKvHeads * rp::kMaxCache * kD * 2;
    DevBuf dq, dk, dv, dqw, dkw, dc, ds, dqr, dkc, dvc;
    RH_CHECK(dq.alloc(QD * 2)); RH_CHECK(dk.alloc(KD * 2)); RH_CHECK(dv.alloc(KD * 2)); RH_CHECK(dqw.alloc(kD * 2));
    RH_CHECK(dkw.alloc(kD * 2)); RH_CHECK(dc.alloc(kD * 2)); RH_CHECK(ds.alloc(kD * 2)); RH_CHECK(dqr.alloc(QD * 2));
    RH_CHECK(dkc.alloc(cb)); RH_CHECK(dvc.alloc(cb));
    RH_CHECK(cudaMemcpy(dq.p, q, dq.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dk.p, k, dk.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dv.p, v, dv.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dqw.p, q_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkw.p, k_norm_w, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dc.p, cosine, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(ds.p, sine, kD * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkc.p, key_cache, cb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvc.p, value_cache, cb, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rp::predictor_qk_norm_rope_cache_m1_kernel, dim3((unsigned)(rp::kQueryHeads + rp::kKvHeads)), dim3(rp::kThreads),
                         0, (cudaStream_t) nullptr, dq.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dqw.as<uint16_t>(),
                         dkw.as<uint16_t>(), dc.as<uint16_t>(), ds.as<uint16_t>(), dqr.as<uint16_t>(), dkc.as<uint16_t>(),
                         dvc.as<uint16_t>(), cache_position);
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(q_rot, dqr.p, dqr.bytes, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(key_cache, dkc.p, cb, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(value_cache, dvc.p, cb, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_predictor_attention_m1(const uint16_t* q_rot, const uint16_t* key_cache, const uint16_t* value_cache, uint16_t* context,
                                 int key_length) {
    constexpr int QD = rp::kQueryDim;
    const size_t cb = (size_t)rp::kKvHeads * rp::kMaxCache * kD * 2;
    if (key_length < 1 || key_length > rp::kMaxCache) return -2;
    DevBuf dq, dkc, dvc, dctx;
    RH_CHECK(dq.alloc(QD * 2)); RH_CHECK(dkc.alloc(cb)); RH_CHECK(dvc.alloc(cb)); RH_CHECK(dctx.alloc(QD * 2));
    RH_CHECK(cudaMemcpy(dq.p, q_rot, dq.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dkc.p, key_cache, cb, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dvc.p, value_cache, cb, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rp::predictor_attention_gqa2_m1_kernel, dim3((unsigned)rp::kKvHeads), dim3(rp::kThreads), 0,
                         (cudaStream_t) nullptr, dq.as<uint16_t>(), dkc.as<uint16_t>(), dvc.as<uint16_t>(), dctx.as<uint16_t>(), key_length);
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(context, dctx.p, dctx.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// out[n] = dot(input, weight[n]) (+ residual[n]); weight [n_dim][k_dim]; residual may be null.
int qmref_predictor_linear_m1(const uint16_t* input, const uint16_t* weight, const uint16_t* residual, uint16_t* out, int n_dim,
                              int k_dim) {
    DevBuf di, dw, dr, dout;
    RH_CHECK(di.alloc((size_t)k_dim * 2)); RH_CHECK(dw.alloc((size_t)n_dim * k_dim * 2)); RH_CHECK(dr.alloc((size_t)n_dim * 2));
    RH_CHECK(dout.alloc((size_t)n_dim * 2));
    RH_CHECK(cudaMemcpy(di.p, input, di.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, weight, dw.bytes, cudaMemcpyHostToDevice));
    if (residual) RH_CHECK(cudaMemcpy(dr.p, residual, dr.bytes, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rp::predictor_linear_m1_fused_kernel, dim3((unsigned)((n_dim + 15) / 16)), dim3(rp::kThreads), (size_t)k_dim * 2,
                         (cudaStream_t) nullptr, di.as<uint16_t>(), dw.as<uint16_t>(), residual ? dr.as<uint16_t>() : (uint16_t*)nullptr,
                         dout.as<uint16_t>(), n_dim, k_dim);
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_predictor_add_postnorm_m1(const uint16_t* hidden, const uint16_t* attention, const uint16_t* norm_w, uint16_t* residual,
                                    uint16_t* normalized) {
    constexpr int H = rp::kHidden;
    DevBuf dh, da, dw, dr, dn;
    RH_CHECK(dh.alloc(H * 2)); RH_CHECK(da.alloc(H * 2)); RH_CHECK(dw.alloc(H * 2)); RH_CHECK(dr.alloc(H * 2)); RH_CHECK(dn.alloc(H * 2));
    RH_CHECK(cudaMemcpy(dh.p, hidden, H * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(da.p, attention, H * 2, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dw.p, norm_w, H * 2, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rp::predictor_add_postnorm_m1_kernel, dim3(1), dim3(rp::kThreads), 0, (cudaStream_t) nullptr, dh.as<uint16_t>(),
                         da.as<uint16_t>(), dw.as<uint16_t>(), dr.as<uint16_t>(), dn.as<uint16_t>());
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(residual, dr.p, H * 2, cudaMemcpyDeviceToHost));
    RH_CHECK(cudaMemcpy(normalized, dn.p, H * 2, cudaMemcpyDeviceToHost));
    return 0;
}

int qmref_predictor_gate_up_swiglu_m1(const uint16_t* input, const uint16_t* gate_w, const uint16_t* up_w, uint16_t* out) {
    constexpr int H = rp::kHidden, I = rp::kIntermediate;
    DevBuf di, dg, du, dout;
    RH_CHECK(di.alloc(H * 2)); RH_CHECK(dg.alloc((size_t)I * H * 2)); RH_CHECK(du.alloc((size_t)I * H * 2)); RH_CHECK(dout.alloc(I * 2));
    RH_CHECK(cudaMemcpy(di.p, input, di.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(dg.p, gate_w, dg.bytes, cudaMemcpyHostToDevice));
    RH_CHECK(cudaMemcpy(du.p, up_w, du.bytes, cudaMemcpyHostToDevice));
    QINGMING_CUDA_LAUNCH(rp::predictor_gate_up_swiglu_m1_kernel, dim3((unsigned)((I + 15) / 16)), dim3(rp::kThreads), (size_t)H * 2,
                         (cudaStream_t) nullptr, di.as<uint16_t>(), dg.as<uint16_t>(), du.as<uint16_t>(), dout.as<uint16_t>());
    RH_CHECK(cudaGetLastError());
    RH_CHECK(cudaDeviceSynchronize());
    RH_CHECK(cudaMemcpy(out, dout.p, dout.bytes, cudaMemcpyDeviceToHost));
    return 0;
}

// Host RoPE table exactly as the engine builds it.
int qmref_make_rope(int rows, int start, uint16_t* cosine, uint16_t* sine) {
    auto r = qwen3_tts::baseline::make_talker_rope(rows, start);
    std::memcpy(cosine, r.cos.data(), r.cos.size() * 2);
    std::memcpy(sine, r.sin.data(), r.sin.size() * 2);
    return 0;
}

}  // extern "C"
