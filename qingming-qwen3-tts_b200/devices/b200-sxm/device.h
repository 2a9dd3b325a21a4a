#pragma once

//   NVIDIA B200 SXM 180GB / GB100
//   CUDA target: sm_100a
//
// Counterpart of devices/rtx4090-24g/device.h in the reference tree: the hardware contract and kernel policy of
// this device directory, plus the device gate its main.cu calls.
//
// Hardware contract (read at run time where the reference hard-codes it):
//   SMs:                       148 (two dies of 74); the count is queried, kernels size their grids from it
//   warp size:                 32
//   shared memory / block max: 227 KiB
//   tensor memory / SM:        256 KiB (tcgen05 accumulators)
//   HBM3e:                     180 GB
//
// Kernel policy:
//   hand-written sm_100a kernels behind the C ABI of qm_attention.h; no cuBLAS / CUTLASS / cuDNN dependency
//   BF16 model storage with FP32 accumulation, the reference's bf16 materialisation points kept
//   KV cache: paged, 64-token pages, pool[page][kv_head][64][128] per layer
//   decode attention: split-KV over 2 x SM-count CTAs, cp.async.bulk + mbarrier ring
//   prefill attention and projections: tcgen05.mma with TMEM accumulators, TMA-fed
//
// Execution families (same translation-unit switch as the other device directories):
//   QINGMING_MODEL_FAMILY_1_7B   hidden 2048, SwiGLU 6144, 28 layers
//   QINGMING_MODEL_FAMILY_0_6B   hidden 1024, SwiGLU 3072, 28 layers
//   both: 16 query / 8 KV heads of 128, RoPE theta 1e6, codec vocabulary 3072
//
// Resident scheduler: one generation stream (cuda non-blocking), many requests batched per step.

#include <stdexcept>
#include <string>

#include "qm_attention.h"

namespace qingming::b200_sxm {

#if defined(QINGMING_MODEL_FAMILY_1_7B)
inline constexpr const char* kFamily = "1.7b";
inline constexpr int kHidden = 2048;
inline constexpr int kIntermediate = 6144;
#elif defined(QINGMING_MODEL_FAMILY_0_6B)
inline constexpr const char* kFamily = "0.6b";
inline constexpr int kHidden = 1024;
inline constexpr int kIntermediate = 3072;
#else
#error "define QINGMING_MODEL_FAMILY_1_7B or QINGMING_MODEL_FAMILY_0_6B (CMake: -DQINGMING_MODEL_FAMILY=1.7b|0.6b)"
#endif
inline constexpr const char* kDevice = "b200-sxm";
inline constexpr int kLayers = 28;
inline constexpr int kQueryHeads = 16;
inline constexpr int kKvHeads = 8;
inline constexpr int kCodecVocab = 3072;

// Stands where validate_rtx4090_24g_device stands in the reference's main (qwen3_tts_1_7b.cu:7769-7804): compute
// capability 10.x and 32-wide warps are required; the SM count is returned, not compared with a constant.
inline int validate_b200_device(int device) {
    int sm_count = 0;
    if (qm_validate_b200_device(device, &sm_count) != QM_OK)
        throw std::runtime_error(std::string("B200 device validation: ") + qm_last_error_string());
    return sm_count;
}

}  // namespace qingming::b200_sxm
