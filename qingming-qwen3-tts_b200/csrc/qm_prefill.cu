// placeholder, replaced below in the same session
#include "qm_common.cuh"
int32_t qm_pool_build_tensor_maps(qm_kv_pool*) { return QM_OK; }
extern "C" int32_t qm_prefill_attention_varlen(qm_kv_pool*, int32_t, const uint16_t*, const int32_t*, const int32_t*,
                                               const int32_t*, int32_t, int32_t, int32_t, int32_t, int32_t, uint16_t*,
                                               void*) {
    return qm_fail(QM_EINVAL, "prefill attention not built yet");
}
