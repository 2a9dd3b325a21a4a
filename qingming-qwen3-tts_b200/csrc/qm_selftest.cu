// Diagnostic entry point: shows that a device-side wait that never gets its signal gives up, reports
// QM_DEVSTAT_TIMEOUT through the pool's status word and leaves the context usable.  It runs the same bounded
// wait the attention kernels use on an mbarrier that nothing ever arrives on; nothing traps or spins forever.
#include "qm_common.cuh"

namespace {

__global__ void qm_wait_without_signal_kernel(uint32_t* status) {
    __shared__ __align__(8) unsigned long long barrier_storage;
    const uint32_t bar = smem_addr(&barrier_storage);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    bool dead = false;
    if (threadIdx.x == 0) {
        if (!mbar_wait_bounded(bar, 0, dead)) atomicOr(status, QM_DEVSTAT_TIMEOUT);
        // a later wait on the same thread returns at once
        if (mbar_wait_bounded(bar, 0, dead)) atomicOr(status, 0x80000000u);
    }
}

}  // namespace

extern "C" int32_t qm_selftest_wait_timeout(qm_kv_pool* pool, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    qm_wait_without_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pool->status_dev);
    QM_CUDA_TRY(cudaGetLastError(), "bounded-wait self test launch");
    return QM_OK;
}
