// Shared declarations of the talker attention library: the pool object, error
// reporting, bf16 helpers and the sm_100a PTX wrappers (mbarrier, bulk copies)
// the kernels use.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/qm_attention.h"

constexpr int kHeadDim = QM_HEAD_DIM;        // 128
constexpr int kPageTokens = QM_PAGE_TOKENS;  // 64
constexpr int kTileElems = kPageTokens * kHeadDim;   // one (page, kv head) tile
constexpr int kTileBytes = kTileElems * 2;           // 16 KB

struct qm_kv_pool {
    int device;
    int layers;
    int num_pages;
    int kv_heads;
    int sm_count;
    size_t layer_elems;      // num_pages * kv_heads * 64 * 128
    uint16_t* key;           // [layers][num_pages][kv_heads][64][128]
    uint16_t* value;
    uint32_t* status_dev;    // QM_DEVSTAT_* bits, written by kernels
    // Tiled tensor maps over one layer's pool viewed as rows of 128 bf16
    // (rows = num_pages * kv_heads * 64), built at creation for the prefill kernel.
    CUtensorMap* key_maps;   // host array [layers]
    CUtensorMap* value_maps;
};

// Records `text` as this thread's last error and returns `code`.
int32_t qm_fail(int32_t code, const char* text);
int32_t qm_fail_cuda(cudaError_t status, const char* operation);

#define QM_CUDA_TRY(expr, what)                                        \
    do {                                                               \
        cudaError_t qm_cuda_status = (expr);                           \
        if (qm_cuda_status != cudaSuccess) return qm_fail_cuda(qm_cuda_status, what); \
    } while (0)

// Launch with programmatic dependent launch allowed: the kernel may start its
// prologue while the previous kernel on the stream drains; it must call
// pdl_wait() before it touches global memory.  Set QM_DISABLE_PDL=1 in the
// environment to launch with plain stream ordering instead.
bool qm_pdl_enabled();

#ifdef __CUDACC__

#include <utility>

template <typename... KArgs, typename... Args>
cudaError_t qm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = qm_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Blocks until the kernels this launch depends on have completed and their writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream begin launching (it still waits in its own pdl_wait()).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- bf16 <-> f32, bit-level (same rounding as 17.cu:15082-15104)

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t v) { return __uint_as_float(v << 16); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float value) {
    uint32_t bits = __float_as_uint(value);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (bits >> 16) | 0x0040u;
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return bits >> 16;
}

__device__ __forceinline__ float round_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

// Low / high bf16 of a packed pair, widened.
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

// Two floats -> packed bf16x2 (a in the low half), round-to-nearest-even, one cvt instruction.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Packed fp32 pair arithmetic (sm_100): both halves in one issue slot.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// max of three in one instruction (sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Packed bf16 pair -> (low, high) as floats.
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t pair) { return make_float2(bf16_lo(pair), bf16_hi(pair)); }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- mbarrier / bulk-copy wrappers (shared::cta addresses as 32-bit)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking look at a barrier phase.  The answer takes a shared-memory round trip (about 190 cycles on
// sm_100a) but the thread only stalls where it first uses it, so a probe issued before a batch of independent
// instructions hides that latency; `mbar_wait_probed` then completes the wait.
__device__ __forceinline__ uint32_t mbar_probe(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Bounded wait.  Returns false when the limit ran out; the caller records
// QM_DEVSTAT_TIMEOUT and carries on with uniform control flow (the data is then
// garbage and the host sees the status bit), so no thread is left behind at a
// later barrier.  `dead` short-circuits every wait after the first failure.
constexpr uint32_t kWaitSpinLimit = 1u << 19;

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, bool& dead) {
    if (dead) return false;
    for (uint32_t spin = 0; spin < kWaitSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spin > 256) __nanosleep(128);
    }
    dead = true;
    return false;
}

__device__ __forceinline__ bool mbar_wait_probed(uint32_t probed, uint32_t bar, uint32_t parity, bool& dead) {
    if (probed) return !dead;
    return mbar_wait_bounded(bar, parity, dead);
}

// 1-D bulk copy global -> shared::cta, completion counted on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// L2 eviction policies for bulk copies: data read once (a streamed KV tile) should leave first, data fetched
// ahead of its use (a prefetched tile) should stay until it is read.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_copy_g2s_hint(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2_hint(const void* src, uint32_t bytes, uint64_t policy) {
    asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(src), "r"(bytes), "l"(policy) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

#endif  // __CUDACC__
