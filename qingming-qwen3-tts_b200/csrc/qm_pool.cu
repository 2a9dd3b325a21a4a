// Host side of the C ABI that is not a kernel launcher: error text, device
// gate, the paged KV pool object and the RoPE table.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "qm_common.cuh"

namespace {
thread_local char g_error_text[512] = "";
}

int32_t qm_fail(int32_t code, const char* text) {
    std::snprintf(g_error_text, sizeof(g_error_text), "%s", text);
    return code;
}

int32_t qm_fail_cuda(cudaError_t status, const char* operation) {
    std::snprintf(g_error_text, sizeof(g_error_text), "%s: %s", operation, cudaGetErrorString(status));
    if (status == cudaErrorMemoryAllocation) return QM_ENOMEM;
    return QM_ECUDA;
}

bool qm_pdl_enabled() {
    static const bool enabled = [] {
        const char* v = std::getenv("QM_DISABLE_PDL");
        return !(v && v[0] == '1');
    }();
    return enabled;
}

// Defined in qm_prefill.cu: builds the per-layer tiled tensor maps.
int32_t qm_pool_build_tensor_maps(qm_kv_pool* pool);

extern "C" {

const char* qm_last_error_string(void) { return g_error_text; }

int32_t qm_validate_b200_device(int32_t device, int32_t* sm_count_out) {
    cudaDeviceProp prop;
    QM_CUDA_TRY(cudaGetDeviceProperties(&prop, device), "query device properties");
    if (prop.major != 10) {
        char text[160];
        std::snprintf(text, sizeof(text), "device %d is compute capability %d.%d; this library is built for 10.x (B200)",
                      device, prop.major, prop.minor);
        return qm_fail(QM_EDEVICE, text);
    }
    if (prop.warpSize != 32) return qm_fail(QM_EDEVICE, "warp size is not 32");
    if (sm_count_out) *sm_count_out = prop.multiProcessorCount;
    return QM_OK;
}

int32_t qm_kv_pool_create(int32_t layers, int32_t num_pages, int32_t kv_heads, qm_kv_pool** pool_out) {
    if (!pool_out) return qm_fail(QM_EINVAL, "pool_out is null");
    *pool_out = nullptr;
    if (layers < 1 || num_pages < 1 || kv_heads < 1 || kv_heads > 64)
        return qm_fail(QM_EINVAL, "layers and num_pages must be >= 1, kv_heads in 1..64");
    const unsigned long long rows = (unsigned long long)num_pages * kv_heads * kPageTokens;
    if (rows >= (1ull << 31)) return qm_fail(QM_ECAPACITY, "pool rows (num_pages * kv_heads * 64) must stay below 2^31");

    int device = 0;
    QM_CUDA_TRY(cudaGetDevice(&device), "get current device");
    int sm_count = 0;
    int32_t gate = qm_validate_b200_device(device, &sm_count);
    if (gate != QM_OK) return gate;

    qm_kv_pool* pool = new (std::nothrow) qm_kv_pool();
    if (!pool) return qm_fail(QM_ENOMEM, "host allocation of pool object failed");
    std::memset(pool, 0, sizeof(*pool));
    pool->device = device;
    pool->layers = layers;
    pool->num_pages = num_pages;
    pool->kv_heads = kv_heads;
    pool->sm_count = sm_count;
    pool->layer_elems = (size_t)rows * kHeadDim;
    const size_t bytes = pool->layer_elems * sizeof(uint16_t) * (size_t)layers;

    cudaError_t status = cudaMalloc(&pool->key, bytes);
    if (status == cudaSuccess) status = cudaMalloc(&pool->value, bytes);
    if (status == cudaSuccess) status = cudaMalloc(&pool->status_dev, sizeof(uint32_t));
    if (status == cudaSuccess) status = cudaMemset(pool->key, 0, bytes);
    if (status == cudaSuccess) status = cudaMemset(pool->value, 0, bytes);
    if (status == cudaSuccess) status = cudaMemset(pool->status_dev, 0, sizeof(uint32_t));
    if (status == cudaSuccess) status = cudaDeviceSynchronize();
    if (status != cudaSuccess) {
        int32_t code = qm_fail_cuda(status, "allocate KV pool");
        qm_kv_pool_destroy(pool);
        return code;
    }
    int32_t maps = qm_pool_build_tensor_maps(pool);
    if (maps != QM_OK) {
        qm_kv_pool_destroy(pool);
        return maps;
    }
    *pool_out = pool;
    return QM_OK;
}

int32_t qm_kv_pool_destroy(qm_kv_pool* pool) {
    if (!pool) return QM_OK;
    if (pool->key) cudaFree(pool->key);
    if (pool->value) cudaFree(pool->value);
    if (pool->status_dev) cudaFree(pool->status_dev);
    delete[] pool->key_maps;
    delete[] pool->value_maps;
    delete pool;
    return QM_OK;
}

int32_t qm_kv_pool_reset(qm_kv_pool* pool, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = pool->layer_elems * sizeof(uint16_t) * (size_t)pool->layers;
    QM_CUDA_TRY(cudaMemsetAsync(pool->key, 0, bytes, s), "reset K pool");
    QM_CUDA_TRY(cudaMemsetAsync(pool->value, 0, bytes, s), "reset V pool");
    QM_CUDA_TRY(cudaMemsetAsync(pool->status_dev, 0, sizeof(uint32_t), s), "reset status word");
    QM_CUDA_TRY(cudaStreamSynchronize(s), "reset request synchronize");
    return QM_OK;
}

uint16_t* qm_kv_pool_key_ptr(qm_kv_pool* pool, int32_t layer) {
    if (!pool || layer < 0 || layer >= pool->layers) return nullptr;
    return pool->key + (size_t)layer * pool->layer_elems;
}

uint16_t* qm_kv_pool_value_ptr(qm_kv_pool* pool, int32_t layer) {
    if (!pool || layer < 0 || layer >= pool->layers) return nullptr;
    return pool->value + (size_t)layer * pool->layer_elems;
}

int32_t qm_kv_pool_num_pages(const qm_kv_pool* pool) { return pool ? pool->num_pages : 0; }
int32_t qm_kv_pool_kv_heads(const qm_kv_pool* pool) { return pool ? pool->kv_heads : 0; }

int32_t qm_kv_pool_status(qm_kv_pool* pool, void* stream, uint32_t* bits_out) {
    if (!pool || !bits_out) return qm_fail(QM_EINVAL, "pool or bits_out is null");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t bits = 0;
    QM_CUDA_TRY(cudaMemcpyAsync(&bits, pool->status_dev, sizeof(bits), cudaMemcpyDeviceToHost, s), "read status word");
    QM_CUDA_TRY(cudaMemsetAsync(pool->status_dev, 0, sizeof(uint32_t), s), "clear status word");
    QM_CUDA_TRY(cudaStreamSynchronize(s), "status synchronize");
    *bits_out = bits;
    return QM_OK;
}

static inline uint16_t host_f32_to_bf16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

int32_t qm_rope_table_fill(uint16_t* cosine_dev, uint16_t* sine_dev, int32_t rows, int32_t start, double theta,
                           void* stream) {
    if (!cosine_dev || !sine_dev) return qm_fail(QM_EINVAL, "rope table pointer is null");
    if (rows < 0 || start < 0 || !(theta > 0.0)) return qm_fail(QM_EINVAL, "invalid RoPE geometry");
    if (rows == 0) return QM_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int half = kHeadDim / 2;
    std::vector<double> inv(half);
    for (int i = 0; i < half; ++i) inv[i] = std::pow(theta, -2.0 * (double)i / (double)kHeadDim);
    std::vector<uint16_t> c((size_t)rows * kHeadDim), sn((size_t)rows * kHeadDim);
    for (int row = 0; row < rows; ++row) {
        const double pos = (double)(start + row);
        const size_t base = (size_t)row * kHeadDim;
        for (int i = 0; i < half; ++i) {
            const double angle = pos * inv[i];
            const uint16_t cv = host_f32_to_bf16((float)std::cos(angle));
            const uint16_t sv = host_f32_to_bf16((float)std::sin(angle));
            c[base + i] = cv;
            c[base + i + half] = cv;
            sn[base + i] = sv;
            sn[base + i + half] = sv;
        }
    }
    const size_t bytes = c.size() * sizeof(uint16_t);
    QM_CUDA_TRY(cudaMemcpyAsync(cosine_dev, c.data(), bytes, cudaMemcpyHostToDevice, s), "upload RoPE cosine");
    QM_CUDA_TRY(cudaMemcpyAsync(sine_dev, sn.data(), bytes, cudaMemcpyHostToDevice, s), "upload RoPE sine");
    QM_CUDA_TRY(cudaStreamSynchronize(s), "RoPE table synchronize");
    return QM_OK;
}

}  // extern "C"
