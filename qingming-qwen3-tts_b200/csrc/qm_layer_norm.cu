// Row RMSNorm and fused residual-add + post-attention RMSNorm for a batch of token rows.
//
// Stand in for code_predictor::rmsnorm_kernel (17.cu:8295-8357, launcher :8927) and
// talker_add_postnorm_fused_kernel (17.cu:16258-16343, launcher :17989), which the reference launches for one
// row at a time.  One 256-thread block per row with the reference's own reduction shape - thread t accumulates
// columns t, t + 256, ... with fmaf, shuffle-down tree per warp, then the tree over the eight warp sums - and its
// two bf16 roundings, so the bits equal the reference kernels'.
#include "qm_common.cuh"

namespace {

constexpr int kNormThreads = 256;

// Value of the reference's block reductions (block_reduce_sum :8266, talker_block_sum :15150) for 256 threads.
__device__ __forceinline__ float block_sum_reference_order(float value, float* warp_values) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffu, value, offset);
    if (lane == 0) warp_values[warp] = value;
    __syncthreads();
    if (warp == 0) {
        value = lane < kNormThreads / 32 ? warp_values[lane] : 0.0f;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_down_sync(0xffffffffu, value, offset);
        if (lane == 0) warp_values[0] = value;
    }
    __syncthreads();
    return warp_values[0];
}

// hidden == nullptr: plain RMSNorm of x.  Otherwise x is the attention branch: residual = bf16(hidden + x) is
// written out and normalised.
__global__ void __launch_bounds__(kNormThreads) qm_rmsnorm_rows_kernel(const uint16_t* __restrict__ x,
                                                                      const uint16_t* __restrict__ hidden,
                                                                      const uint16_t* __restrict__ weight,
                                                                      uint16_t* __restrict__ residual,
                                                                      uint16_t* __restrict__ normalized, int dim,
                                                                      float epsilon) {
    extern __shared__ uint16_t row_values[];
    __shared__ float warp_values[8];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    float local = 0.0f;
    for (int c = threadIdx.x; c < dim; c += kNormThreads) {
        uint32_t bits = x[base + c];
        if (hidden) {
            bits = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(hidden[base + c]), bf16_bits_to_f32(bits)));
            residual[base + c] = (uint16_t)bits;
        }
        row_values[c] = (uint16_t)bits;
        const float v = bf16_bits_to_f32(bits);
        local = fmaf(v, v, local);
    }
    const float sum = block_sum_reference_order(local, warp_values);
    const float inverse_rms = rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)dim), epsilon));
    for (int c = threadIdx.x; c < dim; c += kNormThreads) {
        const float n = round_bf16(__fmul_rn(bf16_bits_to_f32(row_values[c]), inverse_rms));
        normalized[base + c] = (uint16_t)f32_to_bf16_bits(__fmul_rn(n, bf16_bits_to_f32(weight[c])));
    }
}

// bf16(lo) | bf16(hi) << 16 with the reference's rounding: one cvt.rn.bf16x2 for finite values and infinities,
// where it equals the integer rounding bit for bit; a NaN takes the integer path so that its payload matches too.
__device__ __forceinline__ uint32_t round_pair(float lo, float hi) {
    if (lo != lo || hi != hi) return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
    return pack_bf16x2(lo, hi);
}

// The same arithmetic with 16-byte global accesses and packed roundings.  The row (or hidden + x) is staged in
// shared memory by vector loads and each thread then reads ITS columns t, t + 256, ... from there, so the
// accumulation order and with it every output bit stay those of the kernel above; the normalised row leaves as
// 16-byte stores.  Needs dim % 8 == 0 and 16-byte aligned tensors.
__global__ void __launch_bounds__(kNormThreads) qm_rmsnorm_rows_vec_kernel(const uint16_t* __restrict__ x,
                                                                          const uint16_t* __restrict__ hidden,
                                                                          const uint16_t* __restrict__ weight,
                                                                          uint16_t* __restrict__ residual,
                                                                          uint16_t* __restrict__ normalized, int dim,
                                                                          float epsilon) {
    extern __shared__ uint4 row_vectors[];
    __shared__ float warp_values[8];
    pdl_trigger();
    const int vectors = dim >> 3;
    // The norm weight is a constant of the model: this thread's first piece of it is fetched ahead of the dependency
    // wait, so that its round trip is not left standing at the end of the kernel (rows of up to 2048 columns have no
    // other piece).
    uint4 first_weight = make_uint4(0u, 0u, 0u, 0u);
    if ((int)threadIdx.x < vectors) first_weight = __ldg(reinterpret_cast<const uint4*>(weight + 8 * threadIdx.x));
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim;
    for (int v = threadIdx.x; v < vectors; v += kNormThreads) {
        uint4 raw = *reinterpret_cast<const uint4*>(x + base + 8 * v);
        if (hidden) {
            const uint4 h = *reinterpret_cast<const uint4*>(hidden + base + 8 * v);
            uint32_t* rw = reinterpret_cast<uint32_t*>(&raw);
            const uint32_t* hw = reinterpret_cast<const uint32_t*>(&h);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                rw[i] = round_pair(__fadd_rn(bf16_lo(hw[i]), bf16_lo(rw[i])), __fadd_rn(bf16_hi(hw[i]), bf16_hi(rw[i])));
            *reinterpret_cast<uint4*>(residual + base + 8 * v) = raw;
        }
        row_vectors[v] = raw;
    }
    __syncthreads();
    const uint16_t* row_values = reinterpret_cast<const uint16_t*>(row_vectors);
    float local = 0.0f;
    for (int c = threadIdx.x; c < dim; c += kNormThreads) {
        const float v = bf16_bits_to_f32(row_values[c]);
        local = fmaf(v, v, local);
    }
    const float sum = block_sum_reference_order(local, warp_values);
    const float inverse_rms = rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)dim), epsilon));
    for (int v = threadIdx.x; v < vectors; v += kNormThreads) {
        const uint4 raw = row_vectors[v];
        const uint4 wv = v == (int)threadIdx.x ? first_weight : __ldg(reinterpret_cast<const uint4*>(weight + 8 * v));
        const uint32_t* rw = reinterpret_cast<const uint32_t*>(&raw);
        const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
        uint4 outv;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t n = round_pair(__fmul_rn(bf16_lo(rw[i]), inverse_rms), __fmul_rn(bf16_hi(rw[i]), inverse_rms));
            ow[i] = round_pair(__fmul_rn(bf16_lo(n), bf16_lo(ww[i])), __fmul_rn(bf16_hi(n), bf16_hi(ww[i])));
        }
        *reinterpret_cast<uint4*>(normalized + base + 8 * v) = outv;
    }
}

int32_t launch_norm(const uint16_t* x, const uint16_t* hidden, const uint16_t* weight, uint16_t* residual,
                    uint16_t* normalized, int rows, int dim, float epsilon, cudaStream_t stream, const char* what) {
    if (!x || !weight || !normalized) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (rows < 0 || dim < 1 || dim > 24 * 1024) return qm_fail(QM_EINVAL, "invalid geometry");
    if (rows == 0) return QM_OK;
    const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(weight) |
                          reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(normalized);
    if (dim % 8 == 0 && (all & 15u) == 0)
        QM_CUDA_TRY(qm_launch(qm_rmsnorm_rows_vec_kernel, dim3(rows), dim3(kNormThreads), (size_t)dim * sizeof(uint16_t), stream, x,
                              hidden, weight, residual, normalized, dim, epsilon),
                    what);
    else
        QM_CUDA_TRY(qm_launch(qm_rmsnorm_rows_kernel, dim3(rows), dim3(kNormThreads), (size_t)dim * sizeof(uint16_t), stream, x,
                              hidden, weight, residual, normalized, dim, epsilon),
                    what);
    return QM_OK;
}

}  // namespace

extern "C" {

int32_t qm_rmsnorm(const uint16_t* x, const uint16_t* weight, uint16_t* out, int32_t rows, int32_t dim, float epsilon,
                   void* stream) {
    return launch_norm(x, nullptr, weight, nullptr, out, rows, dim, epsilon, static_cast<cudaStream_t>(stream),
                       "RMSNorm launch");
}

int32_t qm_add_postnorm(const uint16_t* hidden, const uint16_t* attention, const uint16_t* weight, uint16_t* residual,
                        uint16_t* normalized, int32_t rows, int32_t dim, float epsilon, void* stream) {
    if (!hidden || !residual) return qm_fail(QM_EINVAL, "null tensor pointer");
    return launch_norm(attention, hidden, weight, residual, normalized, rows, dim, epsilon,
                       static_cast<cudaStream_t>(stream), "add/postnorm launch");
}

}  // extern "C"
