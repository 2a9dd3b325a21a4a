// The end of a talker decode step: codec-head logits -> next code, for a batch
// of streams, and the embedding row gather that feeds the next step.
//
// Stands in for the reference's final-head chain, which runs one stream at a
// time as five launches (17.cu:14052 cast_final_head_logits, :14063
// repetition_penalty, :14102 suppress_tokens, :14126 argmax_final_head or
// :7546 gpu_sample_topk_f32_kernel, :7668 record_sampled_code_kernel; driver
// NativeFinalHead::run_fast / run_fast_device :14384-14560).  Here one launch
// serves every stream, one CTA per stream, with the same arithmetic:
//
//   score      = float(bf16 logit)
//   repetition : a token found in the stream's history gets score * 1.05 when
//                negative, score * 0x3f73cf3e (the float reciprocal the
//                reference spells out) otherwise
//   suppress   : EOS is -inf while generation_index < 2; every token from
//                reserved_begin on, except EOS, is -inf
//   greedy     : highest score, lowest index among equals
//   top-k      : the k best in (score descending, index ascending) order,
//                weights exp((score - best) / temperature) in double, one
//                SplitMix64 draw from the stream's state, cumulative walk
//   record     : history[generation_index] = code
//
// Ordering is done on 64-bit keys (monotone image of the score in the high
// word, inverted index in the low word), so "better" is a plain integer
// compare; -0.0 is folded into +0.0 first because the reference compares
// floats, and NaN sorts below -inf (the reference never selects a NaN either).
#include <math_constants.h>

#include "qm_common.cuh"

namespace {

constexpr int kSampleThreads = 1024;          // one CTA per stream and few streams: the threads are free
constexpr int kParallelWeights = 1024;        // top-k weights worked out one per thread up to this k
constexpr int kSortSize = 4096;              // as the reference's kGpuSamplerSortSize
constexpr int kBitmapWords = kSortSize / 32;

struct SampleArgs {
    const uint16_t* logits;      // [batch][vocab] bf16
    int32_t* history;            // [batch][history_capacity]
    const int32_t* generation_index;
    uint64_t* rng_state;         // [batch]
    int32_t* codes;              // [batch]
    float* processed;            // [batch][vocab] or null
    uint32_t* status;
    int vocab;
    int history_capacity;
    int flags;
    int eos_token;
    int reserved_begin;
    int top_k;
    float temperature;
};

__device__ __forceinline__ unsigned long long score_key(float score, int index) {
    uint32_t bits = __float_as_uint(score);
    if (bits == 0x80000000u) bits = 0u;                          // -0.0 == +0.0 for the reference's compare
    uint32_t image;
    if ((bits & 0x7fffffffu) > 0x7f800000u) image = 0u;          // NaN: below everything
    else image = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return ((unsigned long long)image << 32) | (unsigned long long)(0xffffffffu - (uint32_t)index);
}

__device__ __forceinline__ float key_score(unsigned long long key) {
    const uint32_t image = (uint32_t)(key >> 32);
    if (image == 0u) return __uint_as_float(0x7fc00000u);
    const uint32_t bits = (image & 0x80000000u) ? (image & 0x7fffffffu) : ~image;
    return __uint_as_float(bits);
}

__device__ __forceinline__ int key_index(unsigned long long key) { return (int)(0xffffffffu - (uint32_t)key); }

// One SplitMix64 step (17.cu:7500-7509) and the 53-bit uniform built from it (:7512-7517).
__device__ __forceinline__ double splitmix_uniform(uint64_t* state) {
    uint64_t z = *state + 0x9e3779b97f4a7c15ULL;
    *state = z;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    z ^= z >> 31;
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

// 64 keys held by one warp, two per lane (elements 2 * lane and 2 * lane + 1), through the steps of a bitonic
// network from `first_width` up to 64: first_width = 2 sorts any 64 keys, first_width = 64 merges a bitonic sequence.
// Element pairs at a distance of 1 are the lane's own two keys, larger distances are a shuffle away.
__device__ __forceinline__ void warp_bitonic64(unsigned long long& k0, unsigned long long& k1, int lane, int first_width,
                                               bool descending) {
    for (int width = first_width; width <= 64; width <<= 1) {
        for (int stride = width >> 1; stride > 0; stride >>= 1) {
            // direction of the pair this element is in: the sequence of `width` elements it belongs to is sorted
            // the requested way when its index has the `width` bit clear (or width is 64), the other way otherwise
            const bool down = (((2 * lane) & width) == 0 || width == 64) ? descending : !descending;
            if (stride == 1) {
                const bool swap = down ? k0 < k1 : k0 > k1;
                if (swap) {
                    const unsigned long long t = k0;
                    k0 = k1;
                    k1 = t;
                }
            } else {
                const unsigned long long o0 = __shfl_xor_sync(0xffffffffu, k0, stride >> 1);
                const unsigned long long o1 = __shfl_xor_sync(0xffffffffu, k1, stride >> 1);
                const bool lower = ((2 * lane) & stride) == 0;            // this lane holds the pair's smaller index
                const bool take_max = lower == down;
                k0 = take_max ? (o0 > k0 ? o0 : k0) : (o0 < k0 ? o0 : k0);
                k1 = take_max ? (o1 > k1 ? o1 : k1) : (o1 < k1 ? o1 : k1);
            }
        }
    }
}

__global__ void __launch_bounds__(kSampleThreads, 1) qm_final_head_sample_kernel(const SampleArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem);                 // [kSortSize]
    uint32_t* seen = reinterpret_cast<uint32_t*>(smem + kSortSize * sizeof(unsigned long long));   // [kBitmapWords]

    pdl_trigger();
    const int tid = threadIdx.x;
    const int stream = blockIdx.x;
    for (int i = tid; i < kBitmapWords; i += kSampleThreads) seen[i] = 0u;
    pdl_wait();

    int generation = a.generation_index ? a.generation_index[stream] : 0;
    if (generation < 0) generation = 0;
    int32_t* history = a.history ? a.history + (size_t)stream * a.history_capacity : nullptr;
    __syncthreads();
    if ((a.flags & QM_SAMPLE_REPETITION) && history) {
        const int count = generation < a.history_capacity ? generation : a.history_capacity;
        for (int i = tid; i < count; i += kSampleThreads) {
            const int token = history[i];
            if (token >= 0 && token < a.vocab) atomicOr(&seen[token >> 5], 1u << (token & 31));
        }
        __syncthreads();
    }

    const uint16_t* row = a.logits + (size_t)stream * a.vocab;
    const float reciprocal = __uint_as_float(0x3f73cf3eu);       // float(1) / float(1.05), as 17.cu:14092
    // Only the first power of two that holds the vocabulary is ordered: the padding keys are worse than any real
    // entry, so the entries beyond it would stay where they are anyway.
    int sort_size = 64;
    while (sort_size < a.vocab) sort_size <<= 1;
    for (int token = tid; token < sort_size; token += kSampleThreads) {
        unsigned long long key = 0ull;                            // padding: worse than any real entry
        if (token < a.vocab) {
            float score = bf16_bits_to_f32(row[token]);
            if ((a.flags & QM_SAMPLE_REPETITION) && ((seen[token >> 5] >> (token & 31)) & 1u))
                score = score < 0.0f ? score * 1.05f : score * reciprocal;
            if (a.flags & QM_SAMPLE_SUPPRESS) {
                if (token == a.eos_token && generation < 2) score = -CUDART_INF_F;
                if (token >= a.reserved_begin && token != a.eos_token) score = -CUDART_INF_F;
            }
            if (a.processed) a.processed[(size_t)stream * a.vocab + token] = score;
            key = score_key(score, token);
        }
        keys[token] = key;
    }
    __syncthreads();

    int code = 0;
    if (a.top_k <= 0) {
        // greedy: the largest key
        unsigned long long best = 0ull;
        for (int i = tid; i < sort_size; i += kSampleThreads) best = keys[i] > best ? keys[i] : best;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
            best = other > best ? other : best;
        }
        __syncthreads();
        if ((tid & 31) == 0) keys[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kSampleThreads / 32; ++w) best = keys[w] > best ? keys[w] : best;
            code = best ? key_index(best) : 0;
        }
    } else if (a.top_k <= 64) {
        // The 64 best keys, in order, are all a draw among at most 64 needs.  Every warp sorts blocks of 64 keys in
        // its registers (even blocks descending, odd ones ascending); then, level by level, the element-wise maximum
        // of a descending and an ascending block is the best 64 of the two as a bitonic sequence, which one more
        // merge puts in order.  The keys are distinct (the index is part of them), so what ends up in keys[0..63]
        // is exactly what a full sort would have put there.
        const int warp = tid >> 5, lane = tid & 31;
        constexpr int kWarps = kSampleThreads / 32;
        int blocks = sort_size >> 6;
        for (int b = warp; b < blocks; b += kWarps) {
            unsigned long long k0 = keys[b * 64 + 2 * lane], k1 = keys[b * 64 + 2 * lane + 1];
            warp_bitonic64(k0, k1, lane, 2, (b & 1) == 0 || blocks == 1);
            keys[b * 64 + 2 * lane] = k0;
            keys[b * 64 + 2 * lane + 1] = k1;
        }
        __syncthreads();
        while (blocks > 1) {
            const int pairs = blocks >> 1;
            unsigned long long m0[2], m1[2];                // a warp takes at most two pairs (4096 keys, 32 warps)
            int mine = 0;
            for (int p = warp; p < pairs; p += kWarps, ++mine) {
                const unsigned long long* x = keys + (2 * p) * 64 + 2 * lane;
                const unsigned long long* y = x + 64;
                m0[mine] = x[0] > y[0] ? x[0] : y[0];
                m1[mine] = x[1] > y[1] ? x[1] : y[1];
            }
            __syncthreads();                                 // everyone has read before anyone writes
            mine = 0;
            for (int p = warp; p < pairs; p += kWarps, ++mine) {
                warp_bitonic64(m0[mine], m1[mine], lane, 64, (p & 1) == 0 || pairs == 1);
                keys[p * 64 + 2 * lane] = m0[mine];
                keys[p * 64 + 2 * lane + 1] = m1[mine];
            }
            __syncthreads();
            blocks = pairs;
        }
    } else {
        // bitonic sort of everything, descending
        for (int width = 2; width <= sort_size; width <<= 1) {
            for (int stride = width >> 1; stride > 0; stride >>= 1) {
                for (int index = tid; index < sort_size; index += kSampleThreads) {
                    const int partner = index ^ stride;
                    if (partner <= index) continue;
                    const bool descending = (index & width) == 0;
                    const unsigned long long x = keys[index], y = keys[partner];
                    if (descending ? x < y : x > y) {
                        keys[index] = y;
                        keys[partner] = x;
                    }
                }
                __syncthreads();
            }
        }
    }
    if (a.top_k > 0) {
        // The k weights exp((score - best) / temperature), in double as the reference has them.  One thread each
        // works them out (the exponentials are the expensive part).  Thread 0 adds them up in the reference's order;
        // its running sums are the reference's cumulative sums as well as, at the end, its total (both loops of the
        // reference add the same numbers in the same order), so they are kept, and the first one above the draw is
        // then found by all threads at once.
        __shared__ double weight[kParallelWeights];
        __shared__ double drawn;
        __shared__ int first_above;
        const int keep = a.top_k < a.vocab ? a.top_k : a.vocab;
        const double inv_t = 1.0 / (double)a.temperature;
        const double maximum = (double)key_score(keys[0]) * inv_t;
        if (keep <= kParallelWeights) {
            if (tid < keep) weight[tid] = exp((double)key_score(keys[tid]) * inv_t - maximum);
            __syncthreads();
            if (tid == 0) {
                double running = 0.0;
                for (int i = 0; i < keep; ++i) {
                    running += weight[i];
                    weight[i] = running;
                }
                // no draw (and no step of the generator) when the weights do not add up to something positive
                first_above = running > 0.0 ? keep : -1;
                drawn = running > 0.0 ? splitmix_uniform(a.rng_state + stream) * running : 0.0;
            }
            __syncthreads();
            if (first_above >= 0 && tid < keep && drawn < weight[tid]) atomicMin(&first_above, tid);
            __syncthreads();
            if (tid == 0) code = key_index(keys[first_above < 0 ? 0 : (first_above < keep ? first_above : keep - 1)]);
        } else if (tid == 0) {
            auto weight_of = [&](int i) { return exp((double)key_score(keys[i]) * inv_t - maximum); };
            double total = 0.0;
            for (int i = 0; i < keep; ++i) total += weight_of(i);
            code = key_index(keys[0]);
            if (total > 0.0) {
                const double target = splitmix_uniform(a.rng_state + stream) * total;
                double cumulative = 0.0;
                code = key_index(keys[keep - 1]);
                for (int i = 0; i < keep; ++i) {
                    cumulative += weight_of(i);
                    if (target < cumulative) {
                        code = key_index(keys[i]);
                        break;
                    }
                }
            }
        }
    }
    if (tid == 0) {
        a.codes[stream] = code;
        if ((a.flags & QM_SAMPLE_RECORD) && history) {
            if (generation < a.history_capacity) history[generation] = code;
            else atomicOr(a.status, QM_DEVSTAT_BAD_POS);
        }
    }
}

// out[r][:] = table[ids[r]][:], 16 bytes per thread (gather_embedding_kernel, 17.cu:8875-8893, for a batch of rows).
__global__ void __launch_bounds__(256) qm_embedding_gather_kernel(const uint16_t* __restrict__ table,
                                                                 const int32_t* __restrict__ ids, int vocab, int hidden,
                                                                 uint16_t* __restrict__ out, uint32_t* status) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y;
    int token = ids[row];
    if (token < 0 || token >= vocab) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, QM_DEVSTAT_BAD_POS);
        token = token < 0 ? 0 : vocab - 1;
    }
    const int chunk = blockIdx.x * blockDim.x + threadIdx.x;      // 8 bf16 each
    if (chunk * 8 < hidden) {
        const uint4 v = *reinterpret_cast<const uint4*>(table + (size_t)token * hidden + chunk * 8);
        *reinterpret_cast<uint4*>(out + (size_t)row * hidden + chunk * 8) = v;
    }
}

}  // namespace

extern "C" {

int32_t qm_final_head_sample(qm_kv_pool* pool, const uint16_t* logits, int32_t batch, int32_t vocab, int32_t* history,
                             int32_t history_capacity, const int32_t* generation_index, int32_t flags,
                             int32_t eos_token, int32_t reserved_begin, int32_t top_k, float temperature,
                             uint64_t* rng_state, int32_t* codes_out, float* processed_out, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (!logits || !codes_out) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (batch < 0 || vocab < 1 || vocab > kSortSize) return qm_fail(QM_EINVAL, "vocab must be between 1 and 4096");
    if ((flags & (QM_SAMPLE_REPETITION | QM_SAMPLE_RECORD)) && (!history || history_capacity < 1 || !generation_index))
        return qm_fail(QM_EINVAL, "repetition penalty and recording need the history and generation_index arrays");
    if ((flags & QM_SAMPLE_SUPPRESS) && !generation_index)
        return qm_fail(QM_EINVAL, "token suppression needs generation_index");
    if (top_k > 0 && (!rng_state || !(temperature > 0.0f)))
        return qm_fail(QM_EINVAL, "top-k sampling needs rng_state and a positive temperature");
    if (batch == 0) return QM_OK;
    constexpr int kSmem = kSortSize * sizeof(unsigned long long) + kBitmapWords * sizeof(uint32_t);
    SampleArgs a{};
    a.logits = logits;
    a.history = history;
    a.generation_index = generation_index;
    a.rng_state = rng_state;
    a.codes = codes_out;
    a.processed = processed_out;
    a.status = pool->status_dev;
    a.vocab = vocab;
    a.history_capacity = history_capacity;
    a.flags = flags;
    a.eos_token = eos_token;
    a.reserved_begin = reserved_begin;
    a.top_k = top_k;
    a.temperature = temperature;
    QM_CUDA_TRY(qm_launch(qm_final_head_sample_kernel, dim3(batch), dim3(kSampleThreads), kSmem,
                          static_cast<cudaStream_t>(stream), a),
                "final head sampling launch");
    return QM_OK;
}

int32_t qm_embedding_gather(qm_kv_pool* pool, const uint16_t* table, const int32_t* token_ids, int32_t rows,
                            int32_t vocab, int32_t hidden, uint16_t* out, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (!table || !token_ids || !out) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (rows < 0 || vocab < 1 || hidden < 8 || (hidden & 7)) return qm_fail(QM_EINVAL, "hidden must be a positive multiple of 8");
    if ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return qm_fail(QM_EINVAL, "table and out must be 16-byte aligned");
    if (rows == 0) return QM_OK;
    const int chunks = hidden / 8;
    QM_CUDA_TRY(qm_launch(qm_embedding_gather_kernel, dim3((chunks + 255) / 256, rows), dim3(256), 0,
                          static_cast<cudaStream_t>(stream), table, token_ids, (int)vocab, (int)hidden, out, pool->status_dev),
                "embedding gather launch");
    return QM_OK;
}

}  // extern "C"
