/*
 * CPU oracle for the Qwen3-TTS talker attention path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or
 * calls this file; it is the checker the tests and the benchmark's CPU
 * baseline compare the CUDA path against.
 *
 * It restates, in plain C, the arithmetic of the reference engine's device
 * kernels (file = devices/rtx4090-24g/qwen3_tts_1_7b.cu of the reference):
 *
 *   bf16 <-> f32                         :15072-15104, :21752-21756
 *   SplitMix64 host RNG                  :7147-7169
 *   RoPE table (double -> bf16)          :21758-21772
 *   per-head RMSNorm                     :8295-8357  (== :15472-15508)
 *   RoPE with rotate_half                :15512-15546 (== :15619-15672)
 *   KV cache layout [kv_head][t][128]    :15553-15572, :15719-15734
 *   decode attention, GQA-2, M=1         :16061-16251
 *   generic (prefill, causal) attention  :15791-16054
 *   softmax scale 1/sqrtf(head_dim)      :17910-17914
 *   warp / block reduction trees         :15107-15245, :8253-8292
 *
 * Two modes:
 *   "ref"  reproduces every bf16 materialisation and the reduction shapes of
 *          the reference kernels (lane-strided fmaf chains + shuffle-down
 *          trees).  Differences from the GPU are limited to libm expf versus
 *          the device expf, and 1/sqrtf versus the device rsqrtf.
 *   "fp32" keeps only the roundings of the stored tensors (bf16 inputs and
 *          cache) and accumulates in double; this is what the stated bf16
 *          tolerance (max abs 2e-2, mean relative 1e-2) is measured against.
 *
 * Parity pin: the reference ships no golden vectors for this path.  The
 * restatement is pinned by fixtures under tests/golden/ that were produced by
 * launching the reference's own kernels (compiled unmodified from its source
 * tree by oracle/ref_harness.cu) on a B200.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QMO_D 128
#define QMO_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 */

static inline float bf16_to_f32(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Round-to-nearest-even with NaN quieting (:15082-15104). */
static inline uint16_t f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffU) > 0x7f800000U) {
        return (uint16_t)((bits >> 16) | 0x0040U);
    }
    bits += 0x7fffU + ((bits >> 16) & 1U);
    return (uint16_t)(bits >> 16);
}

static inline float rnd(float value) { return bf16_to_f32(f32_to_bf16(value)); }

QMO_EXPORT uint16_t qmo_f32_to_bf16(float v) { return f32_to_bf16(v); }
QMO_EXPORT float qmo_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }

QMO_EXPORT void qmo_f32_to_bf16_array(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}

/* ------------------------------------------------------------------- RNG */

/* SplitMix64 (:7154-7161). */
static inline uint64_t splitmix64_next(uint64_t* state) {
    *state += 0x9e3779b97f4a7c15ULL;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

static inline double uniform01(uint64_t* state) {
    return (double)(splitmix64_next(state) >> 11) * (1.0 / 9007199254740992.0);
}

QMO_EXPORT uint64_t qmo_splitmix64(uint64_t* state) { return splitmix64_next(state); }

/* N(0,1) by Box-Muller on two 53-bit uniforms, cast to bf16 (RNE).  Both
 * normals of each pair are used, in order. */
QMO_EXPORT void qmo_fill_normal_bf16(uint64_t seed, uint16_t* out, int64_t n) {
    uint64_t state = seed;
    for (int64_t i = 0; i < n; i += 2) {
        double u1 = uniform01(&state);
        double u2 = uniform01(&state);
        if (u1 < 1e-300) u1 = 1e-300;
        double radius = sqrt(-2.0 * log(u1));
        double angle = 6.283185307179586476925286766559 * u2;
        out[i] = f32_to_bf16((float)(radius * cos(angle)));
        if (i + 1 < n) out[i + 1] = f32_to_bf16((float)(radius * sin(angle)));
    }
}

/* lo + next_u64() % (hi - lo + 1) for each element. */
QMO_EXPORT void qmo_fill_uniform_int(uint64_t seed, int32_t lo, int32_t hi, int32_t* out, int64_t n) {
    uint64_t state = seed;
    uint64_t span = (uint64_t)((int64_t)hi - (int64_t)lo + 1);
    for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)((int64_t)lo + (int64_t)(splitmix64_next(&state) % span));
}

/* Fisher-Yates shuffle of 0..n-1. */
QMO_EXPORT void qmo_shuffled_range(uint64_t seed, int32_t* out, int64_t n) {
    uint64_t state = seed;
    for (int64_t i = 0; i < n; ++i) out[i] = (int32_t)i;
    for (int64_t i = n - 1; i > 0; --i) {
        int64_t j = (int64_t)(splitmix64_next(&state) % (uint64_t)(i + 1));
        int32_t t = out[i];
        out[i] = out[j];
        out[j] = t;
    }
}

/* ------------------------------------------------------------ RoPE table */

/* make_talker_rope (:21758-21772): rows [start, start+rows), head_dim 128. */
QMO_EXPORT void qmo_make_rope(int rows, int start, double theta, uint16_t* cosine, uint16_t* sine) {
    const int half = QMO_D / 2;
    for (int row = 0; row < rows; ++row) {
        double pos = (double)(start + row);
        for (int i = 0; i < half; ++i) {
            double inv = pow(theta, -2.0 * (double)i / (double)QMO_D);
            double a = pos * inv;
            uint16_t c = f32_to_bf16((float)cos(a));
            uint16_t s = f32_to_bf16((float)sin(a));
            size_t b = (size_t)row * QMO_D;
            cosine[b + i] = c;
            cosine[b + i + half] = c;
            sine[b + i] = s;
            sine[b + i + half] = s;
        }
    }
}

/* ------------------------------------------------------- reduction trees */

/* Value seen by lane 0 after the shuffle-down tree of a 32-lane warp. */
static inline float warp_tree_sum(float* v) {
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
    return v[0];
}

static inline float warp_tree_max(float* v) {
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) v[i] = v[i] > v[i + off] ? v[i] : v[i + off];
    return v[0];
}

/* talker_block_sum / talker_block_max for `threads` threads (multiple of 32,
 * <= 256): per-warp tree, then a tree over the warp results held in lanes
 * 0..warps-1 of warp 0 (other lanes contribute the identity). */
static float block_tree_sum(const float* per_thread, int threads) {
    float warp_values[32];
    for (int i = 0; i < 32; ++i) warp_values[i] = 0.0f;
    int warps = threads / 32;
    for (int w = 0; w < warps; ++w) {
        float lane[32];
        memcpy(lane, per_thread + w * 32, sizeof(lane));
        warp_values[w] = warp_tree_sum(lane);
    }
    return warp_tree_sum(warp_values);
}

static float block_tree_max(const float* per_thread, int threads) {
    float warp_values[32];
    for (int i = 0; i < 32; ++i) warp_values[i] = -INFINITY;
    int warps = threads / 32;
    for (int w = 0; w < warps; ++w) {
        float lane[32];
        memcpy(lane, per_thread + w * 32, sizeof(lane));
        warp_values[w] = warp_tree_max(lane);
    }
    return warp_tree_max(warp_values);
}

/* -------------------------------------------------- RMSNorm + RoPE (ref) */

/* One head row: RMSNorm (2 roundings) then RoPE (3 roundings).
 * x, w, cosine, sine, out: 128 bf16 each.  One thread per dimension, 4 warps
 * (:15472-15546). */
static void norm_rope_head_ref(const uint16_t* x, const uint16_t* w, const uint16_t* cosine,
                               const uint16_t* sine, float eps, uint16_t* out) {
    float sq[QMO_D];
    for (int d = 0; d < QMO_D; ++d) {
        float v = bf16_to_f32(x[d]);
        sq[d] = v * v;
    }
    float sum = block_tree_sum(sq, QMO_D);
    float inv = 1.0f / sqrtf(sum / (float)QMO_D + eps);
    uint16_t normed[QMO_D];
    for (int d = 0; d < QMO_D; ++d) {
        uint16_t nb = f32_to_bf16(bf16_to_f32(x[d]) * inv);
        normed[d] = f32_to_bf16(bf16_to_f32(nb) * bf16_to_f32(w[d]));
    }
    for (int d = 0; d < QMO_D; ++d) {
        int rd = d < QMO_D / 2 ? d + QMO_D / 2 : d - QMO_D / 2;
        float rot = bf16_to_f32(normed[rd]);
        if (d < QMO_D / 2) rot = -rot;
        uint16_t first = f32_to_bf16(bf16_to_f32(normed[d]) * bf16_to_f32(cosine[d]));
        uint16_t second = f32_to_bf16(rot * bf16_to_f32(sine[d]));
        out[d] = f32_to_bf16(bf16_to_f32(first) + bf16_to_f32(second));
    }
}

QMO_EXPORT void qmo_norm_rope_head(const uint16_t* x, const uint16_t* w, const uint16_t* cosine,
                                   const uint16_t* sine, float eps, uint16_t* out) {
    norm_rope_head_ref(x, w, cosine, sine, eps, out);
}

/* RMSNorm only (prefill spelling, rmsnorm_kernel :8295-8357), rows x 128. */
QMO_EXPORT void qmo_rmsnorm_rows(const uint16_t* x, const uint16_t* w, float eps, uint16_t* out, int64_t rows) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * QMO_D;
        float sq[256];
        for (int d = 0; d < 256; ++d) sq[d] = 0.0f;
        for (int d = 0; d < QMO_D; ++d) {
            float v = bf16_to_f32(xr[d]);
            sq[d] = fmaf(v, v, 0.0f);
        }
        float sum = block_tree_sum(sq, 256);
        float inv = 1.0f / sqrtf(sum / (float)QMO_D + eps);
        for (int d = 0; d < QMO_D; ++d) {
            uint16_t nb = f32_to_bf16(bf16_to_f32(xr[d]) * inv);
            out[r * QMO_D + d] = f32_to_bf16(bf16_to_f32(nb) * bf16_to_f32(w[d]));
        }
    }
}

/* talker_rope_rows_kernel (:15578-15673): x [seq][heads][128], cos/sin [seq][128]. */
QMO_EXPORT void qmo_rope_rows(const uint16_t* x, const uint16_t* cosine, const uint16_t* sine, uint16_t* out,
                              int64_t seq, int heads) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < seq; ++row) {
        for (int h = 0; h < heads; ++h) {
            const uint16_t* xr = x + (row * heads + h) * QMO_D;
            uint16_t* o = out + (row * heads + h) * QMO_D;
            for (int d = 0; d < QMO_D; ++d) {
                int rd = d < QMO_D / 2 ? d + QMO_D / 2 : d - QMO_D / 2;
                float rot = bf16_to_f32(xr[rd]);
                if (d < QMO_D / 2) rot = -rot;
                uint16_t first = f32_to_bf16(bf16_to_f32(xr[d]) * bf16_to_f32(cosine[row * QMO_D + d]));
                uint16_t second = f32_to_bf16(rot * bf16_to_f32(sine[row * QMO_D + d]));
                o[d] = f32_to_bf16(bf16_to_f32(first) + bf16_to_f32(second));
            }
        }
    }
}

/*
 * Fused norm + RoPE + append for `tokens` consecutive positions of one
 * sequence (decode: tokens = 1; prefill: the whole prompt).
 *   q [tokens][q_heads][128], k, v [tokens][kv_heads][128]   (pre-norm projections)
 *   cosine, sine [tokens][128]  rows for positions first_pos .. first_pos+tokens-1
 *   q_rot [tokens][q_heads][128]
 *   key_cache, value_cache [kv_heads][max_cache][128]        (:15553-15572)
 * K is cached after norm and RoPE, V is copied raw.
 */
QMO_EXPORT void qmo_append(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* q_norm_w,
                           const uint16_t* k_norm_w, const uint16_t* cosine, const uint16_t* sine, float eps,
                           int tokens, int first_pos, int q_heads, int kv_heads, int max_cache, uint16_t* q_rot,
                           uint16_t* key_cache, uint16_t* value_cache) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < tokens; ++t) {
        const uint16_t* c = cosine + (size_t)t * QMO_D;
        const uint16_t* s = sine + (size_t)t * QMO_D;
        for (int h = 0; h < q_heads; ++h) {
            size_t base = ((size_t)t * q_heads + h) * QMO_D;
            norm_rope_head_ref(q + base, q_norm_w, c, s, eps, q_rot + base);
        }
        for (int h = 0; h < kv_heads; ++h) {
            size_t src = ((size_t)t * kv_heads + h) * QMO_D;
            size_t dst = ((size_t)h * max_cache + (size_t)(first_pos + t)) * QMO_D;
            norm_rope_head_ref(k + src, k_norm_w, c, s, eps, key_cache + dst);
            memcpy(value_cache + dst, v + src, QMO_D * sizeof(uint16_t));
        }
    }
}

/* ------------------------------------------------------------- attention */

/*
 * One (query head, query row) in "ref" mode: the arithmetic both reference
 * attention kernels share (:15889-16052, :16118-16249).  Keys 0..key_len-1 of
 * kv head `kv_head` in the [kv_heads][max_cache][128] cache.  `scratch` holds
 * key_len bf16 scores.
 */
static void attention_row_ref(const uint16_t* qrow, const uint16_t* key_cache, const uint16_t* value_cache,
                              int kv_head, int max_cache, int key_len, float scale, uint16_t* scratch,
                              uint16_t* out) {
    float qf[QMO_D];
    for (int d = 0; d < QMO_D; ++d) qf[d] = bf16_to_f32(qrow[d]);
    const uint16_t* kbase = key_cache + (size_t)kv_head * max_cache * QMO_D;
    const uint16_t* vbase = value_cache + (size_t)kv_head * max_cache * QMO_D;

    for (int key = 0; key < key_len; ++key) {
        const uint16_t* kr = kbase + (size_t)key * QMO_D;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int d = l; d < QMO_D; d += 32) acc = fmaf(qf[d], bf16_to_f32(kr[d]), acc);
            lane[l] = acc;
        }
        float dot = warp_tree_sum(lane);
        uint16_t raw = f32_to_bf16(dot);
        scratch[key] = f32_to_bf16(bf16_to_f32(raw) * scale);
    }

    float per_thread[256];
    for (int t = 0; t < 256; ++t) {
        float m = -INFINITY;
        for (int key = t; key < key_len; key += 256) {
            float s = bf16_to_f32(scratch[key]);
            m = m > s ? m : s;
        }
        per_thread[t] = m;
    }
    float maximum = block_tree_max(per_thread, 256);

    for (int t = 0; t < 256; ++t) {
        float sum = 0.0f;
        for (int key = t; key < key_len; key += 256) sum += expf(bf16_to_f32(scratch[key]) - maximum);
        per_thread[t] = sum;
    }
    float total = block_tree_sum(per_thread, 256);

    for (int key = 0; key < key_len; ++key) {
        float p = expf(bf16_to_f32(scratch[key]) - maximum) / total;
        scratch[key] = f32_to_bf16(p);
    }

    float acc[QMO_D];
    for (int d = 0; d < QMO_D; ++d) acc[d] = 0.0f;
    for (int key = 0; key < key_len; ++key) {
        float p = bf16_to_f32(scratch[key]);
        const uint16_t* vr = vbase + (size_t)key * QMO_D;
        for (int d = 0; d < QMO_D; ++d) acc[d] = fmaf(p, bf16_to_f32(vr[d]), acc[d]);
    }
    for (int d = 0; d < QMO_D; ++d) out[d] = f32_to_bf16(acc[d]);
}

/* Same row with no intermediate rounding, double accumulation, f32 result. */
static void attention_row_fp32(const uint16_t* qrow, const uint16_t* key_cache, const uint16_t* value_cache,
                               int kv_head, int max_cache, int key_len, float scale, double* scratch,
                               float* out) {
    double qd[QMO_D];
    for (int d = 0; d < QMO_D; ++d) qd[d] = (double)bf16_to_f32(qrow[d]);
    const uint16_t* kbase = key_cache + (size_t)kv_head * max_cache * QMO_D;
    const uint16_t* vbase = value_cache + (size_t)kv_head * max_cache * QMO_D;
    double maximum = -INFINITY;
    for (int key = 0; key < key_len; ++key) {
        const uint16_t* kr = kbase + (size_t)key * QMO_D;
        double dot = 0.0;
        for (int d = 0; d < QMO_D; ++d) dot += qd[d] * (double)bf16_to_f32(kr[d]);
        dot *= (double)scale;
        scratch[key] = dot;
        if (dot > maximum) maximum = dot;
    }
    double total = 0.0;
    for (int key = 0; key < key_len; ++key) {
        scratch[key] = exp(scratch[key] - maximum);
        total += scratch[key];
    }
    double acc[QMO_D];
    for (int d = 0; d < QMO_D; ++d) acc[d] = 0.0;
    for (int key = 0; key < key_len; ++key) {
        double p = scratch[key];
        const uint16_t* vr = vbase + (size_t)key * QMO_D;
        for (int d = 0; d < QMO_D; ++d) acc[d] += p * (double)bf16_to_f32(vr[d]);
    }
    for (int d = 0; d < QMO_D; ++d) out[d] = (float)(acc[d] / total);
}

static float softmax_scale(void) { return 1.0f / sqrtf((float)QMO_D); }

/*
 * Decode attention for a batch of independent streams, each with its own
 * reference-layout cache.  Stream s: query q_rot + s*q_heads*128, caches at
 * key_caches[s] / value_caches[s] with geometry max_caches[s], attends keys
 * 0..key_lens[s]-1 (the just-appended token included, :16080).
 * mode 0: ref -> out_bf16 [streams][q_heads][128]; mode 1: fp32 -> out_f32.
 * Parallel over (stream, kv head), which is also the timed CPU baseline.
 */
QMO_EXPORT int qmo_decode_attention_batch(const uint16_t* q_rot, const uint16_t* const* key_caches,
                                          const uint16_t* const* value_caches, const int32_t* max_caches,
                                          const int32_t* key_lens, int streams, int q_heads, int kv_heads,
                                          int mode, uint16_t* out_bf16, float* out_f32) {
    if (q_heads % kv_heads != 0) return -1;
    const int group = q_heads / kv_heads;
    const float scale = softmax_scale();
    int64_t pairs = (int64_t)streams * kv_heads;
#pragma omp parallel
    {
        int cap = 0;
        void* scratch = NULL;
#pragma omp for schedule(dynamic, 1)
        for (int64_t pair = 0; pair < pairs; ++pair) {
            int s = (int)(pair / kv_heads);
            int h = (int)(pair % kv_heads);
            int len = key_lens[s];
            if (len > cap) {
                free(scratch);
                cap = len;
                scratch = malloc((size_t)cap * sizeof(double));
            }
            for (int g = 0; g < group; ++g) {
                int qh = h * group + g;
                size_t qoff = ((size_t)s * q_heads + qh) * QMO_D;
                if (mode == 0)
                    attention_row_ref(q_rot + qoff, key_caches[s], value_caches[s], h, max_caches[s], len, scale,
                                      (uint16_t*)scratch, out_bf16 + qoff);
                else
                    attention_row_fp32(q_rot + qoff, key_caches[s], value_caches[s], h, max_caches[s], len, scale,
                                       (double*)scratch, out_f32 + qoff);
            }
        }
        free(scratch);
    }
    return 0;
}

/*
 * Causal prefill attention for one sequence of `seq` rows whose keys are
 * already in the cache: row i attends keys 0..cache_before+i (:15832-15852).
 * q_rot / out are [seq][q_heads][128].  Rows [row_begin, row_end) only, so a
 * caller can time or check a sub-sample.  Parallel over (row, head).
 */
QMO_EXPORT int qmo_prefill_attention(const uint16_t* q_rot, const uint16_t* key_cache, const uint16_t* value_cache,
                                     int max_cache, int seq, int cache_before, int q_heads, int kv_heads,
                                     int row_begin, int row_end, int mode, uint16_t* out_bf16, float* out_f32) {
    if (q_heads % kv_heads != 0 || row_begin < 0 || row_end > seq) return -1;
    const int group = q_heads / kv_heads;
    const float scale = softmax_scale();
    int64_t items = (int64_t)(row_end - row_begin) * q_heads;
    int maxlen = cache_before + seq;
#pragma omp parallel
    {
        void* scratch = malloc((size_t)maxlen * sizeof(double));
#pragma omp for schedule(dynamic, 4)
        for (int64_t item = 0; item < items; ++item) {
            int row = row_begin + (int)(item / q_heads);
            int qh = (int)(item % q_heads);
            int len = cache_before + row + 1;
            size_t qoff = ((size_t)row * q_heads + qh) * QMO_D;
            if (mode == 0)
                attention_row_ref(q_rot + qoff, key_cache, value_cache, qh / group, max_cache, len, scale,
                                  (uint16_t*)scratch, out_bf16 + qoff);
            else
                attention_row_fp32(q_rot + qoff, key_cache, value_cache, qh / group, max_cache, len, scale,
                                   (double*)scratch, out_f32 + qoff);
        }
        free(scratch);
    }
    return 0;
}

/* ------------------------------------------------- split-KV partial math */

/*
 * Partial attention state of one query head over keys [key_begin, key_end):
 * m = max scaled score (natural-log domain), l = sum exp(s - m),
 * o[128] = sum exp(s - m) * V (unnormalised).  Double accumulation.  Used to
 * check the sharded long-context path: combining the partials of disjoint
 * key ranges must reproduce full attention.
 */
QMO_EXPORT void qmo_attention_partial(const uint16_t* qrow, const uint16_t* key_cache, const uint16_t* value_cache,
                                      int kv_head, int max_cache, int key_begin, int key_end, float* m_out,
                                      float* l_out, float* o_out) {
    const float scale = softmax_scale();
    const uint16_t* kbase = key_cache + (size_t)kv_head * max_cache * QMO_D;
    const uint16_t* vbase = value_cache + (size_t)kv_head * max_cache * QMO_D;
    int n = key_end - key_begin;
    if (n <= 0) {
        *m_out = -INFINITY;
        *l_out = 0.0f;
        for (int d = 0; d < QMO_D; ++d) o_out[d] = 0.0f;
        return;
    }
    double* sc = (double*)malloc((size_t)n * sizeof(double));
    double maximum = -INFINITY;
    for (int i = 0; i < n; ++i) {
        const uint16_t* kr = kbase + (size_t)(key_begin + i) * QMO_D;
        double dot = 0.0;
        for (int d = 0; d < QMO_D; ++d) dot += (double)bf16_to_f32(qrow[d]) * (double)bf16_to_f32(kr[d]);
        sc[i] = dot * (double)scale;
        if (sc[i] > maximum) maximum = sc[i];
    }
    double acc[QMO_D];
    for (int d = 0; d < QMO_D; ++d) acc[d] = 0.0;
    double total = 0.0;
    for (int i = 0; i < n; ++i) {
        double p = exp(sc[i] - maximum);
        total += p;
        const uint16_t* vr = vbase + (size_t)(key_begin + i) * QMO_D;
        for (int d = 0; d < QMO_D; ++d) acc[d] += p * (double)bf16_to_f32(vr[d]);
    }
    *m_out = (float)maximum;
    *l_out = (float)total;
    for (int d = 0; d < QMO_D; ++d) o_out[d] = (float)acc[d];
    free(sc);
}

/* Log-sum-exp combine of `parts` partial states: M = max m_g,
 * out = sum e^{m_g-M} o_g / sum e^{m_g-M} l_g.  m in natural-log domain. */
QMO_EXPORT void qmo_combine_partials(const float* m, const float* l, const float* o, int parts, float* out) {
    double big = -INFINITY;
    for (int g = 0; g < parts; ++g)
        if ((double)m[g] > big) big = (double)m[g];
    double denom = 0.0;
    double acc[QMO_D];
    for (int d = 0; d < QMO_D; ++d) acc[d] = 0.0;
    for (int g = 0; g < parts; ++g) {
        if (l[g] <= 0.0f) continue;
        double w = exp((double)m[g] - big);
        denom += w * (double)l[g];
        for (int d = 0; d < QMO_D; ++d) acc[d] += w * (double)o[(size_t)g * QMO_D + d];
    }
    for (int d = 0; d < QMO_D; ++d) out[d] = denom > 0.0 ? (float)(acc[d] / denom) : 0.0f;
}

/* ----------------------------------------------------------- paged layout */

/*
 * Gather one stream's keys (or values) out of a paged pool
 * pool[page][kv_heads][page_size][128] through its page-table row into the
 * reference's contiguous [kv_heads][max_cache][128] layout (tokens
 * 0..tokens-1; the rest of `out` is left untouched).
 */
QMO_EXPORT void qmo_gather_paged(const uint16_t* pool, const int32_t* page_row, int tokens, int kv_heads,
                                 int page_size, int max_cache, uint16_t* out) {
    for (int h = 0; h < kv_heads; ++h) {
        for (int t = 0; t < tokens; ++t) {
            int page = page_row[t / page_size];
            int slot = t % page_size;
            const uint16_t* src = pool + (((size_t)page * kv_heads + h) * page_size + slot) * QMO_D;
            memcpy(out + ((size_t)h * max_cache + t) * QMO_D, src, QMO_D * sizeof(uint16_t));
        }
    }
}

/* Inverse of qmo_gather_paged: scatter a contiguous cache into pool pages. */
QMO_EXPORT void qmo_scatter_paged(const uint16_t* cache, const int32_t* page_row, int tokens, int kv_heads,
                                  int page_size, int max_cache, uint16_t* pool) {
    for (int h = 0; h < kv_heads; ++h) {
        for (int t = 0; t < tokens; ++t) {
            int page = page_row[t / page_size];
            int slot = t % page_size;
            uint16_t* dst = pool + (((size_t)page * kv_heads + h) * page_size + slot) * QMO_D;
            memcpy(dst, cache + ((size_t)h * max_cache + t) * QMO_D, QMO_D * sizeof(uint16_t));
        }
    }
}

/* ------------------------------------------------- rest of the talker layer */

/*
 * The non-attention operators of one talker decoder layer, row by row as the
 * reference's M = 1 kernels compute them (the same file as above):
 *   row RMSNorm, any width             rmsnorm_kernel                       :8295-8357
 *   linear (+bias) (+residual)         talker_linear_fused_kernel           :15250-15317
 *                                      talker_qkv_fused_kernel              :15321-15407
 *   residual add + post-norm           talker_add_postnorm_fused_kernel     :16258-16343
 *   gate/up projections + SwiGLU       talker_gate_up_swiglu_fused_kernel   :16348-16416
 * mode 0 keeps the reference's reduction shape (lane k, k+32, ... fmaf chains, shuffle-down tree) and every
 * bf16 materialisation; mode 1 accumulates in double and rounds only what the reference stores.
 */

static float dot_ref(const uint16_t* x, const uint16_t* w, int k_dim) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int k = l; k < k_dim; k += 32) acc = fmaf(bf16_to_f32(x[k]), bf16_to_f32(w[k]), acc);
        lane[l] = acc;
    }
    return warp_tree_sum(lane);
}

static float dot_f64(const uint16_t* x, const uint16_t* w, int k_dim) {
    double acc = 0.0;
    for (int k = 0; k < k_dim; ++k) acc += (double)bf16_to_f32(x[k]) * (double)bf16_to_f32(w[k]);
    return (float)acc;
}

/* out[r][n] = bf16(dot(x[r], w[n]) + bias[n]); with residual: bf16(residual[r][n] + that bf16 value). */
QMO_EXPORT void qmo_linear(const uint16_t* x, const uint16_t* w, const uint16_t* bias, const uint16_t* residual,
                           int rows, int n_dim, int k_dim, int mode, uint16_t* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int n = 0; n < n_dim; ++n) {
            const uint16_t* xr = x + (size_t)r * k_dim;
            const uint16_t* wn = w + (size_t)n * k_dim;
            float acc = mode == 0 ? dot_ref(xr, wn, k_dim) : dot_f64(xr, wn, k_dim);
            if (bias) acc += bf16_to_f32(bias[n]);
            uint16_t v = f32_to_bf16(acc);
            if (residual) v = f32_to_bf16(bf16_to_f32(residual[(size_t)r * n_dim + n]) + bf16_to_f32(v));
            out[(size_t)r * n_dim + n] = v;
        }
    }
}

/* Row RMSNorm of any width with the 256-thread reduction shape of rmsnorm_kernel: thread t accumulates columns
 * t, t+256, ... with fmaf, then the block tree. */
static float sum_squares_block256(const uint16_t* x, int dim, int use_fma) {
    float per_thread[256];
    for (int t = 0; t < 256; ++t) {
        float s = 0.0f;
        for (int c = t; c < dim; c += 256) {
            float v = bf16_to_f32(x[c]);
            s = use_fma ? fmaf(v, v, s) : s + v * v;
        }
        per_thread[t] = s;
    }
    return block_tree_sum(per_thread, 256);
}

QMO_EXPORT void qmo_rmsnorm(const uint16_t* x, const uint16_t* w, float eps, int rows, int dim, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint16_t* xr = x + (size_t)r * dim;
        float sum = sum_squares_block256(xr, dim, 1);
        float inv = 1.0f / sqrtf(sum / (float)dim + eps);
        for (int c = 0; c < dim; ++c) {
            uint16_t nb = f32_to_bf16(bf16_to_f32(xr[c]) * inv);
            out[(size_t)r * dim + c] = f32_to_bf16(bf16_to_f32(nb) * bf16_to_f32(w[c]));
        }
    }
}

/* residual = bf16(hidden + attention); normalized = RMSNorm(residual) (:16258-16343). */
QMO_EXPORT void qmo_add_postnorm(const uint16_t* hidden, const uint16_t* attention, const uint16_t* w, float eps,
                                 int rows, int dim, uint16_t* residual, uint16_t* normalized) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const size_t base = (size_t)r * dim;
        for (int c = 0; c < dim; ++c)
            residual[base + c] = f32_to_bf16(bf16_to_f32(hidden[base + c]) + bf16_to_f32(attention[base + c]));
        float sum = sum_squares_block256(residual + base, dim, 1);
        float inv = 1.0f / sqrtf(sum / (float)dim + eps);
        for (int c = 0; c < dim; ++c) {
            uint16_t nb = f32_to_bf16(bf16_to_f32(residual[base + c]) * inv);
            normalized[base + c] = f32_to_bf16(bf16_to_f32(nb) * bf16_to_f32(w[c]));
        }
    }
}

/* out[r][c] = bf16( bf16(silu(bf16(g))) * bf16(u) ), g = dot(x, gate[c]), u = dot(x, up[c]) (:16348-16416). */
QMO_EXPORT void qmo_gate_up_swiglu(const uint16_t* x, const uint16_t* gate_w, const uint16_t* up_w, int rows,
                                   int hidden, int intermediate, int mode, uint16_t* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < intermediate; ++c) {
            const uint16_t* xr = x + (size_t)r * hidden;
            float g = mode == 0 ? dot_ref(xr, gate_w + (size_t)c * hidden, hidden) : dot_f64(xr, gate_w + (size_t)c * hidden, hidden);
            float u = mode == 0 ? dot_ref(xr, up_w + (size_t)c * hidden, hidden) : dot_f64(xr, up_w + (size_t)c * hidden, hidden);
            float gv = rnd(g);
            float act = rnd(gv / (1.0f + expf(-gv)));
            out[(size_t)r * intermediate + c] = f32_to_bf16(act * rnd(u));
        }
    }
}

/* ---- final head: logits -> next code (:14052-14176, :7546-7600, :7668-7689) ---- */

typedef struct {
    float score;
    int token;
} qmo_candidate;

/* gpu_sampler_better (:7492-7496) as a qsort order: higher score first, lower index among equals. */
static int candidate_order(const void* pa, const void* pb) {
    const qmo_candidate* a = (const qmo_candidate*)pa;
    const qmo_candidate* b = (const qmo_candidate*)pb;
    if (a->score > b->score) return -1;
    if (a->score < b->score) return 1;
    return a->token < b->token ? -1 : (a->token > b->token ? 1 : 0);
}

/* One stream.  `history` holds the codes generated so far, `generation_index` of them.
 *   scores = float(bf16 logits)                                              cast_final_head_logits :14052-14061
 *   flag 1: a token present in the history gets score * 1.05 when negative,
 *           score * 0x3f73cf3e otherwise                                     repetition_penalty :14063-14099
 *   flag 2: EOS is -inf while generation_index < 2; ids from reserved_begin
 *           on, except EOS, are -inf                                         suppress_tokens :14102-14123
 *   top_k <= 0: highest score, lowest index among equals                     argmax_final_head :14126-14176
 *   top_k  > 0: best top_k in (score desc, index asc) order, weights
 *               exp(score / T - best / T) in double, target = u * total with
 *               u one SplitMix64 draw (>> 11, * 2^-53), cumulative walk      gpu_sample_topk_f32_kernel :7546-7600
 *   flag 4: history[generation_index] = code                                 record_sampled_code_kernel :7668-7689
 * Returns the code; `processed` (vocab floats) receives the processed scores when not NULL. */
QMO_EXPORT int qmo_final_head_sample(const uint16_t* logits, int vocab, int32_t* history, int history_capacity,
                                     int generation_index, int flags, int eos_token, int reserved_begin, int top_k,
                                     float temperature, uint64_t* rng_state, float* processed) {
    float* scores = (float*)malloc((size_t)vocab * sizeof(float));
    qmo_candidate* all = (qmo_candidate*)malloc((size_t)vocab * sizeof(qmo_candidate));
    const int count = generation_index < history_capacity ? generation_index : history_capacity;
    union {
        uint32_t u;
        float f;
    } reciprocal = {0x3f73cf3eu};
    for (int token = 0; token < vocab; ++token) {
        float score = bf16_to_f32(logits[token]);
        if (flags & 1) {
            int repeated = 0;
            for (int i = 0; i < count; ++i) {
                if (history[i] == token) {
                    repeated = 1;
                    break;
                }
            }
            if (repeated) score = score < 0.0f ? score * 1.05f : score * reciprocal.f;
        }
        if (flags & 2) {
            if (token == eos_token && generation_index < 2) score = -INFINITY;
            if (token >= reserved_begin && token != eos_token) score = -INFINITY;
        }
        scores[token] = score;
        if (processed) processed[token] = score;
    }
    int code = 0;
    if (top_k <= 0) {
        float best = -INFINITY;
        for (int token = 0; token < vocab; ++token) {
            if (scores[token] > best) {      /* ascending scan: the first of equal scores stays */
                best = scores[token];
                code = token;
            }
        }
    } else {
        for (int token = 0; token < vocab; ++token) {
            all[token].score = scores[token];
            all[token].token = token;
        }
        qsort(all, (size_t)vocab, sizeof(qmo_candidate), candidate_order);
        const int keep = top_k < vocab ? top_k : vocab;
        const double inv_t = 1.0 / (double)temperature;
        const double maximum = (double)all[0].score * inv_t;
        double total = 0.0;
        for (int i = 0; i < keep; ++i) total += exp((double)all[i].score * inv_t - maximum);
        code = all[0].token;
        if (total > 0.0) {
            uint64_t z = *rng_state + 0x9e3779b97f4a7c15ULL;
            *rng_state = z;
            z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
            z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
            z ^= z >> 31;
            const double target = (double)(z >> 11) * (1.0 / 9007199254740992.0) * total;
            double cumulative = 0.0;
            code = all[keep - 1].token;
            for (int i = 0; i < keep; ++i) {
                cumulative += exp((double)all[i].score * inv_t - maximum);
                if (target < cumulative) {
                    code = all[i].token;
                    break;
                }
            }
        }
    }
    if ((flags & 4) && generation_index >= 0 && generation_index < history_capacity) history[generation_index] = code;
    free(scores);
    free(all);
    return code;
}
