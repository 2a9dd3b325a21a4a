// Split-KV flash decoding over the paged bf16 KV cache (GQA group of 2), plus
// the log-sum-exp combine kernels.
//
// Stands in for talker_attention_gqa2_m1_locality_kernel (17.cu:16061-16251,
// dispatch :17916-17952): one new query token per stream, both query heads that
// share a KV head are served by the same K/V read.  Where the reference runs 8
// CTAs and materialises bf16 scores in shared memory, this kernel
//
//   * flattens the work into units, one unit = one (stream, kv head, page)
//     tile pair (K tile + V tile, 16 KB each, contiguous in the pool), ordered
//     stream-major, then kv head, then page;
//   * gives each of G = 2 x SM-count CTAs an equal contiguous run of units
//     (ragged lengths balance to within one tile);
//   * streams the tiles through a 3-stage shared-memory ring with 1-D bulk
//     copies (cp.async.bulk + mbarrier complete_tx) issued by a producer warp,
//     while 8 consumer warps keep an fp32 online softmax per run of units that
//     belong to the same (stream, kv head) segment;
//   * writes a segment's result directly when one CTA saw all of it, else an
//     (m, l, o) partial into slot (cta + segment) of the workspace - that map
//     is injective over the (cta, segment) pairs that occur because both
//     indices only grow along the unit order.  Each CTA then bumps the
//     segment's arrival counter; the CTA that arrives last folds all partials
//     of the segment in CTA order (so the result does not depend on which CTA
//     that is) and sets the counter back to zero for the next call.
//
// Scores live in the log2 domain (q is pre-multiplied by scale * log2 e).
#include <math_constants.h>

#include <cstdlib>
#include <mutex>

#include "qm_exchange_layout.cuh"
#include "qm_norm_rope.cuh"

namespace {

constexpr int kStages = 3;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps;          // issues every bulk copy
constexpr int kPrepWarp = kConsumerWarps + 1;          // fused step: QK-RMSNorm + RoPE of the staged rows
constexpr int kDecodeThreads = kConsumerThreads + 64;
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kMaxBatchPerLaunch = 256;        // one stream per thread in the prologue
static_assert(kMaxBatchPerLaunch <= kDecodeThreads, "the prologue handles one stream per thread");
constexpr int kMaxGrid = 1024;
constexpr int kPartialStride = kHeadDim + 2;   // m, l, o[128]
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeArgs {
    const uint16_t* q_rot;       // normed + roped queries; in the fused step: the raw q projections
    uint16_t* key_pool;
    uint16_t* value_pool;
    const int32_t* seq_lens;     // keys to attend; in the fused step: positions (keys = position + 1)
    // fused step only: raw k / v projections of the new token, norm weights, RoPE table
    const uint16_t* raw_k;
    const uint16_t* raw_v;
    const uint16_t* q_norm_weight;
    const uint16_t* k_norm_weight;
    const uint16_t* rope_cos;
    const uint16_t* rope_sin;
    int rope_rows;
    int len_offset;              // 0, or 1 in the fused step
    float epsilon;
    const int32_t* page_table;
    uint16_t* out;           // mode 0
    float* partial_out;      // mode 1: [batch][q_heads][130]
    float* ws_partials;      // [(grid + segments)][2][130]
    int32_t* ws_count;       // [segments] arrival counters, zero between calls
    uint32_t* status;
    int batch;
    int kv_heads;
    int max_pages;
    int num_pages;
    int mode;                // 0: bf16 context; 1: partial state of this pool's keys; 2: partial state exchanged with
                             //    the other ranks' and folded here (keys split across GPUs), bf16 context
    int prefetch_units;      // units per CTA whose tiles are prefetched into L2 before the dependency wait
    ExchangeView exchange;   // mode 2: every rank's exchange buffer
};

struct SharedLayout {
    static constexpr int kPrefixOff = kStages * kStageBytes;                       // int32[kMaxBatch+1]
    static constexpr int kLenOff = kPrefixOff + ((kMaxBatchPerLaunch + 1) * 4 + 15) / 16 * 16;   // int32[kMaxBatch]: keys per stream
    static constexpr int kScoreOff = kLenOff + kMaxBatchPerLaunch * 4;
    static constexpr int kMergeOff = kScoreOff + 2 * 2 * kPageTokens * 4;          // float[2][2][64]
    static constexpr int kMergeLOff = kMergeOff + kConsumerWarps * 2 * kHeadDim * 4;
    // per stage: q rows of the two heads (512 B); fused step also cos, sin, raw k, raw v rows (256 B each)
    static constexpr int kStagingBytes = 1536;
    static constexpr int kQOff = kMergeLOff + kConsumerWarps * 2 * 4;
    static constexpr int kMetaOff = kQOff + kStages * kStagingBytes;
    static constexpr int kBarOff = kMetaOff + kStages * 32;
    static constexpr int kFlagOff = kBarOff + 3 * kStages * 8;
    static constexpr int kExchangeOff = kFlagOff + 16;           // uint32[2][2]: per query head, for the fused exchange
    static constexpr int kPeerOff = kExchangeOff + 16;           // the ranks' exchange buffer pointers (mode 2)
    static constexpr int kTotal = kPeerOff + kExchangeMaxWorld * 8;
};

__device__ __forceinline__ int clamp_len(int len, int max_pages, uint32_t* status) {
    if (len < 0) len = 0;
    const int cap = max_pages * kPageTokens;
    if (len > cap) {
        atomicOr(status, QM_DEVSTAT_BAD_POS);
        len = cap;
    }
    return len;
}

template <bool kFused, bool kExchange = false>
__global__ void __launch_bounds__(kDecodeThreads, 2) qm_decode_splitkv_kernel(const DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    int32_t* prefix = reinterpret_cast<int32_t*>(smem + SharedLayout::kPrefixOff);
    int32_t* stream_len = reinterpret_cast<int32_t*>(smem + SharedLayout::kLenOff);
    float* score = reinterpret_cast<float*>(smem + SharedLayout::kScoreOff);
    float* merge_o = reinterpret_cast<float*>(smem + SharedLayout::kMergeOff);
    float* merge_l = reinterpret_cast<float*>(smem + SharedLayout::kMergeLOff);
    int4* meta = reinterpret_cast<int4*>(smem + SharedLayout::kMetaOff);      // two int4 per stage
    volatile int* fold_flag = reinterpret_cast<volatile int*>(smem + SharedLayout::kFlagOff);
    const uint32_t bar_base = smem_addr(smem + SharedLayout::kBarOff);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto staged_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int hkv = a.kv_heads;

    pdl_trigger();
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), kFused ? 2 : 1);       // producer (+ bytes) and, in the fused step, the prep warp
            mbar_init(empty_bar(s), kConsumerWarps);
            mbar_init(staged_bar(s), 1);
        }
        fence_mbar_init();
    }
    // Every stage's unit description starts out as a harmless one (segment 0, page 0, no valid keys): a consumer
    // whose bounded wait gave up reads whatever is there, and these values index shared and global memory.
    if (tid < 2 * kStages) meta[tid] = (tid & 1) ? make_int4(0, 0, 0, 0) : make_int4(0, 0, 1, 0);
    // ---- Work done before the dependency wait, and kept if it turns out to be right.
    // A CTA of this launch becomes resident as soon as a CTA of the previous kernel retires, often many
    // microseconds before the last one does, and would otherwise sit idle in the wait below while HBM runs dry.
    // It therefore works out the unit partition and the page ids of its first units from whatever seq_lens and
    // the page table hold right now, and asks the L2 to fetch the K and V tiles of its first units.  These values
    // may be stale when the previous kernel is the one that writes them, so after the wait every length is read
    // again and compared (one L2 round trip instead of the whole partition pipeline); the page ids are read
    // again in any case.  Only if a length changed is the partition rebuilt.  A wrong guess costs a useless
    // prefetch and nothing else.
    const int cap_len = a.max_pages * kPageTokens;
    auto units_of = [&](int len) { return ((len + kPageTokens - 1) >> 6) * hkv; };
    // prefix[s + 1] holds the units of stream s on entry; on exit prefix[s] = first unit of stream s
    auto scan_prefix = [&]() {
        __syncthreads();
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < a.batch; base += 32) {
                const int idx = base + lane;
                int v = idx < a.batch ? prefix[idx + 1] : 0;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, v, off);
                    if (lane >= off) v += t;
                }
                v += carry;
                if (idx < a.batch) prefix[idx + 1] = v;
                carry = __shfl_sync(0xffffffffu, v, 31);
            }
        }
        __syncthreads();
    };
    // One unit's coordinates from the partition in shared memory (no global access).
    struct UnitMeta {
        int seg, page_idx, pages, nvalid, head, len;
        long long table_index;       // page_table entry of the unit's page
    };
    auto locate = [&](int u) {
        int lo = 0, hi = a.batch;       // largest s with prefix[s] <= u and units in s
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= u) lo = mid; else hi = mid;
        }
        UnitMeta um;
        const int r = u - prefix[lo];
        um.pages = (prefix[lo + 1] - prefix[lo]) / hkv;
        um.head = um.pages > 0 ? r / um.pages : 0;
        um.page_idx = r - um.head * um.pages;
        um.seg = lo * hkv + um.head;
        um.len = stream_len[lo];
        const int left = um.len - um.page_idx * kPageTokens;
        um.nvalid = left < kPageTokens ? left : kPageTokens;
        um.table_index = (long long)lo * a.max_pages + um.page_idx;
        return um;
    };

    const bool speculate = a.prefetch_units > 0;
    UnitMeta first_units{};                      // producer warp: lane l holds this CTA's unit l (speculated)
    bool first_units_known = false;
    if (speculate) {
        if (tid < a.batch) {
            int len = a.seq_lens[tid] + a.len_offset;
            len = len < 0 ? 0 : (len > cap_len ? cap_len : len);
            stream_len[tid] = len;
            prefix[tid + 1] = units_of(len);
        }
        if (tid == 0) prefix[0] = 0;
        scan_prefix();
        if (warp == kProducerWarp) {
            const long long total = prefix[a.batch];
            const long long geff = total < (long long)gridDim.x ? total : (long long)gridDim.x;
            if ((long long)blockIdx.x < geff) {
                const long long ub = (long long)blockIdx.x * total / geff;
                const long long ue = (long long)(blockIdx.x + 1) * total / geff;
                first_units_known = true;
                // About a fourteenth of the CTA's share is asked for ahead of the wait, at most prefetch_units tiles:
                // while the kernel in front still runs, these requests compete with its own traffic, and what a
                // short share gains at its head it would lose there (measured: 4 tiles for shares of 59 units, 2 for
                // shares of 28 inside a decoder step, where the kernel in front streams weights).
                int depth = (int)(ue - ub) / 14;
                depth = depth < 1 ? 1 : (depth > a.prefetch_units ? a.prefetch_units : depth);
                if (ub + lane < ue) {
                    first_units = locate((int)(ub + lane));
                    if (lane < depth && first_units.nvalid > 0) {
                        int page_id = a.page_table[first_units.table_index];
                        page_id = page_id < 0 ? 0 : (page_id >= a.num_pages ? a.num_pages - 1 : page_id);
                        const size_t tile = ((size_t)page_id * hkv + first_units.head) * kTileElems;
                        const uint32_t bytes = (uint32_t)first_units.nvalid * (kHeadDim * 2);
                        const uint64_t keep = l2_policy_evict_last();
                        bulk_prefetch_l2_hint(a.key_pool + tile, bytes, keep);
                        bulk_prefetch_l2_hint(a.value_pool + tile, bytes, keep);
                    }
                }
            }
        }
    }
    pdl_wait();      // everything below reads what earlier kernels on the stream wrote

    // The lengths as they are now (one per thread: a launch takes at most kMaxBatchPerLaunch <= blockDim streams).
    int my_len = 0;
    bool changed = !speculate;
    if (tid < a.batch) {
        my_len = clamp_len(a.seq_lens[tid] + a.len_offset, a.max_pages, a.status);
        if (speculate && my_len != stream_len[tid]) changed = true;
    }
    changed = __syncthreads_or(changed ? 1 : 0) != 0;
    if (changed) {
        if (tid < a.batch) {
            stream_len[tid] = my_len;
            prefix[tid + 1] = units_of(my_len);
        }
        if (tid == 0) prefix[0] = 0;
        scan_prefix();
        first_units_known = false;
    }

    // Streams with nothing to attend get a zero row (mode 0) or an empty partial (mode 1); in mode 2 the empty
    // partial takes part in the exchange like any other (the other ranks wait for this rank's copy of every row).
    volatile uint32_t* exchange_words = reinterpret_cast<volatile uint32_t*>(smem + SharedLayout::kExchangeOff);
    ExchangeView xview = a.exchange;
    if (kExchange) {
        xview = exchange_cache_peers(a.exchange, reinterpret_cast<unsigned char**>(smem + SharedLayout::kPeerOff), tid);
        __syncthreads();
    }
    for (int s = blockIdx.x; s < a.batch; s += gridDim.x) {
        if (prefix[s + 1] != prefix[s]) continue;
        if (kExchange) {
            if (tid < kHeadDim) {        // warps 0-3, one row after the other
                for (int h = 0; h < 2 * hkv; ++h) {
                    const int row = s * (2 * hkv) + h;
                    exchange_row(xview, row, tid, -CUDART_INF_F, 0.0f, 0.0f, true, a.out + (size_t)row * kHeadDim, a.status,
                                 exchange_words, [] { named_bar_sync(2, kHeadDim); });
                }
            }
            continue;
        }
        for (int i = tid; i < 2 * hkv * kHeadDim; i += kDecodeThreads) {
            const size_t row = (size_t)s * (2 * hkv) + i / kHeadDim;
            const int d = i % kHeadDim;
            if (a.mode == 0) {
                a.out[row * kHeadDim + d] = 0;
            } else {
                float* dst = a.partial_out + row * kPartialStride;
                dst[2 + d] = 0.0f;
                if (d == 0) {
                    dst[0] = -CUDART_INF_F;
                    dst[1] = 0.0f;
                }
            }
        }
    }

    const long long total_units = prefix[a.batch];
    const long long grid_eff = total_units < (long long)gridDim.x ? total_units : (long long)gridDim.x;
    const int cta = blockIdx.x;
    if (cta >= grid_eff) return;
    const long long unit_begin = (long long)cta * total_units / grid_eff;
    const long long unit_end = (long long)(cta + 1) * total_units / grid_eff;
    const int count = (int)(unit_end - unit_begin);

    bool dead = false;

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ producer
        const uint64_t stream_once = l2_policy_evict_first();     // a KV tile is read once per step
        for (int base = 0; base < count; base += 32) {
            int seg_l = 0, page_idx_l = 0, pages_l = 1, page_id_l = 0, nvalid_l = 0, head_l = 0, len_l = 0;
            if (base + lane < count) {
                // the first 32 units were located before the wait; only their page ids are read again
                const UnitMeta um = (base == 0 && first_units_known) ? first_units : locate((int)(unit_begin + base + lane));
                seg_l = um.seg;
                page_idx_l = um.page_idx;
                pages_l = um.pages;
                nvalid_l = um.nvalid;
                head_l = um.head;
                len_l = um.len;
                page_id_l = a.page_table[um.table_index];
                if (page_id_l < 0 || page_id_l >= a.num_pages) {
                    atomicOr(a.status, QM_DEVSTAT_BAD_PAGE);
                    page_id_l = 0;
                }
            }
            const int batch_units = count - base < 32 ? count - base : 32;
            for (int j = 0; j < batch_units; ++j) {
                const int seg = __shfl_sync(0xffffffffu, seg_l, j);
                const int page_idx = __shfl_sync(0xffffffffu, page_idx_l, j);
                const int pages = __shfl_sync(0xffffffffu, pages_l, j);
                const int page_id = __shfl_sync(0xffffffffu, page_id_l, j);
                const int nvalid = __shfl_sync(0xffffffffu, nvalid_l, j);
                const int head = __shfl_sync(0xffffffffu, head_l, j);
                const int len = __shfl_sync(0xffffffffu, len_l, j);
                if (lane == 0) {
                    const int n = base + j;
                    const int stage = n % kStages;
                    const uint32_t parity = ((n / kStages) & 1) ^ 1;
                    if (!mbar_wait_bounded(empty_bar(stage), parity, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                    meta[2 * stage] = make_int4(seg, page_idx, pages, nvalid);
                    meta[2 * stage + 1] = make_int4(page_id, 0, 0, 0);
                    const size_t tile = ((size_t)page_id * hkv + head) * kTileElems;
                    const uint32_t dst = smem_addr(smem + stage * kStageBytes);
                    const uint32_t staging = smem_addr(smem + SharedLayout::kQOff + stage * SharedLayout::kStagingBytes);
                    const bool new_segment = n == 0 || page_idx == 0;
                    constexpr uint32_t kQBytes = 2 * kHeadDim * 2;         // the two query heads of this KV head
                    constexpr uint32_t kRowBytes = kHeadDim * 2;
                    if (!kFused) {
                        const uint32_t bytes = (uint32_t)nvalid * kRowBytes;
                        mbar_arrive_expect_tx(full_bar(stage), 2 * bytes + (new_segment ? kQBytes : 0u));
                        if (new_segment) bulk_copy_g2s(staging, a.q_rot + (size_t)seg * 2 * kHeadDim, kQBytes, full_bar(stage));
                        bulk_copy_g2s_hint(dst, a.key_pool + tile, bytes, full_bar(stage), stream_once);
                        bulk_copy_g2s_hint(dst + kTileBytes, a.value_pool + tile, bytes, full_bar(stage), stream_once);
                    } else {
                        // The last page of a segment ends with the new token, which is not in the pool yet: its
                        // row is built by the consumers from the raw k / v rows staged here.
                        const bool last_page = page_idx == pages - 1;
                        const uint32_t bytes = (uint32_t)(last_page ? nvalid - 1 : nvalid) * kRowBytes;
                        int position = len - 1;            // fused step: keys = position + 1 (a clamped length is reported)
                        if (position < 0 || position >= a.rope_rows) {
                            atomicOr(a.status, QM_DEVSTAT_BAD_POS);
                            position = position < 0 ? 0 : a.rope_rows - 1;
                        }
                        const bool needs_rope = new_segment || last_page;
                        // small rows first, on their own barrier: the prep warp works on them while the tile lands
                        mbar_arrive_expect_tx(staged_bar(stage), (new_segment ? kQBytes : 0u) + (needs_rope ? 2 * kRowBytes : 0u) +
                                                                     (last_page ? 2 * kRowBytes : 0u));
                        if (new_segment) bulk_copy_g2s(staging, a.q_rot + (size_t)seg * 2 * kHeadDim, kQBytes, staged_bar(stage));
                        if (needs_rope) {
                            bulk_copy_g2s(staging + 512, a.rope_cos + (size_t)position * kHeadDim, kRowBytes, staged_bar(stage));
                            bulk_copy_g2s(staging + 768, a.rope_sin + (size_t)position * kHeadDim, kRowBytes, staged_bar(stage));
                        }
                        if (last_page) {
                            bulk_copy_g2s(staging + 1024, a.raw_k + (size_t)seg * kHeadDim, kRowBytes, staged_bar(stage));
                            bulk_copy_g2s(staging + 1280, a.raw_v + (size_t)seg * kHeadDim, kRowBytes, staged_bar(stage));
                        }
                        mbar_arrive_expect_tx(full_bar(stage), 2 * bytes);
                        if (bytes) {
                            bulk_copy_g2s_hint(dst, a.key_pool + tile, bytes, full_bar(stage), stream_once);
                            bulk_copy_g2s_hint(dst + kTileBytes, a.value_pool + tile, bytes, full_bar(stage), stream_once);
                        }
                    }
                }
                __syncwarp();
            }
        }
        // The consumers wait for every tile before they finish, so no copy is in
        // flight when the CTA retires unless a wait gave up; in that case wait
        // (bounded again) for the last copies issued.
        if (lane == 0 && dead) {
            bool ignore = false;
            const int first = count > kStages ? count - kStages : 0;
            for (int n = first; n < count; ++n) mbar_wait_bounded(full_bar(n % kStages), (n / kStages) & 1, ignore);
        }
        return;
    }

    if (warp == kPrepWarp) {
        // ------------------------------------------------- fused step: norm + RoPE of the staged rows
        // For every unit: wait for the producer's small rows, turn the raw q rows into q_rot in place (new
        // segment), build the new token's K row (normed, roped) and copy its V row into the shared-memory tile
        // and into the pool (last page of a segment), then arrive on the unit's full barrier.  The consumers
        // find everything in place when that barrier completes.
        if (kFused) {
            const uint2 wq = *reinterpret_cast<const uint2*>(a.q_norm_weight + 4 * lane);
            const uint2 wk = *reinterpret_cast<const uint2*>(a.k_norm_weight + 4 * lane);
            for (int n = 0; n < count; ++n) {
                const int stage = n % kStages;
                if (!mbar_wait_bounded(staged_bar(stage), (n / kStages) & 1, dead) && lane == 0)
                    atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                const int4 mt = meta[2 * stage];
                const int seg = mt.x, page_idx = mt.y, pages = mt.z, nvalid = mt.w;
                const int head = seg % hkv;
                const bool new_segment = n == 0 || page_idx == 0;
                const bool last_page = page_idx == pages - 1;
                unsigned char* staging = smem + SharedLayout::kQOff + stage * SharedLayout::kStagingBytes;
                if (new_segment || last_page) {
                    const uint2 craw = *reinterpret_cast<const uint2*>(staging + 512 + lane * 8);
                    const uint2 sraw = *reinterpret_cast<const uint2*>(staging + 768 + lane * 8);
                    if (new_segment) {
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2) {
                            uint2* row = reinterpret_cast<uint2*>(staging + h2 * 256 + lane * 8);
                            *row = norm_rope_row(*row, wq, craw, sraw, lane, a.epsilon);
                        }
                    }
                    if (last_page && nvalid > 0 && !dead) {      // after a wait that gave up nothing here is trustworthy: no stores
                        const uint2 krow = norm_rope_row(*reinterpret_cast<const uint2*>(staging + 1024 + lane * 8), wk, craw, sraw,
                                                         lane, a.epsilon);
                        const uint2 vrow = *reinterpret_cast<const uint2*>(staging + 1280 + lane * 8);
                        const size_t elem = (((size_t)meta[2 * stage + 1].x * hkv + head) * kPageTokens + (nvalid - 1)) * kHeadDim + 4 * lane;
                        unsigned char* tile_row = smem + stage * kStageBytes + (nvalid - 1) * (kHeadDim * 2) + lane * 8;
                        *reinterpret_cast<uint2*>(tile_row) = krow;
                        *reinterpret_cast<uint2*>(tile_row + kTileBytes) = vrow;
                        *reinterpret_cast<uint2*>(a.key_pool + elem) = krow;
                        *reinterpret_cast<uint2*>(a.value_pool + elem) = vrow;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(stage));
            }
        }
        return;
    }

    // --------------------------------------------------------------- consumers
    const int half = lane >> 4;
    const int lp = lane & 15;
    float2 q0[4], q1[4], o0[4], o1[4];          // dims 8*lp .. 8*lp+7 as (even, odd) pairs
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;
    bool seg_from_start = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) q0[j] = q1[j] = o0[j] = o1[j] = make_float2(0.0f, 0.0f);

    for (int n = 0; n < count; ++n) {
        const int stage = n % kStages;
        if (!mbar_wait_bounded(full_bar(stage), (n / kStages) & 1, dead) && lane == 0)
            atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
        const int4 mt = meta[2 * stage];
        const int seg = mt.x, page_idx = mt.y, pages = mt.z, nvalid = mt.w;
        unsigned char* staging = smem + SharedLayout::kQOff + stage * SharedLayout::kStagingBytes;
        const int stream = seg / hkv;
        const int head = seg - stream * hkv;

        if (n == 0 || page_idx == 0) {
            // New segment: fetch the two query heads of this KV head (q_rot rows 2*head, 2*head+1 of this
            // stream, staged beside the tile by the producer).
            const float qscale = kLog2e / sqrtf((float)kHeadDim);
            const float2 qs2 = make_float2(qscale, qscale);
            const unsigned char* qp = staging + lp * 16;
            const uint4 qa = *reinterpret_cast<const uint4*>(qp);
            const uint4 qb = *reinterpret_cast<const uint4*>(qp + kHeadDim * 2);
            q0[0] = fmul2(bf16x2_to_float2(qa.x), qs2); q0[1] = fmul2(bf16x2_to_float2(qa.y), qs2);
            q0[2] = fmul2(bf16x2_to_float2(qa.z), qs2); q0[3] = fmul2(bf16x2_to_float2(qa.w), qs2);
            q1[0] = fmul2(bf16x2_to_float2(qb.x), qs2); q1[1] = fmul2(bf16x2_to_float2(qb.y), qs2);
            q1[2] = fmul2(bf16x2_to_float2(qb.z), qs2); q1[3] = fmul2(bf16x2_to_float2(qb.w), qs2);
#pragma unroll
            for (int j = 0; j < 4; ++j) o0[j] = o1[j] = make_float2(0.0f, 0.0f);
            m0 = m1 = -CUDART_INF_F;
            l0 = l1 = 0.0f;
            seg_from_start = page_idx == 0;
        }

        const unsigned char* ktile = smem + stage * kStageBytes;
        const unsigned char* vtile = ktile + kTileBytes;
        float* sc = score + (n & 1) * (2 * kPageTokens);

        // ---- scores: 8 keys per warp, half-warp per key row
        float acc[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = 8 * warp + 2 * i + half;
            const uint4 kk = *reinterpret_cast<const uint4*>(ktile + key * (kHeadDim * 2) + lp * 16);
            const float2 kf[4] = {bf16x2_to_float2(kk.x), bf16x2_to_float2(kk.y), bf16x2_to_float2(kk.z),
                                  bf16x2_to_float2(kk.w)};
            float2 d0 = make_float2(0.0f, 0.0f), d1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                d0 = ffma2(q0[j], kf[j], d0);
                d1 = ffma2(q1[j], kf[j], d1);
            }
            acc[2 * i] = d0.x + d0.y;
            acc[2 * i + 1] = d1.x + d1.y;
        }
        {
            // Reduce-scatter over the 16 lanes of a half-warp: 8 values -> lane
            // lp ends with value index lp >> 1 (duplicated in the odd lane).
            float r[4], r2[2];
            const bool b3 = (lp & 8) != 0, b2 = (lp & 4) != 0, b1 = (lp & 2) != 0;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float mine = b3 ? acc[4 + t] : acc[t];
                const float theirs = b3 ? acc[t] : acc[4 + t];
                r[t] = mine + __shfl_xor_sync(0xffffffffu, theirs, 8);
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const float mine = b2 ? r[2 + t] : r[t];
                const float theirs = b2 ? r[t] : r[2 + t];
                r2[t] = mine + __shfl_xor_sync(0xffffffffu, theirs, 4);
            }
            const float mine = b1 ? r2[1] : r2[0];
            const float theirs = b1 ? r2[0] : r2[1];
            float r3 = mine + __shfl_xor_sync(0xffffffffu, theirs, 2);
            r3 += __shfl_xor_sync(0xffffffffu, r3, 1);
            const int idx = lp >> 1;
            const int key = 8 * warp + 2 * (idx >> 1) + half;
            if ((lp & 1) == 0) sc[(idx & 1) * kPageTokens + key] = key < nvalid ? r3 : -CUDART_INF_F;
        }
        named_bar_sync(1, kConsumerThreads);

        // ---- online softmax over the 64 keys of the tile (same in every warp)
        float x0 = fmaxf(sc[lane], sc[lane + 32]);
        float x1 = fmaxf(sc[kPageTokens + lane], sc[kPageTokens + lane + 32]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, off));
            x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, off));
        }
        const float mn0 = fmaxf(m0, x0), mn1 = fmaxf(m1, x1);
        if (mn0 != m0 || mn1 != m1) {
            const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
            const float2 c02 = make_float2(c0, c0), c12 = make_float2(c1, c1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o0[j] = fmul2(o0[j], c02);
                o1[j] = fmul2(o1[j], c12);
            }
            l0 *= c0;
            l1 *= c1;
            m0 = mn0;
            m1 = mn1;
        }

        // ---- P V for this warp's 8 keys
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = 8 * warp + 2 * i + half;
            if (key < nvalid) {
                const float p0 = fast_exp2(sc[key] - m0);
                const float p1 = fast_exp2(sc[kPageTokens + key] - m1);
                l0 += p0;
                l1 += p1;
                const uint4 vv = *reinterpret_cast<const uint4*>(vtile + key * (kHeadDim * 2) + lp * 16);
                const float2 vf[4] = {bf16x2_to_float2(vv.x), bf16x2_to_float2(vv.y), bf16x2_to_float2(vv.z),
                                      bf16x2_to_float2(vv.w)};
                const float2 p02 = make_float2(p0, p0), p12 = make_float2(p1, p1);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    o0[j] = ffma2(p02, vf[j], o0[j]);
                    o1[j] = ffma2(p12, vf[j], o1[j]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));

        // ---- end of this CTA's share of the segment
        if (n == count - 1 || page_idx == pages - 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o0[j].x += __shfl_xor_sync(0xffffffffu, o0[j].x, 16);
                o0[j].y += __shfl_xor_sync(0xffffffffu, o0[j].y, 16);
                o1[j].x += __shfl_xor_sync(0xffffffffu, o1[j].x, 16);
                o1[j].y += __shfl_xor_sync(0xffffffffu, o1[j].y, 16);
            }
            l0 += __shfl_xor_sync(0xffffffffu, l0, 16);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 16);
            if (half == 0) {
                float* dst0 = merge_o + (warp * 2 + 0) * kHeadDim + 8 * lp;
                float* dst1 = merge_o + (warp * 2 + 1) * kHeadDim + 8 * lp;
                *reinterpret_cast<float4*>(dst0) = make_float4(o0[0].x, o0[0].y, o0[1].x, o0[1].y);
                *reinterpret_cast<float4*>(dst0 + 4) = make_float4(o0[2].x, o0[2].y, o0[3].x, o0[3].y);
                *reinterpret_cast<float4*>(dst1) = make_float4(o1[0].x, o1[0].y, o1[1].x, o1[1].y);
                *reinterpret_cast<float4*>(dst1 + 4) = make_float4(o1[2].x, o1[2].y, o1[3].x, o1[3].y);
            }
            if (lane == 0) {
                merge_l[warp * 2 + 0] = l0;
                merge_l[warp * 2 + 1] = l1;
            }
            named_bar_sync(1, kConsumerThreads);
            {
                const int qh = tid >> 7;           // which of the two query heads
                const int d = tid & 127;
                float sum = 0.0f, lsum = 0.0f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    sum += merge_o[(w * 2 + qh) * kHeadDim + d];
                    lsum += merge_l[w * 2 + qh];
                }
                const float m = qh ? m1 : m0;
                const bool whole = seg_from_start && page_idx == pages - 1;
                const size_t row = (size_t)stream * (2 * hkv) + 2 * head + qh;
                // `dead`: one of this thread's waits gave up (QM_DEVSTAT_TIMEOUT is set).  Its numbers are garbage
                // and the unit description may be a stale one, so it writes nothing to global memory and takes
                // no part in the arrival count; the barriers below are still passed by everyone.
                if (whole) {
                    if (kExchange) {
                        // this CTA saw all of this rank's keys of the segment: its state is the rank's partial
                        exchange_row(xview, (int)row, d, m * kLn2, lsum, sum, !dead, a.out + row * kHeadDim, a.status,
                                     exchange_words + 2 * qh, [qh] { if (qh) named_bar_sync(3, kHeadDim); else named_bar_sync(2, kHeadDim); });
                    } else if (dead) {
                    } else if (a.mode == 0) {
                        a.out[row * kHeadDim + d] = (uint16_t)f32_to_bf16_bits(sum / lsum);
                    } else {
                        float* dst = a.partial_out + row * kPartialStride;
                        dst[2 + d] = sum;
                        if (d == 0) {
                            dst[0] = m * kLn2;
                            dst[1] = lsum;
                        }
                    }
                } else {
                    float* dst = a.ws_partials + ((size_t)(cta + seg) * 2 + qh) * kPartialStride;
                    if (!dead) {
                        dst[2 + d] = sum;
                        if (d == 0) {
                            dst[0] = m;
                            dst[1] = lsum;
                        }
                    }
                    // Which CTAs hold a part of this segment (unit u belongs to CTA ((u + 1) * G - 1) / U).
                    const long long u_first = (long long)prefix[stream] + (long long)head * pages;
                    const int c_first = (int)(((u_first + 1) * grid_eff - 1) / total_units);
                    const int c_last = (int)(((u_first + pages) * grid_eff - 1) / total_units);
                    __threadfence();
                    named_bar_sync(1, kConsumerThreads);
                    if (tid == 0) {
                        int is_last = 0;
                        if (!dead) {
                            const int arrived = atomicAdd(a.ws_count + seg, 1) + 1;
                            is_last = arrived == c_last - c_first + 1;
                            if (is_last) a.ws_count[seg] = 0;          // everyone else is done with it
                        }
                        *fold_flag = is_last;
                    }
                    named_bar_sync(1, kConsumerThreads);
                    if (*fold_flag && (kExchange || !dead)) {
                        __threadfence();
                        // Piece i of the segment sits in slot (c_first + i + seg).  The loads of a batch are issued
                        // together (a rolled loop would pay one L2 round trip per piece, twice); the arithmetic stays
                        // in piece order.
                        const int pieces = c_last - c_first + 1;
                        const float* first = a.ws_partials + ((size_t)(c_first + seg) * 2 + qh) * kPartialStride;
                        constexpr size_t kNext = 2 * kPartialStride;
                        float big = -CUDART_INF_F;
                        for (int i0 = 0; i0 < pieces && !dead; i0 += 8) {
                            float mv[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) mv[j] = i0 + j < pieces ? __ldcg(first + (size_t)(i0 + j) * kNext) : -CUDART_INF_F;
#pragma unroll
                            for (int j = 0; j < 8; ++j) big = fmaxf(big, mv[j]);
                        }
                        float acc = 0.0f, denom = 0.0f;
                        for (int i0 = 0; i0 < pieces && !dead; i0 += 4) {
                            float mv[4], lv[4], ov[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float* src = first + (size_t)(i0 + j < pieces ? i0 + j : pieces - 1) * kNext;
                                mv[j] = __ldcg(src);
                                lv[j] = __ldcg(src + 1);
                                ov[j] = __ldcg(src + 2 + d);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (i0 + j < pieces) {
                                    const float w = fast_exp2(mv[j] - big);
                                    denom = fmaf(w, lv[j], denom);
                                    acc = fmaf(w, ov[j], acc);
                                }
                            }
                        }
                        if (kExchange) {
                            exchange_row(xview, (int)row, d, big * kLn2, denom, acc, !dead, a.out + row * kHeadDim, a.status,
                                         exchange_words + 2 * qh, [qh] { if (qh) named_bar_sync(3, kHeadDim); else named_bar_sync(2, kHeadDim); });
                        } else if (dead) {
                        } else if (a.mode == 0) {
                            a.out[row * kHeadDim + d] = (uint16_t)f32_to_bf16_bits(acc / denom);
                        } else {
                            float* out_partial = a.partial_out + row * kPartialStride;
                            out_partial[2 + d] = acc;
                            if (d == 0) {
                                out_partial[0] = big * kLn2;
                                out_partial[1] = denom;
                            }
                        }
                    }
                }
            }
            named_bar_sync(1, kConsumerThreads);
        }
    }
}

// ---------------------------------------------------------------------------
// Short contexts: every stream fits one page (at most 64 keys), e.g. the code predictor's 16 positions or the
// first steps of a talker request.  The split-KV machinery above (unit partition, ring, partials, fold) is all
// overhead there; one small CTA per (stream, kv head) does the whole segment: the page's valid rows come in with two
// bulk copies, four warps score 8 keys per pass (half-warp per key row, as above), one warp per query head does
// the softmax, and every thread owns two output dimensions of one head.  kFused as above: QK-RMSNorm + RoPE of the
// raw q rows and of the new token's K row, which is appended to the pool and attended in the same launch.
constexpr int kShortThreads = 128;

struct ShortSmem {
    static constexpr int kTile = 0;                               // K rows then V rows, 16 KB each
    static constexpr int kQ = 2 * kTileBytes;                     // two q rows (bf16)
    static constexpr int kScore = kQ + 2 * kHeadDim * 2;          // float[2][64]
    static constexpr int kBar = kScore + 2 * kPageTokens * 4;
    static constexpr int kStats = kBar + 8;                       // float[2][2]: row maximum and row sum per query head
    static constexpr int kTotal = kStats + 16;
};

template <bool kFused>
__global__ void __launch_bounds__(kShortThreads) qm_decode_short_kernel(const DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ktile = smem + ShortSmem::kTile;
    unsigned char* vtile = ktile + kTileBytes;
    unsigned char* qrows = smem + ShortSmem::kQ;
    float* score = reinterpret_cast<float*>(smem + ShortSmem::kScore);
    const uint32_t bar = smem_addr(smem + ShortSmem::kBar);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hkv = a.kv_heads;
    const int stream = blockIdx.x / hkv;
    const int head = blockIdx.x - stream * hkv;
    const int seg = blockIdx.x;

    pdl_trigger();
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    pdl_wait();
    const int len = clamp_len(a.seq_lens[stream] + a.len_offset, 1, a.status);       // keys to attend, at most one page
    int page_id = a.page_table[(size_t)stream * a.max_pages];
    if (page_id < 0 || page_id >= a.num_pages) {
        if (tid == 0 && len > 0) atomicOr(a.status, QM_DEVSTAT_BAD_PAGE);
        page_id = 0;
    }
    const size_t row0 = (size_t)seg * 2;                  // the two query rows of this KV head
    if (len == 0) {                                       // nothing to attend: zero row / empty partial
        for (int i = tid; i < 2 * kHeadDim; i += kShortThreads) {
            const size_t row = row0 + i / kHeadDim;
            const int d = i % kHeadDim;
            if (a.mode == 0) {
                a.out[row * kHeadDim + d] = 0;
            } else {
                float* dst = a.partial_out + row * kPartialStride;
                dst[2 + d] = 0.0f;
                if (d == 0) {
                    dst[0] = -CUDART_INF_F;
                    dst[1] = 0.0f;
                }
            }
        }
        return;
    }
    const size_t tile = ((size_t)page_id * hkv + head) * kTileElems;
    const int stored = kFused ? len - 1 : len;            // rows already in the pool
    __syncthreads();                                      // the barrier is initialised
    bool dead = false;
    if (tid == 0) {
        const uint32_t bytes = (uint32_t)stored * (kHeadDim * 2);
        mbar_arrive_expect_tx(bar, 2 * bytes);
        if (bytes) {
            bulk_copy_g2s(smem_addr(ktile), a.key_pool + tile, bytes, bar);
            bulk_copy_g2s(smem_addr(vtile), a.value_pool + tile, bytes, bar);
        }
    }
    if (kFused) {
        // warps 0, 1: the two q rows; warp 2: the new token's K row; warp 3: its V row
        int position = len - 1;
        if (position >= a.rope_rows) {
            if (tid == 0) atomicOr(a.status, QM_DEVSTAT_BAD_POS);
            position = a.rope_rows - 1;
        }
        const uint2 craw = *reinterpret_cast<const uint2*>(a.rope_cos + (size_t)position * kHeadDim + 4 * lane);
        const uint2 sraw = *reinterpret_cast<const uint2*>(a.rope_sin + (size_t)position * kHeadDim + 4 * lane);
        const size_t new_row = tile + (size_t)(len - 1) * kHeadDim + 4 * lane;
        if (warp < 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(a.q_rot + (row0 + warp) * kHeadDim + 4 * lane);
            const uint2 wq = *reinterpret_cast<const uint2*>(a.q_norm_weight + 4 * lane);
            *reinterpret_cast<uint2*>(qrows + warp * 256 + lane * 8) = norm_rope_row(raw, wq, craw, sraw, lane, a.epsilon);
        } else if (warp == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(a.raw_k + (size_t)seg * kHeadDim + 4 * lane);
            const uint2 wk = *reinterpret_cast<const uint2*>(a.k_norm_weight + 4 * lane);
            const uint2 krow = norm_rope_row(raw, wk, craw, sraw, lane, a.epsilon);
            *reinterpret_cast<uint2*>(ktile + (len - 1) * (kHeadDim * 2) + lane * 8) = krow;
            *reinterpret_cast<uint2*>(a.key_pool + new_row) = krow;
        } else {
            const uint2 vrow = *reinterpret_cast<const uint2*>(a.raw_v + (size_t)seg * kHeadDim + 4 * lane);
            *reinterpret_cast<uint2*>(vtile + (len - 1) * (kHeadDim * 2) + lane * 8) = vrow;
            *reinterpret_cast<uint2*>(a.value_pool + new_row) = vrow;
        }
    } else if (warp < 2) {
        *reinterpret_cast<uint2*>(qrows + warp * 256 + lane * 8) =
            *reinterpret_cast<const uint2*>(a.q_rot + (row0 + warp) * kHeadDim + 4 * lane);
    }
    if (!mbar_wait_bounded(bar, 0, dead) && lane == 0) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
    if (__syncthreads_or(dead ? 1 : 0)) {
        // The page never arrived: report it (done above), give the copies one more bounded chance to land so that
        // none is in flight into this CTA's shared memory when it retires, and write nothing.
        if (tid == 0) {
            bool ignore = false;
            mbar_wait_bounded(bar, 0, ignore);
        }
        return;
    }

    // ---- scores in the log2 domain: half-warp per key row, 8 keys per pass over the four warps
    const int half = lane >> 4, lp = lane & 15;
    const float qscale = kLog2e / sqrtf((float)kHeadDim);
    float2 q0[4], q1[4];
    {
        const uint4 qa = *reinterpret_cast<const uint4*>(qrows + lp * 16);
        const uint4 qb = *reinterpret_cast<const uint4*>(qrows + 256 + lp * 16);
        const float2 qs2 = make_float2(qscale, qscale);
        q0[0] = fmul2(bf16x2_to_float2(qa.x), qs2); q0[1] = fmul2(bf16x2_to_float2(qa.y), qs2);
        q0[2] = fmul2(bf16x2_to_float2(qa.z), qs2); q0[3] = fmul2(bf16x2_to_float2(qa.w), qs2);
        q1[0] = fmul2(bf16x2_to_float2(qb.x), qs2); q1[1] = fmul2(bf16x2_to_float2(qb.y), qs2);
        q1[2] = fmul2(bf16x2_to_float2(qb.z), qs2); q1[3] = fmul2(bf16x2_to_float2(qb.w), qs2);
    }
    for (int key0 = 0; key0 < len; key0 += 8) {
        const int key = key0 + 2 * warp + half;
        float d0 = 0.0f, d1 = 0.0f;
        if (key < len) {
            const uint4 kk = *reinterpret_cast<const uint4*>(ktile + key * (kHeadDim * 2) + lp * 16);
            const float2 kf[4] = {bf16x2_to_float2(kk.x), bf16x2_to_float2(kk.y), bf16x2_to_float2(kk.z), bf16x2_to_float2(kk.w)};
            float2 s0 = make_float2(0.0f, 0.0f), s1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s0 = ffma2(q0[j], kf[j], s0);
                s1 = ffma2(q1[j], kf[j], s1);
            }
            d0 = s0.x + s0.y;
            d1 = s1.x + s1.y;
        }
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) {
            d0 += __shfl_xor_sync(0xffffffffu, d0, off);
            d1 += __shfl_xor_sync(0xffffffffu, d1, off);
        }
        if (lp == 0 && key < len) {
            score[key] = d0;
            score[kPageTokens + key] = d1;
        }
    }
    __syncthreads();

    // ---- softmax: warp qh owns query head qh; probabilities replace the scores
    float* stats = reinterpret_cast<float*>(smem + ShortSmem::kStats);
    if (warp < 2) {
        float* sc = score + warp * kPageTokens;
        const float x0 = lane < len ? sc[lane] : -CUDART_INF_F;
        const float x1 = lane + 32 < len ? sc[lane + 32] : -CUDART_INF_F;
        float m = fmaxf(x0, x1);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        const float p0 = lane < len ? fast_exp2(x0 - m) : 0.0f;
        const float p1 = lane + 32 < len ? fast_exp2(x1 - m) : 0.0f;
        float l = p0 + p1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        sc[lane] = p0;
        sc[lane + 32] = p1;
        if (lane == 0) {
            stats[2 * warp] = m;
            stats[2 * warp + 1] = l;
        }
    }
    __syncthreads();

    // ---- O = P V: thread = (query head, two output dimensions)
    {
        const int qh = tid >> 6, dp = tid & 63;
        const float* pr = score + qh * kPageTokens;
        float2 acc = make_float2(0.0f, 0.0f);
        for (int key = 0; key < len; ++key) {
            const float p = pr[key];
            const float2 vv = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(vtile + key * (kHeadDim * 2) + dp * 4));
            acc = ffma2(make_float2(p, p), vv, acc);
        }
        const float m = stats[2 * qh];
        const float l = stats[2 * qh + 1];
        const size_t row = row0 + qh;
        if (a.mode == 0) {
            *reinterpret_cast<uint32_t*>(a.out + row * kHeadDim + 2 * dp) =
                f32_to_bf16_bits(acc.x / l) | (f32_to_bf16_bits(acc.y / l) << 16);
        } else {
            float* dst = a.partial_out + row * kPartialStride;
            *reinterpret_cast<float2*>(dst + 2 + 2 * dp) = acc;
            if (dp == 0) {
                dst[0] = m * kLn2;
                dst[1] = l;
            }
        }
    }
}

// partials [parts][rows][130] (m in natural-log domain) -> out [rows][128] bf16.
__global__ void __launch_bounds__(128) qm_combine_partials_kernel(const float* __restrict__ partials, int parts,
                                                                  int rows, uint16_t* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    float big = -CUDART_INF_F;
    for (int g = 0; g < parts; ++g) big = fmaxf(big, partials[((size_t)g * rows + row) * kPartialStride]);
    float acc = 0.0f, denom = 0.0f;
    for (int g = 0; g < parts; ++g) {
        const float* src = partials + ((size_t)g * rows + row) * kPartialStride;
        if (!(src[1] > 0.0f)) continue;
        const float w = __expf(src[0] - big);
        denom = fmaf(w, src[1], denom);
        acc = fmaf(w, src[2 + d], acc);
    }
    out[(size_t)row * kHeadDim + d] = denom > 0.0f ? (uint16_t)f32_to_bf16_bits(acc / denom) : (uint16_t)0;
}

size_t partials_bytes(int segments) { return (size_t)(kMaxGrid + segments) * 2 * kPartialStride * sizeof(float); }

// Scratch layout: the per-segment arrival counters come first, at a fixed place (counter i at byte 4 * i, room for
// the largest launch: kMaxBatchPerLaunch streams of 64 KV heads), the partial slots after them.  A buffer that serves
// batches of different sizes therefore always finds its counters where the previous call left them at zero, and no
// partial slot can overlap a counter whatever the grid size is.
constexpr size_t kCounterRegionBytes = (size_t)kMaxBatchPerLaunch * 64 * sizeof(int32_t);

// Extra inputs of the fused step (append + attention in one launch); null for plain attention.
struct FusedInputs {
    const uint16_t* k;
    const uint16_t* v;
    const uint16_t* q_norm_weight;
    const uint16_t* k_norm_weight;
    const uint16_t* rope_cos;
    const uint16_t* rope_sin;
    int rope_rows;
    float epsilon;
};

// Units per CTA whose tiles are prefetched into L2 ahead of the dependency wait (0 switches the warm-up off).
// Measured optimum on B200 for the 64-stream ragged batch: 4 (8 and more compete with the launch still running).
// A build with -DQM_DECODE_TUNING reads QM_DECODE_PREFETCH_UNITS from the environment instead.
int decode_prefetch_units() {
#ifdef QM_DECODE_TUNING
    static const int value = [] {
        const char* text = getenv("QM_DECODE_PREFETCH_UNITS");
        int v = text ? atoi(text) : 4;
        return v < 0 ? 0 : (v > 32 ? 32 : v);
    }();
    return value;
#else
    return 4;
#endif
}

int32_t run_decode(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* seq_lens,
                   const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads, uint16_t* out,
                   float* partial_out, void* workspace, int64_t workspace_bytes, cudaStream_t stream, int mode,
                   const FusedInputs* fused = nullptr, const ExchangeView* exchange = nullptr) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (layer < 0 || layer >= pool->layers) return qm_fail(QM_EINVAL, "layer out of range");
    if (!q_rot || !seq_lens || !page_table || !workspace || (mode == 1 ? !partial_out : !out))
        return qm_fail(QM_EINVAL, "null tensor pointer");
    if (mode == 2) {
        if (!exchange || !exchange->peers) return qm_fail(QM_EINVAL, "null pointer");
        if (exchange->world < 1 || exchange->world > kExchangeMaxWorld || exchange->rank < 0 || exchange->rank >= exchange->world ||
            (long long)batch * q_heads > exchange->rows_capacity)
            return qm_fail(QM_EINVAL, "invalid exchange geometry");
        if (batch > kMaxBatchPerLaunch)
            return qm_fail(QM_ECAPACITY, "the fused exchange takes at most 256 streams per call");
    }
    if (q_heads != 2 * pool->kv_heads)
        return qm_fail(QM_EINVAL, "decode attention needs q_heads == 2 * kv_heads (GQA group of 2)");
    if (batch < 0 || max_pages < 1) return qm_fail(QM_EINVAL, "invalid geometry");
    if ((reinterpret_cast<uintptr_t>(q_rot) & 15u) || (reinterpret_cast<uintptr_t>(workspace) & 15u))
        return qm_fail(QM_EINVAL, "q_rot and workspace must be 16-byte aligned");
    if (workspace_bytes < qm_decode_workspace_bytes(batch, pool->kv_heads))
        return qm_fail(QM_EINVAL, "workspace smaller than qm_decode_workspace_bytes()");
    if (batch == 0) return QM_OK;

    static thread_local int attr_device = -1;
    if (attr_device != pool->device) {
        QM_CUDA_TRY(cudaFuncSetAttribute(qm_decode_splitkv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SharedLayout::kTotal),
                    "raise decode kernel shared memory");
        QM_CUDA_TRY(cudaFuncSetAttribute(qm_decode_splitkv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SharedLayout::kTotal),
                    "raise decode kernel shared memory");
        QM_CUDA_TRY(cudaFuncSetAttribute(qm_decode_splitkv_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SharedLayout::kTotal),
                    "raise decode kernel shared memory");
        attr_device = pool->device;
    }
    int grid = 2 * pool->sm_count;
    if (grid > kMaxGrid) grid = kMaxGrid;

    const int chunk_cap = kMaxBatchPerLaunch;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    DecodeArgs a{};
    a.key_pool = qm_kv_pool_key_ptr(pool, layer);
    a.value_pool = qm_kv_pool_value_ptr(pool, layer);
    a.ws_count = reinterpret_cast<int32_t*>(ws);
    a.ws_partials = reinterpret_cast<float*>(ws + kCounterRegionBytes);
    a.status = pool->status_dev;
    a.kv_heads = pool->kv_heads;
    a.max_pages = max_pages;
    a.num_pages = pool->num_pages;
    a.mode = mode;
    a.prefetch_units = decode_prefetch_units();
    if (exchange) a.exchange = *exchange;
    if (fused) {
        a.q_norm_weight = fused->q_norm_weight;
        a.k_norm_weight = fused->k_norm_weight;
        a.rope_cos = fused->rope_cos;
        a.rope_sin = fused->rope_sin;
        a.rope_rows = fused->rope_rows;
        a.epsilon = fused->epsilon;
        a.len_offset = 1;
    }
    for (int begin = 0; begin < batch; begin += chunk_cap) {
        const int n = batch - begin < chunk_cap ? batch - begin : chunk_cap;
        a.q_rot = q_rot + (size_t)begin * q_heads * kHeadDim;
        a.seq_lens = seq_lens + begin;
        a.page_table = page_table + (size_t)begin * max_pages;
        a.out = out ? out + (size_t)begin * q_heads * kHeadDim : nullptr;
        a.partial_out = partial_out ? partial_out + (size_t)begin * q_heads * kPartialStride : nullptr;
        a.batch = n;
        if (fused) {
            a.raw_k = fused->k + (size_t)begin * pool->kv_heads * kHeadDim;
            a.raw_v = fused->v + (size_t)begin * pool->kv_heads * kHeadDim;
        }
        if (max_pages == 1 && mode != 2) {
            // every stream fits one page: one small CTA per (stream, kv head), no scratch involved
            const dim3 short_grid((unsigned)(n * pool->kv_heads));
            if (fused) {
                QM_CUDA_TRY(qm_launch(qm_decode_short_kernel<true>, short_grid, dim3(kShortThreads), ShortSmem::kTotal, stream, a),
                            "fused decode step launch (short contexts)");
            } else {
                QM_CUDA_TRY(qm_launch(qm_decode_short_kernel<false>, short_grid, dim3(kShortThreads), ShortSmem::kTotal, stream, a),
                            "decode attention launch (short contexts)");
            }
            continue;
        }
        if (mode == 2) {
            // the exchange is a variant of its own, so that the other modes compile without it
            QM_CUDA_TRY(qm_launch(qm_decode_splitkv_kernel<false, true>, dim3(grid), dim3(kDecodeThreads), SharedLayout::kTotal,
                                  stream, a),
                        "split-KV decode attention with exchange launch");
        } else if (fused) {
            QM_CUDA_TRY(qm_launch(qm_decode_splitkv_kernel<true>, dim3(grid), dim3(kDecodeThreads), SharedLayout::kTotal,
                                  stream, a),
                        "fused decode step launch");
        } else {
            QM_CUDA_TRY(qm_launch(qm_decode_splitkv_kernel<false>, dim3(grid), dim3(kDecodeThreads), SharedLayout::kTotal,
                                  stream, a),
                        "split-KV decode attention launch");
        }
    }
    return QM_OK;
}

}  // namespace

extern "C" {

int64_t qm_decode_workspace_bytes(int32_t batch, int32_t kv_heads) {
    if (batch < 0 || kv_heads < 1) return 0;
    const int segs = (batch < kMaxBatchPerLaunch ? batch : kMaxBatchPerLaunch) * kv_heads;
    return (int64_t)kCounterRegionBytes + (int64_t)partials_bytes(segs) + 256;
}

int32_t qm_decode_workspace_init(void* workspace, int64_t workspace_bytes, void* stream) {
    if (!workspace || workspace_bytes <= 0) return qm_fail(QM_EINVAL, "workspace is null or empty");
    QM_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)workspace_bytes, static_cast<cudaStream_t>(stream)),
                "clear decode workspace");
    return QM_OK;
}

int32_t qm_decode_attention(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* seq_lens,
                            const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                            uint16_t* out, void* workspace, int64_t workspace_bytes, void* stream) {
    return run_decode(pool, layer, q_rot, seq_lens, page_table, max_pages, batch, q_heads, out, nullptr, workspace,
                      workspace_bytes, static_cast<cudaStream_t>(stream), 0);
}

int32_t qm_decode_step(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                       const uint16_t* q_norm_weight, const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                       const uint16_t* rope_sin, int32_t rope_rows, const int32_t* positions,
                       const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads, float epsilon,
                       uint16_t* out, void* workspace, int64_t workspace_bytes, void* stream) {
    if (!k || !v || !q_norm_weight || !k_norm_weight || !rope_cos || !rope_sin)
        return qm_fail(QM_EINVAL, "null tensor pointer");
    if (rope_rows < 1) return qm_fail(QM_EINVAL, "invalid geometry");
    const uintptr_t all = reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                          reinterpret_cast<uintptr_t>(rope_cos) | reinterpret_cast<uintptr_t>(rope_sin);
    if (all & 15u) return qm_fail(QM_EINVAL, "k, v and the RoPE table must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(q_norm_weight) | reinterpret_cast<uintptr_t>(k_norm_weight)) & 7u)
        return qm_fail(QM_EINVAL, "norm weights must be 8-byte aligned");
    const FusedInputs fused{k, v, q_norm_weight, k_norm_weight, rope_cos, rope_sin, rope_rows, epsilon};
    return run_decode(pool, layer, q, positions, page_table, max_pages, batch, q_heads, out, nullptr, workspace,
                      workspace_bytes, static_cast<cudaStream_t>(stream), 0, &fused);
}

int32_t qm_decode_attention_partial(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                    const int32_t* seq_lens, const int32_t* page_table, int32_t max_pages,
                                    int32_t batch, int32_t q_heads, float* partial, void* workspace,
                                    int64_t workspace_bytes, void* stream) {
    return run_decode(pool, layer, q_rot, seq_lens, page_table, max_pages, batch, q_heads, nullptr, partial,
                      workspace, workspace_bytes, static_cast<cudaStream_t>(stream), 1);
}

int32_t qm_decode_attention_exchange(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* local_seq_lens,
                                     const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                                     uint16_t* out, void* const* peer_buffers_dev, int32_t world, int32_t rank,
                                     int32_t rows_capacity, void* workspace, int64_t workspace_bytes, void* stream) {
    ExchangeView view{};
    view.peers = reinterpret_cast<unsigned char* const*>(peer_buffers_dev);
    view.world = world;
    view.rank = rank;
    view.rows_capacity = rows_capacity;
    return run_decode(pool, layer, q_rot, local_seq_lens, page_table, max_pages, batch, q_heads, out, nullptr, workspace,
                      workspace_bytes, static_cast<cudaStream_t>(stream), 2, nullptr, &view);
}

int32_t qm_attention_combine(const float* partials, int32_t parts, int32_t rows, uint16_t* out, void* stream) {
    if (!partials || !out) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (parts < 1 || rows < 0) return qm_fail(QM_EINVAL, "parts must be >= 1 and rows >= 0");
    if (rows == 0) return QM_OK;
    QM_CUDA_TRY(qm_launch(qm_combine_partials_kernel, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream), partials,
                          (int)parts, (int)rows, out),
                "attention combine launch");
    return QM_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// The split-KV kernel needs scratch for its per-CTA partials.  The regular
// entry point takes that scratch from the caller, who has to cudaMalloc it
// somewhere.  Some hosts of this library cannot: a resident serving loop that
// fixed its device-memory budget at start-up and runs the codec decoder on a
// second stream (cudaMalloc and cudaFree synchronise the whole device and
// would stall that stream in the middle of an audio packet), or an engine
// whose allocator already owns all device memory.  For them the scratch below
// is part of the library image: every GPU that loads the library carries
// these bytes until the process exits, whether or not the entry point is used.
constexpr int kStaticMaxBatch = 64;
constexpr int kStaticMaxKvHeads = 8;
constexpr size_t kStaticScratchBytes =
    kCounterRegionBytes                                                                             // arrival counters
    + (size_t)(kMaxGrid + kStaticMaxBatch * kStaticMaxKvHeads) * 2 * kPartialStride * sizeof(float)  // partials
    + 256;

static __device__ __align__(256) unsigned char qm_static_decode_scratch[kStaticScratchBytes];

namespace {

constexpr int kMaxDevices = 64;

// Device address of the scratch array on `device`, which must be the current
// device.  In host code the array's name is only a handle for the runtime, not
// something a kernel can be given, so the address is looked up once per device
// and remembered.
int32_t static_scratch_address(int device, void** address_out) {
    static std::mutex guard;
    static void* known[kMaxDevices] = {};
    if (device < 0 || device >= kMaxDevices) return qm_fail(QM_EINVAL, "device index out of range for the static scratch");
    // Every call, not only the first: the launch goes to the current device, and the pool's pointers and the
    // address remembered here belong to the pool's device.
    int current = -1;
    QM_CUDA_TRY(cudaGetDevice(&current), "get current device");
    if (current != device)
        return qm_fail(QM_EINVAL, "the pool's device must be the current device for the static-scratch entry points");
    std::lock_guard<std::mutex> lock(guard);
    if (!known[device]) {
        void* address = nullptr;
        QM_CUDA_TRY(cudaGetSymbolAddress(&address, qm_static_decode_scratch), "look up static decode scratch");
        if (!address) return qm_fail(QM_ECUDA, "static decode scratch has no device address");
        known[device] = address;
    }
    *address_out = known[device];
    return QM_OK;
}

}  // namespace

extern "C" int32_t qm_decode_attention_static(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                              const int32_t* seq_lens, const int32_t* page_table,
                                              int32_t max_pages, int32_t batch, int32_t q_heads, uint16_t* out,
                                              void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (batch > kStaticMaxBatch || pool->kv_heads > kStaticMaxKvHeads)
        return qm_fail(QM_ECAPACITY,
                       "qm_decode_attention_static handles at most 64 streams of at most 8 KV heads per call; "
                       "use qm_decode_attention with caller-provided workspace for larger batches");
    void* scratch = nullptr;
    const int32_t looked_up = static_scratch_address(pool->device, &scratch);
    if (looked_up != QM_OK) return looked_up;
    // The only part of the scratch that must start at zero is the per-segment
    // arrival counters.  The array is zero when the library is loaded, and the
    // kernel puts every counter it used back to zero before it finishes, so no
    // clearing is needed here; partial slots are always written before they are
    // read within one call, so leftovers from the previous call are never used.
    // The one exception is a call that reported QM_DEVSTAT_TIMEOUT: it may leave
    // counters behind, and qm_decode_static_scratch_reset puts them back.
    return run_decode(pool, layer, q_rot, seq_lens, page_table, max_pages, batch, q_heads, out, nullptr, scratch,
                      (int64_t)kStaticScratchBytes, static_cast<cudaStream_t>(stream), 0);
}

extern "C" int32_t qm_decode_static_scratch_reset(qm_kv_pool* pool, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    void* scratch = nullptr;
    const int32_t looked_up = static_scratch_address(pool->device, &scratch);
    if (looked_up != QM_OK) return looked_up;
    // a memset on an address that already exists: nothing is allocated
    QM_CUDA_TRY(cudaMemsetAsync(scratch, 0, kCounterRegionBytes, static_cast<cudaStream_t>(stream)),
                "clear static decode scratch counters");
    return QM_OK;
}
