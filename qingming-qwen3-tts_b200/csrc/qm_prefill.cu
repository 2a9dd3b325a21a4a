// Causal GQA prefill attention over the paged bf16 KV cache, on the 5th-gen
// tensor cores: tcgen05.mma with TMEM accumulators, operands staged by TMA.
//
// Stands in for talker_attention_kernel (17.cu:15791-16054, dispatch
// :17954-17985), which runs one CTA per (query row, query head), re-reads K
// and V from global memory for every row and does O(L^2 * D) scalar FMAs.
//
// One CTA owns 128 query positions of one KV head and BOTH query heads that
// share it (two 128 x 128 Q tiles), so every K/V tile fetched serves two
// score tiles.  Per 128-key block j (causal: only blocks up to the diagonal
// are visited):
//
//   S_t = Q_t K_j^T      tcgen05.mma  A, B from shared memory (128B swizzle), D in TMEM
//   P_t = softmax step   4 warps per tile, thread = row: two passes of tcgen05.ld over S
//                        (row max, then exp2 / sum in packed fp32x2), bf16 P written back
//                        over S with tcgen05.st
//   O_t += P_t V_j       tcgen05.mma  A = P from TMEM, B = V tile (MN-major)
//
// Warp roles: warps 0-3 softmax of tile 0, warps 4-7 softmax of tile 1, warp 8
// issues every MMA (one elected lane), warp 9 issues every TMA load.  The two
// tiles interleave on the tensor pipe, so one tile's softmax overlaps the other
// tile's MMAs.  TMEM columns: S0 0-127, S1 128-255, O0 256-383, O1 384-511.
//
// Running maximum: O is only rescaled when a row's maximum grew by more than
// 2^8 since the value in use (probabilities then stay below 256, exact enough
// in bf16 / fp32), which makes the TMEM round trip of a rescale rare.
//
// K/V tiles come straight from the pool through one tiled tensor map per pool
// (rows of 128 bf16, 64 x 64 boxes): a 128-key tile is two pages.  Every wait
// is bounded; a wait that gives up sets QM_DEVSTAT_TIMEOUT and the CTA runs to
// its end (results are then garbage, TMEM is still freed).
#include <math_constants.h>

#include <new>

#include "qm_tcgen05.cuh"

namespace {

constexpr int kBlockM = 128;            // query positions per CTA
constexpr int kBlockN = 128;            // keys per tile (two pages)
constexpr int kPrefillThreads = 320;
constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 9;
constexpr int kTileBytesQ = kBlockM * kHeadDim * 2;      // 32 KB
constexpr int kTileBytesKV = kBlockN * kHeadDim * 2;     // 32 KB
constexpr int kKvStages = 2;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

struct PrefillSmem {
    static constexpr int kQ = 0;                                        // 2 tiles
    static constexpr int kK = kQ + 2 * kTileBytesQ;                     // kKvStages tiles
    static constexpr int kV = kK + kKvStages * kTileBytesKV;
    static constexpr int kBars = kV + kKvStages * kTileBytesKV;
    static constexpr int kTmemSlot = kBars + 16 * 8;
    static constexpr int kTotal = kTmemSlot + 16;
};

// barrier indices
enum { BAR_Q = 0, BAR_KFULL = 1, BAR_KEMPTY = 3, BAR_VFULL = 5, BAR_VEMPTY = 7, BAR_SFULL = 9, BAR_PREADY = 11, BAR_OREADY = 13 };

struct PrefillArgs {
    const int32_t* cu_seqlens;
    const int32_t* start_positions;
    const int32_t* page_table;
    uint16_t* out;
    uint32_t* status;
    int batch;
    int kv_heads;
    int max_pages;
    int num_pages;
    int max_qblocks;
};

__global__ void __launch_bounds__(kPrefillThreads, 1)
qm_prefill_attention_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, const PrefillArgs a) {
    pdl_trigger();
    pdl_wait();
    // ---- which work item: heaviest query blocks first
    const int per_block_row = a.batch * a.kv_heads;
    const int qblock = a.max_qblocks - 1 - (int)(blockIdx.x / per_block_row);
    const int rem = (int)(blockIdx.x % per_block_row);
    const int stream = rem / a.kv_heads;
    const int head = rem % a.kv_heads;
    const int cu0 = a.cu_seqlens[stream];
    const int len = a.cu_seqlens[stream + 1] - cu0;
    const int q0 = qblock * kBlockM;
    if (q0 >= len) return;
    const int start = a.start_positions ? a.start_positions[stream] : 0;
    const int rows_here = len - q0 < kBlockM ? len - q0 : kBlockM;
    const int kv_needed = start + q0 + rows_here;                 // keys 0 .. kv_needed-1
    const int n_tiles = (kv_needed + kBlockN - 1) / kBlockN;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_addr(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    unsigned char* smem = smem_raw + pad;
    const uint32_t sbase = raw_addr + pad;
    const uint32_t bar0 = sbase + PrefillSmem::kBars;
    auto bar = [&](int i) { return bar0 + 8u * i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + PrefillSmem::kTmemSlot);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        mbar_init(bar(BAR_Q), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(BAR_KFULL + s), 1);
            mbar_init(bar(BAR_KEMPTY + s), 1);
            mbar_init(bar(BAR_VFULL + s), 1);
            mbar_init(bar(BAR_VEMPTY + s), 1);
            mbar_init(bar(BAR_SFULL + s), 1);
            mbar_init(bar(BAR_PREADY + s), 128);
            mbar_init(bar(BAR_OREADY + s), 1);
        }
        fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_addr(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    bool dead = false;

    if (warp == kLoadWarp) {
        // ------------------------------------------------------------- TMA loads
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(BAR_Q), 2 * kTileBytesQ);
            for (int t = 0; t < 2; ++t)
                for (int half = 0; half < 2; ++half)
                    tma_load_3d(sbase + PrefillSmem::kQ + t * kTileBytesQ + half * (kTileBytesQ / 2), &q_map, bar(BAR_Q),
                                half * 64, 2 * head + t, cu0 + q0);
            for (int j = 0; j < n_tiles; ++j) {
                int page_id[2];
                for (int p = 0; p < 2; ++p) {
                    int idx = 2 * j + p;
                    if (idx * kPageTokens >= kv_needed || idx >= a.max_pages) idx = 2 * j;   // tile tail: reuse a valid page
                    if (idx >= a.max_pages) {                                                // sequence longer than its table
                        atomicOr(a.status, QM_DEVSTAT_BAD_POS);
                        idx = a.max_pages - 1;
                    }
                    int id = a.page_table[(size_t)stream * a.max_pages + idx];
                    if (id < 0 || id >= a.num_pages) {
                        atomicOr(a.status, QM_DEVSTAT_BAD_PAGE);
                        id = 0;
                    }
                    page_id[p] = id;
                }
                const int st = j % kKvStages;
                const uint32_t parity = ((j / kKvStages) & 1) ^ 1;
                if (!mbar_wait_bounded(bar(BAR_KEMPTY + st), parity, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                mbar_arrive_expect_tx(bar(BAR_KFULL + st), kTileBytesKV);
                for (int p = 0; p < 2; ++p)
                    for (int half = 0; half < 2; ++half)
                        tma_load_2d(sbase + PrefillSmem::kK + st * kTileBytesKV + half * (kTileBytesKV / 2) + p * 8192, &k_map,
                                    bar(BAR_KFULL + st), half * 64, (page_id[p] * a.kv_heads + head) * kPageTokens);
                if (!mbar_wait_bounded(bar(BAR_VEMPTY + st), parity, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                mbar_arrive_expect_tx(bar(BAR_VFULL + st), kTileBytesKV);
                for (int p = 0; p < 2; ++p)
                    for (int half = 0; half < 2; ++half)
                        tma_load_2d(sbase + PrefillSmem::kV + st * kTileBytesKV + half * (kTileBytesKV / 2) + p * 8192, &v_map,
                                    bar(BAR_VFULL + st), half * 64, (page_id[p] * a.kv_heads + head) * kPageTokens);
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------- MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_instr_desc(kBlockM, kBlockN, false);
            constexpr uint32_t idesc_pv = umma_instr_desc(kBlockM, kBlockN, true);
            auto issue_s = [&](int t, int kst) {
                const uint32_t qa = sbase + PrefillSmem::kQ + t * kTileBytesQ;
                const uint32_t ka = sbase + PrefillSmem::kK + kst * kTileBytesKV;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * (kTileBytesQ / 2) + (ks & 3) * 32;
                    mma_ss(tmem_base + t * 128, smem_desc(qa + off, 16, 1024), smem_desc(ka + off, 16, 1024), idesc_qk, ks > 0);
                }
            };
            auto issue_pv = [&](int t, int vst, bool accumulate) {
                const uint32_t va = sbase + PrefillSmem::kV + vst * kTileBytesKV;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    mma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8,
                           smem_desc(va + ks * 2048, kTileBytesKV / 2, 1024), idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
            };
            if (!mbar_wait_bounded(bar(BAR_Q), 0, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
            if (!mbar_wait_bounded(bar(BAR_KFULL + 0), 0, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
            tc_fence_after();
            issue_s(0, 0);
            tc_commit(bar(BAR_SFULL + 0));
            issue_s(1, 0);
            tc_commit(bar(BAR_SFULL + 1));
            tc_commit(bar(BAR_KEMPTY + 0));
            // Barriers that are normally complete by the time they are needed (V, the next K, P of the second
            // head) are probed before the preceding batch of MMAs, so their round trip overlaps the issue.
            uint32_t v_seen = mbar_probe(bar(BAR_VFULL + 0), 0);
            for (int j = 0; j < n_tiles; ++j) {
                const int vst = j % kKvStages;
                const int kst = (j + 1) % kKvStages;
                const bool more = j + 1 < n_tiles;
                if (!mbar_wait_probed(v_seen, bar(BAR_VFULL + vst), (j / kKvStages) & 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                if (!mbar_wait_bounded(bar(BAR_PREADY + 0), j & 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                const uint32_t k_seen = more ? mbar_probe(bar(BAR_KFULL + kst), ((j + 1) / kKvStages) & 1) : 1u;
                const uint32_t p1_seen = mbar_probe(bar(BAR_PREADY + 1), j & 1);
                tc_fence_after();
                issue_pv(0, vst, j > 0);
                tc_commit(bar(BAR_OREADY + 0));
                if (more) {
                    if (!mbar_wait_probed(k_seen, bar(BAR_KFULL + kst), ((j + 1) / kKvStages) & 1, dead))
                        atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                    tc_fence_after();
                    issue_s(0, kst);
                    tc_commit(bar(BAR_SFULL + 0));
                }
                if (!mbar_wait_probed(p1_seen, bar(BAR_PREADY + 1), j & 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                v_seen = more ? mbar_probe(bar(BAR_VFULL + kst), ((j + 1) / kKvStages) & 1) : 1u;
                tc_fence_after();
                issue_pv(1, vst, j > 0);
                tc_commit(bar(BAR_OREADY + 1));
                tc_commit(bar(BAR_VEMPTY + vst));
                if (more) {
                    issue_s(1, kst);
                    tc_commit(bar(BAR_SFULL + 1));
                    tc_commit(bar(BAR_KEMPTY + kst));
                }
            }
        }
        __syncwarp();
    } else {
        // --------------------------------------------------------------- softmax
        const int t = warp >> 2;                       // which Q tile / query head of the pair
        const int row = (warp & 3) * 32 + lane;        // row of the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + t * 128;
        const uint32_t o_addr = tmem_base + lane_base + 256 + t * 128;
        const float c = 1.4426950408889634f / sqrtf((float)kHeadDim);       // scale * log2(e)
        const int qrow = q0 + row < len ? q0 + row : len - 1;
        const int qpos = start + qrow;
        float m_used = -CUDART_INF_F;
        float l = 0.0f;

        for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait_bounded(bar(BAR_SFULL + t), j & 1, dead) && lane == 0) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
            tc_fence_after();
            const int key0 = j * kBlockN;
            const bool diagonal = key0 + kBlockN - 1 > start + q0;       // some key of the tile lies past some row
            const int keys_visible = qpos - key0 + 1;                    // columns [0, keys_visible) of this row count

            // ---- the whole 128-column row of S into registers (one TMEM read)
            uint32_t sreg[4][32];
#pragma unroll
            for (int cch = 0; cch < 4; ++cch) tmem_ld32(s_addr + cch * 32, sreg[cch]);
            tmem_wait_ld();
            if (diagonal) {
#pragma unroll
                for (int cch = 0; cch < 4; ++cch)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (cch * 32 + i >= keys_visible) sreg[cch][i] = __float_as_uint(-CUDART_INF_F);
            }
            // ---- row maximum: 8 independent chains of 3-input max
            float mxa[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mxa[i] = -CUDART_INF_F;
#pragma unroll
            for (int cch = 0; cch < 4; ++cch)
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    mxa[(i >> 1) & 7] = fmax3(mxa[(i >> 1) & 7], __uint_as_float(sreg[cch][i]), __uint_as_float(sreg[cch][i + 1]));
            const float mx = fmax3(fmax3(mxa[0], mxa[1], mxa[2]), fmax3(mxa[3], mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7]));

            const float m_new = fmaxf(m_used, mx * c);
            const bool grow = m_new - m_used > kRescaleThreshold;     // also true on the first tile (m_used = -inf)
            if (j == 0) {
                m_used = m_new;
            } else if (__any_sync(0xffffffffu, grow)) {
                // Rescale O: PV of the previous block must have landed first.
                if (!mbar_wait_bounded(bar(BAR_OREADY + t), (j - 1) & 1, dead) && lane == 0)
                    atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                tc_fence_after();
                const float factor = grow ? fast_exp2(m_used - m_new) : 1.0f;
                if (grow) m_used = m_new;
                l *= factor;
#pragma unroll 1
                for (int cch = 0; cch < 8; ++cch) {
                    uint32_t oreg[16];
                    tmem_ld16(o_addr + cch * 16, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * factor);
                    tmem_st16(o_addr + cch * 16, oreg);
                }
                tmem_wait_st();
            }

            // ---- P = exp2(s * c - m) as bf16 pairs, written over the first 64 columns of S
            float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            const float2 c2 = make_float2(c, c), negm2 = make_float2(-m_used, -m_used);
#pragma unroll
            for (int cch = 0; cch < 4; ++cch) {
                uint32_t preg[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 x = ffma2(make_float2(__uint_as_float(sreg[cch][2 * i]), __uint_as_float(sreg[cch][2 * i + 1])),
                                           c2, negm2);
                    const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    sum2[i & 3] = fadd2(sum2[i & 3], p);
                    preg[i] = pack_bf16x2(p.x, p.y);
                }
                tmem_st16(s_addr + cch * 16, preg);
            }
            l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y) + (sum2[2].x + sum2[2].y) + (sum2[3].x + sum2[3].y);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(BAR_PREADY + t));
        }

        // ---- epilogue: O / l -> bf16 -> global
        if (!mbar_wait_bounded(bar(BAR_OREADY + t), (n_tiles - 1) & 1, dead) && lane == 0)
            atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
        tc_fence_after();
        const float inv_l = 1.0f / l;
        const bool store = q0 + row < len;
        uint16_t* dst = a.out + ((size_t)(cu0 + qrow) * (2 * a.kv_heads) + 2 * head + t) * kHeadDim;
#pragma unroll
        for (int cch = 0; cch < 4; ++cch) {
            uint32_t oreg[32];
            tmem_ld32(o_addr + cch * 32, oreg);
            tmem_wait_ld();
            if (store) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(oreg[i + 0]) * inv_l, __uint_as_float(oreg[i + 1]) * inv_l);
                    w.y = pack_bf16x2(__uint_as_float(oreg[i + 2]) * inv_l, __uint_as_float(oreg[i + 3]) * inv_l);
                    w.z = pack_bf16x2(__uint_as_float(oreg[i + 4]) * inv_l, __uint_as_float(oreg[i + 5]) * inv_l);
                    w.w = pack_bf16x2(__uint_as_float(oreg[i + 6]) * inv_l, __uint_as_float(oreg[i + 7]) * inv_l);
                    *reinterpret_cast<uint4*>(dst + cch * 32 + i) = w;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ----------------------------------------------------------------

// rows x 128 bf16, boxes of 64 rows x 64 columns, 128-byte swizzle.
int32_t encode_pool_map(CUtensorMap* map, void* base, uint64_t rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)kHeadDim * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled failed for a KV pool");
    return QM_OK;
}

// [tokens][heads][128] bf16 viewed as {128, heads, tokens}; boxes of 128 tokens x 1 head x 64 columns.
int32_t encode_query_map(CUtensorMap* map, const void* base, int heads, uint64_t tokens) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)heads, tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)kHeadDim * 2 * heads};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)kBlockM};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled failed for the query tensor");
    return QM_OK;
}

}  // namespace

int32_t qm_pool_build_tensor_maps(qm_kv_pool* pool) {
    pool->key_maps = new (std::nothrow) CUtensorMap[pool->layers];
    pool->value_maps = new (std::nothrow) CUtensorMap[pool->layers];
    if (!pool->key_maps || !pool->value_maps) return qm_fail(QM_ENOMEM, "host allocation of tensor maps failed");
    const uint64_t rows = (uint64_t)pool->num_pages * pool->kv_heads * kPageTokens;
    for (int layer = 0; layer < pool->layers; ++layer) {
        int32_t rc = encode_pool_map(&pool->key_maps[layer], pool->key + (size_t)layer * pool->layer_elems, rows);
        if (rc != QM_OK) return rc;
        rc = encode_pool_map(&pool->value_maps[layer], pool->value + (size_t)layer * pool->layer_elems, rows);
        if (rc != QM_OK) return rc;
    }
    return QM_OK;
}

extern "C" int32_t qm_prefill_attention_varlen(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                               const int32_t* cu_seqlens, const int32_t* start_positions,
                                               const int32_t* page_table, int32_t max_pages, int32_t batch,
                                               int32_t total_tokens, int32_t max_seqlen, int32_t q_heads,
                                               uint16_t* out, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    if (layer < 0 || layer >= pool->layers) return qm_fail(QM_EINVAL, "layer out of range");
    if (!q_rot || !cu_seqlens || !page_table || !out) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (q_heads != 2 * pool->kv_heads)
        return qm_fail(QM_EINVAL, "prefill attention needs q_heads == 2 * kv_heads (GQA group of 2)");
    if (batch < 1 || total_tokens < 0 || max_seqlen < 0 || max_pages < 1) return qm_fail(QM_EINVAL, "invalid geometry");
    if ((reinterpret_cast<uintptr_t>(q_rot) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
        return qm_fail(QM_EINVAL, "q_rot and out must be 16-byte aligned");
    if (total_tokens == 0 || max_seqlen == 0) return QM_OK;

    CUtensorMap q_map;
    int32_t rc = encode_query_map(&q_map, q_rot, q_heads, (uint64_t)total_tokens);
    if (rc != QM_OK) return rc;

    static thread_local int attr_device = -1;
    const int smem_bytes = PrefillSmem::kTotal + 1024;
    if (attr_device != pool->device) {
        QM_CUDA_TRY(cudaFuncSetAttribute(qm_prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes),
                    "raise prefill kernel shared memory");
        attr_device = pool->device;
    }
    PrefillArgs a{};
    a.cu_seqlens = cu_seqlens;
    a.start_positions = start_positions;
    a.page_table = page_table;
    a.out = out;
    a.status = pool->status_dev;
    a.batch = batch;
    a.kv_heads = pool->kv_heads;
    a.max_pages = max_pages;
    a.num_pages = pool->num_pages;
    a.max_qblocks = (max_seqlen + kBlockM - 1) / kBlockM;
    const long long blocks = (long long)a.max_qblocks * batch * pool->kv_heads;
    if (blocks > 0x7fffffffLL) return qm_fail(QM_ECAPACITY, "too many query blocks for one launch");
    QM_CUDA_TRY(qm_launch(qm_prefill_attention_kernel, dim3((unsigned)blocks), dim3(kPrefillThreads), (size_t)smem_bytes,
                          static_cast<cudaStream_t>(stream), q_map, pool->key_maps[layer], pool->value_maps[layer], a),
                "Talker prefill attention launch");
    return QM_OK;
}
