// Skinny GEMM for the talker layer's projections at decode time: out[M][N] = x[M][K] * W[N][K]^T with M <= 64 token
// rows, i.e. pure weight streaming (every weight byte is read once, 2*M flop per byte pair).
//
// Stands in for the reference's M = 1 GEMV kernels, which it launches once per token:
//   talker_linear_fused_kernel           17.cu:15250-15317 (launcher :17646)   o-proj, down-proj (+ residual)
//   talker_qkv_fused_kernel              17.cu:15321-15407 (launcher :17691)   q, k, v projections
//   talker_gate_up_swiglu_fused_kernel   17.cu:16348-16416 (launcher :18020)   gate / up projections + SwiGLU
// and keeps their bf16 materialisation points (projection result, residual sum, gate, up, activation, product).
//
// Mapping: the WEIGHT tile is the tensor core's M operand (128 weight rows per CTA), the token rows are its N
// operand (padded to 32 or 64), so D^T[128 x M] accumulates in 32 / 64 TMEM columns.  K is split across the CTAs
// of a thread-block cluster; each CTA streams its K range through a TMA ring (128B-swizzled 64-column chunks)
// and tcgen05.mma; partial sums meet in distributed shared memory and are folded in cluster-rank order, so the
// result does not depend on timing.  The weight chunks of the first ring stages are requested BEFORE the
// programmatic-dependent-launch wait: weights are constants, so they can stream in while the previous kernel of
// the layer is still finishing; only the activations wait.
#include <cstdlib>
#include <new>

#include "qm_tcgen05.cuh"

namespace {

constexpr int kGemmThreads = 192;      // warps 0-3 epilogue (one TMEM lane each), warp 4 MMA issue, warp 5 TMA
constexpr int kTileRows = 128;         // weight rows per CTA
constexpr int kChunkCols = 64;         // K columns per ring stage (128 bytes: one swizzle atom)
constexpr int kWeightStageBytes = kTileRows * kChunkCols * 2;   // 16 KB

enum { EPI_LINEAR = 0, EPI_SWIGLU = 1 };

// Up to three weight matrices that share the input rows (q, k and v projections) run in one launch; each is a
// segment with its own output tensor.  A plain linear is one segment.
struct GemmArgs {
    const uint16_t* bias[3];     // [N] or null
    uint16_t* out[3];            // [M][N]  (SwiGLU: N = intermediate)
    int out_cols[3];             // N of each segment
    int first_tile[3];           // tile index where each segment starts
    const uint16_t* weight[3];   // raw weight pointers [N][K] (SwiGLU: gate, up), for the L2 warm-up
    int k_dim;                   // K
    const uint16_t* residual;    // [M][N] or null (single-segment calls)
    uint32_t* status;
    int rows;                    // M
    int chunks;                  // K / 64
    int split;                   // cluster size: CTAs sharing one tile's K range
};

template <int kMPad>
struct GemmSmem {
    static constexpr int kStages = kMPad == 32 ? 4 : 3;
    static constexpr int kActStageBytes = kMPad * kChunkCols * 2;
    static constexpr int kStageBytes = kWeightStageBytes + kActStageBytes;
    static constexpr int kRing = 0;
    static constexpr int kReduce = kStages * kStageBytes;                 // float[kMPad][128]
    static constexpr int kBars = kReduce + kMPad * kTileRows * 4;         // full[kStages], empty[kStages], acc
    static constexpr int kTmemSlot = kBars + (2 * kStages + 1) * 8;
    static constexpr int kTotal = kTmemSlot + 16;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local_addr` in the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// Not volatile and no memory clobber on purpose: the loads of one fold are independent and should all be in
// flight together; they sit between two cluster barriers (which are compiler barriers) and read data that is
// not written in between.
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t remote_addr) {
    float4 v;
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote_addr));
    return v;
}
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
template <int kMPad, int kEpilogue>
__global__ void __launch_bounds__(kGemmThreads)
qm_skinny_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap w2_map,
                      const __grid_constant__ CUtensorMap w3_map, const __grid_constant__ CUtensorMap x_map,
                      const GemmArgs a) {
    using L = GemmSmem<kMPad>;
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_addr(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    unsigned char* smem = smem_raw + pad;
    const uint32_t sbase = raw_addr + pad;
    const uint32_t bar0 = sbase + L::kBars;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (L::kStages + s); };
    const uint32_t acc_bar = bar0 + 8u * (2 * L::kStages);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
    float* reduce = reinterpret_cast<float*>(smem + L::kReduce);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int global_tile = blockIdx.x / a.split;
    const int seg = (kEpilogue == EPI_LINEAR) ? (global_tile >= a.first_tile[2] ? 2 : (global_tile >= a.first_tile[1] ? 1 : 0)) : 0;
    const int tile = global_tile - a.first_tile[seg];
    const CUtensorMap* seg_map = seg == 0 ? &w_map : (seg == 1 ? &w2_map : &w3_map);
    // this CTA's share of the K chunks (contiguous, sizes differ by at most one)
    const int chunk_begin = (int)((long long)a.chunks * rank / a.split);
    const int chunk_end = (int)((long long)a.chunks * (rank + 1) / a.split);
    const int n_chunks = chunk_end - chunk_begin;

    // A weight byte is read once per step: it should not push activations and partial sums out of the L2.
    const uint64_t weights_once = l2_policy_evict_first();
    auto load_weights = [&](int i) {
        const int st = i % L::kStages;
        const uint32_t dst = sbase + L::kRing + st * L::kStageBytes;
        const int col = (chunk_begin + i) * kChunkCols;
        mbar_arrive_expect_tx(full_bar(st), L::kStageBytes);
        if (kEpilogue == EPI_SWIGLU) {
            tma_load_2d_hint(dst, &w_map, full_bar(st), col, tile * 64, weights_once);                 // gate rows -> rows 0..63
            tma_load_2d_hint(dst + kWeightStageBytes / 2, &w2_map, full_bar(st), col, tile * 64, weights_once);   // up rows -> 64..127
        } else {
            tma_load_2d_hint(dst, seg_map, full_bar(st), col, tile * kTileRows, weights_once);
        }
    };
    const int head = n_chunks < L::kStages ? n_chunks : L::kStages;
    if (warp == 5 && lane == 0) {
        // The copy warp sets up the barriers itself and asks for its first weight chunks right away - weights are
        // constants, so this may overlap the previous kernel and the TMEM allocation below.
        for (int s = 0; s < L::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        fence_mbar_init();
        for (int i = 0; i < head; ++i) load_weights(i);
    }
    if (warp == 4) {
        tmem_alloc(smem_addr(tmem_slot), kMPad);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    bool dead = false;

    if (warp == 5) {
        // ------------------------------------------------------------------ TMA
        if (lane == 0) {
            auto load_rows = [&](int i) {
                const int st = i % L::kStages;
                tma_load_2d(sbase + L::kRing + st * L::kStageBytes + kWeightStageBytes, &x_map, full_bar(st),
                            (chunk_begin + i) * kChunkCols, 0);
            };
            pdl_wait();                                          // activations come from the previous kernel
            for (int i = 0; i < head; ++i) load_rows(i);
            for (int i = head; i < n_chunks; ++i) {
                const int st = i % L::kStages;
                if (!mbar_wait_bounded(empty_bar(st), ((i / L::kStages) & 1) ^ 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                load_weights(i);
                load_rows(i);
            }
        }
        __syncwarp();
    } else if (warp == 4) {
        // ------------------------------------------------------------------ MMA
        if (lane == 0) {
            constexpr uint32_t idesc = umma_instr_desc(kTileRows, kMPad, false);
            for (int i = 0; i < n_chunks; ++i) {
                const int st = i % L::kStages;
                if (!mbar_wait_bounded(full_bar(st), (i / L::kStages) & 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                tc_fence_after();
                const uint32_t wa = sbase + L::kRing + st * L::kStageBytes;
                const uint32_t xa = wa + kWeightStageBytes;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tmem_base, smem_desc(wa + ks * 32, 16, 1024), smem_desc(xa + ks * 32, 16, 1024), idesc,
                           (i > 0 || ks > 0) ? 1u : 0u);
                tc_commit(empty_bar(st));
            }
            tc_commit(acc_bar);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------- L2 warm-up of this CTA's weight slice
        // Still before the dependency wait: weights are constants.  The ring above holds only its first stages;
        // here every thread asks the L2 for one weight row's share of this CTA's K range, so that HBM streams the
        // whole slice while the previous kernel finishes and the ring's later loads find their bytes in L2.
        {
            const uint16_t* wbase;
            int wrow;
            if (kEpilogue == EPI_SWIGLU) {
                wbase = tid < 64 ? a.weight[0] : a.weight[1];
                wrow = tile * 64 + (tid & 63);
            } else {
                wbase = a.weight[seg];
                wrow = tile * kTileRows + tid;
            }
            // (the ring's own first stages are already on their way)
            if (wrow < a.out_cols[seg] && n_chunks > head)
                bulk_prefetch_l2_hint(wbase + (size_t)wrow * a.k_dim + (size_t)(chunk_begin + head) * kChunkCols,
                                      (uint32_t)((n_chunks - head) * kChunkCols * 2), l2_policy_evict_last());
        }
        // ------------------------------------------------- partial sums -> own shared memory
        if (!mbar_wait_bounded(acc_bar, 0, dead) && lane == 0) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c = 0; c < kMPad / 32; ++c) {
            uint32_t v[32];
            if (n_chunks > 0) {
                tmem_ld32(taddr + c * 32, v);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) reduce[(c * 32 + i) * kTileRows + tid] = __uint_as_float(v[i]);
        }
        pdl_wait();      // the stores below may overwrite what the previous kernel still reads
    }

    // Every CTA of the cluster has its partial tile in shared memory.
    cluster_sync_all();

    if (warp < 4) {
        // ------------------------------------------------- fold in rank order + epilogue
        // Rank r finishes the token rows r, r + split, ...  One work item = one of those token rows x four
        // neighbouring weight rows of the tile (one 16-byte read per peer, one 8-byte store); SwiGLU: four gate
        // rows and the four up rows that go with them.
        const uint32_t reduce_addr = sbase + L::kReduce;
        constexpr int kGroups = kEpilogue == EPI_SWIGLU ? 16 : 32;
        uint32_t peer[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) peer[k] = map_to_rank(reduce_addr, (uint32_t)(k < a.split ? k : 0));
        const int owned = ((int)rank < a.rows) ? (a.rows - 1 - (int)rank) / a.split + 1 : 0;
        const int n_cols = a.out_cols[seg];
        for (int item = tid; item < owned * kGroups; item += 128) {
            const int g = item % kGroups;
            const int m = (int)rank + (item / kGroups) * a.split;
            const uint32_t off = (uint32_t)(m * kTileRows + 4 * g) * 4u;
            float4 part[8], part2[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                part[k] = k < a.split ? ld_cluster_f32x4(peer[k] + off) : make_float4(0.f, 0.f, 0.f, 0.f);
                part2[k] = (kEpilogue == EPI_SWIGLU && k < a.split) ? ld_cluster_f32x4(peer[k] + off + 64u * 4u)
                                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 8; ++k) {       // cluster-rank order; absent ranks contribute +0
                acc[0] += part[k].x; acc[1] += part[k].y; acc[2] += part[k].z; acc[3] += part[k].w;
                acc2[0] += part2[k].x; acc2[1] += part2[k].y; acc2[2] += part2[k].z; acc2[3] += part2[k].w;
            }
            const int col = (kEpilogue == EPI_SWIGLU ? tile * 64 : tile * kTileRows) + 4 * g;
            const size_t o = (size_t)m * n_cols + col;
            uint32_t bits[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (kEpilogue == EPI_SWIGLU) {
                    // bf16(gate), bf16(up), bf16(silu(gate)), bf16(product): 17.cu:16396-16404
                    const float gv = round_bf16(acc[i]), u = round_bf16(acc2[i]);
                    const float act = round_bf16(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))));
                    bits[i] = f32_to_bf16_bits(__fmul_rn(act, u));
                } else {
                    // bf16(dot + bias), then bf16(residual + that): 17.cu:15297-15314
                    float v = acc[i];
                    if (a.bias[seg] && col + i < n_cols) v = __fadd_rn(v, bf16_bits_to_f32(a.bias[seg][col + i]));
                    bits[i] = f32_to_bf16_bits(v);
                    if (a.residual && col + i < n_cols)
                        bits[i] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(a.residual[o + i]), bf16_bits_to_f32(bits[i])));
                }
            }
            uint16_t* dst = (kEpilogue == EPI_SWIGLU ? a.out[0] : a.out[seg]) + o;
            if (col + 3 < n_cols && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(bits[0] | (bits[1] << 16), bits[2] | (bits[3] << 16));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (col + i < n_cols) dst[i] = (uint16_t)bits[i];
            }
        }
    }

    // Nobody leaves while a peer may still read its shared memory.  Only execution order matters here (every
    // remote read above has returned its value), so the arrival carries no release and does not wait for the
    // stores above to drain; the matching wait sits at the very end.
    cluster_arrive_relaxed();
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kMPad);
    }
    cluster_wait();
}

// ---- host side ----------------------------------------------------------------

// [rows][cols] bf16 row-major viewed as {cols, rows}; boxes of box_rows x 64 columns, 128-byte swizzle.
int32_t encode_matrix_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {kChunkCols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return qm_fail(QM_ECUDA, "cuTensorMapEncodeTiled failed for a projection operand");
    return QM_OK;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_cluster(void (*kernel)(KArgs...), unsigned grid, unsigned cluster, size_t smem, cudaStream_t stream,
                           Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = qm_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int sm_count_of_current_device() {
    static thread_local int cached_device = -1, cached_count = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    if (device != cached_device) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return 148;
        cached_device = device;
        cached_count = prop.multiProcessorCount;
    }
    return cached_count;
}

// Cluster size (K split): enough CTAs to occupy every SM about twice, at most 8, at least two chunks each.
int choose_split(int tiles, int chunks) {
#ifdef QM_DECODE_TUNING
    if (const char* forced = std::getenv("QM_GEMM_SPLIT")) {       // tuning builds only
        const int v = std::atoi(forced);
        if (v >= 1 && v <= 8 && chunks / v >= 1) return v;
    }
#endif
    const int target = 2 * sm_count_of_current_device();
    int split = target / (tiles > 0 ? tiles : 1);
    if (split < 1) split = 1;
    if (split > 8) split = 8;
    if (split == 3 || split == 5 || split == 6 || split == 7) split = split >= 4 ? 4 : 2;   // power-of-two clusters only
    while (split > 1 && chunks / split < 2) split >>= 1;
    // More CTAs than SMs with fewer than four chunks each is all fold and no streaming (the code predictor's fused
    // QKV: K = 1024, 32 tiles): halve the cluster there.
    while (split > 1 && chunks / split < 4 && tiles * split > target / 2) split >>= 1;
    return split;
}

struct Segment {
    const uint16_t* weight;
    const uint16_t* bias;
    uint16_t* out;
    int out_cols;
};

template <int kEpilogue>
int32_t run_gemm(const uint16_t* x, const Segment* segs, int n_segs, const uint16_t* up_weight, const uint16_t* residual,
                 int rows, int k_dim, uint32_t* status, cudaStream_t stream, const char* what) {
    if (!x) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (rows < 0 || rows > 64) return qm_fail(QM_ECAPACITY, "projection kernels take at most 64 token rows per call");
    if (k_dim < kChunkCols || k_dim % kChunkCols != 0)
        return qm_fail(QM_EINVAL, "reduction width must be a positive multiple of 64");
    uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(up_weight);
    for (int i = 0; i < n_segs; ++i) {
        if (!segs[i].weight || !segs[i].out || segs[i].out_cols < 1) return qm_fail(QM_EINVAL, "null tensor pointer");
        all |= reinterpret_cast<uintptr_t>(segs[i].weight);
    }
    if (kEpilogue == EPI_SWIGLU && !up_weight) return qm_fail(QM_EINVAL, "null tensor pointer");
    if (all & 15u) return qm_fail(QM_EINVAL, "projection operands must be 16-byte aligned");
    if (rows == 0) return QM_OK;
    const int m_pad = rows <= 32 ? 32 : 64;
    const int rows_per_tile = kEpilogue == EPI_SWIGLU ? 64 : kTileRows;
    CUtensorMap maps[3], x_map;
    GemmArgs a{};
    int tiles = 0;
    for (int i = 0; i < 3; ++i) {
        const Segment& sg = segs[i < n_segs ? i : n_segs - 1];
        const uint16_t* wptr = (kEpilogue == EPI_SWIGLU && i == 1) ? up_weight : sg.weight;
        int32_t rc = encode_matrix_map(&maps[i], wptr, (uint64_t)sg.out_cols, (uint64_t)k_dim, (uint32_t)rows_per_tile);
        if (rc != QM_OK) return rc;
        a.first_tile[i] = i < n_segs ? tiles : 0x7fffffff;
        a.weight[i] = wptr;
        if (i < n_segs) {
            a.bias[i] = sg.bias;
            a.out[i] = sg.out;
            a.out_cols[i] = sg.out_cols;
            tiles += (sg.out_cols + rows_per_tile - 1) / rows_per_tile;
        }
    }
    int32_t rc = encode_matrix_map(&x_map, x, (uint64_t)rows, (uint64_t)k_dim, (uint32_t)m_pad);
    if (rc != QM_OK) return rc;
    a.residual = residual;
    a.k_dim = k_dim;
    a.status = status;
    a.rows = rows;
    a.chunks = k_dim / kChunkCols;
    a.split = choose_split(tiles, a.chunks);
    const unsigned grid = (unsigned)(tiles * a.split);
    cudaError_t err;
    if (m_pad == 32) {
        auto kernel = qm_skinny_gemm_kernel<32, kEpilogue>;
        const size_t smem = GemmSmem<32>::kTotal + 1024;
        QM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), what);
        err = launch_cluster(kernel, grid, (unsigned)a.split, smem, stream, maps[0], maps[1], maps[2], x_map, a);
    } else {
        auto kernel = qm_skinny_gemm_kernel<64, kEpilogue>;
        const size_t smem = GemmSmem<64>::kTotal + 1024;
        QM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), what);
        err = launch_cluster(kernel, grid, (unsigned)a.split, smem, stream, maps[0], maps[1], maps[2], x_map, a);
    }
    QM_CUDA_TRY(err, what);
    return QM_OK;
}


// ---- many token rows (prefill): persistent 128 x 256 output tiles ------------------------------------------------
//
// Stands in for linear_bf16 / linear_warp32_bf16x2_f32acc_kernel (17.cu:142-289) as the prefill loop calls it
// through linear_generic (17.cu:16730-16860), with the residual add (launch_add) and the elementwise SwiGLU
// (swiglu_kernel, 17.cu:8771) of that loop folded into the epilogue at the same bf16 materialisation points.
//
// One CTA per SM walks output tiles of 128 token rows x 256 weight rows; per 64-column K chunk the TMA warp brings a
// 16 KB activation tile and a 32 KB weight tile (two 128-row boxes: consecutive weight rows, or 128 gate rows and
// the matching 128 up rows), the MMA thread issues four 128 x 256 x 16 tcgen05.mma into one of two 256-column
// TMEM accumulators, and the four epilogue warps drain the other accumulator meanwhile.
constexpr int kRowsBM = 128;
constexpr int kRowsBN = 256;
constexpr int kRowsStages = 4;
constexpr int kRowsThreads = 192;
constexpr int kRowsStageA = kRowsBM * kChunkCols * 2;      // 16 KB
constexpr int kRowsStageB = kRowsBN * kChunkCols * 2;      // 32 KB
constexpr int kRowsStageBytes = kRowsStageA + kRowsStageB;

struct RowsSmem {
    static constexpr int kRing = 0;
    static constexpr int kBars = kRowsStages * kRowsStageBytes;            // full[4], empty[4], acc_full[2], acc_empty[2]
    static constexpr int kTmemSlot = kBars + (2 * kRowsStages + 4) * 8;
    static constexpr int kTotal = kTmemSlot + 16;
};

struct RowsArgs {
    const uint16_t* bias;        // [n_cols] or null
    const uint16_t* residual;    // [rows][n_cols] or null
    uint16_t* out;               // [rows][n_cols]
    uint32_t* status;
    int rows;
    int n_cols;                  // output columns
    int k_chunks;
    int m_tiles;
    int n_tiles;
};

template <bool kSwiglu>
__global__ void __launch_bounds__(kRowsThreads, 1)
qm_rows_gemm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w0_map,
                    const __grid_constant__ CUtensorMap w1_map, const RowsArgs a) {
    constexpr int kColsPerTile = kSwiglu ? 128 : 256;
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_addr = smem_addr(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    unsigned char* smem = smem_raw + pad;
    const uint32_t sbase = raw_addr + pad;
    const uint32_t bar0 = sbase + RowsSmem::kBars;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kRowsStages + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * kRowsStages + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * kRowsStages + 2 + b); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + RowsSmem::kTmemSlot);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kRowsStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 128);
        }
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_addr(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const int total_tiles = a.m_tiles * a.n_tiles;
    bool dead = false;
    pdl_wait();

    if (warp == 5) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile / a.n_tiles) * kRowsBM;
                const int n0 = (tile % a.n_tiles) * kColsPerTile;
                for (int kc = 0; kc < a.k_chunks; ++kc, ++it) {
                    const int st = it % kRowsStages;
                    if (!mbar_wait_bounded(empty_bar(st), ((it / kRowsStages) & 1) ^ 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                    const uint32_t dst = sbase + RowsSmem::kRing + st * kRowsStageBytes;
                    mbar_arrive_expect_tx(full_bar(st), kRowsStageBytes);
                    tma_load_2d(dst, &x_map, full_bar(st), kc * kChunkCols, m0);
                    tma_load_2d(dst + kRowsStageA, &w0_map, full_bar(st), kc * kChunkCols, n0);
                    if (kSwiglu)
                        tma_load_2d(dst + kRowsStageA + kRowsStageB / 2, &w1_map, full_bar(st), kc * kChunkCols, n0);
                    else
                        tma_load_2d(dst + kRowsStageA + kRowsStageB / 2, &w0_map, full_bar(st), kc * kChunkCols, n0 + 128);
                }
            }
        }
        __syncwarp();
    } else if (warp == 4) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_instr_desc(kRowsBM, kRowsBN, false);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (!mbar_wait_bounded(acc_empty(buf), ((local >> 1) & 1) ^ 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                tc_fence_after();
                // The next stage's barrier is probed before this stage's MMAs are issued, so that the probe's
                // shared-memory round trip (about 190 cycles) overlaps the issue instead of draining the pipe.
                uint32_t seen = mbar_probe(full_bar(it % kRowsStages), (it / kRowsStages) & 1);
                for (int kc = 0; kc < a.k_chunks; ++kc, ++it) {
                    const int st = it % kRowsStages;
                    if (!mbar_wait_probed(seen, full_bar(st), (it / kRowsStages) & 1, dead)) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
                    seen = kc + 1 < a.k_chunks ? mbar_probe(full_bar((it + 1) % kRowsStages), ((it + 1) / kRowsStages) & 1) : 0u;
                    tc_fence_after();
                    const uint32_t xa = sbase + RowsSmem::kRing + st * kRowsStageBytes;
                    const uint32_t wa = xa + kRowsStageA;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        mma_ss(tmem_base + buf * 256, smem_desc(xa + ks * 32, 16, 1024), smem_desc(wa + ks * 32, 16, 1024), idesc,
                               (kc > 0 || ks > 0) ? 1u : 0u);
                    tc_commit(empty_bar(st));
                }
                tc_commit(acc_full(buf));
            }
        }
        __syncwarp();
    } else {
        const int row_in_tile = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile / a.n_tiles) * kRowsBM;
            const int n0 = (tile % a.n_tiles) * kColsPerTile;
            const int row = m0 + row_in_tile;
            if (!mbar_wait_bounded(acc_full(buf), (local >> 1) & 1, dead) && lane == 0) atomicOr(a.status, QM_DEVSTAT_TIMEOUT);
            tc_fence_after();
            const uint32_t taddr = tmem_base + lane_base + buf * 256;
#pragma unroll 1
            for (int c = 0; c < kColsPerTile / 32; ++c) {
                uint32_t acc[32], acc2[32];
                tmem_ld32(taddr + c * 32, acc);
                if (kSwiglu) tmem_ld32(taddr + 128 + c * 32, acc2);
                tmem_wait_ld();
                const int col = n0 + c * 32;
                if (row < a.rows && col < a.n_cols) {
                    const size_t o = (size_t)row * a.n_cols + col;
                    uint32_t packed[16];
                    if (kSwiglu) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            uint32_t bits[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                // bf16(gate), bf16(up), bf16(silu(gate)), bf16(product): 17.cu:8771-8800
                                const float gv = round_bf16(__uint_as_float(acc[i + h])), u = round_bf16(__uint_as_float(acc2[i + h]));
                                const float act = round_bf16(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))));
                                bits[h] = f32_to_bf16_bits(__fmul_rn(act, u));
                            }
                            packed[i >> 1] = bits[0] | (bits[1] << 16);
                        }
                    } else {
                        uint4 bias4[4] = {}, res4[4] = {};
                        if (a.bias)
#pragma unroll
                            for (int q = 0; q < 4; ++q) bias4[q] = __ldg(reinterpret_cast<const uint4*>(a.bias + col) + q);
                        if (a.residual)
#pragma unroll
                            for (int q = 0; q < 4; ++q) res4[q] = *(reinterpret_cast<const uint4*>(a.residual + o) + q);
                        const uint32_t* bias_w = reinterpret_cast<const uint32_t*>(bias4);
                        const uint32_t* res_w = reinterpret_cast<const uint32_t*>(res4);
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            uint32_t bits[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                // bf16(dot + bias), then bf16(residual + that): 17.cu:234-289 and launch_add
                                float v = __uint_as_float(acc[i + h]);
                                const uint32_t bw = (bias_w[i >> 1] >> (16 * h)) & 0xffffu;
                                if (a.bias) v = __fadd_rn(v, bf16_bits_to_f32((uint16_t)bw));
                                bits[h] = f32_to_bf16_bits(v);
                                if (a.residual) {
                                    const uint32_t rw = (res_w[i >> 1] >> (16 * h)) & 0xffffu;
                                    bits[h] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32((uint16_t)rw), bf16_bits_to_f32((uint16_t)bits[h])));
                                }
                            }
                            packed[i >> 1] = bits[0] | (bits[1] << 16);
                        }
                    }
                    uint4* dst = reinterpret_cast<uint4*>(a.out + o);
#pragma unroll
                    for (int q = 0; q < 4; ++q) dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty(buf));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <bool kSwiglu>
int32_t run_rows_gemm(const uint16_t* x, const uint16_t* w0, const uint16_t* w1, const uint16_t* bias, const uint16_t* residual,
                      uint16_t* out, int rows, int n_cols, int k_dim, uint32_t* status, cudaStream_t stream, const char* what) {
    if (rows < 0 || n_cols < 64 || n_cols % 64 != 0) return qm_fail(QM_EINVAL, "output width must be a positive multiple of 64");
    if (k_dim < kChunkCols || k_dim % kChunkCols != 0)
        return qm_fail(QM_EINVAL, "reduction width must be a positive multiple of 64");
    if (rows == 0) return QM_OK;                      // nothing to do; the row tensors may then be null
    if (!x || !w0 || !out || (kSwiglu && !w1)) return qm_fail(QM_EINVAL, "null tensor pointer");
    const uintptr_t all = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1) |
                          reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out);
    if (all & 15u) return qm_fail(QM_EINVAL, "projection operands must be 16-byte aligned");
    CUtensorMap x_map, w0_map, w1_map;
    int32_t rc = encode_matrix_map(&x_map, x, (uint64_t)rows, (uint64_t)k_dim, 128);
    if (rc != QM_OK) return rc;
    rc = encode_matrix_map(&w0_map, w0, (uint64_t)n_cols, (uint64_t)k_dim, 128);
    if (rc != QM_OK) return rc;
    rc = encode_matrix_map(&w1_map, kSwiglu ? w1 : w0, (uint64_t)n_cols, (uint64_t)k_dim, 128);
    if (rc != QM_OK) return rc;
    RowsArgs a{};
    a.bias = bias;
    a.residual = residual;
    a.out = out;
    a.status = status;
    a.rows = rows;
    a.n_cols = n_cols;
    a.k_chunks = k_dim / kChunkCols;
    a.m_tiles = (rows + kRowsBM - 1) / kRowsBM;
    const int cols_per_tile = kSwiglu ? 128 : 256;
    a.n_tiles = (n_cols + cols_per_tile - 1) / cols_per_tile;
    const long long tiles = (long long)a.m_tiles * a.n_tiles;
    if (tiles > 0x7fffffffLL) return qm_fail(QM_ECAPACITY, "too many output tiles for one launch");
    const int sms = sm_count_of_current_device();
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    auto kernel = qm_rows_gemm_kernel<kSwiglu>;
    const size_t smem = RowsSmem::kTotal + 1024;
    QM_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), what);
    QM_CUDA_TRY(qm_launch(kernel, dim3(grid), dim3(kRowsThreads), smem, stream, x_map, w0_map, w1_map, a), what);
    return QM_OK;
}

}  // namespace

extern "C" {

int32_t qm_linear(qm_kv_pool* pool, const uint16_t* x, const uint16_t* weight, const uint16_t* bias,
                  const uint16_t* residual, uint16_t* out, int32_t rows, int32_t out_features, int32_t in_features,
                  void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    const Segment seg{weight, bias, out, out_features};
    return run_gemm<EPI_LINEAR>(x, &seg, 1, nullptr, residual, rows, in_features, pool->status_dev,
                                static_cast<cudaStream_t>(stream), "projection launch");
}

int32_t qm_qkv_linear(qm_kv_pool* pool, const uint16_t* x, const uint16_t* q_weight, const uint16_t* q_bias,
                      const uint16_t* k_weight, const uint16_t* k_bias, const uint16_t* v_weight, const uint16_t* v_bias,
                      uint16_t* q_out, uint16_t* k_out, uint16_t* v_out, int32_t rows, int32_t hidden, int32_t q_dim,
                      int32_t kv_dim, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    const Segment segs[3] = {{q_weight, q_bias, q_out, q_dim}, {k_weight, k_bias, k_out, kv_dim}, {v_weight, v_bias, v_out, kv_dim}};
    return run_gemm<EPI_LINEAR>(x, segs, 3, nullptr, nullptr, rows, hidden, pool->status_dev, static_cast<cudaStream_t>(stream),
                                "fused QKV projection launch");
}

int32_t qm_gate_up_swiglu(qm_kv_pool* pool, const uint16_t* x, const uint16_t* gate_weight, const uint16_t* up_weight,
                          uint16_t* out, int32_t rows, int32_t hidden, int32_t intermediate, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    const Segment seg{gate_weight, nullptr, out, intermediate};
    return run_gemm<EPI_SWIGLU>(x, &seg, 1, up_weight, nullptr, rows, hidden, pool->status_dev,
                                static_cast<cudaStream_t>(stream), "fused gate/up/SwiGLU launch");
}

int32_t qm_linear_rows(qm_kv_pool* pool, const uint16_t* x, const uint16_t* weight, const uint16_t* bias,
                       const uint16_t* residual, uint16_t* out, int32_t rows, int32_t out_features, int32_t in_features,
                       void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    return run_rows_gemm<false>(x, weight, nullptr, bias, residual, out, rows, out_features, in_features, pool->status_dev,
                                static_cast<cudaStream_t>(stream), "many-row projection launch");
}

int32_t qm_gate_up_swiglu_rows(qm_kv_pool* pool, const uint16_t* x, const uint16_t* gate_weight, const uint16_t* up_weight,
                               uint16_t* out, int32_t rows, int32_t hidden, int32_t intermediate, void* stream) {
    if (!pool) return qm_fail(QM_EINVAL, "pool is null");
    return run_rows_gemm<true>(x, gate_weight, up_weight, nullptr, nullptr, out, rows, intermediate, hidden, pool->status_dev,
                               static_cast<cudaStream_t>(stream), "many-row gate/up/SwiGLU launch");
}

}  // extern "C"
