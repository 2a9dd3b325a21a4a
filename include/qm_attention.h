/*
 * qm_attention.h - C ABI of the B200 (sm_100a) talker attention path.
 *
 * The reference engine (abouya9854/qingming-qwen3-tts) has no FFI: its boundary
 * for this path is the set of private launcher methods of NativeTalkerEngine
 * in devices/rtx4090-24g/qwen3_tts_1_7b.cu ("17.cu" below).  Every entry point
 * here names the launcher (file:line) it stands in for.
 *
 * Conventions (same as the reference's kernels, 17.cu:15414-15423):
 *   - bf16 tensors are `uint16_t*` DEVICE pointers; activations are laid out
 *     [tokens][heads][128]; norm weights are [128].
 *   - int arrays (positions, seq_lens, cu_seqlens, page_table) are `int32_t*`
 *     DEVICE pointers.
 *   - `stream` is a cudaStream_t passed as void*; every launch goes to it and
 *     nothing is synchronised unless the comment says so.
 *   - no function throws; each returns QM_OK (0) or a negative status, and
 *     qm_last_error_string() describes the last failure on the calling thread.
 *   - handles are thread-compatible: one caller at a time per handle.
 *
 * KV cache layout (replaces the per-layer contiguous [kv_head][max_cache][128]
 * caches of LayerCache, 17.cu:16419-16438): per layer one K pool and one V pool
 *     pool[page][kv_head][64][128]  bf16
 * so that one (page, kv_head) tile is 16 KB contiguous.  Token t of stream s
 * lives at page = page_table[s * max_pages + (t >> 6)], slot = t & 63.  K is
 * stored after RMSNorm and RoPE, V raw (17.cu:15553-15572).
 */
#ifndef QM_ATTENTION_H
#define QM_ATTENTION_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QM_OK 0
#define QM_EINVAL (-1)     /* bad argument, detected before any launch          */
#define QM_ECAPACITY (-2)  /* position/page beyond the pool ("cache overflow", 17.cu:17204) */
#define QM_ECUDA (-3)      /* a CUDA runtime call or launch failed               */
#define QM_ETIMEOUT (-4)   /* a bounded device-side wait gave up                 */
#define QM_ENOMEM (-5)     /* device allocation failed                           */
#define QM_EDEVICE (-6)    /* not a compute-capability 10.x device               */
#define QM_ENCCL (-7)      /* an NCCL call failed or reported an asynchronous error (communicator aborted) */

#define QM_HEAD_DIM 128
#define QM_PAGE_TOKENS 64

/* Device status bits written by kernels into the pool's status word. */
#define QM_DEVSTAT_BAD_PAGE 1u   /* page id outside the pool, access skipped     */
#define QM_DEVSTAT_BAD_POS 2u    /* position beyond max_pages * 64, skipped      */
#define QM_DEVSTAT_TIMEOUT 4u    /* bounded mbarrier wait expired                */

typedef struct qm_kv_pool qm_kv_pool;

/* Text for the last non-zero status returned on this thread.  Stands in for the
 * std::runtime_error text built by cuda_check (17.cu:17440-17453). */
const char* qm_last_error_string(void);

/* Replaces validate_rtx4090_24g_device (17.cu:7769-7804): requires compute
 * capability 10.x and 32-wide warps; the SM count is read, not fixed.
 * Optionally returns the SM count. */
int32_t qm_validate_b200_device(int32_t device, int32_t* sm_count_out);

/* ---- KV pool: LayerCache + allocation loop (17.cu:16419-16438, :16506-16533) */

/* Allocates zero-filled K and V pools for `layers` layers of `num_pages` pages
 * on the current device.  kv_heads in 1..64. */
int32_t qm_kv_pool_create(int32_t layers, int32_t num_pages, int32_t kv_heads, qm_kv_pool** pool_out);
int32_t qm_kv_pool_destroy(qm_kv_pool* pool);

/* reset_request (17.cu:16607-16629): zero every page of every layer on
 * `stream`, then synchronise that stream, as the reference does. */
int32_t qm_kv_pool_reset(qm_kv_pool* pool, void* stream);

/* Device pointers of one layer's pools (for tests and for callers that fill
 * or snapshot the cache themselves) and the pool geometry. */
uint16_t* qm_kv_pool_key_ptr(qm_kv_pool* pool, int32_t layer);
uint16_t* qm_kv_pool_value_ptr(qm_kv_pool* pool, int32_t layer);
int32_t qm_kv_pool_num_pages(const qm_kv_pool* pool);
int32_t qm_kv_pool_kv_heads(const qm_kv_pool* pool);

/* Reads and clears the device status word (QM_DEVSTAT_* bits) after
 * synchronising `stream`.  Returns QM_OK and the bits through *bits_out. */
int32_t qm_kv_pool_status(qm_kv_pool* pool, void* stream, uint32_t* bits_out);

/* Diagnostic, no counterpart in the reference (whose kernels never wait on one
 * another): launches one small kernel that waits, with the same bounded wait
 * the attention kernels use, for a signal that is never sent.  After about a
 * second the wait gives up, QM_DEVSTAT_TIMEOUT appears in the status word and
 * the kernel returns normally; the device stays usable. */
int32_t qm_selftest_wait_timeout(qm_kv_pool* pool, void* stream);

/* ---- RoPE table: make_talker_rope (17.cu:21758-21772) */

/* Fills DEVICE arrays cosine/sine [rows][128] bf16 for positions
 * start .. start+rows-1 with the reference's double-precision recipe.  The
 * values are computed on the host and copied on `stream` (synchronised before
 * return).  The reference uploads one row per decode step (17.cu:17221-17239);
 * here the table is built once and indexed by position. */
int32_t qm_rope_table_fill(uint16_t* cosine_dev, uint16_t* sine_dev, int32_t rows, int32_t start, double theta,
                           void* stream);

/* ---- fused QK-RMSNorm + RoPE + paged append */

/* Decode step for `batch` independent streams: launch_qk_norm_rope_cache_m1
 * (17.cu:17741-17778; kernel :15412-15574), batched and paged.
 *   q [batch][q_heads][128], k, v [batch][kv_heads][128]  pre-norm projections
 *   positions[batch]: position of the new token of each stream (the
 *     reference's scalar cache_position)
 *   rope_cos / rope_sin [rope_rows][128], row index = position
 *   q_rot [batch][q_heads][128] receives normed+roped queries
 * K (normed, roped) and V (raw) are written to the pool at (page, slot) of
 * each position.  A position beyond max_pages*64 or a page id outside the pool
 * sets a status bit and skips that row's cache write. */
int32_t qm_decode_append_rope(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                              const uint16_t* v, const uint16_t* q_norm_weight, const uint16_t* k_norm_weight,
                              const uint16_t* rope_cos, const uint16_t* rope_sin, int32_t rope_rows,
                              const int32_t* positions, const int32_t* page_table, int32_t max_pages,
                              int32_t batch, int32_t q_heads, float epsilon, uint16_t* q_rot, void* stream);

/* The same decode step when this pool holds only a slice of each stream (a very
 * long context split across GPUs): launch_qk_norm_rope_cache_m1 (17.cu:17741)
 * with the RoPE row and the cache slot given separately.  positions[batch] is
 * the absolute position (RoPE row); cache_positions[batch] is the slot index
 * inside THIS pool's slice, or -1 on a rank that does not own the new token
 * (q_rot is still produced, K/V are not written). */
int32_t qm_decode_append_rope_sliced(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                                     const uint16_t* v, const uint16_t* q_norm_weight,
                                     const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                                     const uint16_t* rope_sin, int32_t rope_rows, const int32_t* positions,
                                     const int32_t* cache_positions, const int32_t* page_table,
                                     int32_t max_pages, int32_t batch, int32_t q_heads, float epsilon,
                                     uint16_t* q_rot, void* stream);

/* Prefill, packed varlen: the launch_rmsnorm x2 + launch_rope_rows x2 +
 * scatter_prefill_cache sequence of prefill() (17.cu:16763-16798) in one
 * kernel.  Sequence s owns packed rows cu_seqlens[s] .. cu_seqlens[s+1]-1 and
 * its first row has position start_positions[s] (NULL = all zero, as in the
 * reference where prefill starts an empty cache).  total_tokens is
 * cu_seqlens[batch] as known to the host. */
int32_t qm_prefill_append_rope_varlen(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k,
                                      const uint16_t* v, const uint16_t* q_norm_weight,
                                      const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                                      const uint16_t* rope_sin, int32_t rope_rows, const int32_t* cu_seqlens,
                                      const int32_t* start_positions, const int32_t* page_table,
                                      int32_t max_pages, int32_t batch, int32_t total_tokens, int32_t q_heads,
                                      float epsilon, uint16_t* q_rot, void* stream);

/* ---- decode attention: launch_attention with query_length == 1
 *      (17.cu:17895-17952; kernel talker_attention_gqa2_m1_locality_kernel :16061-16251) */

/* Bytes of caller-owned scratch qm_decode_attention needs for a batch. */
int64_t qm_decode_workspace_bytes(int32_t batch, int32_t kv_heads);

/* Zero-fills a freshly allocated workspace on `stream` (the reference clears
 * its buffers the same way when it creates them, 17.cu:16419-16438).  Call it
 * once after allocating: the per-segment arrival counters inside must start
 * at zero; every call leaves them at zero again.  Call it again after a call
 * that reported QM_DEVSTAT_TIMEOUT. */
int32_t qm_decode_workspace_init(void* workspace, int64_t workspace_bytes, void* stream);

/* Split-KV flash decoding over the paged cache, q_heads == 2 * kv_heads.
 *   q_rot [batch][q_heads][128]: output of qm_decode_append_rope
 *   seq_lens[batch]: number of keys each stream attends, i.e. position + 1
 *     (the appended token is included, 17.cu:16080); 0 gives a zero row
 *   out [batch][q_heads][128] bf16, the reference's `context`
 * Softmax scale is 1/sqrtf(128) (17.cu:17910-17914).  Scores, softmax and the
 * PV sum stay in fp32; the result is rounded to bf16 once.  Deterministic:
 * the split of keys over CTAs depends only on seq_lens and the SM count, and
 * partial results are always folded in the same order.  `workspace` must have
 * been prepared once with qm_decode_workspace_init and must not be shared by
 * calls that overlap on the GPU. */
int32_t qm_decode_attention(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* seq_lens,
                            const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                            uint16_t* out, void* workspace, int64_t workspace_bytes, void* stream);

/* The whole decode step of one layer in ONE launch: launch_qk_norm_rope_cache_m1
 * (17.cu:17741) followed by launch_attention (17.cu:17895), as decode_device
 * issues them (17.cu:17284-17309).  Inputs are those of qm_decode_append_rope
 * (raw q, k, v projections, norm weights, RoPE table, positions); every stream
 * attends positions[s] + 1 keys.  QK-RMSNorm and RoPE are applied as q and the
 * new k row are loaded; the new K (normed, roped) and V (raw) rows are written
 * to the pool for later steps and used from shared memory in this one.  The
 * bits written to the pool and the context equal those of the two separate
 * calls.  No q_rot buffer is produced. */
int32_t qm_decode_step(qm_kv_pool* pool, int32_t layer, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                       const uint16_t* q_norm_weight, const uint16_t* k_norm_weight, const uint16_t* rope_cos,
                       const uint16_t* rope_sin, int32_t rope_rows, const int32_t* positions,
                       const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads, float epsilon,
                       uint16_t* out, void* workspace, int64_t workspace_bytes, void* stream);

/* Decode attention without any allocation, here or in the caller.  No counterpart
 * in the reference, whose engine allocates all workspace at construction.
 * Same inputs, outputs and result as qm_decode_attention, but the scratch
 * lives in a fixed array inside the library (about 1.7 MB of device memory on
 * every GPU that loads the library, held until the process exits).  Meant for
 * hosts that cannot cudaMalloc on this path: a resident serving loop whose
 * device memory was budgeted at start-up and whose second stream (the codec
 * decoder) would be stalled by the device-wide synchronisation an allocation
 * implies, or an engine whose own allocator already holds all device memory.
 *   - at most 64 streams and 8 KV heads per call; more returns QM_ECAPACITY.
 *   - the pool's device must be the current device on every call (QM_EINVAL
 *     otherwise); the first call on each device looks up the array's device
 *     address: make that first call before starting any stream capture.
 *   - all calls on a device share the one array and it keeps what the last
 *     call wrote; it starts zeroed and the kernel re-zeroes the counters it
 *     uses, so nothing needs clearing between calls, but two calls
 *     whose kernels overlap on the GPU (different streams, or several
 *     threads) would overwrite each other's partials: issue them on one
 *     stream, or order them with events.
 *   - a call after which qm_kv_pool_status shows QM_DEVSTAT_TIMEOUT may have
 *     left arrival counters behind in the array: call
 *     qm_decode_static_scratch_reset before the next one.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
int32_t qm_decode_attention_static(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                   const int32_t* seq_lens, const int32_t* page_table, int32_t max_pages,
                                   int32_t batch, int32_t q_heads, uint16_t* out, void* stream);

/* Puts the arrival counters of the library's built-in scratch back to zero on
 * `stream` (a memset on memory that already exists; allocates nothing).  No
 * counterpart in the reference.  Needed only after a qm_decode_attention_static
 * call that reported QM_DEVSTAT_TIMEOUT; the pool's device must be current. */
int32_t qm_decode_static_scratch_reset(qm_kv_pool* pool, void* stream);

/* Same, but stops before normalisation and returns the partial softmax state
 * of each (stream, query head) over the keys held in THIS pool:
 *   partial [batch][q_heads][130] fp32 = { m (max scaled score, natural-log
 *   domain), l (sum of exp(s - m)), o[128] (unnormalised) }.
 * Used when one stream's keys are split over several GPUs: each GPU calls this
 * on its slice, the partials are exchanged (33 280 B per rank for 4 streams),
 * and qm_attention_combine finishes.  A stream with seq_len 0 yields
 * m = -inf, l = 0, o = 0. */
int32_t qm_decode_attention_partial(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                    const int32_t* seq_lens, const int32_t* page_table, int32_t max_pages,
                                    int32_t batch, int32_t q_heads, float* partial, void* workspace,
                                    int64_t workspace_bytes, void* stream);

/* Log-sum-exp combine of `parts` partial states per row:
 *   partials [parts][rows][130] fp32, out [rows][128] bf16,
 *   out = sum_g e^{m_g - M} o_g / sum_g e^{m_g - M} l_g,  M = max_g m_g.
 * Parts are folded in index order, so the result does not depend on timing. */
int32_t qm_attention_combine(const float* partials, int32_t parts, int32_t rows, uint16_t* out, void* stream);

/* Exchange + combine in one kernel over peer memory, for streams whose keys are split across the GPUs of one box.
 * No counterpart in the reference (single GPU).  Every rank calls it at the same point of its stream with its own
 * partials (from qm_decode_attention_partial) and the same `rows`; the kernel stores them into every rank's exchange
 * buffer with plain peer-to-peer stores, waits - bounded, QM_DEVSTAT_TIMEOUT if a rank never shows up - until all
 * ranks' copies of each row of this call have arrived in its own buffer, and folds them in rank order into
 * out [rows][128] bf16 (the order and arithmetic of qm_attention_combine: every rank ends with the same bits).
 *   peer_buffers_dev: DEVICE array of `world` pointers, entry r = rank r's exchange buffer mapped into this
 *     process (symmetric / IPC / peer-enabled memory), each of qm_exchange_buffer_bytes(world, rows_capacity) bytes,
 *     zero-filled once when allocated and never touched by the host afterwards.
 * The call number lives in the buffer (one counter per row, advanced by the kernel), so consecutive calls need no
 * host-side bookkeeping, `rows` may differ from call to call (as long as every rank passes the same value), and a
 * launch captured in a CUDA graph can be replayed.  After a call that reported QM_DEVSTAT_TIMEOUT the ranks'
 * counters may disagree: zero every rank's buffer again (all ranks, with a host barrier) before the next call.
 * rows beyond what the GPU can hold resident at once (about 1 700 on B200) are rejected with QM_ECAPACITY. */
int64_t qm_exchange_buffer_bytes(int32_t world, int32_t rows_capacity);
int32_t qm_attention_exchange_combine(qm_kv_pool* pool, const float* local_partials, void* const* peer_buffers_dev,
                                      int32_t world, int32_t rank, int32_t rows, int32_t rows_capacity, uint16_t* out,
                                      void* stream);

/* The split-KV kernel and the exchange in ONE launch, for the same streams-split-across-GPUs case.  No counterpart in
 * the reference.  Same inputs as qm_decode_attention_partial (this pool holds a slice of every stream,
 * local_seq_lens[s] of its keys; 0 is fine) and the same exchange buffers as qm_attention_exchange_combine.  The CTA
 * that finishes a (stream, KV head) segment of this rank holds its two rows' partial state in registers: it stores
 * them straight into every rank's exchange buffer, waits (bounded, QM_DEVSTAT_TIMEOUT) for the same two rows from
 * every other rank and folds them in rank order into out [batch][q_heads][128] - no partial buffer, no second
 * launch, and the NVLink round trip of the early segments overlaps the streaming of the late ones.  Bits equal
 * qm_decode_attention_partial + qm_attention_exchange_combine (and + all-gather + qm_attention_combine).  Every
 * rank calls it at the same point of its stream with the same batch; batch * q_heads <= rows_capacity, batch <= 256.
 * The two exchange entry points may be mixed freely on one set of buffers. */
int32_t qm_decode_attention_exchange(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* local_seq_lens,
                                     const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                                     uint16_t* out, void* const* peer_buffers_dev, int32_t world, int32_t rank,
                                     int32_t rows_capacity, void* workspace, int64_t workspace_bytes, void* stream);

/* The exchange buffers as an object, for hosts that have no symmetric-memory allocator of their own.  No counterpart
 * in the reference.  qm_exchange_create allocates and zeroes this rank's buffer on the current device.  With one
 * process per GPU, every rank exports its buffer with qm_exchange_ipc_handle (QM_IPC_HANDLE_BYTES bytes, a CUDA IPC
 * memory handle), the host passes the handles around by whatever channel it has, and qm_exchange_open_peers maps
 * the others (`handles` = world consecutive handles in rank order; the own entry is ignored).  With one process
 * driving several GPUs, qm_exchange_set_peers takes the other ranks' qm_exchange_local_buffer pointers instead
 * (peer access between the devices must be enabled by the host).  qm_exchange_combine is
 * qm_attention_exchange_combine on these buffers.  qm_exchange_reset zeroes this rank's buffer on `stream` (after
 * a timeout; every rank, then a host barrier).  Creation, mapping and destruction allocate and synchronise;
 * qm_exchange_combine does neither. */
#define QM_IPC_HANDLE_BYTES 64
typedef struct qm_exchange qm_exchange;
int32_t qm_exchange_create(int32_t world, int32_t rank, int32_t rows_capacity, qm_exchange** exchange_out);
int32_t qm_exchange_destroy(qm_exchange* exchange);
void* qm_exchange_local_buffer(qm_exchange* exchange);
int32_t qm_exchange_ipc_handle(qm_exchange* exchange, void* handle_out);
int32_t qm_exchange_open_peers(qm_exchange* exchange, const void* handles);
int32_t qm_exchange_set_peers(qm_exchange* exchange, void* const* peer_buffers);
int32_t qm_exchange_reset(qm_exchange* exchange, void* stream);
int32_t qm_exchange_combine(qm_kv_pool* pool, qm_exchange* exchange, const float* local_partials, int32_t rows,
                            uint16_t* out, void* stream);
/* qm_decode_attention_exchange on these buffers. */
int32_t qm_exchange_decode_attention(qm_kv_pool* pool, qm_exchange* exchange, int32_t layer, const uint16_t* q_rot,
                                     const int32_t* local_seq_lens, const int32_t* page_table, int32_t max_pages,
                                     int32_t batch, int32_t q_heads, uint16_t* out, void* workspace, int64_t workspace_bytes,
                                     void* stream);

/* ---- the same exchange through NCCL, for a C++ host with one process or thread per GPU ----
 * No counterpart in the reference (single GPU; its launch_attention, 17.cu:17895, sees the whole cache). */

/* One layer of decode attention when this pool holds a slice of every stream: the split-KV kernel over the local
 * keys (qm_decode_attention_partial), ONE ncclAllGather of the [batch][q_heads][130] fp32 partials on `stream`,
 * and the rank-order combine, so every rank ends with the same bits in out [batch][q_heads][128].
 *   local_seq_lens[batch]: keys of each stream held in THIS pool (0 is fine)
 *   partial_send [batch][q_heads][130] fp32, partial_recv [world][batch][q_heads][130] fp32: caller-owned device
 *     buffers (registering them with NCCL is the caller's choice)
 *   nccl_comm: the caller's ncclComm_t of `world` ranks; every rank makes the call.
 * Nothing here allocates or synchronises.  A failed NCCL call returns QM_ENCCL.  A collective that never completes
 * (a rank that died) is detected by qm_nccl_wait, not here. */
int32_t qm_decode_attention_sharded(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot, const int32_t* local_seq_lens,
                                    const int32_t* page_table, int32_t max_pages, int32_t batch, int32_t q_heads,
                                    uint16_t* out, float* partial_send, float* partial_recv, int32_t world,
                                    void* workspace, int64_t workspace_bytes, void* nccl_comm, void* stream);

/* Host-side deadline for the collectives queued on `stream`: polls the stream and ncclCommGetAsyncError until the
 * stream's work is done (QM_OK), NCCL reports an asynchronous error (ncclCommAbort, then QM_ENCCL), the stream
 * itself fails (abort, QM_ECUDA) or `deadline_ms` passes (abort, QM_ETIMEOUT).  After anything but QM_OK the
 * communicator is gone and must be rebuilt by the host. */
int32_t qm_nccl_wait(void* nccl_comm, void* stream, int32_t deadline_ms);

/* The NCCL functions used above.  By default they are resolved at first use from libnccl.so.2 (or the file named
 * by the environment variable QM_NCCL_LIBRARY); a host that links NCCL itself, or a test that wants to stand in
 * for it, passes its own table.  Result codes are NCCL's (0 = ncclSuccess, 7 = ncclInProgress); stream_query
 * returns 0 when the stream has finished, 1 while it is busy, a negative value on error (NULL = cudaStreamQuery).
 * qm_nccl_set_api(NULL) goes back to the shared library. */
typedef struct qm_nccl_api {
    int (*all_gather)(const void* send, void* recv, size_t send_count, int datatype, void* comm, void* stream);
    int (*comm_get_async_error)(void* comm, int* async_error);
    int (*comm_abort)(void* comm);
    int (*comm_count)(const void* comm, int* count);
    const char* (*get_error_string)(int result);
    int (*stream_query)(void* stream);
} qm_nccl_api;
int32_t qm_nccl_set_api(const qm_nccl_api* api);

/* Convenience for hosts without NCCL plumbing of their own: ncclGetUniqueId (128 bytes), ncclCommInitRank and
 * ncclCommDestroy through the same lazily loaded library. */
int32_t qm_nccl_unique_id(void* id_out);
int32_t qm_nccl_comm_init_rank(void** comm_out, int32_t world, const void* id, int32_t rank);
int32_t qm_nccl_comm_destroy(void* comm);

/* ---- prefill attention: launch_attention with query_length > 1
 *      (17.cu:17954-17985; kernel talker_attention_kernel :15791-16054) */

/* Causal GQA attention over packed varlen queries whose keys are already in
 * the paged cache (the reference also attends over the cache it has just
 * scattered, 17.cu:16791-16807).  Row i of sequence s (position
 * start_positions[s] + i) attends keys 0 .. start_positions[s] + i.
 *   q_rot, out [total_tokens][q_heads][128] bf16
 * max_seqlen: the longest sequence, as known to the host (sizes the grid).
 * tcgen05 tensor-core kernel with TMEM accumulators; fp32 softmax. */
int32_t qm_prefill_attention_varlen(qm_kv_pool* pool, int32_t layer, const uint16_t* q_rot,
                                    const int32_t* cu_seqlens, const int32_t* start_positions,
                                    const int32_t* page_table, int32_t max_pages, int32_t batch,
                                    int32_t total_tokens, int32_t max_seqlen, int32_t q_heads, uint16_t* out,
                                    void* stream);

/* ---- the rest of the talker decoder layer at decode time (batch of token rows) ----
 * The reference runs these for one token per launch; here `rows` token rows (at most 64 for the projections) go
 * through one launch.  All keep the reference's bf16 materialisation points.  `pool` supplies the device status
 * word that bounded waits report into. */

/* Row RMSNorm: code_predictor::rmsnorm_kernel via launch_rmsnorm (17.cu:8295-8357, :8927); input and final norm
 * of decode_device (17.cu:17259, :17389).  out = bf16(bf16(x * inv_rms) * weight), bit-identical reduction order. */
int32_t qm_rmsnorm(const uint16_t* x, const uint16_t* weight, uint16_t* out, int32_t rows, int32_t dim, float epsilon,
                   void* stream);

/* launch_add_postnorm_m1 (17.cu:17989; kernel :16258-16343): residual = bf16(hidden + attention),
 * normalized = RMSNorm(residual) with `weight`. */
int32_t qm_add_postnorm(const uint16_t* hidden, const uint16_t* attention, const uint16_t* weight, uint16_t* residual,
                        uint16_t* normalized, int32_t rows, int32_t dim, float epsilon, void* stream);

/* launch_linear_m1 / launch_qkv_m1 (17.cu:17646, :17691; kernels :15250-15407):
 * out[r][n] = bf16(dot(x[r], weight[n]) + bias[n]); with `residual`, bf16(residual[r][n] + that value).
 * weight is [out_features][in_features] row-major (q, k and v weights stacked for the fused QKV call);
 * in_features must be a multiple of 64; bias and residual may be NULL.  tcgen05 kernel, fp32 accumulation. */
int32_t qm_linear(qm_kv_pool* pool, const uint16_t* x, const uint16_t* weight, const uint16_t* bias,
                  const uint16_t* residual, uint16_t* out, int32_t rows, int32_t out_features, int32_t in_features,
                  void* stream);

/* launch_qkv_m1 (17.cu:17691; kernel talker_qkv_fused_kernel :15321-15407): the three projections of the
 * normalised hidden rows in one launch, each with its own weight [dim][hidden], optional bias and output tensor
 * (q_out [rows][q_dim], k_out / v_out [rows][kv_dim]) - the layouts qm_decode_step takes. */
int32_t qm_qkv_linear(qm_kv_pool* pool, const uint16_t* x, const uint16_t* q_weight, const uint16_t* q_bias,
                      const uint16_t* k_weight, const uint16_t* k_bias, const uint16_t* v_weight, const uint16_t* v_bias,
                      uint16_t* q_out, uint16_t* k_out, uint16_t* v_out, int32_t rows, int32_t hidden, int32_t q_dim,
                      int32_t kv_dim, void* stream);

/* launch_gate_up_swiglu_m1 (17.cu:18020; kernel :16348-16416):
 * out[r][c] = bf16( bf16(silu(bf16(gate))) * bf16(up) ), gate = dot(x[r], gate_weight[c]), up likewise. */
int32_t qm_gate_up_swiglu(qm_kv_pool* pool, const uint16_t* x, const uint16_t* gate_weight, const uint16_t* up_weight,
                          uint16_t* out, int32_t rows, int32_t hidden, int32_t intermediate, void* stream);

/* ---- the same projections for many token rows at once (prefill) ----
 * linear_bf16 as the prefill loop calls it through linear_generic (17.cu:142-289; call sites :16730-16860), any
 * number of rows: out[r][n] = bf16(dot(x[r], weight[n]) + bias[n]); with `residual` (the loop's launch_add),
 * bf16(residual[r][n] + that value).  out_features and in_features multiples of 64; bias and residual may be NULL.
 * Persistent tcgen05 kernel, 128 x 256 tiles, fp32 accumulation in TMEM. */
int32_t qm_linear_rows(qm_kv_pool* pool, const uint16_t* x, const uint16_t* weight, const uint16_t* bias,
                       const uint16_t* residual, uint16_t* out, int32_t rows, int32_t out_features, int32_t in_features,
                       void* stream);

/* The prefill loop's two linear_generic calls on post_norm_ (gate, up) and its swiglu_kernel (17.cu:8771-8800,
 * call sites :16833-16860) in one launch: out[r][c] = bf16( bf16(silu(bf16(gate))) * bf16(up) ). */
int32_t qm_gate_up_swiglu_rows(qm_kv_pool* pool, const uint16_t* x, const uint16_t* gate_weight, const uint16_t* up_weight,
                               uint16_t* out, int32_t rows, int32_t hidden, int32_t intermediate, void* stream);

/* ---- the end of a decode step: codec-head logits -> next code, and the embedding rows of the next step ---- */

#define QM_SAMPLE_REPETITION 1   /* repetition penalty 1.05 over the stream's history (17.cu:14063-14099)     */
#define QM_SAMPLE_SUPPRESS 2     /* EOS forbidden for generation_index < 2, reserved ids forbidden (:14102-14123) */
#define QM_SAMPLE_RECORD 4       /* history[generation_index] = code (record_sampled_code_kernel, :7668-7689) */

/* NativeFinalHead::run_fast / run_fast_device after the head projection (17.cu:14384-14560), for `batch` streams in
 * one launch: scores = float(logits) (cast_final_head_logits :14052), then the processors selected by `flags`, then
 *   top_k <= 0: argmax_final_head (:14126-14176) - highest score, lowest index among equals;
 *   top_k  > 0: gpu_sample_topk_f32_kernel (:7546-7600) - the top_k best by (score desc, index asc), weights
 *               exp((score - best) / temperature) in double, one SplitMix64 draw from rng_state[stream].
 * logits [batch][vocab] bf16, vocab <= 4096; history [batch][history_capacity] int32 holds the codes generated so
 * far, generation_index[stream] of them; codes_out [batch]; processed_out [batch][vocab] float receives the processed
 * scores when not NULL (what the reference's FinalHeadTrace keeps).  The reference passes eos_token 2150 and
 * reserved_begin vocab - 1024.  Everything stays on the device: nothing here synchronises or copies to the host. */
int32_t qm_final_head_sample(qm_kv_pool* pool, const uint16_t* logits, int32_t batch, int32_t vocab, int32_t* history,
                             int32_t history_capacity, const int32_t* generation_index, int32_t flags,
                             int32_t eos_token, int32_t reserved_begin, int32_t top_k, float temperature,
                             uint64_t* rng_state, int32_t* codes_out, float* processed_out, void* stream);

/* gather_embedding_kernel (17.cu:8875-8893) for a batch of rows: out[r][:] = table[token_ids[r]][:].
 * table [vocab][hidden] bf16, hidden a multiple of 8; an id outside the table is clamped and reported in the
 * pool's status word (QM_DEVSTAT_BAD_POS). */
int32_t qm_embedding_gather(qm_kv_pool* pool, const uint16_t* table, const int32_t* token_ids, int32_t rows,
                            int32_t vocab, int32_t hidden, uint16_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QM_ATTENTION_H */
