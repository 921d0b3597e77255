/* q27b_attn: B200 (sm_100a) attention hot path for qwen27-engine, C ABI.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (passed as
 * void*, it is a cudaStream_t / CUstream). Work is enqueued on that stream on the device that
 * is current at call time; nothing synchronises with the host. All entry points return a
 * status code (0 = ok); q27b_last_error() gives the text of the last failure on the calling
 * thread. No exception crosses this boundary.
 *
 * Each declaration names the interface of the reference engine that it replaces
 * (file:line in avallavall/qwen27-engine).
 *
 * Fixed model constants (reference src/attn.cu:22-28): head dim 256, 6 query heads per KV
 * head, at most 4 query tokens per decode call.
 *
 * Memory: the caller owns every buffer that it passes. The library keeps a workspace per device
 * (see q27b_attn_workspace_*): a status word, the decode partials (fixed size, allocated by the
 * first decode call), the prefill partials (allocated once, by the first prefill call that splits,
 * at a fixed cap - a later, deeper call splits less instead of reallocating, as the reference's
 * fixed buffer, src/attn.cu:954-959) and the partials of the batched paged decode (grow with the
 * batch). Run every shape class once before capturing a CUDA graph (the reference's
 * Decoder::warmup does the same, src/model.cu:910-931), or fix everything up front with
 * q27b_attn_workspace_init.
 * Threading: one caller thread per device at a time (as the reference, src/attn.cu:869-879);
 * different devices may be driven from different threads (the process-wide state - tensor-map
 * cache, kernel choices, one-time set-up - is synchronised).
 */
#ifndef Q27B_ATTN_H_
#define Q27B_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q27B_OK 0
#define Q27B_BAD_SHAPE 1      /* the reference throws "bad shape" here (src/attn.cu:906,929) */
#define Q27B_CUDA_ERROR 2     /* a CUDA runtime / driver call failed (the reference's CK(), src/common.cuh:12-13) */
#define Q27B_UNSUPPORTED 3
#define Q27B_DEVICE_STATUS 4  /* a kernel recorded a bounded wait that ran out */

#define Q27B_HEAD_DIM 256
#define Q27B_GQA 6
#define Q27B_MAX_T 4
#define Q27B_PART_ROW 258 /* floats of one partial row: max, sum, unnormalised O[256] (src/attn.cu:26) */
#define Q27B_PAGE 256     /* positions per page of the paged cache */

/* Text of the last error on this thread ("" if none). */
const char* q27b_last_error(void);

/* Reads (and clears) the device status word of the current device. Synchronises the device:
 * call it after your own synchronisation point. 0 = no kernel reported a problem. */
int q27b_device_status(int* status_out);

/* The per-device workspace (the counterpart of the reference's static AttnWs ws[16] and pbuf[16],
 * src/attn.cu:869-879,954-959), for callers that want control. All three act on the current device.
 *  - query: bytes currently held for the decode partials, the prefill partials and the paged-decode
 *    partials (0 = not allocated yet), and whether the workspace has been fixed.
 *  - init: allocates everything now - the decode partials, the prefill partials at prefill_bytes
 *    (0: the default cap of 128 MiB) and paged_bytes for the batched paged decode (0: none) - and
 *    fixes it: afterwards no entry point allocates or frees device memory (q27b_attn_decode_ref
 *    and the exchange-buffer helpers excepted); a call that would need more splits less (prefill) or
 *    fails with Q27B_UNSUPPORTED and says how much it needs (paged decode).
 *  - destroy: synchronises the device, frees the workspace and lifts the fix. Graphs captured
 *    before must not be replayed afterwards. */
int q27b_attn_workspace_query(uint64_t* decode_bytes, uint64_t* prefill_bytes, uint64_t* paged_bytes, int* fixed);
int q27b_attn_workspace_init(uint64_t prefill_bytes, uint64_t paged_bytes);
int q27b_attn_workspace_destroy(void);

/* Bytes of the K (or V) cache of one layer. q8_0 (q8 != 0): int8 values [nkvh][n_ctx][256]
 * followed by f16 scales [nkvh][n_ctx][8]; else f16 [nkvh][n_ctx][256].
 * Replaces q27::kv_cache_bytes (src/ops.h:53, src/attn.cu:890-892). */
uint64_t q27b_kv_cache_bytes(int nkvh, int n_ctx, int q8);

/* Position chunks per KV head used by the decode kernel on the current device.
 * Replaces q27::attn_chunks (src/ops.h:77, src/attn.cu:883-888). */
int q27b_attn_chunks(int nkvh);

/* Append T tokens' K and V rows (k, v: f32 [T][nkvh][256]) at cache rows *pos0 + t, quantised
 * to q8_0 (d = amax/127 per 32 values, q = round(x/d), f16 scale) or rounded to f16.
 * pos0 is read on the device. Replaces the cache-write tail of q27::attn_prep
 * (src/ops.h:59-62, attn_prep_kernel src/ops.cu:628-652). */
int q27b_kv_append(const float* k, const float* v, void* kcache, void* vcache, const int* pos0, int T, int nkvh,
                   int n_ctx, int q8, void* stream);

/* Full q27::attn_prep (src/ops.h:54-62, src/ops.cu:587-654,798-803): per-head RMSNorm of q and
 * k, NeoX RoPE on the first 64 dims (IMRoPE sections), q -> qn [T][nqh][256], K and V -> cache
 * rows *pos0 + t. rope3 / rdelta may be null. The reference's pf / pf_bytes L2-prefetch hint
 * has no counterpart (the shim ignores it). */
int q27b_attn_prep(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm,
                   float* qn, void* kcache, void* vcache, const int* pos0, int T, float eps, float theta_scale,
                   int nqh, int nkvh, int n_ctx, int q8, void* stream, const int* rope3, const int* rdelta);

/* Decode attention of T = 1..4 query tokens at positions *pos0 + t over cache rows
 * 0 .. *pos0 + t (causal inside the block), GQA 6:1, then o *= sigmoid(gate).
 * qn [T][nqh][256], qg [T][nqh][512] (gate in the second half of each 512), o [T][nqh][256] f32.
 * With xq != null the result goes to q8_1 (xq int8 [T*nqh*256], xd f32 [T*nqh*8]) instead of o.
 * Replaces q27::attn_decode (src/ops.h:63-67, src/attn.cu:894-918). */
int q27b_attn_decode(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o, int8_t* xq,
                     float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                     void* stream);

/* The same result with a simple slow kernel, for checks (plain f32 softmax over all visible
 * positions, roundings of the definition); T may be any size up to 65535. Its score scratch
 * (T * nqh * n_ctx floats) is allocated on demand. Replaces q27::attn_decode_ref (src/ops.h:73-75;
 * src/attn.cu:824-867,976-987), which tools/bench_attn.cu compares the fast kernels with. */
int q27b_attn_decode_ref(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                         const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream);

/* q27b_attn_decode for callers that must not allocate device memory. It has no counterpart in
 * the reference, whose attn_decode allocates its partial buffer on first use
 * (src/attn.cu:898-900). Same arguments, same result as q27b_attn_decode (q8_0 cache only).
 *
 * Who needs it: a host that runs under a fixed device-memory budget fixed at start-up, or that
 * drives several GPUs in lock step - there a cudaMalloc in the middle of a batch synchronises the
 * whole device while its peer is waiting for it (the situation the reference describes at
 * src/attn.cu:954-956) - or an embedding runtime that owns the allocator and forbids the library
 * to touch it. This entry point calls no cudaMalloc / cudaFree and no allocating library routine:
 * the split partials live in an array that is part of the library image (3.96 MB of every GPU
 * that loads the library, held until the process exits), and the result goes to the caller's
 * own buffers.
 *
 * Limit: nkvh * floor(SMs / nkvh) <= 160 chunk partials, i.e. any KV-head count on GPUs of up to
 * 160 SMs; beyond that the call returns Q27B_BAD_SHAPE and says so. A bounded wait that ran out in
 * these kernels shows in q27b_device_status like any other.
 * The first call on a device looks up the array's device address and opts the kernels into their
 * shared-memory size; make that first call before any stream capture starts.
 * Every call on a device uses the same array and leaves its partials there; nothing in it has to
 * start at zero (each call rewrites every partial it later reads). Two calls that can overlap on
 * the GPU (different streams) race on it: keep calls of one device in one stream order. */
int q27b_attn_decode_noalloc(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                             int8_t* xq, float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh,
                             int n_ctx, int q8, void* stream);

/* Same attention, restricted to the cache rows that this GPU holds when one sequence is split
 * by KV length across GPUs: local cache row i is global position base_pos + i, rows
 * 0 .. n_local-1 are attended (a row is visible to token t iff its global position is
 * <= *pos0 + t). Output is not normalised: part [T][nqh][258] = (max, sum, O[256]) per row,
 * ready for q27b_lse_merge. Extends the per-chunk partials of attn_mma_kernel
 * (src/attn.cu:115-120,286-289) to a per-GPU partial; the reference has no multi-GPU split. */
int q27b_attn_decode_partial(const float* qn, const void* kcache, const void* vcache, float* part, const int* pos0,
                             int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos, int n_local,
                             void* stream);

/* Log-sum-exp merge of nparts partials of `rows` rows (partial c, row r at
 * part + c*part_stride + r*258 floats): M = max m, L = sum l e^(m-M), A = sum O e^(m-M),
 * y = A/L * sigmoid(gate) with the gate of row r at qg + r*512 + 256 (qg null: no gate).
 * Output f32 o [rows][256], or q8_1 (xq, xd) when xq != null.
 * Replaces attn_combine_kernel (src/attn.cu:294-316) and attn_pf_combine_kernel
 * (src/attn.cu:803-822). */
int q27b_lse_merge(const float* part, int nparts, int64_t part_stride, int64_t rows, const float* qg, float* o,
                   int8_t* xq, float* xd, void* stream);

/* Batched decode over a paged q8_0 cache: B sequences, T query tokens each at positions
 * seq_len[b] - T + t (seq_len counts the T new tokens, whose K/V are already in the cache).
 * Pool layout (K and V each): int8 values [n_pages][nkvh][256][256] followed by f16 scales
 * [n_pages][nkvh][256][8]; page_table [B][max_pages] int32 (page j of sequence b holds its
 * positions 256*j .. 256*j+255); seq_len int32 [B] on the device.
 * qn [B][T][nqh][256], qg [B][T][nqh][512], o [B][T][nqh][256].
 * The reference is single-sequence with one contiguous cache (src/model.cu:462-472); this is
 * the same operator (src/ops.h:63-67) applied per sequence through a page table. */
int q27b_attn_decode_paged(const float* qn, const float* qg, const void* kpool, const void* vpool,
                           const int* page_table, const int* seq_len, float* o, int B, int T, float kq_scale, int nqh,
                           int nkvh, int n_pages, int max_pages, int max_seq_len, void* stream);

/* q27::attn_prep for a batch over the page pool: B sequences, T new tokens each at positions
 * seq_len[b] - T + t (seq_len counts them). qg [B][T][nqh][512], k / v [B][T][nkvh][256], qn [B][T][nqh][256];
 * rope3 [B][T][3] or null, rdelta [B] or null. With q_norm == null it only appends K and V (no norm, no
 * RoPE; qg, k_norm and qn are not used). The rows are written through page_table [B][max_pages] into the
 * pools of q27b_attn_decode_paged; an entry outside [0, n_pages) sets device status bit 1 and the row is
 * dropped. Same arithmetic as q27b_attn_prep (src/ops.cu:587-654) row by row. */
int q27b_attn_prep_paged(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm,
                         float* qn, void* kpool, void* vpool, const int* page_table, const int* seq_len, int B, int T,
                         float eps, float theta_scale, int nqh, int nkvh, int n_pages, int max_pages, void* stream,
                         const int* rope3, const int* rdelta);

/* Page bookkeeping for those pools (host only, thread-safe): which pages back which positions of which
 * sequence. The reference has one contiguous cache per sequence; what its server relies on when it
 * reuses a prompt prefix is that "KV rows below a position stay valid when the sequence is cut back to it"
 * (src/model.h:177-180, Engine::prepare src/engine.cpp:228-291): q27b_pager_cut keeps the pages that hold
 * rows below the new length and returns the others to the pool.
 *  - create: a pool of n_pages pages, at most max_seqs sequences of at most max_pages_per_seq pages.
 *  - open: a new empty sequence. extend: back positions below new_len (>= the current length) with pages;
 *    Q27B_UNSUPPORTED, and nothing changed, when the pool has too few free pages. close: all pages back.
 *  - fork: a new sequence that starts as the first prefix_len positions of `seq`: the full pages of the
 *    prefix are shared (reference counts, no copy); if the prefix ends inside a page the new sequence gets a
 *    page of its own for it and the call returns the pair to copy (q27b_kv_page_copy, K and V pools), else -1.
 *    Only sequences whose last page is full or not shared can be extended; unshare gives a sequence whose
 *    partly filled last page is shared (after a fork at a page boundary and a cut, say) a page of its own
 *    and returns the pair to copy, or -1 when there was nothing to do.
 *  - tables: page_table [B][max_pages_per_seq] (-1 where no page) and seq_len [B] of the given sequences,
 *    into host memory, in the form the device operators read. */
typedef struct q27b_pager q27b_pager;
int q27b_pager_create(int n_pages, int max_seqs, int max_pages_per_seq, q27b_pager** out);
void q27b_pager_destroy(q27b_pager* pager);
int q27b_pager_open(q27b_pager* pager, int* seq);
int q27b_pager_extend(q27b_pager* pager, int seq, int new_len);
int q27b_pager_cut(q27b_pager* pager, int seq, int new_len);
int q27b_pager_close(q27b_pager* pager, int seq);
int q27b_pager_fork(q27b_pager* pager, int seq, int prefix_len, int* new_seq, int* copy_src_page, int* copy_dst_page,
                    int* copy_rows);
int q27b_pager_unshare(q27b_pager* pager, int seq, int* copy_src_page, int* copy_dst_page, int* copy_rows);
int q27b_pager_free_pages(q27b_pager* pager); /* -1: null */
int q27b_pager_len(q27b_pager* pager, int seq); /* -1: no such sequence */
int q27b_pager_tables(q27b_pager* pager, const int* seqs, int B, int* page_table, int* seq_len);
/* The first `rows` rows of page src_page into page dst_page, all heads, of one pool (K or V). */
int q27b_kv_page_copy(void* pool, int src_page, int dst_page, int rows, int nkvh, int n_pages, void* stream);

/* One sequence split by KV length over the nz GPUs of a head group, exchanged over peer memory
 * instead of a collective. Every rank owns an exchange buffer of q27b_xbuf_bytes(nz, T * nqh) bytes,
 * zeroed once, that its peers can store into (peer-mapped device memory; how it is mapped is the
 * caller's business: CUDA IPC, symmetric memory, one process with several devices).
 * q27b_attn_decode_partial_push = q27b_attn_decode_partial whose merge kernel stores the slice's
 * (m, l, O) rows into slot my_z of all nz buffers (peer_xbuf[k] = buffer of rank k of the group, as
 * seen from this GPU; peer_xbuf[my_z] is this rank's own). Every float travels as one 8-byte word
 * {value, step tag}: an aligned 8-byte store arrives whole, so a word that carries the tag of the current
 * step carries its value, and neither a fence nor a flag is needed. q27b_lse_merge_wait waits (bounded:
 * about a second, then device status bit 0 and nothing is written) for the words of the nz slices in its
 * own buffer, merges them and applies the gate. Steps are counted on the device, so the pair can sit in a
 * CUDA graph; two parities of the data area make it safe for a rank to run one step ahead of a peer. No
 * counterpart in the reference (its two cards split KV heads, never the KV length: src/model.cu:161-164). */
uint64_t q27b_xbuf_bytes(int nz, int64_t rows);
/* Helpers for one process per GPU: an exchange buffer as a cudaMalloc allocation of its own (zeroed),
 * its CUDA IPC handle (64 bytes, to be sent to the peers by any means), and the mapping of a peer's
 * handle into the address space of the calling thread's CURRENT device, which must be the device
 * whose kernels will store into it (a handle opened under another device is not reachable). */
int q27b_xbuf_alloc(int nz, int64_t rows, void** out);
int q27b_xbuf_free(void* xbuf);
/* After a step that ended in device status 1 (a peer's slice or rows never arrived: the waiting kernel
 * gave up without finishing the step's bookkeeping) an exchange buffer is out of step with its peers.
 * Before the group uses its buffers again EVERY rank of the group zeroes its own buffer with this call
 * (`bytes` = the size it was allocated with: the header with the step counters, and the data area, whose
 * words carry step tags that a restarted count would meet again; on `stream`), and the ranks meet on the
 * host (a barrier of whatever they use to talk) between the resets and the next push. Applies to the
 * buffers of both exchanges (q27b_lse_merge_wait and q27b_sum_norm_q8_wait). */
int q27b_xbuf_reset(void* xbuf, uint64_t bytes, void* stream);
int q27b_ipc_export(const void* ptr, unsigned char handle[64]);
int q27b_ipc_open(const unsigned char handle[64], void** out);
int q27b_ipc_close(void* mapped);
int q27b_attn_decode_partial_push(const float* qn, const void* kcache, const void* vcache, const int* pos0, int T,
                                  float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos, int n_local,
                                  void* const* peer_xbuf, int my_z, int nz, void* stream);
int q27b_lse_merge_wait(void* xbuf, int nz, int64_t rows, const float* qg, float* o, void* stream);
/* The two calls above as one: after the split-K kernel a single kernel merges this rank's slice, stores it
 * into the peers' buffers and, having pushed, waits (bounded) for the peers' slices in its own buffer and
 * writes the gated output - one launch less per step. Every rank of the group must run the same call in the
 * same step (each pushes before it waits, so the waits cannot wait for one another). Falls back to the pair
 * when the slice's shape does not take the many-partials form of the merge (more than two KV heads per GPU). */
int q27b_attn_decode_exchange(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                              const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos,
                              int n_local, void* const* peer_xbuf, int my_z, int nz, void* stream);

/* How the path is shared out over the GPUs of one box, as host arithmetic (no GPU needed), for hosts that do
 * not go through the Python helpers (qwen27-engine_b200/shard.py gives the same answers). The reference splits
 * by KV head only (2 KV heads + their 12 query heads per card, src/model.cu:161-164).
 *  - plan_single_sequence: up to nkvh ranks, rank r owns KV heads [kv_head0, kv_head0 + n_kv_heads) and there is
 *    no exchange (nz = 1); beyond, a head belongs to nz = world / nkvh ranks, rank r holding KV-length slice z of it.
 *  - kv_slice: positions [lo, hi) of slice z of nz of a sequence of n positions (boundaries on 64-position tiles).
 *  - plan_prefill: one chunk of M tokens at pos0: KV-head groups first, then up to two query-token ranges
 *    [ranges[2i], ranges[2i+1]) per rank (an early and a late block of equal causal cost, whole 128-token tiles);
 *    each range is one q27b_attn_prefill call at pos0 + ranges[2i]. ranges must hold 4 ints. */
int q27b_plan_single_sequence(int rank, int world, int nkvh, int* kv_head0, int* n_kv_heads, int* z, int* nz);
int q27b_kv_slice(int n, int z, int nz, int* lo, int* hi);
int q27b_plan_prefill(int rank, int world, int M, int pos0, int nkvh, int* kv_head0, int* n_kv_heads, int* ranges,
                      int* n_ranges);

/* The step after the attention output projection (row f4 of the path's neighbours): x [rows][n] +=
 * the sum over the GPUs of their partial rows, then RMSNorm(x) * w -> h (f32, may be null) and q8_1
 * (xq int8 [rows][n], xd f32 [rows * n / 32] = f32(f16(amax / 127)); xq may be null). Replaces
 * q27::sum_norm_q8 (src/ops.h:101-104; kernel src/ops.cu:129-260 with norm_q8_row :89-107; call
 * sites src/model.cu:652-692). n a multiple of 32 up to 16384 (the model has n = 5120).
 *  - q27b_sum_norm_q8: one GPU, or partials already summed (the reference's ar == null branch).
 *  - q27b_sum_push + q27b_sum_norm_q8_wait: `world` GPUs on one NVLink switch. Every rank owns an
 *    exchange buffer of q27b_sum_xbuf_bytes(world, rows, n) bytes (q27b_xbuf_alloc_bytes: zeroed,
 *    an allocation of its own for CUDA IPC) and passes the buffers of all ranks, its own at index
 *    `rank`, as mapped into its address space, in rank order. q27b_sum_push stores this rank's f32
 *    rows into slot `rank` of every buffer, one 8-byte word {value, step tag} per float (no fence, no
 *    flag: a word with the tag of the current step carries its value); q27b_sum_norm_q8_wait waits
 *    (bounded: a missing rank ends in Q27B status 4 / device status 1, not in a hang) for the words of all
 *    ranks, adds the slices in rank order - every rank gets the same bits - and normalises. The reference's
 *    two PCIe cards exchange through mapped host memory in a bf16 or q8 wire format
 *    (src/ops.cu:151-243); over NVLink the f32 rows go as they are. A buffer serves one call site
 *    per step (its header counts steps); rows and n must not change between steps. */
uint64_t q27b_sum_xbuf_bytes(int world, int rows, int n);
int q27b_xbuf_alloc_bytes(uint64_t bytes, void** out);
int q27b_sum_norm_q8(float* x, const float* partial, int n, int rows, const float* w, float eps, float* h, int8_t* xq,
                     float* xd, void* stream);
int q27b_sum_push(const float* partial, int n, int rows, int rank, int world, void* const* xbufs, void* stream);
int q27b_sum_norm_q8_wait(float* x, void* xbuf, int world, int n, int rows, const float* w, float eps, float* h, int8_t* xq,
                          float* xd, void* stream);
/* q27b_sum_push + q27b_sum_norm_q8_wait as one kernel: every CTA stores its row of this rank's partial into the
 * peers' buffers, then waits for theirs and normalises (every rank of the group runs the same call in the same
 * step; each pushes before it waits). */
int q27b_sum_exchange_norm_q8(float* x, const float* partial, int n, int rows, int rank, int world, void* const* xbufs,
                              const float* w, float eps, float* h, int8_t* xq, float* xd, void* stream);

/* Which split-K kernel q27b_attn_decode* uses for q8_0 caches: 0 = default (the warp-specialised
 * kernel), 1 = the single-role warp-MMA kernel (every warp runs both contractions), 2 = the tcgen05
 * kernel (both contractions on the 5th-generation tensor cores), 3 = the warp-specialised kernel
 * (Q K^T warps and P V warps, csrc/decode_ws.cu). All compute the same operator with the same roundings
 * (src/attn.cu:95-292). Process-wide; the environment variable Q27B_DECODE_KERNEL=mma|tc|ws sets the
 * initial value. No counterpart in the reference (it has one kernel). */
int q27b_set_decode_kernel(int which);

/* How the warp-specialised split-K kernel shares out one sequence: pool != 0 (default): every CTA owns
 * about four fifths of an equal share of the 64-position tiles and draws the rest one by one from a
 * pool per KV head, so that CTAs on faster SMs take more (the result then depends on the order of
 * f32 additions and may differ in the last bits from run to run); pool == 0: equal static shares, the
 * same bits on every run. Process-wide; Q27B_DECODE_POOL=0 sets the initial value. No counterpart in
 * the reference. */
int q27b_set_decode_schedule(int pool);

/* Which kernel q27b_attn_prefill* uses for q8_0 caches: 0 = default, 1 = int8 Q K^T
 * (attn_prefill_i8_kernel, src/attn.cu:557-801; the reference's default), 2 = f16 Q K^T on K and V
 * dequantised to f16 on the way to the tensor core (attn_prefill_kernel<PT, true>,
 * src/attn.cu:338-528; the reference's Q27_ATTN_I8=0). Process-wide; the environment variable
 * Q27_ATTN_I8=0 sets the initial value to 2, as in the reference (src/attn.cu:933). f16 caches
 * always use the f16 kernel. */
int q27b_set_prefill_kernel(int which);

/* How a q27b_attn_prefill call of M tokens and nqh heads on a GPU of n_sm SMs splits its positions
 * (host arithmetic only, no GPU needed): the first *split_tiles 128-token query tiles are cut into
 * *pieces pieces each (partials + merge), the others are not split. Few CTAs: every tile is split by
 * the reference's rule (src/attn.cu:945-951, also what Q27_ATTN_SPLIT forces); more CTAs than SMs on
 * a deep prefix: only as many CTAs as do not fill a last full round are cut. 0 / 1 = no split. */
int q27b_prefill_split_plan(int M, int nqh, int n_sm, int depth_hint, int* split_tiles, int* pieces);

/* Test hook for the failure path, no counterpart in the reference: launches one warp that waits on
 * a barrier nobody arrives at, with the bounded wait every kernel of this library uses. After the
 * limit (about two seconds) the wait gives up, the kernel returns normally and
 * q27b_device_status reports bit 0 (wait expired); the context stays usable. */
int q27b_debug_expire_wait(void* stream);

/* Measurement hook, no counterpart in the reference: while `event` (a cudaEvent_t) is set, every
 * q27b_attn_decode / q27b_attn_decode_partial call on the current device records it on the
 * caller's stream between its split-K kernel and its merge kernel, so that a benchmark can time
 * the dominant kernel alone with CUDA events. NULL switches it off. */
int q27b_debug_split_event(void* event);
/* The same with an event before the split-K kernel as well. Inside a stream capture both records
 * become event nodes of the graph (cudaEventRecordExternal) and are taken at every replay, so the
 * kernel can be timed alone, on the launching stream, inside the replayed graph: set a pair of events
 * before each captured call. NULL, NULL switches it off. */
int q27b_debug_split_events(void* begin, void* end);
/* While on, q27b_attn_decode on the current device launches its split-K kernel only (the partials stay
 * in the workspace, the output is not written): a benchmark captures a graph of such calls and times
 * the dominant kernel alone, back to back, with events around the replay (event nodes between the
 * kernels of a graph cost a few microseconds each and distort a 65 us kernel). */
int q27b_debug_split_only(int on);

/* Measurement hook, no counterpart in the reference: while `stamps` (device memory, 8 x uint64 per
 * CTA of the split-K grid, i.e. 8 * q27b_attn_chunks(nkvh) * nkvh values) is set, every CTA of the
 * warp-specialised split-K kernel of q27b_attn_decode / _partial on the current device writes
 * %globaltimer values (ns) there: [0] kernel entry, [1] barriers initialised and the position known,
 * [2] first K tile landed, [3] / [4] Q K^T loop of group 0 / 1 finished, [5] first P tile handed
 * over, [6] P V loop of group 0 finished, [7] partial written. A benchmark reads from them how a
 * launch divides into ramp-up, streaming and drain. NULL switches it off. */
int q27b_debug_decode_trace(unsigned long long* stamps);

/* Measurement hook, no counterpart in the reference: launches the tensor-core peak microbenchmark on
 * the current device (one CTA per SM issuing `iters` x 4 back-to-back tcgen05.mma 128 x 256 tiles from
 * operands resident in shared memory into tensor memory): kind 0 = kind::i8 (s8 x s8 -> s32, K = 32 per
 * instruction), kind 1 = kind::f16 (f16 x f16 -> f32, K = 16). *ops_per_launch = the multiply-adds x 2
 * of one launch; time the launch with events to get the int8 TOPS / f16 TFLOPS that the prefill
 * kernels' tensor-pipe fractions are quoted against (the reference quotes its kernel against its card's
 * tensor peak, docs/PERFORMANCE.md:214). */
int q27b_debug_mma_peak(int kind, int iters, void* stream, double* ops_per_launch);

/* The reference's host ("wire") layout of rows [p0, p1) of one cache, used for its RAM swap of idle
 * slots and its prompt-cache checkpoints (Decoder::kv_copy, src/model.cu:1809-1830): the values
 * [nkvh][p1-p0][256 B], then the scales [nkvh][p1-p0][16 B]; q27b_kv_wire_bytes gives its size
 * (q8_0 caches only). The four functions pack such a buffer on the device from, and unpack it into,
 * the page pool of one sequence (`pages` = its page table row on the device, as in
 * q27b_attn_decode_paged) or a contiguous cache [nkvh][n_ctx]; one contiguous copy between `wire`
 * and pinned host memory completes the transfer. With them a slot written by a paged engine can be
 * restored into the reference's contiguous cache and the other way round. A page index outside
 * [0, n_pages) sets device status bit 1 and skips the row. */
uint64_t q27b_kv_wire_bytes(int nkvh, int n_rows);
int q27b_kv_pages_to_wire(const void* pool, const int* pages, void* wire, int nkvh, int n_pages, int p0, int p1,
                          void* stream);
int q27b_kv_wire_to_pages(void* pool, const int* pages, const void* wire, int nkvh, int n_pages, int p0, int p1,
                          void* stream);
int q27b_kv_cache_to_wire(const void* cache, void* wire, int nkvh, int n_ctx, int p0, int p1, void* stream);
int q27b_kv_wire_to_cache(void* cache, const void* wire, int nkvh, int n_ctx, int p0, int p1, void* stream);

/* Bytes of the K (or V) page pool of q27b_attn_decode_paged. */
uint64_t q27b_kv_pool_bytes(int nkvh, int n_pages);

/* Prefill attention: M query tokens at positions *pos0 .. *pos0+M-1 (their K/V already in the
 * cache), causal, o [M][nqh][256] f32 with the gate applied. q8_0 cache: Q K^T on the int8
 * tensor path (Q rounded to int8 with an f32 scale per 32 dims, K = the cache bytes, one int32
 * dot product per 32-dim block, scaled and summed in f32), P V in f16 with f32 accumulation.
 * f16 cache (q8 = 0): Q * kq_scale rounded to f16, Q K^T and P V in f16 with f32 accumulation
 * (attn_prefill_kernel<PT, false>, src/attn.cu:338-528).
 * depth_hint: host copy of *pos0 or -1. Replaces q27::attn_prefill (src/ops.h:68-72,
 * src/attn.cu:920-974; kernel attn_prefill_i8_kernel src/attn.cu:557-801). */
int q27b_attn_prefill(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                      const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream,
                      int depth_hint);

/* The same with the output quantised to q8_1 in the kernel's epilogue, which is what the reference
 * does with the attention output before its next GEMM (quantize_q8_1 after attn_prefill,
 * src/model.cu:1230,1499; numerics of q8_store, src/common.cuh:72-81): xq int8 [M][nqh][256],
 * xd f32 [M*nqh*8] = f32(f16(amax / 127)) per 32 values. The f32 round trip through `o` is saved. */
int q27b_attn_prefill_q8_1(const float* qn, const float* qg, const void* kcache, const void* vcache, int8_t* xq,
                           float* xd, const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                           void* stream, int depth_hint);

/* Test hook of the prefill kernel's integer stage: quantises `rows` (<= 128) query rows
 * (x [rows][256] f32, already the rows of one head) as the prefill kernel does and multiplies
 * them on the int8 tensor path with npos (<= 64) K rows taken from a q8_0 cache (head kh,
 * first row p0). Outputs: q_i8 [rows][256], q_scale [rows][8] f32, acc [rows][npos][8] int32
 * (the per-32-block accumulators of src/attn.cu:690-691, which must be bit-exact). */
int q27b_prefill_qk_debug(const float* x, int rows, float kq_scale, const void* kcache, int nkvh, int n_ctx, int kh,
                          int p0, int npos, int8_t* q_i8, float* q_scale, int32_t* acc, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q27B_ATTN_H_ */
