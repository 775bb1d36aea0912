/*
 * flywheel_b200.h -- C ABI of the B200 (sm_100a) paged-KV softmax attention path.
 *
 * This is the boundary a host binding (XLA FFI handler, ctypes, cgo ...) calls.
 * Every pointer below is a DEVICE pointer unless a comment says "host".  No
 * entry point allocates, frees or synchronises: work is enqueued on the CUDA
 * stream the caller passes (a cudaStream_t cast to void*), scratch memory is a
 * caller-owned workspace sized by the matching *_workspace_bytes call, and
 * values the reference allows to be traced (lengths, tables, descales, sinks,
 * num_active) are read on the device, never on the host.
 *
 * Reference interfaces these entry points stand behind (paths relative to the
 * heavyball-research/flywheel-tpu project):
 *   fw_decode_kvcache   <- flywheel_tpu/softmax_attention/decode.py:189-625
 *                          (flash_attn_with_kvcache) and the custom call it
 *                          lowers to, kernels/decode.py:2046-2475
 *   fw_append_ragged    <- kernels/kv_append.py:116-184 (append_ragged)
 *   fw_write_kv_pages   <- flywheel_tpu/softmax_attention/page.py:35-73
 *                          (write_kv_cache_pages)
 *   fw_prefill_paged    <- flywheel_tpu/softmax_attention/prefill.py:437-661
 *                          (flash_attn_varlen_func with block_table) and
 *                          kernels/fwd_paged.py:1351-1491
 *   fw_lse_combine      <- patches/tpu-inference.patch:7174-7186 (_merge_states;
 *                          the library itself has no split-KV merge)
 *
 * Return value: FW_OK or a negative FW_ERR_* code; fw_last_error() returns a
 * thread-local message for the last failing call on the calling thread.
 */
#ifndef FLYWHEEL_B200_H_
#define FLYWHEEL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FW_OK 0
#define FW_ERR_BAD_SHAPE (-1)   /* reference raises ValueError               */
#define FW_ERR_BAD_DTYPE (-2)   /* reference raises NotImplementedError      */
#define FW_ERR_UNSUPPORTED (-3) /* valid in the reference, not built here    */
#define FW_ERR_LAUNCH (-4)      /* CUDA refused the launch / descriptor      */
#define FW_ERR_TIMEOUT (-5)     /* a bounded device-side wait gave up        */
#define FW_ERR_WORKSPACE (-6)   /* workspace missing, small or misaligned    */

/* KV cache element types (flywheel_tpu/softmax_attention/kv_layout.py:30-34). */
#define FW_DTYPE_BF16 0
#define FW_DTYPE_E4M3 1
#define FW_DTYPE_E5M2 2

/* Device status word at workspace offset 0: the OR of the bits below, 0 = clean.
 * It stays set until fw_read_status reports and clears it, so it covers every
 * launch since the last read.  WAIT_TIMEOUT: a bounded device-side wait gave up
 * and the results of that launch are void.  BAD_PAGE: a block-table entry
 * outside the pool, or a position past the table row / the contiguous capacity,
 * was met; reads were clamped to page 0 (that request's output is void) and
 * an append to such a position stored nothing.  The first 256 bytes of a
 * workspace belong to this status block and must be zero when the workspace is
 * first used (afterwards the library maintains them). */
#define FW_STATUS_OK 0
#define FW_STATUS_WAIT_TIMEOUT 1
#define FW_STATUS_BAD_PAGE 2

/*
 * Attention of q against a KV cache with the new tokens' K/V appended in the
 * same launch (flash_attn_with_kvcache, decode.py:189-625).
 *
 * head_dim is 64 (bf16 caches only), 128 or 256 (at 256: at most 64 query
 * rows, seqlen_q * nheads / nheads_k, per KV head).
 *
 * Layouts
 *   paged merged (block_table != NULL): kv_cache is one pool
 *     (num_pages, page_size, cache_heads, head_dim) whose token rows hold
 *     [k0, v0, k1, v1, ...] (kv_layout.py:39-46); v_cache must be NULL.
 *     cache_heads = 2*nheads_k, an odd fp8 nheads_k padded by one zero head.
 *     page_size must be a multiple of 16 (the reference asks for 128).
 *   contiguous pair (block_table == NULL): kv_cache and v_cache are
 *     (batch_cache, capacity, nheads_k, head_dim) bf16; cache_batch_idx (or
 *     NULL = identity) picks the cache row of each query row; seqlen_q == 1.
 * q / out: (batch, seqlen_q, nheads, head_dim) bf16.  k_new / v_new: NULL, or
 * (batch, seqlen_q, nheads_k, head_dim) in the cache dtype; token t of row b
 * is written at position cache_seqlens[b] + t and then attended.
 * lse: NULL or (batch, nheads, seqlen_q) f32, natural log.
 * Mask: bottom-right aligned; causal != 0 forces the right bound to 0;
 * window_left < 0 is unbounded.  softcap > 0 maps a scaled score s to
 * softcap * tanh(s / softcap).  sinks: NULL or (nheads,) f32.
 * Rows b >= *num_active (NULL = batch) append nothing and return out 0,
 * lse -inf.
 *
 * partial_out != NULL switches to "partial state" mode for a cache whose
 * pages are split over several GPUs: instead of out/lse the call writes the
 * sink-free normalised f32 state partial_out (batch, seqlen_q, nheads,
 * head_dim) and partial_lse (batch, seqlen_q, nheads); merge the gathered
 * states with fw_lse_combine.
 */
typedef struct FwDecodeArgs {
  const void* q;
  void* out;
  float* lse;
  void* kv_cache;
  void* v_cache;
  const void* k_new;
  const void* v_new;
  const int32_t* cache_seqlens;
  const int32_t* block_table;
  const int32_t* cache_batch_idx;
  const int32_t* num_active;
  const float* k_descale;
  const float* v_descale;
  const float* sinks;
  float* partial_out;
  float* partial_lse;
  void* workspace;
  uint64_t workspace_bytes;
  int64_t num_pages;        /* paged: pool pages; contiguous: batch_cache */
  int32_t page_size;        /* paged: tokens per page; contiguous: capacity */
  int32_t pages_per_seq;    /* block_table row length */
  int32_t batch;
  int32_t seqlen_q;
  int32_t nheads;
  int32_t nheads_k;
  int32_t head_dim;
  int32_t kv_dtype;         /* FW_DTYPE_* */
  int32_t causal;
  int32_t window_left;      /* -1 = unbounded */
  float softmax_scale;
  float softcap;
  int32_t num_ctas;         /* 0 = pick from the device; tests may pin it */
  /* NULL, or one device int read by the kernel: 0 makes the call behave as if
   * k_new / v_new were NULL (nothing appended, the new tokens not attended).
   * Lets one enqueued or graph-captured call serve steps in which this GPU does
   * and does not own the page the new token falls in (see fw_shard_step). */
  const int32_t* append_enable;
} FwDecodeArgs;

uint64_t fw_decode_workspace_bytes(const FwDecodeArgs* args);
int fw_decode_kvcache(const FwDecodeArgs* args, void* stream);

/*
 * fw_decode_kvcache for hosts that must not allocate device memory.
 * (No counterpart in the reference: its kernels get their scratch from XLA.)
 *
 * Some callers cannot hand this library a workspace: a serving engine that
 * has already given every free byte of HBM to its KV-cache pool, a runtime
 * whose allocator must not be re-entered from inside a custom-call handler,
 * or latency-critical code that cannot afford the device-wide synchronisation
 * a cudaMalloc may imply.  For them this entry point keeps the split-KV
 * partial states in a fixed array of FW_STATIC_SCRATCH_BYTES that is part of
 * the library's device image: every GPU that loads the library holds that
 * much memory until the process exits, and nothing is allocated or freed
 * here.  args->workspace and args->workspace_bytes are ignored; inputs and
 * outputs are still the caller's.  A call whose fw_decode_workspace_bytes
 * exceeds FW_STATIC_SCRATCH_BYTES (very large batch x heads) is refused with
 * FW_ERR_WORKSPACE.
 *
 * The first call on each device looks up the array's address on that device
 * (the device must be current, as for every call); make that first call before
 * starting any stream capture.  All calls on one device share the one array:
 * two calls that overlap on the GPU (different streams, no dependency) race on
 * it, so keep them ordered.  The array keeps the previous call's contents;
 * the entry point clears the status word itself, nothing else needs zeroing.
 * Read that word with fw_read_status_static (fw_read_status needs a workspace
 * pointer, which callers of this entry point never hold).
 */
#define FW_STATIC_SCRATCH_BYTES (32ull << 20)
int fw_decode_kvcache_static(const FwDecodeArgs* args, void* stream);

/* The status word of the built-in scratch on the current device, copied to
 * *status (host) after synchronising `stream`, then cleared if it was set.  It
 * describes the most recent fw_decode_kvcache_static call on that device only,
 * because each such call starts by clearing the word.  (No counterpart in the
 * reference.) */
int fw_read_status_static(void* stream, int32_t* status);

/*
 * Packed new K/V rows -> merged pages (append_ragged, kv_append.py:116-184).
 * k_new / v_new: (total_tokens, nheads_k, head_dim) in the pool dtype;
 * request r < *num_active owns rows [cu_seqlens_q[r], cu_seqlens_q[r+1]) and
 * writes them at cache_seqlens[r] + t.  Whole merged rows are written.
 */
typedef struct FwAppendArgs {
  void* kv_cache;
  const void* k_new;
  const void* v_new;
  const int32_t* cu_seqlens_q;   /* (batch + 1,) */
  const int32_t* cache_seqlens;  /* (batch,) lengths before the append */
  const int32_t* block_table;
  const int32_t* num_active;
  int64_t num_pages;
  int32_t page_size;
  int32_t pages_per_seq;
  int32_t batch;
  int32_t total_tokens;
  int32_t nheads_k;
  int32_t head_dim;
  int32_t kv_dtype;
} FwAppendArgs;

int fw_append_ragged(const FwAppendArgs* args, void* stream);

/*
 * Slice-table page writer (write_kv_cache_pages,
 * flywheel_tpu/softmax_attention/page.py:35-73 and
 * kernels/kv_cache_write.py:66-227): the serving caller's prefill cache fill.
 * k_new / v_new: (total_tokens, nheads_k, head_dim) in the pool dtype.
 * slices: i32[3, num_columns] row-major; column j < *num_slices is
 * (cache_row_start, new_row_start, length) in rows of the flat
 * (num_pages * page_size) cache view and of k / v, each piece inside one page;
 * later columns are ignored.  Whole merged rows are written (bits, not values;
 * an fp8 pad head as zeros); rows outside the cache or k / v are skipped.
 */
typedef struct FwWritePagesArgs {
  void* kv_cache;
  const void* k_new;
  const void* v_new;
  const int32_t* slices;
  const int32_t* num_slices;
  int64_t num_pages;
  int32_t page_size;
  int32_t num_columns;
  int32_t total_tokens;
  int32_t nheads_k;
  int32_t head_dim;
  int32_t kv_dtype;
} FwWritePagesArgs;

int fw_write_kv_pages(const FwWritePagesArgs* args, void* stream);

/*
 * Read-only chunked prefill over the merged pool (flash_attn_varlen_func with
 * block_table, prefill.py:437-661).  q / out: head-major (nheads, total_q,
 * head_dim) bf16; lse: NULL or (nheads, total_q) f32.  seqused_k[r] is request
 * r's KV length, its new tokens included, already in the pool.  Rows past
 * cu_seqlens_q[*num_active] return out 0, lse -inf.
 */
typedef struct FwPrefillArgs {
  const void* q;
  void* out;
  float* lse;
  const void* kv_cache;
  const int32_t* cu_seqlens_q;   /* (batch + 1,), cu_seqlens_q[0] == 0 */
  const int32_t* seqused_k;      /* (batch,) */
  const int32_t* block_table;
  const int32_t* num_active;
  const float* k_descale;
  const float* v_descale;
  const float* sinks;
  void* workspace;
  uint64_t workspace_bytes;
  int64_t num_pages;
  int32_t page_size;
  int32_t pages_per_seq;
  int32_t batch;
  int32_t total_q;
  int32_t max_seqlen_q;
  int32_t nheads;
  int32_t nheads_k;
  int32_t head_dim;
  int32_t kv_dtype;
  int32_t causal;
  int32_t window_left;
  float softmax_scale;
  float softcap;
  int32_t token_major;  /* 1: q/out are (total_q, nheads, head_dim) */
  /* Q-only rotary embedding (prefill.py:494-498, rotary.py:27-215): NULL, or
   * (rotary_len, head_dim / 2) cos / sin tables, f32 (rotary_bf16 = 0) or bf16.
   * Token t of request r is rotated at position seqused_k[r] - len_q(r) + t in
   * f32 and rounded once to bf16; the cache holds K already rotated. */
  const void* rotary_cos;
  const void* rotary_sin;
  int32_t rotary_len;
  int32_t rotary_interleaved;
  int32_t rotary_bf16;
  /* Packed K/V (fw_attention_packed only; leave zero for fw_prefill_paged):
   * kv_cache is K and v_packed is V, bf16, (nheads_k, total_k, head_dim) or,
   * with kv_token_major = 1, (total_k, nheads_k, head_dim).  Request r's keys
   * are rows [cu_seqlens_k[r], cu_seqlens_k[r + 1]). */
  const void* v_packed;
  const int32_t* cu_seqlens_k;   /* (batch + 1,) */
  int32_t total_k;
  int32_t kv_token_major;
  int32_t rotary_k;      /* 1: K is rotated too, token t of a request at position t */
  int32_t sink_period;   /* 0: sinks has nheads entries; n > 0: head h uses sinks[h % n] */
  int32_t window_right;  /* > 0 with causal = 0: keys up to this far past a row's diagonal are visible */
  /* Packed K/V in fixed-size request slots instead of cu_seqlens_k: n > 0 puts
   * request r's keys at rows [r * n, r * n + seqused_k[r]) (cu_seqlens_k NULL). */
  int32_t kv_request_stride;
  /* Which kernel serves a paged call: FW_ROUTE_AUTO lets the library choose by
   * chunk length (tensor-core kernel for chunks of 64 tokens and more, the
   * split-KV kernel below that); the other two pin it for this call where the
   * pinned kernel can take the shapes.  Per call, no process-wide switch. */
  int32_t route;
  /* NULL, or one device int: requests below *first_request are left out (no
   * query blocks are made for them and their packed rows are not written), as if
   * the request window started there.  What a mixed step needs: its leading
   * one-token requests go to the decode kernel (see fw_extend_mixed). */
  const int32_t* first_request;
} FwPrefillArgs;

#define FW_ROUTE_AUTO 0
#define FW_ROUTE_TENSOR_CORE 1
#define FW_ROUTE_SPLIT_KV 2

uint64_t fw_prefill_workspace_bytes(const FwPrefillArgs* args);
int fw_prefill_paged(const FwPrefillArgs* args, void* stream);

/*
 * One mixed serving step over the paged pool: the leading *num_decode requests
 * are one-token decode rows, the requests after them (up to *num_active) are
 * prefill chunks; what flywheel_tpu_extend of the reference's serving backend
 * does with a page write, a decode call and a varlen call over a request window
 * slid past the decode rows (patches/tpu-inference.patch:8219-8320).  Here it is
 * one entry point and one launch sequence on `stream`, with every count read on
 * the device: (1) when k_new is given, the slice-table page write of all
 * scheduled tokens (fw_write_kv_pages); (2) the split-KV decode kernel over
 * requests [0, *num_decode), reading the pool (nothing appended: the rows were
 * just written), so a one-token row never occupies a 256-row tensor-core tile;
 * (3) the paged prefill over requests [*num_decode, *num_active), whose query
 * blocks start at the first prefill request without the host sliding any array.
 *
 * attn describes the step like a fw_prefill_paged call with token_major = 1:
 * q / out (total_q, nheads, head_dim) bf16, request r owns rows
 * [cu_seqlens_q[r], cu_seqlens_q[r + 1]) (one row each for the decode requests),
 * seqused_k[r] = its KV length with this step's tokens included.  attn.lse and
 * the rotary fields must be NULL; attn.first_request is ignored.  Rows at or past
 * cu_seqlens_q[*num_active] return 0.  The workspace (fw_extend_workspace_bytes)
 * holds both kernels' scratch; one status word at its head serves both.
 */
typedef struct FwExtendArgs {
  FwPrefillArgs attn;
  const int32_t* num_decode;   /* device int, 0 <= *num_decode <= *num_active */
  /* Optional page write before attention (NULL k_new = the pool is already
   * written); fields as in FwWritePagesArgs. */
  const void* k_new;
  const void* v_new;
  const int32_t* slices;
  const int32_t* num_slices;
  int32_t num_columns;
  int32_t total_tokens;
} FwExtendArgs;

uint64_t fw_extend_workspace_bytes(const FwExtendArgs* args);
int fw_extend_mixed(const FwExtendArgs* args, void* stream);

/*
 * Forward attention of packed q over packed K/V without a block table: the
 * non-paged branch of flash_attn_varlen_func (prefill.py:818-963) and, with one
 * sequence per batch row, flash_attn_func (prefill.py:62-341; its head-major
 * (batch, nheads, seqlen, head_dim) layout is this call with batch * nheads
 * heads over a single sequence, sink_period = nheads).  Causal and left-window
 * masks are bottom-right aligned per sequence (causal = 1 is a right bound of
 * 0, window_right a positive one).  bf16, head_dim 64, 128 or 256, nheads /
 * nheads_k up to 128.  block_table, seqused_k, num_active and the descales must be NULL.
 * Rows past cu_seqlens_q[batch] return out 0, lse -inf.  With rotary tables q
 * (and K when rotary_k = 1) are rotated into scratch copies first.
 */
uint64_t fw_attention_packed_workspace_bytes(const FwPrefillArgs* args);
int fw_attention_packed(const FwPrefillArgs* args, void* stream);

/*
 * Merge `parts` sink-free partial states over disjoint key sets
 * (_merge_states, patches/tpu-inference.patch:7174-7186).
 * partial_out: (parts, rows, head_dim) f32 normalised; partial_lse:
 * (parts, rows) f32 natural log, -inf for an empty part; row = token * nheads
 * + head.  sinks: NULL or (nheads,) f32, joins the denominator once.
 * out: (rows, head_dim) bf16; lse: NULL or (rows,) f32 with stride given by
 * lse_head_stride / lse_token_stride (elements) so it can land in the
 * (batch, nheads, seqlen_q) layout.
 */
typedef struct FwCombineArgs {
  const float* partial_out;
  const float* partial_lse;
  const float* sinks;
  void* out;
  float* lse;
  int32_t parts;
  int32_t rows;
  int32_t nheads;
  int32_t head_dim;
  int32_t lse_head_stride;
  int32_t lse_token_stride;
  /* Elements between consecutive parts of partial_out / partial_lse; 0 means
   * contiguous (rows * head_dim and rows).  Lets the merge read an all-gather
   * buffer whose per-rank slice is [o rows | lse rows] without a repack. */
  int64_t part_stride_out;
  int64_t part_stride_lse;
} FwCombineArgs;

int fw_lse_combine(const FwCombineArgs* args, void* stream);

/*
 * Exchange + merge of per-rank attention states without a collective library:
 * for one long request whose pages are split over the GPUs of a node, every
 * rank runs fw_decode_kvcache in partial-state mode and then this call, which
 * stores the rank's (o, lse) state into every peer's exchange buffer over
 * NVLink as {value, epoch} pairs (each 8-byte store carries its own flag, so
 * there is no separate flag and no system-scope fence), polls (with an
 * iteration limit; FW_STATUS_WAIT_TIMEOUT in *status when a peer does not
 * deliver) its own buffer until every rank's pairs carry the step's epoch and
 * merges the gathered states like fw_lse_combine.  Two launches, capturable in
 * a CUDA graph; every rank must make the same sequence of calls.  With
 * state_out = state_lse = NULL only the merge is enqueued: the states were
 * delivered by fw_sharded_decode_step(deliver_only = 1).  fw_sharded_decode_step
 * is the fused form of the whole step and what a serving loop should call.
 * (No counterpart in the reference, whose library is single-device; the merge
 * is _merge_states, patches/tpu-inference.patch:7174-7186.)
 *
 * Exchange buffers: fw_peer_alloc allocates and zeroes one of
 * fw_exchange_buffer_bytes on the current device and returns a 64-byte handle;
 * the host program passes the handles between the ranks' processes, each rank
 * maps its peers' buffers with fw_peer_open (which also enables peer access)
 * and lists all of them, its own included, in peer_buffers[0 .. world).  These
 * four routines allocate / map memory and belong to set-up, not to the step.
 */
typedef struct FwExchangeArgs {
  void* const* peer_buffers;  /* host array of `world` device pointers */
  const float* state_out;     /* (rows, head_dim) f32: partial_out of the decode call */
  const float* state_lse;     /* (rows,) f32 */
  const float* sinks;         /* NULL or (nheads,) */
  void* out;                  /* (rows, head_dim) bf16 */
  float* lse;                 /* NULL or strided like FwCombineArgs.lse */
  int32_t* status;            /* NULL or a device status word */
  int32_t world;
  int32_t rank;
  int32_t rows;
  int32_t nheads;
  int32_t head_dim;
  int32_t lse_head_stride;
  int32_t lse_token_stride;
  /* Optional round-robin bookkeeping (see fw_shard_step), advanced by the merge
   * once the step is complete so the NEXT step needs no launch for it: when
   * global_len is not NULL the merge adds `advance` to *global_len and writes
   * *local_len / *append_enable for the new length.  Prime the three words with
   * fw_shard_step(advance = 0) before the first step. */
  int32_t* global_len;
  int32_t* local_len;
  int32_t* append_enable;
  int32_t page_size;
  int32_t advance;
} FwExchangeArgs;

uint64_t fw_exchange_buffer_bytes(int32_t world, int32_t rows, int32_t head_dim);

/*
 * Per-step bookkeeping of one request whose logical pages are dealt round-robin
 * over the GPUs: logical page p lives on GPU p % world as that GPU's local page
 * p / world, so the growing tail of a long generation keeps moving from GPU to
 * GPU and every GPU holds the same number of pages to within one.  One thread
 * reads *global_len (tokens cached before this step) and writes
 *   *local_len     = how many of those tokens live in this rank's pages (they
 *                    are a prefix of its local page list), and
 *   *append_enable = 1 on the rank whose page holds position *global_len (for
 *                    that rank local_len is exactly the new token's local
 *                    position), 0 elsewhere,
 * then adds `advance` to *global_len.  Enqueue it before fw_decode_kvcache
 * (cache_seqlens = local_len, append_enable as given) every step: the same
 * captured sequence then serves a whole generation, across page and rank
 * boundaries.  (No counterpart in the reference, whose library is
 * single-device.)
 */
typedef struct FwShardStepArgs {
  int32_t* global_len;
  int32_t* local_len;
  int32_t* append_enable;
  int32_t page_size;
  int32_t world;
  int32_t rank;
  int32_t advance;
} FwShardStepArgs;

int fw_shard_step(const FwShardStepArgs* args, void* stream);

/*
 * One decode step of a request whose pages are split over the GPUs of a node,
 * as three launches: the decode kernel over this rank's pages (with the fused
 * append where append_enable says so), the combine kernel, which stores the
 * rank's sink-free (o, lse) state straight into every rank's exchange buffer
 * over NVLink ({value, epoch} pairs: compute and delivery in one kernel), and
 * the merge kernel, which waits - bounded - for all ranks' states, folds the
 * sink in and writes decode.out / decode.lse on every rank.  decode is filled
 * as for fw_decode_kvcache (workspace of fw_decode_workspace_bytes; out / lse /
 * sinks describe the MERGED result; partial_out / partial_lse NULL; one request
 * or one-token requests; head_dim 128 or 256).  When global_len is not NULL the
 * merge also advances the round-robin bookkeeping for the next step (see
 * FwExchangeArgs), so a captured graph of this one call serves a whole
 * generation.  deliver_only = 1 stops after the delivery (the merge is then
 * enqueued with fw_state_exchange_merge, state_out = NULL): for tests that play
 * several ranks on one GPU, where no kernel may wait for a later one.
 * Device-side trouble is reported in the status word at the head of
 * decode.workspace.
 */
typedef struct FwShardedDecodeArgs {
  FwDecodeArgs decode;
  void* const* peer_buffers;  /* host array of `world` device pointers, own buffer included */
  int32_t world;
  int32_t rank;
  int32_t* global_len;        /* NULL, or the three bookkeeping words */
  int32_t* local_len;
  int32_t* append_enable;
  int32_t advance;
  int32_t deliver_only;
} FwShardedDecodeArgs;

int fw_sharded_decode_step(const FwShardedDecodeArgs* args, void* stream);
int fw_peer_alloc(uint64_t bytes, void** ptr, void* handle64);
int fw_peer_open(const void* handle64, void** ptr);
int fw_peer_close(void* ptr);
int fw_peer_free(void* ptr);
int fw_state_exchange_merge(const FwExchangeArgs* args, void* stream);

/* Copies the device status word at the head of `workspace` to *status (host)
 * and clears it on the device if it was set.  Synchronises `stream`; meant for
 * tests and debugging, not the hot path. */
int fw_read_status(const void* workspace, void* stream, int32_t* status);

/* Failure-detection self test: launches one CTA whose bounded wait can never
 * be satisfied (a barrier nothing arrives on).  After at most spin_limit polls
 * (capped at 2^20) it records FW_STATUS_WAIT_TIMEOUT in the status word at the
 * head of `workspace` and returns; the context stays usable.  No fault, trap
 * or endless loop is involved.  (No counterpart in the reference, which has no
 * runtime error channel.) */
int fw_selftest_wait_timeout(void* workspace, uint32_t spin_limit, void* stream);

/* Thread-local text of the last error on this thread ("" if none). */
const char* fw_last_error(void);

/* ABI version: bumped when a struct above changes. */
int fw_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLYWHEEL_B200_H_ */
