/*
 * paged_attention_b200.h -- C ABI of the B200 paged-attention decode library
 * (libpaged_attention_b200.so).
 *
 * The four launch_kernels_* entry points replace, one for one, the four host
 * launchers of baodii/flash_attention_factory; each takes exactly the
 * quantities the reference's pybind shims unpack from their torch tensors
 * (paged_attention_loop/paged_attention_loop.cpp:44-79) and passes them in one
 * plain struct.  No torch types, no C++ types and no exceptions cross this
 * boundary: every function returns a pa_status code and the message of the
 * last failure on the calling thread is available from pa_last_error().
 *
 * Memory contract (same as the reference): every buffer is allocated and owned
 * by the caller and lives on the current CUDA device; the library allocates
 * nothing on the device.  The only state it keeps between calls is a table of
 * work counters inside its device image, of which every split-context launch
 * takes a row of its own and hands it back zeroed: calls on different streams
 * (with different scratch buffers) may overlap, and a launch recorded into a
 * CUDA graph keeps its row for every replay, in a range direct launches never use.
 *
 * Data layouts (reference paged_attention_kernel_loop.hpp:44-62):
 *   query        fp16  [num_seqs, num_heads, head_size]
 *   key_cache    fp16 or 1-byte FP8  [num_blocks, block_size, num_kv_heads, head_size]
 *   value_cache  same layout and type as key_cache
 *   block_tables int32 (read as uint32) [num_seqs, max_blocks_per_seq]
 *   context_lens int32 (read as uint32) [num_seqs]
 *   out          fp16  [num_seqs, num_heads, head_size]
 *   max_logits   fp32  [num_seqs, num_heads, max_num_partitions]       (reduce only)
 *   exp_sums     fp32  [num_seqs, num_heads, max_num_partitions]       (reduce only)
 *   tmp_out      fp16  [num_seqs, num_heads, max_num_partitions, head_size] (reduce only)
 *   sinks        fp16  [num_heads] or NULL
 */
#ifndef PAGED_ATTENTION_B200_H_
#define PAGED_ATTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_API __attribute__((visibility("default")))

typedef enum pa_status {
  PA_OK = 0,
  /* (head_size, block_size) or num_queries_per_tokens outside the supported
   * set; the message strings are the reference's own
   * (paged_attention_loop/launch_kernels_loop.h:114-115,170-172). */
  PA_ERR_UNSUPPORTED = 1,
  PA_ERR_BAD_ARG = 2, /* null pointer, inconsistent sizes, misaligned buffer */
  PA_ERR_CUDA = 3,    /* a CUDA runtime / driver call failed */
  PA_ERR_TIMEOUT = 4  /* a bounded device-side wait gave up (see pa_device_status) */
} pa_status;

typedef enum pa_kv_dtype {
  PA_KV_F16 = 0,
  PA_KV_FP8_E5M2 = 1, /* the format the reference bindings hard-wire
                         (paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:43) */
  PA_KV_FP8_E4M3 = 2  /* e4m3fn bit layout (no infinities, 0x7F/0xFF = NaN) */
} pa_kv_dtype;

typedef struct pa_params {
  /* outputs */
  void *out;          /* fp16 [num_seqs, num_heads, head_size] */
  float *max_logits;  /* reduce: written for partitions < ceil(ctx/partition_size) */
  float *exp_sums;    /* reduce: same indexing as max_logits */
  void *tmp_out;      /* reduce: fp16 per-partition normalised partial outputs */
  /* inputs */
  const void *query;
  const void *key_cache;
  const void *value_cache;
  const void *sinks;             /* nullable */
  const uint32_t *block_tables;
  const uint32_t *context_lens;
  /* sizes: the values the reference reads from tensor shapes
   * (paged_attention_loop/paged_attention_loop.cpp:60-65) */
  uint32_t num_seqs;               /* query.size(0) */
  uint32_t num_heads;              /* query.size(1) */
  uint32_t head_size;              /* query.size(2): 128 or 64 */
  uint32_t num_kv_heads;           /* key_cache.size(2) */
  uint32_t max_num_partitions;     /* max_logits.size(2); stride of the reduce scratch */
  uint32_t max_blocks_per_seq;     /* block_tables.size(1) */
  uint32_t block_size;             /* tokens per KV block: 16, 32, 64 or 128 */
  uint32_t num_queries_per_tokens; /* GQA group, 1..8; must equal num_heads / num_kv_heads */
  uint32_t max_context_len;        /* scheduling hint only (the reference ignores it); 0 = unknown */
  uint32_t reserved0;
  uint64_t num_blocks;             /* key_cache.size(0); bounds the TMA descriptor, so a
                                      block id >= num_blocks reads zeros instead of faulting */
  float sm_scale;
  float fp8_scale; /* per-tensor dequantisation scale of an FP8 cache; ignored for fp16 */
  int32_t kv_dtype; /* pa_kv_dtype; must match the entry point (fp16 vs FP8) */
  int32_t reserved1;
  /* Optional per-KV-head dequantisation scales of an FP8 cache (device pointers, fp32
   * [num_kv_heads] each, or NULL).  The reference has one scalar fp8_scale
   * (paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:34); when these are set,
   * K of head k dequantises as fp16(code) * k_scale_per_head[k] and V as
   * fp16(code) * v_scale_per_head[k], and fp8_scale is not used for that cache. */
  const float *k_scale_per_head;
  const float *v_scale_per_head;
  /* Opt-in score modifiers.  The reference accepts alibi_slopes and softcap and ignores
   * them (call sites commented out, paged_attention_kernel_loop.hpp:329-342), and so do the
   * Python run() shims; a caller of this ABI enables them by setting these fields:
   * score s of token t becomes softcap * tanh(s / softcap) if softcap > 0 (the formula of
   * the reference oracle, test_paged.py:92-95), then + alibi_slopes[h] * (t - (ctx - 1)) if
   * alibi_slopes != NULL (fp32 [num_heads], device pointer). */
  const float *alibi_slopes;
  float softcap;
  float reserved2;
  /* Optional subset launch (no reference counterpart): a device array of num_seqs sequence
   * ids.  The call then processes exactly those sequences; every tensor is still indexed
   * by the ids themselves (query[id], block_tables[id], out[id], scratch rows of id), so two
   * calls with disjoint lists can share all buffers, e.g. a loop launch for the short and a
   * reduce launch for the long sequences of one batch.  NULL = sequences 0 .. num_seqs-1. */
  const uint32_t *seq_indices;
  /* Optional packed block tables (no reference counterpart; the reference's table is the dense
   * [num_seqs, max_blocks_per_seq] tensor, paged_attention_loop/paged_attention_loop.cpp:57).
   * A device array of num_seqs + 1 offsets (indexed by sequence id like every other tensor):
   * block_tables then is one list of block ids and the row of sequence i is
   * block_tables[block_table_offsets[i] .. block_table_offsets[i + 1]); max_blocks_per_seq is
   * not used.  A ragged batch's tables shrink from num_seqs * max_blocks_per_seq entries to
   * the sum of ceil(ctx / block_size), which is what a host uploads per step.  A context
   * length beyond what its row holds is cut to it.  NULL = dense tables. */
  const uint32_t *block_table_offsets;
  /* Optional per-block dequantisation scales of an FP8 cache (no reference counterpart; the
   * reference has one scalar, paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:34): device
   * arrays fp32 [num_blocks, num_kv_heads], both or neither.  K of block b, head k dequantises as
   * fp16(code) * k_scale_per_block[b * num_kv_heads + k], V likewise; fp8_scale is then not
   * used and the per-head scales must be NULL. */
  const float *k_scale_per_block;
  const float *v_scale_per_block;
} pa_params;

/* Tiling knobs of include/paged_attention_policy_v2.hpp for one
 * (head_size, block_size, group) triple, as run-time values. */
typedef struct pa_policy_info {
  uint32_t partition_size;        /* tokens per partition of the reduce variant */
  uint32_t stages;                /* base policy pipeline depth of the reference (3) */
  uint32_t head_size_stride;      /* reference MMA k-slice (16) */
  uint32_t partition_stride;      /* merge kernel: partitions per step (8) */
  uint32_t max_partitions_per_sg; /* reference merge-kernel register rows */
  uint32_t tokens_per_stage;      /* this library: rows (KV heads x tokens) per shared-memory ring stage */
  uint32_t ring_stages;           /* this library: TMA ring depth for the fp16 cache */
  uint32_t ring_stages_fp8;       /* this library: TMA ring depth for an FP8 cache */
  uint32_t consumer_warps;        /* MMA warps per CTA (one more warp issues TMA) */
  uint32_t threads_per_cta;
} pa_policy_info;

/*
 * The four launchers.  `stream` is a cudaStream_t (NULL = default stream) of
 * the current device.  If `us_out` is NULL the call is asynchronous: kernels
 * are only enqueued.  If `us_out` is non-NULL the call blocks until the work
 * is done and stores device execution time in microseconds, reproducing the
 * reference's blocking launch-and-profile behaviour
 * (paged_attention_loop/launch_kernels_loop.h:32-34,51-53).
 */

/* fp16 KV cache, single pass.  Replaces dispatch_paged_attention_loop +
 * launch_paged_attn_loop (paged_attention_loop/launch_kernels_loop.h:16-54,56-173).
 * Writes `out` only; max_logits / exp_sums / tmp_out are accepted and unused, as
 * in the reference.  us_out[0] = kernel time. */
PA_API int launch_kernels_loop(const pa_params *p, void *stream, float *us_out);

/* fp16 KV cache, split-context: attention kernel per 512-token (256 for
 * head_size 64) partition + merge kernel.  Replaces dispatch_paged_attention +
 * launch_paged_attn_v2 (paged_attention_reduce/launch_kernels_reduce.h:18-78,80-197).
 * us_out[0] = attention kernel, us_out[1] = merge kernel. */
PA_API int launch_kernels_reduce(const pa_params *p, void *stream, float *us_out);

/* FP8 KV cache, single pass.  Replaces dispatch_paged_attention_fp8_loop +
 * launch_paged_attn_fp8_loop
 * (paged_attention_fp8_loop/launch_kernels_fp8_loop.h:17-56,58-175). */
PA_API int launch_kernels_fp8_loop(const pa_params *p, void *stream, float *us_out);

/* FP8 KV cache, split-context.  Replaces dispatch_paged_attention_fp8 +
 * launch_paged_attn_fp8_v2
 * (paged_attention_fp8_reduce/launch_kernels_fp8_reduce.h:16-76,78-196). */
PA_API int launch_kernels_fp8_reduce(const pa_params *p, void *stream, float *us_out);

/* Size in bytes of the scratch array built into the library for
 * launch_kernels_reduce_static_scratch (32 MiB, held by every GPU that loads the library). */
#define PA_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/* fp16 KV cache, split-context, for callers that cannot allocate device memory.
 * No counterpart in the reference: there the caller always allocates max_logits,
 * exp_sums and tem_output itself.
 *
 * Same computation and same two kernels as launch_kernels_reduce, but the
 * per-partition maxima, exp-sums and partial outputs are kept in a fixed
 * PA_STATIC_SCRATCH_BYTES array inside the library's device image, so a host
 * that may not call cudaMalloc (memory owned by a foreign pool, allocation
 * forbidden after start-up, no tolerance for the device-wide synchronisation
 * an allocation implies) can still run the split variant.  The call itself
 * allocates nothing, on the device or through any library, and is always
 * asynchronous on `stream` (no timing, no host synchronisation).
 *
 * The caller passes the inputs and `out` as usual; p->max_logits, p->exp_sums
 * and p->tmp_out are ignored and may be NULL; p->max_num_partitions must still
 * cover ceil(max context / partition size).  The call fails with
 * PA_ERR_BAD_ARG, before any work is enqueued, if
 *   2 * align256(4 * rows) + align256(2 * head_size * rows) > PA_STATIC_SCRATCH_BYTES,
 *   rows = num_seqs * num_heads * max_num_partitions,
 * or if p->seq_indices is not NULL: a subset launch addresses scratch rows by
 * sequence id, ids the host cannot see, so the fixed array cannot be sized for
 * it (use launch_kernels_reduce with caller scratch for subset launches).
 *
 * The first call on each device looks up the array's device address (with
 * that device current) and caches it; make that first call outside of any
 * stream capture.  All calls on a device share the one array and it keeps the
 * previous call's contents: two calls whose kernels overlap on the GPU (other
 * streams, other host threads) race on it, so serialise them.  Nothing in the
 * array needs clearing between calls. */
PA_API int launch_kernels_reduce_static_scratch(const pa_params *p, void *stream);

/* Host side of one decode step, for callers whose per-step inputs live in host memory. */
typedef struct pa_host_step {
  const void *host_in; /* pinned host staging buffer: whatever per-step inputs pa_params reads
                          (query, block tables, context lengths), packed by the caller */
  void *dev_in;        /* its device mirror; the pa_params pointers point into this buffer */
  uint64_t in_bytes;   /* bytes copied host_in -> dev_in before the launch (0: no upload) */
  void *host_out;      /* pinned host buffer that receives pa_params.out after the launch */
  uint64_t out_bytes;  /* bytes copied pa_params.out -> host_out (0: no download, e.g. because
                          pa_params.out already is device-visible pinned host memory and the
                          kernel writes the result there itself) */
} pa_host_step;

typedef enum pa_entry {
  PA_ENTRY_LOOP = 0,
  PA_ENTRY_REDUCE = 1,
  PA_ENTRY_FP8_LOOP = 2,
  PA_ENTRY_FP8_REDUCE = 3
} pa_entry;

/* One decode step with host buffers, in one call (no counterpart in the reference, whose
 * bindings take device tensors): upload of the step's inputs, the asynchronous form of the
 * chosen entry point, download of the result, all on `stream`; if `synchronize` is non-zero
 * the call returns after the stream has drained, i.e. when host_out (or the host memory behind
 * pa_params.out) holds the result.  Allocates nothing. */
PA_API int pa_decode_step_host(int32_t entry, const pa_params *p, const pa_host_step *io, void *stream,
                               int32_t synchronize);

/* Cuts num_seqs sequences into `parts` ranges of consecutive sequences with equal shares of the
 * KV tokens (host arithmetic, no reference counterpart): range r is [bounds[r], bounds[r + 1])
 * and ends behind the sequence whose cumulative context length reaches (r + 1) / parts of the
 * total; ranges may be empty.  Used for the sub-batches of pa_decode_step_host_batch and for
 * sharding a batch over GPUs by sequence.  `bounds` holds parts + 1 entries. */
PA_API int pa_split_by_kv_length(const uint32_t *context_lens, uint32_t num_seqs, uint32_t parts, uint32_t *bounds);

/* Host buffers of one decode step for pa_decode_step_host_batch: the caller's per-step inputs
 * and the result, each in pinned host memory, laid out like their device mirrors in pa_params. */
typedef struct pa_host_batch {
  const void *host_query;                   /* fp16 [num_seqs, num_heads, head_size] */
  const uint32_t *host_block_tables;        /* dense [num_seqs, max_blocks_per_seq], or the packed id list */
  const uint32_t *host_block_table_offsets; /* [num_seqs + 1] for packed tables, NULL for dense ones */
  const uint32_t *host_context_lens;        /* [num_seqs] */
  void *host_out;                           /* fp16 [num_seqs, num_heads, head_size] */
  uint32_t sub_batches;                     /* 0 = chosen from the step's size; 1 = no overlap; at most 8 */
  uint32_t flags;                           /* PA_STEP_* */
  /* Optional: the host inputs above all lie in ONE pinned staging block of staging_bytes at
   * host_staging, and the device mirrors in pa_params lie at the same offsets inside the device
   * block at dev_staging.  A step that is not cut into sub-batches then uploads the block with a
   * single copy instead of one per tensor (a small step is bound by copy latencies, not bytes). */
  const void *host_staging;
  void *dev_staging;
  uint64_t staging_bytes;
} pa_host_batch;

/* The kernels of the last sub-batch write their result straight into host_out (which then has
 * to be device-accessible pinned memory) instead of a download by the copy engine. */
#define PA_STEP_LAST_OUT_DIRECT 1u

/* One decode step with host buffers, pipelined (no counterpart in the reference).  The batch is
 * cut into sub-batches of consecutive sequences by KV tokens (the first and the last a third of
 * the size of the inner ones: their upload and download are the transfers nothing hides); the
 * upload of sub-batch k+1 (its rows of query, context lengths and block tables -- only the
 * entries in use when the tables are packed, see pa_params.block_table_offsets), the kernels of
 * sub-batch k and the download of sub-batch k-1 run at the same time, on two copy streams the
 * library creates once per device and on `stream`.  p holds the device mirrors (query,
 * block_tables, block_table_offsets, context_lens, out, and the scratch of the reduce entry
 * points), all caller-owned; p->seq_indices must be NULL.  A sub-batch is the same call with
 * every per-sequence pointer moved to its first row, so results are those of the chosen entry
 * point on the whole batch for the reduce entry points (bit for bit) and for the loop entry
 * points whenever the same cluster size is chosen.  With `synchronize` non-zero the call returns
 * when host_out holds the whole result; otherwise everything is ordered on `stream`.
 * Allocates no device memory.  One such call at a time per device. */
PA_API int pa_decode_step_host_batch(int32_t entry, const pa_params *p, const pa_host_batch *io, void *stream,
                                     int32_t synchronize);

/* What pa_decode_step_host_batch would do with these arguments: the number of sub-batches and
 * the bytes it moves host -> device and device -> host per step (host arithmetic only). */
PA_API int pa_host_batch_plan(const pa_params *p, const pa_host_batch *io, uint32_t *sub_batches,
                              uint64_t *h2d_bytes, uint64_t *d2h_bytes);

/* ---- several GPUs in one process (no reference counterpart: the reference is single-device,
 * paged_attention_loop/launch_kernels_loop.h:32-34) ---- */

/* Deals num_seqs sequences to `parts` parts, longest first, each to the part that holds the
 * fewest KV tokens so far (ties: lower sequence id, lower part): part_of[i] is the part of
 * sequence i.  Balanced to within a fraction of one sequence where consecutive ranges
 * (pa_split_by_kv_length) can be off by a whole long sequence. */
PA_API int pa_split_lpt(const uint32_t *context_lens, uint32_t num_seqs, uint32_t parts, uint32_t *part_of);

/* One shard of a batch: its GPU, its entry point and its argument block, whose pointers all
 * live on that GPU.  A shard by sequence holds some of the sequences with all heads; a shard
 * by KV head holds all sequences with num_kv_heads / N heads of both caches, the matching
 * query heads and the matching slice of `out`. */
typedef struct pa_device_shard {
  int32_t device; /* CUDA device ordinal */
  int32_t entry;  /* pa_entry */
  pa_params params;
} pa_device_shard;

/* Launcher of one shard; the default calls the library's own entry point for shard->entry. */
typedef int (*pa_shard_launch_fn)(int32_t entry, const pa_params *p, void *stream, void *user);

/* Run without any CUDA call (host threads, barrier and aggregation only; host-clock timing):
 * for tests of the driver logic on machines without a GPU, together with a `launch` stand-in. */
#define PA_MULTI_GPU_HOST_ONLY 1u

typedef struct pa_multi_gpu_options {
  uint32_t calls;            /* calls per shard inside the timed region, at least 1 */
  uint32_t warmup;           /* untimed calls per shard before the common start */
  uint32_t flags;            /* PA_MULTI_GPU_* */
  uint32_t reserved;
  pa_shard_launch_fn launch; /* NULL = the library's entry points */
  void *user;                /* passed to `launch` */
} pa_multi_gpu_options;

/* Runs the shards of one batch at the same time from this process: one host thread and one
 * stream per shard, `warmup` untimed calls each, a common start barrier, then `calls`
 * asynchronous calls per shard timed with CUDA events on the shard's stream.  Stores the mean
 * microseconds per call of the slowest shard (max over shards; the time of the whole batch) and,
 * if us_per_call_each is not NULL, of every shard.  There is no exchange between the shards.  If
 * shards fail, the others still finish; the call returns the first failing shard's code and
 * pa_last_error() names every failing shard.  Blocks until all shards are done.  Several shards
 * may name the same device (they then share it through separate streams). */
PA_API int pa_multi_gpu_run(const pa_device_shard *shards, uint32_t num_shards, const pa_multi_gpu_options *options,
                            float *us_per_call_max, float *us_per_call_each);

#define PA_GATHER_BY_SEQUENCE 0 /* shard i's rows follow those of shard i - 1 in dst */
#define PA_GATHER_BY_KV_HEAD 1  /* shard i's heads follow those of shard i - 1 in every row of dst */

/* Collects the shards' `out` tensors into dst [sum of num_seqs, num_heads, head_size] (by
 * sequence) or [num_seqs, dst_num_heads, head_size] (by KV head) on dst_device, with peer
 * copies, after the shards' work is done; blocks until the copies have finished.  The only
 * cross-GPU step of the path and not part of any timed region. */
PA_API int pa_multi_gpu_gather_out(const pa_device_shard *shards, uint32_t num_shards, int32_t mode,
                                   void *dst, int32_t dst_device, uint32_t dst_num_heads);

/* Arguments of pa_reshape_and_cache. */
typedef struct pa_cache_write_params {
  const void *key;             /* fp16 [num_tokens, num_kv_heads, head_size] */
  const void *value;           /* fp16 [num_tokens, num_kv_heads, head_size] */
  void *key_cache;             /* [num_blocks, block_size, num_kv_heads, head_size], fp16 or FP8 */
  void *value_cache;           /* same layout and type as key_cache */
  const int64_t *slot_mapping; /* [num_tokens]: block_id * block_size + row; negative = skip the token */
  uint32_t num_tokens;
  uint32_t num_kv_heads;
  uint32_t head_size;
  uint32_t block_size;
  uint64_t num_blocks;
  float fp8_scale;             /* stored = x / fp8_scale (the scale the attention entry points take) */
  int32_t kv_dtype;            /* pa_kv_dtype of the cache */
  /* Optional scales of an FP8 cache that take the place of fp8_scale, the very arrays the
   * attention entry points take under the same names (pa_params): per KV head, fp32
   * [num_kv_heads], or per block and KV head, fp32 [num_blocks, num_kv_heads].  K and V
   * both or neither, one kind at most; stored = x / scale of the token's head (and block).
   * All NULL (a zero-initialised tail) = fp8_scale. */
  const float *k_scale_per_head;
  const float *v_scale_per_head;
  const float *k_scale_per_block;
  const float *v_scale_per_block;
} pa_cache_write_params;

/* Appends new K/V tokens to the paged cache in the layout the attention entry points read
 * (reference paged_attention_kernel_loop.hpp:50-51), casting to the cache type: fp16 is
 * copied, FP8 is round-to-nearest-even of x / scale (fp8_scale, or the per-head / per-block
 * scale arrays when given), saturating to the largest finite code.  The reference has no device kernel for this step: its tests fill caches on the host
 * with torch casts (test_paged_fp8cache.py:180-203), which this call reproduces bit for bit for
 * values inside the format's range.  Asynchronous on `stream`. */
PA_API int pa_reshape_and_cache(const pa_cache_write_params *p, void *stream);

/* Compile-time policy of include/paged_attention_policy_v2.hpp as data
 * (reference include/paged_attention_policy_v2.hpp:5-100).  Returns
 * PA_ERR_UNSUPPORTED for triples the launchers reject. */
PA_API int pa_query_policy(uint32_t head_size, uint32_t block_size, uint32_t group,
                           pa_policy_info *info);

/* Partition size the reduce variant uses for a head size (512 / 256), i.e. the
 * divisor callers use to size max_logits / exp_sums / tmp_out; 0 if unsupported. */
PA_API uint32_t pa_partition_size(uint32_t head_size);

/* Message of the last non-PA_OK return on the calling thread ("" if none). */
PA_API const char *pa_last_error(void);

/* Reads (and clears) the device status word of the current device: 0 if no
 * kernel of this library ever gave up a bounded wait, else PA_ERR_TIMEOUT.
 * Synchronises the device. */
PA_API int pa_device_status(void);

/* Library version, "major.minor". */
PA_API const char *pa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_ATTENTION_B200_H_ */
