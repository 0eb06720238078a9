/*
 * C ABI of the B200 fused score + exact Top-K operator (libitk_b200.so).
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, never allocates, never synchronises and never
 * writes its inputs ("_out" convention: the caller owns every buffer).  The
 * return value is 0 on success or a negative ITK_ERR_* code; itk_last_error()
 * gives the message of the calling thread's last failure.  Conditions found on
 * the device (a row the fast path could not prove complete, an inconsistent
 * repair, an expired bounded wait) are reported in device memory: the per-row
 * failure / repair-error flags and the status word.
 *
 * Each declaration names the reference interface it replaces (paths relative to
 * the reference repository root).
 *
 * Tensor contract (src/fused_index_topk/kernel/csrc/long_fused_bindings.cpp:119-153):
 *   q         [Q,64,128]  fp8 e4m3, contiguous, 16-byte aligned
 *   kv        [N,128]     fp8 e4m3, contiguous, 16-byte aligned
 *   kv_scales [N]         fp32
 *   weights   [Q,64]      fp32, 16-byte aligned
 *   k_start, k_end [Q]    int32, end-exclusive key range of each query row
 *   scores are kv_scales[n] * sum_h weights[q,h] * relu(sum_d q[q,h,d]*kv[n,d])
 */
#ifndef ITK_B200_H
#define ITK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* itk_stream_t;

#define ITK_OK 0
#define ITK_ERR_ARGUMENT (-1)
#define ITK_ERR_CUDA (-2)
#define ITK_ERR_UNSUPPORTED (-3)

#define ITK_TOP_K 2048
#define ITK_HEADS 64
#define ITK_HEAD_DIM 128
#define ITK_BLOCK_Q 4
#define ITK_REPAIR_CHUNK 16384
#define ITK_SPILL_U64_PER_ROW 5632      /* 4 segments x 1408 entries */
#define ITK_MAX_KEYS 262144             /* 16-bit segment-relative candidate ids */
#define ITK_MAX_PAIR_SOURCES 16
#define ITK_MAX_CTAS 256                /* the fused kernel's grid never exceeds this (one CTA per SM) */

/* bits of the device status word */
#define ITK_STATUS_WAIT_EXPIRED 1

/* values of the per-row repair error flag */
#define ITK_REPAIR_ERR_COUNT 1
#define ITK_REPAIR_ERR_LOCAL_SELECT 2
#define ITK_REPAIR_ERR_MERGE_SELECT 3

/* Library identity and one-time per-device set-up (raises the dynamic shared-memory
 * limit of the kernels).  itk_init is idempotent and is also called lazily. */
const char* itk_version(void);
const char* itk_last_error(void);
int itk_init(int device);

/* Registers, shared memory and launch shape of every kernel, as "name=value" lines.
 * Replaces resource_report() (sampling_threshold.cu:294-309, long_context_repair.cu:629-651). */
int itk_resource_report(char* buffer, size_t buffer_bytes);

/* Bytes the caller must provide for each workspace of a Q x N problem split into
 * `shards` key ranges.  Replaces the allocations of FusedIndexTopK.prepare
 * (src/fused_index_topk/kernel/plugin.py:202-257). */
typedef struct itk_workspace_sizes {
    size_t spill_bytes;            /* uint64 [min(4*ceil(Q/4)*shards, 4*ITK_MAX_CTAS),4,1408]: one region per CTA
                                    * and row of the CTA's current unit, not per query row */
    size_t repair_pairs_bytes;     /* uint64 [shards*Q,16384] */
    size_t pairs_bytes;            /* uint64 [shards,Q,2048]: local / accumulator / output pairs, each */
    size_t counts_bytes;           /* int32  [shards,Q] */
    size_t flags_bytes;            /* uint8  [shards,Q] */
    size_t thresholds_bytes;       /* float  [shards,Q] */
    size_t chunk_ranges_bytes;     /* int32  [chunks,Q], each of start and end */
    int repair_chunks;
} itk_workspace_sizes;
int itk_workspace_bytes(int rows, int keys, int shards, itk_workspace_sizes* sizes);

/* sampled_kv[s,:] = kv[sample_ids[s],:], sampled_scales[s] = kv_scales[sample_ids[s]].
 * Replaces gather_out (sampling_threshold.cu:185-234). */
int itk_gather_sampled_kv(const void* kv, const float* kv_scales, const int32_t* sample_ids, void* sampled_kv,
                          float* sampled_scales, int keys, int samples, itk_stream_t stream);

/* Threshold prepass in one launch: scores of every query row against the S gathered
 * sample keys on the tensor cores, then per row the sample_rank-th largest score among
 * samples whose key position lies in [k_start,k_end) and whose score is finite;
 * -inf when k_end-k_start <= target_candidates or fewer than sample_rank samples are
 * valid.  Replaces deep_gemm.fp8_mqa_logits on the sample (kernel/plugin.py:272-282)
 * followed by threshold_out (sampling_threshold.cu:236-292).  diag_logits (optional,
 * fp32 [Q,diag_stride]) receives the dense sampled scores; trace (optional, int64 [CTAs,32])
 * the per-CTA phase trace.  Either selects the diagnostic build.  Only the query blocks
 * block_begin + i * block_stride, i < num_blocks, are scored (the blocks one rank owns; 0, 1,
 * ceil(Q/4) for all of them); the thresholds of the other rows are left alone.  With
 * exit_when_no_keys the launch returns at once, writing nothing, when every row's key range is
 * empty (the compacted retry problem of a call without flagged rows). */
int itk_sample_thresholds(const void* q, const void* sampled_kv, const float* sampled_scales, const float* weights,
                          const int32_t* sample_ids, const int32_t* k_start, const int32_t* k_end,
                          float* thresholds, int rows, int samples, int sample_rank, int target_candidates,
                          int block_begin, int block_stride, int num_blocks, int exit_when_no_keys,
                          float* diag_logits, long long diag_stride, long long* trace, int* status,
                          itk_stream_t stream);

/* Arguments of the fused kernel.  Replaces fp8_mqa_topk_out
 * (kernel/csrc/long_fused_bindings.cpp:100-184). */
typedef struct itk_fused_args {
    const void* q;
    const void* kv;
    const float* kv_scales;
    const float* weights;
    const int32_t* k_start;
    const int32_t* k_end;
    const float* thresholds;    /* [Q] */
    int32_t* out_ids;           /* [Q,2048]; may be null when out_pairs is given or every block is split */
    uint64_t* out_pairs;        /* optional [Q,2048]: (ordered score << 32) | key */
    int32_t* out_counts;        /* optional [Q], with out_pairs */
    uint8_t* failure_flags;     /* [Q]: 1 = row must be repaired */
    uint64_t* spill;            /* scratch of itk_workspace_sizes.spill_bytes: bounded overflow of the
                                 * shared-memory candidate lists, one region per CTA and unit row */
    uint64_t* shard_pairs;      /* with shards > 1: [shards,Q,2048] pairs, [shards,Q] counts and [shards,Q] */
    int32_t* shard_counts;      /* overflow flags of the key shards of the split blocks, for          */
    uint8_t* shard_flags;       /* itk_merge_shard_lists; rows of whole blocks are not touched        */
    float* diag_logits;         /* optional fp32 [Q,diag_stride] dense scores (-inf outside the range) */
    long long diag_stride;
    long long* trace;           /* optional int64 [CTAs,32] phase trace; selects the diagnostic build.
                                 * Counterpart of the ITK_LONG_DIAGNOSTIC trace
                                 * (kernel/csrc/include/fused_index_topk/long_cta_topk.cuh:8-29) */
    int* status;                /* device status word (or-ed) */
    unsigned long long wait_limit_ns; /* wall-clock limit of every wait inside the kernel; 0 = 2 s.  A wait that
                                 * runs out sets bit 0 of *status, the kernel drains and returns */
    int withhold_loads;         /* diagnostic build only, for tests of the expiry path: the kernel issues no
                                 * load, so its first wait runs into wait_limit_ns and it returns with the
                                 * status bit set; nothing is computed */
    int rows;                   /* Q */
    int keys;                   /* N */
    int key_lo;                 /* first key scored (multiple of 128) */
    int key_hi;                 /* one past the last key scored */
    int shards;                 /* the key range of a split block is cut into this many equal shards (>= 1) */
    int split_blocks;           /* with shards > 1: how many of the owned blocks are split, namely the ones with the
                                 * lowest block numbers (the fewest keys under a causal mask); 0 = all of them.
                                 * A launch runs its units in waves of one per SM; splitting the blocks of the
                                 * last, partly filled wave fills it.  A shard uses the row's threshold and
                                 * returns everything it found when that is fewer than 2048 candidates; the
                                 * merge decides whether the row is complete.  Whole blocks write out_ids /
                                 * out_pairs and failure_flags as with shards = 1. */
    int block_begin;            /* first owned block of 4 query rows */
    int block_stride;           /* stride between owned blocks (number of ranks) */
    int num_blocks;             /* owned blocks */
    int force_compute;          /* 1: score rows even when all their keys are selected anyway */
    int max_ctas;               /* 0 = one CTA per SM; otherwise the grid is capped (the reference plugin's
                                 * debug_ctas option, kernel/plugin.py:95-130) */
    int exit_when_no_keys;      /* 1: return at once, writing nothing, when every row's key range is empty
                                 * (the compacted retry problem of a call without flagged rows) */
    const int32_t* tile_table;  /* paged keys (null = contiguous): physical 128-key tile of each logical
                                 * tile, [ceil(keys/128)], every entry in [0, physical_keys/128).  kv and
                                 * kv_scales then are the physical pool ([physical_keys,128], [physical_keys]);
                                 * ids, ranges and `keys` stay logical.  Not offered with diag_logits. */
    int physical_keys;          /* rows of the pool, a multiple of 128 (ignored without tile_table) */
    /* Thresholds computed inside this launch (sampled_kv != null): every whole block scores the `samples`
     * gathered sample keys (itk_gather_sampled_kv) in front of its own keys, with the query tile it has in
     * shared memory anyway, and takes each row's threshold from them by the rule of itk_sample_thresholds
     * (same arithmetic, same result); the threshold is also written to thresholds_out [Q].  This saves the
     * separate prepass launch and its second read of q; it pays while the threshold is picked by one warp
     * (samples <= 512, contexts up to 32 K keys).  Needs key_lo = 0 and key_hi = keys.  The shards of split
     * blocks still read `thresholds`, which the caller fills for their rows with itk_sample_thresholds
     * (`thresholds` and thresholds_out may be the same buffer). */
    const void* sampled_kv;     /* [samples,128] e4m3, 16-byte aligned */
    const float* sampled_scales;/* [samples] */
    const int32_t* sample_ids;  /* [samples] key position of every sample */
    float* thresholds_out;      /* [Q] */
    int samples;
    int sample_rank;
    int target_candidates;
} itk_fused_args;
int itk_fused_topk(const itk_fused_args* args, itk_stream_t stream);

/* chunk_start/chunk_end [chunks,Q]: the row ranges rebased into each 16384-key chunk.
 * Replaces update_ranges_out ( long_context_repair.cu:671-701; kernel :653-669). */
int itk_update_chunk_ranges(const int32_t* k_start, const int32_t* k_end, int32_t* chunk_start,
                            int32_t* chunk_end, int rows, int keys, itk_stream_t stream);

/* For rows whose failure flag is set: recompute the scores of keys
 * [chunk_lo, chunk_hi) (at most 16384) and write every pair to
 * repair_pairs[row, key-chunk_lo] (0 where the key is outside the row's range).
 * Replaces produce_repair_candidates_out (kernel/csrc/repair/repair_producer_bindings.cpp:19-30). */
int itk_repair_produce(const void* q, const void* kv, const float* kv_scales, const float* weights,
                       const int32_t* k_start, const int32_t* k_end, const uint8_t* failure_flags,
                       uint64_t* repair_pairs, int rows, int keys, int chunk_lo, int chunk_hi, int block_begin,
                       int block_stride, int num_blocks, int* status, itk_stream_t stream);

/* Exact Top-2048 pairs of one chunk for flagged rows.  chunk_start/chunk_end are the
 * chunk-local ranges of itk_update_chunk_ranges (the number of live pairs must equal
 * their difference, else repair error 1).  Replaces local_topk_pairs_out
 * (long_context_repair.cu:467-527). */
int itk_chunk_local_topk(const uint64_t* repair_pairs, const int32_t* chunk_start, const int32_t* chunk_end,
                         const uint8_t* failure_flags, uint64_t* local_pairs, int32_t* local_counts,
                         uint8_t* repair_error_flags, int rows, int first_chunk, itk_stream_t stream);

/* accumulator <- Top-2048(accumulator U local) for flagged rows.  Replaces
 * merge_topk_pairs_out (long_context_repair.cu:529-576). */
int itk_merge_topk_pairs(uint64_t* accumulator_pairs, int32_t* accumulator_counts, const uint64_t* local_pairs,
                         const int32_t* local_counts, const uint8_t* failure_flags, uint8_t* repair_error_flags,
                         int rows, int first_chunk, itk_stream_t stream);

/* Repaired rows: ids (and optionally pairs / counts) into the operator output, flag
 * cleared.  Replaces finalize_repair_out (long_context_repair.cu:578-616). */
int itk_finalize_repair(const uint64_t* accumulator_pairs, const int32_t* accumulator_counts, int32_t* out_ids,
                        uint64_t* out_pairs, int32_t* out_counts, uint8_t* failure_flags,
                        const uint8_t* repair_error_flags, int rows, itk_stream_t stream);

/* Exact Top-2048 of the union of `sources` candidate lists per row, each
 * [Q,2048] pairs with [Q] counts: the merge step after key-range sharding, across
 * shards of one GPU or across the all-gathered per-GPU candidates.  A row is flagged
 * in failure_flags (optional) when the union holds fewer than min(2048, valid) pairs.
 * Has no counterpart kernel in the reference (which is single-GPU); it applies the
 * selection rule of select_topk_pairs (long_context_repair.cu:139-235). */
int itk_merge_candidate_lists(const uint64_t* const* source_pairs, const int32_t* const* source_counts,
                              int sources, int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts, int rows,
                              itk_stream_t stream);

/* itk_merge_candidate_lists for the key shards of ONE itk_fused_topk launch (shards > 1),
 * which also decides per row whether the result is complete:
 * failure_flags[row] = 1 when any shard of the row reported an overflow
 * (shard_flags [sources, rows]) or the union holds fewer than
 * min(2048, number of keys of the row inside [key_lo, key_hi)) pairs, else 0.  Such rows
 * go to the repair graph.  Only the rows of the query blocks block_begin + i * block_stride,
 * i < num_blocks, are merged (num_blocks = 0: every row).  With out_rows (int32 [rows], optional)
 * the lists, k_start and k_end are those of a compacted problem and row r's ids, pairs, count and
 * flag go to row out_rows[r] of the outputs; r is skipped when out_rows[r] < 0.  mirror_ids
 * (optional, [Q,2048]) receives a second copy of the ids of every row written: a caller that has
 * already copied the fast path's ids to the host passes the mapped host buffer here, so that
 * repaired rows reach it without another copy of the whole output.
 * No counterpart in the reference (one unit per query block there). */
int itk_merge_shard_lists(const uint64_t* const* source_pairs, const int32_t* const* source_counts, int sources,
                          int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts, int rows,
                          const uint8_t* shard_flags, uint8_t* failure_flags, const int32_t* k_start,
                          const int32_t* k_end, int key_lo, int key_hi, int block_begin, int block_stride,
                          int num_blocks, const int32_t* out_rows, int32_t* mirror_ids, itk_stream_t stream);

/* A scope of launches that only matter when a row is flagged (the whole repair stage).  When `stream`
 * is being captured into a CUDA graph, begin adds a one-CTA kernel that looks at failure_flags [rows]
 * and an IF node after it, and returns in *body_stream a stream that captures the node's body: what
 * the caller launches on it until itk_flagged_scope_end runs, in a replay, only if some row was
 * flagged; a replay without flagged rows then pays for two graph nodes instead of for every launch of
 * the stage.  Work enqueued on `stream` after the scope is ordered after the body.  Outside a capture
 * (or where the driver offers no conditional nodes) *body_stream is `stream` itself and the launches
 * run as they are; each of them returns at once on the device when it finds no flagged row.  One
 * scope at a time per device (the library keeps one body stream per device); the first call on a
 * device should come outside a capture, like every other entry point's.  The reference launches its
 * repair graph unconditionally (src/fused_index_topk/kernel/plugin.py:333-377). */
int itk_flagged_scope_begin(const uint8_t* failure_flags, int rows, itk_stream_t stream, itk_stream_t* body_stream);
int itk_flagged_scope_end(itk_stream_t stream, itk_stream_t body_stream);

/* First stage of the retry of flagged rows: the b-th flagged row (in row order) becomes row b of a
 * compact problem of `slots` rows: its query tile, head weights and key range are copied to
 * q_out [slots,64,128], weights_out [slots,64], k_start_out / k_end_out [slots], and slot_rows[b]
 * names it.  Slots beyond the number of flagged rows get an empty key range and slot_rows[b] = -1;
 * flagged rows beyond the slots stay flagged for the dense repair.  The compact problem is then run
 * through itk_sample_thresholds (a lower threshold), itk_fused_topk with key shards and
 * itk_merge_shard_lists with out_rows = slot_rows, which costs the scores of the flagged rows only.
 * The reference repairs every flagged row by the dense rescan (src/fused_index_topk/kernel/plugin.py:333-377). */
int itk_compact_flagged_rows(const uint8_t* failure_flags, const void* q, const float* weights, const int32_t* k_start,
                             const int32_t* k_end, int rows, int slots, void* q_out, float* weights_out,
                             int32_t* k_start_out, int32_t* k_end_out, int32_t* slot_rows, itk_stream_t stream);

/* itk_chunk_local_topk, itk_merge_topk_pairs and (on the last chunk) itk_finalize_repair in one launch:
 * accumulator <- Top-2048(accumulator U the dense pairs of chunk [chunk_lo, chunk_hi)) for flagged rows;
 * the chunk-local key range of each row is derived from k_start / k_end here, so no
 * itk_update_chunk_ranges launch is needed.  With last_chunk the result goes to out_ids / out_pairs /
 * out_counts (and a second copy of the ids to mirror_ids, optional, as in itk_merge_shard_lists)
 * instead and a complete row's failure flag is cleared.  Error codes as in the separate
 * steps (count mismatch 1, selection 3).  Same kernels of the reference as those three
 * (long_context_repair.cu:237-426), launched there once each per chunk. */
int itk_repair_merge_chunk(uint64_t* accumulator_pairs, int32_t* accumulator_counts, const uint64_t* repair_pairs,
                           const int32_t* k_start, const int32_t* k_end, int chunk_lo, int chunk_hi,
                           uint8_t* failure_flags, uint8_t* repair_error_flags, int rows, int first_chunk,
                           int last_chunk, int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts,
                           int32_t* mirror_ids, itk_stream_t stream);

/* Paged forms of itk_gather_sampled_kv and itk_repair_produce: the keys live in a pool of
 * 128-key physical tiles addressed through tile_table as in itk_fused_args.  The reference
 * has no paged layout (src/fused_index_topk/inputs.py:31-32 rejects it); these exist for
 * serving stacks that keep the index keys in a paged cache. */
int itk_gather_sampled_kv_paged(const void* kv, const float* kv_scales, const int32_t* sample_ids,
                                const int32_t* tile_table, void* sampled_kv, float* sampled_scales, int keys,
                                int physical_keys, int samples, itk_stream_t stream);
int itk_repair_produce_paged(const void* q, const void* kv, const float* kv_scales, const float* weights,
                             const int32_t* k_start, const int32_t* k_end, const uint8_t* failure_flags,
                             uint64_t* repair_pairs, int rows, int keys, int chunk_lo, int chunk_hi, int block_begin,
                             int block_stride, int num_blocks, const int32_t* tile_table, int physical_keys,
                             int* status, itk_stream_t stream);

/* Row-wise e4m3 quantisation of operator inputs on the device: the step before the
 * operator.  For each of `rows` rows of ITK_HEAD_DIM elements
 *   scale = max(amax(|x|), 1e-4) / 448 (fp32), value = e4m3(x / scale) with IEEE fp32
 *   division and round-to-nearest-even,
 * the arithmetic of quantize_contiguous_index_kv (src/fused_index_topk/inputs.py:76-90),
 * which the reference runs in torch; results are bit-identical to it for finite inputs.
 * source_dtype: ITK_SOURCE_F32 or ITK_SOURCE_BF16.  `values` gets [rows,128] e4m3 bytes.
 * `scales` ([rows] fp32) may be null when a fold is requested.  With fold and folded set
 * (both [rows] fp32, may alias) folded[r] = fold[r] * scale[r]: quantised queries
 * ([Q*64,128] rows) carry their scale in the head weights, because the operator has no
 * query-scale argument (src/fused_index_topk/contract.py:152-185). */
#define ITK_SOURCE_F32 0
#define ITK_SOURCE_BF16 1
int itk_quantize_rows_e4m3(const void* source, int source_dtype, const float* fold, float* folded, void* values,
                           float* scales, long long rows, itk_stream_t stream);

/* The fused kernel for callers that must not allocate device memory.
 *
 * Some hosts of this operator cannot call cudaMalloc at the point where they run it:
 * an inference engine that has handed the whole device to its own pool allocator and
 * forbids foreign allocations, a plugin loaded into a process whose memory budget is
 * fixed at start-up, or code running inside a region where allocation would
 * synchronise the device.  itk_fused_topk needs one scratch buffer from its caller
 * (the bounded overflow spill, 45056 bytes per CTA and unit row); this variant takes the
 * spill from an array that is part of the library image instead, so the caller passes
 * only inputs, thresholds and outputs.  It has no counterpart in the reference, whose
 * host bindings always receive the spill workspace from the Python plugin.
 *
 * Limits and rules:
 *  - at most ITK_STATIC_MAX_ROWS query rows per call (larger problems are rejected with
 *    ITK_ERR_ARGUMENT; split them by rows); args->spill must be null;
 *    key-range shards (shards > 1) are not offered here;
 *  - the array (ITK_STATIC_MAX_ROWS * 45056 bytes = 11 MiB) lives in every device
 *    context that loads the library, until the process exits;
 *  - the first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call outside any stream capture;
 *  - every call on a device shares the one array: two calls that overlap on the GPU
 *    (different streams, or graphs replayed concurrently) race on it and must be
 *    serialised by the caller.  Nothing in it needs to start at zero: a row's spill is
 *    only read up to the counts the same launch wrote. */
#define ITK_STATIC_MAX_ROWS 256
int itk_fused_topk_static(const itk_fused_args* args, itk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ITK_B200_H */
