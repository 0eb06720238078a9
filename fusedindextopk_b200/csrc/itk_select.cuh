// Plain CUDA kernels around the fused kernel: the sample gather, the per-chunk
// range rebasing, and the exact Top-2048 reducers over packed
// (ordered score << 32 | key) pairs that serve the repair path, the merge of
// key-range shards and the merge of per-GPU candidates.
//
// Counterparts in the reference: gather_sampled_kv
// (kernel/csrc/sampling_threshold.cu:80-97); itk_update_chunk_ranges,
// itk_chunk_local_topk, itk_merge_topk_pairs, itk_finalize_repair
// (kernel/csrc/long_context_repair.cu:653-669, 237-339, 341-405, 407-426).
#pragma once

#include "itk_fused.cuh"

namespace itk {

constexpr int kPairThreads = 512;
constexpr int kPairCapacity = 16384;           // pairs one CTA can hold: 128 KB of shared memory
constexpr int kMaxPairSources = 8;

// ------------------------------------------------------------------ gather

// sampled_kv[s,:] = kv[ids[s],:] (128 bytes as 8 x 16 B), sampled_scales[s] = kv_scales[ids[s]].
// With a tile table, key position k is stored at row tile_table[k / 128] * 128 + k % 128.
__global__ void itk_gather_kernel(const uint8_t* __restrict__ kv, const float* __restrict__ kv_scales,
                                  const int32_t* __restrict__ sample_ids, const int32_t* __restrict__ tile_table,
                                  uint8_t* __restrict__ sampled_kv, float* __restrict__ sampled_scales, int samples) {
    const int work = blockIdx.x * blockDim.x + threadIdx.x;
    if (work >= samples * 8) return;
    const int sample = work >> 3;
    const int part = work & 7;
    long long source = sample_ids[sample];
    if (tile_table != nullptr) source = static_cast<long long>(tile_table[source >> 7]) * 128 + (source & 127);
    reinterpret_cast<uint4*>(sampled_kv)[work] = reinterpret_cast<const uint4*>(kv + source * kHeadDim)[part];
    if (part == 0) sampled_scales[sample] = kv_scales[source];
}

// ------------------------------------------------------------------ chunk ranges

// chunk_start[c,row] = clamp(k_start[row] - c*chunk, 0, width_c), same for the end,
// width_c = min(chunk, keys - c*chunk).
__global__ void itk_chunk_ranges_kernel(const int32_t* __restrict__ k_start, const int32_t* __restrict__ k_end,
                                        int32_t* __restrict__ chunk_start, int32_t* __restrict__ chunk_end, int rows,
                                        int chunks, int keys, int chunk) {
    const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long long>(rows) * chunks) return;
    const int c = static_cast<int>(index / rows);
    const int row = static_cast<int>(index - static_cast<long long>(c) * rows);
    const int offset = c * chunk;
    const int width = min(chunk, keys - offset);
    chunk_start[index] = min(width, max(0, k_start[row] - offset));
    chunk_end[index] = min(width, max(0, k_end[row] - offset));
}

// ------------------------------------------------------------------ pair reducers

struct PairSource {
    const uint64_t* pairs;    // [rows, capacity]
    const int32_t* counts;    // [rows] live entries per row; null: scan all `capacity` entries, 0 = empty
};

struct PairTopKParams {
    PairSource sources[kMaxPairSources];
    int num_sources;
    int first_source;               // sources below this index are ignored (empty accumulator)
    int capacity;                   // entries per row of every source
    int rows;
    int row_period;                 // > 0: `rows` counts (chunk, row) pairs, chunk-major; row_mask and error_flags
                                    // are indexed by row % row_period (one entry per query row)
    const uint8_t* row_mask;        // null, or only rows with row_mask[row] != 0 are processed
    uint8_t* error_flags;           // null, or per-row error code; rows with a nonzero code are skipped
    int clear_errors;               // reset error_flags[row] of processed rows first
    const int32_t* expect_start;    // null, or dense sources are scanned over [expect_start, expect_end) only
                                    // and the live-entry total must equal expect_end - expect_start
    const int32_t* expect_end;
    int error_count_mismatch;       // code stored when that check fails
    int error_selection;            // code stored when the selection is inconsistent
    uint64_t* out_pairs;            // null or [rows, 2048]
    int32_t* out_ids;               // null or [rows, 2048]
    int32_t* out_counts;            // null or [rows]
    uint8_t* clear_flags;           // null, or flag reset to 0 for rows that produced a full result
    // Merge of the key shards of one launch: verdict_flags[row] (null = off) becomes 1 when a shard of
    // the row overflowed (shard_flags [sources, rows]) or the union holds fewer than
    // min(2048, keys of the row inside [key_lo, key_hi)) pairs, else 0.
    uint8_t* verdict_flags;
    const uint8_t* shard_flags;
    const int32_t* k_start;
    const int32_t* k_end;
    int key_lo, key_hi;
};

__device__ __forceinline__ void write_shard_verdict(const PairTopKParams& p, int row, int produced) {
    if (p.verdict_flags == nullptr) return;
    int failed = 0;
    for (int s = 0; s < p.num_sources; ++s) failed |= p.shard_flags[static_cast<long long>(s) * p.rows + row];
    const int wanted = min(max(min(p.k_end[row], p.key_hi) - max(p.k_start[row], p.key_lo), 0), kTopK);
    p.verdict_flags[row] = (failed != 0 || produced < wanted) ? 1 : 0;
}

struct PairShared {
    int hist[256];
    int count;
    int sel_bin;
    int sel_greater;
    int gcount;
    int ecount;
    int skip;
};

// Exact Top-2048 of the union of up to eight pair lists per row.  One CTA per
// row (grid-strided); the union (at most 16384 pairs) is staged in shared memory,
// the 2048-th largest score is found by four 8-bit radix rounds over the ordered
// score bits, then everything above it and the needed number of ties are
// written.  Rows with at most 2048 pairs are copied through.
__global__ void __launch_bounds__(kPairThreads, 1) itk_pair_topk_kernel(const PairTopKParams p) {
    extern __shared__ __align__(16) uint64_t staged[];
    __shared__ PairShared sh;
    const int tx = threadIdx.x;
    const int lane = tx & 31;

    if (p.row_mask != nullptr) {
        // The usual case of the repair graph is that no row is flagged: look at all of this CTA's
        // rows at once instead of paying one dependent global load per row.
        int any = 0;
        for (int row = static_cast<int>(blockIdx.x) + tx * static_cast<int>(gridDim.x); row < p.rows;
             row += kPairThreads * static_cast<int>(gridDim.x))
            any |= p.row_mask[p.row_period > 0 ? row % p.row_period : row];
        if (__syncthreads_or(any) == 0) return;
    }

    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        __syncthreads();
        const int flag_row = p.row_period > 0 ? row % p.row_period : row;
        if (tx == 0) {
            int skip = 0;
            if (p.row_mask != nullptr && p.row_mask[flag_row] == 0) skip = 1;
            if (!skip && p.error_flags != nullptr) {
                if (p.clear_errors) p.error_flags[flag_row] = 0;
                else if (p.error_flags[flag_row] != 0) skip = 1;
            }
            sh.skip = skip;
            sh.count = 0;
            sh.gcount = 0;
            sh.ecount = 0;
        }
        __syncthreads();
        if (sh.skip) continue;

        // stage the live pairs of every source
        for (int s = p.first_source; s < p.num_sources; ++s) {
            const uint64_t* source = p.sources[s].pairs + static_cast<long long>(row) * p.capacity;
            const bool dense = p.sources[s].counts == nullptr;
            // a dense source is only defined inside the row's own range: entries outside it
            // were never written by the producer
            int first = 0;
            int live = dense ? p.capacity : min(p.sources[s].counts[row], p.capacity);
            if (dense && p.expect_start != nullptr) {
                first = max(p.expect_start[row], 0);
                live = min(p.expect_end[row], p.capacity);
            }
            for (int base = first & ~31; base < live; base += kPairThreads) {
                const int i = base + tx;
                const bool inside = i >= first && i < live;
                const uint64_t pair = inside ? source[i] : 0ull;
                const bool keep = inside && (!dense || pair != 0ull);
                const int position = warp_reserve(&sh.count, keep, lane);
                if (keep && position < kPairCapacity) staged[position] = pair;
            }
        }
        __syncthreads();
        const int count = sh.count;
        int error = 0;
        if (count > kPairCapacity) error = p.error_count_mismatch;
        if (p.expect_start != nullptr && count != p.expect_end[row] - p.expect_start[row])
            error = p.error_count_mismatch;
        if (error != 0) {
            if (tx == 0) {
                if (p.error_flags != nullptr) p.error_flags[flag_row] = static_cast<uint8_t>(error);
                if (p.out_counts != nullptr) p.out_counts[row] = 0;
                write_shard_verdict(p, row, 0);
            }
            continue;
        }

        uint64_t* out_pairs = p.out_pairs != nullptr ? p.out_pairs + static_cast<long long>(row) * kTopK : nullptr;
        int32_t* out_ids = p.out_ids != nullptr ? p.out_ids + static_cast<long long>(row) * kTopK : nullptr;
        if (count <= kTopK) {
            for (int i = tx; i < kTopK; i += kPairThreads) {
                const uint64_t pair = i < count ? staged[i] : 0ull;
                if (out_pairs != nullptr) out_pairs[i] = pair;
                if (out_ids != nullptr) out_ids[i] = i < count ? static_cast<int32_t>(static_cast<uint32_t>(pair)) : -1;
            }
            if (tx == 0) {
                if (p.out_counts != nullptr) p.out_counts[row] = count;
                if (p.clear_flags != nullptr && count == kTopK) p.clear_flags[row] = 0;
                write_shard_verdict(p, row, count);
            }
            continue;
        }

        uint32_t prefix = 0, mask = 0;
        int rank = kTopK;
#pragma unroll 1
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tx < 256) sh.hist[tx] = 0;
            __syncthreads();
            for (int i = tx; i < count; i += kPairThreads) {
                const uint32_t score = static_cast<uint32_t>(staged[i] >> 32);
                if ((score & mask) == prefix) atomicAdd(&sh.hist[(score >> shift) & 255u], 1);
            }
            __syncthreads();
            if (tx < 32) {
                int bins[8];
                int mine = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    bins[j] = sh.hist[tx * 8 + j];
                    mine += bins[j];
                }
                int suffix = mine;
#pragma unroll
                for (int offset = 1; offset < 32; offset <<= 1) {
                    const int other = __shfl_down_sync(0xffffffffu, suffix, offset);
                    if (tx + offset < 32) suffix += other;
                }
                int above = suffix - mine;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    const int through = above + bins[j];
                    if (above < rank && rank <= through) {
                        sh.sel_bin = tx * 8 + j;
                        sh.sel_greater = above;
                    }
                    above = through;
                }
            }
            __syncthreads();
            prefix |= static_cast<uint32_t>(sh.sel_bin) << shift;
            rank -= sh.sel_greater;
            mask |= 0xffu << shift;
        }
        const int equal_needed = rank;
        const int greater_total = kTopK - equal_needed;
        for (int base = 0; base < count; base += kPairThreads) {
            const int i = base + tx;
            const bool live = i < count;
            const uint64_t pair = live ? staged[i] : 0ull;
            const uint32_t score = static_cast<uint32_t>(pair >> 32);
            const bool greater = live && score > prefix;
            const bool equal = live && score == prefix;
            const int g = warp_reserve(&sh.gcount, greater, lane);
            const int e = warp_reserve(&sh.ecount, equal, lane);
            int position = -1;
            if (greater) position = g;
            else if (equal && e < equal_needed) position = greater_total + e;
            if (position >= 0 && position < kTopK) {
                // the staged copy is complete, so the output may alias a source
                if (out_pairs != nullptr) out_pairs[position] = pair;
                if (out_ids != nullptr) out_ids[position] = static_cast<int32_t>(static_cast<uint32_t>(pair));
            }
        }
        __syncthreads();
        if (tx == 0) {
            const bool consistent = equal_needed > 0 && sh.gcount == greater_total && sh.ecount >= equal_needed;
            if (!consistent) {
                if (p.error_flags != nullptr) p.error_flags[flag_row] = static_cast<uint8_t>(p.error_selection);
                if (p.out_counts != nullptr) p.out_counts[row] = 0;
            } else {
                if (p.out_counts != nullptr) p.out_counts[row] = kTopK;
                if (p.clear_flags != nullptr) p.clear_flags[row] = 0;
            }
            write_shard_verdict(p, row, consistent ? kTopK : 0);
        }
    }
}

// Rows that were flagged and fully repaired get their ids (and optionally their
// pairs) copied into the operator output, and their failure flag cleared.
__global__ void itk_finalize_repair_kernel(const uint64_t* __restrict__ accumulator_pairs,
                                           const int32_t* __restrict__ accumulator_counts,
                                           int32_t* __restrict__ out_ids, uint64_t* __restrict__ out_pairs,
                                           int32_t* __restrict__ out_counts, uint8_t* __restrict__ failure_flags,
                                           const uint8_t* __restrict__ repair_error_flags, int rows) {
    const int row = blockIdx.x;
    if (row >= rows || failure_flags[row] == 0) return;
    if (repair_error_flags[row] != 0 || accumulator_counts[row] != kTopK) return;
    for (int i = threadIdx.x; i < kTopK; i += blockDim.x) {
        const uint64_t pair = accumulator_pairs[static_cast<long long>(row) * kTopK + i];
        if (out_ids != nullptr) out_ids[static_cast<long long>(row) * kTopK + i] = static_cast<int32_t>(static_cast<uint32_t>(pair));
        if (out_pairs != nullptr) out_pairs[static_cast<long long>(row) * kTopK + i] = pair;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (out_counts != nullptr) out_counts[row] = kTopK;
        failure_flags[row] = 0;
    }
}

}  // namespace itk
