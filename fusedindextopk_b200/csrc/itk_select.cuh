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
constexpr int kPairCapacity = 16384 + 2048;    // pairs one CTA can hold (a dense chunk and one list): 144 KB of shared memory
constexpr int kMaxPairSources = 16;

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

// ------------------------------------------------------------------ flagged rows, compacted

// Slot b of the retry problem takes the b-th flagged row (in row order): its query tile, head weights
// and key range are copied into the compact arrays and slot_rows[b] names the row; slots beyond the
// number of flagged rows get an empty key range and slot_rows[b] = -1.  One CTA per slot; every CTA
// scans the flags itself (16 rows per thread and step), which for a few thousand rows is cheaper
// than a second launch that would hand out the slots.
constexpr int kCompactThreads = 256;

__global__ void __launch_bounds__(kCompactThreads) itk_compact_flagged_kernel(
    const uint8_t* __restrict__ flags, int rows, const uint4* __restrict__ q, const float* __restrict__ weights,
    const int32_t* __restrict__ k_start, const int32_t* __restrict__ k_end, uint4* __restrict__ q_out,
    float* __restrict__ weights_out, int32_t* __restrict__ k_start_out, int32_t* __restrict__ k_end_out,
    int32_t* __restrict__ slot_rows) {
    __shared__ int warp_sums[kCompactThreads / 32];
    __shared__ int found_row;
    const int tx = threadIdx.x;
    const int lane = tx & 31;
    const int slot = blockIdx.x;
    if (tx == 0) found_row = -1;
    int seen = 0;          // flagged rows below `base`
    bool located = false;
    for (int base = 0; base < rows && !located; base += kCompactThreads * 16) {
        const int first = base + tx * 16;
        uint32_t mask = 0;   // bit i: row first + i is flagged
        if (first + 16 <= rows) {
            const uint4 word = *reinterpret_cast<const uint4*>(flags + first);
            const uint32_t parts[4] = {word.x, word.y, word.z, word.w};
#pragma unroll
            for (int i = 0; i < 16; ++i) mask |= ((parts[i >> 2] >> ((i & 3) * 8)) & 0xffu) != 0u ? 1u << i : 0u;
        } else {
            for (int i = 0; i < 16 && first + i < rows; ++i) mask |= flags[first + i] != 0 ? 1u << i : 0u;
        }
        const int mine = __popc(mask);
        if (__syncthreads_count(mask != 0u) == 0) continue;   // no flag in this step (the usual case)
        // inclusive scan of the per-thread counts over the CTA
        int scan = mine;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const int other = __shfl_up_sync(0xffffffffu, scan, offset);
            if (lane >= offset) scan += other;
        }
        if (lane == 31) warp_sums[tx >> 5] = scan;
        __syncthreads();
        int before = 0, step_total = 0;
#pragma unroll
        for (int w = 0; w < kCompactThreads / 32; ++w) {
            if (w < (tx >> 5)) before += warp_sums[w];
            step_total += warp_sums[w];
        }
        const int through = seen + before + scan;   // flagged rows up to and including this thread's 16
        if (slot >= through - mine && slot < through) {
            int skip = slot - (through - mine);
            uint32_t rest = mask;
            while (skip-- > 0) rest &= rest - 1u;
            found_row = first + __ffs(rest) - 1;
        }
        located = slot < seen + step_total;
        seen += step_total;
        __syncthreads();   // warp_sums may be rewritten by the next step
    }
    __syncthreads();
    const int row = found_row;
    if (row < 0) {
        if (tx == 0) {
            slot_rows[slot] = -1;
            k_start_out[slot] = 0;
            k_end_out[slot] = 0;
        }
        return;
    }
    constexpr int kRowVectors = kHeads * kHeadDim / 16;   // 512 x 16 B per query row
    for (int i = tx; i < kRowVectors; i += kCompactThreads)
        q_out[static_cast<long long>(slot) * kRowVectors + i] = q[static_cast<long long>(row) * kRowVectors + i];
    if (tx < kHeads) weights_out[slot * kHeads + tx] = weights[static_cast<long long>(row) * kHeads + tx];
    if (tx == 0) {
        slot_rows[slot] = row;
        k_start_out[slot] = k_start[row];
        k_end_out[slot] = k_end[row];
    }
}

// ------------------------------------------------------------------ is any row flagged?

// Sets the condition of a graph's IF node: 1 when any row is flagged, else 0.  One CTA.
__global__ void __launch_bounds__(256) itk_any_flag_kernel(cudaGraphConditionalHandle condition,
                                                            const uint8_t* __restrict__ flags, int rows) {
    int any = 0;
    for (int i = static_cast<int>(threadIdx.x); i < rows; i += static_cast<int>(blockDim.x)) any |= flags[i];
    any = __syncthreads_or(any);
    if (threadIdx.x == 0) cudaGraphSetConditional(condition, any != 0 ? 1u : 0u);
}

// ------------------------------------------------------------------ pair reducers

struct PairSource {
    const uint64_t* pairs;    // [rows, capacity]
    const int32_t* counts;    // [rows] live entries per row; null: a dense chunk, entry i belongs to key
                              // dense_lo + i, scanned over the row's key range only, 0 = empty
    int capacity;             // entries per row
};

struct PairTopKParams {
    PairSource sources[kMaxPairSources];
    int num_sources;
    int first_source;               // sources below this index are ignored (empty accumulator)
    int stage_capacity;             // pairs the launch's shared memory holds (<= kPairCapacity); a row whose
                                    // union is larger is an error (count mismatch), for a shard merge a failed row
    int rows;
    // Rows taken: all of them, or (owned_blocks > 0) the blocks of 4 rows block_begin + i * block_stride.
    int block_begin, block_stride, owned_blocks;
    const int32_t* out_rows;        // null, or the row of the outputs (ids, pairs, counts, flags) for source row r;
                                    // negative: the source row is an empty slot and is skipped
    const uint8_t* row_mask;        // null, or only rows with row_mask[row] != 0 are processed
    uint8_t* error_flags;           // null, or per-row error code; rows with a nonzero code are skipped
    int clear_errors;               // reset error_flags[row] of processed rows first
    // Dense sources: the chunk holds keys [dense_lo, dense_hi); the live-entry total must equal the number
    // of keys of the row's range [k_start, k_end) inside the chunk (expect_start / expect_end, when given,
    // hold that range rebased into the chunk instead).
    const int32_t* expect_start;
    const int32_t* expect_end;
    int dense_lo, dense_hi;
    int error_count_mismatch;       // code stored when that check fails
    int error_selection;            // code stored when the selection is inconsistent
    uint64_t* out_pairs;            // null or [rows, 2048]
    int32_t* out_ids;               // null or [rows, 2048]
    int32_t* mirror_ids;            // null, or a second copy of the ids ([rows, 2048], e.g. in mapped host memory)
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

__device__ __forceinline__ void write_shard_verdict(const PairTopKParams& p, int row, int out_row, int produced) {
    if (p.verdict_flags == nullptr) return;
    int failed = 0;
    for (int s = 0; s < p.num_sources; ++s) failed |= p.shard_flags[static_cast<long long>(s) * p.rows + row];
    const int wanted = min(max(min(p.k_end[row], p.key_hi) - max(p.k_start[row], p.key_lo), 0), kTopK);
    p.verdict_flags[out_row] = (failed != 0 || produced < wanted) ? 1 : 0;
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

// Exact Top-2048 of the union of up to sixteen pair lists per row.  One CTA per
// row (grid-strided); the union (at most kPairCapacity pairs) is staged in shared memory,
// the 2048-th largest score is found by four 8-bit radix rounds over the ordered
// score bits, then everything above it and the needed number of ties are
// written.  Rows with at most 2048 pairs are copied through.
__global__ void __launch_bounds__(kPairThreads, 3) itk_pair_topk_kernel(const PairTopKParams p) {
    extern __shared__ __align__(16) uint64_t staged[];
    __shared__ PairShared sh;
    const int tx = threadIdx.x;
    const int lane = tx & 31;
    const int items = p.owned_blocks > 0 ? p.owned_blocks * kBlockQ : p.rows;
    const auto row_of = [&](int item) {
        return p.owned_blocks > 0 ? (p.block_begin + (item >> 2) * p.block_stride) * kBlockQ + (item & 3) : item;
    };

    if (p.row_mask != nullptr) {
        // The usual case of the repair graph is that no row is flagged: look at all of this CTA's
        // rows at once instead of paying one dependent global load per row.
        int any = 0;
        for (int item = static_cast<int>(blockIdx.x) + tx * static_cast<int>(gridDim.x); item < items;
             item += kPairThreads * static_cast<int>(gridDim.x)) {
            const int row = row_of(item);
            if (row < p.rows) any |= p.row_mask[row];
        }
        if (__syncthreads_or(any) == 0) return;
    }

    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int row = row_of(item);
        if (row >= p.rows) continue;
        const int out_row = p.out_rows != nullptr ? p.out_rows[row] : row;
        if (out_row < 0) continue;
        __syncthreads();
        if (tx == 0) {
            int skip = 0;
            if (p.row_mask != nullptr && p.row_mask[row] == 0) skip = 1;
            if (!skip && p.error_flags != nullptr) {
                if (p.clear_errors) p.error_flags[row] = 0;
                else if (p.error_flags[row] != 0) skip = 1;
            }
            sh.skip = skip;
            sh.count = 0;
            sh.gcount = 0;
            sh.ecount = 0;
        }
        __syncthreads();
        if (sh.skip) continue;

        // stage the live pairs of every source
        int error = 0;
        for (int s = p.first_source; s < p.num_sources; ++s) {
            const int capacity = p.sources[s].capacity;
            const uint64_t* source = p.sources[s].pairs + static_cast<long long>(row) * capacity;
            const bool dense = p.sources[s].counts == nullptr;
            // a dense source is only defined inside the row's own range: entries outside it
            // were never written by the producer
            int first = 0;
            int live = dense ? capacity : min(p.sources[s].counts[row], capacity);
            if (dense) {
                if (p.expect_start != nullptr) {
                    first = max(p.expect_start[row], 0);
                    live = min(p.expect_end[row], capacity);
                } else {
                    const int width = min(capacity, p.dense_hi - p.dense_lo);
                    first = min(width, max(0, p.k_start[row] - p.dense_lo));
                    live = min(width, max(0, p.k_end[row] - p.dense_lo));
                }
                __syncthreads();
            }
            const int before = dense ? sh.count : 0;
            for (int base = first & ~31; base < live; base += kPairThreads) {
                const int i = base + tx;
                const bool inside = i >= first && i < live;
                const uint64_t pair = inside ? source[i] : 0ull;
                const bool keep = inside && (!dense || pair != 0ull);
                const int position = warp_reserve(&sh.count, keep, lane);
                if (keep && position < p.stage_capacity) staged[position] = pair;
            }
            if (dense) {
                __syncthreads();
                if (sh.count - before != max(live - first, 0)) error = p.error_count_mismatch;
            }
        }
        __syncthreads();
        const int count = sh.count;
        if (count > p.stage_capacity) error = p.error_count_mismatch != 0 ? p.error_count_mismatch : 1;
        if (error != 0) {
            if (tx == 0) {
                if (p.error_flags != nullptr) p.error_flags[row] = static_cast<uint8_t>(error);
                if (p.out_counts != nullptr) p.out_counts[out_row] = 0;
                write_shard_verdict(p, row, out_row, 0);
            }
            continue;
        }

        uint64_t* out_pairs = p.out_pairs != nullptr ? p.out_pairs + static_cast<long long>(out_row) * kTopK : nullptr;
        int32_t* out_ids = p.out_ids != nullptr ? p.out_ids + static_cast<long long>(out_row) * kTopK : nullptr;
        int32_t* mirror_ids = p.mirror_ids != nullptr ? p.mirror_ids + static_cast<long long>(out_row) * kTopK : nullptr;
        if (count <= kTopK) {
            for (int i = tx; i < kTopK; i += kPairThreads) {
                const uint64_t pair = i < count ? staged[i] : 0ull;
                const int32_t id = i < count ? static_cast<int32_t>(static_cast<uint32_t>(pair)) : -1;
                if (out_pairs != nullptr) out_pairs[i] = pair;
                if (out_ids != nullptr) out_ids[i] = id;
                if (mirror_ids != nullptr) mirror_ids[i] = id;
            }
            if (tx == 0) {
                if (p.out_counts != nullptr) p.out_counts[out_row] = count;
                if (p.clear_flags != nullptr && count == kTopK) p.clear_flags[out_row] = 0;
                write_shard_verdict(p, row, out_row, count);
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
                if (mirror_ids != nullptr) mirror_ids[position] = static_cast<int32_t>(static_cast<uint32_t>(pair));
            }
        }
        __syncthreads();
        if (tx == 0) {
            const bool consistent = equal_needed > 0 && sh.gcount == greater_total && sh.ecount >= equal_needed;
            if (!consistent) {
                if (p.error_flags != nullptr) p.error_flags[row] = static_cast<uint8_t>(p.error_selection);
                if (p.out_counts != nullptr) p.out_counts[out_row] = 0;
            } else {
                if (p.out_counts != nullptr) p.out_counts[out_row] = kTopK;
                if (p.clear_flags != nullptr) p.clear_flags[out_row] = 0;
            }
            write_shard_verdict(p, row, out_row, consistent ? kTopK : 0);
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
