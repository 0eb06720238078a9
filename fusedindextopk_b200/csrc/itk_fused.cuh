// The persistent fused score + exact Top-K kernel for sm_100a.
//
// One CTA per SM walks a static list of work units.  A unit is one block of
// kBlockQ = 4 consecutive query rows against one contiguous key range.  For
// every 128-key tile of the range the CTA computes
//
//     acc[key, (row, head)] = sum_d kv[key, d] * q[row, head, d]        (fp8 x fp8 -> fp32)
//
// as one 128 x 256 x 128 contraction on the tensor cores (four tcgen05.mma of
// K = 32 into a TMEM accumulator), then the epilogue warps read the accumulator
// back with tcgen05.ld (one warp per TMEM lane quarter and query row) and form
//
//     score[row, key] = (sum_h relu(acc) * w[row, h]) * kv_scale[key].
//
// The dense score matrix is never written.  What happens to a score depends on
// the kernel mode:
//   kModeTopK    keep (score, key) when the key is inside the row's range and
//                score >= threshold[row]; candidates go to per-row shared-memory
//                segments (overflow to a bounded global spill) and are counted in a
//                per-row histogram; when the unit's last tile is done the four
//                epilogue warps of a row select its exact Top-2048 in place;
//   kModeSample  the "keys" are S gathered sample keys; one warp per row picks the
//                rank-th largest valid sampled score = the row's threshold;
//   kModeRepair  for rows flagged as failed, write every (score, key) of one
//                16 K-key chunk to global memory for the exact repair reducers.
//
// Warp roles (640 threads): warp 0 TMA producer, warp 1 UMMA issuer and TMEM
// owner, warps 2-3 idle, warps 4-19 epilogue and selection.  All hand-offs are
// mbarriers with bounded waits; a wait that expires sets bit 0 of *status and
// the CTA drains.
//
// Counterparts in the reference (sm_90a, WGMMA): the persistent kernel
// kernel/csrc/include/fused_index_topk/long_fused_topk.cuh:64-672 and its
// consumer kernel/csrc/include/fused_index_topk/long_cta_topk.cuh:116-309; the
// masked chunk producer kernel/csrc/repair/include/fused_index_topk/repair_producer.cuh:48-430;
// the sampled threshold kernel/csrc/sampling_threshold.cu:99-178.
#pragma once

#include "itk_ptx.cuh"

// Build-time experiment switch for timing studies (0 in every shipped build):
//   1 = epilogue only drains TMEM and hands the buffer back, 2 = drain + head reduction, no filtering,
//   6 = everything but the per-row Top-K selection, 7 = additionally no filter / compaction.
#ifndef ITK_EXPERIMENT
#define ITK_EXPERIMENT 0
#endif

// Heartbeat builds (-DITK_HEARTBEAT, diagnostic kernels only): lane 0 of every warp records the last
// point it reached in trace[32 + warp], so that a host thread can read a stuck kernel's state from
// mapped host memory.
#ifdef ITK_HEARTBEAT
#define ITK_BEAT(code)                                                                                        \
    do {                                                                                                      \
        if (DIAG && p.trace != nullptr && lane == 0)                                                          \
            *reinterpret_cast<volatile long long*>(p.trace + static_cast<long long>(blockIdx.x) * kTraceFields + \
                                                   32 + warp) = (code);                                        \
    } while (0)
#else
#define ITK_BEAT(code) do { } while (0)
#endif

#include <type_traits>

namespace itk {

constexpr int kHeads = 64;
constexpr int kHeadDim = 128;
constexpr int kBlockQ = 4;                     // query rows per unit
constexpr int kTileKeys = 128;                 // keys per UMMA tile (= TMEM lanes)
constexpr int kUmmaN = kBlockQ * kHeads;       // 256 accumulator columns per tile
constexpr int kKvStages = 4;
constexpr int kAccBuffers = 2;
constexpr int kTmemColumns = kAccBuffers * kUmmaN;  // 512 = all of TMEM
constexpr int kTopK = 2048;

constexpr int kSegments = 4;                   // one per TMEM lane quarter: segment = (key >> 5) & 3
constexpr int kSegCap = 1280;                  // shared-memory candidates per (row, segment)
constexpr int kRowCap = kSegments * kSegCap;   // 5120
constexpr int kSpillSegCap = 1408;             // global spill entries per (row, segment)
constexpr int kSpillRow = kSegments * kSpillSegCap;  // 5632 u64 per row
constexpr int kRepairChunk = 16384;

// Warp 0: TMA producer; warp 1: UMMA issuer; warps 2-3: idle (they complete the first warpgroup);
// warps 4-19: epilogue and per-row selection.  65536 / 640 rounded down to the allocation unit of 8
// gives every thread 96 registers.
constexpr int kThreads = 640;
constexpr int kEpilogueWarp0 = 4;
constexpr int kEpilogueThreads = 512;
constexpr int kEpilogueWarps = kEpilogueThreads / 32;
constexpr int kScoreBins = 256;
constexpr int kBinListCap = 64;     // scores of the histogram bin that holds the cutoff; more: radix fallback
constexpr int kRankDirect = 48;    // lists up to this size are ranked without a second histogram level

constexpr uint32_t kQBytes = kUmmaN * kHeadDim;       // 32768
constexpr uint32_t kKvBytes = kTileKeys * kHeadDim;   // 16384

constexpr int kModeTopK = 0;
constexpr int kModeSample = 1;
constexpr int kModeRepair = 2;

constexpr int kStatusWaitExpired = 1;

// Per-CTA phase trace of diagnostic builds (clock64 cycles unless noted).
#ifdef ITK_HEARTBEAT
constexpr int kTraceFields = 64;
#else
constexpr int kTraceFields = 32;
#endif
constexpr int kTraceMmaTotal = 0, kTraceMmaWaitAcc = 1, kTraceMmaWaitKv = 2, kTraceMmaWaitQ = 3, kTraceMmaTiles = 4;
constexpr int kTraceTmaTotal = 8, kTraceTmaWaitKv = 9, kTraceTmaWaitQ = 10;
constexpr int kTraceEpiTotal = 12, kTraceEpiWaitAcc = 13, kTraceEpiSelect = 14, kTraceEpiWaitW = 15;  // +4 for query row 1
constexpr int kTraceSm = 24, kTraceNsBegin = 25, kTraceNsEnd = 26;

struct FusedParams {
    CUtensorMap map_q;    // [rows*64, 128] bytes, box 256 x 128, 128-byte swizzle
    CUtensorMap map_kv;   // [keys, 128] bytes (PAGED: the physical pool), box 128 x 128, 128-byte swizzle
    const float* kv_scales;     // [keys] (PAGED: [physical keys])
    const int32_t* tile_table;  // PAGED builds: physical 128-key tile of every logical tile, [ceil(keys/128)]
    const float* weights;       // [rows, 64]
    const int32_t* k_start;     // [rows]
    const int32_t* k_end;       // [rows]
    const float* thresholds;    // [shards, rows]      kModeTopK input
    float* thresholds_out;      // [rows]              kModeSample output
    const int32_t* sample_ids;  // [keys]              kModeSample: key position of each sample
    int32_t* out_ids;           // [rows, 2048]        kModeTopK output (may be null when out_pairs is set)
    uint64_t* out_pairs;        // [shards, rows, 2048] kModeTopK optional (ordered score << 32 | key)
    int32_t* out_counts;        // [shards, rows]      number of pairs written (with out_pairs)
    uint8_t* failure_flags;     // [shards, rows]      kModeTopK output / kModeRepair input
    uint64_t* spill;            // [shards, rows, 8, kSpillSegCap]
    uint64_t* repair_pairs;     // [shards*rows, 16384] kModeRepair output, dense by key - chunk_lo
    float* diag_logits;         // [rows, diag_stride] dense scores, diagnostic builds only
    long long diag_stride;
    long long* trace;           // [grid, kTraceFields] per-CTA cycle counters, diagnostic builds only
    int debug_skip;             // diagnostic builds only: 1 no selection, 2 no compaction, 4 no head reduction
    int* status;                // device status word, bits are or-ed in
    int rows;                   // Q
    int keys;                   // N (or S in kModeSample)
    int key_lo;                 // first key of shard 0 (multiple of 128)
    int key_hi;                 // end of the last shard
    int shard_keys;             // keys per shard (multiple of 128)
    int shards;
    int block_begin;            // first owned query block
    int block_stride;           // stride between owned query blocks
    int num_blocks;             // owned query blocks
    int sample_rank;            // kModeSample
    int target_candidates;      // kModeSample
    int top_k_min_valid;        // rows with at most this many valid keys need no selection (= 2048)
    int row_thresholds;         // 1: thresholds are per row (shared by the row's shards); a shard that finds
                                // fewer than 2048 candidates returns them all instead of failing
    int flags_per_row;          // kModeRepair with shards > 1: failure_flags has [rows] entries (one launch over
                                // all repair chunks of every flagged row), repair_pairs stays [shards*rows, 16384]
};

// Per-row scratch of the selection.
struct RowSelect {
    int hist[256];                      // second-level histogram / digit histogram of the radix fallback
    uint32_t bin_scores[kBinListCap];   // the scores of the histogram bin that holds the cutoff
    int position;     // next free output position of the row
    int bin_count;
    int tickets;
    int bin;          // radix fallback: digit of the round
    int above;
    uint32_t reference;
    uint32_t differing;
};

struct __align__(16) FusedShared {
    float weights[2][kBlockQ * kHeads];
    uint32_t cand_scores[kBlockQ][kRowCap];
    uint16_t cand_ids[kBlockQ][kRowCap];
    int counts[kBlockQ][kSegments];
    // Score histogram of every row's candidates, filled by the epilogue as it finds them:
    // kScoreBins bins of the distance to the row threshold, two 16-bit counters per word.
    uint32_t row_hist[kBlockQ][kScoreBins / 2];
    RowSelect select[kBlockQ];
    uint32_t tmem_base;
    int abort;
    uint64_t kv_full[kKvStages];
    uint64_t tile_done[kKvStages];   // one arrival per finished tile: frees the key stage and publishes the accumulator
    uint64_t q_full;
    uint64_t q_empty;
    uint64_t w_full[2];
    uint64_t w_empty[2];
    uint64_t acc_empty[kAccBuffers];
    uint64_t row_bar[kBlockQ];       // barrier of the four epilogue warps of a query row
};

constexpr size_t kSmemTileBytes = kQBytes + kKvStages * kKvBytes;
constexpr size_t kFusedSmemBytes = 1024 + kSmemTileBytes + sizeof(FusedShared);
static_assert(kFusedSmemBytes <= 232448, "fused kernel exceeds the 227 KB shared-memory limit");
static_assert(kSegCap % 32 == 0 && kSpillSegCap % 32 == 0, "segment capacities are warp multiples");

// mbar_wait that adds the cycles it took to `cycles` in diagnostic builds.
template <bool DIAG, uint32_t PARK_NS = kWaitParkNs>
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           long long& cycles) {
    if (DIAG) {
        const long long begin = clock64();
        const bool ok = mbar_wait<PARK_NS>(bar, parity, abort_flag);
        cycles += clock64() - begin;
        return ok;
    }
    return mbar_wait<PARK_NS>(bar, parity, abort_flag);
}

// ------------------------------------------------------------------ work units

struct Unit {
    int block;       // query block index
    int shard;
    int row0;
    int nrows;
    int key_lo;
    int key_hi;
    int tile_begin;  // global tile indices (key >> 7)
    int tile_end;    // tile_begin == tile_end: nothing to compute
};

// Unit `iter` of this CTA.  Units are ordered longest first (later query blocks
// see more keys) and dealt to the CTAs in a serpentine so that every CTA gets a
// similar amount of work.  Every role of the CTA derives the same list.
template <int MODE>
__device__ __forceinline__ bool load_unit(const FusedParams& p, int iter, Unit& u) {
    const int grid = static_cast<int>(gridDim.x);
    const int cta = (iter & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
    const long long index = static_cast<long long>(iter) * grid + cta;
    const long long total = static_cast<long long>(p.num_blocks) * p.shards;
    if (index >= total) return false;
    const int ordinal = static_cast<int>(index / p.shards);
    u.shard = static_cast<int>(index - static_cast<long long>(ordinal) * p.shards);
    u.block = p.block_begin + (p.num_blocks - 1 - ordinal) * p.block_stride;
    u.row0 = u.block * kBlockQ;
    u.nrows = min(kBlockQ, p.rows - u.row0);
    u.key_lo = p.key_lo + u.shard * p.shard_keys;
    u.key_hi = min(p.key_hi, u.key_lo + p.shard_keys);
    int lo = 0x7fffffff, hi = 0;
    for (int r = 0; r < u.nrows; ++r) {
        const int row = u.row0 + r;
        const int start = __ldg(p.k_start + row);
        const int end = __ldg(p.k_end + row);
        bool needed;
        int s, e;
        if (MODE == kModeSample) {
            needed = end - start > p.target_candidates;
            s = 0;
            e = p.keys;
        } else {
            s = max(start, u.key_lo);
            e = min(min(end, p.keys), u.key_hi);
            if (MODE == kModeTopK) {
                needed = e - s > (p.out_pairs != nullptr ? 0 : p.top_k_min_valid);
            } else {
                needed = e > s && p.failure_flags[(p.flags_per_row ? 0ll : static_cast<long long>(u.shard) * p.rows) + row] != 0;
            }
        }
        if (needed) {
            lo = min(lo, s);
            hi = max(hi, e);
        }
    }
    if (hi > lo) {
        u.tile_begin = lo >> 7;
        u.tile_end = (hi + kTileKeys - 1) >> 7;
    } else {
        u.tile_begin = 0;
        u.tile_end = 0;
    }
    return true;
}

// ------------------------------------------------------------------ selection helpers

// ------------------------------------------------------------------ per-row selection

// The four epilogue warps that score one query row (one per TMEM lane quarter) also select its
// Top-K when the unit's last tile is done: 128 threads per row, the four rows of a unit side by side.
constexpr int kRowThreads = 128;

// Barrier of the four warps of one query row: an mbarrier that the four warps arrive on and all
// 128 threads then poll, so that the wait is bounded like every other wait of the kernel (the waits
// are short: the four warps work in step, and nothing else wants the issue slots meanwhile).  When the limit
// expires (or another role already gave up) the abort flag is set and the call returns as if the
// barrier had completed: the results are garbage then, but every later wait sees the flag, the
// kernel ends and the host reads the failure from the status word.
struct RowBarrier {
    uint64_t* bar;
    uint32_t phase;
    volatile int* abort_flag;
    long long* lap;        // diagnostic builds: cycle counters of the selection steps (else null)
    long long lap_start;
};

// Adds the cycles since the previous lap to counter `index` (diagnostic builds only).
__device__ __forceinline__ void lap(RowBarrier& rb, int index) {
    if (rb.lap != nullptr) {
        const long long now = clock64();
        rb.lap[index] += now - rb.lap_start;
        rb.lap_start = now;
    }
}

__device__ __forceinline__ void row_sync(RowBarrier& rb) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) mbar_arrive(rb.bar);   // one arrival per warp
    if (!mbar_wait<kHotWait>(rb.bar, rb.phase & 1u, rb.abort_flag)) *rb.abort_flag = 1;
    ++rb.phase;
}

// The same barrier for warps that expect to wait long (one warp of the row works alone): a failed
// probe parks the warp instead of competing with the working warp for issue slots.
__device__ __forceinline__ void row_sync_parked(RowBarrier& rb) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) mbar_arrive(rb.bar);
    if (!mbar_wait<500>(rb.bar, rb.phase & 1u, rb.abort_flag)) *rb.abort_flag = 1;
    ++rb.phase;
}

__device__ __forceinline__ int decode_key(uint32_t packed, int segment) {
    return static_cast<int>(((packed >> 5) << 7) | (static_cast<uint32_t>(segment) << 5) | (packed & 31u));
}

__device__ __forceinline__ uint16_t encode_key(int key) {
    const uint32_t k = static_cast<uint32_t>(key);
    return static_cast<uint16_t>(((k >> 7) << 5) | (k & 31u));
}

// Warp-aggregated slot reservation: every lane calls, active lanes get distinct slots.
__device__ __forceinline__ int warp_reserve(int* counter, bool active, int lane) {
    const unsigned mask = __ballot_sync(0xffffffffu, active);
    if (mask == 0u) return -1;
    const int leader = __ffs(mask) - 1;
    int base = 0;
    if (lane == leader) base = atomicAdd(counter, __popc(mask));
    base = __shfl_sync(0xffffffffu, base, leader);
    return active ? base + __popc(mask & ((1u << lane) - 1u)) : -1;
}

// The view a warp has of the candidates it owns during the selection: the segment it filled itself
// (its TMEM lane quarter) and that segment's spill region in global memory.
struct RowView {
    const uint32_t* scores;        // [kSegCap] of the warp's segment
    const uint16_t* ids;           // [kSegCap]
    const uint64_t* spill;         // [kSpillSegCap] of the warp's segment
    int in_smem;                   // candidates of the segment in shared memory
    int in_spill;                  // ... and in the spill region
    int segment;
};

// Histogram bin of a candidate: the binary exponent of its distance to the row threshold (in value,
// not in bit patterns: scores may straddle zero).  One bin per octave covers every float, so the
// histogram needs no knowledge of the scale of the scores; the octave that holds the Top-K cutoff is
// resolved by a second histogram over the next eight bits of the distance.
__device__ __forceinline__ uint32_t distance_bits(uint32_t score_bits, float threshold) {
    return __float_as_uint(ordered_to_float(score_bits) - threshold);   // >= +0 for every candidate
}

// visit(score) for every candidate of the calling lane (candidate i of the segment belongs to lane
// i % 32).  The passes of a selection run once per unit, far apart in time, so their instructions
// come from a cold instruction cache: they are kept as short rolled loops over shared memory rather
// than unrolled passes over a register cache, which took several times longer.
// Four candidates are loaded before the first is visited: a visit may contain a shared-memory atomic,
// above which the compiler cannot move the next load, and a lone warp cannot hide a load per step.
// Missing candidates are passed as the score 0, which is below every real score (finite scores map
// to ordered bits above 0x00800000) and whose distance to a threshold is a NaN pattern that belongs
// to no bin, so a visit needs no liveness test.
template <typename Visit>
__device__ __forceinline__ void for_scores(const RowView& v, int lane, Visit&& visit) {
    const uint32_t* scores = v.scores;
    const int in_smem = v.in_smem;
#pragma unroll 1
    for (int i = lane; i < in_smem; i += 128) {
        const uint32_t s0 = scores[i];
        const uint32_t s1 = i + 32 < in_smem ? scores[i + 32] : 0u;
        const uint32_t s2 = i + 64 < in_smem ? scores[i + 64] : 0u;
        const uint32_t s3 = i + 96 < in_smem ? scores[i + 96] : 0u;
        visit(s0);
        visit(s1);
        visit(s2);
        visit(s3);
    }
#pragma unroll 1
    for (int e = lane; e < v.in_spill; e += 32) visit(static_cast<uint32_t>(v.spill[e] >> 32));
}

// Lane l owns entries 8l .. 8l+7 of a 256-entry histogram (counts[j] = entry 8l + j).  Finds the
// entry that holds the rank-th largest candidate, counting from the top: returns true in the lane
// that owns it, with its index, the number of candidates above it and its own count.
__device__ __forceinline__ bool find_rank(const int (&counts)[8], int lane, int rank, int& entry, int& above_out,
                                          int& inside) {
    int mine = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) mine += counts[j];
    int suffix = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const int other = __shfl_down_sync(0xffffffffu, suffix, offset);
        if (lane + offset < 32) suffix += other;
    }
    int above = suffix - mine;
    bool found = false;
#pragma unroll
    for (int j = 7; j >= 0; --j) {
        const int through = above + counts[j];
        if (above < rank && rank <= through) {
            found = true;
            entry = lane * 8 + j;
            above_out = above;
            inside = counts[j];
        }
        above = through;
    }
    return found;
}

// Warp-wide result of find_rank: every lane gets the values of the lane that found the entry.
__device__ __forceinline__ void share_rank(bool found, int& entry, int& above, int& inside) {
    const unsigned who = __ballot_sync(0xffffffffu, found);
    const int source = __ffs(who) - 1;
    entry = __shfl_sync(0xffffffffu, entry, source);
    above = __shfl_sync(0xffffffffu, above, source);
    inside = __shfl_sync(0xffffffffu, inside, source);
}

// Selection from the histogram that the epilogue filled while it found the candidates.  The octave
// (of the distance to the threshold) that holds the rank-th largest score is read off that histogram;
// the candidates of that octave are histogrammed again by the next eight bits of the distance; the
// handful of scores in the sub-bin that holds the cutoff are gathered and ranked against one another.
// The small steps (reading a histogram, ranking the list) are done by every warp redundantly, which
// costs a few dozen instructions and saves a barrier and a broadcast each.  Returns false (outputs
// untouched) when the last list holds more than kBinListCap scores (many equal or nearly equal
// scores); the caller then falls back to the radix selection.  Called by the 128 threads of a row
// after the barrier that publishes the row's counts; rs.hist and rs.bin_count are zero on entry;
// needs rank_in <= number of candidates.
__device__ __forceinline__ bool bin_select(RowSelect& rs, const RowView& v, const uint32_t* row_hist, float threshold,
                                           RowBarrier& rb, int tid, int rank_in, uint32_t& cutoff,
                                           int& equal_needed) {
    const int lane = tid & 31;
    int octave_entry, above, in_list;
    {
        int counts[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t word = row_hist[lane * 4 + j];
            counts[2 * j] = static_cast<int>(word & 0xffffu);
            counts[2 * j + 1] = static_cast<int>(word >> 16);
        }
        const bool found = find_rank(counts, lane, rank_in, octave_entry, above, in_list);
        share_rank(found, octave_entry, above, in_list);
    }
    lap(rb, 1);
    const uint32_t octave = static_cast<uint32_t>(octave_entry);
    int sub_bin = -1;            // -1: the whole octave is the list
    // octave 255 (infinite distances: the threshold is -inf) holds no usable order; the radix
    // selection sorts such rows out
    if (octave >= 255u) return false;
    if (in_list > kRankDirect) {
        // second level: the next eight bits of the distance inside the octave
        for_scores(v, lane, [&](uint32_t score) {
            const uint32_t d = distance_bits(score, threshold);
            if (d >> 23 == octave) atomicAdd(&rs.hist[(d >> 15) & 255u], 1);
        });
        lap(rb, 8);
        row_sync(rb);
        lap(rb, 9);
        int counts[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) counts[j] = rs.hist[lane * 8 + j];
        int above2 = 0;
        const bool found = find_rank(counts, lane, rank_in - above, sub_bin, above2, in_list);
        share_rank(found, sub_bin, above2, in_list);
        above += above2;
        lap(rb, 2);
    }
    if (in_list > kBinListCap) return false;
    const int need = rank_in - above;       // how many of the list's scores belong to the top rank_in
    // gather the list: the candidates whose distance starts with (octave) or (octave, sub-bin)
    const int list_shift = sub_bin < 0 ? 23 : 15;
    const uint32_t list_prefix = sub_bin < 0 ? octave : (octave << 8 | static_cast<uint32_t>(sub_bin));
    for_scores(v, lane, [&](uint32_t score) {
        if (distance_bits(score, threshold) >> list_shift == list_prefix) {
            const int at = atomicAdd(&rs.bin_count, 1);
            if (at < kBinListCap) rs.bin_scores[at] = score;
        }
    });
    lap(rb, 10);
    row_sync(rb);
    lap(rb, 3);
    // The need-th largest of the list: the score with fewer than `need` scores above it and at least
    // `need` scores above or equal to it.  Every warp ranks the whole list (two entries per lane).
    uint32_t found_cutoff = 0u;
    int found_equal = 0;
    bool found = false;
#pragma unroll 1
    for (int k = 0; k < kBinListCap / 32; ++k) {
        const int i = lane + 32 * k;
        const uint32_t mine = i < in_list ? rs.bin_scores[i] : 0u;
        int greater = 0, equal = 0;
#pragma unroll 4
        for (int j = 0; j < in_list; ++j) {
            const uint32_t other = rs.bin_scores[j];
            greater += other > mine ? 1 : 0;
            equal += other == mine ? 1 : 0;
        }
        if (i < in_list && greater < need && need <= greater + equal) {
            found = true;
            found_cutoff = mine;
            found_equal = need - greater;
        }
    }
    const unsigned who = __ballot_sync(0xffffffffu, found);
    const int source = __ffs(who) - 1;
    cutoff = __shfl_sync(0xffffffffu, found_cutoff, source);
    equal_needed = __shfl_sync(0xffffffffu, found_equal, source);
    lap(rb, 4);
    return true;
}

// Radix selection over the ordered score bits of one row, up to 8 bits per round: the fallback for
// rows whose cutoff bin is too full (many equal or nearly equal scores).  On return `cutoff` is the
// rank-th largest score and `equal_needed` the number of candidates equal to it that belong to the
// top `rank_in`.  The leading bits that all candidates share are found first and skipped.
__device__ __forceinline__ void radix_select(RowSelect& rs, const RowView& v, RowBarrier& rb, int tid, int rank_in,
                                             uint32_t& cutoff, int& equal_needed) {
    const int lane = tid & 31;
    if (tid == 0) rs.differing = 0u;
    if (lane == 0 && v.in_smem > 0) rs.reference = v.scores[0];   // any candidate of the row (the row has at least
    row_sync(rb);                                                  // rank_in >= 1 candidates, so some segment has one)
    const uint32_t reference = rs.reference;
    uint32_t differing = 0u;
    for_scores(v, lane, [&](uint32_t score) { differing |= score ^ reference; });
    differing = __reduce_or_sync(0xffffffffu, differing);
    if (lane == 0 && differing != 0u) atomicOr(&rs.differing, differing);
    row_sync(rb);
    differing = rs.differing;

    int bits = differing == 0u ? 0 : 32 - __clz(differing);   // low bits in which candidates may differ
    uint32_t mask = bits == 32 ? 0u : 0xffffffffu << bits;
    uint32_t prefix = reference & mask;
    int rank = rank_in;
#pragma unroll 1
    while (bits > 0) {
        const int width = min(8, bits);
        const int shift = bits - width;
        const uint32_t digit_mask = (1u << width) - 1u;
        for (int bin = tid; bin < 256; bin += kRowThreads) rs.hist[bin] = 0;
        row_sync(rb);
        for_scores(v, lane, [&](uint32_t score) {
            if ((score & mask) == prefix) atomicAdd(&rs.hist[(score >> shift) & digit_mask], 1);
        });
        row_sync(rb);
        if (tid < 32) {
            int bins[8];
            int mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bins[j] = rs.hist[lane * 8 + j];
                mine += bins[j];
            }
            int suffix = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const int other = __shfl_down_sync(0xffffffffu, suffix, offset);
                if (lane + offset < 32) suffix += other;
            }
            int above = suffix - mine;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                const int through = above + bins[j];
                if (above < rank && rank <= through) {
                    rs.bin = lane * 8 + j;
                    rs.above = above;
                }
                above = through;
            }
        }
        row_sync(rb);
        prefix |= static_cast<uint32_t>(rs.bin) << shift;
        rank -= rs.above;
        mask |= digit_mask << shift;
        bits = shift;
        row_sync(rb);   // everybody has read the round's result before the histogram is cleared again
    }
    cutoff = prefix;
    equal_needed = rank;
}

// Writes the selected candidates of one row: everything above `cutoff`, then `equal_needed` of the
// candidates equal to it (any of them); cutoff 0 takes every candidate.  Every warp counts its
// candidates above the cutoff, reserves that many output positions with one atomic add and fills
// them in ballot order, 32 candidates at a time, so that the stores of a warp instruction fall into
// a few sectors.  The few candidates equal to the cutoff draw tickets for the positions behind.
// rs.position and rs.tickets must be 0 on entry (a row barrier before the call publishes that).
__device__ __forceinline__ void emit_row(RowSelect& rs, const RowView& v, int lane, uint32_t cutoff, int equal_needed,
                                         int greater_total, int32_t* out_ids, uint64_t* out_pairs,
                                         RowBarrier* timer = nullptr) {
    int greater = 0;
    for_scores(v, lane, [&](uint32_t score) { greater += score > cutoff ? 1 : 0; });
    greater = __reduce_add_sync(0xffffffffu, greater);
    if (timer != nullptr) lap(*timer, 12);
    int position = 0;
    if (lane == 0 && greater > 0) position = atomicAdd(&rs.position, greater);
    position = __shfl_sync(0xffffffffu, position, 0);
    if (timer != nullptr) lap(*timer, 13);
    const unsigned below = (1u << lane) - 1u;
    const auto write = [&](int at, uint32_t score, int key) {
        if (at >= kTopK) return;
        if (out_ids != nullptr) out_ids[at] = key;
        if (out_pairs != nullptr) out_pairs[at] = (static_cast<uint64_t>(score) << 32) | static_cast<uint32_t>(key);
    };
    // One candidate per lane (score 0: none); `key()` is only evaluated for the candidates that are written.
    // No divergent branch on the common path: a lane that writes nothing aims past the end, and the
    // tie tickets (about one per row) sit behind a warp-uniform test.
    const auto place = [&](uint32_t score, auto&& key) {
        const bool is_greater = score > cutoff;
        const unsigned ballot = __ballot_sync(0xffffffffu, is_greater);
        const bool tie = score == cutoff && cutoff != 0u;
        int at = is_greater ? position + __popc(ballot & below) : kTopK;
        if (__any_sync(0xffffffffu, tie)) {
            if (tie) {
                const int ticket = atomicAdd(&rs.tickets, 1);
                if (ticket < equal_needed) at = greater_total + ticket;
            }
        }
        write(at, score, key());
        position += __popc(ballot);
    };
    {
        // four candidates (score and id) are loaded before the first is placed, see for_scores
        const uint32_t* scores = v.scores;
        const uint16_t* ids = v.ids;
        const int in_smem = v.in_smem, segment = v.segment;
#pragma unroll 1
        for (int base = 0; base < in_smem; base += 128) {
            uint32_t score[4];
            uint32_t id[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = base + 32 * k + lane;
                const bool live = i < in_smem;
                score[k] = live ? scores[i] : 0u;
                id[k] = live ? ids[i] : 0u;
            }
            // The four ballots first, then the positions, then the stores: the votes of one group do not
            // wait for each other's stores, and the tie test costs one vote per group (dead lanes carry
            // score 0, which is neither greater than nor tied with a cutoff).
            unsigned ballot[4];
            bool tie = false;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                ballot[k] = __ballot_sync(0xffffffffu, score[k] > cutoff);
                tie = tie || (score[k] == cutoff && cutoff != 0u);
            }
            int at[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                at[k] = score[k] > cutoff ? position + __popc(ballot[k] & below) : kTopK;
                position += __popc(ballot[k]);
            }
            if (__any_sync(0xffffffffu, tie)) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (score[k] == cutoff && cutoff != 0u) {
                        const int ticket = atomicAdd(&rs.tickets, 1);
                        if (ticket < equal_needed) at[k] = greater_total + ticket;
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) write(at[k], score[k], decode_key(id[k], segment));
        }
    }
#pragma unroll 1
    for (int base = 0; base < v.in_spill; base += 32) {
        const int e = base + lane;
        const uint64_t pair = e < v.in_spill ? v.spill[e] : 0ull;
        place(static_cast<uint32_t>(pair >> 32), [&]() { return static_cast<int>(static_cast<uint32_t>(pair)); });
    }
}

// Exact Top-2048 of one row from its candidates.  Called by the 128 threads of row r after the
// row's four segment counts are in shared memory and the row barrier has been passed; returns with
// the row barrier passed again (the candidate buffers and the histogram may be reused).
__device__ __forceinline__ void select_topk_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                bool has_tiles, RowBarrier& rb, int tid) {
    const int row = u.row0 + r;
    const long long row_slot = static_cast<long long>(u.shard) * p.rows + row;
    const int start = max(__ldg(p.k_start + row), u.key_lo);
    const int end = min(min(__ldg(p.k_end + row), p.keys), u.key_hi);
    const int valid = max(end - start, 0);
    int32_t* out_ids = p.out_ids != nullptr ? p.out_ids + static_cast<long long>(row) * kTopK : nullptr;
    uint64_t* out_pairs = p.out_pairs != nullptr ? p.out_pairs + row_slot * kTopK : nullptr;

    if (out_pairs == nullptr && valid <= p.top_k_min_valid) {
        // every valid key is selected; no scores are needed
        for (int i = tid; i < kTopK; i += kRowThreads) out_ids[i] = i < valid ? start + i : -1;
        if (tid == 0) p.failure_flags[row_slot] = 0;
        return;
    }
    const auto fill_empty = [&](int from) {
        for (int i = from + tid; i < kTopK; i += kRowThreads) {
            if (out_ids != nullptr) out_ids[i] = -1;
            if (out_pairs != nullptr) out_pairs[i] = 0ull;
        }
    };
    if (!has_tiles) {
        // pairs requested but the row has no key in this shard
        fill_empty(0);
        if (tid == 0) {
            p.failure_flags[row_slot] = 0;
            if (p.out_counts != nullptr) p.out_counts[row_slot] = 0;
        }
        return;
    }

    RowSelect& rs = sh.select[r];
    const int lane = tid & 31;
    const int segment = tid >> 5;
    int total = 0;
    bool overflow = false;
#pragma unroll
    for (int s = 0; s < kSegments; ++s) {
        total += sh.counts[r][s];
        overflow = overflow || sh.counts[r][s] > kSegCap + kSpillSegCap;
    }
    RowView view;
    view.segment = segment;
    view.scores = sh.cand_scores[r] + segment * kSegCap;
    view.ids = sh.cand_ids[r] + segment * kSegCap;
    view.spill = p.spill + row_slot * kSpillRow + segment * kSpillSegCap;
    view.in_smem = min(sh.counts[r][segment], kSegCap);
    view.in_spill = min(max(sh.counts[r][segment] - kSegCap, 0), kSpillSegCap);
    const int wanted = min(valid, kTopK);
    uint32_t* row_hist = sh.row_hist[r];
    if (overflow || (total < wanted && !p.row_thresholds)) {
        // too many candidates for the buffers or too few for a full answer: the repair pass redoes the row
        // (with per-row thresholds a shard may come up short: the merge of the shards checks the total)
        fill_empty(0);
        if (tid == 0) {
            p.failure_flags[row_slot] = 1;
            if (p.out_counts != nullptr) p.out_counts[row_slot] = 0;
        }
    } else {
        if (rb.lap != nullptr) rb.lap_start = clock64();
        if (total <= kTopK) {
            // only reachable when valid <= 2048 (threshold forced to -inf): take everything
            emit_row(rs, view, lane, 0u, 0, 0, out_ids, out_pairs);
            fill_empty(total);
        } else {
            uint32_t cutoff;
            int equal_needed;
            const float threshold =
                valid > kTopK ? __ldg(p.thresholds + (p.row_thresholds ? row : row_slot)) : __int_as_float(0xff800000);
            if (!bin_select(rs, view, row_hist, threshold, rb, tid, kTopK, cutoff, equal_needed))
                radix_select(rs, view, rb, tid, kTopK, cutoff, equal_needed);
            emit_row(rs, view, lane, cutoff, equal_needed, kTopK - equal_needed, out_ids, out_pairs, &rb);
            lap(rb, 11);
        }
        if (tid == 0) {
            p.failure_flags[row_slot] = 0;
            if (p.out_counts != nullptr) p.out_counts[row_slot] = min(total, kTopK);
        }
    }
    for (int i = tid; i < kScoreBins / 2; i += kRowThreads) row_hist[i] = 0u;   // for the next unit
    row_sync(rb);
    // the selection's scratch is clean again for the row's next selection, whose first barrier
    // (the one that publishes the counts) orders these stores before any use
    for (int i = tid; i < 256; i += kRowThreads) rs.hist[i] = 0;
    if (tid == 0) {
        rs.position = 0;
        rs.tickets = 0;
        rs.bin_count = 0;
    }
    if (!(overflow || total < wanted) && total > kTopK) lap(rb, 6);
}

// The rank-th largest (1-based) of at most 32 * SLOTS ordered score words spread over the four
// segments of a row, by ONE warp: every lane keeps SLOTS values in registers and the answer is
// fixed bit by bit from the top, counting the live values that have the bit set (one warp reduction per bit).
// No shared-memory histogram and no barrier between the row's warps.
template <int SLOTS>
__device__ __forceinline__ uint32_t ballot_rank_select(const uint32_t* row_scores, const int (&counts)[kSegments],
                                                       int total, int rank, int lane) {
    static_assert(kSegments == 4, "the segment lookup below is written for four segments");
    const int b1 = counts[0], b2 = b1 + counts[1], b3 = b2 + counts[2];
    // a value that can no longer be the answer is set to 0, which has no bit to count
    uint32_t value[SLOTS];
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int index = lane + 32 * i;
        const bool valid = index < total;
        const int segment = (index >= b1) + (index >= b2) + (index >= b3);
        const int base = segment == 0 ? 0 : segment == 1 ? b1 : segment == 2 ? b2 : b3;
        value[i] = valid ? row_scores[segment * kSegCap + (index - base)] : 0u;
    }
    // Bits above the highest one in which two values differ are common to all of them; below, every
    // bit about halves the live set, and once a single value is left it is the answer.
    uint32_t any_bits = 0, all_bits = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        any_bits |= value[i];
        all_bits &= lane + 32 * i < total ? value[i] : 0xffffffffu;
    }
    any_bits = __reduce_or_sync(0xffffffffu, any_bits);
    all_bits = __reduce_and_sync(0xffffffffu, all_bits);
    const uint32_t differing = any_bits ^ all_bits;
    if (differing == 0u) return all_bits;                      // all values are equal
    const int top = 31 - __clz(static_cast<int>(differing));
    uint32_t prefix = top == 31 ? 0u : all_bits & ~((2u << top) - 1u);
    int alive = total;
#pragma unroll 1
    for (int bit = top; bit >= 0 && alive > 1; --bit) {
        const uint32_t probe = 1u << bit;
        int mine = 0;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) mine += static_cast<int>((value[i] >> bit) & 1u);
        const int with_bit = __reduce_add_sync(0xffffffffu, mine);
        const bool take = rank <= with_bit;   // the answer has this bit set
        if (take) prefix |= probe;
        else rank -= with_bit;
        alive = take ? with_bit : alive - with_bit;
        // keep the values that agree with the answer on this bit (zeros stay zero either way)
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) value[i] = ((value[i] & probe) != 0) == take ? value[i] : 0u;
    }
    if (alive == 1) {
        // the one value left (everything else is zero by now)
        uint32_t last = 0;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) last = max(last, value[i]);
        return __reduce_max_sync(0xffffffffu, last);
    }
    return prefix;
}

// Threshold of one row = rank-th largest valid sampled score (kModeSample).  Up to 512 samples are
// selected by one warp from registers (ballot_rank_select; row r by its warp of lane quarter r, the
// other three warps park at the row barrier); more samples go through the radix rounds of the row's
// four warps.  Called by the 128 threads of the row after the barrier that publishes the counts;
// returns whether the one-warp path was taken.
__device__ __forceinline__ bool sample_threshold_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                     bool has_tiles, RowBarrier& rb, int tid) {
    const int row = u.row0 + r;
    const int start = __ldg(p.k_start + row);
    const int end = __ldg(p.k_end + row);
    float result = __int_as_float(0xff800000);
    bool solo = false;   // the row's first warp selected alone; the others only wait for it
    if (has_tiles && end - start > p.target_candidates) {
        const int segment = tid >> 5;
        int total = 0;
        bool overflow = false;
#pragma unroll
        for (int s = 0; s < kSegments; ++s) {
            total += sh.counts[r][s];
            overflow = overflow || sh.counts[r][s] > kSegCap;
        }
        if (!overflow && total >= p.sample_rank && total <= 512) {
            // row r is selected by its warp of lane quarter r: the four working warps of a unit then sit on
            // four different schedulers
            solo = true;
            if (segment == (r & 3)) {
                const int counts[kSegments] = {sh.counts[r][0], sh.counts[r][1], sh.counts[r][2], sh.counts[r][3]};
                const uint32_t cutoff = total <= 256
                    ? ballot_rank_select<8>(sh.cand_scores[r], counts, total, p.sample_rank, tid & 31)
                    : ballot_rank_select<16>(sh.cand_scores[r], counts, total, p.sample_rank, tid & 31);
                result = ordered_to_float(cutoff);
            }
        } else if (!overflow && total >= p.sample_rank) {   // the same decision in all 128 threads
            RowView view;
            view.segment = segment;
            view.scores = sh.cand_scores[r] + segment * kSegCap;
            view.ids = sh.cand_ids[r] + segment * kSegCap;
            view.spill = nullptr;
            view.in_smem = sh.counts[r][segment];
            view.in_spill = 0;
            uint32_t cutoff;
            int equal_needed;
            radix_select(sh.select[r], view, rb, tid, p.sample_rank, cutoff, equal_needed);
            result = ordered_to_float(cutoff);
        }
    }
    if (solo ? tid == (r & 3) * 32 : tid == 0) p.thresholds_out[row] = result;
    return solo;
}

// ------------------------------------------------------------------ the kernel

__device__ __forceinline__ uint64_t pack_pair(float lo, float hi) {
    uint64_t packed;
    asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(lo), "f"(hi));
    return packed;
}

__device__ __forceinline__ void unpack_pair(uint64_t packed, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(packed));
}

__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// ------------------------------------------------------------------ epilogue helpers

// What the epilogue needs to know about one query row of a unit.
struct RowState {
    int lo, hi;          // key range of the row inside the unit's key slice
    float threshold;
    bool on;             // the row takes part in this launch
    long long slot;      // row index in the per-shard arrays (thresholds, spill, repair pairs)
};

template <int MODE>
__device__ __forceinline__ RowState load_row_state(const FusedParams& p, int row0, int nrows, int shard,
                                                   int unit_key_lo, int unit_key_hi, int r) {
    RowState state{0, 0, __int_as_float(0xff800000), r < nrows, 0};
    if (state.on) {
        const int row = row0 + r;
        state.slot = static_cast<long long>(shard) * p.rows + row;
        const int start = __ldg(p.k_start + row);
        const int end = __ldg(p.k_end + row);
        if (MODE == kModeSample) {
            state.lo = start;
            state.hi = end;
            state.on = end - start > p.target_candidates;
        } else {
            state.lo = max(start, unit_key_lo);
            state.hi = min(min(end, p.keys), unit_key_hi);
            if (MODE == kModeTopK) {
                const int valid = state.hi - state.lo;
                if (valid > kTopK) state.threshold = __ldg(p.thresholds + (p.row_thresholds ? row : state.slot));
                state.on = valid > (p.out_pairs != nullptr ? 0 : p.top_k_min_valid);
            } else {
                state.on = p.failure_flags[p.flags_per_row ? row : state.slot] != 0;
            }
        }
    }
    return state;
}

// Lane 0 waits on the barrier, the warp then reconverges: one poller per warp.
template <bool DIAG, uint32_t PARK_NS = kWaitParkNs>
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane,
                                          long long& cycles) {
    int ok = 1;
    if (lane == 0) ok = timed_wait<DIAG, PARK_NS>(bar, parity, abort_flag, cycles) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

// Per-tile wait of an epilogue warp.  The whole warp probes the barrier (no lane-0 branch and
// broadcast).  A first probe that fails parks the warp in the hardware for a short time: with four
// epilogue warps per scheduler the issue slots are the scarce resource, so a waiting warp must not
// spin.  Lanes of one probe can disagree when the phase completes while the probe is in flight, so
// every decision is taken by a warp vote and the warp leaves only when all of its lanes have seen
// the phase.  Bounded like mbar_wait.
constexpr uint32_t kTileParkNs = 2000;
// The UMMA issuer usually waits for the epilogue (an accumulator buffer to come back).  It shares its
// scheduler with four epilogue warps, so it parks between probes instead of spinning; the park is short
// because the hand-off it waits for is one tile (a microsecond or so) away.
constexpr uint32_t kIssuerParkNs = 200;

template <bool DIAG>
__device__ __forceinline__ bool warp_tile_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               long long& cycles) {
    if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
    const long long begin = DIAG ? clock64() : 0;
    uint64_t deadline = 0;
    bool ok = true;
    for (uint32_t spin = 1;; ++spin) {
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity, kTileParkNs))) break;
        if ((spin & 63u) == 0u) {
            const uint64_t now = global_timer_ns();
            if (deadline == 0) deadline = now + kWaitLimitNs;
            if (__any_sync(0xffffffffu, *abort_flag != 0 || now > deadline)) {
                *abort_flag = 1;
                ok = false;
                break;
            }
        }
    }
    if (DIAG) cycles += clock64() - begin;
    return ok;
}

template <int MODE, bool DIAG, bool PAGED = false>
__global__ void __launch_bounds__(kThreads, 1) itk_fused_kernel(const __grid_constant__ FusedParams p) {
    extern __shared__ uint8_t smem_raw[];
    // Align by pointer arithmetic on the shared array (not through an integer cast) so that the
    // compiler keeps the shared address space: LDS/STS/ATOMS instead of generic accesses.
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_q = smem;
    uint8_t* smem_kv = smem + kQBytes;
    FusedShared& sh = *reinterpret_cast<FusedShared*>(smem + kSmemTileBytes);
    volatile int* abort_flag = &sh.abort;

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;

    if (MODE == kModeRepair) {
        // The usual case is that the fast path flagged no row: find that out with one parallel scan
        // of the flags before any barrier, TMEM or descriptor is set up.
        int any = 0;
        const int flags = (p.flags_per_row ? 1 : p.shards) * p.rows;
        for (int i = static_cast<int>(threadIdx.x); i < flags; i += kThreads) any |= p.failure_flags[i];
        if (__syncthreads_or(any) == 0) return;
    }

    for (int i = static_cast<int>(threadIdx.x); i < kBlockQ * kScoreBins / 2; i += kThreads)
        (&sh.row_hist[0][0])[i] = 0u;
    for (int i = static_cast<int>(threadIdx.x); i < kBlockQ * 256; i += kThreads) sh.select[i >> 8].hist[i & 255] = 0;
    if (threadIdx.x < kBlockQ) {
        sh.select[threadIdx.x].position = 0;
        sh.select[threadIdx.x].tickets = 0;
        sh.select[threadIdx.x].bin_count = 0;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kKvStages; ++i) {
            mbar_init(&sh.kv_full[i], 1);
            mbar_init(&sh.tile_done[i], 1);
        }
        mbar_init(&sh.q_full, 1);
        mbar_init(&sh.q_empty, 1);
        for (int i = 0; i < kBlockQ; ++i) mbar_init(&sh.row_bar[i], kRowThreads / 32);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.w_full[i], 1);
            mbar_init(&sh.w_empty[i], kEpilogueWarps);
            mbar_init(&sh.acc_empty[i], kEpilogueWarps);
        }
        sh.abort = 0;
        fence_mbar_init();
        prefetch_tensormap(&p.map_q);
        prefetch_tensormap(&p.map_kv);
    }
    if (warp == 1) {
        tmem_alloc(&sh.tmem_base, kTmemColumns);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = sh.tmem_base;
    ITK_BEAT(2);

    const bool is_epilogue = warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + kEpilogueWarps;
    if (!is_epilogue) {
    if (warp == 0) {
        // ============================================================ TMA producer
        if (lane == 0) {
            int kv_iter = 0, q_iter = 0;
            bool ok = true;
            long long wait_kv = 0, wait_q = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                if (u.tile_end == u.tile_begin) continue;
                ok = timed_wait<DIAG>(&sh.q_empty, (q_iter & 1) ^ 1, abort_flag, wait_q);
                if (!ok) break;
                mbar_arrive_expect_tx(&sh.q_full, kQBytes);
                tma_load_2d(smem_q, &p.map_q, &sh.q_full, 0, u.block * kUmmaN);
                ITK_BEAT(10);
                const int ws = q_iter & 1;
                ok = timed_wait<DIAG>(&sh.w_empty[ws], ((q_iter >> 1) & 1) ^ 1, abort_flag, wait_q);
                if (!ok) break;
                const uint32_t w_bytes = static_cast<uint32_t>(u.nrows) * kHeads * sizeof(float);
                mbar_arrive_expect_tx(&sh.w_full[ws], w_bytes);
                bulk_load(sh.weights[ws], p.weights + static_cast<long long>(u.row0) * kHeads, w_bytes,
                          &sh.w_full[ws]);
                for (int t = u.tile_begin; t < u.tile_end; ++t, ++kv_iter) {
                    const int stage = kv_iter % kKvStages;
                    ok = timed_wait<DIAG>(&sh.tile_done[stage], ((kv_iter / kKvStages) & 1) ^ 1, abort_flag, wait_kv);
                    if (!ok) break;
#if ITK_EXPERIMENT == 4
                    mbar_arrive(&sh.kv_full[stage]);
#else
                    mbar_arrive_expect_tx(&sh.kv_full[stage], kKvBytes);
                    tma_load_2d(smem_kv + stage * kKvBytes, &p.map_kv, &sh.kv_full[stage], 0,
                                (PAGED ? __ldg(p.tile_table + t) : t) * kTileKeys);
#endif
                    ITK_BEAT(100 + kv_iter);
                }
                ++q_iter;
            }
            if (DIAG && p.trace != nullptr) {
                long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields;
                trace[kTraceTmaTotal] = clock64() - role_begin;
                trace[kTraceTmaWaitKv] = wait_kv;
                trace[kTraceTmaWaitQ] = wait_q;
            }
            if (!ok) {
                atomicOr(p.status, kStatusWaitExpired);
                // give loads already in flight a bounded chance to land before the CTA exits
                const uint64_t until = global_timer_ns() + 2000000ull;
                while (global_timer_ns() < until) {
                }
            }
        }
    } else if (warp == 1) {
        // ============================================================ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_e4m3_f32(kTileKeys, kUmmaN);
            const uint64_t desc_q = umma_desc_sw128_kmajor(smem_u32(smem_q));
            int kv_iter = 0, q_iter = 0;
            bool ok = true;
            long long wait_acc = 0, wait_kv = 0, wait_q = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                if (u.tile_end == u.tile_begin) continue;
                ok = timed_wait<DIAG>(&sh.q_full, q_iter & 1, abort_flag, wait_q);
                if (!ok) break;
                ITK_BEAT(10);
                // The tensor pipe accepts only a couple of UMMAs ahead of the one it executes, so
                // every cycle this thread spends between two batches of issues is a bubble.  The
                // barriers of tile t+1 are therefore probed while the UMMAs of tile t execute
                // (a probe takes less time than one UMMA); the blocking waits at the top are
                // normally satisfied already.
                bool acc_ready = false, kv_ready = false;
                for (int t = u.tile_begin; t < u.tile_end; ++t, ++kv_iter) {
                    const int buffer = kv_iter & 1;
                    const int stage = kv_iter % kKvStages;
                    ITK_BEAT(1000 + kv_iter * 10 + 1);
                    if (!acc_ready) {
                        ok = timed_wait<DIAG, kIssuerParkNs>(&sh.acc_empty[buffer], ((kv_iter >> 1) & 1) ^ 1, abort_flag, wait_acc);
                        if (!ok) break;
                    }
                    if (!kv_ready) {
                        ok = timed_wait<DIAG, kHotWait>(&sh.kv_full[stage], (kv_iter / kKvStages) & 1, abort_flag, wait_kv);
                        if (!ok) break;
                    }
                    tcgen05_fence_after_sync();
                    const uint64_t desc_kv = umma_desc_sw128_kmajor(smem_u32(smem_kv + stage * kKvBytes));
                    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buffer * kUmmaN);
                    const int next = kv_iter + 1;
                    const bool more = t + 1 < u.tile_end;
                    // advance both operands by 32 bytes (= 2 descriptor address units) per K step
                    umma_f8(tmem_d, desc_kv, desc_q, idesc, 0u);
                    acc_ready = more && mbar_test_wait(&sh.acc_empty[next & 1], ((next >> 1) & 1) ^ 1);
                    umma_f8(tmem_d, desc_kv + 2, desc_q + 2, idesc, 1u);
                    kv_ready = more && mbar_test_wait(&sh.kv_full[next % kKvStages], (next / kKvStages) & 1);
                    umma_f8(tmem_d, desc_kv + 4, desc_q + 4, idesc, 1u);
                    if (more && !acc_ready) acc_ready = mbar_test_wait(&sh.acc_empty[next & 1], ((next >> 1) & 1) ^ 1);
                    umma_f8(tmem_d, desc_kv + 6, desc_q + 6, idesc, 1u);
                    // a single commit per tile frees the key stage and publishes the accumulator
                    umma_commit(&sh.tile_done[stage]);
                    ITK_BEAT(1000 + kv_iter * 10 + 2);
                }
                if (!ok) break;
                umma_commit(&sh.q_empty);
                ++q_iter;
            }
            if (DIAG && p.trace != nullptr) {
                long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields;
                trace[kTraceMmaTotal] = clock64() - role_begin;
                trace[kTraceMmaWaitAcc] = wait_acc;
                trace[kTraceMmaWaitKv] = wait_kv;
                trace[kTraceMmaWaitQ] = wait_q;
                trace[kTraceMmaTiles] = kv_iter;
                unsigned sm;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
                trace[kTraceSm] = sm;
            }
            if (!ok) atomicOr(p.status, kStatusWaitExpired);
        }
    }
    } else {
        // ============================================================ epilogue
        // Sixteen warps share every tile: warp (quarter, row) reads the 32 TMEM lanes (= keys) of
        // its lane quarter, which is also its candidate segment, and the 64 accumulator columns
        // (= heads) of one query row.  Accumulators come out of TMEM in the 16x256b fragment
        // layout, 32 columns at a time: thread t of a warp holds, for lanes l = t/4 and l+8 of a
        // 16-lane half, the column pairs 8n + 2(t%4) + {0,1}, n = 0..3.  So a thread needs only 16
        // of the row's 64 head weights, kept in registers for the whole unit: no shared-memory
        // traffic in the hot loop.  The four threads of a quad combine their partial head sums
        // with two shuffles, after which every thread owns the score of exactly one key of the
        // tile.  Four warps per scheduler hide one another's TMEM and arithmetic latencies.
        const int ew = warp - kEpilogueWarp0;
        const int quarter = ew & 3;             // = warp % 4, the TMEM lane quarter this warp may read
        const int own_r = ew >> 2;              // query row of the unit this warp finishes
        const int quad = lane & 3;              // column-pair selector inside the fragment
        int own_lane = (lane >> 2) + 8 * quad;   // key (TMEM lane) of the quarter this thread finishes
        uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(own_r * kHeads);
        keep_in_register(own_lane);
        keep_in_register(tmem_lane);
        int unit_iter = 0;  // units with tiles
        int acc_iter = 0;   // tiles
        bool ok = true;
        long long wait_acc = 0, wait_w = 0, select_cycles = 0;
        const long long role_begin = DIAG ? clock64() : 0;
        if (DIAG && p.trace != nullptr && ew == 0 && lane == 0)
            p.trace[static_cast<long long>(blockIdx.x) * kTraceFields + kTraceNsBegin] = global_timer_ns();
        // What the row's four warps do when the unit's candidates are complete (or the unit has no tile
        // at all): exact Top-K of the row, or its sampled threshold.  All four warps of a row call it.
        long long laps[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
        RowBarrier rb{&sh.row_bar[own_r], 0u, abort_flag, DIAG ? laps : nullptr, 0};
        const auto finish_row = [&](const Unit& u, bool has_tiles) {
            const long long begin = DIAG ? clock64() : 0;
            bool solo = false;
            if (own_r < u.nrows) {
                if (MODE == kModeTopK) {
#if ITK_EXPERIMENT < 6
                    if (!(DIAG && (p.debug_skip & 1))) select_topk_row(sh, p, u, own_r, has_tiles, rb, quarter * 32 + lane);
#endif
                } else if (MODE == kModeSample) {
                    solo = sample_threshold_row(sh, p, u, own_r, has_tiles, rb, quarter * 32 + lane);
                }
            }
            if (MODE == kModeSample) {   // the row's buffers may be written again
                if (solo && quarter != (own_r & 3)) row_sync_parked(rb);
                else row_sync(rb);
            }
            if (DIAG) select_cycles += clock64() - begin;
        };
        for (int iter = 0; ok; ++iter) {
            Unit u;
            if (!load_unit<MODE>(p, iter, u)) break;
            if (u.tile_end == u.tile_begin) {
                finish_row(u, false);
                continue;
            }
            const int slot = unit_iter & 1;   // weight buffer of the unit
            const uint32_t use_parity = (unit_iter >> 1) & 1;
            ok = warp_wait<DIAG>(&sh.w_full[slot], use_parity, abort_flag, lane, wait_w);
            if (!ok) break;
            ITK_BEAT(11 + 100000 * unit_iter);

            // candidate segment of (row, quarter) and the number of candidates in it (warp-uniform)
            uint32_t score_slots = smem_u32(&sh.cand_scores[own_r][quarter * kSegCap]);
            uint32_t id_slots = smem_u32(&sh.cand_ids[own_r][quarter * kSegCap]);
            keep_in_register(score_slots);
            keep_in_register(id_slots);
            const uint32_t hist_slots = smem_u32(&sh.row_hist[own_r][0]);
            int count = 0;
            // Filter state of the row, arranged so that the tile loop needs no branch: a key passes when
            // it lies in [row_lo, row_lo + row_span) and its score reaches the threshold (-inf for rows
            // that keep every key); a row that is switched off has an empty range.
            const RowState row = load_row_state<MODE>(p, u.row0, u.nrows, u.shard, u.key_lo, u.key_hi, own_r);
            int row_lo = row.lo;
            unsigned row_span = row.on && row.hi > row.lo ? static_cast<unsigned>(row.hi - row.lo) : 0u;
            float threshold = row.threshold;
            // the compiler would otherwise re-derive these per tile from thread and unit indices
            keep_in_register(row_lo);
            keep_in_register(row_span);
            keep_in_register(threshold);

            // head weights of this thread's column pairs
            uint64_t w[8];
#pragma unroll
            for (int n = 0; n < 8; ++n)
                w[n] = *reinterpret_cast<const uint64_t*>(&sh.weights[slot][own_r * kHeads + 8 * n + 2 * quad]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.w_empty[slot]);   // weights are in registers now
            ITK_BEAT(12 + 100000 * unit_iter);

            // scale and range key of the key this thread finishes in tile t
            const auto per_key = [&](int t, float& scale, int& range_key) {
                const int key = t * kTileKeys + quarter * 32 + own_lane;
                const bool key_ok = key < p.keys;
                // a paged key keeps its logical position (ids, ranges); only its storage moves
                const int stored = PAGED ? __ldg(p.tile_table + t) * kTileKeys + quarter * 32 + own_lane : key;
                scale = key_ok ? __ldg(p.kv_scales + stored) : 0.0f;
                if (MODE == kModeSample) range_key = key_ok ? __ldg(p.sample_ids + key) : 0x7fffffff;
            };
            // ReLU is applied in place on the fragment registers, which are consecutive pairs
            // already, so the packed multiply-add can read them without any move.
            const auto relu_fma = [](uint32_t& x0, uint32_t& x1, uint64_t wpair, uint64_t& acc) {
                asm("{\n\t"
                    ".reg .b64 t;\n\t"
                    "max.f32 %0, %0, 0f00000000;\n\t"
                    "max.f32 %1, %1, 0f00000000;\n\t"
                    "mov.b64 t, {%0, %1};\n\t"
                    "fma.rn.f32x2 %2, t, %3, %2;\n\t"
                    "}"
                    : "+f"(*reinterpret_cast<float*>(&x0)), "+f"(*reinterpret_cast<float*>(&x1)), "+l"(acc)
                    : "l"(wpair));
            };
            // one fragment (32 columns, lanes l and l+8) into the packed accumulators of the two lanes
            const auto partial = [&](uint32_t (&r)[16], int w0, uint64_t (&acc_a)[2], uint64_t (&acc_b)[2]) {
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    relu_fma(r[4 * n + 0], r[4 * n + 1], w[w0 + n], acc_a[n & 1]);
                    relu_fma(r[4 * n + 2], r[4 * n + 3], w[w0 + n], acc_b[n & 1]);
                }
            };
            const auto head_sum = [](const uint64_t (&acc)[2]) -> float {
                float x0, x1, x2, x3;
                unpack_pair(acc[0], x0, x1);
                unpack_pair(acc[1], x2, x3);
                return (x0 + x1) + (x2 + x3);
            };
            // Quad reduce-scatter of the four partial sums (lanes l, l+8, l+16, l+24 of the quarter):
            // thread `quad` ends up with the complete head sum number `quad`.
            const auto quad_reduce = [&](float v0, float v1, float v2, float v3) -> float {
                const bool odd = (quad & 1) != 0;
                const float send_a = odd ? v0 : v1;
                const float send_b = odd ? v2 : v3;
                const float keep_a = (odd ? v1 : v0) + __shfl_xor_sync(0xffffffffu, send_a, 1);
                const float keep_b = (odd ? v3 : v2) + __shfl_xor_sync(0xffffffffu, send_b, 1);
                const bool upper = (quad & 2) != 0;
                return (upper ? keep_b : keep_a) + __shfl_xor_sync(0xffffffffu, upper ? keep_a : keep_b, 2);
            };
            // threshold filter and warp-level compaction of the 32 scores of this warp in one tile
            // Filter and warp-level compaction of the 32 scores of this warp in one tile.
            const auto finish = [&](int t, float sum, float scale, int sample_key) {
                const float score = sum * scale;
                const int key = t * kTileKeys + quarter * 32 + own_lane;
                const int range_key = MODE == kModeSample ? sample_key : key;   // the sampled key's position in the context
                const bool in_range = static_cast<unsigned>(range_key - row_lo) < row_span;
                if (DIAG) {
                    const bool key_ok = key < p.keys;
                    if (own_r < u.nrows && key_ok && p.diag_logits != nullptr) {
                        const bool shown = MODE == kModeSample ? true : (range_key >= row.lo && range_key < row.hi);
                        p.diag_logits[static_cast<long long>(u.row0 + own_r) * p.diag_stride + key] =
                            shown ? score : __int_as_float(0xff800000);
                    }
                }
                if (MODE == kModeRepair) {
                    if (row.on && key < p.keys && key >= u.key_lo && key < u.key_hi) {
                        p.repair_pairs[row.slot * kRepairChunk + (key - u.key_lo)] =
                            (range_key >= row.lo && range_key < row.hi) ? pack_score_id(score, static_cast<uint32_t>(key))
                                                                        : 0ull;
                    }
                    return;
                }
                bool active = in_range;
                if (DIAG && (p.debug_skip & 2)) active = false;
                if (MODE == kModeTopK) active = active && score >= threshold;
                else active = active && (fabsf(score) <= 3.4028234663852886e38f);  // finite
                const unsigned ballot = __ballot_sync(0xffffffffu, active);
                const int position = count + __popc(ballot & ((1u << lane) - 1u));
                count += __popc(ballot);
                const uint32_t score_bits = ordered_bits(score);
                if (MODE == kModeTopK && active) {
                    // one more candidate in its bin of the row's score histogram (16-bit counters)
                    const uint32_t bin = __float_as_uint(ordered_to_float(score_bits) - threshold) >> 23;
                    red_shared_add_u32(hist_slots + 4u * (bin >> 1), 1u << ((bin & 1u) * 16u));
                }
                if (active && position < kSegCap) {
                    st_shared_u32(score_slots + 4u * static_cast<uint32_t>(position), score_bits);
                    // id = (tile << 5) | (key & 31); the segment number carries the lane quarter
                    st_shared_u16(id_slots + 2u * static_cast<uint32_t>(position), static_cast<uint32_t>(t * 32 + own_lane));
                }
                if (MODE == kModeTopK && count > kSegCap) {
                    // warp-uniform and rare: the segment is full, later candidates go to the global spill
                    if (active && position >= kSegCap && position < kSegCap + kSpillSegCap) {
                        const long long row_slot = static_cast<long long>(u.shard) * p.rows + u.row0 + own_r;
                        p.spill[row_slot * kSpillRow + quarter * kSpillSegCap + (position - kSegCap)] =
                            pack_score_id(score, static_cast<uint32_t>(key));
                    }
                }
            };

            // Four fragment loads per tile, (half 0, heads 0-31), (half 0, heads 32-63), (half 1, heads
            // 0-31), (half 1, heads 32-63), through one 16-register buffer: the register budget has no
            // room for a second one, and the other three epilogue warps of the scheduler cover the TMEM
            // latency.  The accumulator buffer goes back to the UMMA issuer as soon as the fourth
            // fragment has landed; the first fragment of the next tile is requested before the filter step.
            uint32_t fa[16];
            float scale, next_scale = 0.0f;
            int range_key = 0, next_range_key = 0;   // sample mode only
            per_key(u.tile_begin, scale, range_key);
            ok = warp_tile_wait<DIAG>(&sh.tile_done[acc_iter % kKvStages], (acc_iter / kKvStages) & 1, abort_flag, wait_acc);
            if (!ok) break;
            tcgen05_fence_after_sync();
            tmem_load_frag16(tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN), fa);
            for (int t = u.tile_begin; t < u.tile_end; ++t, ++acc_iter) {
                ITK_BEAT(100 * acc_iter + 20);
                const uint32_t taddr = tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN);
                const uint32_t upper_half = 16u << 16;
                const bool more = t + 1 < u.tile_end;
                if (more) per_key(t + 1, next_scale, next_range_key);
                uint64_t acc_a[2] = {0, 0}, acc_b[2] = {0, 0};

                tmem_load_wait16(fa);                                 // (half 0, heads 0-31)
                ITK_BEAT(100 * acc_iter + 21);
#if ITK_EXPERIMENT != 1
                partial(fa, 0, acc_a, acc_b);
#else
                if (fa[3] == 0x7fc12345u) count += 1;
#endif
                tmem_load_frag16(taddr + 32, fa);
                tmem_load_wait16(fa);                                 // (half 0, heads 32-63)
                ITK_BEAT(100 * acc_iter + 22);
#if ITK_EXPERIMENT != 1
                partial(fa, 4, acc_a, acc_b);
#else
                if (fa[3] == 0x7fc12345u) count += 1;
#endif
                tmem_load_frag16(taddr + upper_half, fa);
                const float sum0 = head_sum(acc_a), sum1 = head_sum(acc_b);   // lanes l and l+8 of the quarter
                acc_a[0] = acc_a[1] = acc_b[0] = acc_b[1] = 0;
                tmem_load_wait16(fa);                                 // (half 1, heads 0-31)
                ITK_BEAT(100 * acc_iter + 23);
#if ITK_EXPERIMENT != 1
                partial(fa, 0, acc_a, acc_b);
#else
                if (fa[3] == 0x7fc12345u) count += 1;
#endif
                tmem_load_frag16(taddr + upper_half + 32, fa);
                tmem_load_wait16(fa);                                 // (half 1, heads 32-63): buffer fully read
                ITK_BEAT(100 * acc_iter + 24);
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.acc_empty[acc_iter & 1]);
                ITK_BEAT(100 * acc_iter + 25);
#if ITK_EXPERIMENT != 1
                partial(fa, 4, acc_a, acc_b);
#else
                if (fa[3] == 0x7fc12345u) count += 1;
#endif
                if (more) {
                    const int next = acc_iter + 1;
                    ok = warp_tile_wait<DIAG>(&sh.tile_done[next % kKvStages], (next / kKvStages) & 1, abort_flag, wait_acc);
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                    tmem_load_frag16(tmem_lane + static_cast<uint32_t>((next & 1) * kUmmaN), fa);
                }
                ITK_BEAT(100 * acc_iter + 26);
#if ITK_EXPERIMENT == 0 || ITK_EXPERIMENT == 6
                finish(t, quad_reduce(sum0, sum1, head_sum(acc_a), head_sum(acc_b)), scale, range_key);
#elif ITK_EXPERIMENT == 7   // no filter / compaction
                if (quad_reduce(sum0, sum1, head_sum(acc_a), head_sum(acc_b)) * scale >= threshold) count += 1;
#elif ITK_EXPERIMENT == 2
                if (sum0 + sum1 + head_sum(acc_a) + head_sum(acc_b) == 1.2345e38f) count += 1;
#endif
                scale = next_scale;
                range_key = next_range_key;
                ITK_BEAT(100 * acc_iter + 27);
            }
            if (!ok) break;
            if (MODE != kModeRepair) {
                if (lane == 0) sh.counts[own_r][quarter] = count;
                row_sync(rb);   // the four segments of the row are complete and counted
            }
            finish_row(u, true);
            ++unit_iter;
        }
        if (DIAG && p.trace != nullptr && quarter == 0 && own_r < 2 && lane == 0) {
            long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields + 4 * own_r;
            trace[kTraceEpiTotal] = clock64() - role_begin;
            trace[kTraceEpiWaitAcc] = wait_acc;
            trace[kTraceEpiSelect] = select_cycles;
            trace[kTraceEpiWaitW] = wait_w;
            if (own_r == 0) {
                long long* cta_trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields;
                cta_trace[27] = laps[0];   // candidate caching
                cta_trace[28] = laps[1];   // octave from the histogram
                cta_trace[29] = laps[2];   // second-level histogram
                cta_trace[30] = laps[3];   // list gathering
                cta_trace[31] = laps[4];   // list ranking
                cta_trace[20] = laps[11];  // emission: placing
                cta_trace[22] = laps[12];  // emission: counting
                cta_trace[23] = laps[13];  // emission: position reservation
                cta_trace[21] = laps[6];   // clean-up and last barrier
                cta_trace[5] = laps[8];    // second level: histogram pass
                cta_trace[6] = laps[9];    // second level: barrier
                cta_trace[7] = laps[10];   // gathering pass
                cta_trace[kTraceNsEnd] = global_timer_ns();
            }
        }
        if (!ok && lane == 0) atomicOr(p.status, kStatusWaitExpired);
    }

    // ---------------------------------------------------------------- teardown
    ITK_BEAT(900000);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

}  // namespace itk
