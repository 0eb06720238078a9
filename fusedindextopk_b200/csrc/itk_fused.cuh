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
//                score >= threshold[row]; every epilogue thread appends to its own
//                candidate list in shared memory (overflow to a bounded global
//                spill); when the unit's last tile is done the four epilogue warps
//                of a row select its exact Top-2048 in place.  With sample_tiles > 0
//                the unit first scores the gathered sample keys and takes its rows'
//                thresholds from them; the blocks of the last wave may be cut into
//                key shards whose lists a merge kernel combines;
//   kModeSample  the "keys" are S gathered sample keys; one warp per row picks the
//                rank-th largest valid sampled score = the row's threshold;
//   kModeRepair  for rows flagged as failed, write every (score, key) of one
//                16 K-key chunk to global memory for the exact repair reducers.
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 UMMA issuer and TMEM
// owner, warps 2-17 epilogue and selection.  All hand-offs are mbarriers with
// bounded waits; a wait that expires sets bit 0 of *status and the CTA drains.
//
// Counterparts in the reference (sm_90a, WGMMA): the persistent kernel
// kernel/csrc/include/fused_index_topk/long_fused_topk.cuh:64-672 and its
// consumer kernel/csrc/include/fused_index_topk/long_cta_topk.cuh:116-309; the
// masked chunk producer kernel/csrc/repair/include/fused_index_topk/repair_producer.cuh:48-430;
// the sampled threshold kernel/csrc/sampling_threshold.cu:99-178.
#pragma once

#include "itk_ptx.cuh"

#include <cstddef>
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
constexpr int kSegCap = 1248;                  // shared-memory candidates per (row, segment)
constexpr int kRowCap = kSegments * kSegCap;   // 4992
constexpr int kSpillSegCap = 1408;             // global spill entries per (row, segment)
constexpr int kSpillRow = kSegments * kSpillSegCap;  // 5632 u64 per row
constexpr int kRepairChunk = 16384;

// Warp 0: TMA producer; warp 1: UMMA issuer; warps 2-17: epilogue and per-row selection (a warp may
// only read the TMEM lane quarter warp % 4, so sixteen consecutive warps cover every quarter four
// times: once per query row of the unit).  Five warps share the first two schedulers, which caps
// the kernel at 96 registers per thread.
constexpr int kThreads = 576;
constexpr int kEpilogueWarp0 = 2;
constexpr int kEpilogueThreads = 512;
constexpr int kEpilogueWarps = kEpilogueThreads / 32;
constexpr int kScoreBins = 256;
constexpr int kBinListCap = 128;    // scores of the histogram bin that holds the cutoff; more: radix fallback

constexpr uint32_t kQBytes = kUmmaN * kHeadDim;       // 32768
constexpr uint32_t kKvBytes = kTileKeys * kHeadDim;   // 16384

constexpr int kModeTopK = 0;
constexpr int kModeSample = 1;
constexpr int kModeRepair = 2;

constexpr int kStatusWaitExpired = 1;
constexpr int kStatusBadSharedBase = 2;   // the dynamic shared memory does not start on a 1 KB boundary

// Per-CTA phase trace of diagnostic builds (clock64 cycles unless noted).
constexpr int kTraceFields = 32;
constexpr int kTraceMmaTotal = 0, kTraceMmaWaitAcc = 1, kTraceMmaWaitKv = 2, kTraceMmaWaitQ = 3, kTraceMmaTiles = 4;
constexpr int kTraceTmaTotal = 8, kTraceTmaWaitKv = 9, kTraceTmaWaitQ = 10;
constexpr int kTraceEpiTotal = 12, kTraceEpiWaitAcc = 13, kTraceEpiSelect = 14, kTraceEpiWaitW = 15;  // +4 for query row 1
constexpr int kTraceSm = 24, kTraceNsBegin = 25, kTraceNsEnd = 26;

struct FusedParams {
    CUtensorMap map_q;    // [rows*64, 128] bytes, box 256 x 128, 128-byte swizzle
    CUtensorMap map_kv;   // [keys, 128] bytes (PAGED: the physical pool), box 128 x 128, 128-byte swizzle
    CUtensorMap map_sample;     // [samples, 128] gathered sample keys, kModeTopK with sample_tiles > 0
    const float* sample_scales; // [samples]           their scales
    const float* kv_scales;     // [keys] (PAGED: [physical keys])
    const int32_t* tile_table;  // PAGED builds: physical 128-key tile of every logical tile, [ceil(keys/128)]
    const float* weights;       // [rows, 64]
    const int32_t* k_start;     // [rows]
    const int32_t* k_end;       // [rows]
    const float* thresholds;    // [rows]              kModeTopK input
    float* thresholds_out;      // [rows]              kModeSample output
    const int32_t* sample_ids;  // [keys]              kModeSample: key position of each sample
    int32_t* out_ids;           // [rows, 2048]        kModeTopK output (may be null when out_pairs is set)
    uint64_t* out_pairs;        // [rows, 2048]        kModeTopK optional (ordered score << 32 | key)
    int32_t* out_counts;        // [rows]              number of pairs written (with out_pairs)
    uint8_t* failure_flags;     // [rows]              kModeTopK output / kModeRepair input
    uint64_t* shard_pairs;      // [shards, rows, 2048] pairs, counts and flags of the units that are one key
    int32_t* shard_counts;      // [shards, rows]       shard of a split query block (the merge of a row's
    uint8_t* shard_flags;       // [shards, rows]       shards decides about the row)
    uint64_t* spill;            // [4 * grid, 4, kSpillSegCap]: one region per CTA and query row of its current unit
    uint64_t* repair_pairs;     // [shards*rows, 16384] kModeRepair output, dense by key - chunk_lo
    float* diag_logits;         // [rows, diag_stride] dense scores, diagnostic builds only
    long long diag_stride;
    long long* trace;           // [grid, kTraceFields] per-CTA cycle counters, diagnostic builds only
    int* status;                // device status word, bits are or-ed in
    unsigned long long wait_limit_ns;  // wall-clock limit of every wait inside the kernel
    int withhold_q_loads;       // diagnostic builds only: the producer issues no load at all, so that the
                                // first wait for the query tile runs into wait_limit_ns (tests of the expiry path)
    int rows;                   // Q
    int keys;                   // N (or S in kModeSample)
    int key_lo;                 // first key of shard 0 (multiple of 128)
    int key_hi;                 // end of the last shard
    int shard_keys;             // keys per shard (multiple of 128)
    int shards;
    int split_blocks;           // the key range of this many owned blocks (the ones with the fewest keys: the
                                // lowest block numbers) is cut into `shards` units; the others are one unit each
    int block_begin;            // first owned query block
    int block_stride;           // stride between owned query blocks
    int num_blocks;             // owned query blocks
    int sample_rank;            // kModeSample, and kModeTopK with sample_tiles > 0
    int target_candidates;      // the same
    int sample_tiles;           // kModeTopK, > 0: a whole block scores the sample_count gathered sample keys (that many
    int sample_count;           // 128-key tiles) in front of its own keys and takes its rows' thresholds from them
                                // (written to thresholds_out as well), instead of reading `thresholds`
    int top_k_min_valid;        // rows with at most this many valid keys need no selection (= 2048)
    int exit_when_no_keys;      // 1: return at once when every row's key range is empty (nothing is written then)
};

// Per-row scratch of the selection.
struct RowSelect {
    union {
        int hist[256];                          // digit histogram of the radix selection, which clears it itself
        struct {                                // the binned selection, which never runs beside the radix one:
            uint32_t bin_scores[kBinListCap];   // the candidates of the histogram bin that holds the cutoff
            int32_t bin_keys[kBinListCap];
        };
    };
    int position;     // next free output position of the row
    int bin_count;
    int tickets;
    int bin;          // radix fallback: digit of the round
    int above;
    uint32_t reference;
    uint32_t differing;
};

struct __align__(16) FusedShared {
    // Histogram of a row's candidates over the binary exponent of their distance to the row
    // threshold (first pass of the selection).
    uint32_t row_hist[kBlockQ][kScoreBins];
    float weights[2][kBlockQ * kHeads];
    uint32_t cand_scores[kBlockQ][kRowCap];
    uint16_t cand_ids[kBlockQ][kRowCap];
    int counts[kBlockQ][kSegments];         // candidates of every (row, segment) in shared memory
    int spill_counts[kBlockQ][kSegments];   // candidates that went (or would have gone) to the segment's spill
    uint32_t scale_part[kBlockQ][kSegments];   // sampled median distance to the threshold, per segment
    float unit_threshold[kBlockQ];             // thresholds the unit computed itself (sample_tiles > 0)
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
constexpr size_t kFusedSmemBytes = kSmemTileBytes + sizeof(FusedShared);
static_assert(kSmemTileBytes % 1024 == 0, "FusedShared must start on a 1 KB boundary");
static_assert(kFusedSmemBytes <= 232448, "fused kernel exceeds the 227 KB shared-memory limit");
static_assert(kSegCap % 32 == 0 && kSpillSegCap % 32 == 0, "segment capacities are warp multiples");

// What a bounded wait needs besides the barrier: the CTA's abort flag and the time limit.
struct WaitCtl {
    volatile int* abort_flag;
    uint64_t limit_ns;
};

// mbar_wait that adds the cycles it took to `cycles` in diagnostic builds.
template <bool DIAG, uint32_t PARK_NS = kWaitParkNs>
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, long long& cycles) {
    if (DIAG) {
        const long long begin = clock64();
        const bool ok = mbar_wait<PARK_NS>(bar, parity, ctl.abort_flag, ctl.limit_ns);
        cycles += clock64() - begin;
        return ok;
    }
    return mbar_wait<PARK_NS>(bar, parity, ctl.abort_flag, ctl.limit_ns);
}

// ------------------------------------------------------------------ work units

struct Unit {
    int block;       // query block index
    int shard;
    bool split;      // one key shard of a split block: the result are pairs for the merge, and a shard that
                     // finds fewer than 2048 candidates returns them all instead of failing
    int row0;
    int nrows;
    int key_lo;
    int key_hi;
    int tile_begin;  // global tile indices (key >> 7)
    int tile_end;    // tile_begin == tile_end: nothing to compute
    int sample_tiles;  // tiles of gathered sample keys in front of the unit's own (its rows' thresholds come from them)
};

// Unit `iter` of this CTA.  Units are ordered longest first (later query blocks
// see more keys) and dealt to the CTAs in a serpentine so that every CTA gets a
// similar amount of work.  Every role of the CTA derives the same list.
template <int MODE>
__device__ __forceinline__ bool load_unit(const FusedParams& p, int iter, Unit& u) {
    const int grid = static_cast<int>(gridDim.x);
    const int cta = (iter & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
    const long long index = static_cast<long long>(iter) * grid + cta;
    // whole blocks first (the longest units), then the shards of the split blocks
    const long long whole = p.num_blocks - p.split_blocks;
    const long long total = whole + static_cast<long long>(p.split_blocks) * p.shards;
    if (index >= total) return false;
    int ordinal = static_cast<int>(index);
    u.shard = 0;
    u.split = index >= whole;
    if (u.split) {
        const long long inside = index - whole;
        ordinal = static_cast<int>(whole + inside / p.shards);
        u.shard = static_cast<int>(inside % p.shards);
    }
    u.block = p.block_begin + (p.num_blocks - 1 - ordinal) * p.block_stride;
    u.row0 = u.block * kBlockQ;
    u.nrows = min(kBlockQ, p.rows - u.row0);
    u.key_lo = u.split ? p.key_lo + u.shard * p.shard_keys : p.key_lo;
    u.key_hi = u.split ? min(p.key_hi, u.key_lo + p.shard_keys) : p.key_hi;
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
                needed = e - s > ((u.split || p.out_pairs != nullptr) ? 0 : p.top_k_min_valid);
            } else {
                needed = e > s && p.failure_flags[row] != 0;
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
    u.sample_tiles = (MODE == kModeTopK && !u.split && hi > lo) ? p.sample_tiles : 0;
    return true;
}

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
// A waiting warp parks in the hardware between probes: the warps of the other three rows share its
// scheduler and its shared-memory pipe, and a warp that polls without pause slows them several times.
constexpr uint32_t kRowParkNs = 200;

struct RowBarrier {
    uint64_t* bar;
    uint32_t phase;
    WaitCtl ctl;
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
    if (!mbar_wait<kRowParkNs>(rb.bar, rb.phase & 1u, rb.ctl.abort_flag, rb.ctl.limit_ns)) *rb.ctl.abort_flag = 1;
    ++rb.phase;
}

// The same barrier for warps that expect to wait long (one warp of the row works alone): a failed
// probe parks the warp instead of competing with the working warp for issue slots.
__device__ __forceinline__ void row_sync_parked(RowBarrier& rb) {
    __syncwarp();
    if ((threadIdx.x & 31u) == 0u) mbar_arrive(rb.bar);
    if (!mbar_wait<500>(rb.bar, rb.phase & 1u, rb.ctl.abort_flag, rb.ctl.limit_ns)) *rb.ctl.abort_flag = 1;
    ++rb.phase;
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

__device__ __forceinline__ int decode_key(uint32_t packed, int segment) {
    return static_cast<int>(((packed >> 5) << 7) | (static_cast<uint32_t>(segment) << 5) | (packed & 31u));
}

// The view a warp has of the candidates it owns during the selection: the segment it filled itself
// (its TMEM lane quarter) and that segment's spill region in global memory.  Lane l owns the
// entries j * 32 + l, j < lane_entries, of the segment: in the Top-K mode every thread of the
// epilogue appends to its own list (no warp vote per tile), in the sample mode the segment is
// filled densely and lane l simply has ceil((count - l) / 32) entries.
//
// Score words in shared memory are the float itself in the Top-K mode (RAW = true in the functions
// below: the selection works on distances to the row threshold) and its ordered integer image in the
// sample mode; the spill always holds (ordered score << 32 | key).
// A unit's spill is written and read back by the same CTA before its next unit starts, so the
// spill is addressed by CTA and row of the unit, not by query row: 4 regions per CTA.
__device__ __forceinline__ long long spill_slot(int r) { return static_cast<long long>(blockIdx.x) * kBlockQ + r; }

struct RowView {
    const uint32_t* scores;        // [kSegCap] of the warp's segment
    const uint16_t* ids;           // [kSegCap]
    const uint64_t* spill;         // [kSpillSegCap] of the warp's segment
    int lane_entries;              // entries of the calling lane in shared memory
    int max_entries;               // largest lane_entries of the warp
    int in_spill;                  // entries in the spill region
    int segment;
};

// The float `steps` representable values above (below, for negative steps) x.
__device__ __forceinline__ float neighbour_float(float x, int steps) {
    return ordered_to_float(ordered_bits(x) + static_cast<uint32_t>(steps));
}

template <bool RAW>
__device__ __forceinline__ uint32_t word_to_ordered(uint32_t word) {
    return RAW ? ordered_bits(__uint_as_float(word)) : word;
}

template <bool RAW>
__device__ __forceinline__ float word_to_value(uint32_t word) {
    return RAW ? __uint_as_float(word) : ordered_to_float(word);
}

// visit(ordered score) for every candidate of the calling lane: its list in shared memory, four
// entries at a time so that the loads of a group are in flight together, then its share of the spill
// region.  A visit may use shared-memory atomics but no warp-collective operation.
template <bool RAW, typename Visit>
__device__ __forceinline__ void for_scores(const RowView& v, int lane, Visit&& visit) {
    const uint32_t* scores = v.scores + lane;
    const int mine = v.lane_entries;
#pragma unroll 1
    for (int j = 0; j < mine; j += 4) {
        uint32_t s[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) s[k] = j + k < mine ? scores[(j + k) * 32] : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (j + k < mine) visit(word_to_ordered<RAW>(s[k]));
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

// Warp-wide result of find_rank: every lane gets the values of the lane that found the entry
// (entry -1 when no lane found it: the histogram holds fewer than `rank` candidates).
__device__ __forceinline__ void share_rank(bool found, int& entry, int& above, int& inside) {
    const unsigned who = __ballot_sync(0xffffffffu, found);
    const int source = who != 0u ? __ffs(who) - 1 : 0;
    entry = __shfl_sync(0xffffffffu, who != 0u ? entry : -1, source);
    above = __shfl_sync(0xffffffffu, above, source);
    inside = __shfl_sync(0xffffffffu, inside, source);
}

// One pass of a warp over its candidates that writes the selected ones.  classify(word) (the score
// word as stored in shared memory; spill entries are passed converted to the same form) returns 2
// for a candidate that is selected, 1 for one that is handed to on_listed(ordered score, key), 0
// otherwise.  Selected candidates get consecutive output positions from rs.position: four entries
// per lane are classified at a time, one shared-memory atomic per such group reserves the positions,
// the position inside the group comes from warp votes, so the stores of a warp instruction fall into
// a few sectors (every lane keeping its own run of positions made each store touch 32 sectors, which
// took several times longer).
template <bool RAW, typename Classify, typename Listed>
__device__ __forceinline__ void emit_pass(RowSelect& rs, const RowView& v, int lane, int32_t* out_ids,
                                          uint64_t* out_pairs, Classify&& classify, Listed&& on_listed) {
    const unsigned below = (1u << lane) - 1u;
    const auto write = [&](int at, uint32_t word, int key) {
        at = min(at, kTopK - 1);
        if (out_ids != nullptr) out_ids[at] = key;
        if (out_pairs != nullptr)
            out_pairs[at] = (static_cast<uint64_t>(word_to_ordered<RAW>(word)) << 32) | static_cast<uint32_t>(key);
    };
    const uint32_t* scores = v.scores + lane;
    const uint16_t* ids = v.ids + lane;
    const int mine = v.lane_entries, segment = v.segment;
#pragma unroll 1
    for (int j = 0; j < v.max_entries; j += 4) {
        uint32_t word[4], id[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const bool live = j + k < mine;
            word[k] = live ? scores[(j + k) * 32] : 0u;
            id[k] = live ? ids[(j + k) * 32] : 0u;
        }
        int kind[4];
        unsigned ballot[4];
        int group = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            kind[k] = j + k < mine ? classify(word[k]) : 0;
            ballot[k] = __ballot_sync(0xffffffffu, kind[k] == 2);
            group += __popc(ballot[k]);
        }
        int position = 0;
        if (lane == 0 && group > 0) position = atomicAdd(&rs.position, group);
        position = __shfl_sync(0xffffffffu, position, 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int key = decode_key(id[k], segment);
            if (kind[k] == 2) write(position + __popc(ballot[k] & below), word[k], key);
            else if (kind[k] == 1) on_listed(word_to_ordered<RAW>(word[k]), key);
            position += __popc(ballot[k]);
        }
    }
#pragma unroll 1
    for (int base = 0; base < v.in_spill; base += 32) {
        const int e = base + lane;
        const bool live = e < v.in_spill;
        const uint64_t pair = live ? v.spill[e] : 0ull;
        const uint32_t ordered = static_cast<uint32_t>(pair >> 32);
        const uint32_t word = RAW ? __float_as_uint(ordered_to_float(ordered)) : ordered;
        const int key = static_cast<int>(static_cast<uint32_t>(pair));
        const int kind = live ? classify(word) : 0;
        const unsigned ballot = __ballot_sync(0xffffffffu, kind == 2);
        int position = 0;
        if (lane == 0 && ballot != 0u) position = atomicAdd(&rs.position, __popc(ballot));
        position = __shfl_sync(0xffffffffu, position, 0);
        if (kind == 2) write(position + __popc(ballot & below), word, key);
        else if (kind == 1) on_listed(ordered, key);
    }
}

// Median (upper median) of the calling warp's valid values, one per lane, as a warp-uniform result;
// 0 when fewer than four lanes hold a valid value.  Values are compared as unsigned integers.
__device__ __forceinline__ uint32_t warp_median(uint32_t value, bool valid, int lane) {
    const unsigned who = __ballot_sync(0xffffffffu, valid);
    const int live = __popc(who);
    int below = 0;   // valid values that sort before this lane's (ties: the lower lane first)
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
        const uint32_t other = __shfl_sync(0xffffffffu, value, k);
        const bool counts = ((who >> k) & 1u) != 0u && (other < value || (other == value && k < lane));
        below += counts ? 1 : 0;
    }
    const unsigned median_lane = __ballot_sync(0xffffffffu, valid && below == live / 2);
    const uint32_t median = __shfl_sync(0xffffffffu, value, median_lane != 0u ? __ffs(median_lane) - 1 : 0);
    return live >= 4 ? median : 0u;
}

// Exact Top-2048 of a row whose candidates lie above a finite threshold (Top-K mode: the score words
// are floats).  `width` is a robust scale of the candidates' distances to the threshold (four times
// the median of a sample of them): 256 equal bins over [0, width) resolve the lower, densely
// populated part of the distances, where the 2048th largest score lies, to a couple of dozen
// candidates per bin; the few large distances beyond (all of them selected anyway) share the last bin.
//   1. histogram of the bins (one pass of every warp over its own candidates); the bin that holds
//      the 2048th largest score is read off it, by every warp redundantly;
//   2. the bin's two edges are turned into score values (exactly: the edge is moved until the bin
//      arithmetic agrees), so that the second pass classifies a candidate with two comparisons: above
//      the bin it goes to the output, inside the bin onto a list;
//   3. one warp ranks the list and writes its largest entries to the remaining positions (ties: the
//      first ones of the list).
// Returns false, with nothing written, when the list would hold more than kBinListCap scores (many
// equal or nearly equal scores, or a scale that does not fit the row); the caller then falls back to
// the radix selection.  Called by the 128 threads of a row after the barrier that publishes the
// row's counts; row_hist, rs.bin_count and rs.position are zero on entry.
__device__ __forceinline__ bool binned_select(RowSelect& rs, const RowView& v, uint32_t* row_hist, float threshold,
                                              float width, RowBarrier& rb, int tid, int32_t* out_ids,
                                              uint64_t* out_pairs) {
    const int lane = tid & 31;
    const float bins_per_unit = static_cast<float>(kScoreBins) / width;
    const auto bin_of = [&](float score) -> int {
        return __float2int_rz(fminf((score - threshold) * bins_per_unit, static_cast<float>(kScoreBins - 1)));
    };
    {
        const uint32_t* scores = v.scores + lane;
        const int mine = v.lane_entries;
#pragma unroll 1
        for (int j = 0; j < mine; j += 4) {
            float s[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] = j + k < mine ? __uint_as_float(scores[(j + k) * 32]) : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (j + k < mine) atomicAdd(&row_hist[bin_of(s[k])], 1u);
        }
#pragma unroll 1
        for (int e = lane; e < v.in_spill; e += 32)
            atomicAdd(&row_hist[bin_of(ordered_to_float(static_cast<uint32_t>(v.spill[e] >> 32)))], 1u);
    }
    lap(rb, 1);
    row_sync(rb);
    int cutoff_bin, above, in_list;
    {
        int counts[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) counts[j] = static_cast<int>(row_hist[lane * 8 + j]);
        const bool found = find_rank(counts, lane, kTopK, cutoff_bin, above, in_list);
        share_rank(found, cutoff_bin, above, in_list);
    }
    if (cutoff_bin < 0 || in_list > kBinListCap) {
        if (rb.lap != nullptr) rb.lap[0] = cutoff_bin < 0 ? 1000000 : 2000000 + in_list * 256 + cutoff_bin;
        return false;
    }
    // Smallest score of bin `b` (bin_of is monotone in the score).  Start from the arithmetic edge and
    // move by single floats; that settles within a step or two unless the edge lies much closer to zero
    // than the threshold does (a negative threshold, scores around zero): there one float of the edge
    // is far smaller than the rounding of threshold + distance, and the edge is bisected over the
    // ordered images of the floats between the threshold and the end of the bins instead.
    const auto lower_edge = [&](int b) -> float {
        if (b <= 0) return threshold;   // every candidate is at or above the threshold
        float edge = threshold + static_cast<float>(b) / bins_per_unit;
#pragma unroll 1
        for (int step = 0; step < 8 && bin_of(edge) < b; ++step) edge = neighbour_float(edge, 1);
#pragma unroll 1
        for (int step = 0; step < 8; ++step) {
            const float lower = neighbour_float(edge, -1);
            if (bin_of(lower) < b) break;
            edge = lower;
        }
        if (bin_of(edge) >= b && bin_of(neighbour_float(edge, -1)) < b) return edge;
        uint32_t below = ordered_bits(threshold);           // bin 0 < b
        uint32_t reached = ordered_bits(threshold + width);  // the last bin
#pragma unroll 1
        while (reached - below > 1u) {
            const uint32_t middle = below + ((reached - below) >> 1);
            if (bin_of(ordered_to_float(middle)) >= b) reached = middle;
            else below = middle;
        }
        return ordered_to_float(reached);
    };
    const float list_from = lower_edge(cutoff_bin);
    const float take_from = cutoff_bin >= kScoreBins - 1 ? __int_as_float(0x7f800000) : lower_edge(cutoff_bin + 1);
    // the edges must agree with the histogram, else the counts would not add up: check them
    bool edges_ok = bin_of(list_from) == cutoff_bin && (cutoff_bin >= kScoreBins - 1 || bin_of(take_from) == cutoff_bin + 1);
    edges_ok = edges_ok && !(cutoff_bin > 0 && bin_of(neighbour_float(list_from, -1)) >= cutoff_bin);
    edges_ok = edges_ok && !(cutoff_bin < kScoreBins - 1 && bin_of(neighbour_float(take_from, -1)) > cutoff_bin);
    if (!edges_ok) {
        if (rb.lap != nullptr) rb.lap[0] = 3000000 + cutoff_bin;
        return false;
    }
    lap(rb, 2);
    emit_pass<true>(rs, v, lane, out_ids, out_pairs,
                    [&](uint32_t word) {
                        const float score = __uint_as_float(word);
                        return score >= take_from ? 2 : (score >= list_from ? 1 : 0);
                    },
                    [&](uint32_t ordered, int key) {
                        const int at = atomicAdd(&rs.bin_count, 1);
                        if (at < kBinListCap) {
                            rs.bin_scores[at] = ordered;
                            rs.bin_keys[at] = key;
                        }
                    });
    lap(rb, 3);
    row_sync(rb);
    // The list's `need` largest scores complete the row: an entry is taken when fewer than `need`
    // entries are above it, counting equal scores that come earlier in the list as above.
    if (tid < 32) {
        const int need = kTopK - above;
        in_list = min(in_list, kBinListCap);
#pragma unroll 1
        for (int k = 0; k * 32 < in_list; ++k) {
            const int i = lane + 32 * k;
            const uint32_t mine = i < in_list ? rs.bin_scores[i] : 0u;
            int before = 0;
#pragma unroll 4
            for (int j = 0; j < in_list; ++j) {
                const uint32_t other = rs.bin_scores[j];
                before += (other > mine || (other == mine && j < i)) ? 1 : 0;
            }
            if (i < in_list && before < need) {
                const int key = rs.bin_keys[i];
                if (out_ids != nullptr) out_ids[above + before] = key;
                if (out_pairs != nullptr) out_pairs[above + before] = (static_cast<uint64_t>(mine) << 32) | static_cast<uint32_t>(key);
            }
        }
    }
    lap(rb, 4);
    return true;
}

// Radix selection over the ordered score bits of one row, up to 8 bits per round: the fallback for
// rows whose cutoff bin is too full (many equal or nearly equal scores), and the selection of the
// sample mode beyond 512 samples.  On return `cutoff` is the rank-th largest score and
// `equal_needed` the number of candidates equal to it that belong to the top `rank_in`.  The leading
// bits that all candidates share are found first and skipped.
template <bool RAW>
__device__ __forceinline__ void radix_select(RowSelect& rs, const RowView& v, RowBarrier& rb, int tid, int rank_in,
                                             uint32_t& cutoff, int& equal_needed) {
    const int lane = tid & 31;
    if (tid == 0) {
        rs.differing = 0u;
        rs.reference = 0u;
    }
    row_sync(rb);
    // any candidate of the row serves as the reference (the row has at least rank_in >= 1 candidates)
    if (lane == 0 && v.lane_entries > 0) atomicMax(&rs.reference, word_to_ordered<RAW>(v.scores[0]));
    if (lane == 0 && v.lane_entries == 0 && v.in_spill > 0) atomicMax(&rs.reference, static_cast<uint32_t>(v.spill[0] >> 32));
    row_sync(rb);
    const uint32_t reference = rs.reference;
    uint32_t differing = 0u;
    for_scores<RAW>(v, lane, [&](uint32_t score) { differing |= score ^ reference; });
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
        for_scores<RAW>(v, lane, [&](uint32_t score) {
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

// Writes the selected candidates of one row when the cutoff (an ordered score) is known: everything
// above `cutoff`, then `equal_needed` of the candidates equal to it (any of them); cutoff 0 takes
// every candidate.  greater_total = number of candidates above the cutoff (their positions come
// first).  rs.position and rs.tickets must be 0 on entry (a row barrier before the call publishes that).
template <bool RAW>
__device__ __forceinline__ void emit_row(RowSelect& rs, const RowView& v, int lane, uint32_t cutoff, int equal_needed,
                                         int greater_total, int32_t* out_ids, uint64_t* out_pairs) {
    emit_pass<RAW>(rs, v, lane, out_ids, out_pairs,
                   [&](uint32_t word) {
                       const uint32_t score = word_to_ordered<RAW>(word);
                       return score > cutoff ? 2 : (score == cutoff && cutoff != 0u ? 1 : 0);
                   },
                   [&](uint32_t ordered, int key) {
                       const int ticket = atomicAdd(&rs.tickets, 1);
                       if (ticket < equal_needed) {
                           const int at = min(greater_total + ticket, kTopK - 1);
                           if (out_ids != nullptr) out_ids[at] = key;
                           if (out_pairs != nullptr) out_pairs[at] = (static_cast<uint64_t>(ordered) << 32) | static_cast<uint32_t>(key);
                       }
                   });
}

// Exact Top-2048 of one row from its candidates.  Called by the 128 threads of row r after the
// row's four segment totals are in shared memory and the row barrier has been passed (lane_entries:
// the calling lane's own number of entries in its segment); returns with the row barrier passed
// again (the candidate buffers and the histograms may be reused).
__device__ __forceinline__ void select_topk_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                bool has_tiles, RowBarrier& rb, int tid, int lane_entries) {
    const int row = u.row0 + r;
    // a shard of a split block writes pairs, count and flag of its own; a whole block the row's
    const long long row_slot = u.split ? static_cast<long long>(u.shard) * p.rows + row : row;
    const int start = max(__ldg(p.k_start + row), u.key_lo);
    const int end = min(min(__ldg(p.k_end + row), p.keys), u.key_hi);
    const int valid = max(end - start, 0);
    int32_t* out_ids = !u.split && p.out_ids != nullptr ? p.out_ids + static_cast<long long>(row) * kTopK : nullptr;
    uint64_t* const pair_base = u.split ? p.shard_pairs : p.out_pairs;
    uint64_t* out_pairs = pair_base != nullptr ? pair_base + row_slot * kTopK : nullptr;
    int32_t* const out_counts = u.split ? p.shard_counts : p.out_counts;
    uint8_t* const failure_flags = u.split ? p.shard_flags : p.failure_flags;

    if (out_pairs == nullptr && valid <= p.top_k_min_valid) {
        // every valid key is selected; no scores are needed
        for (int i = tid; i < kTopK; i += kRowThreads) out_ids[i] = i < valid ? start + i : -1;
        if (tid == 0) failure_flags[row_slot] = 0;
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
            failure_flags[row_slot] = 0;
            if (out_counts != nullptr) out_counts[row_slot] = 0;
        }
        return;
    }

    RowSelect& rs = sh.select[r];
    const int lane = tid & 31;
    const int segment = tid >> 5;
    const float threshold = valid > kTopK ? (u.sample_tiles > 0 ? sh.unit_threshold[r] : __ldg(p.thresholds + row))
                                          : __int_as_float(0xff800000);
    RowView view;
    view.segment = segment;
    view.scores = sh.cand_scores[r] + segment * kSegCap;
    view.ids = sh.cand_ids[r] + segment * kSegCap;
    view.spill = p.spill + spill_slot(r) * kSpillRow + segment * kSpillSegCap;
    view.lane_entries = lane_entries;
    view.max_entries = __reduce_max_sync(0xffffffffu, lane_entries);
    // Every warp publishes the number of candidates in its segment and the median distance to the
    // threshold of a sample of them (the first entry of every lane); one barrier, after which all
    // four warps of the row know the totals and agree on a scale for the selection's bins.
    {
        // sample: the last entry of every lane (the first ones are the lowest key positions, where
        // attention sinks sit)
        const uint32_t sample = lane_entries > 0
            ? __float_as_uint(__uint_as_float(view.scores[(lane_entries - 1) * 32 + lane]) - threshold) : 0u;
        const uint32_t median = warp_median(sample, lane_entries > 0 && sample < 0x7f800000u, lane);
        const int in_segment = __reduce_add_sync(0xffffffffu, lane_entries);
        if (lane == 0) {
            sh.counts[r][segment] = in_segment;
            sh.scale_part[r][segment] = median;
        }
    }
    row_sync(rb);
    int total = 0;
    bool overflow = false;
    uint32_t scale_bits = 0u;
#pragma unroll
    for (int s = 0; s < kSegments; ++s) {
        total += sh.counts[r][s] + min(sh.spill_counts[r][s], kSpillSegCap);
        overflow = overflow || sh.spill_counts[r][s] > kSpillSegCap;
        scale_bits = max(scale_bits, sh.scale_part[r][s]);
    }
    view.in_spill = min(sh.spill_counts[r][segment], kSpillSegCap);
    const int wanted = min(valid, kTopK);
    uint32_t* row_hist = sh.row_hist[r];
    if (overflow || (total < wanted && !u.split)) {
        // too many candidates for the buffers or too few for a full answer: the repair pass redoes the row
        // (a shard of a split block may come up short: the merge of the shards checks the total)
        fill_empty(0);
        if (tid == 0) {
            failure_flags[row_slot] = 1;
            if (out_counts != nullptr) out_counts[row_slot] = 0;
        }
    } else {
        if (rb.lap != nullptr) rb.lap_start = clock64();
        if (total <= kTopK) {
            // only reachable when valid <= 2048 or a shard came up short: take everything
            emit_row<true>(rs, view, lane, 0u, 0, 0, out_ids, out_pairs);
            fill_empty(total);
        } else {
            // bins of the selection: 256 over [0, 4 x the largest of the four sampled medians)
            const float width = 4.0f * __uint_as_float(scale_bits);
            const bool usable = scale_bits != 0u && width < 3.0e38f;
            if (!usable || !binned_select(rs, view, row_hist, threshold, width, rb, tid, out_ids, out_pairs)) {
                if (rb.lap != nullptr) {
                    rb.lap[7] += 1;
                    if (!usable) rb.lap[0] = 4000000;
                }
                uint32_t cutoff;
                int equal_needed;
                radix_select<true>(rs, view, rb, tid, kTopK, cutoff, equal_needed);
                emit_row<true>(rs, view, lane, cutoff, equal_needed, kTopK - equal_needed, out_ids, out_pairs);
            }
            lap(rb, 5);
        }
        if (tid == 0) {
            failure_flags[row_slot] = 0;
            if (out_counts != nullptr) out_counts[row_slot] = min(total, kTopK);
        }
    }
    row_sync(rb);   // every warp is done with the candidates, the histograms and the list
    // leave the selection's scratch clean for the row's next selection, whose first barrier
    // (the one that publishes the counts) orders these stores before any use
    for (int i = tid; i < kScoreBins; i += kRowThreads) {
        row_hist[i] = 0u;
        rs.hist[i] = 0;
    }
    if (tid < kSegments) sh.spill_counts[r][tid] = 0;
    if (tid == 0) {
        rs.position = 0;
        rs.tickets = 0;
        rs.bin_count = 0;
    }
    lap(rb, 6);
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
            // the dense segment as per-lane lists: lane l owns the entries l, l + 32, ...
            view.lane_entries = max(sh.counts[r][segment] - (tid & 31) + 31, 0) >> 5;
            view.max_entries = (sh.counts[r][segment] + 31) >> 5;
            view.in_spill = 0;
            uint32_t cutoff;
            int equal_needed;
            radix_select<false>(sh.select[r], view, rb, tid, p.sample_rank, cutoff, equal_needed);
            result = ordered_to_float(cutoff);
        }
    }
    if (solo ? tid == (r & 3) * 32 : tid == 0) {
        p.thresholds_out[row] = result;
        sh.unit_threshold[r] = result;   // read by the row's warps after their next barrier
    }
    return solo;
}

// ------------------------------------------------------------------ epilogue arithmetic

// ReLU of two neighbouring accumulator columns and their packed multiply-add with the two head
// weights.  The ReLU is fma.rn.sat(x, 2^-25, 0) on the FMA pipe rather than max(x, 0), which the
// integer/compare pipe issues at half rate: |x| <= 128 * 448^2 < 2^25, so the saturating multiply
// by 2^-25 is exact for x > 0, clamps x <= 0 (and NaN) to +0 and never reaches the upper clamp; the
// head weights are pre-multiplied by 2^25 (exact for |w| < 2^103), so that every product, and with
// it every partial sum, is bit-identical to the max form.  The two accumulator registers are
// neighbours of an even/odd register pair already (they come out of one tcgen05.ld), so packing them
// costs no move.
template <bool FIRST>
__device__ __forceinline__ void relu_fma(uint32_t& x0, uint32_t& x1, uint64_t wpair, uint64_t& acc) {
    float& f0 = *reinterpret_cast<float*>(&x0);
    float& f1 = *reinterpret_cast<float*>(&x1);
    if (FIRST) {
        asm("{\n\t.reg .b64 t;\n\t"
            "fma.rn.sat.f32 %0, %0, 0f33000000, 0f00000000;\n\t"
            "fma.rn.sat.f32 %1, %1, 0f33000000, 0f00000000;\n\t"
            "mov.b64 t, {%0, %1};\n\tmul.rn.f32x2 %2, t, %3;\n\t}"
            : "+f"(f0), "+f"(f1), "=l"(acc)
            : "l"(wpair));
    } else {
        asm("{\n\t.reg .b64 t;\n\t"
            "fma.rn.sat.f32 %0, %0, 0f33000000, 0f00000000;\n\t"
            "fma.rn.sat.f32 %1, %1, 0f33000000, 0f00000000;\n\t"
            "mov.b64 t, {%0, %1};\n\tfma.rn.f32x2 %2, t, %3, %2;\n\t}"
            : "+f"(f0), "+f"(f1), "+l"(acc)
            : "l"(wpair));
    }
}

constexpr float kSatUnscale = 33554432.0f;   // 2^25

// One fragment (all 64 accumulator columns of a query row for TMEM lanes l and l+8: r[4n], r[4n+1]
// belong to lane l, r[4n+2], r[4n+3] to lane l+8, column pair n = 0..7) into the packed partial
// sums of the two lanes.
__device__ __forceinline__ void fragment_fma(uint32_t (&r)[32], const uint64_t (&w)[8], uint64_t& acc_a,
                                             uint64_t& acc_b) {
#define ITK_STEP(N, F)                                          \
    relu_fma<F>(r[4 * N + 0], r[4 * N + 1], w[N], acc_a);       \
    relu_fma<F>(r[4 * N + 2], r[4 * N + 3], w[N], acc_b);
    ITK_STEP(0, true)
    ITK_STEP(1, false)
    ITK_STEP(2, false)
    ITK_STEP(3, false)
    ITK_STEP(4, false)
    ITK_STEP(5, false)
    ITK_STEP(6, false)
    ITK_STEP(7, false)
#undef ITK_STEP
}

__device__ __forceinline__ float pair_sum(uint64_t packed) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(packed));
    return lo + hi;
}

// Threshold filter and store of one score in the Top-K mode, without a branch and without a warp
// vote: the thread appends to its own candidate list (entry j of lane l of the segment sits at index
// j * 32 + l, so the stores of a warp never meet in a bank).  score_at / id_at are the byte addresses
// of the thread's next free entry, limit_at the end of its list.  Returns nonzero when the score is a
// candidate but the list is full (the caller spills it).
__device__ __forceinline__ uint32_t filter_store(float score, uint32_t score_bits, int key, int row_lo, unsigned row_span,
                                                 float threshold, uint32_t id16, uint32_t& score_at, uint32_t& id_at,
                                                 uint32_t limit_at) {
    uint32_t full;
    asm volatile(
        "{\n\t"
        ".reg .pred in_range, active, room;\n\t"
        ".reg .u32 offset;\n\t"
        "sub.u32 offset, %3, %4;\n\t"
        "setp.lt.u32 in_range, offset, %5;\n\t"
        "setp.ge.and.f32 active, %6, %7, in_range;\n\t"
        "setp.lt.and.u32 room, %0, %8, active;\n\t"
        "@room st.shared.u32 [%0], %9;\n\t"
        "@room st.shared.u16 [%1], %10;\n\t"
        "@room add.u32 %0, %0, 128;\n\t"
        "@room add.u32 %1, %1, 64;\n\t"
        "xor.pred room, room, active;\n\t"
        "selp.u32 %2, 1, 0, room;\n\t"
        "}"
        : "+r"(score_at), "+r"(id_at), "=r"(full)
        : "r"(key), "r"(row_lo), "r"(row_span), "f"(score), "f"(threshold), "r"(limit_at), "r"(score_bits),
          "h"(static_cast<uint16_t>(id16))
        : "memory");
    return full;
}

// One lane of the warp (elected by the hardware) arrives on the barrier; no branch.
__device__ __forceinline__ void mbar_arrive_elected(uint32_t bar_address) {
    asm volatile(
        "{\n\t"
        ".reg .pred leader;\n\t"
        "elect.sync _|leader, 0xffffffff;\n\t"
        "@leader mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
        "}"
        ::"r"(bar_address)
        : "memory");
}

// ------------------------------------------------------------------ the Top-K tile loop in PTX

// The tile loop of an epilogue warp in the Top-K mode, written in PTX as one block: every branch in
// it is uniform (warp votes decide), every per-thread decision is a predicate, and the addresses and
// counters that change from tile to tile are carried in registers.  The same loop written in C++
// compiled to about a third more instructions per tile (divergence scaffolding around votes,
// shuffles and the one-lane barrier arrival, re-derived indices, register moves), and the epilogue
// is bound by instruction issue.
//
// Per tile: wait for the accumulator (one parked probe and a vote; if that fails the loop is left
// so that the caller can do the bounded wait), load the 16-lane halves of the warp's TMEM quarter
// one after the other through the same 32 registers, ReLU and packed multiply-add with the head
// weights, hand the accumulator back after the second load, reduce the four partial head sums of a
// quad so that every thread owns the score of one key, multiply by the key scale (prefetched one
// tile ahead), filter against range and threshold and append the candidate to the thread's own list.
//
// Returns why it stopped: kLoopDone (tile_end reached), kLoopNeedWait (the accumulator of tile t is
// not there yet), kLoopSpill (some thread's list is full: `full` is nonzero in those threads, whose
// candidate of the tile just finished, key - 128 with score last_score, goes to the spill).
constexpr uint32_t kLoopDone = 0, kLoopNeedWait = 1, kLoopSpill = 2;

#define ITK_PTX_RELU(r) "fma.rn.sat.f32 " r ", " r ", 0f33000000, 0f00000000;\n\t"
// column pair of TMEM lane l (registers a0, a1) and of lane l+8 (b0, b1) with weight pair W
#define ITK_PTX_PAIR_FIRST(a0, a1, b0, b1, W)                                                        \
    ITK_PTX_RELU(a0) ITK_PTX_RELU(a1) "mov.b64 pa, {" a0 ", " a1 "};\n\tmul.rn.f32x2 acc_a, pa, " W ";\n\t" \
    ITK_PTX_RELU(b0) ITK_PTX_RELU(b1) "mov.b64 pb, {" b0 ", " b1 "};\n\tmul.rn.f32x2 acc_b, pb, " W ";\n\t"
#define ITK_PTX_PAIR(a0, a1, b0, b1, W)                                                                      \
    ITK_PTX_RELU(a0) ITK_PTX_RELU(a1) "mov.b64 pa, {" a0 ", " a1 "};\n\tfma.rn.f32x2 acc_a, pa, " W ", acc_a;\n\t" \
    ITK_PTX_RELU(b0) ITK_PTX_RELU(b1) "mov.b64 pb, {" b0 ", " b1 "};\n\tfma.rn.f32x2 acc_b, pb, " W ", acc_b;\n\t"
#define ITK_PTX_FRAGMENT                                       \
    ITK_PTX_PAIR_FIRST("r0", "r1", "r2", "r3", "%21")          \
    ITK_PTX_PAIR("r4", "r5", "r6", "r7", "%22")                \
    ITK_PTX_PAIR("r8", "r9", "r10", "r11", "%23")              \
    ITK_PTX_PAIR("r12", "r13", "r14", "r15", "%24")            \
    ITK_PTX_PAIR("r16", "r17", "r18", "r19", "%25")            \
    ITK_PTX_PAIR("r20", "r21", "r22", "r23", "%26")            \
    ITK_PTX_PAIR("r24", "r25", "r26", "r27", "%27")            \
    ITK_PTX_PAIR("r28", "r29", "r30", "r31", "%28")
#define ITK_PTX_LOAD_FRAGMENT                                                                                  \
    "tcgen05.ld.sync.aligned.16x256b.x8.b32 "                                                                  \
    "{r0, r1, r2, r3, r4, r5, r6, r7, r8, r9, r10, r11, r12, r13, r14, r15, "                                  \
    "r16, r17, r18, r19, r20, r21, r22, r23, r24, r25, r26, r27, r28, r29, r30, r31}, [taddr];\n\t"

__device__ __forceinline__ uint32_t topk_tile_loop(int& t, int& acc_iter, int& key, uint16_t& id16, float& scale,
                                                   uint32_t& score_at, uint32_t& id_at, uint32_t& full,
                                                   float& last_score, int tile_end, uint32_t limit_at, int row_lo,
                                                   unsigned row_span, float threshold, const float* kv_scales,
                                                   int last_key, uint32_t tile_done_bars, uint32_t acc_empty_bars,
                                                   uint32_t tmem_lane, int lane, const uint64_t (&w)[8]) {
    uint32_t why;
    asm volatile(
        "{\n\t"
        ".reg .pred p_odd, p_upper, p_ready, p_in, p_act, p_room, p_full, p_any, p_more, p_lead;\n\t"
        ".reg .b32 r<32>;\n\t"
        ".reg .b64 acc_a, acc_b, pa, pb, scale_at;\n\t"
        ".reg .f32 lo, hi, v0, v1, v2, v3, sa, sb, ka, kb, ra, rb, kk, ss, rr, sum, nscale;\n\t"
        ".reg .u32 stage, bar, parity, buf, taddr, abar, off, tmp;\n\t"
        ".reg .s32 knext;\n\t"
        "and.b32 tmp, %20, 1;\n\t"
        "setp.ne.u32 p_odd, tmp, 0;\n\t"
        "and.b32 tmp, %20, 2;\n\t"
        "setp.ne.u32 p_upper, tmp, 0;\n\t"
        "mov.u32 %8, 0;\n\t"
        "mov.f32 %9, 0f00000000;\n\t"
        "mov.u32 %7, 0;\n\t"
        "setp.lt.s32 p_more, %0, %10;\n\t"
        "@!p_more bra.uni ITK_LOOP_END;\n"
        "ITK_LOOP:\n\t"
        // the tile's barrier: stage = tile counter % 4, phase parity = (tile counter / 4) % 2
        "and.b32 stage, %1, 3;\n\t"
        "mad.lo.u32 bar, stage, 8, %17;\n\t"
        "shr.u32 parity, %1, 2;\n\t"
        "and.b32 parity, parity, 1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p_ready, [bar], parity, 2000;\n\t"
        "vote.sync.all.pred p_ready, p_ready, 0xffffffff;\n\t"
        "@!p_ready bra.uni ITK_LOOP_WAIT;\n\t"
        "tcgen05.fence::after_thread_sync;\n\t"
        "and.b32 buf, %1, 1;\n\t"
        "mad.lo.u32 taddr, buf, 256, %19;\n\t"
        ITK_PTX_LOAD_FRAGMENT
        // the next tile's key scale (an index past the last key is clamped: such a key is outside every range)
        "add.s32 knext, %2, 128;\n\t"
        "min.s32 knext, knext, %16;\n\t"
        "mad.wide.s32 scale_at, knext, 4, %15;\n\t"
        "ld.global.nc.f32 nscale, [scale_at];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n\t"
        ITK_PTX_FRAGMENT
        "add.u32 taddr, taddr, 1048576;\n\t"   // TMEM lanes 16-31 of the quarter
        ITK_PTX_LOAD_FRAGMENT
        "mov.b64 {lo, hi}, acc_a;\n\t"
        "add.f32 v0, lo, hi;\n\t"
        "mov.b64 {lo, hi}, acc_b;\n\t"
        "add.f32 v1, lo, hi;\n\t"
        "tcgen05.wait::ld.sync.aligned;\n\t"
        // the accumulator buffer is fully read: hand it back
        "tcgen05.fence::before_thread_sync;\n\t"
        "mad.lo.u32 abar, buf, 8, %18;\n\t"
        "elect.sync _|p_lead, 0xffffffff;\n\t"
        "@p_lead mbarrier.arrive.shared::cta.b64 _, [abar];\n\t"
        ITK_PTX_FRAGMENT
        "mov.b64 {lo, hi}, acc_a;\n\t"
        "add.f32 v2, lo, hi;\n\t"
        "mov.b64 {lo, hi}, acc_b;\n\t"
        "add.f32 v3, lo, hi;\n\t"
        // reduce-scatter of the four partial sums over the four threads of a quad
        "selp.f32 sa, v0, v1, p_odd;\n\t"
        "selp.f32 sb, v2, v3, p_odd;\n\t"
        "selp.f32 ka, v1, v0, p_odd;\n\t"
        "selp.f32 kb, v3, v2, p_odd;\n\t"
        "shfl.sync.bfly.b32 ra, sa, 1, 0x1f, 0xffffffff;\n\t"
        "shfl.sync.bfly.b32 rb, sb, 1, 0x1f, 0xffffffff;\n\t"
        "add.f32 ka, ka, ra;\n\t"
        "add.f32 kb, kb, rb;\n\t"
        "selp.f32 kk, kb, ka, p_upper;\n\t"
        "selp.f32 ss, ka, kb, p_upper;\n\t"
        "shfl.sync.bfly.b32 rr, ss, 2, 0x1f, 0xffffffff;\n\t"
        "add.f32 sum, kk, rr;\n\t"
        // score (the fused add of +0 turns a -0 product into +0), filter, append to the thread's list
        "fma.rn.f32 %9, sum, %4, 0f00000000;\n\t"
        "sub.u32 off, %2, %12;\n\t"
        "setp.lt.u32 p_in, off, %13;\n\t"
        "setp.ge.and.f32 p_act, %9, %14, p_in;\n\t"
        "setp.lt.and.u32 p_room, %5, %11, p_act;\n\t"
        "@p_room st.shared.b32 [%5], %9;\n\t"
        "@p_room st.shared.u16 [%6], %3;\n\t"
        "@p_room add.u32 %5, %5, 128;\n\t"
        "@p_room add.u32 %6, %6, 64;\n\t"
        "xor.pred p_full, p_room, p_act;\n\t"
        "vote.sync.any.pred p_any, p_full, 0xffffffff;\n\t"
        // next tile
        "add.s32 %0, %0, 1;\n\t"
        "add.s32 %1, %1, 1;\n\t"
        "add.s32 %2, %2, 128;\n\t"
        "add.u16 %3, %3, 32;\n\t"
        "mov.f32 %4, nscale;\n\t"
        "@p_any bra.uni ITK_LOOP_SPILL;\n\t"
        "setp.lt.s32 p_more, %0, %10;\n\t"
        "@p_more bra.uni ITK_LOOP;\n\t"
        "bra.uni ITK_LOOP_END;\n"
        "ITK_LOOP_WAIT:\n\t"
        "mov.u32 %7, 1;\n\t"
        "bra.uni ITK_LOOP_END;\n"
        "ITK_LOOP_SPILL:\n\t"
        "selp.u32 %8, 1, 0, p_full;\n\t"
        "mov.u32 %7, 2;\n"
        "ITK_LOOP_END:\n\t"
        "}"
        : "+r"(t), "+r"(acc_iter), "+r"(key), "+h"(id16), "+f"(scale), "+r"(score_at), "+r"(id_at), "=&r"(why),
          "=&r"(full), "=&f"(last_score)
        : "r"(tile_end), "r"(limit_at), "r"(row_lo), "r"(row_span), "f"(threshold), "l"(kv_scales), "r"(last_key),
          "r"(tile_done_bars), "r"(acc_empty_bars), "r"(tmem_lane), "r"(lane), "l"(w[0]), "l"(w[1]), "l"(w[2]),
          "l"(w[3]), "l"(w[4]), "l"(w[5]), "l"(w[6]), "l"(w[7])
        : "memory");
    return why;
}
#undef ITK_PTX_LOAD_FRAGMENT
#undef ITK_PTX_FRAGMENT
#undef ITK_PTX_PAIR
#undef ITK_PTX_PAIR_FIRST
#undef ITK_PTX_RELU

// What the epilogue needs to know about one query row of a unit.
struct RowState {
    int lo, hi;          // key range of the row inside the unit's key slice
    float threshold;
    bool on;             // the row takes part in this launch
    long long slot;      // the row
};

template <int MODE>
__device__ __forceinline__ RowState load_row_state(const FusedParams& p, int row0, int nrows, bool split,
                                                   int unit_key_lo, int unit_key_hi, int r) {
    RowState state{0, 0, __int_as_float(0xff800000), r < nrows, 0};
    if (state.on) {
        const int row = row0 + r;
        state.slot = row;
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
                if (valid > kTopK) state.threshold = __ldg(p.thresholds + row);
                state.on = valid > ((split || p.out_pairs != nullptr) ? 0 : p.top_k_min_valid);
            } else {
                state.on = p.failure_flags[state.slot] != 0;
            }
        }
    }
    return state;
}

// Lane 0 waits on the barrier, the warp then reconverges: one poller per warp.
template <bool DIAG, uint32_t PARK_NS = kWaitParkNs>
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int lane,
                                          long long& cycles) {
    int ok = 1;
    if (lane == 0) ok = timed_wait<DIAG, PARK_NS>(bar, parity, ctl, cycles) ? 1 : 0;
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
// scheduler with four epilogue warps, so it parks between probes instead of spinning.
constexpr uint32_t kIssuerParkNs = 200;

template <bool DIAG>
__device__ __noinline__ bool warp_tile_wait_slow(uint32_t bar_address, uint32_t parity, const WaitCtl ctl, long long* cycles) {
    uint64_t* bar = reinterpret_cast<uint64_t*>(__cvta_shared_to_generic(bar_address));
    const long long begin = DIAG ? clock64() : 0;
    uint64_t deadline = 0;
    bool ok = true;
    for (uint32_t spin = 1;; ++spin) {
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity, kTileParkNs))) break;
        if ((spin & 63u) == 0u) {
            const uint64_t now = global_timer_ns();
            if (deadline == 0) deadline = now + ctl.limit_ns;
            if (__any_sync(0xffffffffu, *ctl.abort_flag != 0 || now > deadline)) {
                *ctl.abort_flag = 1;
                ok = false;
                break;
            }
        }
    }
    if (DIAG) *cycles += clock64() - begin;
    return ok;
}

// The common case in one probe and one vote: the tile is there already.
template <bool DIAG>
__device__ __forceinline__ bool warp_tile_wait(uint32_t bar_address, uint32_t parity, const WaitCtl& ctl, long long& cycles) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "vote.sync.all.pred p, p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar_address), "r"(parity)
        : "memory");
    if (done != 0u) return true;
    return warp_tile_wait_slow<DIAG>(bar_address, parity, ctl, &cycles);
}

template <int MODE, bool DIAG, bool PAGED = false>
__global__ void __launch_bounds__(kThreads, 1) itk_fused_kernel(const __grid_constant__ FusedParams p) {
    // The operand tiles (128-byte swizzle) and the histogram blocks need a 1 KB-aligned base; the
    // kernel has no static shared memory in front of the dynamic block, and checks the address below.
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* smem_q = smem;
    uint8_t* smem_kv = smem + kQBytes;
    FusedShared& sh = *reinterpret_cast<FusedShared*>(smem + kSmemTileBytes);
    const WaitCtl ctl{&sh.abort, p.wait_limit_ns};

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;

    if ((smem_u32(smem) & 1023u) != 0u) {   // the same in every thread
        if (threadIdx.x == 0) atomicOr(p.status, kStatusBadSharedBase);
        return;
    }
    if (MODE == kModeRepair) {
        // The usual case is that the fast path flagged no row: find that out with one parallel scan
        // of the flags before any barrier, TMEM or descriptor is set up.
        int any = 0;
        const int flags = p.rows;
        for (int i = static_cast<int>(threadIdx.x); i < flags; i += kThreads) any |= p.failure_flags[i];
        if (__syncthreads_or(any) == 0) return;
    } else if (p.exit_when_no_keys) {
        // The compacted retry problem usually has no row at all (every slot has an empty key range).
        int any = 0;
        for (int i = static_cast<int>(threadIdx.x); i < p.rows; i += kThreads) any |= p.k_end[i] > p.k_start[i] ? 1 : 0;
        if (__syncthreads_or(any) == 0) return;
    }

    for (int i = static_cast<int>(threadIdx.x); i < kBlockQ * kScoreBins; i += kThreads) {
        (&sh.row_hist[0][0])[i] = 0u;
        sh.select[i >> 8].hist[i & 255] = 0;
    }
    if (threadIdx.x < kBlockQ * kSegments) (&sh.spill_counts[0][0])[threadIdx.x] = 0;
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
        if (MODE == kModeTopK && p.sample_tiles > 0) prefetch_tensormap(&p.map_sample);
    }
    if (warp == 1) {
        tmem_alloc(&sh.tmem_base, kTmemColumns);
        tmem_relinquish_alloc_permit();
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = sh.tmem_base;

    if (warp == 0) {
        // ============================================================ TMA producer
        if (lane == 0) {
            int kv_iter = 0, q_iter = 0;
            bool ok = true;
            long long wait_kv = 0, wait_q = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            const bool withhold = DIAG && p.withhold_q_loads != 0;
            for (int iter = 0; ok && !withhold; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                if (u.tile_end == u.tile_begin) continue;
                ok = timed_wait<DIAG>(&sh.q_empty, (q_iter & 1) ^ 1, ctl, wait_q);
                if (!ok) break;
                mbar_arrive_expect_tx(&sh.q_full, kQBytes);
                tma_load_2d(smem_q, &p.map_q, &sh.q_full, 0, u.block * kUmmaN);
                const int ws = q_iter & 1;
                ok = timed_wait<DIAG>(&sh.w_empty[ws], ((q_iter >> 1) & 1) ^ 1, ctl, wait_q);
                if (!ok) break;
                const uint32_t w_bytes = static_cast<uint32_t>(u.nrows) * kHeads * sizeof(float);
                mbar_arrive_expect_tx(&sh.w_full[ws], w_bytes);
                bulk_load(sh.weights[ws], p.weights + static_cast<long long>(u.row0) * kHeads, w_bytes,
                          &sh.w_full[ws]);
                // the gathered sample keys first (when the unit takes its thresholds from them), then its own
                for (int t = u.tile_begin - u.sample_tiles; t < u.tile_end; ++t, ++kv_iter) {
                    const int stage = kv_iter % kKvStages;
                    ok = timed_wait<DIAG>(&sh.tile_done[stage], ((kv_iter / kKvStages) & 1) ^ 1, ctl, wait_kv);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sh.kv_full[stage], kKvBytes);
                    if (t < u.tile_begin) {
                        tma_load_2d(smem_kv + stage * kKvBytes, &p.map_sample, &sh.kv_full[stage], 0,
                                    (t - u.tile_begin + u.sample_tiles) * kTileKeys);
                    } else {
                        tma_load_2d(smem_kv + stage * kKvBytes, &p.map_kv, &sh.kv_full[stage], 0,
                                    (PAGED ? __ldg(p.tile_table + t) : t) * kTileKeys);
                    }
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
            const uint64_t desc_kv0 = umma_desc_sw128_kmajor(smem_u32(smem_kv));
            int kv_iter = 0, q_iter = 0;
            bool ok = true;
            long long wait_acc = 0, wait_kv = 0, wait_q = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                if (u.tile_end == u.tile_begin) continue;
                ok = timed_wait<DIAG>(&sh.q_full, q_iter & 1, ctl, wait_q);
                if (!ok) break;
                // Issuing a tile's four UMMAs occupies this thread for about as long as the tensor pipe
                // needs for them, so the barriers of tile t+1 are probed while the UMMAs of tile t
                // execute; the blocking waits at the top are normally satisfied already.
                bool acc_ready = false, kv_ready = false;
                for (int t = u.tile_begin - u.sample_tiles; t < u.tile_end; ++t, ++kv_iter) {
                    const int buffer = kv_iter & 1;
                    const int stage = kv_iter % kKvStages;
                    if (!acc_ready) {
                        ok = timed_wait<DIAG, kIssuerParkNs>(&sh.acc_empty[buffer], ((kv_iter >> 1) & 1) ^ 1, ctl, wait_acc);
                        if (!ok) break;
                    }
                    if (!kv_ready) {
                        ok = timed_wait<DIAG, kHotWait>(&sh.kv_full[stage], (kv_iter / kKvStages) & 1, ctl, wait_kv);
                        if (!ok) break;
                    }
                    tcgen05_fence_after_sync();
                    // key tile of the stage: 16 KB = 1024 descriptor address units apart; both operands
                    // advance by 32 bytes (= 2 units) per K step
                    const uint64_t desc_kv = desc_kv0 + static_cast<uint64_t>(stage * (kKvBytes >> 4));
                    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buffer * kUmmaN);
                    const int next = kv_iter + 1;
                    const bool more = t + 1 < u.tile_end;
                    umma_f8(tmem_d, desc_kv, desc_q, idesc, 0u);
                    acc_ready = more && mbar_test_wait(&sh.acc_empty[next & 1], ((next >> 1) & 1) ^ 1);
                    umma_f8(tmem_d, desc_kv + 2, desc_q + 2, idesc, 1u);
                    kv_ready = more && mbar_test_wait(&sh.kv_full[next % kKvStages], (next / kKvStages) & 1);
                    umma_f8(tmem_d, desc_kv + 4, desc_q + 4, idesc, 1u);
                    if (more && !acc_ready) acc_ready = mbar_test_wait(&sh.acc_empty[next & 1], ((next >> 1) & 1) ^ 1);
                    umma_f8(tmem_d, desc_kv + 6, desc_q + 6, idesc, 1u);
                    // a single commit per tile frees the key stage and publishes the accumulator
                    umma_commit(&sh.tile_done[stage]);
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
    } else if (warp >= kEpilogueWarp0) {
        // ============================================================ epilogue
        // Sixteen warps share every tile: warp (quarter, row) reads the 32 TMEM lanes (= keys) of
        // its lane quarter, which is also its candidate segment, and the 64 accumulator columns
        // (= heads) of one query row.  Accumulators come out of TMEM in the 16x256b fragment
        // layout, 16 lanes at a time: thread t of a warp holds, for lanes l = t/4 and l+8 of a
        // 16-lane half, the column pairs 8n + 2(t%4) + {0,1}, n = 0..7.  So a thread needs only 16
        // of the row's 64 head weights, kept in registers for the whole unit: no shared-memory
        // traffic in the hot loop.  The four threads of a quad combine their partial head sums
        // with two shuffles, after which every thread owns the score of exactly one key of the
        // tile.  Four warps per scheduler hide one another's TMEM and arithmetic latencies.
        const int ew = warp - kEpilogueWarp0;
        const int quarter = warp & 3;           // the TMEM lane quarter this warp may read
        const int own_r = ew >> 2;              // query row of the unit this warp finishes
        const int quad = lane & 3;              // column-pair selector inside the fragment
        int own_key = quarter * 32 + (lane >> 2) + 8 * quad;   // key of a tile (= TMEM lane) this thread finishes
        uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(own_r * kHeads);
        keep_in_register(own_key);
        keep_in_register(tmem_lane);
        // this thread's candidate list: entries j * 32 + lane of the (row, quarter) segment
        uint32_t score_list = smem_u32(&sh.cand_scores[own_r][quarter * kSegCap + lane]);
        uint32_t id_list = smem_u32(&sh.cand_ids[own_r][quarter * kSegCap + lane]);
        keep_in_register(score_list);
        keep_in_register(id_list);
        const uint32_t tile_done_bars = smem_u32(&sh.tile_done[0]);
        const uint32_t acc_empty_bars = smem_u32(&sh.acc_empty[0]);
        int unit_iter = 0;  // units with tiles
        int acc_iter = 0;   // tiles
        bool ok = true;
        long long wait_acc = 0, wait_w = 0, select_cycles = 0;

        const long long role_begin = DIAG ? clock64() : 0;
        if (DIAG && p.trace != nullptr && ew == 0 && lane == 0)
            p.trace[static_cast<long long>(blockIdx.x) * kTraceFields + kTraceNsBegin] = global_timer_ns();
        // What the row's four warps do when the unit's candidates are complete (or the unit has no tile
        // at all): exact Top-K of the row, or its sampled threshold.  All four warps of a row call it.
        long long laps[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        RowBarrier rb{&sh.row_bar[own_r], 0u, ctl, DIAG ? laps : nullptr, 0};
        const auto finish_row = [&](const Unit& u, bool has_tiles, int lane_entries) {
            const long long begin = DIAG ? clock64() : 0;
            bool solo = false;
            if (own_r < u.nrows) {
                if (MODE == kModeTopK) {
                    select_topk_row(sh, p, u, own_r, has_tiles, rb, quarter * 32 + lane, lane_entries);
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
                finish_row(u, false, 0);
                continue;
            }
            const int slot = unit_iter & 1;   // weight buffer of the unit
            const uint32_t use_parity = (unit_iter >> 1) & 1;
            ok = warp_wait<DIAG>(&sh.w_full[slot], use_parity, ctl, lane, wait_w);
            if (!ok) break;

            // Filter state of the row, arranged so that the tile loop needs no branch: a key passes when
            // it lies in [row_lo, row_lo + row_span) and its score reaches the threshold (-inf for rows
            // that keep every key); a row that is switched off has an empty range.
            const RowState row = load_row_state<MODE>(p, u.row0, u.nrows, u.split, u.key_lo, u.key_hi, own_r);
            int row_lo = row.lo;
            unsigned row_span = row.on && row.hi > row.lo ? static_cast<unsigned>(row.hi - row.lo) : 0u;
            float threshold = row.threshold;
            // the compiler would otherwise re-derive these per tile from thread and unit indices
            keep_in_register(row_lo);
            keep_in_register(row_span);
            keep_in_register(threshold);

            // head weights of this thread's column pairs, times 2^25 (the ReLU is a saturating multiply
            // by 2^-25)
            uint64_t w[8];
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float2 pair = *reinterpret_cast<const float2*>(&sh.weights[slot][own_r * kHeads + 8 * n + 2 * quad]);
                const float lo = pair.x * kSatUnscale, hi = pair.y * kSatUnscale;
                asm("mov.b64 %0, {%1, %2};" : "=l"(w[n]) : "f"(lo), "f"(hi));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.w_empty[slot]);   // weights are in registers now

            // scale and range key of the key this thread finishes in tile t
            const auto per_key = [&](int t, float& scale, int& range_key) {
                const int key = t * kTileKeys + own_key;
                const bool key_ok = key < p.keys;
                // a paged key keeps its logical position (ids, ranges); only its storage moves
                const int stored = PAGED ? __ldg(p.tile_table + t) * kTileKeys + own_key : key;
                scale = key_ok ? __ldg(p.kv_scales + stored) : 0.0f;
                if (MODE == kModeSample) range_key = key_ok ? __ldg(p.sample_ids + key) : 0x7fffffff;
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

            // Top-K mode: the thread's own candidate list (next free entry, end of the list)
            uint32_t score_at = score_list, id_at = id_list;
            const uint32_t limit_at = score_list + static_cast<uint32_t>(kSegCap / 32) * 128u;
            int count = 0;   // sample mode: candidates of the warp's segment (dense, warp-uniform)

            // What happens to the 32 scores of this warp in one tile.
            const auto finish = [&](int t, float sum, float scale, int sample_key) {
                // the fused add of +0 turns a -0 product into +0 and changes no other value
                const float score = __fmaf_rn(sum, scale, 0.0f);
                const int key = t * kTileKeys + own_key;
                const int range_key = MODE == kModeSample ? sample_key : key;   // the sampled key's position in the context
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
                const uint32_t bits = __float_as_uint(score);
                const uint32_t score_bits = bits ^ (static_cast<uint32_t>(static_cast<int32_t>(bits) >> 31) | 0x80000000u);
                // id = (tile << 5) | (key & 31); the segment number carries the lane quarter
                const uint32_t id16 = static_cast<uint32_t>(t * 32 + (own_key & 31));
                if (MODE == kModeTopK) {
                    if (filter_store(score, bits, key, row_lo, row_span, threshold, id16, score_at, id_at, limit_at)) {
                        // rare: this thread's list is full, the candidate goes to the segment's global spill
                        const int at = atomicAdd(&sh.spill_counts[own_r][quarter], 1);
                        if (at < kSpillSegCap)
                            p.spill[spill_slot(own_r) * kSpillRow + quarter * kSpillSegCap + at] =
                                (static_cast<uint64_t>(score_bits) << 32) | static_cast<uint32_t>(key);
                    }
                } else {
                    // sample mode: dense segment, filled in warp-vote order
                    const bool active = static_cast<unsigned>(range_key - row_lo) < row_span &&
                                        fabsf(score) <= 3.4028234663852886e38f;   // finite
                    const unsigned ballot = __ballot_sync(0xffffffffu, active);
                    const int position = count + __popc(ballot & lanemask_lt());
                    count += __popc(ballot);
                    if (active && position < kSegCap) {
                        sh.cand_scores[own_r][quarter * kSegCap + position] = score_bits;
                        sh.cand_ids[own_r][quarter * kSegCap + position] = static_cast<uint16_t>(id16);
                    }
                }
            };

            // Two fragment loads per tile, one per 16-lane half of the quarter, through one 32-register
            // buffer; the other three epilogue warps of the scheduler cover the TMEM latency.  The
            // accumulator buffer goes back to the UMMA issuer as soon as the second fragment has landed.
            uint32_t frag[32];
            if (MODE == kModeTopK && u.sample_tiles > 0) {
                // The unit's first tiles are the gathered sample keys: score them like any tile, keep the
                // scores of samples inside the row's key range as a dense segment, and let the row's warps
                // pick the threshold from them (the arithmetic and the choice of the sample kernel).
                const int start = own_r < u.nrows ? __ldg(p.k_start + u.row0 + own_r) : 0;
                const int end = own_r < u.nrows ? __ldg(p.k_end + u.row0 + own_r) : 0;
                const unsigned sample_span = end - start > p.target_candidates ? static_cast<unsigned>(end - start) : 0u;
                int sampled = 0;
                for (int st = 0; st < u.sample_tiles; ++st, ++acc_iter) {
                    const int sample = st * kTileKeys + own_key;
                    const bool sample_ok = sample < p.sample_count;
                    const float sample_scale = sample_ok ? __ldg(p.sample_scales + sample) : 0.0f;
                    const int position = sample_ok ? __ldg(p.sample_ids + sample) : 0x7fffffff;
                    ok = warp_tile_wait<DIAG>(tile_done_bars + 8u * static_cast<uint32_t>(acc_iter % kKvStages),
                                              (acc_iter / kKvStages) & 1, ctl, wait_acc);
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                    const uint32_t taddr = tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN);
                    tmem_load_frag(taddr, frag);
                    uint64_t acc_a, acc_b;
                    tmem_load_wait(frag);
                    fragment_fma(frag, w, acc_a, acc_b);
                    tmem_load_frag(taddr + (16u << 16), frag);
                    const float sum0 = pair_sum(acc_a), sum1 = pair_sum(acc_b);
                    tmem_load_wait(frag);
                    tcgen05_fence_before_sync();
                    mbar_arrive_elected(acc_empty_bars + 8u * static_cast<uint32_t>(acc_iter & 1));
                    fragment_fma(frag, w, acc_a, acc_b);
                    const float score = __fmaf_rn(quad_reduce(sum0, sum1, pair_sum(acc_a), pair_sum(acc_b)), sample_scale, 0.0f);
                    const uint32_t bits = __float_as_uint(score);
                    const bool active = static_cast<unsigned>(position - start) < sample_span &&
                                        fabsf(score) <= 3.4028234663852886e38f;   // finite
                    const unsigned ballot = __ballot_sync(0xffffffffu, active);
                    const int slot_at = sampled + __popc(ballot & lanemask_lt());
                    sampled += __popc(ballot);
                    if (active && slot_at < kSegCap)
                        sh.cand_scores[own_r][quarter * kSegCap + slot_at] =
                            bits ^ (static_cast<uint32_t>(static_cast<int32_t>(bits) >> 31) | 0x80000000u);
                }
                if (!ok) break;
                if (lane == 0) sh.counts[own_r][quarter] = sampled;
                row_sync(rb);   // the four segments of the row are complete and counted
                bool solo = false;
                if (own_r < u.nrows) solo = sample_threshold_row(sh, p, u, own_r, true, rb, quarter * 32 + lane);
                if (solo && quarter != (own_r & 3)) row_sync_parked(rb);
                else row_sync(rb);   // the threshold is in shared memory, the segments may be written again
                if (row_span != 0u && row.hi - row.lo > kTopK) threshold = sh.unit_threshold[own_r];
                keep_in_register(threshold);
            }
            float scale, next_scale = 0.0f;
            int range_key = 0, next_range_key = 0;   // sample mode only
            per_key(u.tile_begin, scale, range_key);
            int t = u.tile_begin;
            if (MODE == kModeTopK && !DIAG && !PAGED) {
                // the product path of the Top-K mode runs the tile loop in its PTX form; this C++ loop
                // serves the diagnostic, paged, sample and repair instances (same arithmetic, same order)
                int key = t * kTileKeys + own_key;
                uint16_t id16 = static_cast<uint16_t>(t * 32 + (own_key & 31));
                for (;;) {
                    uint32_t full;
                    float last_score;
                    const uint32_t why = topk_tile_loop(t, acc_iter, key, id16, scale, score_at, id_at, full, last_score,
                                                        u.tile_end, limit_at, row_lo, row_span, threshold, p.kv_scales,
                                                        p.keys - 1, tile_done_bars, acc_empty_bars, tmem_lane, lane, w);
                    if (why == kLoopDone) break;
                    if (why == kLoopNeedWait) {
                        ok = warp_tile_wait_slow<DIAG>(tile_done_bars + 8u * static_cast<uint32_t>(acc_iter % kKvStages),
                                                       (acc_iter / kKvStages) & 1, ctl, &wait_acc);
                        if (!ok) break;
                    } else if (full != 0u) {
                        const int at = atomicAdd(&sh.spill_counts[own_r][quarter], 1);
                        if (at < kSpillSegCap)
                            p.spill[spill_slot(own_r) * kSpillRow + quarter * kSpillSegCap + at] =
                                pack_score_id(last_score, static_cast<uint32_t>(key - kTileKeys));
                    }
                }
                t = u.tile_end;
            }
            for (; t < u.tile_end; ++t, ++acc_iter) {
                ok = warp_tile_wait<DIAG>(tile_done_bars + 8u * static_cast<uint32_t>(acc_iter % kKvStages),
                                          (acc_iter / kKvStages) & 1, ctl, wait_acc);
                if (!ok) break;
                tcgen05_fence_after_sync();
                const uint32_t taddr = tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN);
                tmem_load_frag(taddr, frag);                          // lanes 0-15 of the quarter
                if (t + 1 < u.tile_end) per_key(t + 1, next_scale, next_range_key);
                uint64_t acc_a, acc_b;
                tmem_load_wait(frag);
                fragment_fma(frag, w, acc_a, acc_b);
                tmem_load_frag(taddr + (16u << 16), frag);            // lanes 16-31 of the quarter
                const float sum0 = pair_sum(acc_a), sum1 = pair_sum(acc_b);   // lanes l and l+8 of the quarter
                tmem_load_wait(frag);                                 // the accumulator buffer is fully read
                tcgen05_fence_before_sync();
                mbar_arrive_elected(acc_empty_bars + 8u * static_cast<uint32_t>(acc_iter & 1));
                fragment_fma(frag, w, acc_a, acc_b);
                finish(t, quad_reduce(sum0, sum1, pair_sum(acc_a), pair_sum(acc_b)), scale, range_key);
                scale = next_scale;
                range_key = next_range_key;
            }
            if (!ok) break;
            int lane_entries = 0;
            if (MODE == kModeTopK) lane_entries = static_cast<int>(score_at - score_list) >> 7;
            if (MODE == kModeSample) {
                if (lane == 0) sh.counts[own_r][quarter] = count;
                row_sync(rb);   // the four segments of the row are complete and counted
            }
            finish_row(u, true, lane_entries);
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
                cta_trace[27] = laps[1];   // histogram pass
                cta_trace[28] = laps[2];   // bin of the cutoff and its exact edges
                cta_trace[29] = laps[3];   // emission
                cta_trace[30] = laps[4];   // list ranking
                cta_trace[31] = laps[5];   // whole selection incl. fallback
                cta_trace[20] = laps[6];   // clean-up
                cta_trace[5] = laps[7];    // rows (of the unit's first row slot) that fell back to the radix selection
                cta_trace[6] = laps[0];    // why the last of them did
                cta_trace[kTraceNsEnd] = global_timer_ns();
            }
        }
        if (!ok && lane == 0) atomicOr(p.status, kStatusWaitExpired);
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        if (sh.abort != 0) {
            // a wait expired: UMMAs issued before that may still be in the tensor pipe (a tile takes
            // well under a microsecond); TMEM is not freed under them
            const uint64_t until = global_timer_ns() + 2000000ull;
            while (global_timer_ns() < until) {
            }
        }
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

}  // namespace itk
