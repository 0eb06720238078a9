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
// back with tcgen05.ld, one TMEM lane = one key per thread, and form
//
//     score[row, key] = (sum_h relu(acc) * w[row, h]) * kv_scale[key].
//
// The dense score matrix is never written.  What happens to a score depends on
// the kernel mode:
//   kModeTopK    keep (score, key) when the key is inside the row's range and
//                score >= threshold[row]; candidates go to per-row shared-memory
//                segments (overflow to a bounded global spill), and consumer
//                warps of the same CTA radix-select the exact Top-2048 of the
//                previous unit while the next unit's scores are produced;
//   kModeSample  the "keys" are S gathered sample keys; consumer warps pick the
//                rank-th largest valid sampled score of each row = its threshold;
//   kModeRepair  for rows flagged as failed, write every (score, key) of one
//                16 K-key chunk to global memory for the exact repair reducers.
//
// Warp roles (512 threads): warp 0 TMA producer, warp 1 UMMA issuer and TMEM
// owner, warps 4-11 epilogue (two warpgroups, one per TMEM accumulator buffer),
// warps 2, 3, 12-15 Top-K consumers.  All hand-offs are mbarriers with bounded
// waits; a wait that expires sets bit 0 of *status and the CTA drains.
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
//   6 = everything but the Top-K selection of the consumer warps.
#ifndef ITK_EXPERIMENT
#define ITK_EXPERIMENT 0
#endif

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
constexpr int kSegCap = 640;                   // shared-memory candidates per (row, segment)
constexpr int kRowCap = kSegments * kSegCap;   // 2560
constexpr int kSpillSegCap = 1408;             // global spill entries per (row, segment)
constexpr int kSpillRow = kSegments * kSpillSegCap;  // 5632 u64 per row
constexpr int kRepairChunk = 16384;

constexpr int kThreads = 512;
constexpr int kEpilogueWarp0 = 4;
constexpr int kEpilogueThreads = 256;
constexpr int kEpilogueWarps = kEpilogueThreads / 32;
constexpr int kEpilogueRegisters = 144;        // per-thread budget of the two epilogue warpgroups
constexpr int kOtherRegisters = 112;            // ... and of the producer / issuer / consumer warpgroups
static_assert(256 * kEpilogueRegisters + 256 * kOtherRegisters <= 65536, "register pool of one SM");
constexpr int kConsumerThreads = 192;
constexpr int kConsumerWarps = kConsumerThreads / 32;

constexpr uint32_t kQBytes = kUmmaN * kHeadDim;       // 32768
constexpr uint32_t kKvBytes = kTileKeys * kHeadDim;   // 16384

constexpr int kModeTopK = 0;
constexpr int kModeSample = 1;
constexpr int kModeRepair = 2;

constexpr int kStatusWaitExpired = 1;

// Per-CTA phase trace of diagnostic builds (clock64 cycles unless noted).
constexpr int kTraceFields = 32;
constexpr int kTraceMmaTotal = 0, kTraceMmaWaitAcc = 1, kTraceMmaWaitKv = 2, kTraceMmaWaitQ = 3, kTraceMmaTiles = 4;
constexpr int kTraceTmaTotal = 8, kTraceTmaWaitKv = 9, kTraceTmaWaitQ = 10;
constexpr int kTraceEpiTotal = 12, kTraceEpiWaitAcc = 13, kTraceEpiWaitFree = 14, kTraceEpiWaitW = 15;  // +4 for warpgroup 1
constexpr int kTraceConTotal = 20, kTraceConWaitReady = 21, kTraceConSelect = 22, kTraceConUnits = 23;
constexpr int kTraceSm = 24, kTraceNsBegin = 25, kTraceNsEnd = 26;

struct FusedParams {
    CUtensorMap map_q;    // [rows*64, 128] bytes, box 256 x 128, 128-byte swizzle
    CUtensorMap map_kv;   // [keys, 128] bytes, box 128 x 128, 128-byte swizzle
    const float* kv_scales;     // [keys]
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
};

struct __align__(16) FusedShared {
    float weights[2][kBlockQ * kHeads];
    uint32_t cand_scores[2][kBlockQ][kRowCap];
    uint16_t cand_ids[2][kBlockQ][kRowCap];
    int counts[2][kBlockQ][kSegments];
    int hist[kConsumerWarps][256];   // one digit histogram per consumer warp
    int warp_greater[kConsumerWarps];
    int warp_equal[kConsumerWarps];
    uint32_t sel_ref;
    uint32_t sel_or;
    int sel_bin;
    int sel_greater;
    int sel_failed;
    int sel_total;
    int sel_gcount;
    int sel_ecount;
    uint32_t tmem_base;
    int abort;
    uint64_t kv_full[kKvStages];
    uint64_t tile_done[kKvStages];   // one arrival per finished tile: frees the key stage and publishes the accumulator
    uint64_t q_full;
    uint64_t q_empty;
    uint64_t w_full[2];
    uint64_t w_empty[2];
    uint64_t acc_empty[kAccBuffers];
    uint64_t cand_ready[2];
    uint64_t cand_free[2];
};

constexpr size_t kSmemTileBytes = kQBytes + kKvStages * kKvBytes;
constexpr size_t kFusedSmemBytes = 1024 + kSmemTileBytes + sizeof(FusedShared);
static_assert(kFusedSmemBytes <= 232448, "fused kernel exceeds the 227 KB shared-memory limit");
static_assert(kSegCap % 32 == 0 && kSpillSegCap % 32 == 0, "segment capacities are warp multiples");

// mbar_wait that adds the cycles it took to `cycles` in diagnostic builds.
template <bool DIAG, bool HOT = false>
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           long long& cycles) {
    if (DIAG) {
        const long long begin = clock64();
        const bool ok = mbar_wait<HOT>(bar, parity, abort_flag);
        cycles += clock64() - begin;
        return ok;
    }
    return mbar_wait<HOT>(bar, parity, abort_flag);
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
                needed = e > s && p.failure_flags[static_cast<long long>(u.shard) * p.rows + row] != 0;
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

// ------------------------------------------------------------------ consumer helpers

__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// Key index of shared-memory candidate `packed` stored in segment `segment`.
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
    const int leader = __ffs(static_cast<int>(mask)) - 1;
    int base = 0;
    if (lane == leader) base = atomicAdd(counter, __popc(mask));
    base = __shfl_sync(0xffffffffu, base, leader);
    return active ? base + __popc(mask & ((1u << lane) - 1u)) : -1;
}

// The view the consumer has of one row's candidates: counted shared-memory
// segments plus the row's spill region in global memory.
struct RowCandidates {
    const uint32_t* scores;   // [kRowCap]
    const uint16_t* ids;      // [kRowCap]
    const int* counts;        // [kSegments], may exceed the capacities
    const uint64_t* spill;    // [kSegments][kSpillSegCap], null when the mode has no spill
};

// Every consumer thread keeps "its" candidates of the row in registers for the whole
// selection, so the radix rounds touch neither shared nor global memory for them:
//   * shared-memory candidate i of a segment belongs to thread i % 192, slot i / 192
//     (at most kSegCap / 192 rounded up = 4 slots per segment, 16 in all);
//   * spill entry e (the segments' spill regions concatenated) belongs to thread e % 192,
//     slot e / 192, for the first 192 * kSpillRegs entries; later ones stay in global memory
//     and are re-read in every pass (only when a threshold is far too low).
constexpr int kSmemSlots = (kSegCap + kConsumerThreads - 1) / kConsumerThreads;   // 4
constexpr int kOwnSmem = kSegments * kSmemSlots;                                   // 16
constexpr int kSpillRegs = 8;
constexpr int kSpillCached = kSpillRegs * kConsumerThreads;

struct OwnCandidates {
    uint32_t smem_score[kOwnSmem];
    uint32_t spill_score[kSpillRegs];
    uint32_t spill_key[kSpillRegs];
    uint32_t smem_live;               // bit j: smem_score[j] holds a candidate
    uint32_t spill_live;              // bit k: spill_score[k] holds a candidate
    int spill_first[kSegments + 1];   // prefix sums of the per-segment spill counts
};

__device__ __forceinline__ uint64_t spill_entry(const RowCandidates& c, const OwnCandidates& own, int e) {
    int segment = 0;
    int begin = 0;
#pragma unroll
    for (int i = 1; i < kSegments; ++i) {
        if (e >= own.spill_first[i]) {
            segment = i;
            begin = own.spill_first[i];
        }
    }
    return c.spill[segment * kSpillSegCap + (e - begin)];
}

__device__ __forceinline__ void load_own(const RowCandidates& c, OwnCandidates& own, int ctid) {
    own.smem_live = 0u;
    own.spill_live = 0u;
    own.spill_first[0] = 0;
#pragma unroll
    for (int s = 0; s < kSegments; ++s) {
        const int count = c.counts[s];
        const int in_smem = min(count, kSegCap);
        const int spilled = c.spill == nullptr ? 0 : min(max(count - kSegCap, 0), kSpillSegCap);
        own.spill_first[s + 1] = own.spill_first[s] + spilled;
#pragma unroll
        for (int k = 0; k < kSmemSlots; ++k) {
            const int i = ctid + k * kConsumerThreads;
            const bool live = i < in_smem;
            own.smem_score[s * kSmemSlots + k] = live ? c.scores[s * kSegCap + i] : 0u;
            own.smem_live |= live ? 1u << (s * kSmemSlots + k) : 0u;
        }
    }
    const int total = own.spill_first[kSegments];
#pragma unroll
    for (int k = 0; k < kSpillRegs; ++k) {
        const int e = ctid + k * kConsumerThreads;
        uint64_t pair = 0ull;
        if (e < total) {
            pair = spill_entry(c, own, e);
            own.spill_live |= 1u << k;
        }
        own.spill_score[k] = static_cast<uint32_t>(pair >> 32);
        own.spill_key[k] = static_cast<uint32_t>(pair);
    }
}

// visit(score) for every candidate this thread owns in registers.
template <typename Visit>
__device__ __forceinline__ void for_own_scores(const OwnCandidates& own, Visit&& visit) {
#pragma unroll
    for (int j = 0; j < kOwnSmem; ++j)
        if (own.smem_live >> j & 1u) visit(own.smem_score[j]);
#pragma unroll
    for (int k = 0; k < kSpillRegs; ++k)
        if (own.spill_live >> k & 1u) visit(own.spill_score[k]);
}

// visit(pair) for the spill entries beyond the register cache, split over the threads.
template <typename Visit>
__device__ __forceinline__ void for_excess_spill(const RowCandidates& c, const OwnCandidates& own, int ctid,
                                                 Visit&& visit) {
    const int total = own.spill_first[kSegments];
    for (int e = kSpillCached + ctid; e < total; e += kConsumerThreads) visit(spill_entry(c, own, e));
}

// Radix selection over the ordered score bits of one row, up to 8 bits per round.
// On return `cutoff` is the rank-th largest score and `equal_needed` the number of
// candidates equal to it that belong to the top `rank_in`.  Needs rank_in <= number of
// candidates.  Called by all consumer threads.  The leading bits that all candidates
// share are found first and skipped; every warp counts into its own histogram, so
// the only contention on the shared-memory atomics is inside a warp.
__device__ __forceinline__ void radix_select(FusedShared& sh, const RowCandidates& c, const OwnCandidates& own,
                                             int ctid, int rank_in, uint32_t& cutoff, int& equal_needed) {
    const int lane = ctid & 31;
    const int cwarp = ctid >> 5;
    int* my_hist = sh.hist[cwarp];
    if (ctid == 0) {
        int s = 0;
        while (s < kSegments - 1 && c.counts[s] == 0) ++s;
        sh.sel_ref = c.scores[s * kSegCap];   // any candidate of the row
        sh.sel_or = 0u;
    }
    consumer_sync();
    const uint32_t reference = sh.sel_ref;
    uint32_t differing = 0u;
    for_own_scores(own, [&](uint32_t score) { differing |= score ^ reference; });
    for_excess_spill(c, own, ctid, [&](uint64_t pair) { differing |= static_cast<uint32_t>(pair >> 32) ^ reference; });
    differing = __reduce_or_sync(0xffffffffu, differing);
    if (lane == 0 && differing != 0u) atomicOr(&sh.sel_or, differing);
    consumer_sync();
    differing = sh.sel_or;

    int bits = differing == 0u ? 0 : 32 - __clz(differing);   // low bits in which candidates may differ
    uint32_t mask = bits == 32 ? 0u : 0xffffffffu << bits;
    uint32_t prefix = reference & mask;
    int rank = rank_in;
#pragma unroll 1
    while (bits > 0) {
        const int width = min(8, bits);
        const int shift = bits - width;
        const uint32_t digit_mask = (1u << width) - 1u;
        for (int bin = lane; bin < 256; bin += 32) my_hist[bin] = 0;
        __syncwarp();
        for_own_scores(own, [&](uint32_t score) {
            if ((score & mask) == prefix) atomicAdd(&my_hist[(score >> shift) & digit_mask], 1);
        });
        for_excess_spill(c, own, ctid, [&](uint64_t pair) {
            const uint32_t score = static_cast<uint32_t>(pair >> 32);
            if ((score & mask) == prefix) atomicAdd(&my_hist[(score >> shift) & digit_mask], 1);
        });
        consumer_sync();
        if (ctid < 32) {
            // lane l owns bins 8l .. 8l+7 (summed over the warps' histograms); `above` =
            // candidates in bins owned by higher lanes
            int bins[8];
            int mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) sum += sh.hist[w][ctid * 8 + j];
                bins[j] = sum;
                mine += sum;
            }
            int suffix = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const int other = __shfl_down_sync(0xffffffffu, suffix, offset);
                if (ctid + offset < 32) suffix += other;
            }
            int above = suffix - mine;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                const int through = above + bins[j];
                if (above < rank && rank <= through) {
                    sh.sel_bin = ctid * 8 + j;
                    sh.sel_greater = above;
                }
                above = through;
            }
        }
        consumer_sync();
        prefix |= static_cast<uint32_t>(sh.sel_bin) << shift;
        rank -= sh.sel_greater;
        mask |= digit_mask << shift;
        bits = shift;
    }
    cutoff = prefix;
    equal_needed = rank;
}

// Writes the selected candidates of one row: everything above `cutoff`, then
// `equal_needed` of the candidates equal to it (any of them); with take_all every
// candidate.  Two passes without atomics: per-warp totals first, then each warp writes
// behind the totals of the warps before it, lanes ordered by ballot.
__device__ __forceinline__ void emit_row(FusedShared& sh, const RowCandidates& c, const OwnCandidates& own, int ctid,
                                         uint32_t cutoff, int equal_needed, int greater_total, bool take_all,
                                         int32_t* out_ids, uint64_t* out_pairs) {
    const int lane = ctid & 31;
    const int cwarp = ctid >> 5;
    const int total_spill = own.spill_first[kSegments];
    int greater = 0, equal = 0;
    const auto tally = [&](uint32_t score) {
        greater += (take_all || score > cutoff) ? 1 : 0;
        equal += (!take_all && score == cutoff) ? 1 : 0;
    };
    for_own_scores(own, tally);
    for_excess_spill(c, own, ctid, [&](uint64_t pair) { tally(static_cast<uint32_t>(pair >> 32)); });
    greater = __reduce_add_sync(0xffffffffu, greater);
    equal = __reduce_add_sync(0xffffffffu, equal);
    if (lane == 0) {
        sh.warp_greater[cwarp] = greater;
        sh.warp_equal[cwarp] = equal;
    }
    consumer_sync();
    int next_greater = 0, next_equal = 0;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
        next_greater += w < cwarp ? sh.warp_greater[w] : 0;
        next_equal += w < cwarp ? sh.warp_equal[w] : 0;
    }
    const unsigned below = (1u << lane) - 1u;
    const auto place = [&](bool live, uint32_t score) -> int {
        const bool is_greater = live && (take_all || score > cutoff);
        const bool is_equal = live && !take_all && score == cutoff;
        const unsigned ballot_g = __ballot_sync(0xffffffffu, is_greater);
        const unsigned ballot_e = __ballot_sync(0xffffffffu, is_equal);
        int position = -1;
        if (is_greater) {
            position = next_greater + __popc(ballot_g & below);
        } else if (is_equal) {
            const int e = next_equal + __popc(ballot_e & below);
            if (e < equal_needed) position = greater_total + e;
        }
        next_greater += __popc(ballot_g);
        next_equal += __popc(ballot_e);
        return position < kTopK ? position : -1;
    };
    const auto write = [&](int position, uint32_t score, int key) {
        if (out_ids != nullptr) out_ids[position] = key;
        if (out_pairs != nullptr) out_pairs[position] = (static_cast<uint64_t>(score) << 32) | static_cast<uint32_t>(key);
    };
#pragma unroll
    for (int j = 0; j < kOwnSmem; ++j) {
        const int s = j / kSmemSlots;
        const int i = ctid + (j % kSmemSlots) * kConsumerThreads;
        const int position = place((own.smem_live >> j & 1u) != 0u, own.smem_score[j]);
        if (position >= 0) write(position, own.smem_score[j], decode_key(c.ids[s * kSegCap + i], s));
    }
#pragma unroll
    for (int k = 0; k < kSpillRegs; ++k) {
        if (k * kConsumerThreads < total_spill) {
            const int position = place((own.spill_live >> k & 1u) != 0u, own.spill_score[k]);
            if (position >= 0) write(position, own.spill_score[k], static_cast<int>(own.spill_key[k]));
        }
    }
    for (int base = kSpillCached + cwarp * 32; base < total_spill; base += kConsumerThreads) {
        const int e = base + lane;
        const bool live = e < total_spill;
        const uint64_t pair = live ? spill_entry(c, own, e) : 0ull;
        const int position = place(live, static_cast<uint32_t>(pair >> 32));
        if (position >= 0) write(position, static_cast<uint32_t>(pair >> 32), static_cast<int>(static_cast<uint32_t>(pair)));
    }
}

// Exact Top-2048 of one row from its candidates (kModeTopK consumer).
__device__ __forceinline__ void consume_topk_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                 int slot, bool has_tiles, int ctid, long long* phase = nullptr) {
    const int row = u.row0 + r;
    const long long row_slot = static_cast<long long>(u.shard) * p.rows + row;
    const int start = max(__ldg(p.k_start + row), u.key_lo);
    const int end = min(min(__ldg(p.k_end + row), p.keys), u.key_hi);
    const int valid = max(end - start, 0);
    int32_t* out_ids = p.out_ids != nullptr ? p.out_ids + static_cast<long long>(row) * kTopK : nullptr;
    uint64_t* out_pairs = p.out_pairs != nullptr ? p.out_pairs + row_slot * kTopK : nullptr;

    if (out_pairs == nullptr && valid <= p.top_k_min_valid) {
        // every valid key is selected; no scores are needed
        for (int i = ctid; i < kTopK; i += kConsumerThreads) out_ids[i] = i < valid ? start + i : -1;
        if (ctid == 0) p.failure_flags[row_slot] = 0;
        return;
    }
    if (!has_tiles) {
        // pairs requested but the row has no key in this shard
        for (int i = ctid; i < kTopK; i += kConsumerThreads) {
            if (out_ids != nullptr) out_ids[i] = -1;
            out_pairs[i] = 0ull;
        }
        if (ctid == 0) {
            p.failure_flags[row_slot] = 0;
            if (p.out_counts != nullptr) p.out_counts[row_slot] = 0;
        }
        return;
    }

    RowCandidates c;
    c.scores = sh.cand_scores[slot][r];
    c.ids = sh.cand_ids[slot][r];
    c.counts = sh.counts[slot][r];
    c.spill = p.spill + row_slot * kSpillRow;

    if (ctid == 0) {
        int total = 0;
        int overflow = 0;
        for (int s = 0; s < kSegments; ++s) {
            total += c.counts[s];
            overflow |= c.counts[s] > kSegCap + kSpillSegCap;
        }
        const int wanted = min(valid, kTopK);
        sh.sel_total = total;
        sh.sel_failed = (overflow || total < wanted) ? 1 : 0;
        sh.sel_gcount = 0;
        sh.sel_ecount = 0;
    }
    consumer_sync();
    const int total = sh.sel_total;
    const bool failed = sh.sel_failed != 0;
    if (failed) {
        for (int i = ctid; i < kTopK; i += kConsumerThreads) {
            if (out_ids != nullptr) out_ids[i] = -1;
            if (out_pairs != nullptr) out_pairs[i] = 0ull;
        }
        if (ctid == 0) {
            p.failure_flags[row_slot] = 1;
            if (p.out_counts != nullptr) p.out_counts[row_slot] = 0;
        }
        consumer_sync();
        return;
    }
    OwnCandidates view;
    long long stamp = phase != nullptr ? clock64() : 0;
    load_own(c, view, ctid);
    if (phase != nullptr) {
        // the cached entries are only complete once their loads have returned
        uint32_t touch = 0;
#pragma unroll
        for (int k = 0; k < kSpillRegs; ++k) touch |= view.spill_score[k];
        if (touch == 0x80000001u) phase[3] += 1;
        const long long now = clock64();
        phase[0] += now - stamp;
        stamp = now;
    }
    if (total <= kTopK) {
        // only reachable when valid <= 2048 (threshold forced to -inf): take everything
        emit_row(sh, c, view, ctid, 0u, 0, 0, true, out_ids, out_pairs);
        for (int i = total + ctid; i < kTopK; i += kConsumerThreads) {
            if (out_ids != nullptr) out_ids[i] = -1;
            if (out_pairs != nullptr) out_pairs[i] = 0ull;
        }
    } else {
        uint32_t cutoff;
        int equal_needed;
        radix_select(sh, c, view, ctid, kTopK, cutoff, equal_needed);
        if (phase != nullptr) {
            const long long now = clock64();
            phase[1] += now - stamp;
            stamp = now;
        }
        emit_row(sh, c, view, ctid, cutoff, equal_needed, kTopK - equal_needed, false, out_ids, out_pairs);
    }
    if (ctid == 0) {
        p.failure_flags[row_slot] = 0;
        if (p.out_counts != nullptr) p.out_counts[row_slot] = min(total, kTopK);
    }
    consumer_sync();
    if (phase != nullptr) phase[2] += clock64() - stamp;
}

// Threshold of one row = rank-th largest valid sampled score (kModeSample consumer).
// One warp per row, no block-level synchronisation: the warp walks the row's candidates in
// shared memory once per score bit (most significant differing bit first), counts the
// candidates that agree with the prefix found so far and have the bit set, and keeps or
// clears the bit so that exactly rank-1 candidates stay above the prefix.
__device__ __forceinline__ void sample_threshold_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                     int slot, bool has_tiles, int lane) {
    const int row = u.row0 + r;
    const int start = __ldg(p.k_start + row);
    const int end = __ldg(p.k_end + row);
    const float minus_inf = __int_as_float(0xff800000);
    float result = minus_inf;
    if (has_tiles && end - start > p.target_candidates) {
        const uint32_t* scores = sh.cand_scores[slot][r];
        const int* counts = sh.counts[slot][r];
        int total = 0;
        bool overflow = false;
        uint32_t reference = 0u;
#pragma unroll
        for (int s = kSegments - 1; s >= 0; --s) {
            total += counts[s];
            overflow = overflow || counts[s] > kSegCap;
            if (counts[s] > 0) reference = scores[s * kSegCap];
        }
        if (!overflow && total >= p.sample_rank) {
            // candidate g of the row (segments concatenated) belongs to lane g % 32; the first
            // kCached of a lane's candidates live in registers, the rest is re-read from shared
            // memory four at a time (a single warp is latency-bound, so loads must overlap)
            constexpr int kCached = 16;
            const int first1 = counts[0], first2 = first1 + counts[1], first3 = first2 + counts[2];
            const auto fetch = [&](int g) -> uint32_t {
                int segment = 0, begin = 0;
                if (g >= first1) { segment = 1; begin = first1; }
                if (g >= first2) { segment = 2; begin = first2; }
                if (g >= first3) { segment = 3; begin = first3; }
                return scores[segment * kSegCap + (g - begin)];
            };
            uint32_t own[kCached];
            uint32_t live = 0u;
#pragma unroll
            for (int m = 0; m < kCached; ++m) {
                const int g = lane + 32 * m;
                own[m] = g < total ? fetch(g) : 0u;
                live |= g < total ? 1u << m : 0u;
            }
            const auto for_rest = [&](auto&& visit) {
#pragma unroll 1
                for (int g = lane + 32 * kCached; g < total; g += 128) {
                    uint32_t x[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) x[k] = g + 32 * k < total ? fetch(g + 32 * k) : 0u;
#pragma unroll
                    for (int k = 0; k < 4; ++k) visit(g + 32 * k < total, x[k]);
                }
            };
            uint32_t differing = 0u;
#pragma unroll
            for (int m = 0; m < kCached; ++m) differing |= (live >> m & 1u) ? own[m] ^ reference : 0u;
            for_rest([&](bool valid, uint32_t score) { differing |= valid ? score ^ reference : 0u; });
            differing = __reduce_or_sync(0xffffffffu, differing);
            const int bits = differing == 0u ? 0 : 32 - __clz(differing);
            uint32_t mask = bits == 32 ? 0u : 0xffffffffu << bits;
            uint32_t prefix = reference & mask;
            int rank = p.sample_rank;
#pragma unroll 1
            for (int bit = bits - 1; bit >= 0; --bit) {
                const uint32_t probe = 1u << bit;
                const uint32_t want = prefix | probe;       // agrees with the prefix and has the bit set
                const uint32_t care = mask | probe;
                int above = 0;
#pragma unroll
                for (int m = 0; m < kCached; ++m)
                    above += static_cast<int>(live >> m & 1u) & static_cast<int>((own[m] & care) == want);
                for_rest([&](bool valid, uint32_t score) {
                    above += static_cast<int>(valid) & static_cast<int>((score & care) == want);
                });
                above = __reduce_add_sync(0xffffffffu, above);
                if (above >= rank) prefix |= probe;   // the rank-th largest has this bit set
                else rank -= above;                   // it lies among the candidates with the bit clear
                mask |= probe;
            }
            result = ordered_to_float(prefix);
        }
    }
    if (lane == 0) p.thresholds_out[row] = result;
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

// Lane 0 waits on the barrier, the warp then reconverges: one poller per warp.
template <bool DIAG, bool HOT = false>
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane,
                                          long long& cycles) {
    int ok = 1;
    if (lane == 0) ok = timed_wait<DIAG, HOT>(bar, parity, abort_flag, cycles) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

// The whole warp polls the barrier (one warp-wide probe per iteration, no parking, no
// lane-0 branch and broadcast): for the per-tile waits on the critical path.  Bounded like mbar_wait.
template <bool DIAG>
__device__ __forceinline__ bool warp_hot_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              long long& cycles) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long begin = DIAG ? clock64() : 0;
    uint64_t deadline = 0;
    bool ok = true;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_test_wait(bar, parity)) break;
        if ((spin & 4095u) == 0u) {
            const uint64_t now = global_timer_ns();
            if (deadline == 0) deadline = now + kWaitLimitNs;
            if (*abort_flag != 0 || now > deadline) {
                *abort_flag = 1;
                ok = false;
                break;
            }
        }
    }
    if (DIAG) cycles += clock64() - begin;
    return __all_sync(0xffffffffu, ok);
}

template <int MODE, bool DIAG>
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

    if (threadIdx.x == 0) {
        for (int i = 0; i < kKvStages; ++i) {
            mbar_init(&sh.kv_full[i], 1);
            mbar_init(&sh.tile_done[i], 1);
        }
        mbar_init(&sh.q_full, 1);
        mbar_init(&sh.q_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.w_full[i], 1);
            mbar_init(&sh.w_empty[i], kEpilogueWarps);
            mbar_init(&sh.acc_empty[i], kEpilogueWarps);
            mbar_init(&sh.cand_ready[i], kEpilogueWarps);
            mbar_init(&sh.cand_free[i], 1);
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

    const bool is_epilogue = warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + kEpilogueWarps;
    if (!is_epilogue) {
    // Register budget per warpgroup: producer / issuer / consumer warpgroups give registers back ...
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegisters));
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
                    tma_load_2d(smem_kv + stage * kKvBytes, &p.map_kv, &sh.kv_full[stage], 0, t * kTileKeys);
#endif
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
                // The tensor pipe accepts only a couple of UMMAs ahead of the one it executes, so
                // every cycle this thread spends between two batches of issues is a bubble.  The
                // barriers of tile t+1 are therefore probed while the UMMAs of tile t execute
                // (a probe takes less time than one UMMA); the blocking waits at the top are
                // normally satisfied already.
                bool acc_ready = false, kv_ready = false;
                for (int t = u.tile_begin; t < u.tile_end; ++t, ++kv_iter) {
                    const int buffer = kv_iter & 1;
                    const int stage = kv_iter % kKvStages;
                    if (!acc_ready) {
                        ok = timed_wait<DIAG, true>(&sh.acc_empty[buffer], ((kv_iter >> 1) & 1) ^ 1, abort_flag, wait_acc);
                        if (!ok) break;
                    }
                    if (!kv_ready) {
                        ok = timed_wait<DIAG, true>(&sh.kv_full[stage], (kv_iter / kKvStages) & 1, abort_flag, wait_kv);
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
    } else {
        // ============================================================ Top-K / threshold consumers
        if (MODE != kModeRepair) {
            const int cwarp = warp < kEpilogueWarp0 ? warp - 2 : warp - 12 + 2;   // warps 2,3,12..15 -> 0..5
            const int ctid = cwarp * 32 + lane;
            int unit_iter = 0;
            bool ok = true;
            long long wait_ready = 0, select_cycles = 0;
            long long phase[4] = {0, 0, 0, 0};
            const long long role_begin = DIAG ? clock64() : 0;
            if (DIAG && p.trace != nullptr && ctid == 0)
                p.trace[static_cast<long long>(blockIdx.x) * kTraceFields + kTraceNsBegin] = global_timer_ns();
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                const bool has_tiles = u.tile_end > u.tile_begin;
                const int slot = unit_iter & 1;
                if (has_tiles) {
                    // one thread polls; the others sleep in the named barrier until it is through
                    if (ctid == 0) {
                        const bool got = timed_wait<DIAG>(&sh.cand_ready[slot], (unit_iter >> 1) & 1, abort_flag, wait_ready);
                        sh.sel_failed = got ? 0 : -1;
                    }
                    consumer_sync();
                    ok = sh.sel_failed != -1;
                    consumer_sync();
                    if (!ok) break;
                }
                const long long select_begin = DIAG ? clock64() : 0;
                if (MODE == kModeTopK) {
                    for (int r = 0; r < u.nrows; ++r) {
                        if (DIAG && (p.debug_skip & 1)) continue;
#if ITK_EXPERIMENT == 6
                        continue;
#endif
                        consume_topk_row(sh, p, u, r, slot, has_tiles, ctid, DIAG ? phase : nullptr);
                    }
                } else if (cwarp < u.nrows) {
                    sample_threshold_row(sh, p, u, cwarp, slot, has_tiles, lane);   // one warp per row
                }
                if (DIAG) select_cycles += clock64() - select_begin;
                if (has_tiles) {
                    consumer_sync();
                    if (ctid == 0) mbar_arrive(&sh.cand_free[slot]);
                    ++unit_iter;
                }
            }
            if (DIAG && p.trace != nullptr && ctid == 0) {
                long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields;
                trace[kTraceConTotal] = clock64() - role_begin;
                trace[kTraceConWaitReady] = wait_ready;
                trace[kTraceConSelect] = select_cycles;
                trace[kTraceConUnits] = unit_iter;
                trace[27] = phase[0];   // spill caching
                trace[28] = phase[1];   // radix rounds
                trace[29] = phase[2];   // emit
                trace[kTraceNsEnd] = global_timer_ns();
            }
            if (!ok && lane == 0) atomicOr(p.status, kStatusWaitExpired);
        }
    }
    } else {
        // ... and the two epilogue warpgroups (warps 4-11) take most of the register file.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpilogueRegisters));
        // ============================================================ epilogue
        // Every tile is shared by both warpgroups: warpgroup g owns query rows 2g and 2g+1
        // (accumulator columns [128g, 128g+128)); a warp reads the 32 TMEM lanes (= keys) of
        // its quarter, which is also its candidate segment.  Accumulators come out of TMEM in
        // the 16x256b fragment layout: thread t of a warp holds, for lanes l = t/4 and l+8 of
        // a 16-lane half, the column pairs 8n + 2(t%4) + {0,1}, n = 0..7, of one query row.
        // So a thread only ever needs 16 of the 64 head weights of each of its two rows, kept
        // in registers for the whole unit: no shared-memory traffic in the hot loop.  The
        // four threads of a quad then combine their partial head sums with two shuffles.
        const int ew = warp - kEpilogueWarp0;
        const int wg = ew >> 2;
        const int quarter = ew & 3;             // = warp % 4, the TMEM lane quarter this warp may read
        const int quad = lane & 3;              // column-pair selector inside the fragment
        const int own_i = quad & 1;             // which of the warpgroup's two rows this thread finishes
        const int own_lane = (lane >> 2) + 8 * (quad >> 1);   // lane inside a 16-lane half it finishes
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(wg * 2 * kHeads);
        const float minus_inf = __int_as_float(0xff800000);
        int unit_iter = 0;  // units with tiles
        int acc_iter = 0;   // tiles
        bool ok = true;
        long long wait_acc = 0, wait_free = 0, wait_w = 0;
        const long long role_begin = DIAG ? clock64() : 0;
        for (int iter = 0; ok; ++iter) {
            Unit u;
            if (!load_unit<MODE>(p, iter, u)) break;
            if (u.tile_end == u.tile_begin) continue;
            const int slot = unit_iter & 1;
            const uint32_t use_parity = (unit_iter >> 1) & 1;
            if (MODE != kModeRepair) {
                ok = warp_wait<DIAG>(&sh.cand_free[slot], use_parity ^ 1, abort_flag, lane, wait_free);
                if (!ok) break;
            }
            ok = warp_wait<DIAG>(&sh.w_full[slot], use_parity, abort_flag, lane, wait_w);
            if (!ok) break;

            // the row this thread finishes: range, threshold, whether it is wanted at all
            const int own_r = wg * 2 + own_i;
            int row_lo = 0, row_hi = 0;
            float threshold = minus_inf;
            bool row_on = own_r < u.nrows;
            long long own_slot = 0;
            if (row_on) {
                const int row = u.row0 + own_r;
                own_slot = static_cast<long long>(u.shard) * p.rows + row;
                const int start = __ldg(p.k_start + row);
                const int end = __ldg(p.k_end + row);
                if (MODE == kModeSample) {
                    row_lo = start;
                    row_hi = end;
                    row_on = end - start > p.target_candidates;
                } else {
                    row_lo = max(start, u.key_lo);
                    row_hi = min(min(end, p.keys), u.key_hi);
                    if (MODE == kModeTopK) {
                        const int valid = row_hi - row_lo;
                        if (valid > kTopK) threshold = __ldg(p.thresholds + own_slot);
                        row_on = valid > (p.out_pairs != nullptr ? 0 : p.top_k_min_valid);
                    } else {
                        row_on = p.failure_flags[own_slot] != 0;
                    }
                }
            }
            // Candidate compaction: even lanes finish row 2g, odd lanes row 2g+1, so one ballot per
            // 16-lane half serves both rows and every thread keeps the running count of its own row.
            const unsigned row_mask = own_i == 0 ? 0x55555555u : 0xaaaaaaaau;
            const unsigned row_below = row_mask & ((1u << lane) - 1u);
            const uint32_t score_slots = smem_u32(&sh.cand_scores[slot][own_r][quarter * kSegCap]);
            const uint32_t id_slots = smem_u32(&sh.cand_ids[slot][own_r][quarter * kSegCap]);
            int own_count = 0;
            // tiles [interior_lo, interior_hi) lie inside the row's key range: there the threshold alone
            // decides (a NaN threshold rejects everything for rows that are switched off)
            const int interior_lo = (row_lo + kTileKeys - 1) / kTileKeys;
            const int interior_hi = row_hi / kTileKeys;
            const float pass_threshold = row_on ? threshold : __int_as_float(0x7fc00000);

            // head weights of this thread's column pairs, both rows
            uint64_t w0[8], w1[8];
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                w0[n] = *reinterpret_cast<const uint64_t*>(&sh.weights[slot][(wg * 2 + 0) * kHeads + 8 * n + 2 * quad]);
                w1[n] = *reinterpret_cast<const uint64_t*>(&sh.weights[slot][(wg * 2 + 1) * kHeads + 8 * n + 2 * quad]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.w_empty[slot]);   // weights are in registers now

            // scale and range key of the two keys this thread finishes in tile t (one per 16-lane half)
            const auto per_key = [&](int t, float (&scale)[2], int (&range_key)[2]) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int key = t * kTileKeys + quarter * 32 + h * 16 + own_lane;
                    const bool key_ok = key < p.keys;
                    scale[h] = key_ok ? __ldg(p.kv_scales + key) : 0.0f;
                    range_key[h] = key;
                    if (MODE == kModeSample) range_key[h] = key_ok ? __ldg(p.sample_ids + key) : 0x7fffffff;
                }
            };
            // partial head sums of one fragment load: lanes l and l+8, this thread's 16 heads.
            // ReLU is applied in place on the fragment registers, which are consecutive pairs
            // already, so the packed multiply-add can read them without any move.
            const auto relu_fma = [](uint32_t& x0, uint32_t& x1, uint64_t w, uint64_t& acc) {
                asm("{\n\t"
                    ".reg .b64 t;\n\t"
                    "max.f32 %0, %0, 0f00000000;\n\t"
                    "max.f32 %1, %1, 0f00000000;\n\t"
                    "mov.b64 t, {%0, %1};\n\t"
                    "fma.rn.f32x2 %2, t, %3, %2;\n\t"
                    "}"
                    : "+f"(*reinterpret_cast<float*>(&x0)), "+f"(*reinterpret_cast<float*>(&x1)), "+l"(acc)
                    : "l"(w));
            };
            const auto partial = [&](uint32_t (&r)[32], const uint64_t (&w)[8], float& lane_a, float& lane_b) {
                uint64_t a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
                for (int n = 0; n < 8; n += 2) {
                    relu_fma(r[4 * n + 0], r[4 * n + 1], w[n], a0);
                    relu_fma(r[4 * n + 2], r[4 * n + 3], w[n], b0);
                    relu_fma(r[4 * n + 4], r[4 * n + 5], w[n + 1], a1);
                    relu_fma(r[4 * n + 6], r[4 * n + 7], w[n + 1], b1);
                }
                float x0, x1, x2, x3;
                unpack_pair(a0, x0, x1);
                unpack_pair(a1, x2, x3);
                lane_a = (x0 + x1) + (x2 + x3);
                unpack_pair(b0, x0, x1);
                unpack_pair(b1, x2, x3);
                lane_b = (x0 + x1) + (x2 + x3);
            };
            // Quad reduce-scatter of (lane a,row 0), (lane a,row 1), (lane b,row 0), (lane b,row 1):
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
            // threshold filter and warp-level compaction of the 32 scores of one 16-lane half.
            // Even lanes finish row 2g, odd lanes row 2g+1, so one ballot serves both rows.
            const auto finish_half = [&](int h, int t, float head_sum, float scale, int range_key) {
                const float score = head_sum * scale;
                const int key = t * kTileKeys + quarter * 32 + h * 16 + own_lane;
                bool active;
                if (MODE == kModeTopK && !DIAG && t >= interior_lo && t < interior_hi) {
                    active = score >= pass_threshold;
                } else {
                    const bool key_ok = key < p.keys;
                    const bool in_range = key_ok && range_key >= row_lo && range_key < row_hi;
                    if (DIAG) {
                        if (own_r < u.nrows && key_ok && p.diag_logits != nullptr) {
                            const bool shown = MODE == kModeSample ? true : in_range;
                            p.diag_logits[static_cast<long long>(u.row0 + own_r) * p.diag_stride + key] =
                                shown ? score : minus_inf;
                        }
                    }
                    if (MODE == kModeRepair) {
                        if (row_on && key_ok && key >= u.key_lo && key < u.key_hi) {
                            p.repair_pairs[own_slot * kRepairChunk + (key - u.key_lo)] =
                                in_range ? pack_score_id(score, static_cast<uint32_t>(key)) : 0ull;
                        }
                        return;
                    }
                    active = row_on && in_range;
                    if (DIAG && (p.debug_skip & 2)) active = false;
                    if (MODE == kModeTopK) active = active && score >= threshold;
                    else active = active && (fabsf(score) <= 3.4028234663852886e38f);  // finite
                }
                const unsigned ballot = __ballot_sync(0xffffffffu, active);
                const int position = own_count + __popc(ballot & row_below);
                own_count += __popc(ballot & row_mask);
                if (active) {
                    if (position < kSegCap) {
                        st_shared_u32(score_slots + 4u * static_cast<uint32_t>(position), ordered_bits(score));
                        // id = (tile << 5) | (key & 31); the segment number carries the lane quarter
                        st_shared_u16(id_slots + 2u * static_cast<uint32_t>(position),
                                      static_cast<uint32_t>(t * 32 + h * 16 + own_lane));
                    } else if (MODE == kModeTopK && position < kSegCap + kSpillSegCap) {
                        p.spill[own_slot * kSpillRow + quarter * kSpillSegCap + (position - kSegCap)] =
                            pack_score_id(score, static_cast<uint32_t>(key));
                    }
                }
            };

            // Software pipeline over the four fragment loads of a tile, (half 0,row 0), (half 0,row 1),
            // (half 1,row 0), (half 1,row 1): while one fragment is reduced on the CUDA cores the
            // next is on its way out of TMEM (TMEM read bandwidth, about 350 cycles per tile, hides
            // under the arithmetic).  The accumulator buffer goes back to the UMMA issuer as soon
            // as the fourth fragment has landed; the first fragment of the next tile is requested
            // before the last filter step so that its latency is covered too.
            uint32_t fx[32], fy[32];
            float scale[2], next_scale[2] = {0.0f, 0.0f};
            int range_key[2], next_range_key[2] = {0, 0};
            per_key(u.tile_begin, scale, range_key);
            ok = warp_hot_wait<DIAG>(&sh.tile_done[acc_iter % kKvStages], (acc_iter / kKvStages) & 1, abort_flag, wait_acc);
            if (!ok) break;
            tcgen05_fence_after_sync();
            tmem_load_frag(tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN), fx);
            for (int t = u.tile_begin; t < u.tile_end; ++t, ++acc_iter) {
                const uint32_t taddr = tmem_lane + static_cast<uint32_t>((acc_iter & 1) * kUmmaN);
                const uint32_t upper_half = 16u << 16;
                const bool more = t + 1 < u.tile_end;
                if (more) per_key(t + 1, next_scale, next_range_key);
                float a_r0, b_r0, a_r1, b_r1, c_r0, d_r0, c_r1, d_r1;

                tmem_load_wait(fx);                                   // (half 0, row 0)
                tmem_load_frag(taddr + kHeads, fy);
#if ITK_EXPERIMENT != 1
                partial(fx, w0, a_r0, b_r0);
#else
                if (fx[3] == 0x7fc12345u) own_count += 1;
#endif
                tmem_load_wait(fy);                                   // (half 0, row 1)
                tmem_load_frag(taddr + upper_half, fx);
#if ITK_EXPERIMENT != 1
                partial(fy, w1, a_r1, b_r1);
#else
                if (fy[3] == 0x7fc12345u) own_count += 1;
#endif
                tmem_load_wait(fx);                                   // (half 1, row 0)
                tmem_load_frag(taddr + upper_half + kHeads, fy);
#if ITK_EXPERIMENT == 0 || ITK_EXPERIMENT == 6
                finish_half(0, t, quad_reduce(a_r0, a_r1, b_r0, b_r1), scale[0], range_key[0]);
#elif ITK_EXPERIMENT == 2
                if (a_r0 + a_r1 + b_r0 + b_r1 == 1.2345e38f) own_count += 1;
#endif
#if ITK_EXPERIMENT != 1
                partial(fx, w0, c_r0, d_r0);
#else
                if (fx[3] == 0x7fc12345u) own_count += 1;
#endif
                tmem_load_wait(fy);                                   // (half 1, row 1): buffer fully read
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.acc_empty[acc_iter & 1]);
#if ITK_EXPERIMENT != 1
                partial(fy, w1, c_r1, d_r1);
#else
                if (fx[0] == 0x7fc12345u && fy[1] == 7u) own_count += 1;
#endif
                if (more) {
                    const int next = acc_iter + 1;
                    ok = warp_hot_wait<DIAG>(&sh.tile_done[next % kKvStages], (next / kKvStages) & 1, abort_flag, wait_acc);
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                    tmem_load_frag(tmem_lane + static_cast<uint32_t>((next & 1) * kUmmaN), fx);
                }
#if ITK_EXPERIMENT == 0 || ITK_EXPERIMENT == 6
                finish_half(1, t, quad_reduce(c_r0, c_r1, d_r0, d_r1), scale[1], range_key[1]);
#elif ITK_EXPERIMENT == 2
                if (c_r0 + c_r1 + d_r0 + d_r1 == 1.2345e38f) own_count += 1;
#endif
                scale[0] = next_scale[0];
                scale[1] = next_scale[1];
                range_key[0] = next_range_key[0];
                range_key[1] = next_range_key[1];
            }
            if (!ok) break;
            __syncwarp();
            if (MODE != kModeRepair) {
                // lane 0 finishes row 2g, lane 1 row 2g+1: their running counts are the segment sizes
                if (lane < 2) sh.counts[slot][own_r][quarter] = own_count;
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.cand_ready[slot]);
            }
            ++unit_iter;
        }
        if (DIAG && p.trace != nullptr && quarter == 0 && lane == 0) {
            long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields + 4 * wg;
            trace[kTraceEpiTotal] = clock64() - role_begin;
            trace[kTraceEpiWaitAcc] = wait_acc;
            trace[kTraceEpiWaitFree] = wait_free;
            trace[kTraceEpiWaitW] = wait_w;
        }
        if (!ok && lane == 0) atomicOr(p.status, kStatusWaitExpired);
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

}  // namespace itk
