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

constexpr int kSegments = 8;                   // one per epilogue warp: segment = (key >> 5) & 7
constexpr int kSegCap = 320;                   // shared-memory candidates per (row, segment)
constexpr int kRowCap = kSegments * kSegCap;   // 2560
constexpr int kSpillSegCap = 704;              // global spill entries per (row, segment)
constexpr int kSpillRow = kSegments * kSpillSegCap;  // 5632 u64 per row
constexpr int kRepairChunk = 16384;

constexpr int kThreads = 512;
constexpr int kEpilogueWarp0 = 4;
constexpr int kEpilogueThreads = 256;
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
    int hist[256];
    int sel_bin;
    int sel_greater;
    int sel_failed;
    int sel_total;
    int sel_gcount;
    int sel_ecount;
    uint32_t tmem_base;
    int abort;
    uint64_t kv_full[kKvStages];
    uint64_t kv_empty[kKvStages];
    uint64_t q_full;
    uint64_t q_empty;
    uint64_t w_full[2];
    uint64_t w_empty[2];
    uint64_t acc_full[kAccBuffers];
    uint64_t acc_empty[kAccBuffers];
    uint64_t cand_ready[2];
    uint64_t cand_free[2];
};

constexpr size_t kSmemTileBytes = kQBytes + kKvStages * kKvBytes;
constexpr size_t kFusedSmemBytes = 1024 + kSmemTileBytes + sizeof(FusedShared);
static_assert(kFusedSmemBytes <= 232448, "fused kernel exceeds the 227 KB shared-memory limit");
static_assert(kSegCap % 32 == 0 && kSpillSegCap % 32 == 0, "segment capacities are warp multiples");

// mbar_wait that adds the cycles it took to `cycles` in diagnostic builds.
template <bool DIAG>
__device__ __forceinline__ bool timed_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           long long& cycles) {
    if (DIAG) {
        const long long begin = clock64();
        const bool ok = mbar_wait(bar, parity, abort_flag);
        cycles += clock64() - begin;
        return ok;
    }
    return mbar_wait(bar, parity, abort_flag);
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
    return static_cast<int>(((packed >> 5) << 8) | (static_cast<uint32_t>(segment) << 5) | (packed & 31u));
}

__device__ __forceinline__ uint16_t encode_key(int key) {
    const uint32_t k = static_cast<uint32_t>(key);
    return static_cast<uint16_t>(((k >> 8) << 5) | (k & 31u));
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
    const uint64_t* spill;    // [kSegments][kSpillSegCap]
};

// Four rounds of 8-bit radix selection over the ordered score bits of one row.
// On return `prefix` is the rank-th largest score and `rank` the number of
// candidates equal to it that belong to the top `rank_in`.  Needs
// rank_in <= number of candidates.  Called by all consumer threads.
__device__ __forceinline__ void radix_select(FusedShared& sh, const RowCandidates& c, int ctid, int rank_in,
                                             uint32_t& prefix, int& rank) {
    prefix = 0;
    rank = rank_in;
    uint32_t mask = 0;
#pragma unroll 1
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int bin = ctid; bin < 256; bin += kConsumerThreads) sh.hist[bin] = 0;
        consumer_sync();
#pragma unroll 1
        for (int s = 0; s < kSegments; ++s) {
            const int count = c.counts[s];
            const int in_smem = min(count, kSegCap);
            for (int i = ctid; i < in_smem; i += kConsumerThreads) {
                const uint32_t score = c.scores[s * kSegCap + i];
                if ((score & mask) == prefix) atomicAdd(&sh.hist[(score >> shift) & 255u], 1);
            }
            const int spilled = min(count, kSegCap + kSpillSegCap) - kSegCap;
            for (int i = ctid; i < spilled; i += kConsumerThreads) {
                const uint32_t score = static_cast<uint32_t>(c.spill[s * kSpillSegCap + i] >> 32);
                if ((score & mask) == prefix) atomicAdd(&sh.hist[(score >> shift) & 255u], 1);
            }
        }
        consumer_sync();
        if (ctid < 32) {
            // lane l owns bins 8l .. 8l+7; `above` = candidates in bins owned by higher lanes
            int bins[8];
            int mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bins[j] = sh.hist[ctid * 8 + j];
                mine += bins[j];
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
        mask |= 0xffu << shift;
    }
}

// Writes the selected candidates of one row: everything above `cutoff`, then
// `equal_needed` of the candidates equal to it (any of them).  With
// take_all = true every candidate is written.  Returns nothing; the number of
// entries written is greater_total + equal_needed (or the candidate total).
__device__ __forceinline__ void emit_row(FusedShared& sh, const RowCandidates& c, int ctid, uint32_t cutoff,
                                         int equal_needed, int greater_total, bool take_all, int32_t* out_ids,
                                         uint64_t* out_pairs) {
    const int lane = ctid & 31;
    const int cwarp = ctid >> 5;
#pragma unroll 1
    for (int s = 0; s < kSegments; ++s) {
        const int count = c.counts[s];
        const int in_smem = min(count, kSegCap);
        for (int base = cwarp * 32; base < in_smem; base += kConsumerThreads) {
            const int i = base + lane;
            const bool live = i < in_smem;
            const uint32_t score = live ? c.scores[s * kSegCap + i] : 0u;
            const bool greater = live && (take_all || score > cutoff);
            const bool equal = live && !take_all && score == cutoff;
            const int g = warp_reserve(&sh.sel_gcount, greater, lane);
            const int e = warp_reserve(&sh.sel_ecount, equal, lane);
            int position = -1;
            if (greater) position = g;
            else if (equal && e < equal_needed) position = greater_total + e;
            if (position >= 0 && position < kTopK) {
                const int key = decode_key(c.ids[s * kSegCap + i], s);
                if (out_ids != nullptr) out_ids[position] = key;
                if (out_pairs != nullptr)
                    out_pairs[position] = (static_cast<uint64_t>(score) << 32) | static_cast<uint32_t>(key);
            }
        }
        const int spilled = min(count, kSegCap + kSpillSegCap) - kSegCap;
        for (int base = cwarp * 32; base < spilled; base += kConsumerThreads) {
            const int i = base + lane;
            const bool live = i < spilled;
            const uint64_t pair = live ? c.spill[s * kSpillSegCap + i] : 0ull;
            const uint32_t score = static_cast<uint32_t>(pair >> 32);
            const bool greater = live && (take_all || score > cutoff);
            const bool equal = live && !take_all && score == cutoff;
            const int g = warp_reserve(&sh.sel_gcount, greater, lane);
            const int e = warp_reserve(&sh.sel_ecount, equal, lane);
            int position = -1;
            if (greater) position = g;
            else if (equal && e < equal_needed) position = greater_total + e;
            if (position >= 0 && position < kTopK) {
                if (out_ids != nullptr) out_ids[position] = static_cast<int32_t>(static_cast<uint32_t>(pair));
                if (out_pairs != nullptr) out_pairs[position] = pair;
            }
        }
    }
}

// Exact Top-2048 of one row from its candidates (kModeTopK consumer).
__device__ __forceinline__ void consume_topk_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                 int slot, bool has_tiles, int ctid) {
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
    if (total <= kTopK) {
        // only reachable when valid <= 2048 (threshold forced to -inf): take everything
        emit_row(sh, c, ctid, 0u, 0, 0, true, out_ids, out_pairs);
        for (int i = total + ctid; i < kTopK; i += kConsumerThreads) {
            if (out_ids != nullptr) out_ids[i] = -1;
            if (out_pairs != nullptr) out_pairs[i] = 0ull;
        }
    } else {
        uint32_t cutoff;
        int equal_needed;
        radix_select(sh, c, ctid, kTopK, cutoff, equal_needed);
        emit_row(sh, c, ctid, cutoff, equal_needed, kTopK - equal_needed, false, out_ids, out_pairs);
    }
    if (ctid == 0) {
        p.failure_flags[row_slot] = 0;
        if (p.out_counts != nullptr) p.out_counts[row_slot] = min(total, kTopK);
    }
    consumer_sync();
}

// Threshold of one row = rank-th largest valid sampled score (kModeSample consumer).
__device__ __forceinline__ void consume_sample_row(FusedShared& sh, const FusedParams& p, const Unit& u, int r,
                                                   int slot, bool has_tiles, int ctid) {
    const int row = u.row0 + r;
    const int start = __ldg(p.k_start + row);
    const int end = __ldg(p.k_end + row);
    const float minus_inf = __int_as_float(0xff800000);
    if (!has_tiles || end - start <= p.target_candidates) {
        if (ctid == 0) p.thresholds_out[row] = minus_inf;
        return;
    }
    RowCandidates c;
    c.scores = sh.cand_scores[slot][r];
    c.ids = sh.cand_ids[slot][r];
    c.counts = sh.counts[slot][r];
    c.spill = nullptr;
    if (ctid == 0) {
        int total = 0;
        int overflow = 0;
        for (int s = 0; s < kSegments; ++s) {
            total += c.counts[s];
            overflow |= c.counts[s] > kSegCap;
        }
        sh.sel_total = total;
        sh.sel_failed = overflow;
    }
    consumer_sync();
    const int total = sh.sel_total;
    const bool overflow = sh.sel_failed != 0;
    if (overflow || total < p.sample_rank) {
        if (ctid == 0) p.thresholds_out[row] = minus_inf;
        consumer_sync();
        return;
    }
    uint32_t cutoff;
    int unused;
    radix_select(sh, c, ctid, p.sample_rank, cutoff, unused);
    if (ctid == 0) p.thresholds_out[row] = ordered_to_float(cutoff);
    consumer_sync();
}

// ------------------------------------------------------------------ the kernel

template <int MODE, bool DIAG>
__global__ void __launch_bounds__(kThreads, 1) itk_fused_kernel(const __grid_constant__ FusedParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;
    uint8_t* smem_kv = smem + kQBytes;
    FusedShared& sh = *reinterpret_cast<FusedShared*>(smem + kSmemTileBytes);
    volatile int* abort_flag = &sh.abort;

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kKvStages; ++i) {
            mbar_init(&sh.kv_full[i], 1);
            mbar_init(&sh.kv_empty[i], 1);
        }
        mbar_init(&sh.q_full, 1);
        mbar_init(&sh.q_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.w_full[i], 1);
            mbar_init(&sh.w_empty[i], kEpilogueThreads);
            mbar_init(&sh.acc_full[i], 1);
            mbar_init(&sh.acc_empty[i], kEpilogueThreads / 2);
            mbar_init(&sh.cand_ready[i], kEpilogueThreads);
            mbar_init(&sh.cand_free[i], kConsumerThreads);
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
                ok = mbar_wait(&sh.w_empty[ws], ((q_iter >> 1) & 1) ^ 1, abort_flag);
                if (!ok) break;
                const uint32_t w_bytes = static_cast<uint32_t>(u.nrows) * kHeads * sizeof(float);
                mbar_arrive_expect_tx(&sh.w_full[ws], w_bytes);
                bulk_load(sh.weights[ws], p.weights + static_cast<long long>(u.row0) * kHeads, w_bytes,
                          &sh.w_full[ws]);
                for (int t = u.tile_begin; t < u.tile_end; ++t, ++kv_iter) {
                    const int stage = kv_iter % kKvStages;
                    ok = timed_wait<DIAG>(&sh.kv_empty[stage], ((kv_iter / kKvStages) & 1) ^ 1, abort_flag, wait_kv);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sh.kv_full[stage], kKvBytes);
                    tma_load_2d(smem_kv + stage * kKvBytes, &p.map_kv, &sh.kv_full[stage], 0, t * kTileKeys);
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
            int acc_iter[kAccBuffers] = {0, 0};
            bool ok = true;
            long long wait_acc = 0, wait_kv = 0, wait_q = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                if (u.tile_end == u.tile_begin) continue;
                ok = timed_wait<DIAG>(&sh.q_full, q_iter & 1, abort_flag, wait_q);
                if (!ok) break;
                for (int t = u.tile_begin; t < u.tile_end; ++t, ++kv_iter) {
                    const int buffer = t & 1;
                    const int stage = kv_iter % kKvStages;
                    ok = timed_wait<DIAG>(&sh.acc_empty[buffer], (acc_iter[buffer] & 1) ^ 1, abort_flag, wait_acc);
                    if (!ok) break;
                    ok = timed_wait<DIAG>(&sh.kv_full[stage], (kv_iter / kKvStages) & 1, abort_flag, wait_kv);
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                    const uint64_t desc_kv = umma_desc_sw128_kmajor(smem_u32(smem_kv + stage * kKvBytes));
                    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buffer * kUmmaN);
#pragma unroll
                    for (int k = 0; k < kHeadDim / 32; ++k) {
                        // advance both operands by 32 bytes (= 2 descriptor address units) per K step
                        umma_f8(tmem_d, desc_kv + 2 * k, desc_q + 2 * k, idesc, k > 0 ? 1u : 0u);
                    }
                    umma_commit(&sh.kv_empty[stage]);
                    umma_commit(&sh.acc_full[buffer]);
                    ++acc_iter[buffer];
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
    } else if (warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + kEpilogueThreads / 32) {
        // ============================================================ epilogue
        const int ew = warp - kEpilogueWarp0;   // 0..7 = candidate segment
        const int wg = ew >> 2;                 // TMEM buffer / tile parity served by this warpgroup
        const int quarter = ew & 3;             // TMEM lane quarter this warp may read (= warp % 4)
        const int lane_key = quarter * 32 + lane;
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(wg * kUmmaN);
        const float minus_inf = __int_as_float(0xff800000);
        int unit_iter = 0;  // units with tiles
        int acc_iter = 0;   // tiles of this warpgroup's parity
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
                ok = timed_wait<DIAG>(&sh.cand_free[slot], use_parity ^ 1, abort_flag, wait_free);
                if (!ok) break;
            }
            ok = timed_wait<DIAG>(&sh.w_full[slot], use_parity, abort_flag, wait_w);
            if (!ok) break;

            int row_lo[kBlockQ], row_hi[kBlockQ], count[kBlockQ];
            float threshold[kBlockQ];
            bool row_on[kBlockQ];
#pragma unroll
            for (int r = 0; r < kBlockQ; ++r) {
                count[r] = 0;
                row_on[r] = r < u.nrows;
                row_lo[r] = 0;
                row_hi[r] = 0;
                threshold[r] = minus_inf;
                if (row_on[r]) {
                    const int row = u.row0 + r;
                    const long long row_slot = static_cast<long long>(u.shard) * p.rows + row;
                    const int start = __ldg(p.k_start + row);
                    const int end = __ldg(p.k_end + row);
                    if (MODE == kModeSample) {
                        row_lo[r] = start;
                        row_hi[r] = end;
                        row_on[r] = end - start > p.target_candidates;
                    } else {
                        row_lo[r] = max(start, u.key_lo);
                        row_hi[r] = min(min(end, p.keys), u.key_hi);
                        if (MODE == kModeTopK) {
                            const int valid = row_hi[r] - row_lo[r];
                            if (valid > kTopK) threshold[r] = __ldg(p.thresholds + row_slot);
                            row_on[r] = valid > (p.out_pairs != nullptr ? 0 : p.top_k_min_valid);
                        } else {
                            row_on[r] = p.failure_flags[row_slot] != 0;
                        }
                    }
                }
            }

            for (int t = u.tile_begin; t < u.tile_end; ++t) {
                if ((t & 1) != wg) continue;
                const int key = t * kTileKeys + lane_key;   // key (or sample position) of this thread
                const bool key_ok = key < p.keys;
                const float scale = key_ok ? __ldg(p.kv_scales + key) : 0.0f;
                int range_key = key;
                if (MODE == kModeSample) range_key = key_ok ? __ldg(p.sample_ids + key) : 0x7fffffff;

                ok = timed_wait<DIAG>(&sh.acc_full[wg], acc_iter & 1, abort_flag, wait_acc);
                if (!ok) break;
                ++acc_iter;
                __syncwarp();
                tcgen05_fence_after_sync();

                uint32_t ra[32], rb[32];
                tmem_load_32(tmem_lane, ra);
#pragma unroll
                for (int r = 0; r < kBlockQ; ++r) {
                    const float4* w4 = reinterpret_cast<const float4*>(&sh.weights[slot][r * kHeads]);
                    float2 acc0 = make_float2(0.0f, 0.0f);
                    float2 acc1 = make_float2(0.0f, 0.0f);
                    // first half of the heads is in ra, second half is loaded into rb meanwhile
                    tmem_load_wait(ra);
                    tmem_load_32(tmem_lane + static_cast<uint32_t>(r * kHeads + 32), rb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 w = w4[j];
                        const float2 x0 = make_float2(fmaxf(__uint_as_float(ra[4 * j + 0]), 0.0f),
                                                      fmaxf(__uint_as_float(ra[4 * j + 1]), 0.0f));
                        const float2 x1 = make_float2(fmaxf(__uint_as_float(ra[4 * j + 2]), 0.0f),
                                                      fmaxf(__uint_as_float(ra[4 * j + 3]), 0.0f));
                        acc0 = fma2(x0, make_float2(w.x, w.y), acc0);
                        acc1 = fma2(x1, make_float2(w.z, w.w), acc1);
                    }
                    tmem_load_wait(rb);
                    if (r + 1 < kBlockQ) {
                        tmem_load_32(tmem_lane + static_cast<uint32_t>((r + 1) * kHeads), ra);
                    } else {
                        // every column of this buffer has been read: hand it back to the UMMA issuer
                        tcgen05_fence_before_sync();
                        mbar_arrive(&sh.acc_empty[wg]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 w = w4[8 + j];
                        const float2 x0 = make_float2(fmaxf(__uint_as_float(rb[4 * j + 0]), 0.0f),
                                                      fmaxf(__uint_as_float(rb[4 * j + 1]), 0.0f));
                        const float2 x1 = make_float2(fmaxf(__uint_as_float(rb[4 * j + 2]), 0.0f),
                                                      fmaxf(__uint_as_float(rb[4 * j + 3]), 0.0f));
                        acc0 = fma2(x0, make_float2(w.x, w.y), acc0);
                        acc1 = fma2(x1, make_float2(w.z, w.w), acc1);
                    }
                    const float score = ((acc0.x + acc0.y) + (acc1.x + acc1.y)) * scale;
                    const bool in_range = key_ok && range_key >= row_lo[r] && range_key < row_hi[r];

                    if (DIAG) {
                        if (r < u.nrows && key_ok && p.diag_logits != nullptr) {
                            const bool shown = MODE == kModeSample ? true : in_range;
                            p.diag_logits[static_cast<long long>(u.row0 + r) * p.diag_stride + key] =
                                shown ? score : minus_inf;
                        }
                    }

                    if (MODE == kModeRepair) {
                        if (row_on[r] && key_ok && key >= u.key_lo && key < u.key_hi) {
                            const long long row_slot = static_cast<long long>(u.shard) * p.rows + u.row0 + r;
                            p.repair_pairs[row_slot * kRepairChunk + (key - u.key_lo)] =
                                in_range ? pack_score_id(score, static_cast<uint32_t>(key)) : 0ull;
                        }
                    } else {
                        bool active = row_on[r] && in_range;
                        if (MODE == kModeTopK) active = active && score >= threshold[r];
                        else active = active && (fabsf(score) <= 3.4028234663852886e38f);  // finite
                        const unsigned ballot = __ballot_sync(0xffffffffu, active);
                        const int position = count[r] + __popc(ballot & ((1u << lane) - 1u));
                        count[r] += __popc(ballot);
                        if (active) {
                            if (position < kSegCap) {
                                sh.cand_scores[slot][r][ew * kSegCap + position] = ordered_bits(score);
                                sh.cand_ids[slot][r][ew * kSegCap + position] = encode_key(key);
                            } else if (MODE == kModeTopK && position < kSegCap + kSpillSegCap) {
                                const long long row_slot = static_cast<long long>(u.shard) * p.rows + u.row0 + r;
                                p.spill[row_slot * kSpillRow + ew * kSpillSegCap + (position - kSegCap)] =
                                    pack_score_id(score, static_cast<uint32_t>(key));
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            if (MODE != kModeRepair) {
                if (lane == 0) {
#pragma unroll
                    for (int r = 0; r < kBlockQ; ++r) sh.counts[slot][r][ew] = count[r];
                }
                __syncwarp();
                mbar_arrive(&sh.cand_ready[slot]);
            }
            mbar_arrive(&sh.w_empty[slot]);
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
    } else {
        // ============================================================ Top-K / threshold consumers
        if (MODE != kModeRepair) {
            const int cwarp = warp < kEpilogueWarp0 ? warp - 2 : warp - 12 + 2;   // warps 2,3,12..15 -> 0..5
            const int ctid = cwarp * 32 + lane;
            int unit_iter = 0;
            bool ok = true;
            long long wait_ready = 0, select_cycles = 0;
            const long long role_begin = DIAG ? clock64() : 0;
            if (DIAG && p.trace != nullptr && ctid == 0)
                p.trace[static_cast<long long>(blockIdx.x) * kTraceFields + kTraceNsBegin] = global_timer_ns();
            for (int iter = 0; ok; ++iter) {
                Unit u;
                if (!load_unit<MODE>(p, iter, u)) break;
                const bool has_tiles = u.tile_end > u.tile_begin;
                const int slot = unit_iter & 1;
                if (has_tiles) {
                    ok = timed_wait<DIAG>(&sh.cand_ready[slot], (unit_iter >> 1) & 1, abort_flag, wait_ready);
                    if (!ok) break;
                }
                const long long select_begin = DIAG ? clock64() : 0;
                for (int r = 0; r < u.nrows; ++r) {
                    if (MODE == kModeTopK) consume_topk_row(sh, p, u, r, slot, has_tiles, ctid);
                    else consume_sample_row(sh, p, u, r, slot, has_tiles, ctid);
                }
                if (DIAG) select_cycles += clock64() - select_begin;
                if (has_tiles) {
                    mbar_arrive(&sh.cand_free[slot]);
                    ++unit_iter;
                }
            }
            if (DIAG && p.trace != nullptr && ctid == 0) {
                long long* trace = p.trace + static_cast<long long>(blockIdx.x) * kTraceFields;
                trace[kTraceConTotal] = clock64() - role_begin;
                trace[kTraceConWaitReady] = wait_ready;
                trace[kTraceConSelect] = select_cycles;
                trace[kTraceConUnits] = unit_iter;
                trace[kTraceNsEnd] = global_timer_ns();
            }
            if (!ok && lane == 0) atomicOr(p.status, kStatusWaitExpired);
        }
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
