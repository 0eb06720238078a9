// C-ABI entry points of libitk_b200.so: argument validation, TMA descriptor
// construction and kernel launches.  Ahead-of-time compiled for sm_100a; there is
// no JIT step and no dependency beyond the CUDA runtime and driver.
#include "../../include/itk_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "itk_quantize.cuh"
#include "itk_select.cuh"

namespace {

using namespace itk;

thread_local std::string g_last_error;

int fail(int code, const char* format, ...) {
    char buffer[512];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof(buffer), format, args);
    va_end(args);
    g_last_error = buffer;
    return code;
}

#define ITK_REQUIRE(condition, ...)                             \
    do {                                                        \
        if (!(condition)) return fail(ITK_ERR_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define ITK_CUDA(call)                                                                        \
    do {                                                                                      \
        const cudaError_t status_ = (call);                                                   \
        if (status_ != cudaSuccess)                                                           \
            return fail(ITK_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(status_));   \
    } while (0)

bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

// ---------------------------------------------------------------- driver entry point

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled_entry() {
    static EncodeTiled entry = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* symbol = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) == cudaSuccess &&
            query == cudaDriverEntryPointSuccess) {
            entry = reinterpret_cast<EncodeTiled>(symbol);
        }
    });
    return entry;
}

// [rows, 128] bytes, row-major, box of `box_rows` rows x 128 bytes, 128-byte swizzle.
int make_row_map(CUtensorMap* map, const void* base, long long rows, int box_rows) {
    EncodeTiled encode = encode_tiled_entry();
    if (encode == nullptr) return fail(ITK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kHeadDim)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kHeadDim), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result =
        encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, element_strides,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return fail(ITK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(result));
    return ITK_OK;
}

// ---------------------------------------------------------------- per-device set-up

constexpr int kMaxDevices = 64;
std::mutex g_init_mutex;
bool g_initialised[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
cudaStream_t g_body_stream[kMaxDevices] = {};   // captures the body of a conditional graph node

constexpr size_t kPairSmemBytes = static_cast<size_t>(kPairCapacity) * sizeof(uint64_t);
constexpr int kShardMergeCapacity = 6144;   // pairs staged per row by the merge of one launch's key shards

template <typename Kernel>
cudaError_t raise_smem(Kernel kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

int init_current_device(int* device_out) {
    int device = 0;
    ITK_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(ITK_ERR_UNSUPPORTED, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(g_init_mutex);
    if (!g_initialised[device]) {
        cudaDeviceProp properties;
        ITK_CUDA(cudaGetDeviceProperties(&properties, device));
        if (properties.major != 10)
            return fail(ITK_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                        properties.major, properties.minor);
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeTopK, false>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeTopK, true>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeSample, false>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeSample, true>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeRepair, false>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeTopK, false, true>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_fused_kernel<kModeRepair, false, true>, kFusedSmemBytes));
        ITK_CUDA(raise_smem(itk_pair_topk_kernel, kPairSmemBytes));
        g_sm_count[device] = properties.multiProcessorCount;
        // (a stream cannot be created while this thread captures in the global mode; the scope then stays unconditional)
        if (cudaStreamCreateWithFlags(&g_body_stream[device], cudaStreamNonBlocking) != cudaSuccess) {
            g_body_stream[device] = nullptr;
            (void)cudaGetLastError();
        }
        g_initialised[device] = true;
    }
    if (device_out != nullptr) *device_out = device;
    return ITK_OK;
}

int launch_check(const char* what) {
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(ITK_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(status));
    return ITK_OK;
}

int fused_grid(int device, long long units, int max_ctas) {
    long long grid = g_sm_count[device];
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    if (units < grid) grid = units;
    if (grid > ITK_MAX_CTAS) grid = ITK_MAX_CTAS;   // the spill workspace has one region per CTA and unit row
    return static_cast<int>(grid < 1 ? 1 : grid);
}

template <int MODE>
int launch_fused(const FusedParams& params, bool diagnostic, int grid, cudaStream_t stream) {
    if (diagnostic) {
        if (params.tile_table != nullptr) return fail(ITK_ERR_UNSUPPORTED, "paged keys have no diagnostic build");
        if (MODE == kModeRepair) return fail(ITK_ERR_UNSUPPORTED, "the repair producer has no diagnostic build");
        if (MODE == kModeTopK)
            itk_fused_kernel<kModeTopK, true><<<grid, kThreads, kFusedSmemBytes, stream>>>(params);
        else
            itk_fused_kernel<kModeSample, true><<<grid, kThreads, kFusedSmemBytes, stream>>>(params);
    } else if (params.tile_table != nullptr) {
        if (MODE == kModeSample) return fail(ITK_ERR_UNSUPPORTED, "the sample prepass reads gathered keys, not pages");
        if (MODE == kModeTopK)
            itk_fused_kernel<kModeTopK, false, true><<<grid, kThreads, kFusedSmemBytes, stream>>>(params);
        else
            itk_fused_kernel<kModeRepair, false, true><<<grid, kThreads, kFusedSmemBytes, stream>>>(params);
    } else {
        itk_fused_kernel<MODE, false><<<grid, kThreads, kFusedSmemBytes, stream>>>(params);
    }
    return launch_check("itk_fused_kernel");
}

int pair_grid(int device, int rows) {
    const int sms = g_sm_count[device];
    return rows < sms ? (rows < 1 ? 1 : rows) : sms;
}

}  // namespace

extern "C" {

const char* itk_version(void) { return "fusedindextopk_b200 0.1.0 (sm_100a)"; }

const char* itk_last_error(void) { return g_last_error.c_str(); }

int itk_init(int device) {
    ITK_CUDA(cudaSetDevice(device));
    return init_current_device(nullptr);
}

int itk_resource_report(char* buffer, size_t buffer_bytes) {
    ITK_REQUIRE(buffer != nullptr && buffer_bytes > 0, "resource report needs a buffer");
    int device = 0;
    const int status = init_current_device(&device);
    if (status != ITK_OK) return status;
    std::string text;
    char line[256];
    auto add = [&](const char* name, const void* function, int threads, size_t dynamic_smem) -> int {
        cudaFuncAttributes attributes{};
        ITK_CUDA(cudaFuncGetAttributes(&attributes, function));
        snprintf(line, sizeof(line),
                 "%s.registers_per_thread=%d\n%s.static_shared_bytes=%zu\n%s.dynamic_shared_bytes=%zu\n"
                 "%s.local_bytes_per_thread=%zu\n%s.threads=%d\n",
                 name, attributes.numRegs, name, attributes.sharedSizeBytes, name, dynamic_smem, name,
                 attributes.localSizeBytes, name, threads);
        text += line;
        return ITK_OK;
    };
    int rc;
    if ((rc = add("fused_topk", (const void*)itk_fused_kernel<kModeTopK, false>, kThreads, kFusedSmemBytes))) return rc;
    if ((rc = add("fused_sample", (const void*)itk_fused_kernel<kModeSample, false>, kThreads, kFusedSmemBytes))) return rc;
    if ((rc = add("fused_repair", (const void*)itk_fused_kernel<kModeRepair, false>, kThreads, kFusedSmemBytes))) return rc;
    if ((rc = add("pair_topk", (const void*)itk_pair_topk_kernel, kPairThreads, kPairSmemBytes))) return rc;
    if ((rc = add("gather", (const void*)itk_gather_kernel, 256, 0))) return rc;
    snprintf(line, sizeof(line),
             "sm_count=%d\nblock_q=%d\nkv_stages=%d\nsegment_capacity=%d\nspill_segment_capacity=%d\n"
             "tmem_columns=%d\n",
             g_sm_count[device], kBlockQ, kKvStages, kSegCap, kSpillSegCap, kTmemColumns);
    text += line;
    if (text.size() + 1 > buffer_bytes) return fail(ITK_ERR_ARGUMENT, "resource report needs %zu bytes", text.size() + 1);
    memcpy(buffer, text.c_str(), text.size() + 1);
    return ITK_OK;
}

int itk_workspace_bytes(int rows, int keys, int shards, itk_workspace_sizes* sizes) {
    ITK_REQUIRE(sizes != nullptr, "sizes must not be null");
    ITK_REQUIRE(rows > 0 && keys > 0 && shards >= 1 && shards <= ITK_MAX_PAIR_SOURCES,
                "need rows > 0, keys > 0 and 1 <= shards <= %d", ITK_MAX_PAIR_SOURCES);
    const size_t slots = static_cast<size_t>(rows) * shards;
    // the spill is addressed by CTA and row of the CTA's current unit: 4 regions per CTA, never more CTAs than units
    const size_t unit_rows = static_cast<size_t>((rows + kBlockQ - 1) / kBlockQ) * shards * kBlockQ;
    const size_t spill_rows = unit_rows < static_cast<size_t>(ITK_MAX_CTAS) * kBlockQ ? unit_rows
                                                                                      : static_cast<size_t>(ITK_MAX_CTAS) * kBlockQ;
    sizes->spill_bytes = spill_rows * kSpillRow * sizeof(uint64_t);
    sizes->repair_pairs_bytes = slots * kRepairChunk * sizeof(uint64_t);
    sizes->pairs_bytes = slots * kTopK * sizeof(uint64_t);
    sizes->counts_bytes = slots * sizeof(int32_t);
    sizes->flags_bytes = slots;
    sizes->thresholds_bytes = slots * sizeof(float);
    sizes->repair_chunks = (keys + kRepairChunk - 1) / kRepairChunk;
    sizes->chunk_ranges_bytes = static_cast<size_t>(sizes->repair_chunks) * rows * sizeof(int32_t);
    return ITK_OK;
}

int itk_gather_sampled_kv_paged(const void* kv, const float* kv_scales, const int32_t* sample_ids,
                                const int32_t* tile_table, void* sampled_kv, float* sampled_scales, int keys,
                                int physical_keys, int samples, itk_stream_t stream) {
    ITK_REQUIRE(kv && kv_scales && sample_ids && sampled_kv && sampled_scales, "gather pointers must not be null");
    ITK_REQUIRE(keys > 0 && samples > 0 && samples <= keys, "need 0 < samples <= keys");
    ITK_REQUIRE(tile_table == nullptr || (physical_keys >= kTileKeys && physical_keys % kTileKeys == 0),
                "physical_keys must be a positive multiple of 128");
    ITK_REQUIRE(aligned16(kv) && aligned16(sampled_kv), "kv and sampled_kv must be 16-byte aligned");
    const int work = samples * 8;
    itk_gather_kernel<<<(work + 255) / 256, 256, 0, stream>>>(
        static_cast<const uint8_t*>(kv), kv_scales, sample_ids, tile_table, static_cast<uint8_t*>(sampled_kv),
        sampled_scales, samples);
    return launch_check("itk_gather_kernel");
}

int itk_gather_sampled_kv(const void* kv, const float* kv_scales, const int32_t* sample_ids, void* sampled_kv,
                          float* sampled_scales, int keys, int samples, itk_stream_t stream) {
    return itk_gather_sampled_kv_paged(kv, kv_scales, sample_ids, nullptr, sampled_kv, sampled_scales, keys, 0, samples,
                                       stream);
}

int itk_quantize_rows_e4m3(const void* source, int source_dtype, const float* fold, float* folded, void* values,
                           float* scales, long long rows, itk_stream_t stream) {
    static_assert(kQuantDim == ITK_HEAD_DIM, "rows are one index head wide");
    ITK_REQUIRE(source && values, "source and values must not be null");
    ITK_REQUIRE(source_dtype == ITK_SOURCE_F32 || source_dtype == ITK_SOURCE_BF16,
                "source_dtype must be ITK_SOURCE_F32 or ITK_SOURCE_BF16");
    ITK_REQUIRE((fold == nullptr) == (folded == nullptr), "fold and folded go together");
    ITK_REQUIRE(scales || folded, "nothing would receive the row scales");
    ITK_REQUIRE(rows > 0 && rows <= (1ll << 31) * kQuantRowsPerBlock / 2, "rows out of range");
    ITK_REQUIRE(aligned16(source) && aligned16(values), "source and values must be 16-byte aligned");
    const unsigned blocks = static_cast<unsigned>((rows + kQuantRowsPerBlock - 1) / kQuantRowsPerBlock);
    if (source_dtype == ITK_SOURCE_F32) {
        itk_quantize_rows_kernel<float><<<blocks, kQuantThreads, 0, stream>>>(
            static_cast<const float*>(source), fold, folded, static_cast<uint8_t*>(values), scales, rows);
    } else {
        itk_quantize_rows_kernel<__nv_bfloat16><<<blocks, kQuantThreads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(source), fold, folded, static_cast<uint8_t*>(values), scales, rows);
    }
    return launch_check("itk_quantize_rows_kernel");
}

int itk_sample_thresholds(const void* q, const void* sampled_kv, const float* sampled_scales, const float* weights,
                          const int32_t* sample_ids, const int32_t* k_start, const int32_t* k_end,
                          float* thresholds, int rows, int samples, int sample_rank, int target_candidates,
                          int block_begin, int block_stride, int num_blocks, int exit_when_no_keys,
                          float* diag_logits, long long diag_stride, long long* trace, int* status,
                          itk_stream_t stream) {
    ITK_REQUIRE(q && sampled_kv && sampled_scales && weights && sample_ids && k_start && k_end && thresholds && status,
                "sample threshold pointers must not be null");
    ITK_REQUIRE(rows > 0 && samples > 0, "need rows > 0 and samples > 0");
    ITK_REQUIRE(samples <= kRowCap - kSegments * 32 && samples <= kTopK,
                "at most %d samples fit the shared-memory candidate segments", kTopK);
    ITK_REQUIRE(sample_rank >= 1 && sample_rank <= samples, "sample_rank must lie in [1, samples]");
    ITK_REQUIRE(target_candidates > 0, "target_candidates must be positive");
    ITK_REQUIRE(aligned16(q) && aligned16(sampled_kv) && aligned16(weights), "q, sampled_kv, weights must be 16-byte aligned");
    ITK_REQUIRE(diag_logits == nullptr || diag_stride >= samples, "diag_stride must cover the samples");
    const int sample_blocks = (rows + kBlockQ - 1) / kBlockQ;
    ITK_REQUIRE(block_stride >= 1 && block_begin >= 0 && num_blocks >= 0 &&
                    (num_blocks == 0 || block_begin + static_cast<long long>(num_blocks - 1) * block_stride < sample_blocks),
                "owned query blocks must lie inside the %d blocks of the problem", sample_blocks);
    if (num_blocks == 0) return ITK_OK;
    int device = 0;
    int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    FusedParams params{};
    if ((rc = make_row_map(&params.map_q, q, static_cast<long long>(rows) * kHeads, kUmmaN)) != ITK_OK) return rc;
    if ((rc = make_row_map(&params.map_kv, sampled_kv, samples, kTileKeys)) != ITK_OK) return rc;
    params.kv_scales = sampled_scales;
    params.weights = weights;
    params.k_start = k_start;
    params.k_end = k_end;
    params.thresholds_out = thresholds;
    params.sample_ids = sample_ids;
    params.diag_logits = diag_logits;
    params.diag_stride = diag_stride;
    params.trace = trace;
    params.status = status;
    params.rows = rows;
    params.keys = samples;
    params.key_lo = 0;
    params.key_hi = samples;
    params.shard_keys = (samples + kTileKeys - 1) / kTileKeys * kTileKeys;
    params.shards = 1;
    params.block_begin = block_begin;
    params.block_stride = block_stride;
    params.num_blocks = num_blocks;
    params.sample_rank = sample_rank;
    params.target_candidates = target_candidates;
    params.top_k_min_valid = kTopK;
    params.wait_limit_ns = kWaitLimitNs;
    params.exit_when_no_keys = exit_when_no_keys != 0 ? 1 : 0;
    return launch_fused<kModeSample>(params, diag_logits != nullptr || trace != nullptr,
                                     fused_grid(device, params.num_blocks, 0), stream);
}

int itk_fused_topk(const itk_fused_args* args, itk_stream_t stream) {
    ITK_REQUIRE(args != nullptr, "args must not be null");
    const itk_fused_args& a = *args;
    ITK_REQUIRE(a.q && a.kv && a.kv_scales && a.weights && a.k_start && a.k_end && a.thresholds && a.spill && a.status,
                "fused top-k pointers must not be null");
    ITK_REQUIRE(a.rows > 0 && a.keys > 0 && a.keys <= ITK_MAX_KEYS, "need rows > 0 and 0 < keys <= %d", ITK_MAX_KEYS);
    ITK_REQUIRE(a.key_lo >= 0 && a.key_lo % kTileKeys == 0 && a.key_hi > a.key_lo && a.key_hi <= a.keys,
                "need 0 <= key_lo < key_hi <= keys with key_lo a multiple of 128");
    ITK_REQUIRE(a.shards >= 1 && a.shards <= ITK_MAX_PAIR_SOURCES, "need 1 <= shards <= %d", ITK_MAX_PAIR_SOURCES);
    ITK_REQUIRE(a.shards == 1 || (a.shard_pairs && a.shard_counts && a.shard_flags),
                "key-range shards need shard_pairs, shard_counts and shard_flags");
    ITK_REQUIRE(a.split_blocks >= 0 && a.split_blocks <= a.num_blocks, "split_blocks must lie in [0, num_blocks]");
    const int split_blocks = a.shards == 1 ? 0 : (a.split_blocks == 0 ? a.num_blocks : a.split_blocks);
    ITK_REQUIRE(split_blocks == a.num_blocks || (a.failure_flags && (a.out_ids != nullptr || a.out_pairs != nullptr)),
                "whole blocks need failure_flags and out_ids or out_pairs");
    const int total_blocks = (a.rows + kBlockQ - 1) / kBlockQ;
    ITK_REQUIRE(a.block_stride >= 1 && a.block_begin >= 0 && a.num_blocks >= 0 &&
                    (a.num_blocks == 0 || a.block_begin + static_cast<long long>(a.num_blocks - 1) * a.block_stride < total_blocks),
                "owned query blocks must lie inside the %d blocks of the problem", total_blocks);
    ITK_REQUIRE(aligned16(a.q) && aligned16(a.kv) && aligned16(a.weights), "q, kv, weights must be 16-byte aligned");
    ITK_REQUIRE(a.diag_logits == nullptr || a.diag_stride >= a.keys, "diag_stride must cover the keys");
    if (a.num_blocks == 0) return ITK_OK;
    int device = 0;
    int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    FusedParams params{};
    if ((rc = make_row_map(&params.map_q, a.q, static_cast<long long>(a.rows) * kHeads, kUmmaN)) != ITK_OK) return rc;
    if (a.tile_table != nullptr)
        ITK_REQUIRE(a.physical_keys >= kTileKeys && a.physical_keys % kTileKeys == 0,
                    "physical_keys must be a positive multiple of 128");
    if ((rc = make_row_map(&params.map_kv, a.kv, a.tile_table != nullptr ? a.physical_keys : a.keys, kTileKeys)) != ITK_OK)
        return rc;
    params.kv_scales = a.kv_scales;
    params.tile_table = a.tile_table;
    params.weights = a.weights;
    params.k_start = a.k_start;
    params.k_end = a.k_end;
    params.thresholds = a.thresholds;
    params.out_ids = a.out_ids;
    params.out_pairs = a.out_pairs;
    params.out_counts = a.out_counts;
    params.failure_flags = a.failure_flags;
    params.spill = a.spill;
    params.shard_pairs = a.shard_pairs;
    params.shard_counts = a.shard_counts;
    params.shard_flags = a.shard_flags;
    params.diag_logits = a.diag_logits;
    params.diag_stride = a.diag_stride;
    params.trace = a.trace;
    params.wait_limit_ns = a.wait_limit_ns != 0 ? a.wait_limit_ns : kWaitLimitNs;
    params.withhold_q_loads = a.withhold_loads;
    params.status = a.status;
    params.rows = a.rows;
    params.keys = a.keys;
    params.key_lo = a.key_lo;
    params.key_hi = a.key_hi;
    const int span = a.key_hi - a.key_lo;
    const int per_shard = (span + a.shards - 1) / a.shards;
    params.shard_keys = (per_shard + kTileKeys - 1) / kTileKeys * kTileKeys;
    params.shards = a.shards;
    params.split_blocks = split_blocks;
    params.block_begin = a.block_begin;
    params.block_stride = a.block_stride;
    params.num_blocks = a.num_blocks;
    params.top_k_min_valid = a.force_compute ? 0 : kTopK;
    params.exit_when_no_keys = a.exit_when_no_keys != 0 ? 1 : 0;
    if (a.sampled_kv != nullptr) {
        ITK_REQUIRE(a.sampled_scales && a.sample_ids && a.thresholds_out, "in-kernel thresholds need sampled_scales, sample_ids, thresholds_out");
        ITK_REQUIRE(a.samples > 0 && a.samples <= kRowCap - kSegments * 32 && a.samples <= kTopK,
                    "at most %d samples fit the shared-memory candidate segments", kTopK);
        ITK_REQUIRE(a.sample_rank >= 1 && a.sample_rank <= a.samples, "sample_rank must lie in [1, samples]");
        ITK_REQUIRE(a.target_candidates > 0, "target_candidates must be positive");
        ITK_REQUIRE(a.key_lo == 0 && a.key_hi == a.keys, "in-kernel thresholds need the whole key range");
        ITK_REQUIRE(a.diag_logits == nullptr, "in-kernel thresholds are not offered with diag_logits");
        ITK_REQUIRE(aligned16(a.sampled_kv), "sampled_kv must be 16-byte aligned");
        if ((rc = make_row_map(&params.map_sample, a.sampled_kv, a.samples, kTileKeys)) != ITK_OK) return rc;
        params.sample_scales = a.sampled_scales;
        params.sample_ids = a.sample_ids;
        params.thresholds_out = a.thresholds_out;
        params.sample_count = a.samples;
        params.sample_tiles = (a.samples + kTileKeys - 1) / kTileKeys;
        params.sample_rank = a.sample_rank;
        params.target_candidates = a.target_candidates;
    }
    const long long units = (a.num_blocks - split_blocks) + static_cast<long long>(split_blocks) * a.shards;
    return launch_fused<kModeTopK>(params, a.diag_logits != nullptr || a.trace != nullptr,
                                   fused_grid(device, units, a.max_ctas), stream);
}

int itk_update_chunk_ranges(const int32_t* k_start, const int32_t* k_end, int32_t* chunk_start,
                            int32_t* chunk_end, int rows, int keys, itk_stream_t stream) {
    ITK_REQUIRE(k_start && k_end && chunk_start && chunk_end, "chunk range pointers must not be null");
    ITK_REQUIRE(rows > 0 && keys > 0, "need rows > 0 and keys > 0");
    const int chunks = (keys + kRepairChunk - 1) / kRepairChunk;
    const long long work = static_cast<long long>(rows) * chunks;
    itk_chunk_ranges_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
        k_start, k_end, chunk_start, chunk_end, rows, chunks, keys, kRepairChunk);
    return launch_check("itk_chunk_ranges_kernel");
}

int itk_repair_produce(const void* q, const void* kv, const float* kv_scales, const float* weights,
                       const int32_t* k_start, const int32_t* k_end, const uint8_t* failure_flags,
                       uint64_t* repair_pairs, int rows, int keys, int chunk_lo, int chunk_hi, int block_begin,
                       int block_stride, int num_blocks, int* status, itk_stream_t stream) {
    return itk_repair_produce_paged(q, kv, kv_scales, weights, k_start, k_end, failure_flags, repair_pairs, rows, keys,
                                    chunk_lo, chunk_hi, block_begin, block_stride, num_blocks, nullptr, 0, status,
                                    stream);
}

int itk_repair_produce_paged(const void* q, const void* kv, const float* kv_scales, const float* weights,
                             const int32_t* k_start, const int32_t* k_end, const uint8_t* failure_flags,
                             uint64_t* repair_pairs, int rows, int keys, int chunk_lo, int chunk_hi, int block_begin,
                             int block_stride, int num_blocks, const int32_t* tile_table, int physical_keys,
                             int* status, itk_stream_t stream) {
    ITK_REQUIRE(tile_table == nullptr || (physical_keys >= kTileKeys && physical_keys % kTileKeys == 0),
                "physical_keys must be a positive multiple of 128");
    ITK_REQUIRE(q && kv && kv_scales && weights && k_start && k_end && failure_flags && repair_pairs && status,
                "repair producer pointers must not be null");
    ITK_REQUIRE(rows > 0 && keys > 0 && keys <= ITK_MAX_KEYS, "need rows > 0 and 0 < keys <= %d", ITK_MAX_KEYS);
    ITK_REQUIRE(chunk_lo >= 0 && chunk_lo % kTileKeys == 0 && chunk_hi > chunk_lo && chunk_hi <= keys &&
                    chunk_hi - chunk_lo <= kRepairChunk,
                "need a chunk of at most %d keys starting at a multiple of 128", kRepairChunk);
    const int total_blocks = (rows + kBlockQ - 1) / kBlockQ;
    ITK_REQUIRE(block_stride >= 1 && block_begin >= 0 && num_blocks >= 0 &&
                    (num_blocks == 0 || block_begin + static_cast<long long>(num_blocks - 1) * block_stride < total_blocks),
                "owned query blocks must lie inside the %d blocks of the problem", total_blocks);
    ITK_REQUIRE(aligned16(q) && aligned16(kv) && aligned16(weights), "q, kv, weights must be 16-byte aligned");
    if (num_blocks == 0) return ITK_OK;
    int device = 0;
    int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    FusedParams params{};
    if ((rc = make_row_map(&params.map_q, q, static_cast<long long>(rows) * kHeads, kUmmaN)) != ITK_OK) return rc;
    if ((rc = make_row_map(&params.map_kv, kv, tile_table != nullptr ? physical_keys : keys, kTileKeys)) != ITK_OK) return rc;
    params.kv_scales = kv_scales;
    params.tile_table = tile_table;
    params.weights = weights;
    params.k_start = k_start;
    params.k_end = k_end;
    params.failure_flags = const_cast<uint8_t*>(failure_flags);
    params.repair_pairs = repair_pairs;
    params.status = status;
    params.rows = rows;
    params.keys = keys;
    params.key_lo = chunk_lo;
    params.key_hi = chunk_hi;
    params.shard_keys = kRepairChunk;
    params.shards = 1;
    params.block_begin = block_begin;
    params.block_stride = block_stride;
    params.num_blocks = num_blocks;
    params.top_k_min_valid = kTopK;
    params.wait_limit_ns = kWaitLimitNs;
    return launch_fused<kModeRepair>(params, false, fused_grid(device, num_blocks, 0), stream);
}

int itk_chunk_local_topk(const uint64_t* repair_pairs, const int32_t* chunk_start, const int32_t* chunk_end,
                         const uint8_t* failure_flags, uint64_t* local_pairs, int32_t* local_counts,
                         uint8_t* repair_error_flags, int rows, int first_chunk, itk_stream_t stream) {
    ITK_REQUIRE(repair_pairs && chunk_start && chunk_end && failure_flags && local_pairs && local_counts &&
                    repair_error_flags,
                "chunk top-k pointers must not be null");
    ITK_REQUIRE(rows > 0, "need rows > 0");
    int device = 0;
    const int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    PairTopKParams params{};
    params.sources[0] = PairSource{repair_pairs, nullptr, kRepairChunk};
    params.num_sources = 1;
    params.rows = rows;
    params.row_mask = failure_flags;
    params.error_flags = repair_error_flags;
    params.clear_errors = first_chunk ? 1 : 0;
    params.expect_start = chunk_start;
    params.expect_end = chunk_end;
    params.error_count_mismatch = ITK_REPAIR_ERR_COUNT;
    params.error_selection = ITK_REPAIR_ERR_LOCAL_SELECT;
    params.out_pairs = local_pairs;
    params.out_counts = local_counts;
    params.stage_capacity = kPairCapacity;
    itk_pair_topk_kernel<<<pair_grid(device, rows), kPairThreads, kPairSmemBytes, stream>>>(params);
    return launch_check("itk_pair_topk_kernel (chunk)");
}

int itk_merge_topk_pairs(uint64_t* accumulator_pairs, int32_t* accumulator_counts, const uint64_t* local_pairs,
                         const int32_t* local_counts, const uint8_t* failure_flags, uint8_t* repair_error_flags,
                         int rows, int first_chunk, itk_stream_t stream) {
    ITK_REQUIRE(accumulator_pairs && accumulator_counts && local_pairs && local_counts && failure_flags &&
                    repair_error_flags,
                "merge pointers must not be null");
    ITK_REQUIRE(rows > 0, "need rows > 0");
    int device = 0;
    const int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    PairTopKParams params{};
    params.sources[0] = PairSource{accumulator_pairs, accumulator_counts, kTopK};
    params.sources[1] = PairSource{local_pairs, local_counts, kTopK};
    params.num_sources = 2;
    params.first_source = first_chunk ? 1 : 0;
    params.rows = rows;
    params.row_mask = failure_flags;
    params.error_flags = repair_error_flags;
    params.error_count_mismatch = ITK_REPAIR_ERR_MERGE_SELECT;
    params.error_selection = ITK_REPAIR_ERR_MERGE_SELECT;
    params.out_pairs = accumulator_pairs;
    params.out_counts = accumulator_counts;
    params.stage_capacity = kPairCapacity;
    itk_pair_topk_kernel<<<pair_grid(device, rows), kPairThreads, kPairSmemBytes, stream>>>(params);
    return launch_check("itk_pair_topk_kernel (merge)");
}

int itk_finalize_repair(const uint64_t* accumulator_pairs, const int32_t* accumulator_counts, int32_t* out_ids,
                        uint64_t* out_pairs, int32_t* out_counts, uint8_t* failure_flags,
                        const uint8_t* repair_error_flags, int rows, itk_stream_t stream) {
    ITK_REQUIRE(accumulator_pairs && accumulator_counts && failure_flags && repair_error_flags,
                "finalize pointers must not be null");
    ITK_REQUIRE(out_ids != nullptr || out_pairs != nullptr, "need out_ids or out_pairs");
    ITK_REQUIRE(rows > 0, "need rows > 0");
    itk_finalize_repair_kernel<<<rows, 256, 0, stream>>>(accumulator_pairs, accumulator_counts, out_ids, out_pairs,
                                                        out_counts, failure_flags, repair_error_flags, rows);
    return launch_check("itk_finalize_repair_kernel");
}

int itk_merge_candidate_lists(const uint64_t* const* source_pairs, const int32_t* const* source_counts,
                              int sources, int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts, int rows,
                              itk_stream_t stream) {
    return itk_merge_shard_lists(source_pairs, source_counts, sources, out_ids, out_pairs, out_counts, rows, nullptr,
                                 nullptr, nullptr, nullptr, 0, 0, 0, 1, 0, nullptr, nullptr, stream);
}

int itk_merge_shard_lists(const uint64_t* const* source_pairs, const int32_t* const* source_counts, int sources,
                          int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts, int rows,
                          const uint8_t* shard_flags, uint8_t* failure_flags, const int32_t* k_start,
                          const int32_t* k_end, int key_lo, int key_hi, int block_begin, int block_stride,
                          int num_blocks, const int32_t* out_rows, int32_t* mirror_ids, itk_stream_t stream) {
    ITK_REQUIRE(source_pairs && source_counts, "source tables must not be null");
    ITK_REQUIRE(failure_flags == nullptr || (shard_flags && k_start && k_end && key_hi > key_lo && key_lo >= 0),
                "a row verdict needs shard_flags, k_start, k_end and 0 <= key_lo < key_hi");
    ITK_REQUIRE(sources >= 1 && sources <= kMaxPairSources, "need 1 <= sources <= %d", kMaxPairSources);
    ITK_REQUIRE(out_ids != nullptr || out_pairs != nullptr, "need out_ids or out_pairs");
    ITK_REQUIRE(rows > 0, "need rows > 0");
    const int total_blocks = (rows + kBlockQ - 1) / kBlockQ;
    ITK_REQUIRE(block_stride >= 1 && block_begin >= 0 && num_blocks >= 0 &&
                    (num_blocks == 0 || block_begin + static_cast<long long>(num_blocks - 1) * block_stride < total_blocks),
                "owned query blocks must lie inside the %d blocks of the problem", total_blocks);
    int device = 0;
    const int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    PairTopKParams params{};
    for (int s = 0; s < sources; ++s) {
        ITK_REQUIRE(source_pairs[s] && source_counts[s], "source %d has a null pointer", s);
        params.sources[s] = PairSource{source_pairs[s], source_counts[s], kTopK};
    }
    params.num_sources = sources;
    params.rows = rows;
    params.block_begin = block_begin;
    params.block_stride = block_stride;
    params.owned_blocks = num_blocks;
    params.out_rows = out_rows;
    params.mirror_ids = out_ids != nullptr ? mirror_ids : nullptr;
    params.out_ids = out_ids;
    params.out_pairs = out_pairs;
    params.out_counts = out_counts;
    params.verdict_flags = failure_flags;
    params.shard_flags = shard_flags;
    params.k_start = k_start;
    params.k_end = k_end;
    params.key_lo = key_lo;
    params.key_hi = key_hi;
    const int items = num_blocks > 0 ? num_blocks * kBlockQ : rows;
    // The shards of one launch share the row's threshold, so their union is about as large as the
    // candidate set of an unsharded row (some 3 to 5 thousand pairs): a small staging area lets three
    // CTAs share an SM, and the rare row that exceeds it is flagged and goes to the retry.  Merges
    // without that way out (no verdict, or the retry's own merge) get room for every list in full.
    int capacity = sources * kTopK < kPairCapacity ? sources * kTopK : kPairCapacity;
    if (failure_flags != nullptr && out_rows == nullptr && capacity > kShardMergeCapacity) capacity = kShardMergeCapacity;
    params.stage_capacity = capacity;
    const size_t smem = static_cast<size_t>(capacity) * sizeof(uint64_t);
    const int per_sm = smem <= 72 * 1024 ? 3 : (smem <= 110 * 1024 ? 2 : 1);   // the kernel is built for 3 CTAs of 512 threads per SM
    int grid = g_sm_count[device] * per_sm;
    if (grid > items) grid = items;
    itk_pair_topk_kernel<<<grid, kPairThreads, smem, stream>>>(params);
    return launch_check("itk_pair_topk_kernel (lists)");
}

int itk_flagged_scope_begin(const uint8_t* failure_flags, int rows, itk_stream_t stream, itk_stream_t* body_stream) {
    ITK_REQUIRE(failure_flags != nullptr && rows > 0 && body_stream != nullptr, "need failure_flags, rows > 0 and body_stream");
    *body_stream = stream;   // outside a capture, or when a step below is refused: the launches run as they are
    int device = 0;
    const int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    cudaGraph_t graph = nullptr;
    const cudaGraphNode_t* dependencies = nullptr;
    size_t count = 0;
    ITK_CUDA(cudaStreamGetCaptureInfo_v2(stream, &status, nullptr, &graph, &dependencies, &count));
    if (status != cudaStreamCaptureStatusActive || g_body_stream[device] == nullptr) return ITK_OK;
    cudaGraphConditionalHandle condition;
    if (cudaGraphConditionalHandleCreate(&condition, graph, 0, cudaGraphCondAssignDefault) != cudaSuccess) {
        (void)cudaGetLastError();   // no conditional nodes here: stay unconditional
        return ITK_OK;
    }
    // from here on the capture is being changed: a failure is an error of the call
    itk_any_flag_kernel<<<1, 256, 0, stream>>>(condition, failure_flags, rows);
    const int launched = launch_check("itk_any_flag_kernel");
    if (launched != ITK_OK) return launched;
    ITK_CUDA(cudaStreamGetCaptureInfo_v2(stream, &status, nullptr, &graph, &dependencies, &count));
    cudaGraphNodeParams node_params{};
    node_params.type = cudaGraphNodeTypeConditional;
    node_params.conditional.handle = condition;
    node_params.conditional.type = cudaGraphCondTypeIf;
    node_params.conditional.size = 1;
    cudaGraphNode_t node = nullptr;
    ITK_CUDA(cudaGraphAddNode(&node, graph, dependencies, count, &node_params));
    // what the caller enqueues on `stream` after the scope comes after the conditional node
    ITK_CUDA(cudaStreamUpdateCaptureDependencies(stream, &node, 1, cudaStreamSetCaptureDependencies));
    cudaGraph_t body = node_params.conditional.phGraph_out[0];
    ITK_CUDA(cudaStreamBeginCaptureToGraph(g_body_stream[device], body, nullptr, nullptr, 0, cudaStreamCaptureModeRelaxed));
    *body_stream = g_body_stream[device];
    return ITK_OK;
}

int itk_flagged_scope_end(itk_stream_t stream, itk_stream_t body_stream) {
    if (body_stream == stream || body_stream == nullptr) return ITK_OK;
    cudaGraph_t body = nullptr;
    ITK_CUDA(cudaStreamEndCapture(body_stream, &body));
    return ITK_OK;
}

int itk_compact_flagged_rows(const uint8_t* failure_flags, const void* q, const float* weights, const int32_t* k_start,
                             const int32_t* k_end, int rows, int slots, void* q_out, float* weights_out,
                             int32_t* k_start_out, int32_t* k_end_out, int32_t* slot_rows, itk_stream_t stream) {
    ITK_REQUIRE(failure_flags && q && weights && k_start && k_end && q_out && weights_out && k_start_out && k_end_out &&
                    slot_rows,
                "compaction pointers must not be null");
    ITK_REQUIRE(rows > 0 && slots > 0 && slots <= 4096, "need rows > 0 and 0 < slots <= 4096");
    ITK_REQUIRE(aligned16(failure_flags) && aligned16(q) && aligned16(q_out),
                "failure_flags, q and q_out must be 16-byte aligned");
    itk_compact_flagged_kernel<<<slots, kCompactThreads, 0, stream>>>(
        failure_flags, rows, static_cast<const uint4*>(q), weights, k_start, k_end, static_cast<uint4*>(q_out),
        weights_out, k_start_out, k_end_out, slot_rows);
    return launch_check("itk_compact_flagged_kernel");
}

int itk_repair_merge_chunk(uint64_t* accumulator_pairs, int32_t* accumulator_counts, const uint64_t* repair_pairs,
                           const int32_t* k_start, const int32_t* k_end, int chunk_lo, int chunk_hi,
                           uint8_t* failure_flags, uint8_t* repair_error_flags, int rows, int first_chunk,
                           int last_chunk, int32_t* out_ids, uint64_t* out_pairs, int32_t* out_counts,
                           int32_t* mirror_ids, itk_stream_t stream) {
    ITK_REQUIRE(accumulator_pairs && accumulator_counts && repair_pairs && k_start && k_end && failure_flags &&
                    repair_error_flags,
                "repair merge pointers must not be null");
    ITK_REQUIRE(rows > 0, "need rows > 0");
    ITK_REQUIRE(chunk_lo >= 0 && chunk_hi > chunk_lo && chunk_hi - chunk_lo <= kRepairChunk,
                "need a chunk of at most %d keys", kRepairChunk);
    ITK_REQUIRE(!last_chunk || out_ids != nullptr || out_pairs != nullptr, "the last chunk needs out_ids or out_pairs");
    int device = 0;
    const int rc = init_current_device(&device);
    if (rc != ITK_OK) return rc;
    PairTopKParams params{};
    params.sources[0] = PairSource{accumulator_pairs, accumulator_counts, kTopK};
    params.sources[1] = PairSource{repair_pairs, nullptr, kRepairChunk};
    params.num_sources = 2;
    params.first_source = first_chunk ? 1 : 0;
    params.rows = rows;
    params.row_mask = failure_flags;
    params.error_flags = repair_error_flags;
    params.clear_errors = first_chunk ? 1 : 0;
    params.k_start = k_start;
    params.k_end = k_end;
    params.dense_lo = chunk_lo;
    params.dense_hi = chunk_hi;
    params.error_count_mismatch = ITK_REPAIR_ERR_COUNT;
    params.error_selection = ITK_REPAIR_ERR_MERGE_SELECT;
    if (last_chunk) {
        // the result of the last chunk is the row's answer: it goes to the operator output and a full
        // result clears the row's failure flag
        params.out_ids = out_ids;
        params.mirror_ids = out_ids != nullptr ? mirror_ids : nullptr;
        params.out_pairs = out_pairs;
        params.out_counts = out_counts;
        params.clear_flags = failure_flags;
    } else {
        params.out_pairs = accumulator_pairs;
        params.out_counts = accumulator_counts;
    }
    params.stage_capacity = kPairCapacity;
    itk_pair_topk_kernel<<<pair_grid(device, rows), kPairThreads, kPairSmemBytes, stream>>>(params);
    return launch_check("itk_pair_topk_kernel (chunk merge)");
}

}  // extern "C"

// ---------------------------------------------------------------- no-allocation variant

namespace {

constexpr int kStaticMaxRows = ITK_STATIC_MAX_ROWS;

// Spill scratch of the no-allocation entry point: part of the library image, one copy per
// device context.  In host code this name is only a handle; the kernel must be given the
// device address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned long long g_static_spill[static_cast<size_t>(kStaticMaxRows) * itk::kSpillRow];

std::mutex g_static_mutex;
uint64_t* g_static_spill_address[kMaxDevices] = {};

}  // namespace

extern "C" int itk_fused_topk_static(const itk_fused_args* args, itk_stream_t stream) {
    ITK_REQUIRE(args != nullptr, "args must not be null");
    ITK_REQUIRE(args->spill == nullptr, "the no-allocation variant owns its spill; pass spill = null");
    ITK_REQUIRE(args->rows > 0 && args->rows <= kStaticMaxRows,
                "the no-allocation variant handles at most %d query rows per call (got %d); split the call by rows",
                kStaticMaxRows, args->rows);
    ITK_REQUIRE(args->shards == 1, "the no-allocation variant does not offer key-range shards");
    int device = 0;
    ITK_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(ITK_ERR_UNSUPPORTED, "device index %d out of range", device);
    uint64_t* spill = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (g_static_spill_address[device] == nullptr) {
            // once per device, with that device current: resolve the symbol to a device address
            void* address = nullptr;
            ITK_CUDA(cudaGetSymbolAddress(&address, g_static_spill));
            if (address == nullptr) return fail(ITK_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
            g_static_spill_address[device] = static_cast<uint64_t*>(address);
        }
        spill = g_static_spill_address[device];
    }
    itk_fused_args with_spill = *args;
    with_spill.spill = spill;
    return itk_fused_topk(&with_spill, stream);
}
