// Row-wise e4m3 quantisation of the operator's inputs on the device.
//
// The reference quantises the index keys with torch before the operator runs
// (src/fused_index_topk/inputs.py:76-90): per 128-element row
//     scale = max(amax(|x|), 1e-4) / 448        (fp32)
//     value = e4m3(x / scale)                   (IEEE fp32 division, round to nearest even)
// This kernel does the same arithmetic in one pass over HBM, for fp32 or bf16
// sources, and can fold the row scale into a second vector
// (folded[row] = fold[row] * scale[row]): the operator takes no query scale, so
// quantised queries carry theirs inside the head weights.
//
// Layout: eight lanes share a row.  Load i of lane l takes the 16-byte vector
// i*8 + l of the row, so that every load instruction of a warp reads four rows
// as four fully used 128-byte lines, and the matching store writes whole 32-byte
// sectors.  The kernel is bound by HBM: 4 (or 2) bytes read and 1 byte written
// per element.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

#include "itk_ptx.cuh"

namespace itk {

constexpr int kQuantDim = 128;   // elements per row (the index head dimension)
constexpr int kQuantRowLanes = 8;
constexpr int kQuantThreads = 256;
constexpr int kQuantRowsPerBlock = kQuantThreads / kQuantRowLanes;
constexpr float kE4m3Max = 448.0f;
constexpr float kQuantAmaxFloor = 1e-4f;

// Two floats -> two e4m3 bytes (first argument in the low byte), round to nearest even.
__device__ __forceinline__ uint32_t e4m3x2(float low, float high) {
    uint16_t packed;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(high), "f"(low));
    return packed;
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    return e4m3x2(a, b) | (e4m3x2(c, d) << 16);
}

__device__ __forceinline__ uint4 load_stream16(const void* address) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(address));
    return v;
}

// Correctly rounded x / scale for the 16 elements a lane divides by the same scale, at
// three instructions each instead of a full IEEE division.  With r = RN(1/scale),
// q0 = RN(x*r) lies within one ulp of x/scale, the FMA gives the remainder
// x - q0*scale exactly, and RN(q0 + remainder*r) is then the correctly rounded
// quotient (Markstein's theorem on FMA division).  The remainder is exact while it is
// a normal number, which holds for |x| >= 2^-100; below that the quotient is smaller
// than 2^-78 (scale >= 1e-4/448) and every value in reach encodes to a signed e4m3
// zero, so the e4m3 result equals that of the IEEE division for every finite input.
struct RowDivisor {
    float scale, reciprocal;
    __device__ __forceinline__ float quotient(float x) const {
        const float q0 = __fmul_rn(x, reciprocal);
        const float remainder = __fmaf_rn(-q0, scale, x);
        // a zero remainder added to -0 would give +0: the quotient has the sign of x (scale > 0)
        return copysignf(__fmaf_rn(remainder, reciprocal, q0), x);
    }
};

__device__ __forceinline__ RowDivisor make_row_divisor(float scale) {
    RowDivisor divisor;
    divisor.scale = scale;
    divisor.reciprocal = __fdiv_rn(1.0f, scale);
    return divisor;
}

template <typename Source>
struct QuantSource;

template <>
struct QuantSource<float> {
    static constexpr int kVector = 4;  // elements per 16-byte load
    static __device__ __forceinline__ void unpack(const uint4& raw, float* out) {
        out[0] = __uint_as_float(raw.x);
        out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z);
        out[3] = __uint_as_float(raw.w);
    }
};

template <>
struct QuantSource<__nv_bfloat16> {
    static constexpr int kVector = 8;
    static __device__ __forceinline__ void unpack(const uint4& raw, float* out) {
        const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(words[i] << 16);
            out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
        }
    }
};

template <typename Source>
__global__ void __launch_bounds__(kQuantThreads)
itk_quantize_rows_kernel(const Source* __restrict__ source, const float* __restrict__ fold,
                         float* __restrict__ folded, uint8_t* __restrict__ values, float* __restrict__ scales,
                         long long rows) {
    constexpr int kVector = QuantSource<Source>::kVector;
    constexpr int kLoads = kQuantDim / (kVector * kQuantRowLanes);
    const int lane = threadIdx.x % kQuantRowLanes;
    const long long row = static_cast<long long>(blockIdx.x) * kQuantRowsPerBlock + threadIdx.x / kQuantRowLanes;
    const bool live = row < rows;

    float x[kLoads][kVector];
    float amax = 0.0f;
    if (live) {
        const uint4* row_vectors = reinterpret_cast<const uint4*>(source + row * kQuantDim);
        uint4 raw[kLoads];
#pragma unroll
        for (int i = 0; i < kLoads; ++i) raw[i] = load_stream16(row_vectors + i * kQuantRowLanes + lane);
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            QuantSource<Source>::unpack(raw[i], x[i]);
#pragma unroll
            for (int j = 0; j < kVector; ++j) amax = fmaxf(amax, fabsf(x[i][j]));
        }
    }
    // the eight lanes of a row are neighbours inside one warp
#pragma unroll
    for (int step = 1; step < kQuantRowLanes; step <<= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, step));
    if (!live) return;

    const float scale = __fdiv_rn(fmaxf(amax, kQuantAmaxFloor), kE4m3Max);
    const RowDivisor divisor = make_row_divisor(scale);
    uint8_t* row_values = values + row * kQuantDim;
#pragma unroll
    for (int i = 0; i < kLoads; ++i) {
        uint32_t packed[kVector / 4];
#pragma unroll
        for (int j = 0; j < kVector / 4; ++j)
            packed[j] = e4m3x4(divisor.quotient(x[i][4 * j]), divisor.quotient(x[i][4 * j + 1]),
                               divisor.quotient(x[i][4 * j + 2]), divisor.quotient(x[i][4 * j + 3]));
        uint8_t* target = row_values + (i * kQuantRowLanes + lane) * kVector;
        if constexpr (kVector == 4) {
            *reinterpret_cast<uint32_t*>(target) = packed[0];
        } else {
            *reinterpret_cast<uint2*>(target) = make_uint2(packed[0], packed[1]);
        }
    }
    if (lane == 0) {
        if (scales != nullptr) scales[row] = scale;
        if (folded != nullptr) folded[row] = fold[row] * scale;
    }
}

}  // namespace itk
