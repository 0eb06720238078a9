// Thin inline-PTX wrappers for the sm_100a features the fused kernel uses:
// mbarrier, TMA (tiled and untiled bulk copies into this CTA's shared memory),
// tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads) and packed fp32 math.
// Every wait on an mbarrier is bounded: it gives up after a wall-clock limit and
// reports failure instead of spinning forever.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace itk {

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    return now;
}

// ------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// One probe of the barrier.  The thread may be parked by the hardware until the phase
// completes or the time hint (nanoseconds) runs out, whichever comes first, so a waiting
// thread does not spend issue slots on a hot spin loop.
constexpr uint32_t kWaitParkNs = 20000;

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t park_ns = kWaitParkNs) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(park_ns)
        : "memory");
    return done != 0;
}

// Non-blocking probe, for waits that sit on the critical path (the wake-up from a parked
// probe costs more than the hand-off it waits for).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Default wall-clock limit of one wait.  The longest legitimate wait is the UMMA issuer or the
// TMA producer waiting out the Top-K selection at the end of a unit (microseconds).
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Waits for the phase with the given parity.  Returns false when limit_ns
// expired or another thread of the CTA already gave up (*abort_flag != 0); the
// caller then leaves its role loop.  PARK_NS = 0 polls without parking, otherwise a
// failed probe suspends the thread for up to PARK_NS nanoseconds.
constexpr uint32_t kHotWait = 0;

template <uint32_t PARK_NS = kWaitParkNs>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
    constexpr bool kHot = PARK_NS == kHotWait;
    if (mbar_test_wait(bar, parity)) return true;
    uint64_t deadline = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (kHot ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity, PARK_NS)) return true;
        if ((spin & (kHot ? 1023u : 15u)) == 0u) {
            if (*abort_flag != 0) return false;
            const uint64_t now = global_timer_ns();
            if (deadline == 0) {
                deadline = now + limit_ns;
            } else if (now > deadline) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Makes a value opaque to the compiler, which then keeps it in a register instead of
// recomputing it from its inputs at every use inside a hot loop.
__device__ __forceinline__ void keep_in_register(int& value) { asm volatile("" : "+r"(value)); }
__device__ __forceinline__ void keep_in_register(unsigned& value) { asm volatile("" : "+r"(value)); }
__device__ __forceinline__ void keep_in_register(float& value) { asm volatile("" : "+f"(value)); }

// Mask of the lanes below the calling one.
__device__ __forceinline__ uint32_t lanemask_lt() {
    uint32_t mask;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
    return mask;
}

// Stores through a 32-bit shared-memory address (no generic address arithmetic).
__device__ __forceinline__ void st_shared_u32(uint32_t address, uint32_t value) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}

__device__ __forceinline__ void st_shared_u16(uint32_t address, uint32_t value) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(address), "h"(static_cast<uint16_t>(value)) : "memory");
}

// Shared-memory add without a return value.
__device__ __forceinline__ void red_shared_add_u32(uint32_t address, uint32_t value) {
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}

// ------------------------------------------------------------------ TMA

// Tiled 2-D load of one box into this CTA's shared memory; completion is
// signalled as transaction bytes on `bar`.  c0 is the innermost (byte) coordinate
// and must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t c0,
                                            int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* global_src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(global_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes `bar` receive one arrival once every tcgen05 operation this thread
// issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128
// bytes long and stored with the 128-byte swizzle (the layout a 128-byte-wide
// TMA box with SWIZZLE_128B produces).  Eight-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128_kmajor(uint32_t smem_address) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_address & 0x3FFFFu) >> 4);  // start address, 16-byte units
    desc |= static_cast<uint64_t>(1) << 16;                          // leading byte offset (unused here)
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset: 8 rows * 128 B
    desc |= static_cast<uint64_t>(1) << 46;                          // descriptor version of sm_100
    desc |= static_cast<uint64_t>(2) << 61;                          // SWIZZLE_128B
    return desc;
}

// Instruction descriptor of kind::f8f6f4 with e4m3 A and B (both K-major) and fp32 D.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(uint32_t m, uint32_t n) {
    return (1u << 4)            // D format: F32
           | (0u << 7)          // A format: E4M3
           | (0u << 10)         // B format: E4M3
           | (0u << 15)         // A K-major
           | (0u << 16)         // B K-major
           | ((n >> 3) << 17)   // N / 8
           | ((m >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]^T, one UMMA of shape M x N x 32 (fp8).
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane (lane = 32*(warp%4) + laneid).
__device__ __forceinline__ void tmem_load_32(uint32_t tmem_address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(tmem_address)
        : "memory");
}

// 16 TMEM lanes x 64 fp32 columns in the 16x256b fragment layout: thread t of the warp gets,
// for n = 0..7, r[4n], r[4n+1] = (lane t/4, columns 8n + 2(t%4) + {0,1}) and
// r[4n+2], r[4n+3] = (lane t/4 + 8, same columns).  The lane field of the address selects
// the 16-lane half inside the warp's own 32-lane quarter.
__device__ __forceinline__ void tmem_load_frag(uint32_t tmem_address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(tmem_address)
        : "memory");
}

// Half-width fragment: 16x256b.x4 = 32 columns, 16 registers (thread t: r[4n], r[4n+1] = lane t/4,
// columns 8n + 2(t%4) + {0,1}; r[4n+2], r[4n+3] = lane t/4 + 8, same columns; n = 0..3).
__device__ __forceinline__ void tmem_load_frag16(uint32_t tmem_address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(tmem_address)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15])
                 :
                 : "memory");
}

// Waits for this thread's outstanding TMEM loads.  The registers are listed as
// read-write operands so that no use of them is scheduled above the wait.
__device__ __forceinline__ void tmem_load_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// ------------------------------------------------------------------ packed fp32

// d = a * b + c on two fp32 lanes at once (sm_100 packed FMA).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    uint64_t ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// ------------------------------------------------------------------ score bits

// Monotone uint32 image of a float: -0 reads as +0, negatives are inverted,
// non-negatives get the sign bit set.  Larger score <=> larger integer.
__host__ __device__ __forceinline__ uint32_t ordered_bits(float value) {
#ifdef __CUDA_ARCH__
    // adding +0 turns -0 into +0 and leaves every other value alone; the sign then selects the flip mask
    const uint32_t bits = __float_as_uint(value + 0.0f);
    return bits ^ (static_cast<uint32_t>(static_cast<int32_t>(bits) >> 31) | 0x80000000u);
#else
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    if ((bits & 0x7fffffffu) == 0u) bits = 0u;
    return (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
#endif
}

__host__ __device__ __forceinline__ float ordered_to_float(uint32_t ordered) {
    const uint32_t bits = (ordered & 0x80000000u) ? (ordered ^ 0x80000000u) : ~ordered;
#ifdef __CUDA_ARCH__
    return __uint_as_float(bits);
#else
    float value;
    memcpy(&value, &bits, sizeof(value));
    return value;
#endif
}

__host__ __device__ __forceinline__ uint64_t pack_score_id(float score, uint32_t id) {
    return (static_cast<uint64_t>(ordered_bits(score)) << 32) | id;
}

}  // namespace itk
