#pragma once
// UMMA (tcgen05.mma) descriptor construction and the CTA role layout.
// Takes the place of the reference's WGMMA selector and thread-count helpers
// (yan/include/gemm/mma_utils.cuh:17-84): instead of one 64xNx32 WGMMA atom per math
// warpgroup writing registers, ONE thread issues 128xNx32 `kind::f8f6f4` MMAs whose fp32
// accumulator lives in tensor memory; the math warpgroups become promotion warpgroups.

#include <cstdint>

#include "utils.cuh"

namespace yan {

// --- CTA role layout -------------------------------------------------------------------------
// warp 0      : TMA producer (one elected lane)
// warp 1      : MMA issuer   (one elected lane)
// warp 2      : TMEM allocator / deallocator
// warp 3      : spare (keeps the first four warps a full warpgroup for setmaxnreg)
// warps 4..   : promotion/epilogue warpgroups; warpgroup h owns output columns
//               [h*BLOCK_N/G, (h+1)*BLOCK_N/G) of the tile, warp (w%4) owns TMEM lanes 32*(w%4)..+31.
// G = 2 everywhere.  G = 4 (sixteen promotion warps, 64 columns each, 112 registers) was measured slower
// for BLOCK_N = 256 (851 vs 805 cycles per k-block): all promotion warps are released by the same barrier, so
// they load TMEM in lockstep and then issue FMAs in lockstep, and extra warps add contention, not overlap.
constexpr uint32_t kNumControlThreads = 128;
constexpr uint32_t kNumMathThreadsPerGroup = 128;

#ifndef YAN_NUM_MATH_WARPGROUPS
#define YAN_NUM_MATH_WARPGROUPS 2
#endif
__host__ __device__ constexpr uint32_t get_num_math_warpgroups(uint32_t block_n) {
    return (YAN_NUM_MATH_WARPGROUPS == 4 && block_n % 64 == 0) ? 4 : 2;
}

template <uint32_t kNumTMAThreads = kNumControlThreads, uint32_t kNumMathThreads = kNumMathThreadsPerGroup>
__host__ __device__ constexpr uint32_t get_num_threads_per_sm(uint32_t block_n) {
    static_assert(kNumMathThreads == 128, "a promotion warpgroup is 128 threads (4 TMEM lane quarters)");
    return get_num_math_warpgroups(block_n) * kNumMathThreads + kNumTMAThreads;
}

// Registers after setmaxnreg (the mechanism of fp8_gemm.cuh:171-181 in the reference).  The pool that
// setmaxnreg.inc draws from is what the CTA was given at launch (registers per thread at launch x threads),
// NOT the whole register file: an increase that the control warpgroup's decrease does not cover blocks
// forever.  Launch allocation = floor(65536 / threads / 8) * 8 registers per thread.
//   2 math warpgroups: launch 168 x 384; 128*40 + 256*232 = 64512 = 168*384
//   4 math warpgroups: launch  96 x 640; 128*32 + 512*112 = 61440 =  96*640
__host__ __device__ constexpr uint32_t get_num_launch_registers(uint32_t block_n) {
    return (65536u / get_num_threads_per_sm<>(block_n)) / 8u * 8u;
}
__host__ __device__ constexpr uint32_t get_num_control_registers(uint32_t block_n) {
    return get_num_math_warpgroups(block_n) == 4 ? 32 : 40;
}
__host__ __device__ constexpr uint32_t get_num_math_registers(uint32_t block_n) {
    return get_num_math_warpgroups(block_n) == 4 ? 112 : 232;
}

template <uint32_t BLOCK_N>
struct RegisterBudgetCheck {
    static constexpr uint32_t launch = get_num_launch_registers(BLOCK_N);
    static constexpr uint32_t freed = kNumControlThreads * (launch - get_num_control_registers(BLOCK_N));
    static constexpr uint32_t wanted =
        get_num_math_warpgroups(BLOCK_N) * kNumMathThreadsPerGroup * (get_num_math_registers(BLOCK_N) - launch);
    static_assert(wanted <= freed, "setmaxnreg.inc would wait forever: the decrease does not cover the increase");
    static constexpr bool ok = true;
};

// --- instruction descriptor (32 bit) for tcgen05.mma kind::f8f6f4 ------------------------------
//  [4,6)  accumulator format: 1 = fp32
//  [7,10) A format: 0 = e4m3      [10,13) B format: 0 = e4m3
//  [15]   A major: 0 = K-major    [16]    B major: 0 = K-major
//  [17,23) N >> 3                 [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_instr_desc_e4m3_f32(uint32_t umma_m, uint32_t umma_n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

// --- shared-memory matrix descriptor (64 bit), K-major operand, 128-byte swizzle ---------------
// The tile is rows x 128 bytes, written by TMA with CU_TENSOR_MAP_SWIZZLE_128B into a 1024-byte
// aligned buffer: 8 rows form one 1024-byte swizzle atom.
//  [0,14)  start address >> 4
//  [16,30) leading-dimension byte offset >> 4 (unused for swizzled K-major; canonical value 1)
//  [32,46) stride byte offset >> 4 = 1024 >> 4 (distance between 8-row groups)
//  [46,48) descriptor version = 1 on sm_100
//  [61,64) layout type: 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t make_smem_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>(1) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

// Advancing by one UMMA K step (32 e4m3 = 32 bytes) inside the 128-byte swizzle row adds
// 32 >> 4 = 2 to the start-address field.
constexpr uint32_t kUmmaK = 32;
constexpr uint32_t kDescKStep = (kUmmaK * 1) >> 4;

}  // namespace yan
