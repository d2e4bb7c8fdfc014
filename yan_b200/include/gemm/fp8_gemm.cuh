#pragma once
// FP8 (e4m3) fine-grained-scaled GEMM for sm_100a:  D[M,N] (bf16 or fp32) = A[M,K] . B[N,K]^T with
//   A scales: one fp32 per (row, 128-wide k-block), stored k-block-major (M contiguous)
//   B scales: one fp32 per 128x128 block, [N/128, K/128] row-major.
//
// This is the kernel the reference leaves unfinished at yan/include/gemm/fp8_gemm.cuh:32-197
// (persistent, warp-specialised, TMA-fed, per-k-block scale promotion), rebuilt for Blackwell:
//   * operands: TMA 2D tiled loads (128-byte swizzle) into a kNumStages-deep shared-memory ring,
//     each CTA loading its own tiles (no cluster multicast);
//   * math: ONE thread issues `tcgen05.mma.kind::f8f6f4` 128 x BLOCK_N x 32; the first MMA of each
//     128-wide k-block overwrites a TMEM accumulator buffer, so a buffer holds exactly one
//     k-block's partial sum  P_kb = A8_kb . B8_kb^T;
//   * promotion: two warpgroups read P_kb from TMEM (`tcgen05.ld`), multiply by
//     sA[row,kb] * sB[n/128,kb] and accumulate in fp32 registers, while the MMA thread already
//     fills the next TMEM buffer (2 or 4 buffers rotate);
//   * epilogue: registers -> bf16 -> global (16-byte stores), overlapped with the next tile's MMAs.
// Every mbarrier wait is bounded: on expiry the kernel records a code in a status word, all roles
// drain, TMEM is freed and the kernel returns normally.

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "mma_utils.cuh"
#include "ptx.cuh"
#include "scheduler.cuh"
#include "tma_utils.cuh"
#include "utils.cuh"

namespace yan {

constexpr uint32_t kBlockM = 128;
constexpr uint32_t kBlockK = 128;

// Device-side view of one launch.
struct GemmParams {
    const float* scales_a;      // [K/128][sa_ld], element (kb, row) at kb * sa_ld + row
    const float* scales_b;      // [groups][ceil(N/128)][K/128]
    const int* grouped_layout;  // Contiguous: [M] group per row (-1 = padding); Masked: [G] valid rows
    void* out;                  // [rows][ldd]
    float* out_scales;          // e4m3 output only: [N/128][out_scales_ld], element (nb, row) at nb * out_scales_ld + row
    uint32_t out_scales_ld;
    uint32_t sa_ld;
    uint32_t ldd;
    uint32_t shape_m;  // Normal/Contiguous: total rows; Masked: rows per group (M_max)
    uint32_t shape_n;
    uint32_t shape_k;
    uint32_t num_groups;
    // Whole-tile launch: only tiles [0, tile_limit) of the scheduler's order are computed (0 = all).
    // Tail launch (kTail instance): CTA b computes k-blocks slice b % tail_slices of tile tail_first_tile + b / tail_slices
    // and writes its fp32 partial tile to slot (b % tail_slices) * tail_tiles + b / tail_slices of `out`.
    uint32_t tile_limit = 0;
    uint32_t tail_first_tile = 0, tail_tiles = 0, tail_slices = 0;
    // Scatter instance (kScatter, K-split over several GPUs): the tile of m-block mb is not stored to `out` but to the
    // staging buffer of the rank that owns it, rank mb % scatter_world, at [scatter_rank][row][col] of that rank's
    // [world][rows][ldd] array; scatter_base[r] is rank r's array as mapped into this process (entry [scatter_rank] is local).
    void* scatter_base[8] = {};
    uint32_t scatter_world = 0, scatter_rank = 0, scatter_rows = 0;
    int* status;  // optional device word: 0 = fine, otherwise (kDeviceTimeout << 8) | site
    unsigned long long timeout_ns;
    // optional: CTA 0 writes {clock64, globaltimer} when it starts and when it ends (4 values), so that the host can
    // derive the SM clock the kernel really ran at (cycles / nanoseconds), which a millisecond-period NVML sample misses
    long long* clock_probe = nullptr;
};

namespace detail {

// Wait on an mbarrier phase with a wall-clock bound.  Returns false when the wait ran out or another
// role already gave up; the caller then leaves its loop.
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             const GemmParams& p, int site) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    // Fast path first: when the phase is already complete (the usual case for the role that bounds the kernel) the
    // timer is never read.
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
#if defined(YAN_PRODUCER_POLL_SLEEP_NS) && YAN_PRODUCER_POLL_SLEEP_NS > 0
        if (site == 1) __nanosleep(YAN_PRODUCER_POLL_SLEEP_NS);  // the TMA producer runs stages ahead: it can poll lazily
#endif
        if ((++spins & 0x3Fu) == 0) {
            if (*abort_flag != 0) return false;
            if (ptx::globaltimer_ns() - t0 > p.timeout_ns) {
                *abort_flag = 1;
                if (p.status != nullptr) atomicCAS(p.status, 0, (static_cast<int>(kDeviceTimeout) << 8) | site);
                return false;
            }
        }
    }
    return true;
}

template <typename out_t, uint32_t kCols>
__device__ __forceinline__ void store_row(out_t* dst, const float (&acc)[kCols], uint32_t n_first, uint32_t shape_n) {
    if constexpr (sizeof(out_t) == 2) {
#pragma unroll
        for (uint32_t j = 0; j < kCols / 8; ++j) {
            if (n_first + j * 8 < shape_n) {
                uint4 v;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[j * 8 + 0], acc[j * 8 + 1]);
                __nv_bfloat162 t1 = __floats2bfloat162_rn(acc[j * 8 + 2], acc[j * 8 + 3]);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[j * 8 + 4], acc[j * 8 + 5]);
                __nv_bfloat162 t3 = __floats2bfloat162_rn(acc[j * 8 + 6], acc[j * 8 + 7]);
                v.x = *reinterpret_cast<uint32_t*>(&t0);
                v.y = *reinterpret_cast<uint32_t*>(&t1);
                v.z = *reinterpret_cast<uint32_t*>(&t2);
                v.w = *reinterpret_cast<uint32_t*>(&t3);
                *reinterpret_cast<uint4*>(dst + j * 8) = v;
            }
        }
    } else {
#pragma unroll
        for (uint32_t j = 0; j < kCols / 4; ++j) {
            if (n_first + j * 4 < shape_n) {
                float4 v = make_float4(acc[j * 4 + 0], acc[j * 4 + 1], acc[j * 4 + 2], acc[j * 4 + 3]);
                *reinterpret_cast<float4*>(dst + j * 4) = v;
            }
        }
    }
}

// Epilogue of the e4m3 output (the next layer's activation operand): the thread holds one whole 1 x 128 group of its
// row, so the per-token-group quantizer runs in registers.  The values are rounded to bf16 first and then quantized
// with the quantizer's own three fp32 operations (amax_c = max(amax, 1e-4); inv = 448 / amax_c; q = e4m3_rne(x * inv);
// scale = amax_c / 448), so that the result is bit-identical to the bf16 GEMM followed by per_token_cast_to_fp8.
__device__ __forceinline__ void store_row_e4m3(uint8_t* dst, float* scale_dst, float (&acc)[128]) {
    float amax = 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < 128; ++j) {
        acc[j] = __bfloat162float(__float2bfloat16_rn(acc[j]));
        amax = fmaxf(amax, fabsf(acc[j]));
    }
    const float amax_c = fmaxf(amax, 1e-4f);
    const float inv = __fdiv_rn(448.0f, amax_c);
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j) {
        uint32_t w[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const float* a = acc + j * 16 + i * 4;
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[0], inv), __fmul_rn(a[1], inv)),
                                                         __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[2], inv), __fmul_rn(a[3], inv)),
                                                         __NV_SATFINITE, __NV_E4M3);
            w[i] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4*>(dst + j * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *scale_dst = __fdiv_rn(amax_c, 448.0f);
}

}  // namespace detail

// Output element type of the quantized-output GEMM: e4m3 codes plus one fp32 scale per (row, 128 columns).
struct E4m3Out {
    uint8_t code;
};

template <uint32_t BLOCK_N, uint32_t kNumStages, bool kWideBoxes = false>
struct GemmSmemLayout {
    static constexpr uint32_t kNumTmemBufs = (BLOCK_N > 128) ? 2 : 4;
    static constexpr uint32_t kTmemColsUsed = kNumTmemBufs * BLOCK_N;
    static constexpr uint32_t kTmemCols =  // allocations are powers of two
        kTmemColsUsed <= 32 ? 32 : kTmemColsUsed <= 64 ? 64 : kTmemColsUsed <= 128 ? 128 : kTmemColsUsed <= 256 ? 256 : 512;
    static constexpr uint32_t SMEM_A_SIZE_PER_STAGE = kBlockM * kBlockK;
    static constexpr uint32_t SMEM_B_SIZE_PER_STAGE = BLOCK_N * kBlockK;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + kNumStages * SMEM_A_SIZE_PER_STAGE;
    // Output staging: every promotion warp owns one 32-row x 64-byte box (2 KB).  A lane writes 64 bytes of its own
    // output row into the box, the warp reads the box back eight rows at a time and stores 64 contiguous bytes per
    // row piece, so that one store instruction covers 8 x 64 bytes instead of 32 x 16 bytes of 32 different lines.
    // kWideBoxes (the scatter instance, whose pieces cross NVLink): 32 rows x 128 bytes per box, so that a store
    // instruction covers 4 x 128 bytes -- whole 128-byte lines on the link instead of half lines.
    static constexpr uint32_t kStoreRowBytes = kWideBoxes ? 128 : 64;
    static constexpr uint32_t kStoreBoxBytes = 32 * kStoreRowBytes;
    static constexpr uint32_t kNumStoreBoxes = 8;
    static constexpr uint32_t kOffStore = kOffB + kNumStages * SMEM_B_SIZE_PER_STAGE;
    static constexpr uint32_t kStoreBytes =
        (kOffStore + kNumStoreBoxes * kStoreBoxBytes + 2048 <= 232448) ? kNumStoreBoxes * kStoreBoxBytes : 0;
    static constexpr uint32_t kOffBarriers = kOffStore + kStoreBytes;
    // ring full/empty, TMEM full/empty per buffer and column half
    static constexpr uint32_t kNumBarriers = 2 * kNumStages + 4 * kNumTmemBufs;
    static constexpr uint32_t kOffTmemSlot = kOffBarriers + kNumBarriers * 8;
    static constexpr uint32_t kOffAbort = kOffTmemSlot + 4;
    // +1024: the dynamic shared-memory base is re-aligned to 1024 bytes inside the kernel.
    static constexpr uint32_t kSmemSize = kOffAbort + 4 + 1024;
    static_assert(kTmemColsUsed <= 512, "tensor memory has 512 columns");
    static_assert(BLOCK_N % 32 == 0 && BLOCK_N >= 32 && BLOCK_N <= 256, "UMMA M=128 needs N % 16 == 0, N <= 256");
};

// Compile-time knobs of the promotion (defaults = the measured best on B200; the others stay selectable for the tuner
// and for measurements):
//   YAN_PROMO_CHUNK        columns per tcgen05.ld (8, 16 or 32).
//   YAN_PROMO_SPLIT_HALVES 1: the MMA thread issues each k-block as two half-width MMA streams (columns [0, N/2) then
//                          [N/2, N)), each with its own TMEM-full / TMEM-empty barrier: warpgroup 0 is released half a
//                          k-block before warpgroup 1 (so the two warps that share an SM sub-partition do not load and
//                          multiply in lockstep) and each half of a TMEM buffer is recycled as soon as its own
//                          warpgroup has read it.  0: one full-width stream, one barrier pair per buffer.
//   YAN_PROMO_EARLY_PROBE  1: the next k-block's TMEM-full barrier is probed (without blocking) right after this
//                          k-block's last load, so that the answer arrives under the last FMAs.
//   YAN_WIDE_STORE_BOXES   1: every instance stages its output in 32 x 128-byte boxes (the scatter instance always does);
//                          for a local output it measured within +-1 % on the large shapes and 3 % slower on
//                          M=8192 N=3584 K=8192, so the default keeps the 64-byte rows and the 16 KB of shared memory.
// Measured and dropped: handing the TMEM read port back and forth between the two warps of a sub-partition through
// mbarriers (an arrive-to-wait hand-over costs ~100 cycles: 778 and 1163 cycles per k-block for 64- and 32-column turns
// against 343 without), and four promotion warpgroups (874 cycles per k-block against 733: the per-k-block bookkeeping
// of sixteen warps fills the issue slots).
#ifndef YAN_PROMO_CHUNK
#define YAN_PROMO_CHUNK 16
#endif
#ifndef YAN_PROMO_SPLIT_HALVES
#define YAN_PROMO_SPLIT_HALVES 0
#endif
#ifndef YAN_TAIL_MIN_K_BLOCKS
#define YAN_TAIL_MIN_K_BLOCKS 96
#endif
#ifndef YAN_PROMO_EARLY_PROBE
#define YAN_PROMO_EARLY_PROBE 0
#endif
#ifndef YAN_WIDE_STORE_BOXES
#define YAN_WIDE_STORE_BOXES 0
#endif

// -DYAN_PHASE_STAMPS: CTA 0 also accumulates, per role, the cycles it spends waiting and working and writes them
// behind the four clock values of GemmParams::clock_probe (the per-SM clock64 stamps of the reference's
// yan/include/flash_attn/flash_attn_tk.cuh:56-63,159-164).  Slots: [4] producer waiting for a free stage,
// [5] MMA thread waiting for operands, [6] MMA thread waiting for a free TMEM buffer, [7] MMA thread total,
// [8] promotion warp 4 waiting for a full TMEM buffer, [9] its TMEM loads, [10] its FMAs (issue time),
// [11] its total, [12] k-blocks it promoted, [13] its epilogue stores.  The clock reads perturb the schedule
// a little: use the flag to see where time goes, not to time the kernel.
#ifdef YAN_PHASE_STAMPS
#define YAN_STAMP(var) const long long var = clock64()
#define YAN_STAMP_ADD(acc, from, to) acc += (to) - (from)
#else
#define YAN_STAMP(var)
#define YAN_STAMP_ADD(acc, from, to)
#endif

// kTail: the instance that finishes a launch whose last wave would be nearly empty.  With T tiles on G CTAs and
// r = T mod G small, the whole-tile instance computes the first T - r tiles (full waves) and this one computes the last
// r: every tile is cut along K into floor(G / r) slices, one CTA per (tile, slice), each writing an fp32 partial tile;
// reduce_tail_partials_kernel then adds a tile's partials in slice order, rounds once and stores.  It is a separate
// instance (and the k-range, tile choice and output slot are compile-time branches) because the code of the hot loop
// is sensitive to everything else the kernel holds: an earlier form that taught the one kernel to cut tiles lost a
// fifth of the whole-tile schedule's speed.
// kScatter: the instance of the row-parallel (K-split) GEMM whose epilogue is the reduce-scatter half of the
// allreduce: every finished bf16 tile goes straight to the rank that will sum it (plain stores to peer-mapped memory,
// 128 contiguous bytes per row piece), while the MMAs of the next tiles run; gather_staged_allreduce_bf16_kernel in
// comm/peer_allreduce.cuh is the other half.  This is the per-tile hand-over of the reference's epilogue (comm/gemm_allreduce.cu:339-410) without NVSHMEM.
template <uint32_t BLOCK_N, uint32_t kNumStages, GemmType kGemmType, typename out_t, bool kTail = false, bool kScatter = false>
__global__ void __launch_bounds__(get_num_threads_per_sm<>(BLOCK_N), 1)
    fp8_gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tensor_map_a,
                    const __grid_constant__ CUtensorMap tensor_map_b) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    using L = GemmSmemLayout<BLOCK_N, kNumStages, (kScatter || YAN_WIDE_STORE_BOXES != 0) && GemmSmemLayout<BLOCK_N, kNumStages, true>::kStoreBytes != 0>;
    using Sched = Scheduler<kGemmType, kBlockM, BLOCK_N>;
    constexpr uint32_t kNumTmemBufs = L::kNumTmemBufs;
    constexpr uint32_t kNumMathWGs = get_num_math_warpgroups(BLOCK_N);
    static_assert(kNumMathWGs == 2 || YAN_PROMO_SPLIT_HALVES == 0, "the half-width streams assume two promotion warpgroups");
    static_assert(RegisterBudgetCheck<BLOCK_N>::ok);
    constexpr uint32_t kColsPerWG = BLOCK_N / kNumMathWGs;
    constexpr uint32_t kNumMathWarps = 4 * kNumMathWGs;
    // Columns move TMEM -> registers in chunks of 32 (the fastest tcgen05.ld shape measured) plus, when BLOCK_N/2 is
    // not a multiple of 32 (BLOCK_N = 224, 160, 96), one chunk of 16.
    static_assert(kColsPerWG % 16 == 0, "a promotion warpgroup owns a multiple of 16 columns");
    static_assert(YAN_PROMO_CHUNK == 8 || YAN_PROMO_CHUNK == 16 || YAN_PROMO_CHUNK == 32);
    constexpr uint32_t kChunk = kColsPerWG < YAN_PROMO_CHUNK ? kColsPerWG : YAN_PROMO_CHUNK;
    constexpr bool kEarlyProbe = (YAN_PROMO_EARLY_PROBE != 0);
    constexpr uint32_t kNumChunks = kColsPerWG / kChunk;
    constexpr uint32_t kTailChunk = kColsPerWG - kNumChunks * kChunk;  // 0 or 16
    static_assert(kTailChunk == 0 || kTailChunk == 16);
    // A warpgroup's column range lies inside one 128-column scale block when it divides 128 or is a multiple of it
    // starting on a block boundary (BLOCK_N = 32, 64, 128, 256).  Otherwise it can straddle one boundary, at a
    // multiple of 16 columns: two B scales per k-block, chosen per group of 16 columns (the case the reference
    // handles for BLOCK_N not dividing BLOCK_K, fp8_gemm.cuh:55-61,149-160).
    constexpr bool kTwoScales = (128 % kColsPerWG != 0) && (kColsPerWG % 128 != 0);
    // k-blocks between the load of a scale and its use (the promotion loop is unrolled by this number).  0 = by tile
    // width: 2 for the wide tiles, whose k-block lasts about as long as an L2 round trip, 4 for the narrow ones.
    // Measured on 256-wide tiles (C4, same box): 4 -> 1736 us, 3 -> 1737 us, 2 -> 1654 us, 1 -> 1680 us on a second box
    // where 2 gave 1692 us; the shorter loop body is what helps.
#ifndef YAN_PROMO_SCALE_DEPTH
#define YAN_PROMO_SCALE_DEPTH 0
#endif
    constexpr uint32_t kScaleDepth = YAN_PROMO_SCALE_DEPTH != 0 ? YAN_PROMO_SCALE_DEPTH : (BLOCK_N >= 128 ? 2 : 4);
    // The wide tiles run a single copy of the loop body and shift the ring instead (C4: 1654 -> 1616 us on one box;
    // with three slots the same form measured 1672 us); YAN_PROMO_SHIFT_RING = 0 / 1 forces either form.
#ifndef YAN_PROMO_SHIFT_RING
#define YAN_PROMO_SHIFT_RING (-1)
#endif
    constexpr bool kShiftRing = YAN_PROMO_SHIFT_RING >= 0 ? (YAN_PROMO_SHIFT_RING != 0) : (kScaleDepth == 2);
    constexpr uint32_t kLoopUnroll = kShiftRing ? 1 : kScaleDepth;
    // bf16 / fp32 output through the staging boxes (see GemmSmemLayout) when a warpgroup's columns are whole 64-byte pieces.
    constexpr bool kStagedStore = L::kStoreBytes != 0 && sizeof(out_t) >= 2 && kNumMathWarps == L::kNumStoreBoxes &&
                                  (kColsPerWG * sizeof(out_t)) % L::kStoreRowBytes == 0;
    constexpr uint32_t kStoreCols = L::kStoreRowBytes / (sizeof(out_t) >= 2 ? sizeof(out_t) : 2);  // columns per box row
    // Half-width MMA streams: each warpgroup's columns are produced and recycled on their own barriers.
    constexpr bool kSplitHalves = (YAN_PROMO_SPLIT_HALVES != 0);
    constexpr uint32_t kNumHalves = kSplitHalves ? 2 : 1;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);

    uint64_t* full_barriers = reinterpret_cast<uint64_t*>(smem + L::kOffBarriers);
    uint64_t* empty_barriers = full_barriers + kNumStages;
    uint64_t* tmem_full_barriers = empty_barriers + kNumStages;            // [buf][half]
    uint64_t* tmem_empty_barriers = tmem_full_barriers + 2 * kNumTmemBufs;  // [buf][half]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffTmemSlot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kOffAbort);

    const uint32_t warp_idx = __shfl_sync(0xffffffffu, threadIdx.x / 32, 0);
    const uint32_t lane_idx = ptx::lane_id();
    const uint32_t num_k_blocks = p.shape_k / kBlockK;
    const uint32_t num_sb_rows = ceil_div(p.shape_n, 128u);
    static_assert(!kTail || (kGemmType == GemmType::Normal && sizeof(out_t) == 4), "the tail instance writes fp32 partials");
    static_assert(!kScatter || (kGemmType == GemmType::Normal && sizeof(out_t) == 2 && !kTail), "the scatter instance writes bf16 tiles");
    // k-blocks [kb_begin, kb_begin + kb_count) of every tile this CTA computes: all of them, or the CTA's slice
    const uint32_t tail_slice = kTail ? blockIdx.x % p.tail_slices : 0u, tail_tile = kTail ? blockIdx.x / p.tail_slices : 0u;
    const uint32_t kb_begin = kTail ? (tail_slice * num_k_blocks) / p.tail_slices : 0u;
    const uint32_t kb_count = kTail ? ((tail_slice + 1) * num_k_blocks) / p.tail_slices - kb_begin : num_k_blocks;
    // next tile of this CTA: the persistent walk, or the tail instance's single tile
    [[maybe_unused]] bool tail_taken = false;
    auto next_tile = [&](Sched& sched, uint32_t& m_block_idx, uint32_t& n_block_idx) -> bool {
        if constexpr (kTail) {
            if (tail_taken || tail_tile >= p.tail_tiles) return false;
            tail_taken = true;
            sched.swizzle(p.tail_first_tile + tail_tile, sched.num_m_blocks, m_block_idx, n_block_idx);
            return true;
        } else {
            return sched.get_next_block(m_block_idx, n_block_idx);
        }
    };

    // A whole-tile launch that is followed by a tail launch lets that one be scheduled at once: its CTAs take the SMs as
    // this kernel's CTAs leave them (they read operands and write scratch only, nothing this kernel produces).
    if (!kTail && p.tile_limit != 0) ptx::grid_dependency_launch_dependents();
    if (warp_idx == 0 && lane_idx == 0) {
        ptx::tma_prefetch_desc(&tensor_map_a);
        ptx::tma_prefetch_desc(&tensor_map_b);
    }
    if (warp_idx == 1 && lane_idx == 0) {
#pragma unroll
        for (uint32_t i = 0; i < kNumStages; ++i) {
            ptx::mbar_init(full_barriers + i, 1);   // producer's arrive.expect_tx
            ptx::mbar_init(empty_barriers + i, 1);  // tcgen05.commit of the MMA thread
        }
#pragma unroll
        for (uint32_t i = 0; i < 2 * kNumTmemBufs; ++i) {
            ptx::mbar_init(tmem_full_barriers + i, 1);                             // tcgen05.commit
            ptx::mbar_init(tmem_empty_barriers + i, kNumMathWarps / kNumHalves);  // one arrival per promotion warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp_idx == 2) {
        ptx::tmem_alloc(tmem_slot, L::kTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clock_probe[0] = clock64();
        p.clock_probe[1] = static_cast<long long>(ptx::globaltimer_ns());
    }

    if (warp_idx < 4) {
        ptx::reg_dealloc<get_num_control_registers(BLOCK_N)>();

        if (warp_idx == 0 && lane_idx == 0) {
            // ------------------------------ TMA producer ------------------------------
            Sched sched(p.shape_m, p.shape_n, p.grouped_layout, p.num_groups);
            if (p.tile_limit != 0) sched.num_blocks = min(sched.num_blocks, p.tile_limit);
            uint32_t m_block_idx, n_block_idx, stage = 0, phase = 0;
            bool alive = true;
            [[maybe_unused]] long long waited_empty = 0;
            while (alive && next_tile(sched, m_block_idx, n_block_idx)) {
                const int group = sched.get_group(m_block_idx);
                if (group < 0) continue;
                const int32_t a_row = static_cast<int32_t>(sched.get_row_base(m_block_idx));
                const int32_t b_row = static_cast<int32_t>(group * p.shape_n + n_block_idx * BLOCK_N);
                for (uint32_t kb = kb_begin; kb < kb_begin + kb_count; ++kb) {
                    YAN_STAMP(w0);
                    if (!detail::bounded_wait(empty_barriers + stage, phase ^ 1, abort_flag, p, 1)) {
                        alive = false;
                        break;
                    }
                    YAN_STAMP(w1);
                    YAN_STAMP_ADD(waited_empty, w0, w1);
                    ptx::mbar_arrive_expect_tx(full_barriers + stage,
                                               L::SMEM_A_SIZE_PER_STAGE + L::SMEM_B_SIZE_PER_STAGE);
                    ptx::tma_load_2d(smem + L::kOffA + stage * L::SMEM_A_SIZE_PER_STAGE, &tensor_map_a,
                                     full_barriers + stage, static_cast<int32_t>(kb * kBlockK), a_row);
                    ptx::tma_load_2d(smem + L::kOffB + stage * L::SMEM_B_SIZE_PER_STAGE, &tensor_map_b,
                                     full_barriers + stage, static_cast<int32_t>(kb * kBlockK), b_row);
                    if (++stage == kNumStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
#ifdef YAN_PHASE_STAMPS
            if (p.clock_probe != nullptr && blockIdx.x == 0) p.clock_probe[4] = waited_empty;
#endif
            if (!alive) {
                // Give copies still in flight time to land before the CTA's shared memory is released.
                const uint64_t t0 = ptx::globaltimer_ns();
                while (ptx::globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
            }
        } else if (warp_idx == 1 && lane_idx == 0) {
            // ------------------------------ MMA issuer ------------------------------
            Sched sched(p.shape_m, p.shape_n, p.grouped_layout, p.num_groups);
            if (p.tile_limit != 0) sched.num_blocks = min(sched.num_blocks, p.tile_limit);
            constexpr uint32_t kUmmaN = BLOCK_N / kNumHalves;
            constexpr uint32_t idesc = make_instr_desc_e4m3_f32(kBlockM, kUmmaN);
            // rows [kUmmaN, BLOCK_N) of the B tile start kUmmaN 128-byte rows further on (whole 8-row swizzle atoms)
            constexpr uint32_t kDescHalfStep = (kUmmaN * kBlockK) >> 4;
            static_assert(kUmmaN % 16 == 0, "UMMA with M = 128 needs N % 16 == 0");
            uint32_t m_block_idx, n_block_idx, stage = 0, phase = 0, buf = 0, buf_phase = 0;
            bool alive = true;
            [[maybe_unused]] long long waited_full = 0, waited_tmem = 0;
            YAN_STAMP(mma_begin);
            while (alive && next_tile(sched, m_block_idx, n_block_idx)) {
                if (sched.get_group(m_block_idx) < 0) continue;
                for (uint32_t kb = 0; kb < kb_count && alive; ++kb) {
                    YAN_STAMP(w0);
                    if (!detail::bounded_wait(full_barriers + stage, phase, abort_flag, p, 2)) {
                        alive = false;
                        break;
                    }
                    YAN_STAMP(w1);
                    YAN_STAMP_ADD(waited_full, w0, w1);
                    const uint64_t a_desc =
                        make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L::kOffA + stage * L::SMEM_A_SIZE_PER_STAGE));
                    const uint64_t b_desc =
                        make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L::kOffB + stage * L::SMEM_B_SIZE_PER_STAGE));
#pragma unroll
                    for (uint32_t h = 0; h < kNumHalves; ++h) {
                        YAN_STAMP(w2);
                        if (!detail::bounded_wait(tmem_empty_barriers + buf * 2 + h, buf_phase ^ 1, abort_flag, p, 3)) {
                            alive = false;
                            break;
                        }
                        YAN_STAMP(w3);
                        YAN_STAMP_ADD(waited_tmem, w2, w3);
                        ptx::tcgen05_fence_after_thread_sync();
                        const uint32_t tmem_d = tmem_base + buf * BLOCK_N + h * kUmmaN;
#pragma unroll
                        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                            ptx::umma_f8f6f4_ss(tmem_d, a_desc + k * kDescKStep, b_desc + h * kDescHalfStep + k * kDescKStep,
                                                idesc, k > 0);
                        if (h + 1 == kNumHalves)
                            ptx::umma_commit(empty_barriers + stage);       // smem stage reusable once these MMAs are done
                        ptx::umma_commit(tmem_full_barriers + buf * 2 + h);  // partial sum of this k-block is complete
                    }
                    if (++stage == kNumStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                    if (++buf == kNumTmemBufs) {
                        buf = 0;
                        buf_phase ^= 1;
                    }
                }
            }
#ifdef YAN_PHASE_STAMPS
            if (p.clock_probe != nullptr && blockIdx.x == 0) {
                p.clock_probe[5] = waited_full;
                p.clock_probe[6] = waited_tmem;
                p.clock_probe[7] = clock64() - mma_begin;
            }
#endif
        }
        __syncwarp();
    } else {
        // ------------------------------ promotion + epilogue warpgroups ------------------------------
        ptx::reg_alloc<get_num_math_registers(BLOCK_N)>();

        const uint32_t wg = (warp_idx - 4) / 4;
        const uint32_t quarter = warp_idx % 4;
        const uint32_t row_in_tile = quarter * 32 + lane_idx;
        const uint32_t col0 = wg * kColsPerWG;
        const uint32_t tmem_lane_base = tmem_base + ((quarter * 32u) << 16) + col0;
        const uint32_t half = kSplitHalves ? wg : 0;

        Sched sched(p.shape_m, p.shape_n, p.grouped_layout, p.num_groups);
        if (p.tile_limit != 0) sched.num_blocks = min(sched.num_blocks, p.tile_limit);
        uint32_t m_block_idx, n_block_idx, buf = 0, buf_phase = 0;
        bool alive = true, next_ready = false;
        float acc[kColsPerWG];
        [[maybe_unused]] long long waited_tmem_full = 0, in_loads = 0, in_fmas = 0, in_stores = 0, promoted = 0;
        YAN_STAMP(promo_begin);

        while (alive && next_tile(sched, m_block_idx, n_block_idx)) {
            const int group = sched.get_group(m_block_idx);
            if (group < 0) continue;
            const uint32_t row = sched.get_row_base(m_block_idx) + row_in_tile;
            const bool row_ok = row < sched.get_row_limit();
            const uint32_t n_first = n_block_idx * BLOCK_N + col0;
            const uint32_t sb_row = min(n_first / 128u, num_sb_rows - 1);
            const float* sa_ptr = p.scales_a + (kTail ? static_cast<size_t>(kb_begin) * p.sa_ld : 0) + row;
            const float* sb_ptr =
                p.scales_b + (static_cast<size_t>(group) * num_sb_rows + sb_row) * num_k_blocks + (kTail ? kb_begin : 0u);
            const float* sa_next = sa_ptr + static_cast<size_t>(kScaleDepth) * p.sa_ld;  // row's scale kScaleDepth k-blocks ahead
            // two-scale case: groups of 16 columns from `hi_from` on belong to the next 128-column block
            const uint32_t hi_from = kTwoScales ? (128u - n_first % 128u) / 16u : 0xFFFFu;
            const float* sb_hi_ptr = p.scales_b +
                                     (static_cast<size_t>(group) * num_sb_rows + min(sb_row + 1, num_sb_rows - 1)) * num_k_blocks +
                                     (kTail ? kb_begin : 0u);

            // Scales are prefetched kScaleDepth k-blocks ahead: one L2 round trip is longer than one k-block.
            float sa_ring[kScaleDepth], sb_ring[kScaleDepth], sb_hi_ring[kTwoScales ? kScaleDepth : 1];
#pragma unroll
            for (uint32_t i = 0; i < kScaleDepth; ++i) {
                sa_ring[i] = (row_ok && i < kb_count) ? __ldg(sa_ptr + static_cast<size_t>(i) * p.sa_ld) : 0.0f;
                sb_ring[i] = (i < kb_count) ? __ldg(sb_ptr + i) : 0.0f;
                if constexpr (kTwoScales) sb_hi_ring[i] = (i < kb_count) ? __ldg(sb_hi_ptr + i) : 0.0f;
            }
#pragma unroll
            for (uint32_t j = 0; j < kColsPerWG; ++j) acc[j] = 0.0f;

            // kShiftRing: one copy of the loop body, the ring of scales moved down one slot per k-block (a few register
            // moves); otherwise the body is unrolled once per ring slot and every copy uses its own slot.
            for (uint32_t kb0 = 0; kb0 < kb_count && alive; kb0 += kLoopUnroll) {
#pragma unroll(kLoopUnroll)
                for (uint32_t i = 0; i < kLoopUnroll; ++i) {
                    const uint32_t kb = kb0 + i;
                    if (!alive || (kLoopUnroll > 1 && kb >= kb_count)) continue;
                    const uint32_t use = kShiftRing ? 0 : i, fill = kShiftRing ? kScaleDepth - 1 : i;
                    const float scale = sa_ring[use] * sb_ring[use];
                    float scale_hi = scale;
                    if constexpr (kTwoScales) scale_hi = sa_ring[use] * sb_hi_ring[use];
                    if constexpr (kShiftRing) {
#pragma unroll
                        for (uint32_t r = 0; r + 1 < kScaleDepth; ++r) {
                            sa_ring[r] = sa_ring[r + 1];
                            sb_ring[r] = sb_ring[r + 1];
                            if constexpr (kTwoScales) sb_hi_ring[r] = sb_hi_ring[r + 1];
                        }
                    }
                    if (kb + kScaleDepth < kb_count) {
                        sa_ring[fill] = row_ok ? __ldg(sa_next) : 0.0f;
                        sa_next += p.sa_ld;
                        sb_ring[fill] = __ldg(sb_ptr + kb + kScaleDepth);
                        if constexpr (kTwoScales) sb_hi_ring[fill] = __ldg(sb_hi_ptr + kb + kScaleDepth);
                    }
                    YAN_STAMP(w0);
                    const bool ok = (kEarlyProbe && next_ready) ||
                                    detail::bounded_wait(tmem_full_barriers + buf * 2 + half, buf_phase, abort_flag, p, 4);
                    if (!__all_sync(0xffffffffu, ok)) {
                        alive = false;
                        continue;
                    }
                    YAN_STAMP(w1);
                    YAN_STAMP_ADD(waited_tmem_full, w0, w1);
                    YAN_STAMP_ADD(promoted, 0, 1);
                    ptx::tcgen05_fence_after_thread_sync();
                    const uint32_t taddr = tmem_lane_base + buf * BLOCK_N;

                    // The TMEM buffer is handed back as soon as the last columns have landed, before their FMAs.
                    // Nothing is scheduled between a tcgen05.ld and its wait: FMAs issued while a load is
                    // outstanding were measured ~10x slower than after it (the load does not overlap with the
                    // issuing warp's own arithmetic), so the overlap has to come from the sibling warp.
                    auto release_buffer = [&]() {
                        ptx::tcgen05_fence_before_thread_sync();
                        __syncwarp();
                        if (lane_idx == 0) ptx::mbar_arrive(tmem_empty_barriers + buf * 2 + half);
                    };
                    auto group_scale = [&](uint32_t group16) { return (kTwoScales && group16 >= hi_from) ? scale_hi : scale; };
#pragma unroll
                    for (uint32_t c = 0; c < kNumChunks; ++c) {
                        uint32_t t[kChunk];
                        YAN_STAMP(l0);
                        ptx::tmem_ld_32x32b<kChunk>(taddr + c * kChunk, t);
                        ptx::tmem_ld_wait<kChunk>(t);
                        YAN_STAMP(l1);
                        YAN_STAMP_ADD(in_loads, l0, l1);
                        if (kTailChunk == 0 && c + 1 == kNumChunks) {
                            release_buffer();
                            if constexpr (kEarlyProbe) {
                                const uint32_t nb = (buf + 1 == kNumTmemBufs) ? 0 : buf + 1;
                                const uint32_t np = (buf + 1 == kNumTmemBufs) ? buf_phase ^ 1 : buf_phase;
                                next_ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(tmem_full_barriers + nb * 2 + half, np));
                            }
                        }
#pragma unroll
                        for (uint32_t j = 0; j < kChunk; ++j) {
                            const float sc = group_scale((c * kChunk + j) / 16);
                            acc[c * kChunk + j] = fmaf(sc, __uint_as_float(t[j]), acc[c * kChunk + j]);
                        }
                        YAN_STAMP(l2);
                        YAN_STAMP_ADD(in_fmas, l1, l2);
                    }
                    if constexpr (kTailChunk != 0) {
                        uint32_t t[16];
                        ptx::tmem_ld_32x32b<16>(taddr + kNumChunks * kChunk, t);
                        ptx::tmem_ld_wait<16>(t);
                        release_buffer();
                        const float sc = group_scale((kNumChunks * kChunk) / 16);
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j)
                            acc[kNumChunks * kChunk + j] = fmaf(sc, __uint_as_float(t[j]), acc[kNumChunks * kChunk + j]);
                    }
                    if (++buf == kNumTmemBufs) {
                        buf = 0;
                        buf_phase ^= 1;
                    }
                }
            }
            YAN_STAMP(s0);
            if (alive && row_ok) {
                if constexpr (sizeof(out_t) == 1 && kColsPerWG != 128) {
                    // the e4m3 output needs one 128-column group per thread (BLOCK_N = 256, two warpgroups): the launcher
                    // refuses every other shape of CTA
                } else if constexpr (sizeof(out_t) == 1) {
                    if (n_first < p.shape_n)
                        detail::store_row_e4m3(
                            reinterpret_cast<uint8_t*>(p.out) + static_cast<size_t>(row) * p.ldd + n_first,
                            p.out_scales + static_cast<size_t>(n_first / 128u) * p.out_scales_ld + row, acc);
                } else if constexpr (!kStagedStore) {
                    out_t* dst = reinterpret_cast<out_t*>(p.out) + static_cast<size_t>(row) * p.ldd + n_first;
                    detail::store_row<out_t, kColsPerWG>(dst, acc, n_first, p.shape_n);
                }
            }
            if constexpr (kStagedStore) {
                if (alive) {
                    // Lane r fills row r (64 bytes; 128 in the wide boxes) of the warp's box; 16-byte chunk j of a row sits
                    // at chunk j ^ ((r / 2) % 4) (j ^ (r % 8) in the wide boxes), which keeps both the row-wise writes and
                    // the read-back free of bank conflicts.
                    constexpr uint32_t kRowBytes = L::kStoreRowBytes, kChunksPerRow = kRowBytes / 16;
                    constexpr uint32_t kRowsPerStore = 32 / kChunksPerRow;  // box rows one store instruction covers
                    auto swizzled = [](uint32_t chunk, uint32_t r) {
                        return kChunksPerRow == 4 ? (chunk ^ ((r >> 1) & 3u)) : (chunk ^ (r & 7u));
                    };
                    const uint32_t box = ptx::smem_u32(smem + L::kOffStore + (warp_idx - 4) * L::kStoreBoxBytes);
                    const uint32_t row_addr = box + lane_idx * kRowBytes;
                    constexpr uint32_t kElemsPerChunk = 16 / sizeof(out_t);
                    // the tail instance writes whole partial tiles into its slot of the scratch: [slot][128][BLOCK_N]
                    const uint32_t tile_row0 =
                        (kTail ? (tail_slice * p.tail_tiles + tail_tile) * kBlockM : sched.get_row_base(m_block_idx)) + quarter * 32u;
                    const uint32_t row_limit = kTail ? 0xFFFFFFFFu : sched.get_row_limit();
                    const uint32_t out_ld = kTail ? BLOCK_N : p.ldd, out_cols = kTail ? BLOCK_N : p.shape_n;
                    const uint32_t n_store = kTail ? col0 : n_first;
                    out_t* out_base = reinterpret_cast<out_t*>(p.out);
                    if constexpr (kScatter)
                        out_base = reinterpret_cast<out_t*>(p.scatter_base[m_block_idx % p.scatter_world]) +
                                   static_cast<size_t>(p.scatter_rank) * p.scatter_rows * p.ldd;
#pragma unroll
                    for (uint32_t pass = 0; pass < kColsPerWG / kStoreCols; ++pass) {
                        __syncwarp();  // the read-back of the previous pass is over
#pragma unroll
                        for (uint32_t j = 0; j < kChunksPerRow; ++j) {
                            const float* a = acc + pass * kStoreCols + j * kElemsPerChunk;
                            uint4 v;
                            if constexpr (sizeof(out_t) == 2) {
                                __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(a[4], a[5]), t3 = __floats2bfloat162_rn(a[6], a[7]);
                                v.x = *reinterpret_cast<uint32_t*>(&t0);
                                v.y = *reinterpret_cast<uint32_t*>(&t1);
                                v.z = *reinterpret_cast<uint32_t*>(&t2);
                                v.w = *reinterpret_cast<uint32_t*>(&t3);
                            } else {
                                v = make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]),
                                               __float_as_uint(a[3]));
                            }
                            ptx::st_shared_v4(row_addr + (swizzled(j, lane_idx) << 4), v);
                        }
                        __syncwarp();
                        // read back: instruction i covers box rows 8i .. 8i+7, lane l -> row 8i + l/4, chunk l%4
                        // (wide boxes: rows 4i .. 4i+3, lane l -> row 4i + l/8, chunk l%8)
                        const uint32_t my_chunk = lane_idx % kChunksPerRow;
                        const uint32_t n_chunk = n_store + pass * kStoreCols + my_chunk * kElemsPerChunk;
#pragma unroll
                        for (uint32_t i = 0; i < 32 / kRowsPerStore; ++i) {
                            const uint32_t r = i * kRowsPerStore + lane_idx / kChunksPerRow;
                            const uint4 v = ptx::ld_shared_v4(box + r * kRowBytes + (swizzled(my_chunk, r) << 4));
                            const uint32_t out_row = tile_row0 + r;
                            if (out_row < row_limit && n_chunk < out_cols)
                                *reinterpret_cast<uint4*>(out_base + static_cast<size_t>(out_row) * out_ld + n_chunk) = v;
                        }
                    }
                }
            }
            YAN_STAMP(s1);
            YAN_STAMP_ADD(in_stores, s0, s1);
        }
#ifdef YAN_PHASE_STAMPS
        if (p.clock_probe != nullptr && blockIdx.x == 0 && warp_idx == 4 && lane_idx == 0) {
            p.clock_probe[8] = waited_tmem_full;
            p.clock_probe[9] = in_loads;
            p.clock_probe[10] = in_fmas;
            p.clock_probe[11] = clock64() - promo_begin;
            p.clock_probe[12] = promoted;
            p.clock_probe[13] = in_stores;
        }
#endif
        __syncwarp();
    }

    // Every role has left its loop (normally or through the bounded-wait path): free tensor memory.
    if constexpr (kTail) {
        // launched programmatically behind the whole-tile kernel: do not complete before that kernel has (the kernel
        // that sums the partials waits for this one only), and let that kernel be scheduled now
        ptx::grid_dependency_launch_dependents();
        ptx::grid_dependency_wait();
    }
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp_idx == 2) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(tmem_base, L::kTmemCols);
    }
    if (p.clock_probe != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        p.clock_probe[2] = clock64();
        p.clock_probe[3] = static_cast<long long>(ptx::globaltimer_ns());
    }
#endif
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct GemmArgs {
    const void* lhs = nullptr;         // e4m3 [rows, K]
    const float* lhs_scales = nullptr; // k-block-major, leading dimension lhs_scales_ld (>= rows)
    uint32_t lhs_scales_ld = 0;
    const void* rhs = nullptr;         // e4m3 [groups * N, K]
    const float* rhs_scales = nullptr; // [groups, ceil(N/128), K/128]
    void* out = nullptr;               // [rows, ldd]
    uint32_t ldd = 0;
    float* out_scales = nullptr;       // e4m3 output only: [N/128, out_scales_ld]
    uint32_t out_scales_ld = 0;
    const int* grouped_layout = nullptr;
    uint32_t m = 0, n = 0, k = 0, num_groups = 1;
    int num_sms = 0;
    int* status = nullptr;
    unsigned long long timeout_ns = 2000000000ull;
    long long* clock_probe = nullptr;  // optional: 4 values written by CTA 0 (see GemmParams)
    // optional scratch (tail_workspace_bytes) that lets a Normal bf16 launch cut the tiles of a nearly empty last wave
    // along K; its contents are rewritten by every launch that uses it, nothing needs to be cleared
    void* tail_workspace = nullptr;
    size_t tail_workspace_bytes = 0;
    // K-split with the reduce-scatter in the epilogue: staging arrays of all ranks (see GemmParams::scatter_base);
    // scatter_world = 0: ordinary output
    void* scatter_base[8] = {};
    uint32_t scatter_world = 0, scatter_rank = 0;
};

// Bytes of scratch a grid of `num_sms` CTAs can use for the tail of a launch of BLOCK_N-wide tiles.
constexpr size_t tail_workspace_bytes(uint32_t num_sms, uint32_t block_n) {
    return static_cast<size_t>(num_sms) * kBlockM * block_n * sizeof(float);
}

// How to finish `tiles` tiles on `grid` CTAs: slices per tile of the last `tiles % grid` tiles, or 0 to run them as one
// more wave of whole tiles.  Cutting pays when that wave would be less than half full, costs at least 5 % of the launch,
// and K is long: the two extra launches and the tail CTAs' prologue and epilogue cost about 25 us, which a wave of
// 64 k-blocks (K = 8192, ~30 us) does not repay and a wave of 144 (K = 18432, ~70 us) does
// (measured on B200: M=4096 N=7168 K=18432 533 -> 505 us; M=8192 N=3584 K=8192 230 -> 232 us).
inline uint32_t choose_tail_slices(uint32_t tiles, uint32_t grid, uint32_t num_k_blocks) {
    const uint32_t rest = tiles % grid;
    if (grid < 2 || tiles < grid || rest == 0 || 2 * rest > grid || num_k_blocks < YAN_TAIL_MIN_K_BLOCKS) return 0;
    const uint32_t waves = tiles / grid + 1;
    if (static_cast<double>(grid - rest) / (static_cast<double>(waves) * grid) < 0.05) return 0;
    uint32_t slices = grid / rest;
    if (slices > num_k_blocks / 3) slices = num_k_blocks / 3;
    return slices >= 2 ? slices : 0;
}

// Adds the fp32 partial tiles of a tail launch in slice order, rounds once and stores bf16.  One thread per 8 columns.
template <uint32_t BLOCK_N>
__global__ void __launch_bounds__(256) reduce_tail_partials_kernel(const float* __restrict__ partials,
                                                                    __nv_bfloat16* __restrict__ out, uint32_t ldd,
                                                                    uint32_t shape_m, uint32_t shape_n, uint32_t first_tile,
                                                                    uint32_t tail_tiles, uint32_t slices) {
    constexpr uint32_t kChunksPerRow = BLOCK_N / 8;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the partial tiles are complete (no-op for an ordinary launch)
    const uint32_t t = blockIdx.x;
    const uint32_t idx = blockIdx.y * 256 + threadIdx.x;
    const uint32_t row = idx / kChunksPerRow, chunk = idx % kChunksPerRow;
    if (row >= kBlockM) return;
    Scheduler<GemmType::Normal, kBlockM, BLOCK_N> sched(shape_m, shape_n);
    uint32_t m_block_idx, n_block_idx;
    sched.swizzle(first_tile + t, sched.num_m_blocks, m_block_idx, n_block_idx);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t sl = 0; sl < slices; ++sl) {
        const float4* src = reinterpret_cast<const float4*>(
            partials + (static_cast<size_t>(sl * tail_tiles + t) * kBlockM + row) * BLOCK_N + chunk * 8);
        const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
        acc[0] += lo.x, acc[1] += lo.y, acc[2] += lo.z, acc[3] += lo.w;
        acc[4] += hi.x, acc[5] += hi.y, acc[6] += hi.z, acc[7] += hi.w;
    }
    const uint32_t out_row = m_block_idx * kBlockM + row, out_col = n_block_idx * BLOCK_N + chunk * 8;
    if (out_row >= shape_m || out_col >= shape_n) return;
    uint4 v;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]), t1 = __floats2bfloat162_rn(acc[2], acc[3]);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]), t3 = __floats2bfloat162_rn(acc[6], acc[7]);
    v.x = *reinterpret_cast<uint32_t*>(&t0);
    v.y = *reinterpret_cast<uint32_t*>(&t1);
    v.z = *reinterpret_cast<uint32_t*>(&t2);
    v.w = *reinterpret_cast<uint32_t*>(&t3);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(out_row) * ldd + out_col) = v;
}

inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <uint32_t BLOCK_N, uint32_t kNumStages, GemmType kGemmType, typename out_t>
struct GemmLauncher {
    using L = GemmSmemLayout<BLOCK_N, kNumStages, YAN_WIDE_STORE_BOXES != 0 && GemmSmemLayout<BLOCK_N, kNumStages, true>::kStoreBytes != 0>;
    static constexpr uint32_t kSmemSize = L::kSmemSize;

    static int launch(const GemmArgs& a, cudaStream_t stream) {
        if (a.lhs == nullptr || a.lhs_scales == nullptr || a.rhs == nullptr || a.rhs_scales == nullptr ||
            a.out == nullptr)
            return kBadArgument;
        if (a.m == 0 || a.n == 0 || a.k == 0 || a.k % kBlockK != 0 || a.n % 16 != 0 || a.num_groups == 0)
            return kBadArgument;
        constexpr uint32_t kVec = 16 / sizeof(out_t);
        if (a.ldd < a.n || a.ldd % kVec != 0 || a.lhs_scales_ld == 0) return kBadArgument;
        if (!is_aligned(a.lhs, 16) || !is_aligned(a.rhs, 16) || !is_aligned(a.out, 16) || !is_aligned(a.lhs_scales, 4) ||
            !is_aligned(a.rhs_scales, 4))
            return kBadArgument;
        if (sizeof(out_t) == 1 &&
            (a.out_scales == nullptr || a.out_scales_ld < a.m || a.n % 128 != 0 || !is_aligned(a.out_scales, 4)))
            return kBadArgument;
        if (kGemmType != GemmType::Normal && a.grouped_layout == nullptr) return kBadArgument;
        if (kGemmType == GemmType::Normal && a.num_groups != 1) return kBadArgument;
        if (a.num_sms <= 0) return kBadArgument;

        int device = 0, max_smem = 0, sm_count = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return kLaunchFailed;
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (static_cast<int>(kSmemSize) > max_smem) return kSmemTooLarge;
        if (a.num_sms > sm_count) return kBadArgument;

        const uint64_t a_rows =
            (kGemmType == GemmType::GroupedMasked) ? static_cast<uint64_t>(a.m) * a.num_groups : a.m;
        const uint64_t b_rows = static_cast<uint64_t>(a.n) * a.num_groups;
        if (a_rows > 0x7fffffffull || b_rows > 0x7fffffffull) return kBadArgument;
        if (kGemmType == GemmType::GroupedMasked ? a.lhs_scales_ld < a_rows : a.lhs_scales_ld < a.m)
            return kBadArgument;

        bool ok = true;
        const CUtensorMap map_a = make_2d_tma_desc_u8_sw128(a.lhs, a_rows, a.k, a.k, kBlockM, ok);
        const CUtensorMap map_b = make_2d_tma_desc_u8_sw128(a.rhs, b_rows, a.k, a.k, BLOCK_N, ok);
        if (!ok) return kTensorMapFailed;

        GemmParams p;
        p.scales_a = a.lhs_scales;
        p.scales_b = a.rhs_scales;
        p.grouped_layout = a.grouped_layout;
        p.out = a.out;
        p.out_scales = a.out_scales;
        p.out_scales_ld = a.out_scales_ld;
        p.sa_ld = a.lhs_scales_ld;
        p.ldd = a.ldd;
        p.shape_m = a.m;
        p.shape_n = a.n;
        p.shape_k = a.k;
        p.num_groups = a.num_groups;
        p.status = a.status;
        p.timeout_ns = a.timeout_ns;
        p.clock_probe = a.clock_probe;

        auto kernel = fp8_gemm_kernel<BLOCK_N, kNumStages, kGemmType, out_t>;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemSize) != cudaSuccess) {
            cudaGetLastError();
            return kSmemTooLarge;
        }
        uint32_t grid = static_cast<uint32_t>(a.num_sms);
        if (kGemmType != GemmType::GroupedMasked) {
            const uint32_t tiles = ceil_div(a.m, kBlockM) * ceil_div(a.n, BLOCK_N);
            grid = tiles < grid ? tiles : grid;
        }
        if constexpr (kGemmType == GemmType::Normal && sizeof(out_t) == 2 && L::kStoreBytes != 0) {
            if (a.scatter_world != 0) {
                // only the widths whose epilogue goes through the staging boxes know the owners' staging arrays
                if (BLOCK_N != 256 && BLOCK_N != 128) return kBadArgument;
                if (a.scatter_world < 2 || a.scatter_world > 8 || a.scatter_rank >= a.scatter_world) return kBadArgument;
                for (uint32_t r = 0; r < a.scatter_world; ++r) {
                    if (a.scatter_base[r] == nullptr || !is_aligned(a.scatter_base[r], 16)) return kBadArgument;
                    p.scatter_base[r] = a.scatter_base[r];
                }
                p.scatter_world = a.scatter_world;
                p.scatter_rank = a.scatter_rank;
                p.scatter_rows = a.m;
                auto scatter_kernel = fp8_gemm_kernel<BLOCK_N, kNumStages, GemmType::Normal, out_t, false, true>;
                // the scatter instance stages its output in wider boxes where they fit (same rule as in the kernel)
                using Wide = GemmSmemLayout<BLOCK_N, kNumStages, true>;
                constexpr uint32_t kScatterSmem = Wide::kStoreBytes != 0 ? Wide::kSmemSize : kSmemSize;
                if (static_cast<int>(kScatterSmem) > max_smem) return kSmemTooLarge;
                if (cudaFuncSetAttribute(scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScatterSmem) != cudaSuccess) {
                    cudaGetLastError();
                    return kSmemTooLarge;
                }
                scatter_kernel<<<grid, get_num_threads_per_sm<>(BLOCK_N), kScatterSmem, stream>>>(p, map_a, map_b);
                return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
            }
        } else {
            if (a.scatter_world != 0) return kBadArgument;
        }
        // A nearly empty last wave: whole tiles for the full waves, then the rest cut along K, then the sum of the cuts.
        if constexpr (kGemmType == GemmType::Normal && sizeof(out_t) == 2 && L::kStoreBytes != 0) {
            const uint32_t tiles = ceil_div(a.m, kBlockM) * ceil_div(a.n, BLOCK_N);
            const uint32_t slices = (a.tail_workspace != nullptr && is_aligned(a.tail_workspace, 16))
                                        ? choose_tail_slices(tiles, grid, a.k / kBlockK) : 0;
            const uint32_t rest = tiles % grid;
            if (slices != 0 && a.tail_workspace_bytes >= static_cast<size_t>(rest) * slices * kBlockM * BLOCK_N * sizeof(float)) {
                auto tail_kernel = fp8_gemm_kernel<BLOCK_N, kNumStages, GemmType::Normal, float, true>;
                if (cudaFuncSetAttribute(tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemSize) != cudaSuccess) {
                    cudaGetLastError();
                    return kSmemTooLarge;
                }
                p.tile_limit = tiles - rest;
                kernel<<<grid, get_num_threads_per_sm<>(BLOCK_N), kSmemSize, stream>>>(p, map_a, map_b);
                GemmParams tail = p;
                tail.tile_limit = 0;
                tail.out = a.tail_workspace;
                tail.tail_first_tile = tiles - rest;
                tail.tail_tiles = rest;
                tail.tail_slices = slices;
                tail.clock_probe = nullptr;
                // both follow-up kernels are launched with programmatic stream serialization: the launch latencies
                // hide behind the kernel before; ordering is kept by the waits inside them
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(rest * slices);
                cfg.blockDim = dim3(get_num_threads_per_sm<>(BLOCK_N));
                cfg.dynamicSmemBytes = kSmemSize;
                cfg.stream = stream;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                if (cudaLaunchKernelEx(&cfg, tail_kernel, tail, map_a, map_b) != cudaSuccess) {
                    cudaGetLastError();
                    return kLaunchFailed;
                }
                cfg.gridDim = dim3(rest, kBlockM * (BLOCK_N / 8) / 256);
                cfg.blockDim = dim3(256);
                cfg.dynamicSmemBytes = 0;
                const float* partials = static_cast<const float*>(a.tail_workspace);
                __nv_bfloat16* out_bf16 = static_cast<__nv_bfloat16*>(a.out);
                const uint32_t first_tile = tiles - rest;
                if (cudaLaunchKernelEx(&cfg, reduce_tail_partials_kernel<BLOCK_N>, partials, out_bf16, a.ldd, a.m, a.n,
                                       first_tile, rest, slices) != cudaSuccess) {
                    cudaGetLastError();
                    return kLaunchFailed;
                }
                return kOk;
            }
        }
        kernel<<<grid, get_num_threads_per_sm<>(BLOCK_N), kSmemSize, stream>>>(p, map_a, map_b);
        return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
    }
};

// ---------------------------------------------------------------------------------------------
// `Gemm<...>`: the host class the reference's launch template instantiates but never defines
// (yan/jit_kernels/gemm.py:20-30).  Template parameter order and the member names are the
// template's; the eighth parameter (the reference's TMA multicast width) is accepted for source
// compatibility and must be 1: this kernel never multicasts.  The scale and output "descriptors" carry plain pointers because the kernel
// reads scales with ordinary loads and writes D with 16-byte stores.
// ---------------------------------------------------------------------------------------------
// A kernel library compiled by the JIT layer (-DYAN_JIT_KERNEL) has a status word and a wait bound of its own, read
// and set through two extra exports next to `launch`; the prebuilt library passes its own through GemmArgs instead.
#ifdef YAN_JIT_KERNEL
namespace jit_state {
__device__ int g_status_word = 0;
inline unsigned long long g_timeout_ns = 2000000000ull;
inline int* status_word() {
    static int* ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        ptr[dev] = static_cast<int*>(p);
    }
    return ptr[dev];
}
}  // namespace jit_state

// 0 on success; *status = 0 or (kDeviceTimeout << 8) | site.  Synchronises the device.
extern "C" __attribute__((visibility("default"))) inline __attribute__((used)) int yan_jit_read_device_status(int* status,
                                                                                                               int reset) {
    int* word = jit_state::status_word();
    if (status == nullptr || word == nullptr) return kLaunchFailed;
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return kLaunchFailed;
    }
    if (reset != 0 && *status != 0) {
        const int zero = 0;
        if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            return kLaunchFailed;
        }
    }
    return kOk;
}
extern "C" __attribute__((visibility("default"))) inline __attribute__((used)) void yan_jit_set_wait_timeout_ns(
    unsigned long long timeout_ns) {
    jit_state::g_timeout_ns = timeout_ns == 0 ? 1 : timeout_ns;
}
#endif

struct ScalesADesc {
    const float* ptr;
    uint32_t ld;
};
struct OutDesc {
    __nv_bfloat16* ptr;
    uint32_t ld;
};

template <uint32_t SHAPE_N, uint32_t SHAPE_K, uint32_t BLOCK_M, uint32_t BLOCK_N, uint32_t BLOCK_K, uint32_t kNumGroups,
          uint32_t kNumStages, uint32_t kNumCtasPerLoad, GemmType kGemmType>
class Gemm {
    static_assert(BLOCK_M == kBlockM && BLOCK_K == kBlockK, "this kernel is built around 128 x BLOCK_N x 128 tiles");
    static_assert(kNumCtasPerLoad == 1, "every CTA loads its own tiles: the load width must be 1");
    static_assert(SHAPE_K % BLOCK_K == 0, "K must be a multiple of 128");

public:
    using Launcher = GemmLauncher<BLOCK_N, kNumStages, kGemmType, __nv_bfloat16>;
    static constexpr uint32_t kSmemSize = Launcher::kSmemSize;

    struct TmaDesc {
        const void* ptr;
        uint32_t rows;
    };

    template <typename T>
    static TmaDesc make_2d_tma_a_desc(T* lhs, uint32_t m) {
        return {lhs, m};
    }
    template <typename T>
    static TmaDesc make_2d_tma_b_desc(T* rhs) {
        return {rhs, SHAPE_N * kNumGroups};
    }
    static ScalesADesc make_2d_tma_scales_a_desc(const float* lhs_scales, uint32_t m) { return {lhs_scales, m}; }
    static OutDesc make_2d_tma_d_desc(__nv_bfloat16* out, uint32_t /*m*/) { return {out, SHAPE_N}; }

    // Returns a ReturnCode; the generated `launch` stores it in `__return_code`.
    static int run(__nv_bfloat16* out, float* rhs_scales, int* grouped_layout, uint32_t m, const TmaDesc& a_desc,
                   const TmaDesc& b_desc, const ScalesADesc& scales_a_desc, const OutDesc& d_desc, cudaStream_t stream,
                   int num_sms, uint32_t smem_size) {
        if (smem_size != 0 && smem_size < kSmemSize) return kSmemTooLarge;
        GemmArgs a;
        a.lhs = a_desc.ptr;
        a.lhs_scales = scales_a_desc.ptr;
        a.lhs_scales_ld = scales_a_desc.ld;
        a.rhs = b_desc.ptr;
        a.rhs_scales = rhs_scales;
        a.out = out;
        a.ldd = d_desc.ld;
        a.grouped_layout = grouped_layout;
        a.m = m;
        a.n = SHAPE_N;
        a.k = SHAPE_K;
        a.num_groups = kNumGroups;
        a.num_sms = num_sms;
#ifdef YAN_JIT_KERNEL
        a.status = jit_state::status_word();
        a.timeout_ns = jit_state::g_timeout_ns;
#endif
        return Launcher::launch(a, stream);
    }
};

}  // namespace yan
