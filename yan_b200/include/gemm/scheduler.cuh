#pragma once
// Persistent tile scheduler.  Completes what the reference sketches at
// yan/include/gemm/scheduler.cuh:7-58: `GemmType` with the three kinds it declares, one
// scheduler object per role, `get_next_block` handing out (m_block, n_block) pairs in an
// L2-friendly order (bands of kNum1DBlocksPerGroup = 16 tile rows, scheduler.cuh:20).

#include <cstdint>

#include "utils.cuh"

namespace yan {

enum class GemmType {
    Normal,             // D[M,N] = A[M,K] . B[N,K]^T
    GroupedContiguous,  // rows of A belong to groups (128-row aligned); B is [G,N,K]; grouped_layout[m] = group or -1
    GroupedMasked       // A is [G,M_max,K], B is [G,N,K]; grouped_layout[g] = valid rows of group g
};

#ifndef YAN_SCHED_BAND
#define YAN_SCHED_BAND 16
#endif

template <GemmType kGemmType, uint32_t BLOCK_M, uint32_t BLOCK_N, uint32_t kNum1DBlocksPerGroup = YAN_SCHED_BAND>
struct Scheduler {
    int current_iter = -1;
    uint32_t num_m_blocks;  // Normal / Contiguous: over shape_m; Masked: per group maximum
    uint32_t num_n_blocks;
    uint32_t num_blocks;
    uint32_t shape_m;
    uint32_t shape_n;
    uint32_t num_groups;
    const int* grouped_layout;
    // GroupedMasked walk state
    uint32_t curr_group_idx = 0, curr_cumsum = 0;

    __device__ __forceinline__ Scheduler(uint32_t shape_m_, uint32_t shape_n_, const int* grouped_layout_ = nullptr,
                                         uint32_t num_groups_ = 1)
        : shape_m(shape_m_), shape_n(shape_n_), num_groups(num_groups_), grouped_layout(grouped_layout_) {
        num_m_blocks = ceil_div(shape_m, BLOCK_M);
        num_n_blocks = ceil_div(shape_n, BLOCK_N);
        num_blocks = num_m_blocks * num_n_blocks;
    }

    // Band-major order: tiles of 16 consecutive m-blocks sweep all n-blocks before the next band
    // starts, so the CTAs running at one time share a few A row-panels and a few B column-panels.
    __device__ __forceinline__ void swizzle(uint32_t idx, uint32_t m_blocks, uint32_t& m_block_idx,
                                            uint32_t& n_block_idx) const {
        const uint32_t per_band = kNum1DBlocksPerGroup * num_n_blocks;
        const uint32_t band = idx / per_band;
        const uint32_t first_m = band * kNum1DBlocksPerGroup;
        const uint32_t rows = min(kNum1DBlocksPerGroup, m_blocks - first_m);
        const uint32_t in_band = idx - band * per_band;
        m_block_idx = first_m + in_band % rows;
        n_block_idx = in_band / rows;
    }

    __device__ __forceinline__ bool get_next_block(uint32_t& m_block_idx, uint32_t& n_block_idx) {
        const uint32_t next = static_cast<uint32_t>(++current_iter) * gridDim.x + blockIdx.x;
        if constexpr (kGemmType == GemmType::GroupedMasked) {
            while (true) {
                if (curr_group_idx == num_groups) return false;
                const uint32_t m_blocks_g = ceil_div(get_masked_rows(curr_group_idx), BLOCK_M);
                if (next < (curr_cumsum + m_blocks_g) * num_n_blocks) {
                    swizzle(next - curr_cumsum * num_n_blocks, m_blocks_g, m_block_idx, n_block_idx);
                    return true;
                }
                ++curr_group_idx;
                curr_cumsum += m_blocks_g;
            }
        } else {
            if (next >= num_blocks) return false;
            swizzle(next, num_m_blocks, m_block_idx, n_block_idx);
            return true;
        }
    }

    // Group that owns the current tile (Normal: 0).  Contiguous: read from the layout at the tile's
    // first row; negative = padding tile with nothing to compute.
    __device__ __forceinline__ int get_group(uint32_t m_block_idx) const {
        if constexpr (kGemmType == GemmType::GroupedContiguous) return __ldg(grouped_layout + m_block_idx * BLOCK_M);
        if constexpr (kGemmType == GemmType::GroupedMasked) return static_cast<int>(curr_group_idx);
        return 0;
    }

    // First row of the tile in the (flattened) A / D / scales-A row space.
    __device__ __forceinline__ uint32_t get_row_base(uint32_t m_block_idx) const {
        if constexpr (kGemmType == GemmType::GroupedMasked) return curr_group_idx * shape_m + m_block_idx * BLOCK_M;
        return m_block_idx * BLOCK_M;
    }

    // One past the last row the tile may store (tail guard).
    __device__ __forceinline__ uint32_t get_row_limit() const {
        if constexpr (kGemmType == GemmType::GroupedMasked)
            return curr_group_idx * shape_m + get_masked_rows(curr_group_idx);
        return shape_m;
    }

    // Valid rows of a masked group, clamped to [0, M_max]: the count lives in device memory where the host cannot
    // check it, and an oversized or negative value must not make a tile store into the next group or past the output.
    __device__ __forceinline__ uint32_t get_masked_rows(uint32_t group) const {
        const int rows = __ldg(grouped_layout + group);
        return static_cast<uint32_t>(min(max(rows, 0), static_cast<int>(shape_m)));
    }
};

}  // namespace yan
