#pragma once
// Weight-streaming FP8 GEMM for M <= 32 without any cross-CTA reduction ("stacked K").
//
// The operands are swapped as in fp8_gemm_small_m.cuh (weight rows on the UMMA M side, activation rows on the N
// side), but a CTA owns only 32 weight rows and ALL of K.  The four lane quarters of the 128-row MMA operand hold
// the same 32 weight rows at four different k-blocks (quarter q of step s holds k-block q*steps + s), and the
// activation operand stacks the four matching activation tiles along N:
//
//        A operand (128 x 128 B)            B operand (4*M_PAD x 128 B)          D in TMEM (128 lanes x 4*M_PAD cols)
//   rows  0..31 : W[n0.., kb(0,s)]     rows 0..M_PAD-1     : X[.., kb(0,s)]      lanes  0..31, cols 0..M_PAD-1      useful
//   rows 32..63 : W[n0.., kb(1,s)]     rows M_PAD..2M_PAD-1: X[.., kb(1,s)]      lanes 32..63, cols M_PAD..2M_PAD-1 useful
//   ...                                                                           (the off-diagonal blocks are waste)
//
// Three quarters of the MMA work are thrown away, which costs nothing here: the kernel is bound by HBM, the tensor
// pipe idles.  What it buys: N/32 small CTAs (224 for N = 7168) instead of N/128 pairs, two of them resident per SM
// (96 KB of shared memory at M_PAD = 16), so that with programmatic dependent launch the next GEMM's CTAs start
// streaming weights beside the current ones; and the k-quarters of a weight row meet in ONE CTA, so the final sum is a
// shared-memory exchange between its four promotion warps -- no cluster, no distributed shared memory.
//
// Everything else follows the pair kernel: all TMA loads up front (no ring), one mbarrier and one TMEM column range
// per step, promotion per step as its MMAs finish (thread = lane = (k-quarter, weight row)), weights loaded before
// griddepcontrol.wait and activations after it, bounded waits.
// Limits (host-checked, otherwise the pair kernel or the general kernel runs): M <= 32, N % 32 == 0,
// K % 512 == 0, steps = K/512 <= 8, steps * 4*M_PAD <= 512 TMEM columns, shared memory fits.
// For M <= 16 and more than four steps (K up to 16384) the ring variant further down takes over.

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "fp8_gemm_small_m.cuh"

namespace yan {

constexpr uint32_t kStackedThreads = 160;  // warps 0-3: promotion (warp = lane quarter = k-quarter), warp 4: TMA + MMA
constexpr uint32_t kStackFactor = 4;
constexpr uint32_t kStackedRows = 128 / kStackFactor;  // weight rows per CTA
constexpr uint32_t kStackedMaxSteps = 8;

struct StackedSmem {
    uint32_t off_w, off_x, off_scales, off_reduce, off_barriers, off_tmem_slot, off_abort, total;
};

__host__ __device__ inline StackedSmem stacked_k_smem_layout(uint32_t m_pad, uint32_t steps) {
    StackedSmem s;
    s.off_w = 0;                                              // steps x [128 x 128 B] stacked weight tiles
    s.off_x = s.off_w + steps * 16384u;                       // steps x [4*m_pad x 128 B] stacked activation tiles
    s.off_scales = s.off_x + steps * kStackFactor * m_pad * 128u;  // [4][steps][m_pad] floats: sA * sB per (quarter, step, row)
    s.off_reduce = s.off_scales + kStackFactor * steps * m_pad * 4u;  // [4][m_pad][32] floats
    s.off_barriers = align_up(s.off_reduce + kStackFactor * m_pad * kStackedRows * 4u, 8u);
    s.off_tmem_slot = s.off_barriers + 2 * kStackedMaxSteps * 8u;
    s.off_abort = s.off_tmem_slot + 4;
    s.total = s.off_abort + 4 + 1024;
    return s;
}

template <uint32_t M_PAD>
__global__ void __launch_bounds__(kStackedThreads, 2)
    fp8_gemm_stacked_k_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tensor_map_w,
                              const __grid_constant__ CUtensorMap tensor_map_x) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    static_assert(M_PAD == 16 || M_PAD == 32, "activation rows are padded to 16 or 32");
    constexpr uint32_t kMmaN = kStackFactor * M_PAD;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t num_k_blocks = p.shape_k / kBlockK;
    const uint32_t steps = num_k_blocks / kStackFactor;
    const StackedSmem L = stacked_k_smem_layout(M_PAD, steps);
    uint64_t* full_barriers = reinterpret_cast<uint64_t*>(smem + L.off_barriers);
    uint64_t* done_barriers = full_barriers + kStackedMaxSteps;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.off_tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L.off_abort);
    float* s_scales = reinterpret_cast<float*>(smem + L.off_scales);
    float* s_reduce = reinterpret_cast<float*>(smem + L.off_reduce);

    const uint32_t warp_idx = __shfl_sync(0xffffffffu, threadIdx.x / 32, 0);
    const uint32_t lane_idx = ptx::lane_id();
    const uint32_t n0 = blockIdx.x * kStackedRows;
    const uint32_t tmem_cols = small_m_tmem_cols(kMmaN, steps);
    constexpr uint32_t kStepBytes = 16384u + kMmaN * 128u;

    // Let the next kernel of the stream begin its own weight loads right away.
    ptx::grid_dependency_launch_dependents();

    if (warp_idx == 4) {
        if (lane_idx == 0) {
            ptx::tma_prefetch_desc(&tensor_map_w);
            ptx::tma_prefetch_desc(&tensor_map_x);
            for (uint32_t s = 0; s < steps; ++s) {
                ptx::mbar_init(full_barriers + s, 1);
                ptx::mbar_init(done_barriers + s, 1);
            }
            *abort_flag = 0;
            ptx::fence_barrier_init();
            ptx::fence_proxy_async_smem();
            for (uint32_t s = 0; s < steps; ++s) ptx::mbar_arrive_expect_tx(full_barriers + s, kStepBytes);
        }
        __syncwarp();
        // One load per lane: lane = (step, quarter).  Weights first (they are parameters, not products of the kernel
        // before this one), activations after the grid dependency has been satisfied.
        const uint32_t s = lane_idx / kStackFactor, q = lane_idx % kStackFactor;
        if (s < steps)
            ptx::tma_load_2d(smem + L.off_w + s * 16384u + q * (kStackedRows * 128u), &tensor_map_w, full_barriers + s,
                             static_cast<int32_t>((q * steps + s) * kBlockK), static_cast<int32_t>(n0));
        ptx::grid_dependency_wait();
        if (s < steps)
            ptx::tma_load_2d(smem + L.off_x + s * (kMmaN * 128u) + q * (M_PAD * 128u), &tensor_map_x, full_barriers + s,
                             static_cast<int32_t>((q * steps + s) * kBlockK), 0);
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, tmem_cols);
        ptx::tmem_relinquish_alloc_permit();
    } else {
        // Promotion warps: fold both scale factors of every (quarter, step, row) while the weights stream in.
        const float* sb_ptr = p.scales_b + static_cast<size_t>(n0 / 128u) * num_k_blocks;
        ptx::grid_dependency_wait();
        for (uint32_t i = threadIdx.x; i < kStackFactor * steps * M_PAD; i += 128) {
            const uint32_t m = i % M_PAD, qs = i / M_PAD;  // qs = q * steps + s = the k-block index
            const float sa = (m < p.shape_m) ? __ldg(p.scales_a + static_cast<size_t>(qs) * p.sa_ld + m) : 0.0f;
            s_scales[i] = sa * __ldg(sb_ptr + qs);
        }
    }
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp_idx == 4) {
        if (lane_idx == 0) {
            constexpr uint32_t idesc = make_instr_desc_e4m3_f32(128, kMmaN);
            for (uint32_t s = 0; s < steps; ++s) {
                if (!detail::bounded_wait(full_barriers + s, 0, abort_flag, p, 5)) break;
                ptx::tcgen05_fence_after_thread_sync();
                const uint64_t w_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_w + s * 16384u));
                const uint64_t x_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_x + s * (kMmaN * 128u)));
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                    ptx::umma_f8f6f4_ss(tmem_base + s * kMmaN, w_desc + k * kDescKStep, x_desc + k * kDescKStep, idesc,
                                        k > 0);
                ptx::umma_commit(done_barriers + s);
            }
        }
        __syncwarp();
    } else {
        // Thread = TMEM lane 32*q + r: k-quarter q (= warp), weight row n0 + r.  Its useful columns of step s are
        // [s*kMmaN + q*M_PAD, +M_PAD).
        const uint32_t q = warp_idx;
        const uint32_t taddr = tmem_base + ((q * 32u) << 16) + q * M_PAD;
        float acc[M_PAD];
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; ++m) acc[m] = 0.0f;
        bool alive = true;
        for (uint32_t s = 0; s < steps && alive; ++s) {
            const bool ok = detail::bounded_wait(done_barriers + s, 0, abort_flag, p, 6);
            alive = __all_sync(0xffffffffu, ok);
            if (alive) {
                ptx::tcgen05_fence_after_thread_sync();
                uint32_t t[M_PAD];
                ptx::tmem_ld_32x32b<M_PAD>(taddr + s * kMmaN, t);
                ptx::tmem_ld_wait<M_PAD>(t);
                const float* sc = s_scales + (q * steps + s) * M_PAD;
#pragma unroll
                for (uint32_t m = 0; m < M_PAD; ++m) acc[m] = fmaf(sc[m], __uint_as_float(t[m]), acc[m]);
            }
        }
        ptx::tcgen05_fence_before_thread_sync();
        // The four k-quarters of a weight row sit in four warps: exchange through shared memory, [q][m][r].
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; ++m) s_reduce[(q * M_PAD + m) * kStackedRows + lane_idx] = acc[m];
        ptx::named_barrier_sync(1, 128);
        if (alive && *abort_flag == 0) {
            // warp q finishes activation rows m = q, q+4, ...: all loads first, then the stores
            float v[M_PAD / kStackFactor];
            const uint32_t base = ptx::smem_u32(s_reduce) + lane_idx * 4u;
#pragma unroll
            for (uint32_t j = 0; j < M_PAD / kStackFactor; ++j) {
                const uint32_t m = q + j * kStackFactor;
                v[j] = 0.0f;
#pragma unroll
                for (uint32_t qq = 0; qq < kStackFactor; ++qq)
                    v[j] += ptx::ld_shared_f32(base + ((qq * M_PAD + m) * kStackedRows) * 4u);
            }
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + n0 + lane_idx;
#pragma unroll
            for (uint32_t j = 0; j < M_PAD / kStackFactor; ++j) {
                const uint32_t m = q + j * kStackFactor;
                if (m < p.shape_m) out[static_cast<size_t>(m) * p.ldd] = __float2bfloat16_rn(v[j]);
            }
        }
    }

    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp_idx == 4) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(tmem_base, tmem_cols);
    }
#endif
}

// ---------------------------------------------------------------------------------------------------------------
// Long K (more than four steps, K > 2048): the same kernel with its step buffers recycled.  Four step slots of shared
// memory (96 KB: still two CTAs per SM) and four accumulator slots of tensor memory rotate: the loads of step s + 4 go
// out as soon as the MMAs of step s are complete, the MMAs of step s + 4 wait until the promotion warps have read the
// accumulator of step s.  Four steps per CTA stay in flight for the whole K loop.  M <= 32 (M_PAD 16 or 32).
//   warps 0-3: promotion; warp 4: sixteen producer lanes, lane = (slot, k-quarter); warp 5: TMEM + MMA issuer.
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t kRingThreads = 192;
constexpr uint32_t kRingMaxSteps = 32;
// Slots per CTA: 4 (96 KB, two CTAs per SM) when the grid is larger than the GPU, 8 (192 KB, all 512 TMEM columns)
// when every CTA has an SM to itself anyway (N/32 <= number of SMs), which doubles the bytes a CTA keeps in flight.

struct StackedRingSmem {
    uint32_t off_w, off_x, off_scales, off_reduce, off_barriers, off_tmem_slot, off_abort, total;
};

__host__ __device__ inline StackedRingSmem stacked_k_ring_smem_layout(uint32_t m_pad, uint32_t steps,
                                                                      uint32_t kRingSlots) {
    StackedRingSmem s;
    s.off_w = 0;                                                   // slots x [128 x 128 B]
    s.off_x = s.off_w + kRingSlots * 16384u;                       // slots x [4*m_pad x 128 B]
    s.off_scales = s.off_x + kRingSlots * kStackFactor * m_pad * 128u;  // [4][steps][m_pad] floats
    s.off_reduce = s.off_scales + kStackFactor * steps * m_pad * 4u;    // [4][m_pad][32] floats
    s.off_barriers = align_up(s.off_reduce + kStackFactor * m_pad * kStackedRows * 4u, 8u);
    s.off_tmem_slot = s.off_barriers + 3 * kRingSlots * 8u;  // full, done, tmem_empty per slot
    s.off_abort = s.off_tmem_slot + 4;
    s.total = s.off_abort + 4 + 1024;
    return s;
}

template <uint32_t M_PAD, uint32_t kRingSlots>
__global__ void __launch_bounds__(kRingThreads, (M_PAD == 16 && kRingSlots == 4) ? 2 : 1)
    fp8_gemm_stacked_k_ring_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tensor_map_w,
                                   const __grid_constant__ CUtensorMap tensor_map_x) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    constexpr uint32_t kMmaN = kStackFactor * M_PAD;  // 64 or 128
    constexpr uint32_t kStepBytes = 16384u + kMmaN * 128u;
    constexpr uint32_t kTmemCols = kRingSlots * kMmaN;  // 256 or 512
    static_assert(M_PAD == 16 || M_PAD == 32, "activation rows are padded to 16 or 32");
    static_assert(kRingSlots == 4 || kRingSlots == 8, "one producer lane per (slot, k-quarter): at most 8 slots");
    static_assert(kTmemCols <= 512, "tensor memory has 512 columns");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t num_k_blocks = p.shape_k / kBlockK;
    const uint32_t steps = num_k_blocks / kStackFactor;
    const StackedRingSmem L = stacked_k_ring_smem_layout(M_PAD, steps, kRingSlots);
    uint64_t* full_barriers = reinterpret_cast<uint64_t*>(smem + L.off_barriers);
    uint64_t* done_barriers = full_barriers + kRingSlots;
    uint64_t* tmem_empty_barriers = done_barriers + kRingSlots;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.off_tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L.off_abort);
    float* s_scales = reinterpret_cast<float*>(smem + L.off_scales);
    float* s_reduce = reinterpret_cast<float*>(smem + L.off_reduce);

    const uint32_t warp_idx = __shfl_sync(0xffffffffu, threadIdx.x / 32, 0);
    const uint32_t lane_idx = ptx::lane_id();
    const uint32_t n0 = blockIdx.x * kStackedRows;

    ptx::grid_dependency_launch_dependents();

    if (warp_idx == 4) {
        if (lane_idx == 0) {
            ptx::tma_prefetch_desc(&tensor_map_w);
            ptx::tma_prefetch_desc(&tensor_map_x);
            for (uint32_t r = 0; r < kRingSlots; ++r) {
                ptx::mbar_init(full_barriers + r, 1);        // the producer's arrive.expect_tx
                ptx::mbar_init(done_barriers + r, 1);        // tcgen05.commit
                ptx::mbar_init(tmem_empty_barriers + r, 4);  // one arrival per promotion warp
            }
            *abort_flag = 0;
            ptx::fence_barrier_init();
            ptx::fence_proxy_async_smem();
        }
        __syncwarp();
    }
    __syncthreads();  // barriers are initialised before any role uses them

    if (warp_idx == 4) {
        if (lane_idx < kRingSlots * kStackFactor) {
            const uint32_t r = lane_idx / kStackFactor, q = lane_idx % kStackFactor;
            const uint32_t group_mask = 0xFu << (r * kStackFactor);  // the four lanes of slot r
            uint8_t* w_dst = smem + L.off_w + r * 16384u + q * (kStackedRows * 128u);
            uint8_t* x_dst = smem + L.off_x + r * (kMmaN * 128u) + q * (M_PAD * 128u);
            // first fill: weights before the grid dependency (they are parameters), activations after it
            if (r < steps) {
                if (q == 0) ptx::mbar_arrive_expect_tx(full_barriers + r, kStepBytes);
                __syncwarp(group_mask);
                ptx::tma_load_2d(w_dst, &tensor_map_w, full_barriers + r, static_cast<int32_t>((q * steps + r) * kBlockK),
                                 static_cast<int32_t>(n0));
            }
            ptx::grid_dependency_wait();
            if (r < steps)
                ptx::tma_load_2d(x_dst, &tensor_map_x, full_barriers + r, static_cast<int32_t>((q * steps + r) * kBlockK), 0);
            // refills: slot r is free again when the MMAs of the step it held are complete
            for (uint32_t s = r + kRingSlots; s < steps; s += kRingSlots) {
                const uint32_t it = s / kRingSlots;
                bool ok = detail::bounded_wait(done_barriers + r, (it - 1) & 1, abort_flag, p, 7);
                ok = __all_sync(group_mask, ok);
                if (!ok) break;
                if (q == 0) ptx::mbar_arrive_expect_tx(full_barriers + r, kStepBytes);
                __syncwarp(group_mask);
                ptx::tma_load_2d(w_dst, &tensor_map_w, full_barriers + r, static_cast<int32_t>((q * steps + s) * kBlockK),
                                 static_cast<int32_t>(n0));
                ptx::tma_load_2d(x_dst, &tensor_map_x, full_barriers + r, static_cast<int32_t>((q * steps + s) * kBlockK), 0);
            }
        } else {
            ptx::grid_dependency_wait();
        }
        __syncwarp();
    } else if (warp_idx == 5) {
        ptx::grid_dependency_wait();
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    } else {
        const float* sb_ptr = p.scales_b + static_cast<size_t>(n0 / 128u) * num_k_blocks;
        ptx::grid_dependency_wait();
        for (uint32_t i = threadIdx.x; i < kStackFactor * steps * M_PAD; i += 128) {
            const uint32_t m = i % M_PAD, qs = i / M_PAD;  // qs = q * steps + s = the k-block index
            const float sa = (m < p.shape_m) ? __ldg(p.scales_a + static_cast<size_t>(qs) * p.sa_ld + m) : 0.0f;
            s_scales[i] = sa * __ldg(sb_ptr + qs);
        }
    }
    // TMEM address and scales become visible to the MMA and promotion roles.  The producer lanes are in their refill
    // loop until the last load has gone out, and that loop needs the other roles to make progress, so the barrier
    // below is among warps 0-3 and 5 only (128 + 32 = 160 threads); warp 4 joins the others at the end of the kernel.
    ptx::tcgen05_fence_before_thread_sync();
    if (warp_idx != 4) ptx::named_barrier_sync(2, 160);
    ptx::tcgen05_fence_after_thread_sync();

    if (warp_idx == 5) {
        const uint32_t tmem_base = *tmem_slot;
        if (lane_idx == 0) {
            constexpr uint32_t idesc = make_instr_desc_e4m3_f32(128, kMmaN);
            for (uint32_t s = 0; s < steps; ++s) {
                const uint32_t r = s % kRingSlots, it = s / kRingSlots;
                if (!detail::bounded_wait(full_barriers + r, it & 1, abort_flag, p, 5)) break;
                if (it > 0 && !detail::bounded_wait(tmem_empty_barriers + r, (it - 1) & 1, abort_flag, p, 8)) break;
                ptx::tcgen05_fence_after_thread_sync();
                const uint64_t w_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_w + r * 16384u));
                const uint64_t x_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_x + r * (kMmaN * 128u)));
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                    ptx::umma_f8f6f4_ss(tmem_base + r * kMmaN, w_desc + k * kDescKStep, x_desc + k * kDescKStep, idesc,
                                        k > 0);
                ptx::umma_commit(done_barriers + r);
            }
        }
        __syncwarp();
    } else if (warp_idx < 4) {
        const uint32_t tmem_base = *tmem_slot;
        const uint32_t q = warp_idx;
        const uint32_t taddr = tmem_base + ((q * 32u) << 16) + q * M_PAD;
        float acc[M_PAD];
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; ++m) acc[m] = 0.0f;
        bool alive = true;
        for (uint32_t s = 0; s < steps && alive; ++s) {
            const uint32_t r = s % kRingSlots, it = s / kRingSlots;
            const bool ok = detail::bounded_wait(done_barriers + r, it & 1, abort_flag, p, 6);
            alive = __all_sync(0xffffffffu, ok);
            if (alive) {
                ptx::tcgen05_fence_after_thread_sync();
                uint32_t t[M_PAD];
                ptx::tmem_ld_32x32b<M_PAD>(taddr + r * kMmaN, t);
                ptx::tmem_ld_wait<M_PAD>(t);
                ptx::tcgen05_fence_before_thread_sync();
                __syncwarp();
                if (lane_idx == 0) ptx::mbar_arrive(tmem_empty_barriers + r);  // the accumulator slot may be overwritten
                const float* sc = s_scales + (q * steps + s) * M_PAD;
#pragma unroll
                for (uint32_t m = 0; m < M_PAD; ++m) acc[m] = fmaf(sc[m], __uint_as_float(t[m]), acc[m]);
            }
        }
        ptx::tcgen05_fence_before_thread_sync();
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; ++m) s_reduce[(q * M_PAD + m) * kStackedRows + lane_idx] = acc[m];
        ptx::named_barrier_sync(1, 128);
        if (alive && *abort_flag == 0) {
            float v[M_PAD / kStackFactor];
            const uint32_t base = ptx::smem_u32(s_reduce) + lane_idx * 4u;
#pragma unroll
            for (uint32_t j = 0; j < M_PAD / kStackFactor; ++j) {
                const uint32_t m = q + j * kStackFactor;
                v[j] = 0.0f;
#pragma unroll
                for (uint32_t qq = 0; qq < kStackFactor; ++qq)
                    v[j] += ptx::ld_shared_f32(base + ((qq * M_PAD + m) * kStackedRows) * 4u);
            }
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + n0 + lane_idx;
#pragma unroll
            for (uint32_t j = 0; j < M_PAD / kStackFactor; ++j) {
                const uint32_t m = q + j * kStackFactor;
                if (m < p.shape_m) out[static_cast<size_t>(m) * p.ldd] = __float2bfloat16_rn(v[j]);
            }
        }
    }

    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    if (warp_idx == 5) {
        ptx::tcgen05_fence_after_thread_sync();
        ptx::tmem_dealloc(*tmem_slot, kTmemCols);
    }
#endif
}

inline bool stacked_k_ring_supported(uint32_t m, uint32_t n, uint32_t k, int max_smem) {
    if (m == 0 || m > 32 || n % kStackedRows != 0 || k % (kBlockK * kStackFactor) != 0) return false;
    const uint32_t steps = k / (kBlockK * kStackFactor);
    if (steps <= 4 || steps > kRingMaxSteps) return false;  // up to four steps need no ring
    return stacked_k_ring_smem_layout(m <= 16 ? 16 : 32, steps, 4).total <= static_cast<uint32_t>(max_smem);
}

template <uint32_t M_PAD, uint32_t kRingSlots>
inline int launch_stacked_k_ring_instance(const GemmParams& p, const CUtensorMap& map_w, const CUtensorMap& map_x,
                                          uint32_t steps, uint32_t grid, cudaStream_t stream, bool programmatic) {
    auto kernel = fp8_gemm_stacked_k_ring_kernel<M_PAD, kRingSlots>;
    const uint32_t smem_ring = stacked_k_ring_smem_layout(M_PAD, steps, kRingSlots).total;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_ring) != cudaSuccess) {
        cudaGetLastError();
        return kSmemTooLarge;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kRingThreads);
    cfg.dynamicSmemBytes = smem_ring;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kernel, p, map_w, map_x) != cudaSuccess) {
        cudaGetLastError();
        return kLaunchFailed;
    }
    return kOk;
}

inline bool stacked_k_supported(uint32_t m, uint32_t n, uint32_t k, int max_smem) {
    if (m == 0 || m > 32 || n % kStackedRows != 0 || k % (kBlockK * kStackFactor) != 0) return false;
    const uint32_t m_pad = m <= 16 ? 16 : 32;
    const uint32_t steps = k / (kBlockK * kStackFactor);
    if (steps > kStackedMaxSteps || steps * kStackFactor * m_pad > 512) return false;
    return stacked_k_smem_layout(m_pad, steps).total <= static_cast<uint32_t>(max_smem);
}

// True where the stacked form is the faster of the two weight-streaming kernels: M <= 16 and two CTAs resident per SM
// (measured at N = 7168, K = 2048 with programmatic launch: 5.4 us against 6.3 us at M = 16; at M = 32 its CTAs
// need 128 KB each, only one fits per SM, and the pair kernel wins, 7.2 us against 7.9 us).
inline bool stacked_k_preferred(uint32_t m, uint32_t n, uint32_t k, int max_smem_per_block, int max_smem_per_sm,
                                int num_sms) {
    // Long K: the ring variant against the general kernel, the only alternative there.  M <= 16: 96 KB + scales, two
    // CTAs per SM, always faster (M=16, N=7168, K=4096: 9.7 vs 16.3 us).  M <= 32: 128 KB + scales, one CTA per SM:
    // faster while the grid fits the GPU in one wave (N=4096, K=7168: 12.9 vs 15.8 us), slower beyond
    // (N=7168, K=4096: 15.2 vs 11.6 us).
    if (stacked_k_ring_supported(m, n, k, max_smem_per_block))
        return m <= 16 || n / kStackedRows <= static_cast<uint32_t>(num_sms);
    if (m > 16 || !stacked_k_supported(m, n, k, max_smem_per_block)) return false;
    const uint32_t per_cta = stacked_k_smem_layout(16, k / (kBlockK * kStackFactor)).total + 1024u;  // + driver reserve
    return 2 * per_cta <= static_cast<uint32_t>(max_smem_per_sm);
}

template <uint32_t M_PAD>
inline int launch_stacked_k_instance(const GemmParams& p, const CUtensorMap& map_w, const CUtensorMap& map_x,
                                     uint32_t smem_bytes, uint32_t grid, cudaStream_t stream, bool programmatic) {
    auto kernel = fp8_gemm_stacked_k_kernel<M_PAD>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
        cudaGetLastError();
        return kSmemTooLarge;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kStackedThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p, map_w, map_x);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return kLaunchFailed;
    }
    return kOk;
}

// Host launcher.  Arguments as GemmLauncher::launch (Normal GEMM, bf16 output).
inline int launch_fp8_gemm_stacked_k(const GemmArgs& a, cudaStream_t stream, bool programmatic = false) {
    if (a.lhs == nullptr || a.lhs_scales == nullptr || a.rhs == nullptr || a.rhs_scales == nullptr || a.out == nullptr)
        return kBadArgument;
    if (a.ldd < a.n || a.lhs_scales_ld < a.m) return kBadArgument;
    if (!is_aligned(a.lhs, 16) || !is_aligned(a.rhs, 16) || !is_aligned(a.out, 2)) return kBadArgument;
    int device = 0, max_smem = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return kLaunchFailed;
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    const bool ring = stacked_k_ring_supported(a.m, a.n, a.k, max_smem);
    if (!ring && !stacked_k_supported(a.m, a.n, a.k, max_smem)) return kBadArgument;
    const uint32_t m_pad = a.m <= 16 ? 16 : 32;
    const uint32_t steps = a.k / (kBlockK * kStackFactor);

    bool ok = true;
    const CUtensorMap map_w = make_2d_tma_desc_u8_sw128(a.rhs, a.n, a.k, a.k, kStackedRows, ok);
    const CUtensorMap map_x = make_2d_tma_desc_u8_sw128(a.lhs, a.m, a.k, a.k, m_pad, ok);
    if (!ok) return kTensorMapFailed;

    GemmParams p;
    p.scales_a = a.lhs_scales;
    p.scales_b = a.rhs_scales;
    p.grouped_layout = nullptr;
    p.out = a.out;
    p.out_scales = nullptr;
    p.out_scales_ld = 0;
    p.sa_ld = a.lhs_scales_ld;
    p.ldd = a.ldd;
    p.shape_m = a.m;
    p.shape_n = a.n;
    p.shape_k = a.k;
    p.num_groups = 1;
    p.status = a.status;
    p.timeout_ns = a.timeout_ns;
    const uint32_t grid = a.n / kStackedRows;
    if (ring) {
        int sm_count = 0;
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (m_pad == 32)  // four slots of 128 accumulator columns are all of tensor memory
            return launch_stacked_k_ring_instance<32, 4>(p, map_w, map_x, steps, grid, stream, programmatic);
        const bool alone_on_sm = grid <= static_cast<uint32_t>(sm_count) && steps > 4 &&
                                 stacked_k_ring_smem_layout(16, steps, 8).total <= static_cast<uint32_t>(max_smem);
        if (alone_on_sm) return launch_stacked_k_ring_instance<16, 8>(p, map_w, map_x, steps, grid, stream, programmatic);
        return launch_stacked_k_ring_instance<16, 4>(p, map_w, map_x, steps, grid, stream, programmatic);
    }
    const uint32_t smem_bytes = stacked_k_smem_layout(m_pad, steps).total;
    if (m_pad == 16) return launch_stacked_k_instance<16>(p, map_w, map_x, smem_bytes, grid, stream, programmatic);
    return launch_stacked_k_instance<32>(p, map_w, map_x, smem_bytes, grid, stream, programmatic);
}

}  // namespace yan
