#pragma once
// Weight-streaming form of the FP8 GEMM for M <= 64 (decode): D[M,N] = A[M,K] . B[N,K]^T, same scales,
// same arithmetic per k-block as fp8_gemm_kernel, organised for HBM bandwidth instead of tensor throughput.
//
//   * operands swapped: 128 rows of B (the weights) are the UMMA "M" side, the M_PAD (16/32/64) activation
//     rows the UMMA "N" side, so a tile is 128 weight rows x all activations and the accumulator of one
//     128-wide k-block is only M_PAD TMEM columns;
//   * split-K over a cluster of two CTAs: CTA r of a pair handles k-blocks [r*KB/2, (r+1)*KB/2) of the same
//     128 weight rows; N/128 * 2 CTAs stream B (112 CTAs for N = 7168);
//   * nothing is recycled: every k-block of a CTA has its own shared-memory tile, its own mbarrier and its
//     own TMEM columns, so all TMA loads are issued at kernel start (the whole of B is in flight at once),
//     the MMA thread never waits for the promotion warps and there is one commit at the end;
//   * each k-block is promoted as soon as its four MMAs are done (one commit and one mbarrier per k-block), so
//     only the last k-block's promotion trails the weight stream: thread = weight row,
//     acc[m] += sA[m,kb]*sB[kb]*P_kb[n,m];
//   * programmatic dependent launch: the weight loads are issued before griddepcontrol.wait, everything that
//     touches activations or the output after it; with the launch attribute set (see the host launcher) the
//     weight loads of GEMM i+1 may start while GEMM i finishes.  Weights must therefore not be produced by the
//     kernel that precedes the GEMM in the stream when that attribute is used;
//   * the second CTA of a pair sends its fp32 partial through distributed shared memory (16-byte st.shared::cluster),
//     the first adds its own, transposes the bf16 tile through shared memory and writes it with 16-byte stores.  No multicast, no remote global memory.  (Measured alternatives,
//     all slower end to end: a 4-CTA cluster with bulk-copy exchange -- the partial sums then cross the
//     SM-to-SM network at about 2 TB/s for the whole chip, a third of the weight bytes again at M = 64 -- and
//     one-way mbarrier hand-shakes instead of the two cluster barriers: a remote arrive costs ~300 ns.)
// Limits (checked on the host; otherwise the general kernel is used): N % 128 == 0, K % 256 == 0,
// (K/256) * M_PAD <= 512 TMEM columns, (K/256) * (16384 + 128*M_PAD) bytes of shared memory.

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "fp8_gemm.cuh"

namespace yan {

constexpr uint32_t kSmallMThreads = 160;   // warps 0-3: promotion (TMEM lane quarter = warp), warp 4: TMA + MMA + TMEM
constexpr uint32_t kSmallMMaxKBlocks = 32;  // k-blocks per CTA

struct SmallMSmem {
    uint32_t off_w, off_x, off_scales, off_stage, off_barriers, off_tmem_slot, off_abort, total;
};

// One weight row's partial sums in the exchange buffer: m_pad floats plus 4 of padding, so that the 16-byte accesses of
// a warp (one row per lane) fall on all 32 banks.
__host__ __device__ constexpr uint32_t small_m_exchange_row_bytes(uint32_t m_pad) { return (m_pad + 4u) * 4u; }

__host__ __device__ inline SmallMSmem small_m_smem_layout(uint32_t m_pad, uint32_t kbh) {
    SmallMSmem s;
    s.off_w = 0;  // kbh x [128 x 128 B] weight tiles; later the exchange buffer [128 weight rows][m_pad + 4] fp32
    const uint32_t w_bytes = kbh * 16384u, exchange_bytes = 128u * small_m_exchange_row_bytes(m_pad);
    s.off_x = s.off_w + (w_bytes > exchange_bytes ? w_bytes : exchange_bytes);  // kbh x [m_pad x 128 B] activation tiles
    s.off_scales = s.off_x + kbh * m_pad * 128u;  // kbh x m_pad floats: sA[m,kb] * sB[kb]
    s.off_stage = align_up(s.off_scales + kbh * m_pad * 4u, 16u);  // [m_pad][128] bf16: the output tile, row-major
    s.off_barriers = align_up(s.off_stage + m_pad * 256u, 8u);
    s.off_tmem_slot = s.off_barriers + 2 * kSmallMMaxKBlocks * 8u;  // full[kb] and done[kb]
    s.off_abort = s.off_tmem_slot + 4;
    s.total = s.off_abort + 4 + 1024;
    return s;
}

__host__ __device__ inline uint32_t small_m_tmem_cols(uint32_t m_pad, uint32_t kbh) {
    uint32_t need = m_pad * kbh, cols = 32;
    while (cols < need) cols *= 2;
    return cols;
}

namespace ptx {
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4_f32(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}
__device__ __forceinline__ float4 ld_shared_v4_f32(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
}  // namespace ptx

template <uint32_t M_PAD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kSmallMThreads, 1)
    fp8_gemm_small_m_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tensor_map_w,
                            const __grid_constant__ CUtensorMap tensor_map_x) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    static_assert(M_PAD == 16 || M_PAD == 32 || M_PAD == 64, "activation rows are padded to 16, 32 or 64");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t num_k_blocks = p.shape_k / kBlockK;
    const uint32_t kbh = num_k_blocks / 2;  // k-blocks of this CTA
    const SmallMSmem L = small_m_smem_layout(M_PAD, kbh);
    uint64_t* full_barriers = reinterpret_cast<uint64_t*>(smem + L.off_barriers);
    uint64_t* done_barriers = full_barriers + kSmallMMaxKBlocks;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.off_tmem_slot);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L.off_abort);
    float* s_scales = reinterpret_cast<float*>(smem + L.off_scales);

    const uint32_t warp_idx = __shfl_sync(0xffffffffu, threadIdx.x / 32, 0);
    const uint32_t lane_idx = ptx::lane_id();
    const uint32_t cta_rank = ptx::cluster_ctarank();
    const uint32_t n_block = blockIdx.x / 2;
    const uint32_t kb_first = cta_rank * kbh;
    const uint32_t tmem_cols = small_m_tmem_cols(M_PAD, kbh);

    // Let the next kernel of the stream begin its own weight loads right away.
    ptx::grid_dependency_launch_dependents();

    if (warp_idx == 4) {
        if (lane_idx == 0) {
            ptx::tma_prefetch_desc(&tensor_map_w);
            ptx::tma_prefetch_desc(&tensor_map_x);
            for (uint32_t i = 0; i < kbh; ++i) {
                ptx::mbar_init(full_barriers + i, 1);
                ptx::mbar_init(done_barriers + i, 1);
            }
            *abort_flag = 0;
            ptx::fence_barrier_init();
            ptx::fence_proxy_async_smem();
            // Every load of this CTA goes out now: nothing below ever waits for a buffer to be recycled.
            // Weights first: they are parameters, not products of the kernel before this one, so under
            // programmatic dependent launch they may be fetched while that kernel is still running.
            for (uint32_t i = 0; i < kbh; ++i) {
                ptx::mbar_arrive_expect_tx(full_barriers + i, 16384u + M_PAD * 128u);
                ptx::tma_load_2d(smem + L.off_w + i * 16384u, &tensor_map_w, full_barriers + i,
                                 static_cast<int32_t>((kb_first + i) * kBlockK), static_cast<int32_t>(n_block * 128u));
            }
            ptx::grid_dependency_wait();  // activations and the output buffer belong to the stream order
            for (uint32_t i = 0; i < kbh; ++i)
                ptx::tma_load_2d(smem + L.off_x + i * M_PAD * 128u, &tensor_map_x, full_barriers + i,
                                 static_cast<int32_t>((kb_first + i) * kBlockK), 0);
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, tmem_cols);
        ptx::tmem_relinquish_alloc_permit();
    } else {
        // Promotion warps: while the weights stream in, fold both scale factors of every (k-block, row) pair.
        const float* sb_ptr = p.scales_b + static_cast<size_t>(n_block) * num_k_blocks + kb_first;
        ptx::grid_dependency_wait();
        for (uint32_t i = threadIdx.x; i < kbh * M_PAD; i += 128) {
            const uint32_t kb = i / M_PAD, m = i % M_PAD;
            const float sa = (m < p.shape_m) ? __ldg(p.scales_a + static_cast<size_t>(kb_first + kb) * p.sa_ld + m) : 0.0f;
            s_scales[i] = sa * __ldg(sb_ptr + kb);
        }
    }
    ptx::tcgen05_fence_before_thread_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;

    float acc[M_PAD];
#pragma unroll
    for (uint32_t m = 0; m < M_PAD; ++m) acc[m] = 0.0f;
    bool alive = true;

    if (warp_idx == 4) {
        if (lane_idx == 0) {
            constexpr uint32_t idesc = make_instr_desc_e4m3_f32(128, M_PAD);
            for (uint32_t i = 0; i < kbh; ++i) {
                if (!detail::bounded_wait(full_barriers + i, 0, abort_flag, p, 5)) break;
                ptx::tcgen05_fence_after_thread_sync();
                const uint64_t w_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_w + i * 16384u));
                const uint64_t x_desc = make_smem_desc_k_major_sw128(ptx::smem_u32(smem + L.off_x + i * M_PAD * 128u));
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k)
                    ptx::umma_f8f6f4_ss(tmem_base + i * M_PAD, w_desc + k * kDescKStep, x_desc + k * kDescKStep, idesc,
                                        k > 0);
                ptx::umma_commit(done_barriers + i);  // this k-block's partial product can be promoted
            }
        }
        __syncwarp();
    } else {
        const uint32_t taddr = tmem_base + ((warp_idx * 32u) << 16);
        constexpr uint32_t kChunk = M_PAD < 32 ? M_PAD : 32;
        for (uint32_t i = 0; i < kbh && alive; ++i) {
            const bool ok = detail::bounded_wait(done_barriers + i, 0, abort_flag, p, 6);
            alive = __all_sync(0xffffffffu, ok);
            if (alive) {
                ptx::tcgen05_fence_after_thread_sync();
#pragma unroll
                for (uint32_t c = 0; c < M_PAD / kChunk; ++c) {
                    uint32_t t[kChunk];
                    ptx::tmem_ld_32x32b<kChunk>(taddr + i * M_PAD + c * kChunk, t);
                    ptx::tmem_ld_wait<kChunk>(t);
#pragma unroll
                    for (uint32_t j = 0; j < kChunk; ++j)
                        acc[c * kChunk + j] = fmaf(s_scales[i * M_PAD + c * kChunk + j], __uint_as_float(t[j]),
                                                   acc[c * kChunk + j]);
                }
            }
        }
        ptx::tcgen05_fence_before_thread_sync();
    }

    // Both CTAs of the pair are past their MMAs and TMEM reads: the weight tiles of CTA 0 are dead and become
    // the landing area for CTA 1's partial sums, one padded row of M_PAD floats per weight row (= per thread), so that
    // both sides move 16 bytes per instruction.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    constexpr uint32_t kRowBytes = small_m_exchange_row_bytes(M_PAD);
    const uint32_t n_in_tile = warp_idx * 32 + lane_idx;
    const uint32_t exchange = ptx::smem_u32(smem + L.off_w) + n_in_tile * kRowBytes;
    if (warp_idx < 4 && cta_rank == 1) {
        const uint32_t remote = ptx::map_to_cta(exchange, 0);
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; m += 4)
            ptx::st_cluster_v4_f32(remote + m * 4u, acc[m], acc[m + 1], acc[m + 2], acc[m + 3]);
    }
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp_idx < 4 && cta_rank == 0 && alive && *abort_flag == 0) {
#pragma unroll
        for (uint32_t m = 0; m < M_PAD; m += 4) {
            const float4 v = ptx::ld_shared_v4_f32(exchange + m * 4u);
            acc[m] += v.x, acc[m + 1] += v.y, acc[m + 2] += v.z, acc[m + 3] += v.w;
        }
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + n_block * 128u;
        const bool vector_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (p.ldd % 8 == 0);
        if (vector_ok) {
            // Transpose through shared memory: [m][128 weight rows] bf16, then 16-byte global stores (a thread-per-
            // weight-row store would write 2 bytes per lane and M_PAD instructions per thread).
            __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + L.off_stage);
#pragma unroll
            for (uint32_t m = 0; m < M_PAD; ++m) stage[m * 128u + n_in_tile] = __float2bfloat16_rn(acc[m]);
            ptx::named_barrier_sync(1, 128);
            for (uint32_t c = threadIdx.x; c < M_PAD * 16u; c += 128) {
                const uint32_t m = c / 16u, part = c % 16u;
                if (m < p.shape_m)
                    *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * p.ldd + part * 8u) =
                        *reinterpret_cast<const uint4*>(stage + m * 128u + part * 8u);
            }
        } else {
#pragma unroll
            for (uint32_t m = 0; m < M_PAD; ++m)
                if (m < p.shape_m) out[static_cast<size_t>(m) * p.ldd + n_in_tile] = __float2bfloat16_rn(acc[m]);
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

// True when the weight-streaming kernel can take the problem (see the limits at the top of this file).
inline bool small_m_supported(uint32_t m, uint32_t n, uint32_t k, int max_smem) {
    if (m == 0 || m > 64 || n % 128 != 0 || k % 256 != 0) return false;
    const uint32_t m_pad = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    const uint32_t kbh = k / 256;
    if (kbh > kSmallMMaxKBlocks || kbh * m_pad > 512) return false;
    return small_m_smem_layout(m_pad, kbh).total <= static_cast<uint32_t>(max_smem);
}

template <uint32_t M_PAD>
inline int launch_small_m_instance(const GemmParams& p, const CUtensorMap& map_w, const CUtensorMap& map_x,
                                   uint32_t smem_bytes, uint32_t grid, cudaStream_t stream, bool programmatic) {
    auto kernel = fp8_gemm_small_m_kernel<M_PAD>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
        cudaGetLastError();
        return kSmemTooLarge;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kSmallMThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];  // the cluster shape is compiled into the kernel (__cluster_dims__)
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
inline int launch_fp8_gemm_small_m(const GemmArgs& a, cudaStream_t stream, bool programmatic = false) {
    if (a.lhs == nullptr || a.lhs_scales == nullptr || a.rhs == nullptr || a.rhs_scales == nullptr || a.out == nullptr)
        return kBadArgument;
    if (a.ldd < a.n || a.lhs_scales_ld < a.m) return kBadArgument;
    if (!is_aligned(a.lhs, 16) || !is_aligned(a.rhs, 16) || !is_aligned(a.out, 2)) return kBadArgument;
    int device = 0, max_smem = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return kLaunchFailed;
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (!small_m_supported(a.m, a.n, a.k, max_smem)) return kBadArgument;
    const uint32_t m_pad = a.m <= 16 ? 16 : (a.m <= 32 ? 32 : 64);
    const uint32_t kbh = a.k / 256;

    bool ok = true;
    const CUtensorMap map_w = make_2d_tma_desc_u8_sw128(a.rhs, a.n, a.k, a.k, 128, ok);
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
    const uint32_t smem_bytes = small_m_smem_layout(m_pad, kbh).total;
    const uint32_t grid = 2 * (a.n / 128);
    switch (m_pad) {
        case 16: return launch_small_m_instance<16>(p, map_w, map_x, smem_bytes, grid, stream, programmatic);
        case 32: return launch_small_m_instance<32>(p, map_w, map_x, smem_bytes, grid, stream, programmatic);
        default: return launch_small_m_instance<64>(p, map_w, map_x, smem_bytes, grid, stream, programmatic);
    }
}

}  // namespace yan
