#pragma once
// bf16 -> e4m3 quantizers with fp32 scales.
//   per_token_cast_to_fp8 : 1 x 128 groups along K (activations); scales written k-block-major
//                           (M contiguous per k-block), the layout the GEMM reads
//                           (yan/include/gemm/fp8_gemm.cuh:59 sizes one stage of A scales as BLOCK_M floats).
//   per_block_cast_to_fp8 : 128 x 128 blocks (weights); scales [N/128, K/128]
//                           (the `scales_b` operand of fp8_gemm.cuh:41).
// The reference has no quantizer; the load/reduce idiom (128-bit loads, shuffle reduction) is the
// one its reduction kernels use (yan/include/reduce/reduce.cuh:30-40,74).
//
// Arithmetic contract (bit-exact against the CPU oracle): per group
//     amax_c = max(max|x|, 1e-4f);  inv = 448 / amax_c  (IEEE RN division)
//     q      = e4m3_rne(x * inv)                          (IEEE RN multiply, then RNE conversion)
//     scale  = amax_c / 448                                (IEEE RN division)
// Must be compiled WITHOUT --use_fast_math.

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../gemm/utils.cuh"

namespace yan {

constexpr float kFp8Max = 448.0f;
constexpr float kAmaxFloor = 1e-4f;

namespace detail {

__device__ __forceinline__ float amax8(const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    __nv_bfloat162 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
    return fmaxf(__low2float(m), __high2float(m));
}

__device__ __forceinline__ uint2 quantize8(const uint4& v, float inv) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 f0 = __bfloat1622float2(h[2 * i]);
        const float2 f1 = __bfloat1622float2(h[2 * i + 1]);
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(__fmul_rn(f0.x, inv), __fmul_rn(f0.y, inv)), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(__fmul_rn(f1.x, inv), __fmul_rn(f1.y, inv)), __NV_SATFINITE, __NV_E4M3);
        w[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    return make_uint2(w[0], w[1]);
}

}  // namespace detail

// One CTA = 256 threads = 16 half-warps covers kRows rows x 4 k-groups; a half-warp owns one
// (row, group) item at a time: 16 lanes x 16 bytes = 128 bf16.  All loads of a thread are issued
// before the first reduction.  Scales are staged in shared memory and written kRows-contiguous.
template <uint32_t kRows>
__global__ void __launch_bounds__(256) per_token_cast_to_fp8_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    uint8_t* __restrict__ q,
                                                                    float* __restrict__ scales, uint32_t m, uint32_t k,
                                                                    uint32_t x_ld, uint32_t sa_ld) {
    constexpr uint32_t kGroups = 4;
    constexpr uint32_t kItems = kRows * kGroups / 16;  // per half-warp
    __shared__ float s_scales[kGroups][kRows];
    // A GEMM launched behind this kernel with programmatic stream serialization may start its weight loads now;
    // it waits for this grid to complete before it touches the quantized activations.  No effect otherwise.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // When this kernel itself was launched with programmatic stream serialization its CTAs may be resident before the
    // kernel that produces x has finished: wait for it (and for the previous readers of q / scales) here.  No effect
    // for an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t hw = threadIdx.x / 16, l = threadIdx.x % 16;
    const uint32_t row0 = blockIdx.y * kRows, kb0 = blockIdx.x * kGroups;
    const uint32_t num_kb = k / 128;

    uint4 v[kItems];
#pragma unroll
    for (uint32_t j = 0; j < kItems; ++j) {
        const uint32_t item = hw + 16 * j, r = item / kGroups, g = item % kGroups;
        const uint32_t row = row0 + r, kb = kb0 + g;
        v[j] = make_uint4(0, 0, 0, 0);
        if (row < m && kb < num_kb)
            v[j] = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * x_ld + kb * 128 + l * 8));
    }
#pragma unroll
    for (uint32_t j = 0; j < kItems; ++j) {
        const uint32_t item = hw + 16 * j, r = item / kGroups, g = item % kGroups;
        const uint32_t row = row0 + r, kb = kb0 + g;
        float amax = detail::amax8(v[j]);
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float amax_c = fmaxf(amax, kAmaxFloor);
        const float inv = __fdiv_rn(kFp8Max, amax_c);
        if (row < m && kb < num_kb) {
            *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * k + kb * 128 + l * 8) =
                detail::quantize8(v[j], inv);
            if (l == 0) s_scales[g][r] = __fdiv_rn(amax_c, kFp8Max);
        }
    }
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < kGroups * kRows; t += 256) {
        const uint32_t g = t / kRows, r = t % kRows;
        if (row0 + r < m && kb0 + g < num_kb) scales[static_cast<size_t>(kb0 + g) * sa_ld + row0 + r] = s_scales[g][r];
    }
}

// One CTA (256 threads) per 128 x 128 block.
__global__ void __launch_bounds__(256) per_block_cast_to_fp8_kernel(const __nv_bfloat16* __restrict__ w,
                                                                    uint8_t* __restrict__ q,
                                                                    float* __restrict__ scales, uint32_t n, uint32_t k) {
    __shared__ float s_amax[8];
    const uint32_t nb = blockIdx.y, kb = blockIdx.x, num_kb = k / 128;
    const uint32_t r0 = threadIdx.x / 16, c = (threadIdx.x % 16) * 8;
    uint4 v[8];
    float amax = 0.0f;
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j) {
        const size_t row = static_cast<size_t>(nb) * 128 + j * 16 + r0;
        v[j] = __ldg(reinterpret_cast<const uint4*>(w + row * k + kb * 128 + c));
        amax = fmaxf(amax, detail::amax8(v[j]));
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (threadIdx.x % 32 == 0) s_amax[threadIdx.x / 32] = amax;
    __syncthreads();
    amax = s_amax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_amax[i]);
    const float amax_c = fmaxf(amax, kAmaxFloor);
    const float inv = __fdiv_rn(kFp8Max, amax_c);
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j) {
        const size_t row = static_cast<size_t>(nb) * 128 + j * 16 + r0;
        *reinterpret_cast<uint2*>(q + row * k + kb * 128 + c) = detail::quantize8(v[j], inv);
    }
    if (threadIdx.x == 0) scales[static_cast<size_t>(nb) * num_kb + kb] = __fdiv_rn(amax_c, kFp8Max);
}

// Host launchers.  Return a ReturnCode.
// programmatic: launch with programmatic stream serialization, so that the launch latency overlaps the tail of the
// kernel before it in the stream (the kernel waits for that kernel before it reads or writes anything).
inline int launch_per_token_cast_to_fp8(const void* x, void* q, float* scales, uint32_t m, uint32_t k, uint32_t x_ld,
                                        uint32_t sa_ld, cudaStream_t stream, bool programmatic = false) {
    if (x == nullptr || q == nullptr || scales == nullptr || m == 0 || k == 0 || k % 128 != 0) return kBadArgument;
    if (x_ld < k || x_ld % 8 != 0 || sa_ld < m) return kBadArgument;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(q) % 8 != 0) return kBadArgument;
    const uint32_t num_kb = k / 128;
    const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x);
    auto* qp = reinterpret_cast<uint8_t*>(q);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    cudaError_t e;
    if (m >= 1024) {
        cfg.gridDim = dim3(ceil_div(num_kb, 4u), ceil_div(m, 32u));
        if (cfg.gridDim.y > 65535) return kBadArgument;
        e = cudaLaunchKernelEx(&cfg, per_token_cast_to_fp8_kernel<32>, xp, qp, scales, m, k, x_ld, sa_ld);
    } else {
        cfg.gridDim = dim3(ceil_div(num_kb, 4u), ceil_div(m, 8u));
        e = cudaLaunchKernelEx(&cfg, per_token_cast_to_fp8_kernel<8>, xp, qp, scales, m, k, x_ld, sa_ld);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return kLaunchFailed;
    }
    return kOk;
}

inline int launch_per_block_cast_to_fp8(const void* w, void* q, float* scales, uint32_t n, uint32_t k,
                                        cudaStream_t stream) {
    if (w == nullptr || q == nullptr || scales == nullptr || n == 0 || k == 0 || n % 128 != 0 || k % 128 != 0)
        return kBadArgument;
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0 || reinterpret_cast<uintptr_t>(q) % 8 != 0) return kBadArgument;
    dim3 grid(k / 128, n / 128);
    if (grid.y > 65535) return kBadArgument;
    per_block_cast_to_fp8_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w),
                                                         reinterpret_cast<uint8_t*>(q), scales, n, k);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace yan
