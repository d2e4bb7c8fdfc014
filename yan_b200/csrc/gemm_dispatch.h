#pragma once
// Internal interface between the C-ABI translation unit and the per-BLOCK_N GEMM instantiation units
// (gemm_inst.cu is compiled once per BLOCK_N so the instantiations build in parallel).
#include <cuda_runtime.h>

#include "gemm/fp8_gemm.cuh"

namespace yan {

enum class OutKind { BF16 = 0, F32 = 1, E4M3 = 2 };

int launch_gemm_bn32(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn64(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn96(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn128(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn160(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn192(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn224(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);
int launch_gemm_bn256(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream);

// Default pipeline depth per BLOCK_N: 128-wide k-block stages (16 KB of A + BLOCK_N * 128 bytes of B each) that fit
// in 227 KB next to the barriers, at most 8.
#ifndef YAN_STAGES_256
#define YAN_STAGES_256 4
#endif
constexpr uint32_t default_num_stages(uint32_t block_n) {
    return block_n == 256 ? YAN_STAGES_256 : block_n >= 192 ? 5 : block_n == 160 ? 6 : block_n == 128 ? 6 : 8;
}

}  // namespace yan
