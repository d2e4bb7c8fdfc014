// One instantiation unit of the FP8 GEMM per BLOCK_N (compile with -DYAN_BLOCK_N=32|64|96|128|160|192|224|256).
#include "gemm_dispatch.h"

#ifndef YAN_BLOCK_N
#error "compile with -DYAN_BLOCK_N=<32|64|96|128|160|192|224|256>"
#endif

#define YAN_CAT_(a, b) a##b
#define YAN_CAT(a, b) YAN_CAT_(a, b)

namespace yan {

int YAN_CAT(launch_gemm_bn, YAN_BLOCK_N)(GemmType type, OutKind out, const GemmArgs& args, cudaStream_t stream) {
    constexpr uint32_t BN = YAN_BLOCK_N;
    constexpr uint32_t S = default_num_stages(BN);
    if (out == OutKind::F32) {
        if (type != GemmType::Normal) return kBadArgument;
        return GemmLauncher<BN, S, GemmType::Normal, float>::launch(args, stream);
    }
    if (out == OutKind::E4M3) {
        // one 1 x 128 quantization group per epilogue thread: only the 256-wide tile has it
        if constexpr (BN == 256) {
            if (type != GemmType::Normal) return kBadArgument;
            return GemmLauncher<BN, S, GemmType::Normal, E4m3Out>::launch(args, stream);
        } else {
            return kBadArgument;
        }
    }
    switch (type) {
        case GemmType::Normal:
            return GemmLauncher<BN, S, GemmType::Normal, __nv_bfloat16>::launch(args, stream);
        case GemmType::GroupedContiguous:
            return GemmLauncher<BN, S, GemmType::GroupedContiguous, __nv_bfloat16>::launch(args, stream);
        case GemmType::GroupedMasked:
            return GemmLauncher<BN, S, GemmType::GroupedMasked, __nv_bfloat16>::launch(args, stream);
    }
    return kBadArgument;
}

}  // namespace yan
