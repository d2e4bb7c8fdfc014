#pragma once
// Small integer helpers shared by host and device code of the FP8 GEMM.
// Same role as the reference's yan/include/gemm/utils.cuh:5-13 (ceil_div, constexpr_gcd).

#include <cstdint>

namespace yan {

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) {
    return (a + b - 1) / b;
}

template <typename T>
__host__ __device__ constexpr T constexpr_gcd(T a, T b) {
    return b == 0 ? a : constexpr_gcd(b, a % b);
}

template <typename T>
__host__ __device__ constexpr T align_up(T a, T b) {
    return ceil_div(a, b) * b;
}

// Error codes written to `__return_code` by every C-ABI entry point.  0 = launched.
// The tuner treats non-zero as "illegal configuration, skip" (yan/jit_kernels/tuner.py:45-50).
enum ReturnCode : int {
    kOk = 0,
    kBadArgument = 1,       // null pointer, non-positive size, misaligned pointer / stride, K % 128 != 0 ...
    kSmemTooLarge = 2,      // requested dynamic shared memory exceeds the device opt-in maximum
    kTensorMapFailed = 3,   // cuTensorMapEncodeTiled refused the descriptor
    kLaunchFailed = 4,      // cudaGetLastError() after the launch (or a runtime call) was not cudaSuccess
    kCommFailed = 5,        // collective library reported an error
    kDeviceTimeout = 6,     // a bounded device-side wait ran out (read back through the status word)
    kWorkspaceTooSmall = 7, // caller-provided or static scratch cannot hold the intermediates
};

}  // namespace yan
