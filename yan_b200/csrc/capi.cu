// C ABI of the FP8 fine-grained-scaled GEMM path (declarations and layouts: include/yan_b200.h).
// Every entry point validates on the host, enqueues on the caller's stream and reports through
// `return_code`; nothing allocates, frees or synchronises (except the explicit status read).

#include <cstdint>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/yan_b200.h"
#include "gemm_dispatch.h"
#include "gemm/fp8_gemm_small_m.cuh"
#include "gemm/fp8_gemm_stacked_k.cuh"
#include "comm/peer_allreduce.cuh"
#include "quant/fp8_cast.cuh"

namespace {

// One status word per device image of this library; kernels report bounded-wait expiry here.
__device__ int g_status_word = 0;

unsigned long long g_timeout_ns = 2000000000ull;
// The waits between ranks have a bound of their own: ranks of one job drift apart by seconds for ordinary reasons
// (first-call module loading, a garbage collection, a stalled data loader), which no wait inside one kernel does.
unsigned long long g_collective_timeout_ns = 10000000000ull;
int g_programmatic_launch = 0;
long long* g_clock_probe = nullptr;

constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {};

int* status_word_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (g_status_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        g_status_ptr[dev] = static_cast<int*>(p);
    }
    return g_status_ptr[dev];
}

// Scratch of the allocation-free entry point: quantized activations followed by their scales.
// Every device that loads this library holds these bytes until the process exits.
constexpr size_t kStaticScratchQBytes = YAN_B200_STATIC_SCRATCH_MAX_ELEMENTS;  // one byte per element
constexpr size_t kStaticScratchScaleBytes = kStaticScratchQBytes / 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchQBytes + kStaticScratchScaleBytes];

unsigned char* g_static_scratch_ptr[kMaxDevices] = {};

// In host code `g_static_scratch` is only a handle; the device address has to be asked for, once per
// device, with that device current.
unsigned char* static_scratch_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (g_static_scratch_ptr[dev] == nullptr) {
        unsigned char* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        g_static_scratch_ptr[dev] = p;
    }
    return g_static_scratch_ptr[dev];
}

// Diagnostic kernel: one thread waits, with the same bounded wait the GEMMs use, on an mbarrier that nothing
// ever arrives on.  The wait runs out, the status word is written, the kernel returns.
__global__ void wait_probe_kernel(yan::GemmParams p) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        yan::ptx::mbar_init(&bar, 1);
        abort_flag = 0;
        yan::ptx::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) yan::detail::bounded_wait(&bar, 0, &abort_flag, p, 15);
    __syncthreads();
}

inline void set_rc(int* rc, int v) {
    if (rc != nullptr) *rc = v;
}

// Picks BLOCK_N by a wave model: cost = waves * (time of one tile relative to a 256-wide one).  The relative tile
// times are measured (time per wave on M = 8192, N = 26880, K = 4096, a shape every width divides): the promotion of a
// k-block has a large fixed part, so a narrower tile is far from proportionally cheaper, and the widths without
// shared-memory room for the staged epilogue (224, 192, 160, 96) or with a second B scale and a 16-column tail chunk
// pay for that.  Large problems therefore get 256; narrower tiles win when they fill the machine better.
int choose_block_n(int m, int n, int k, int num_sms, bool can_cut_tail) {
    static const struct { int bn; double tile_cost; } candidates[8] = {
        {256, 1.000}, {224, 1.08}, {192, 0.84}, {160, 0.82}, {128, 0.67}, {96, 0.72}, {64, 0.57}, {32, 0.50}};
    int best = 256;
    double best_cost = -1.0;
    for (const auto& c : candidates) {
        if (c.bn > 32 && n < c.bn) continue;
        const long tiles = static_cast<long>((m + 127) / 128) * ((n + c.bn - 1) / c.bn);
        double waves = static_cast<double>((tiles + num_sms - 1) / num_sms);
        // with scratch for partial tiles the rest of a nearly empty last wave is cut along K (about a third of a wave)
        if (can_cut_tail && (c.bn == 256 || c.bn == 128 || c.bn == 64) &&
            yan::choose_tail_slices(static_cast<uint32_t>(tiles), static_cast<uint32_t>(num_sms), static_cast<uint32_t>(k / 128)) != 0)
            waves = static_cast<double>(tiles / num_sms) + 0.35;
        const double cost = waves * c.tile_cost;
        if (best_cost < 0.0 || cost < best_cost * 0.98) {  // a narrower tile must win by 2 % to be taken
            best_cost = cost;
            best = c.bn;
        }
    }
    return best;
}

int dispatch_gemm(yan::GemmType type, yan::OutKind out_kind, yan::GemmArgs& a, int block_n, void* stream,
                  bool after_own_quantizer = false) {
    if (a.m == 0 || a.n == 0 || a.k == 0) return yan::kBadArgument;
    if (a.num_sms <= 0) return yan::kBadArgument;
    const bool want_auto = (block_n == 0);
    if (block_n == 0) {
        const int rows = (type == yan::GemmType::GroupedMasked) ? static_cast<int>(a.m * a.num_groups) : static_cast<int>(a.m);
        block_n = choose_block_n(rows, static_cast<int>(a.n), static_cast<int>(a.k), a.num_sms,
                                 type == yan::GemmType::Normal && out_kind == yan::OutKind::BF16 && a.tail_workspace != nullptr);
    }
    a.status = status_word_of_current_device();
    a.timeout_ns = g_timeout_ns;
    a.clock_probe = g_clock_probe;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // M <= 64: the weight-streaming kernels.  block_n 1 asks for the pair-cluster kernel, 2 for the stacked-K kernel
    // (M <= 32), 0 picks the stacked one where it is the faster (M <= 16, two CTAs per SM), else the pair kernel.
    if (type == yan::GemmType::Normal && out_kind == yan::OutKind::BF16 && (want_auto || block_n == 1 || block_n == 2)) {
        int dev = 0, max_smem = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        const bool programmatic = g_programmatic_launch != 0 || after_own_quantizer;
        if (block_n == 2) {
            if (!yan::stacked_k_supported(a.m, a.n, a.k, max_smem) && !yan::stacked_k_ring_supported(a.m, a.n, a.k, max_smem))
                return yan::kBadArgument;
            return yan::launch_fp8_gemm_stacked_k(a, s, programmatic);
        }
        if (want_auto) {
            int max_smem_sm = 0, sm_count = 0;
            cudaDeviceGetAttribute(&max_smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
            if (yan::stacked_k_preferred(a.m, a.n, a.k, max_smem, max_smem_sm, sm_count))
                return yan::launch_fp8_gemm_stacked_k(a, s, programmatic);
        }
        if (yan::small_m_supported(a.m, a.n, a.k, max_smem)) return yan::launch_fp8_gemm_small_m(a, s, programmatic);
        if (block_n == 1) return yan::kBadArgument;
    }
    switch (block_n) {
        case 32: return yan::launch_gemm_bn32(type, out_kind, a, s);
        case 64: return yan::launch_gemm_bn64(type, out_kind, a, s);
        case 96: return yan::launch_gemm_bn96(type, out_kind, a, s);
        case 128: return yan::launch_gemm_bn128(type, out_kind, a, s);
        case 160: return yan::launch_gemm_bn160(type, out_kind, a, s);
        case 192: return yan::launch_gemm_bn192(type, out_kind, a, s);
        case 224: return yan::launch_gemm_bn224(type, out_kind, a, s);
        case 256: return yan::launch_gemm_bn256(type, out_kind, a, s);
        default: return yan::kBadArgument;
    }
}

bool positive(int a, int b, int c) { return a > 0 && b > 0 && c > 0; }

// The GEMM of a quantize-then-GEMM call.  Its predecessor in the stream is this library's own quantizer, which never
// writes weights, so the weight-streaming kernel (M <= 64) is always launched with programmatic stream serialization
// here: its weight loads run while the quantizer does, and it waits for the quantizer before reading the activations.
int gemm_after_quantizer(const void* q, const float* scales, const void* rhs, const void* rhs_scales, void* out, int m,
                         int n, int k, int ldd, void* stream, int num_sms, int block_n) {
    if (ldd <= 0) return yan::kBadArgument;
    yan::GemmArgs a;
    a.lhs = q;
    a.lhs_scales = scales;
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(ldd);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    return dispatch_gemm(yan::GemmType::Normal, yan::OutKind::BF16, a, block_n, stream, true);
}

}  // namespace

extern "C" {

#define YAN_EXPORT __attribute__((visibility("default")))

YAN_EXPORT int yan_b200_abi_version(void) { return YAN_B200_ABI_VERSION; }

YAN_EXPORT const char* yan_b200_return_code_string(int code) {
    switch (code) {
        case YAN_B200_OK: return "ok";
        case YAN_B200_BAD_ARGUMENT: return "bad argument (null/misaligned pointer, size, stride or K % 128 != 0)";
        case YAN_B200_SMEM_TOO_LARGE: return "configuration needs more shared memory than the device offers";
        case YAN_B200_TENSOR_MAP_FAILED: return "cuTensorMapEncodeTiled failed";
        case YAN_B200_LAUNCH_FAILED: return "kernel launch or CUDA runtime call failed";
        case YAN_B200_COMM_FAILED: return "collective communication failed";
        case YAN_B200_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case YAN_B200_WORKSPACE_TOO_SMALL: return "workspace too small";
        default: return "unknown code";
    }
}

YAN_EXPORT void yan_b200_gemm_fp8_fp8_bf16_nt(const void* lhs, const void* lhs_scales, const void* rhs,
                                              const void* rhs_scales, void* out, int m, int n, int k, int ldd,
                                              void* stream, int num_sms, int block_n, int* return_code) {
    if (!positive(m, n, k) || ldd <= 0) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(ldd);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    set_rc(return_code, dispatch_gemm(yan::GemmType::Normal, yan::OutKind::BF16, a, block_n, stream));
}

YAN_EXPORT size_t yan_b200_gemm_tail_workspace_bytes(int num_sms) {
    return num_sms > 0 ? yan::tail_workspace_bytes(static_cast<uint32_t>(num_sms), 256) : 0;
}

YAN_EXPORT void yan_b200_gemm_fp8_fp8_bf16_nt_tail(const void* lhs, const void* lhs_scales, const void* rhs,
                                                   const void* rhs_scales, void* out, int m, int n, int k, int ldd,
                                                   void* stream, int num_sms, int block_n, void* workspace,
                                                   size_t workspace_bytes, int* return_code) {
    if (!positive(m, n, k) || ldd <= 0) return set_rc(return_code, yan::kBadArgument);
    if (workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(ldd);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    a.tail_workspace = workspace;
    a.tail_workspace_bytes = workspace_bytes;
    set_rc(return_code, dispatch_gemm(yan::GemmType::Normal, yan::OutKind::BF16, a, block_n, stream));
}

YAN_EXPORT void yan_b200_gemm_fp8_fp8_f32_nt(const void* lhs, const void* lhs_scales, const void* rhs,
                                             const void* rhs_scales, void* out, int m, int n, int k, int ldd,
                                             void* stream, int num_sms, int block_n, int* return_code) {
    if (!positive(m, n, k) || ldd <= 0) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(ldd);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    set_rc(return_code, dispatch_gemm(yan::GemmType::Normal, yan::OutKind::F32, a, block_n, stream));
}

YAN_EXPORT void yan_b200_gemm_fp8_fp8_e4m3_nt(const void* lhs, const void* lhs_scales, const void* rhs,
                                              const void* rhs_scales, void* out, void* out_scales, int m, int n, int k,
                                              int ldd, int out_scales_ld, void* stream, int num_sms,
                                              int* return_code) {
    if (!positive(m, n, k) || ldd <= 0 || out_scales_ld <= 0) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(ldd);
    a.out_scales = static_cast<float*>(out_scales);
    a.out_scales_ld = static_cast<uint32_t>(out_scales_ld);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    // the epilogue quantizes one 1 x 128 group per thread, which only the 256-wide tile provides
    set_rc(return_code, dispatch_gemm(yan::GemmType::Normal, yan::OutKind::E4M3, a, 256, stream));
}

YAN_EXPORT void yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_contiguous(const void* lhs, const void* lhs_scales,
                                                                   const void* rhs, const void* rhs_scales, void* out,
                                                                   const int* m_indices, int m, int n, int k,
                                                                   int num_groups, void* stream, int num_sms,
                                                                   int block_n, int* return_code) {
    if (!positive(m, n, k) || num_groups <= 0 || m % 128 != 0) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(n);
    a.grouped_layout = m_indices;
    a.m = m, a.n = n, a.k = k;
    a.num_groups = static_cast<uint32_t>(num_groups);
    a.num_sms = num_sms;
    if (n % 128 != 0) return set_rc(return_code, yan::kBadArgument);
    set_rc(return_code, dispatch_gemm(yan::GemmType::GroupedContiguous, yan::OutKind::BF16, a, block_n, stream));
}

YAN_EXPORT void yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_masked(const void* lhs, const void* lhs_scales, const void* rhs,
                                                               const void* rhs_scales, void* out, const int* masked_m,
                                                               int m_max, int n, int k, int num_groups, void* stream,
                                                               int num_sms, int block_n, int* return_code) {
    if (!positive(m_max, n, k) || num_groups <= 0 || n % 128 != 0) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m_max) * static_cast<uint32_t>(num_groups);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = out;
    a.ldd = static_cast<uint32_t>(n);
    a.grouped_layout = masked_m;
    a.m = m_max, a.n = n, a.k = k;
    a.num_groups = static_cast<uint32_t>(num_groups);
    a.num_sms = num_sms;
    set_rc(return_code, dispatch_gemm(yan::GemmType::GroupedMasked, yan::OutKind::BF16, a, block_n, stream));
}

YAN_EXPORT void yan_b200_per_token_cast_to_fp8(const void* x, void* out, void* out_scales, int m, int k, int x_ld,
                                               int scales_ld, void* stream, int* return_code) {
    if (m <= 0 || k <= 0 || x_ld <= 0 || scales_ld <= 0) return set_rc(return_code, yan::kBadArgument);
    set_rc(return_code,
           yan::launch_per_token_cast_to_fp8(x, out, static_cast<float*>(out_scales), m, k, x_ld, scales_ld,
                                             static_cast<cudaStream_t>(stream)));
}

YAN_EXPORT void yan_b200_per_block_cast_to_fp8(const void* w, void* out, void* out_scales, int n, int k, void* stream,
                                               int* return_code) {
    if (n <= 0 || k <= 0) return set_rc(return_code, yan::kBadArgument);
    set_rc(return_code, yan::launch_per_block_cast_to_fp8(w, out, static_cast<float*>(out_scales), n, k,
                                                          static_cast<cudaStream_t>(stream)));
}

YAN_EXPORT size_t yan_b200_fp8_linear_workspace_bytes(int m, int k) {
    if (m <= 0 || k <= 0 || k % 128 != 0) return 0;
    const size_t q_bytes = yan::align_up(static_cast<size_t>(m) * k, static_cast<size_t>(256));
    const size_t s_bytes = yan::align_up(static_cast<size_t>(m) * (k / 128) * sizeof(float), static_cast<size_t>(256));
    return q_bytes + s_bytes;
}

YAN_EXPORT void yan_b200_fp8_linear_bf16(const void* a, const void* rhs, const void* rhs_scales, void* out,
                                         void* workspace, size_t workspace_bytes, int m, int n, int k, int ldd,
                                         void* stream, int num_sms, int block_n, int* return_code) {
    if (!positive(m, n, k) || k % 128 != 0 || workspace == nullptr) return set_rc(return_code, yan::kBadArgument);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return set_rc(return_code, yan::kBadArgument);
    if (workspace_bytes < yan_b200_fp8_linear_workspace_bytes(m, k))
        return set_rc(return_code, yan::kWorkspaceTooSmall);
    uint8_t* q = static_cast<uint8_t*>(workspace);
    float* scales = reinterpret_cast<float*>(q + yan::align_up(static_cast<size_t>(m) * k, static_cast<size_t>(256)));
    int rc = yan::launch_per_token_cast_to_fp8(a, q, scales, m, k, k, m, static_cast<cudaStream_t>(stream),
                                               g_programmatic_launch != 0);
    if (rc != yan::kOk) return set_rc(return_code, rc);
    set_rc(return_code, gemm_after_quantizer(q, scales, rhs, rhs_scales, out, m, n, k, ldd, stream, num_sms, block_n));
}

YAN_EXPORT void yan_b200_fp8_linear_bf16_static(const void* a, const void* rhs, const void* rhs_scales, void* out,
                                                int m, int n, int k, int ldd, void* stream, int num_sms, int block_n,
                                                int* return_code) {
    if (!positive(m, n, k) || k % 128 != 0) return set_rc(return_code, yan::kBadArgument);
    const size_t elements = static_cast<size_t>(m) * static_cast<size_t>(k);
    if (elements > kStaticScratchQBytes || elements / 128 * sizeof(float) > kStaticScratchScaleBytes)
        return set_rc(return_code, yan::kWorkspaceTooSmall);  // M * K exceeds the built-in scratch
    unsigned char* scratch = static_scratch_of_current_device();
    if (scratch == nullptr) return set_rc(return_code, yan::kLaunchFailed);
    uint8_t* q = scratch;
    float* scales = reinterpret_cast<float*>(scratch + kStaticScratchQBytes);
    const int rc = yan::launch_per_token_cast_to_fp8(a, q, scales, m, k, k, m, static_cast<cudaStream_t>(stream),
                                                     g_programmatic_launch != 0);
    if (rc != yan::kOk) return set_rc(return_code, rc);
    set_rc(return_code, gemm_after_quantizer(q, scales, rhs, rhs_scales, out, m, n, k, ldd, stream, num_sms, block_n));
}

YAN_EXPORT void yan_b200_read_device_status(int* status, int reset, int* return_code) {
    if (status == nullptr) return set_rc(return_code, yan::kBadArgument);
    int* word = status_word_of_current_device();
    if (word == nullptr) return set_rc(return_code, yan::kLaunchFailed);
    // cudaMemcpy alone only orders against the legacy default stream; kernels on non-blocking streams must finish too
    if (cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        return set_rc(return_code, yan::kLaunchFailed);
    }
    if (cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return set_rc(return_code, yan::kLaunchFailed);
    }
    if (reset != 0 && *status != 0) {
        const int zero = 0;
        if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            return set_rc(return_code, yan::kLaunchFailed);
        }
    }
    set_rc(return_code, yan::kOk);
}

YAN_EXPORT void yan_b200_wait_probe(unsigned long long timeout_ns, void* stream, int* return_code) {
    yan::GemmParams p = {};
    p.status = status_word_of_current_device();
    p.timeout_ns = timeout_ns == 0 ? 1 : timeout_ns;
    if (p.status == nullptr) return set_rc(return_code, yan::kLaunchFailed);
    if (p.timeout_ns > 1000000000ull) return set_rc(return_code, yan::kBadArgument);  // a probe waits at most 1 s
    wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    set_rc(return_code, cudaGetLastError() == cudaSuccess ? yan::kOk : yan::kLaunchFailed);
}

// ---- peer-mapped memory and the two-shot allreduce of the K-split GEMM ----

YAN_EXPORT void yan_b200_ipc_export(const void* ptr, void* handle, unsigned long long* offset, int* return_code) {
    if (ptr == nullptr || handle == nullptr || offset == nullptr) return set_rc(return_code, yan::kBadArgument);
    static_assert(sizeof(cudaIpcMemHandle_t) == YAN_B200_IPC_HANDLE_BYTES, "handle size is part of the ABI");
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range = []() -> RangeFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<RangeFn>(p);
    }();
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range == nullptr || range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
        return set_rc(return_code, yan::kCommFailed);
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
        cudaGetLastError();
        return set_rc(return_code, yan::kCommFailed);
    }
    memcpy(handle, &h, sizeof(h));
    *offset = static_cast<unsigned long long>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    set_rc(return_code, yan::kOk);
}

YAN_EXPORT void yan_b200_ipc_open(const void* handle, void** base, int* return_code) {
    if (handle == nullptr || base == nullptr) return set_rc(return_code, yan::kBadArgument);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return set_rc(return_code, yan::kCommFailed);
    }
    *base = p;
    set_rc(return_code, yan::kOk);
}

YAN_EXPORT void yan_b200_ipc_close(void* base, int* return_code) {
    if (base == nullptr) return set_rc(return_code, yan::kBadArgument);
    if (cudaIpcCloseMemHandle(base) != cudaSuccess) {
        cudaGetLastError();
        return set_rc(return_code, yan::kCommFailed);
    }
    set_rc(return_code, yan::kOk);
}

YAN_EXPORT void yan_b200_allreduce_bf16_two_shot(void* const* data, void* const* signals, int world, int rank,
                                                 unsigned long long elem_begin, unsigned long long elem_count,
                                                 unsigned int epoch, unsigned int counter_target, int num_ctas,
                                                 int exclusive_sms, void* stream, int* return_code) {
    if (data == nullptr || world < 2 || world > yan::kMaxPeers || (epoch != 0 && signals == nullptr))
        return set_rc(return_code, yan::kBadArgument);
    yan::AllreduceArgs a;
    for (int r = 0; r < world; ++r) {
        a.data.p[r] = data[r];
        a.signals.p[r] = (epoch != 0) ? signals[r] : nullptr;
    }
    a.world = world;
    a.rank = rank;
    a.elem_begin = elem_begin;
    a.elem_count = elem_count;
    a.epoch = epoch;
    a.counter_target = counter_target;
    a.num_ctas = num_ctas;
    a.exclusive = exclusive_sms != 0;
    a.status = status_word_of_current_device();
    a.timeout_ns = g_collective_timeout_ns;
    set_rc(return_code, yan::launch_two_shot_allreduce_bf16(a, static_cast<cudaStream_t>(stream)));
}

YAN_EXPORT void yan_b200_allreduce_bf16_in_switch(void* multicast, void* const* signals, int world, int rank,
                                                  unsigned long long elem_begin, unsigned long long elem_count,
                                                  unsigned int epoch, unsigned int counter_target, int num_ctas,
                                                  int exclusive_sms, void* stream, int* return_code) {
    if (multicast == nullptr || world < 2 || world > yan::kMaxPeers || (epoch != 0 && signals == nullptr))
        return set_rc(return_code, yan::kBadArgument);
    yan::AllreduceArgs a;
    a.multicast = multicast;
    for (int r = 0; r < world; ++r) a.signals.p[r] = (epoch != 0) ? signals[r] : nullptr;
    a.world = world;
    a.rank = rank;
    a.elem_begin = elem_begin;
    a.elem_count = elem_count;
    a.epoch = epoch;
    a.counter_target = counter_target;
    a.num_ctas = num_ctas;
    a.exclusive = exclusive_sms != 0;
    a.status = status_word_of_current_device();
    a.timeout_ns = g_collective_timeout_ns;
    set_rc(return_code, yan::launch_two_shot_allreduce_bf16(a, static_cast<cudaStream_t>(stream)));
}

YAN_EXPORT void yan_b200_gemm_fp8_fp8_bf16_nt_scatter(const void* lhs, const void* lhs_scales, const void* rhs,
                                                      const void* rhs_scales, void* const* stage, int world, int rank,
                                                      int m, int n, int k, int ldd, void* stream, int num_sms, int block_n,
                                                      int* return_code) {
    if (!positive(m, n, k) || ldd <= 0 || stage == nullptr || world < 2 || world > yan::kMaxPeers || rank < 0 || rank >= world)
        return set_rc(return_code, yan::kBadArgument);
    if (block_n != 0 && block_n != 256 && block_n != 128) return set_rc(return_code, yan::kBadArgument);
    yan::GemmArgs a;
    a.lhs = lhs;
    a.lhs_scales = static_cast<const float*>(lhs_scales);
    a.lhs_scales_ld = static_cast<uint32_t>(m);
    a.rhs = rhs;
    a.rhs_scales = static_cast<const float*>(rhs_scales);
    a.out = stage[rank];  // every tile goes to a staging array; `out` only has to be a valid pointer
    a.ldd = static_cast<uint32_t>(ldd);
    a.m = m, a.n = n, a.k = k;
    a.num_sms = num_sms;
    for (int r = 0; r < world; ++r) a.scatter_base[r] = stage[r];
    a.scatter_world = static_cast<uint32_t>(world);
    a.scatter_rank = static_cast<uint32_t>(rank);
    // the staged epilogue exists for the 256- and 128-wide tiles; the general width choice may pick others
    set_rc(return_code, dispatch_gemm(yan::GemmType::Normal, yan::OutKind::BF16, a, block_n == 0 ? 256 : block_n, stream));
}

YAN_EXPORT void yan_b200_allreduce_bf16_gather_staged(const void* stage, void* const* data, void* const* signals,
                                                      int world, int rank, int rows, int ld, unsigned int epoch,
                                                      unsigned int counter_target, int num_ctas, void* stream,
                                                      int* return_code) {
    if (stage == nullptr || data == nullptr || signals == nullptr || world < 2 || world > yan::kMaxPeers || rows <= 0 || ld <= 0)
        return set_rc(return_code, yan::kBadArgument);
    yan::AllreduceArgs a;
    for (int r = 0; r < world; ++r) {
        a.data.p[r] = data[r];
        a.signals.p[r] = signals[r];
    }
    a.world = world;
    a.rank = rank;
    a.epoch = epoch;
    a.counter_target = counter_target;
    a.num_ctas = num_ctas;
    a.status = status_word_of_current_device();
    a.timeout_ns = g_collective_timeout_ns;
    a.stage = stage;
    a.rows = static_cast<uint32_t>(rows);
    a.ld = static_cast<uint32_t>(ld);
    set_rc(return_code, yan::launch_gather_staged_allreduce_bf16(a, static_cast<cudaStream_t>(stream)));
}

YAN_EXPORT void yan_b200_set_programmatic_dependent_launch(int enabled) { g_programmatic_launch = enabled; }

YAN_EXPORT void yan_b200_set_clock_probe(void* device_buffer) { g_clock_probe = static_cast<long long*>(device_buffer); }

YAN_EXPORT void yan_b200_set_wait_timeout_ns(unsigned long long timeout_ns) {
    g_timeout_ns = timeout_ns == 0 ? 1 : timeout_ns;
}

YAN_EXPORT void yan_b200_set_collective_timeout_ns(unsigned long long timeout_ns) {
    g_collective_timeout_ns = timeout_ns == 0 ? 1 : timeout_ns;
}

}  // extern "C"
