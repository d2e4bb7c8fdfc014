/*
 * yan_b200 -- C ABI of the B200 (sm_100a) FP8 fine-grained-scaled GEMM path.
 *
 * Conventions (the same as the reference's generated entry point
 * `extern "C" void launch(<args>, int& __return_code)`, yan/jit/template.py:130-137, called by
 * yan/jit/runtime.py:30-68 through ctypes):
 *   - every tensor is a raw device pointer (`tensor.data_ptr()`), every stream a `cudaStream_t`
 *     passed as void* (`stream.cuda_stream`), sizes are C `int` (template.py:12-49);
 *   - the caller allocates every buffer including the output; nothing here allocates or frees
 *     device memory or synchronises the device; work is enqueued on the given stream only;
 *   - the last parameter receives 0 when the work was enqueued, otherwise a YAN_B200_* code;
 *     nothing is thrown across the boundary (runtime.py:66-68, yan/jit_kernels/tuner.py:45-50).
 *   `int* return_code` is ABI-identical to the reference's `int& __return_code`.
 *
 * Layouts:
 *   lhs         e4m3 [M, K] row-major                      (yan/include/gemm/fp8_gemm.cuh:43,57)
 *   lhs_scales  fp32, k-block-major: element (kb, row) at kb * M + row, kb = k / 128
 *                                                           (fp8_gemm.cuh:59; yan/jit_kernels/gemm.py:25)
 *   rhs         e4m3 [N, K] row-major ("NT")                (fp8_gemm.cuh:44,58)
 *   rhs_scales  fp32 [ceil(N/128), K/128] row-major         (fp8_gemm.cuh:41,55,60-61)
 *   out         bf16 [M, ldd] row-major, ldd >= N           (fp8_gemm.cuh:56,87)
 *   K % 128 == 0, N % 16 == 0; lhs/rhs/out 16-byte aligned; ldd % 8 == 0.
 */
#ifndef YAN_B200_H_
#define YAN_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YAN_B200_ABI_VERSION 1

enum {
    YAN_B200_OK = 0,
    YAN_B200_BAD_ARGUMENT = 1,
    YAN_B200_SMEM_TOO_LARGE = 2,
    YAN_B200_TENSOR_MAP_FAILED = 3,
    YAN_B200_LAUNCH_FAILED = 4,
    YAN_B200_COMM_FAILED = 5,
    YAN_B200_DEVICE_TIMEOUT = 6,
    YAN_B200_WORKSPACE_TOO_SMALL = 7
};

/* Library identification.  No reference counterpart (the reference identifies a build by the hash
 * of its headers, yan/jit/compiler.py:32-53). */
int yan_b200_abi_version(void);
const char* yan_b200_return_code_string(int code);

/*
 * FP8 GEMM, D = A . B^T with per-128-K scale promotion.  Replaces the launch the reference's template
 * describes: yan/jit_kernels/gemm.py:9-31 (`Gemm<...>::run(out, rhs_scales, nullptr, m, descs..., stream,
 * num_sms, smem_size)`) and the kernel yan/include/gemm/fp8_gemm.cuh:32-197.
 * block_n: 0 = choose; 32, 64, 96, 128, 160, 192, 224 or 256 = tile width of the general kernel; 1 = the weight-streaming kernel
 * for M <= 64 (split-K over a pair of CTAs), 2 = the weight-streaming kernel for M <= 32 that keeps all of K in one
 * CTA (YAN_B200_BAD_ARGUMENT when the problem does not fit the kernel asked for).
 * num_sms: CTAs of the persistent grid (<= device SMs).
 */
void yan_b200_gemm_fp8_fp8_bf16_nt(const void* lhs, const void* lhs_scales, const void* rhs, const void* rhs_scales,
                                   void* out, int m, int n, int k, int ldd, void* stream, int num_sms, int block_n,
                                   int* return_code);

/*
 * The same GEMM, allowed to cut the tiles of a nearly empty last wave along K.  896 tiles on 148 SMs run as 7 waves
 * for 6.05 waves of work; with a workspace the launch becomes three: the whole-tile kernel over the full waves, a
 * second instance of it in which every CTA computes one K-slice of one of the remaining tiles into an fp32 partial
 * tile, and a small kernel that adds a tile's partials in slice order, rounds once and stores.  The result can differ
 * from yan_b200_gemm_fp8_fp8_bf16_nt in the last bit of those tiles (a sum of partial sums instead of one running
 * sum) and meets the same tolerance against the dequantize-and-matmul result; it does not depend on timing.
 * workspace: device memory, 256-byte aligned, at least yan_b200_gemm_tail_workspace_bytes(num_sms) bytes, contents
 * irrelevant; NULL = whole tiles only.  Two launches that may run at the same time need a workspace each.
 * Extends the persistent scheduler the reference sketches (yan/include/gemm/scheduler.cuh:20,39-41), which only
 * knows whole tiles.
 */
size_t yan_b200_gemm_tail_workspace_bytes(int num_sms);
void yan_b200_gemm_fp8_fp8_bf16_nt_tail(const void* lhs, const void* lhs_scales, const void* rhs, const void* rhs_scales,
                                        void* out, int m, int n, int k, int ldd, void* stream, int num_sms, int block_n,
                                        void* workspace, size_t workspace_bytes, int* return_code);

/* Same GEMM with the next layer's quantizer fused into the epilogue: out = e4m3 [M, ldd] (ldd % 16 == 0, 16-byte
 * aligned) and out_scales = fp32, k-block-major [N/128][out_scales_ld] (out_scales_ld >= m), i.e. exactly what
 * yan_b200_per_token_cast_to_fp8 would produce from the bf16 output of yan_b200_gemm_fp8_fp8_bf16_nt (the accumulator is
 * rounded to bf16, then quantized with the same three fp32 operations), bit for bit, without the bf16 tensor ever
 * reaching memory.  N % 128 == 0.  No reference counterpart: the reference's epilogue writes bf16 only
 * (yan/include/gemm/fp8_gemm.cuh:56,87). */
void yan_b200_gemm_fp8_fp8_e4m3_nt(const void* lhs, const void* lhs_scales, const void* rhs, const void* rhs_scales,
                                   void* out, void* out_scales, int m, int n, int k, int ldd, int out_scales_ld,
                                   void* stream, int num_sms, int* return_code);

/* Same GEMM with an fp32 output [M, ldd] (ldd % 4 == 0): the K-split path can then sum fp32 partials.
 * Takes the place of the fp32 partial tiles comm/gemm_allreduce.cu:57-60 reduces across ranks. */
void yan_b200_gemm_fp8_fp8_f32_nt(const void* lhs, const void* lhs_scales, const void* rhs, const void* rhs_scales,
                                  void* out, int m, int n, int k, int ldd, void* stream, int num_sms, int block_n,
                                  int* return_code);

/*
 * Grouped GEMMs the reference's scheduler declares (yan/include/gemm/scheduler.cuh:7-11,42-48;
 * `grouped_layout` kernel argument, fp8_gemm.cuh:41).
 * contiguous: lhs [M, K] whose rows are grouped in 128-row-aligned runs
 *             (yan/jit_kernels/utils.py:46-55), m_indices[M] = group of each row (-1 = padding row),
 *             rhs [G, N, K], rhs_scales [G, N/128, K/128], out [M, N].
 * masked:     lhs [G, m_max, K], lhs_scales k-block-major over G*m_max rows, rhs [G, N, K],
 *             out [G, m_max, N]; only the first masked_m[g] rows of group g are computed.
 */
void yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_contiguous(const void* lhs, const void* lhs_scales, const void* rhs,
                                                        const void* rhs_scales, void* out, const int* m_indices, int m,
                                                        int n, int k, int num_groups, void* stream, int num_sms,
                                                        int block_n, int* return_code);
void yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_masked(const void* lhs, const void* lhs_scales, const void* rhs,
                                                    const void* rhs_scales, void* out, const int* masked_m, int m_max,
                                                    int n, int k, int num_groups, void* stream, int num_sms,
                                                    int block_n, int* return_code);

/*
 * Activation quantizer: bf16 [M, x_ld] -> e4m3 [M, K] + fp32 scales (k-block-major, leading dimension
 * scales_ld >= M), 1 x 128 groups, scale = amax/448.  The reference names this component but holds no
 * code for it; the output feeds `lhs` / `lhs_scales` of the GEMM (yan/jit_kernels/gemm.py:23-25).
 */
void yan_b200_per_token_cast_to_fp8(const void* x, void* out, void* out_scales, int m, int k, int x_ld, int scales_ld,
                                    void* stream, int* return_code);

/* Weight quantizer: bf16 [N, K] -> e4m3 [N, K] + fp32 scales [N/128, K/128] (128 x 128 blocks); produces
 * `rhs` / `rhs_scales` (fp8_gemm.cuh:41,44). */
void yan_b200_per_block_cast_to_fp8(const void* w, void* out, void* out_scales, int n, int k, void* stream,
                                    int* return_code);

/*
 * Quantize-then-GEMM in one call: out = bf16( quant_1x128(a) . rhs^T ).  `workspace` is caller-owned
 * scratch of at least yan_b200_fp8_linear_workspace_bytes(m, k) bytes (256-byte aligned) that holds the
 * quantized activations and their scales between the two kernels.  This is the path the north-star
 * names end to end (bf16 A in, bf16 D out); the reference has no such function.
 */
size_t yan_b200_fp8_linear_workspace_bytes(int m, int k);
void yan_b200_fp8_linear_bf16(const void* a, const void* rhs, const void* rhs_scales, void* out, void* workspace,
                              size_t workspace_bytes, int m, int n, int k, int ldd, void* stream, int num_sms,
                              int block_n, int* return_code);

/*
 * Quantize-then-GEMM for callers that must not allocate.  No counterpart in the reference.
 *
 * Some hosts of this library cannot call cudaMalloc or let a framework allocator do it for them: a
 * serving loop that has handed all of its device memory to a KV-cache pool, a plugin running inside
 * another runtime's memory budget, code on a latency path where an allocation may synchronise the
 * device.  For them this variant of yan_b200_fp8_linear_bf16 keeps the intermediate (quantized
 * activations and their scales) in a fixed array inside the library's device image instead of a
 * caller-provided workspace.  Inputs and the output are still the caller's.
 *
 *   - Limit: m * k <= YAN_B200_STATIC_SCRATCH_MAX_ELEMENTS (8 Mi elements; 8.25 MiB of device memory
 *     per GPU that loads the library, held until the process exits).  Larger problems return
 *     YAN_B200_WORKSPACE_TOO_SMALL; use yan_b200_fp8_linear_bf16 with your own workspace instead.
 *   - The first call on each device looks up the array's device address (one cudaGetSymbolAddress, made
 *     with that device current).  Make that first call before any stream capture begins.
 *   - The call allocates and frees nothing and calls no allocating library routine.
 *   - All calls on a device share the one array, which keeps whatever the last call left there.  Nothing
 *     in it needs to start at zero (the quantizer rewrites every byte the GEMM reads), but two calls
 *     that overlap on the GPU -- different streams, or graphs replayed concurrently -- race on it.
 *     Order them on one stream or with events.
 */
#define YAN_B200_STATIC_SCRATCH_MAX_ELEMENTS (8u << 20)
void yan_b200_fp8_linear_bf16_static(const void* a, const void* rhs, const void* rhs_scales, void* out, int m, int n,
                                     int k, int ldd, void* stream, int num_sms, int block_n, int* return_code);

/*
 * Device status word of the current device: 0, or (YAN_B200_DEVICE_TIMEOUT << 8) | site when a bounded
 * device-side wait of the GEMM ran out.  Synchronises the device.  reset != 0 clears the word.
 * Plays the role of the reference's error conventions (yan/jit/template.py:134 return code;
 * comm/helper.h:26-53 CUDA_CHECK) for failures that only the device can see.
 */
void yan_b200_read_device_status(int* status, int reset, int* return_code);

/*
 * Self-test of the bounded-wait machinery: launches one tiny kernel whose only thread waits (at most timeout_ns,
 * <= 1 s) on an mbarrier nothing arrives on, so the wait runs out, the status word becomes
 * (YAN_B200_DEVICE_TIMEOUT << 8) | 15 and the kernel returns normally.  No counterpart in the reference (it has no
 * device-side waits outside CUTLASS).
 */
void yan_b200_wait_probe(unsigned long long timeout_ns, void* stream, int* return_code);

/*
 * Peer-mapped device memory inside one NVSwitch box (CUDA IPC), for the K-split GEMM's exchange step.  They stand in
 * for the NVSHMEM symmetric heap of the reference (comm/gemm_allreduce.cu:238-259: nvshmem_malloc / nvshmem_ptr).
 * yan_b200_ipc_export: handle (YAN_B200_IPC_HANDLE_BYTES bytes, to be sent to the other processes of the box) of the
 *   allocation that contains `ptr`, and the offset of `ptr` inside it.  The memory must come from cudaMalloc (the
 *   default allocator of PyTorch qualifies; its expandable segments do not).
 * yan_b200_ipc_open: maps another process's allocation into this process (peer access is enabled on first use);
 *   *base + offset is the peer's `ptr`.  yan_b200_ipc_close unmaps it.  None of the three touches a stream.
 */
#define YAN_B200_IPC_HANDLE_BYTES 64
void yan_b200_ipc_export(const void* ptr, void* handle, unsigned long long* offset, int* return_code);
void yan_b200_ipc_open(const void* handle, void** base, int* return_code);
void yan_b200_ipc_close(void* base, int* return_code);

/*
 * In-place allreduce (sum) of bf16 elements [elem_begin, elem_begin + elem_count) of `world` same-shaped buffers,
 * one per rank of the box: data[r] is rank r's buffer as seen from this process (data[rank] local, the others mapped
 * with yan_b200_ipc_open).  Every rank calls it with the same range.  Rank r sums the r-th 1/world of the range in
 * fp32 (rank order, one rounding) and stores the result into all buffers: plain peer loads and stores, no multimem.
 * Replaces the per-tile NVLS reduction of comm/gemm_allreduce.cu:57-60,339-401.
 * epoch != 0: signals[r] is rank r's zero-initialised 128-byte signal block (peer-mapped like data); the kernel waits
 *   on entry until every rank has reached the same epoch and on exit until every rank's stores have landed.  epoch
 *   must grow by one per call and counter_target must be the sum of num_ctas over all calls so far (this one
 *   included), identically on every rank.  Waits are bounded (yan_b200_set_wait_timeout_ns) and report
 *   (YAN_B200_DEVICE_TIMEOUT << 8) | 16 or 17 through the status word.
 * epoch == 0: no device-side waiting; the caller orders the ranks before and after the call.
 * elem_begin and elem_count are multiples of 8; 2 <= world <= 8; num_ctas > 0.
 * exclusive_sms == 0: CTAs of 512 threads, the faster shape when the collective has the GPU to itself.
 * exclusive_sms != 0: CTAs of 1024 threads that fill an SM each, so the collective occupies exactly num_ctas SMs and a
 *   GEMM running beside it on another stream (given the other SMs through its num_sms) is not displaced.
 */
void yan_b200_allreduce_bf16_two_shot(void* const* data, void* const* signals, int world, int rank,
                                      unsigned long long elem_begin, unsigned long long elem_count, unsigned int epoch,
                                      unsigned int counter_target, int num_ctas, int exclusive_sms, void* stream,
                                      int* return_code);

/*
 * The same allreduce with the sum formed inside the NVSwitch (multimem.ld_reduce / multimem.st, the instruction pair
 * of comm/gemm_allreduce.cu:57-60,386-395).  `multicast` is the multicast address of the ranks' buffers: memory
 * that every rank has bound to one multicast object (cuMulticastBindMem; torch.distributed._symmetric_memory provides
 * such allocations).  signals[r] are ordinary peer addresses as above.  Everything else as
 * yan_b200_allreduce_bf16_two_shot.
 */
void yan_b200_allreduce_bf16_in_switch(void* multicast, void* const* signals, int world, int rank,
                                       unsigned long long elem_begin, unsigned long long elem_count, unsigned int epoch,
                                       unsigned int counter_target, int num_ctas, int exclusive_sms, void* stream,
                                       int* return_code);

/*
 * Row-parallel (K-split) GEMM fused with its allreduce, tile by tile: what comm/gemm_allreduce.cu:339-410 does with
 * NVSHMEM tile collectives, on plain peer-mapped memory.
 *   _scatter: the GEMM of one rank's K shard; its epilogue stores every finished bf16 tile of m-block mb into the staging
 *             array of the rank that owns it, rank mb % world, at [rank][row][col] (stage[r]: rank r's
 *             [world][M][ldd] bf16 array as mapped into this process, 16-byte aligned) -- the reduce-scatter half of the
 *             allreduce, overlapped with the MMAs of the following tiles.  block_n 0, 128 or 256.
 *   _gather_staged: every rank sums, for the m-blocks it owns, the `world` staged copies (fp32 in rank order, one
 *             rounding: the two-shot kernel's arithmetic, bit for bit) and stores the rows to all ranks' outputs
 *             (data[r]: rank r's [rows][ld] bf16 buffer).  signals / epoch / counter_target as for the two-shot kernel
 *             (epoch > 0: the entry barrier is what tells a rank that every peer's tiles have landed).
 */
void yan_b200_gemm_fp8_fp8_bf16_nt_scatter(const void* lhs, const void* lhs_scales, const void* rhs, const void* rhs_scales,
                                           void* const* stage, int world, int rank, int m, int n, int k, int ldd,
                                           void* stream, int num_sms, int block_n, int* return_code);
void yan_b200_allreduce_bf16_gather_staged(const void* stage, void* const* data, void* const* signals, int world, int rank,
                                           int rows, int ld, unsigned int epoch, unsigned int counter_target,
                                           int num_ctas, void* stream, int* return_code);

/*
 * Programmatic dependent launch for the weight-streaming (M <= 64) kernel.  When enabled, that kernel is
 * launched with cudaLaunchAttributeProgrammaticStreamSerialization: its weight loads (rhs) may start while the
 * previous kernel of the stream is still running; activations, scales of the activations and the output are
 * only touched after the previous kernel has completed.  Enable it only when `rhs` / `rhs_scales` are not
 * written by the kernel that precedes the GEMM in its stream (true for inference weights).  Default: off.
 * While enabled, the quantizer inside yan_b200_fp8_linear_bf16(_static) is launched the same way: its launch overlaps
 * the tail of the previous kernel of the stream, and it waits for that kernel before it reads or writes anything.
 * No reference counterpart (the reference launches every kernel with plain <<<>>>, e.g.
 * yan/include/gemm/cute_gemm.cuh:373).
 */
void yan_b200_set_programmatic_dependent_launch(int enabled);

/*
 * Clock probe.  `device_buffer` = 16 int64 in device memory of the current device, or NULL to switch the probe off
 * (default).  While set, CTA 0 of every general-kernel GEMM launch writes {clock64, globaltimer ns} when it starts
 * ([0], [1]) and when it ends ([2], [3]); ([2]-[0]) / ([3]-[1]) is the SM clock in GHz the kernel really ran at, which
 * a millisecond-period NVML sample cannot show for a kernel of a millisecond or two.  A library built with
 * -DYAN_PHASE_STAMPS also fills [4..13] with per-role wait / work cycles of CTA 0 (slot list: include/gemm/fp8_gemm.cuh).
 * Follows the reference's in-kernel clock64 stamps (yan/include/flash_attn/flash_attn_tk.cuh:56-63,159-164).
 */
void yan_b200_set_clock_probe(void* device_buffer);

/* Sets the bound (nanoseconds, default 2e9) of every device-side wait of later GEMM launches. */
void yan_b200_set_wait_timeout_ns(unsigned long long timeout_ns);

/* Sets the bound (nanoseconds, default 1e10) of the waits between ranks in later allreduce launches.  It is separate
 * from the bound above because ranks drift apart by seconds for ordinary host-side reasons.  When such a wait runs out
 * the kernel leaves the data alone, records YAN_B200_DEVICE_TIMEOUT in the status word and still keeps its counters
 * and epoch flags in step with the host, so a later launch is not poisoned; the buffer's contents of that call are
 * undefined.  No reference counterpart (nvshmem's tile collectives wait without a bound,
 * comm/gemm_allreduce.cu:403-410). */
void yan_b200_set_collective_timeout_ns(unsigned long long timeout_ns);

#ifdef __cplusplus
}
#endif

#endif /* YAN_B200_H_ */
