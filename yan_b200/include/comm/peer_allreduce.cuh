#pragma once
// Two-shot allreduce of a bf16 tensor over peer-mapped memory inside one NVSwitch box: the exchange step of the
// K-split (row-parallel) GEMM, in place on the buffer the GEMM wrote its partial product to.
//
// The reference sums per-tile partials inside its GEMM epilogue through an NVSHMEM symmetric heap and NVLS multimem
// instructions (comm/gemm_allreduce.cu:57-60,339-401).  Here every rank's buffer is ordinary device memory that the
// other ranks of the box have mapped (CUDA IPC), and one kernel per rank does both halves of the collective:
//   reduce-scatter: rank r owns the r-th 1/W of the range; it loads that slice from all W buffers (coalesced 16-byte
//                   peer loads, all W in flight per thread), sums in fp32 in rank order and rounds to bf16 once;
//   all-gather    : it stores the result to the same slice of all W buffers.
// Inbound (loads) and outbound (stores) traffic run at the same time, NVLink being full duplex; per GPU
// (W-1)/W of the tensor crosses each direction once, the minimum for an allreduce without in-switch reduction.
// Plain ld/st on peer pointers only.  A second kernel does the same collective with multimem instructions (the sum
// is formed inside the switch) for buffers that are bound to a multicast object.
//
// Ordering between ranks, with epoch > 0, is part of the kernel: on entry a rank tells every peer that its partial
// is complete (st.release.sys of the epoch into the peer's `arrive` slot) and waits until all peers said so; on exit,
// after a system-scope fence, the last CTA tells every peer that its stores are done and waits for the same from
// all, so completion of the kernel on one rank means the whole tensor is final there.  Every wait is bounded by a
// wall-clock limit and reports through the status word; no CTA waits for another CTA of its own grid, so the kernel
// finishes whatever part of the GPU it is given.  With epoch == 0 the caller provides both barriers (e.g. with a
// collective of its communication library).

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../gemm/utils.cuh"

namespace yan {

constexpr int kMaxPeers = 8;
// Two CTA shapes.  512 threads with about sixteen 16-byte loads in flight per thread is the faster one when the
// collective has the GPU to itself (8 GPUs, 64 MiB: 196 us against 219 us).  1024 threads at <= 64 registers fill an SM,
// so a grid of n such CTAs occupies exactly n SMs however the hardware places it and a GEMM running beside the
// collective keeps the others (smaller CTAs are spread one per SM over the whole GPU and the persistent GEMM loses
// those SMs).  Bandwidth grows with the number of SMs issuing peer accesses -- an SM sustains roughly 20 GB/s of
// peer traffic -- so the collective is only link-bound from about 64 SMs up.
constexpr int kAllreduceThreads = 512;
constexpr int kAllreduceThreadsExclusive = 1024;

struct PeerPtrs {
    void* p[kMaxPeers];
};

// Layout of one rank's signal block (peer-mapped like the data; zero before first use).
struct PeerSignals {
    uint32_t arrive[kMaxPeers];  // arrive[r] = last epoch for which rank r's input is complete
    uint32_t done[kMaxPeers];    // done[r]   = last epoch for which rank r's stores are complete
    uint32_t cta_counter;        // CTAs of this rank that finished their stores, cumulative over launches
    uint32_t pad[15];
};

namespace comm_detail {

__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const uint4* addr) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Wait until *flag (local memory, written by a peer) has reached `epoch`.  Epochs only grow; the comparison is
// wrap-safe.  Returns false after timeout_ns.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns) {
    const uint64_t t0 = timer_ns();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
        if ((++spins & 0xFu) == 0 && timer_ns() - t0 > timeout_ns) return false;
    }
    return true;
}

__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}

}  // namespace comm_detail

// Entry barrier: tells every peer that this rank's input is complete and waits for the same from all.
// Returns false (after recording the status) when a wait ran out; the whole CTA gets the same answer.
template <int W>
__device__ __forceinline__ bool enter_collective(const PeerPtrs& signals, PeerSignals* my_signals, int rank,
                                                 uint32_t epoch, int* status, unsigned long long timeout_ns) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < W)
        comm_detail::st_release_sys(&static_cast<PeerSignals*>(signals.p[threadIdx.x])->arrive[rank], epoch);
    if (threadIdx.x < W && !comm_detail::wait_flag(&my_signals->arrive[threadIdx.x], epoch, timeout_ns)) {
        s_ok = 0;
        if (status != nullptr) atomicCAS(status, 0, (static_cast<int>(kDeviceTimeout) << 8) | 16);
    }
    __syncthreads();
    return s_ok != 0;
}

// Exit barrier: after a system-scope fence by every thread, the last CTA of the grid tells every peer that this rank's
// stores are done and waits for the same from all.  A CTA whose entry wait ran out (`entered` false) still counts
// itself and the last one still publishes `done`, so the CTA counter and the epoch flags stay in step with the host's
// bookkeeping and the next launch works; it does not wait for the peers a second time.
template <int W>
__device__ __forceinline__ void leave_collective(const PeerPtrs& signals, PeerSignals* my_signals, int rank,
                                                 uint32_t epoch, uint32_t counter_target, int* status,
                                                 unsigned long long timeout_ns, bool entered = true) {
    __shared__ int s_last;
    comm_detail::fence_sys();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&my_signals->cta_counter, 1u) + 1u == counter_target);
    __syncthreads();
    if (s_last && threadIdx.x < W) {
        comm_detail::fence_sys();
        comm_detail::st_release_sys(&static_cast<PeerSignals*>(signals.p[threadIdx.x])->done[rank], epoch);
        if (entered && !comm_detail::wait_flag(&my_signals->done[threadIdx.x], epoch, timeout_ns) && status != nullptr)
            atomicCAS(status, 0, (static_cast<int>(kDeviceTimeout) << 8) | 17);
    }
}

// vec_begin / vec_count: the range to reduce, in 16-byte vectors (8 bf16) from the start of every buffer.
template <int W, int kThreads>
__global__ void __launch_bounds__(kThreads)
    two_shot_allreduce_bf16_kernel(const PeerPtrs data, const PeerPtrs signals, const int rank, const size_t vec_begin,
                                   const size_t vec_count, const uint32_t epoch, const uint32_t counter_target,
                                   int* status, const unsigned long long timeout_ns) {
    static_assert(W >= 2 && W <= kMaxPeers, "one NVSwitch box");
    PeerSignals* my_signals = static_cast<PeerSignals*>(signals.p[rank]);
    // inputs incomplete after the bound: leave the buffers alone (the host reads the status word), keep the counters right
    if (epoch != 0 && !enter_collective<W>(signals, my_signals, rank, epoch, status, timeout_ns)) {
        leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns, false);
        return;
    }

    // ---- this rank's slice: loads from all W buffers, one fp32 sum in rank order, stores to all W buffers ----
    const size_t per_rank = (vec_count + W - 1) / W;
    const size_t first = vec_begin + static_cast<size_t>(rank) * per_rank;
    const size_t last = (first + per_rank < vec_begin + vec_count) ? first + per_rank : vec_begin + vec_count;
    // kUnroll vectors per thread and trip, all kUnroll * W loads issued before the first use (what the register
    // budget of the CTA shape allows: about 16 vectors at 512 threads, 8 at 1024).
    constexpr int kVectors = (kThreads <= 512) ? 16 : 8;
    constexpr int kUnroll = (kVectors / W) > 0 ? (kVectors / W) : 1;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < last;
         i0 += stride * kUnroll) {
        uint4 v[kUnroll][W];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < last) {
#pragma unroll
                for (int r = 0; r < W; ++r) v[u][r] = comm_detail::ld_sys_v4(static_cast<const uint4*>(data.p[r]) + i);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < last) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < W; ++r) comm_detail::accumulate(acc, v[u][r]);
                uint4 o;
                __nv_bfloat162 t;
                t = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
#pragma unroll
                for (int r = 0; r < W; ++r) {
                    const int peer = (rank + r) % W;  // spread the ranks over the destinations at any instant
                    static_cast<uint4*>(data.p[peer])[i] = o;
                }
            }
        }
    }

    if (epoch != 0) leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns);
}

// The same collective with the sum formed inside the NVSwitch: `mc` is the multicast address of the buffers (memory
// bound to one multicast object on all ranks).  multimem.ld_reduce returns the sum over all ranks' copies of a vector
// (fp32 accumulation in the switch), multimem.st writes the result to all copies.  Per GPU about (1 + 1/W) of the
// tensor crosses each NVLink direction instead of 2 (W-1)/W: at W = 8, 1.125 against 1.75.  This is the instruction
// pair the reference's epilogue uses (comm/gemm_allreduce.cu:57-60,386-395).
template <int W, int kThreads>
__global__ void __launch_bounds__(kThreads)
    in_switch_allreduce_bf16_kernel(uint4* mc, const PeerPtrs signals, const int rank, const size_t vec_begin,
                                    const size_t vec_count, const uint32_t epoch, const uint32_t counter_target,
                                    int* status, const unsigned long long timeout_ns) {
    PeerSignals* my_signals = static_cast<PeerSignals*>(signals.p[rank]);
    if (epoch != 0 && !enter_collective<W>(signals, my_signals, rank, epoch, status, timeout_ns)) {
        leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns, false);
        return;
    }

    const size_t per_rank = (vec_count + W - 1) / W;
    const size_t first = vec_begin + static_cast<size_t>(rank) * per_rank;
    const size_t last = (first + per_rank < vec_begin + vec_count) ? first + per_rank : vec_begin + vec_count;
    // vectors per thread and trip.  Measured on 64 MiB: 4 ranks 169 / 173 / 182 / 192 us with 1 / 2 / 4 / 8, 8 ranks
    // 171-191 us with 4 and 207 us with 8: more loads in flight per thread do not help, more (shorter) trips do a little,
    // because the stores of one trip then overlap the loads of the next.
#ifndef YAN_IN_SWITCH_UNROLL
#define YAN_IN_SWITCH_UNROLL 2
#endif
    constexpr int kUnroll = YAN_IN_SWITCH_UNROLL;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < last;
         i0 += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < last)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                             : "l"(mc + i)
                             : "memory");
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < last)
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc + i),
                             "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w)
                             : "memory");
        }
    }

    if (epoch != 0) leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns);
}

// Second half of the allreduce whose first half ran inside the GEMM epilogue (fp8_gemm_kernel's scatter instance): the
// tiles of m-block mb were stored by every rank into the staging array of rank mb % W, at [source rank][row][col].
// This kernel sums, for the rows this rank owns, the W staged copies (local loads only; fp32 in rank order, one
// rounding -- the arithmetic of the two-shot kernel, bit for bit) and stores the result to the same rows of all W
// output buffers.  Per GPU only the all-gather half, (W-1)/W of the tensor outbound, crosses NVLink here; the
// reduce-scatter half crossed it tile by tile while the MMAs ran.  Entry / exit ordering as in the two-shot kernel.
// stage: this rank's [W][rows][ld / 8] array of 16-byte vectors; data.p[r]: rank r's [rows][ld / 8] output.
template <int W, int kThreads>
__global__ void __launch_bounds__(kThreads)
    gather_staged_allreduce_bf16_kernel(const uint4* __restrict__ stage, const PeerPtrs data, const PeerPtrs signals,
                                        const int rank, const uint32_t rows, const uint32_t vectors_per_row,
                                        const uint32_t epoch, const uint32_t counter_target, int* status,
                                        const unsigned long long timeout_ns) {
    static_assert(W >= 2 && W <= kMaxPeers, "one NVSwitch box");
    PeerSignals* my_signals = static_cast<PeerSignals*>(signals.p[rank]);
    if (epoch != 0 && !enter_collective<W>(signals, my_signals, rank, epoch, status, timeout_ns)) {
        leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns, false);
        return;
    }
    constexpr uint32_t kRowsPerBlock = 128;  // the GEMM's BLOCK_M: ownership goes by m-blocks
    const uint32_t num_m_blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
    const uint32_t owned_blocks = (num_m_blocks > static_cast<uint32_t>(rank)) ? (num_m_blocks - rank + W - 1) / W : 0;
    const size_t total = static_cast<size_t>(owned_blocks) * kRowsPerBlock * vectors_per_row;
    const size_t copy_stride = static_cast<size_t>(rows) * vectors_per_row;  // one source rank's [rows][ld] copy
    constexpr int kVectors = (kThreads <= 512) ? 16 : 8;
    constexpr int kUnroll = (kVectors / W) > 0 ? (kVectors / W) : 1;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * kUnroll) {
        uint4 v[kUnroll][W];
        size_t at[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            at[u] = static_cast<size_t>(-1);
            if (i < total) {
                const size_t owned_row = i / vectors_per_row, col = i - owned_row * vectors_per_row;
                const size_t row = ((owned_row / kRowsPerBlock) * W + rank) * kRowsPerBlock + owned_row % kRowsPerBlock;
                if (row < rows) {
                    at[u] = row * vectors_per_row + col;
#pragma unroll
                    for (int r = 0; r < W; ++r) v[u][r] = comm_detail::ld_sys_v4(stage + r * copy_stride + at[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (at[u] != static_cast<size_t>(-1)) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < W; ++r) comm_detail::accumulate(acc, v[u][r]);
                uint4 o;
                __nv_bfloat162 t;
                t = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
#pragma unroll
                for (int r = 0; r < W; ++r) {
                    const int peer = (rank + r) % W;
                    static_cast<uint4*>(data.p[peer])[at[u]] = o;
                }
            }
        }
    }
    if (epoch != 0) leave_collective<W>(signals, my_signals, rank, epoch, counter_target, status, timeout_ns);
}

struct AllreduceArgs {
    PeerPtrs data{};     // the same-shaped bf16 buffer on every rank; entry [rank] is local, the others peer-mapped
    void* multicast = nullptr;  // in-switch form only: the multicast address of the buffers (data is then unused)
    PeerPtrs signals{};  // PeerSignals blocks, same convention; unused when epoch == 0
    int world = 0, rank = 0;
    size_t elem_begin = 0, elem_count = 0;  // range in bf16 elements, both multiples of 8
    uint32_t epoch = 0;                     // 0: the caller orders the ranks; otherwise a per-launch growing number
    uint32_t counter_target = 0;            // sum of the grid sizes of all launches so far on this rank, this one included
    int num_ctas = 0;                       // grid size (> 0)
    bool exclusive = false;                 // true: 1024-thread CTAs, one per SM: the grid occupies exactly num_ctas SMs
    int* status = nullptr;
    unsigned long long timeout_ns = 2000000000ull;
    // gather_staged form only: this rank's staging array and the matrix shape (rows, row pitch in bf16 elements)
    const void* stage = nullptr;
    uint32_t rows = 0, ld = 0;
};

inline int launch_gather_staged_allreduce_bf16(const AllreduceArgs& a, cudaStream_t stream) {
    if (a.world < 2 || a.world > kMaxPeers || a.rank < 0 || a.rank >= a.world || a.num_ctas <= 0) return kBadArgument;
    if (a.stage == nullptr || reinterpret_cast<uintptr_t>(a.stage) % 16 != 0 || a.rows == 0 || a.ld == 0 || a.ld % 8 != 0 ||
        a.epoch == 0)
        return kBadArgument;
    for (int r = 0; r < a.world; ++r) {
        if (a.data.p[r] == nullptr || reinterpret_cast<uintptr_t>(a.data.p[r]) % 16 != 0) return kBadArgument;
        if (a.signals.p[r] == nullptr || reinterpret_cast<uintptr_t>(a.signals.p[r]) % 4 != 0) return kBadArgument;
    }
    const dim3 grid(static_cast<unsigned>(a.num_ctas));
    const uint4* stage = static_cast<const uint4*>(a.stage);
#define YAN_LAUNCH_GATHER(W)                                                                                          \
    gather_staged_allreduce_bf16_kernel<W, kAllreduceThreads><<<grid, kAllreduceThreads, 0, stream>>>(                \
        stage, a.data, a.signals, a.rank, a.rows, a.ld / 8, a.epoch, a.counter_target, a.status, a.timeout_ns)
    switch (a.world) {
        case 2: YAN_LAUNCH_GATHER(2); break;
        case 3: YAN_LAUNCH_GATHER(3); break;
        case 4: YAN_LAUNCH_GATHER(4); break;
        case 5: YAN_LAUNCH_GATHER(5); break;
        case 6: YAN_LAUNCH_GATHER(6); break;
        case 7: YAN_LAUNCH_GATHER(7); break;
        default: YAN_LAUNCH_GATHER(8); break;
    }
#undef YAN_LAUNCH_GATHER
    return cudaGetLastError() == cudaSuccess ? kOk : kCommFailed;
}

inline int launch_two_shot_allreduce_bf16(const AllreduceArgs& a, cudaStream_t stream) {
    if (a.world < 2 || a.world > kMaxPeers || a.rank < 0 || a.rank >= a.world || a.num_ctas <= 0) return kBadArgument;
    if (a.elem_begin % 8 != 0 || a.elem_count % 8 != 0 || a.elem_count == 0) return kBadArgument;
    if (a.multicast != nullptr && reinterpret_cast<uintptr_t>(a.multicast) % 16 != 0) return kBadArgument;
    for (int r = 0; r < a.world; ++r) {
        if (a.multicast == nullptr && (a.data.p[r] == nullptr || reinterpret_cast<uintptr_t>(a.data.p[r]) % 16 != 0))
            return kBadArgument;
        if (a.epoch != 0 && (a.signals.p[r] == nullptr || reinterpret_cast<uintptr_t>(a.signals.p[r]) % 4 != 0))
            return kBadArgument;
    }
    const size_t vb = a.elem_begin / 8, vc = a.elem_count / 8;
    const dim3 grid(static_cast<unsigned>(a.num_ctas));
#define YAN_LAUNCH_ALLREDUCE(W, T)                                                                                  \
    if (a.multicast != nullptr)                                                                                     \
        in_switch_allreduce_bf16_kernel<W, T><<<grid, T, 0, stream>>>(static_cast<uint4*>(a.multicast), a.signals,  \
                                                                      a.rank, vb, vc, a.epoch, a.counter_target,    \
                                                                      a.status, a.timeout_ns);                      \
    else                                                                                                            \
        two_shot_allreduce_bf16_kernel<W, T><<<grid, T, 0, stream>>>(a.data, a.signals, a.rank, vb, vc, a.epoch,    \
                                                                     a.counter_target, a.status, a.timeout_ns)
#define YAN_LAUNCH_ALLREDUCE_W(W)                                          \
    if (a.exclusive) {                                                     \
        YAN_LAUNCH_ALLREDUCE(W, kAllreduceThreadsExclusive);               \
    } else {                                                               \
        YAN_LAUNCH_ALLREDUCE(W, kAllreduceThreads);                        \
    }
    switch (a.world) {
        case 2: YAN_LAUNCH_ALLREDUCE_W(2) break;
        case 3: YAN_LAUNCH_ALLREDUCE_W(3) break;
        case 4: YAN_LAUNCH_ALLREDUCE_W(4) break;
        case 5: YAN_LAUNCH_ALLREDUCE_W(5) break;
        case 6: YAN_LAUNCH_ALLREDUCE_W(6) break;
        case 7: YAN_LAUNCH_ALLREDUCE_W(7) break;
        default: YAN_LAUNCH_ALLREDUCE_W(8) break;
    }
#undef YAN_LAUNCH_ALLREDUCE_W
#undef YAN_LAUNCH_ALLREDUCE
    return cudaGetLastError() == cudaSuccess ? kOk : kCommFailed;
}

}  // namespace yan
