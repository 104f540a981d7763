// Per-block execution context of the PTO backend for B200, and the host-side launch helper.
//
// One thread block (256 threads) is one "AI core".  All threads run the same instruction stream of the
// tile program; every PTO instruction is executed cooperatively by the block.  Dynamic shared memory holds
//   [ control | arena ]
// control = the tensor-memory base, the table of flags (one mbarrier per (source pipe, destination pipe,
// event id), the direct counterpart of the reference's set_flag / wait_flag, include/pto/common/cpu_stub.hpp:
// 85-86 and docs/coding/Event.md in the reference) and each warp's flag phases; arena = the space that TASSIGN
// addresses index into.  The NPU has separate address spaces for L1 / UB (Mat and Vec tiles), L0A (Left) and
// L0B (Right), each starting at 0; here they are windows of the one arena:
//   Vec, Mat : [0, PTO_B200_L0A_OFFSET)            default 96 KiB  (two 128x64 + two 64x256 fp16 staging tiles)
//   Left     : [PTO_B200_L0A_OFFSET, PTO_B200_L0B_OFFSET)   48 KiB  (ping at 0, pong at 32 KiB, 16 KiB each)
//   Right    : [PTO_B200_L0B_OFFSET, end of arena)          64 KiB+ (ping at 0, pong at 32 KiB, 32 KiB each)
//   Bias     : a 1 KiB table in the control block (one row of up to 256 floats for TMATMUL_BIAS)
// Define the two macros before including the PTO headers to move the windows.
// 512 tensor-memory columns are allocated per block for Acc tiles.
#pragma once

#include <cuda.h>

#include "tile.hpp"

namespace pto {
namespace b200 {

#ifndef PTO_B200_L0A_OFFSET
#define PTO_B200_L0A_OFFSET (96 * 1024)
#endif
#ifndef PTO_B200_L0B_OFFSET
#define PTO_B200_L0B_OFFSET (144 * 1024)
#endif

constexpr int kBlockThreads = 256;
constexpr int kNumPipes = 8;
constexpr int kNumFlags = kNumPipes * kNumPipes * EVENT_ID_MAX; // 512
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct Control {
    uint32_t tmem_base;
    int abort_flag;
    int error_code;
    int pad;
    uint64_t flags[kNumFlags];
    uint32_t phase[kNumFlags / 32][kBlockThreads / 32]; // phase bit of every flag, per warp
    uint8_t bias_table[1024];                            // the address space of TileType::Bias tiles (the NPU's bias table)
};
constexpr int kControlBytes = ((int)sizeof(Control) + 1023) / 1024 * 1024;
constexpr int kDefaultSmemBytes = 227 * 1024; // 1 KiB alignment slack + control (6 KiB) + 220 KiB arena

#if PTO_B200_DEVICE_CODE
__device__ __forceinline__ uint8_t *smem_base()
{
    extern __shared__ uint8_t pto_b200_dynamic_smem[];
    return reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(pto_b200_dynamic_smem) + 1023) & ~uintptr_t(1023));
}
__device__ __forceinline__ Control *control()
{
    return reinterpret_cast<Control *>(smem_base());
}
__device__ __forceinline__ uint8_t *arena()
{
    return smem_base() + kControlBytes;
}
// start of the window of the arena that tiles of a location index into
template <TileType Loc>
__device__ __forceinline__ uint8_t *arena_of()
{
    if constexpr (Loc == TileType::Bias) {
        return control()->bias_table;
    } else {
        return arena() + (Loc == TileType::Left ? PTO_B200_L0A_OFFSET : (Loc == TileType::Right ? PTO_B200_L0B_OFFSET : 0));
    }
}
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ int flag_index(int src, int dst, int id)
{
    return ((src & 7) * kNumPipes + (dst & 7)) * EVENT_ID_MAX + (id & 7);
}

// ---- mbarrier primitives (bounded waits: a wait that runs out raises the block's abort flag)
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrives once all cp.async copies issued so far by this thread have landed
__device__ __forceinline__ void mbar_arrive_after_copies(uint64_t *bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    volatile int *abort_flag = &control()->abort_flag;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
                return false;
            }
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > kWaitLimitNs) {
                break; // two seconds on the global timer: give up instead of hanging the device
            }
            if (i > 4096) {
                __nanosleep(64);
            }
        }
    }
    *abort_flag = 1;
    return false;
}

// ---- tcgen05 helpers
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Block prologue / epilogue (called by the launch trampoline, not by tile programs).
__device__ __forceinline__ void block_begin()
{
    Control *ctl = control();
    const int nthreads = blockDim.x;
    for (int f = threadIdx.x; f < kNumFlags; f += nthreads) {
        // a flag raised by the matrix pipe is signalled by one tcgen05.commit; every other pipe's work is
        // done by all threads, so all of them arrive
        const int src = f / (kNumPipes * EVENT_ID_MAX);
        mbar_init(&ctl->flags[f], src == PIPE_M ? 1u : static_cast<uint32_t>(nthreads));
    }
    if ((threadIdx.x & 31) == 0) {
        for (int w = 0; w < kNumFlags / 32; ++w) {
            ctl->phase[w][threadIdx.x >> 5] = 0;
        }
    }
    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        ctl->error_code = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
}

__device__ __forceinline__ void block_end(int *status)
{
    asm volatile("cp.async.wait_all;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    Control *ctl = control();
    if (ctl->abort_flag && threadIdx.x == 0 && status != nullptr) {
        atomicCAS(status, 0, 4); // a bounded wait gave up
    }
    if (threadIdx.x < 32) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(ctl->tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}
#endif // PTO_B200_DEVICE_CODE

// The real kernel that hosts a tile program.  It is declared here, before `__global__` loses its CUDA
// meaning for the rest of the translation unit (see pto-inst.hpp).
template <typename Program>
__global__ void __launch_bounds__(kBlockThreads, 1) block_kernel(Program program, int *status)
{
#if PTO_B200_DEVICE_CODE
    block_begin();
    program();
    block_end(status);
#endif
}

// Launches `program` (a __device__ callable) on `blocks` thread blocks of the stream.  `status`, if given,
// is a device word that receives 4 when a block gave up on a flag wait.
template <typename Program>
inline cudaError_t launch(uint32_t blocks, void *stream, Program program, int *status = nullptr,
                          int smem_bytes = kDefaultSmemBytes)
{
    cudaError_t e = cudaFuncSetAttribute(block_kernel<Program>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    block_kernel<Program><<<blocks, kBlockThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(program, status);
    return cudaGetLastError();
}

} // namespace b200
} // namespace pto

// Launch statement for kernels written in the reference's style.  `kernel` is the parenthesised kernel
// name (with its template arguments), followed by the block count, the stream and the kernel's arguments.
#define PTO_B200_LAUNCH(kernel, blocks, stream, ...) \
    (void)pto::b200::launch((blocks), (stream), [=] __device__() { kernel(__VA_ARGS__); })

// ---------------------------------------------------------------- block id, flags
PTO_INTERNAL uint32_t get_block_idx()
{
#if PTO_B200_DEVICE_CODE
    return blockIdx.x;
#else
    return 0;
#endif
}
PTO_INTERNAL uint32_t get_block_num()
{
#if PTO_B200_DEVICE_CODE
    return gridDim.x;
#else
    return 1;
#endif
}

// set_flag(src, dst, id): the flag is raised once everything issued so far on pipe `src` is complete.
//   PIPE_M    : tcgen05.commit by the issuing thread (covers all earlier tcgen05.mma)
//   PIPE_MTE2 : every thread arrives when its own asynchronous copies have landed
//   others    : their work is synchronous per thread, every thread arrives
PTO_INTERNAL void set_flag(pipe_t src, pipe_t dst, event_t id)
{
#if PTO_B200_DEVICE_CODE
    uint64_t *bar = &pto::b200::control()->flags[pto::b200::flag_index(src, dst, id)];
    if (src == PIPE_M) {
        if (threadIdx.x == 0) {
            pto::b200::tc_commit(bar);
        }
    } else if (src == PIPE_MTE2) {
        pto::b200::mbar_arrive_after_copies(bar);
    } else {
        // shared-memory writes of this thread become visible to the tensor core's (asynchronous-proxy) reads
        pto::b200::fence_async_proxy();
        pto::b200::tc_fence_before();
        pto::b200::mbar_arrive(bar);
    }
#else
    (void)src;
    (void)dst;
    (void)id;
#endif
}

// wait_flag(src, dst, id): every thread waits for the matching set_flag (the n-th wait pairs with the n-th set).
PTO_INTERNAL void wait_flag(pipe_t src, pipe_t dst, event_t id)
{
#if PTO_B200_DEVICE_CODE
    pto::b200::Control *ctl = pto::b200::control();
    const int f = pto::b200::flag_index(src, dst, id);
    // all lanes of a warp run the same instruction stream, so the phase is kept once per warp
    volatile uint32_t *word = &ctl->phase[f >> 5][threadIdx.x >> 5];
    const uint32_t bit = 1u << (f & 31);
    const uint32_t parity = (*word & bit) ? 1u : 0u;
    pto::b200::mbar_wait(&ctl->flags[f], parity);
    __syncwarp();
    if ((threadIdx.x & 31) == 0) {
        *word ^= bit;
    }
    __syncwarp();
    pto::b200::tc_fence_after();
    pto::b200::fence_async_proxy();
#else
    (void)src;
    (void)dst;
    (void)id;
#endif
}

PTO_INTERNAL void pipe_barrier(pipe_t pipe)
{
    (void)pipe;
#if PTO_B200_DEVICE_CODE
    __syncthreads();
#endif
}
