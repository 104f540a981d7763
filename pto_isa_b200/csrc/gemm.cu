// fp16 x fp16 -> fp32 GEMM for sm_100a: the B200 form of the reference's GEMM tile program
// (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:67-230, paths relative to the
// reference root).  The mapping of its PTO instructions:
//   TLOAD    (GM -> L1 "Mat" tile, :91-102)      -> TMA bulk-tensor loads into 128B-swizzled shared memory,
//                                                   completion counted on an mbarrier
//   TEXTRACT (L1 -> L0A/L0B window, :106-115)    -> no data movement: the k-window of the staged tile is
//                                                   addressed by advancing the UMMA shared-memory descriptor
//   TMATMUL / TMATMUL_ACC (:27-35, :123-125)     -> tcgen05.mma.kind::f16, M128 x N256 x K16, fp32
//                                                   accumulator in tensor memory (256 columns per C tile)
//   TSTORE   (L0C -> GM, :131-149)               -> tcgen05.ld of the accumulator + 128-bit global stores
//   set_flag / wait_flag ping-pong (:151-165)    -> a 4-stage full/empty mbarrier ring between a TMA
//                                                   producer warp and an MMA issuer warp, and a 2-deep
//                                                   full/empty pair on the accumulators so the TSTORE of C
//                                                   tile i overlaps the k loop of tile i+1
// The base tile is the reference's 128 x 256 with a 64-wide k step.  CTAs are persistent: one per SM,
// each walking the C-tile list with a stride of the grid size.
//
// B is accepted in both layouts the path uses: k x n row-major (Layout::ND, an MN-major UMMA operand)
// and n x k row-major (Layout::DN view, a K-major UMMA operand).
#include "ptx.cuh"
#include "internal.h"

#include <mutex>

#include <cstdlib>
#include <cstring>

namespace pto_b200 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;           // 16 KiB
constexpr int kBBytes = BN * BK * 2;           // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes; // 48 KiB
constexpr int kThreads = 192;                  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kTmemCols = 512;                 // two 256-column accumulators

struct Control {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kSmemBytes = kStages * kStageBytes + sizeof(Control) + 1024; // + slack for 1 KiB alignment

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int &tm, int &tn)
{
    tm = t % tiles_m;
    tn = t / tiles_m;
}

template <int kBLayout>
__global__ void __launch_bounds__(kThreads, 1)
gemm_f16f32_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   float *__restrict__ c, int m, int n, int k, DeviceStatus *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Control *ctl = reinterpret_cast<Control *>(smem + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (m + BM - 1) / BM;
    const int tiles_n = (n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = (k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&ctl->acc_full[a], 1);
            mbar_init(&ctl->acc_empty[a], 4); // one arrival per epilogue warp
        }
        ctl->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(&ctl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int *abort_flag = &ctl->abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ TLOAD: TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, tiles_m, tm, tn);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + stage * kStageBytes;
                    uint8_t *sb = sa + kABytes;
                    mbar_arrive_expect_tx(&ctl->full[stage], kStageBytes);
                    tma_load_2d(sa, &tmap_a, &ctl->full[stage], kb * BK, tm * BM);
                    if (kBLayout == 1) {
                        tma_load_2d(sb, &tmap_b, &ctl->full[stage], kb * BK, tn * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) {
                            tma_load_2d(sb + j * (64 * BK * 2), &tmap_b, &ctl->full[stage], tn * BN + j * 64, kb * BK);
                        }
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ TEXTRACT + TMATMUL: MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BM, BN, 0, kBLayout == 0 ? 1 : 0);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(&ctl->acc_empty[acc], acc_phase ^ 1u, abort_flag)) {
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_base = smem_u32(smem + stage * kStageBytes);
                    const uint32_t b_base = a_base + kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // the 16-wide k window of the staged tiles (the TEXTRACT step)
                        const uint64_t a_desc = make_sw128_desc(a_base + kk * 32, 16, 1024);
                        const uint64_t b_desc = (kBLayout == 1)
                                                    ? make_sw128_desc(b_base + kk * 32, 16, 1024)
                                                    : make_sw128_desc(b_base + kk * (16 * 128), 64 * BK * 2, 1024);
                        tc_mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
                    }
                    tc_commit(&ctl->empty[stage]); // stage reusable once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                tc_commit(&ctl->acc_full[acc]); // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ TSTORE: epilogue warps
        const int quarter = warp & 3; // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = ((n & 3) == 0) && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0);
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            int tm, tn;
            tile_coords(t, tiles_m, tm, tn);
            if (!mbar_wait(&ctl->acc_full[acc], acc_phase, abort_flag)) {
                break;
            }
            tc_fence_after();
            const int row = tm * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            float *crow = c + static_cast<int64_t>(row) * n + static_cast<int64_t>(tn) * BN;
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + cb * 32, r);
                tmem_ld_wait();
                const int col0 = tn * BN + cb * 32;
                if (row < m) {
                    if (vec_ok && col0 + 32 <= n) {
                        float4 *dst = reinterpret_cast<float4 *>(crow + cb * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < n) {
                                crow[cb * 32 + j] = __uint_as_float(r[j]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->acc_empty[acc]);
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ctl->abort_flag) {
        // a wait gave up: give copies still in flight time to land before shared memory is released
        for (int i = 0; i < 1024; ++i) {
            __nanosleep(1000);
        }
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, kErrDeviceWaitTimeout) == 0) {
            status->block = blockIdx.x;
            status->where = 1;
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

} // namespace

int launch_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                       cudaStream_t stream, const float *bias)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0 || (b_layout != 0 && b_layout != 1)) {
        set_error_text("gemm: bad argument");
        return kErrBadArgument;
    }
    // TMA needs 16-byte aligned bases and row pitches that are multiples of 16 bytes
    if ((k % 8) != 0 || (b_layout == 0 && (n % 8) != 0) || (reinterpret_cast<uintptr_t>(a) & 15u) ||
        (reinterpret_cast<uintptr_t>(b) & 15u)) {
        set_error_text("gemm: k (and n for a k x n B) must be multiples of 8 and operands 16-byte aligned");
        return kErrUnsupportedShape;
    }
    // default: the kernel that puts two thread blocks on one 256 x 256 tile (gemm_2cta.cu);
    // PTO_B200_GEMM_MODE=1cta selects the one-block-per-tile kernel of this file
    static const bool one_block = [] {
        const char *e = getenv("PTO_B200_GEMM_MODE");
        return e != nullptr && strcmp(e, "1cta") == 0;
    }();
    if (!one_block) {
        return launch_gemm2_f16f32(a, b, c, m, n, k, b_layout, stream, bias);
    }
    if (bias != nullptr) {
        set_error_text("gemm: the bias form runs on the default kernel only (unset PTO_B200_GEMM_MODE)");
        return kErrUnsupportedShape;
    }
    CUtensorMap tmap_a, tmap_b;
    int rc = make_tmap_2d(&tmap_a, a, 2, m, k, k, BM, BK, true);
    if (rc != kOk) {
        return rc;
    }
    if (b_layout == 1) {
        rc = make_tmap_2d(&tmap_b, b, 2, n, k, k, BN, BK, true);
    } else {
        rc = make_tmap_2d(&tmap_b, b, 2, k, n, n, BK, 64, true);
    }
    if (rc != kOk) {
        return rc;
    }
    const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    DeviceStatus *status = device_status_ptr();
    if (status == nullptr) {
        return kErrCuda;
    }
    if (b_layout == 1) {
        if ((rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm_f16f32_kernel<1>), kSmemBytes)) != kOk) {
            return rc;
        }
        gemm_f16f32_kernel<1><<<grid, kThreads, kSmemBytes, stream>>>(tmap_a, tmap_b, c, m, n, k, status);
    } else {
        if ((rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm_f16f32_kernel<0>), kSmemBytes)) != kOk) {
            return rc;
        }
        gemm_f16f32_kernel<0><<<grid, kThreads, kSmemBytes, stream>>>(tmap_a, tmap_b, c, m, n, k, status);
    }
    return check_launch();
}

// ======================================================================================================
// Host-buffer GEMM that allocates nothing.
//
// For callers that must not (or cannot) allocate device memory at call time: a host process whose device
// memory is entirely owned by another allocator, so that a cudaMalloc of even a few bytes fails or
// fragments its pool; a plugin running under a policy that forbids allocation calls after start-up; or a
// latency-critical path where an allocation's implicit device synchronisation is not acceptable.  The
// regular entry points allocate on first use (the status record; the host variants also their staging
// buffers).  This one keeps everything it needs - the status record and the device copies of A, B and C -
// in one file-scope array that every GPU loading the library holds from module load until exit.
//
// Layout of the array: [0, 4096) header (the status record the kernel's bounded waits report into),
// then A, B and C, each rounded up to 256 bytes.  Problems that do not fit are rejected.
// All calls share the array and it keeps the previous call's contents: the status record is cleared at
// the start of every call, A and B are overwritten by the copies in, and every element of C that is
// copied out is written by the kernel.  Two calls that overlap on the GPU (from two threads or
// processes' worth of streams) would race on it; calls are serialised on the legacy default stream and
// the function returns only after its result has been copied out.
namespace {

constexpr size_t kStaticScratchBytes = 36u << 20; // 36 MiB per GPU
constexpr size_t kStaticHeaderBytes = 4096;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address is
// looked up once per device (with that device current) and cached here.
constexpr int kMaxDevicesStatic = 64;
unsigned char *g_static_scratch_addr[kMaxDevicesStatic] = {nullptr};
std::mutex g_static_mutex; // guards the table above

size_t round256(size_t x)
{
    return (x + 255u) & ~static_cast<size_t>(255u);
}

} // namespace

size_t gemm_static_scratch_bytes()
{
    return kStaticScratchBytes;
}

int gemm_f16f32_host_static(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0 || (b_layout != 0 && b_layout != 1)) {
        set_error_text("gemm_host_static: bad argument");
        return kErrBadArgument;
    }
    if ((k % 8) != 0 || (b_layout == 0 && (n % 8) != 0)) {
        set_error_text("gemm_host_static: k (and n for a k x n B) must be multiples of 8");
        return kErrUnsupportedShape;
    }
    // extents far beyond the scratch are turned away before any byte count is formed (no product can wrap)
    const bool huge = m > (1 << 20) || n > (1 << 20) || k > (1 << 20);
    const size_t a_bytes = static_cast<size_t>(m) * k * 2, b_bytes = static_cast<size_t>(n) * k * 2,
                 c_bytes = static_cast<size_t>(m) * n * 4;
    const size_t need = huge ? ~static_cast<size_t>(0)
                             : kStaticHeaderBytes + round256(a_bytes) + round256(b_bytes) + round256(c_bytes);
    if (need > kStaticScratchBytes) {
        set_error_text("gemm_host_static: A, B and C need %zu bytes of device staging but the built-in scratch holds "
                       "%zu (about m = n = k = 2048); use pto_b200_gemm_f16f32_host for larger problems",
                       need, kStaticScratchBytes);
        return kErrTooLarge;
    }
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc != kOk) {
        return rc;
    }
    if (dev < 0 || dev >= kMaxDevicesStatic) {
        set_error_text("gemm_host_static: device ordinal %d out of range", dev);
        return kErrBadArgument;
    }
    unsigned char *base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (g_static_scratch_addr[dev] == nullptr) {
            // one-time set-up for this device: resolve the array's device address and raise the kernels' dynamic
            // shared-memory limit.  Neither allocates, but CUDA loads a module's code and data when it is first
            // touched: this is the moment the array's 36 MiB are taken from the device, which is why the first call
            // belongs to start-up, before another allocator is handed the rest of the memory.
            unsigned char *p = nullptr;
            rc = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch),
                            "cudaGetSymbolAddress(static scratch; the first call on a device must run while the "
                            "device still has 36 MiB free)");
            if (rc != kOk) {
                return rc;
            }
            if ((rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm_f16f32_kernel<0>), kSmemBytes)) != kOk ||
                (rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm_f16f32_kernel<1>), kSmemBytes)) != kOk) {
                return rc;
            }
            g_static_scratch_addr[dev] = p;
        }
        base = g_static_scratch_addr[dev];
    }
    DeviceStatus *status = reinterpret_cast<DeviceStatus *>(base);
    uint16_t *da = reinterpret_cast<uint16_t *>(base + kStaticHeaderBytes);
    uint16_t *db = reinterpret_cast<uint16_t *>(base + kStaticHeaderBytes + round256(a_bytes));
    float *dc = reinterpret_cast<float *>(base + kStaticHeaderBytes + round256(a_bytes) + round256(b_bytes));
    cudaStream_t s = nullptr; // legacy default stream: serialises the calls that share the array

    // the tensor maps first: a failure here leaves nothing in flight
    CUtensorMap tmap_a, tmap_b;
    rc = make_tmap_2d(&tmap_a, da, 2, m, k, k, BM, BK, true);
    if (rc == kOk) {
        rc = (b_layout == 1) ? make_tmap_2d(&tmap_b, db, 2, n, k, k, BN, BK, true)
                             : make_tmap_2d(&tmap_b, db, 2, k, n, n, BK, 64, true);
    }
    if (rc != kOk) {
        return rc;
    }
    // from the first enqueue on, every error path waits for the stream: no copy may stay in flight on the caller's buffers
    auto fail = [&](int code) {
        cudaStreamSynchronize(s);
        return code;
    };
    // the status record must start at zero; everything else is overwritten before it is read
    if ((rc = check_cuda(cudaMemsetAsync(status, 0, sizeof(DeviceStatus), s), "cudaMemsetAsync(status)")) != kOk ||
        (rc = check_cuda(cudaMemcpyAsync(da, a, a_bytes, cudaMemcpyHostToDevice, s), "H2D A")) != kOk ||
        (rc = check_cuda(cudaMemcpyAsync(db, b, b_bytes, cudaMemcpyHostToDevice, s), "H2D B")) != kOk) {
        return fail(rc);
    }
    const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    if (b_layout == 1) {
        gemm_f16f32_kernel<1><<<grid, kThreads, kSmemBytes, s>>>(tmap_a, tmap_b, dc, m, n, k, status);
    } else {
        gemm_f16f32_kernel<0><<<grid, kThreads, kSmemBytes, s>>>(tmap_a, tmap_b, dc, m, n, k, status);
    }
    if ((rc = check_launch()) != kOk) {
        return fail(rc);
    }
    DeviceStatus host_status;
    if ((rc = check_cuda(cudaMemcpyAsync(c, dc, c_bytes, cudaMemcpyDeviceToHost, s), "D2H C")) != kOk ||
        (rc = check_cuda(cudaMemcpyAsync(&host_status, status, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, s),
                         "D2H status")) != kOk) {
        return fail(rc);
    }
    if ((rc = check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize")) != kOk) {
        return rc;
    }
    if (host_status.code != 0) {
        set_error_text("gemm_host_static: device-side wait gave up (code %d, block %d)", host_status.code,
                       host_status.block);
        return host_status.code;
    }
    return kOk;
}

} // namespace pto_b200
