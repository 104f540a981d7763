// fp16 x fp16 -> fp32 GEMM for sm_100a on CTA pairs (tcgen05 cta_group::2): the same mapping of the reference's
// GEMM tile program as gemm.cu (TLOAD -> TMA, TEXTRACT -> descriptor window, TMATMUL -> tcgen05.mma, TSTORE ->
// tcgen05.ld + stores, flags -> mbarrier rings), with two thread blocks of a cluster working on one
// 256 x 256 C tile.  Each block stages its own 128 rows of A and only *half* of the B tile per k step
// (for a 128-deep k step 64 KiB instead of 96 KiB: a ring of three stages), the MMA of the pair reads both
// halves, so the L2 -> SM traffic per FLOP drops by a third.  Each block ends up with 128 rows x 256 columns
// of the accumulator in its own tensor memory and stores them itself.
//
// Cross-block signalling (no multicast anywhere):
//   full[s]   lives in the leader (rank 0): both blocks' TMA loads complete their bytes on it
//   empty[s]  one per block: the leader commits the MMAs of a stage to its own and to the peer's barrier
//   acc_full  one per block, committed the same way; acc_empty lives in the leader, the peer's epilogue
//             warps arrive on it remotely.
#include "ptx.cuh"
#include "internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace pto_b200 {

namespace {

constexpr int BM = 128;       // rows of A / C per block (256 per pair)
// Columns of C per pair (kBN): 256, or 128 for problems whose 256-wide tiles would leave block pairs idle
// (launch_pair_auto); a block stages kBN / 2 columns of B.
#ifndef PTO_B200_GEMM2_BK
#define PTO_B200_GEMM2_BK 128
#endif
constexpr int kBaseBK = PTO_B200_GEMM2_BK; // k extent of a stage of the 256-column instance
constexpr int kBoxK = 64;                  // k extent of one TMA box (128 bytes, the swizzle span)
constexpr int kMaxStages = 4;
constexpr int kThreads = 192; // warp 0 TMA, warp 1 MMA (leader only), warps 2..5 epilogue
constexpr int kTmemCols = 512;

struct Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// TSTORE staging: each epilogue warp owns two 32 x 32 fp32 slabs (4 KiB, 128-byte rows, 128-byte swizzle) that it
// fills from tensor memory and hands to a TMA store, so that the accumulator leaves the SM as full 128-byte
// lines issued by one instruction instead of 32 row-strided stores per register.
constexpr int kSlabBytes = 32 * 32 * 4;
constexpr int kStagingBytes = 4 * 2 * kSlabBytes;
// what follows from the tile width
template <int kBN>
struct Shape {
    static constexpr int BN = kBN;
    static constexpr int BNH = kBN / 2;                                           // columns of B staged per block
    // k extent of a stage = BK / 16 products per full / empty barrier round trip.  A stage of the narrow instance is
    // twice as deep: its products take half as long, and the per-stage costs of the loading and the issuing thread
    // (about 580 and 320 cycles) hide behind 1024 cycles of products, not behind 512.
    static constexpr int BK = (kBN == 128) ? 2 * kBaseBK : kBaseBK;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kStages = (192 * 1024) / ((BM + BNH) * BK * 2);          // 3 (256 wide) or 2 (128 wide)
    static constexpr int kBBytes = BNH * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + static_cast<int>(sizeof(Control)) + 1024;
    static_assert(kStages >= 2 && kStages <= kMaxStages && BNH % 64 == 0, "tile width");
};

// C tiles are walked in bands of kGroupN tile columns; inside a band the tile column moves fastest, then the
// tile row, so that the tiles in flight at any time (one per block pair: 74 tiles = about nine tile rows of a
// band) form a roughly square patch whose A and B panels stay in L2.
constexpr int kGroupN = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn)
{
    const int band = t / (kGroupN * tiles_m);
    const int first_n = band * kGroupN;
    const int width = (tiles_n - first_n) < kGroupN ? (tiles_n - first_n) : kGroupN;
    const int in_band = t - band * kGroupN * tiles_m;
    tm = in_band / width;
    tn = first_n + in_band % width;
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `p` (a location in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(const void *p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}

__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// commit of the pair's MMAs to a barrier given by its shared::cluster address
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}

// TMA load whose completion bytes are counted on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, uint32_t leader_bar, int c0,
                                                 int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(void *smem_dst, const CUtensorMap *map, uint32_t leader_bar, int c0,
                                                      int c1, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}

// L2 residency: the operands are read by many block pairs and should stay in L2, C is written once and should leave it
// first.  PTO_B200_GEMM2_L2_HINTS: 0 none, 1 C stores evict-first, 2 also operand loads evict-last.  Measured at 6144^3
// in one process, three libraries interleaved: 1405 / 1415 / 1419 TFLOP/s for eight launches after a pause and no
// difference beyond the run-to-run drift of the power-capped loop (1240 - 1420 for all three), so the default is 0.
#ifndef PTO_B200_GEMM2_L2_HINTS
#define PTO_B200_GEMM2_L2_HINTS 0
#endif
#if PTO_B200_GEMM2_L2_HINTS >= 2
#define PTO_GEMM2_LOAD(dst, map, bar, c0, c1) tma_load_2d_pair_hint(dst, map, bar, c0, c1, l2_policy_evict_last())
#else
#define PTO_GEMM2_LOAD(dst, map, bar, c0, c1) tma_load_2d_pair(dst, map, bar, c0, c1)
#endif
#if PTO_B200_GEMM2_L2_HINTS >= 1
#define PTO_GEMM2_STORE(map, src, c0, c1) tma_store_2d_hint(map, src, c0, c1, l2_policy_evict_first())
#else
#define PTO_GEMM2_STORE(map, src, c0, c1) tma_store_2d(map, src, c0, c1)
#endif

__device__ __forceinline__ void tc_mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// the same instruction on signed 8-bit operands with 32-bit integer accumulation (k = 32 per instruction)
__device__ __forceinline__ void tc_mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// instruction descriptor of kind::i8: signed 8-bit A and B (K-major), 32-bit integer accumulator
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// kMode: bit 0 = layout of B (0: k x n, 1: n x k), bit 1 = the TMATMUL_BIAS epilogue, bit 2 = int8 operands with an
// int32 result (TMATMUL's (int8, int8 -> int32) form, include/pto/cpu/TMatmul.hpp:46-51).  In the int8 form the rows
// of A and B are handed to TMA as 16-bit elements, two int8 each, so `k` and every k coordinate below count pairs:
// a 128-byte box is 64 of them, and an MMA still advances 32 bytes (32 int8, its k extent) inside the box.  The
// accumulator words go out bit for bit, as in the float form.  Bits 3-4 = 16-bit output: the accumulator is rounded
// (nearest even) to fp16 (1) or bf16 (2) before it is stored, the conversion TSTORE offers on the way out of the
// accumulator (docs/isa/TSTORE.md:67-72 in the reference).
template <int kMode, int kBN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2_f16f32_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, int c_by_tma, float *__restrict__ c,
                    const float *__restrict__ bias, int m, int n, int k, DeviceStatus *status)
{
    constexpr int BN = Shape<kBN>::BN, BNH = Shape<kBN>::BNH, kStages = Shape<kBN>::kStages;
    constexpr int BK = Shape<kBN>::BK, kABytes = Shape<kBN>::kABytes, kStageBytes = Shape<kBN>::kStageBytes;
    constexpr int kBLayout = kMode & 1;
    constexpr bool kBias = (kMode & 2) != 0;
    constexpr bool kInt8 = (kMode & 4) != 0;
    constexpr bool kBf16In = (kMode & 32) != 0; // bfloat16 operands (bit 5), fp32 accumulate and output
    constexpr int kOut16 = (kMode >> 3) & 3; // 0: fp32 C; 1: C rounded to fp16 on the way out; 2: to bf16 (TSTORE's conversion)
    static_assert(kOut16 == 0 || (!kInt8 && !kBias), "16-bit output: plain fp16 product");
    static_assert(!kInt8 || (kBLayout == 1 && !kBias), "int8: B is n x k, no bias");
    if (threadIdx.x == kThreads - 1) {
        profile_stamp(status, 0);
    }
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *staging = smem + kStages * kStageBytes;
    Control *ctl = reinterpret_cast<Control *>(staging + kStagingBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(); // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    const int tiles_m = (m + 2 * BM - 1) / (2 * BM);
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
            mbar_init(&ctl->acc_empty[a], 8); // four epilogue warps in each of the two blocks
        }
        ctl->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        if (c_by_tma) {
            tma_prefetch_desc(&tmap_c);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync(); // both blocks' barriers exist before anything is signalled across blocks
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int *abort_flag = &ctl->abort_flag;
    const uint32_t peer_abort = map_to_rank(&ctl->abort_flag, rank ^ 1u);

    if (warp == 0) {
        // ------------------------------------------------------------ TLOAD: TMA producer (both blocks)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, tm, tn);
                const int row0 = tm * 2 * BM + static_cast<int>(rank) * BM; // this block's rows of A and C
                const int col0 = tn * BN + static_cast<int>(rank) * BNH;    // this block's half of the B tile
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_pair(&ctl->empty[stage], phase ^ 1u, abort_flag, peer_abort)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + stage * kStageBytes;
                    uint8_t *sb = sa + kABytes;
                    const uint32_t leader_full = map_to_rank(&ctl->full[stage], 0);
                    if (rank == 0) {
                        mbar_arrive_expect_tx(&ctl->full[stage], 2 * kStageBytes); // bytes of both blocks
                    }
#pragma unroll
                    for (int h = 0; h < BK / kBoxK; ++h) {
                        PTO_GEMM2_LOAD(sa + h * (BM * kBoxK * 2), &tmap_a, leader_full, kb * BK + h * kBoxK, row0);
                    }
                    if (kBLayout == 1) {
#pragma unroll
                        for (int h = 0; h < BK / kBoxK; ++h) {
                            PTO_GEMM2_LOAD(sb + h * (BNH * kBoxK * 2), &tmap_b, leader_full, kb * BK + h * kBoxK,
                                             col0);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < BNH / 64; ++j) {
                            PTO_GEMM2_LOAD(sb + j * (64 * BK * 2), &tmap_b, leader_full, col0 + j * 64, kb * BK);
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
        // ------------------------------------------------------------ TEXTRACT + TMATMUL: MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc =
                kInt8 ? make_idesc_i8(2 * BM, BN) : make_idesc_f16(2 * BM, BN, 0, kBLayout == 0 ? 1 : 0, kBf16In ? 1 : 0);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            // descriptors of stage 0; a stage or a k step further on only moves the 16-byte-unit address field
            const uint64_t a_desc0 = make_sw128_desc(smem_u32(smem), 16, 1024);
            const uint64_t b_desc0 = (kBLayout == 1) ? make_sw128_desc(smem_u32(smem) + kABytes, 16, 1024)
                                                     : make_sw128_desc(smem_u32(smem) + kABytes, 64 * BK * 2, 1024);
            constexpr uint32_t kBStep = (kBLayout == 1) ? (32 >> 4) : ((16 * 128) >> 4);
            const uint32_t empty_mine = map_to_rank(&ctl->empty[0], 0);
            const uint32_t empty_peer = map_to_rank(&ctl->empty[0], 1);
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                if (!mbar_wait_pair(&ctl->acc_empty[acc], acc_phase ^ 1u, abort_flag, peer_abort)) {
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_pair(&ctl->full[stage], phase, abort_flag, peer_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kStageBytes >> 4));
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage * (kStageBytes >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // K-major operands: 64-element boxes side by side, 32 bytes per k step inside a box
                        const uint32_t a_off = ((kk >> 2) * (BM * kBoxK * 2) + (kk & 3) * 32) >> 4;
                        const uint32_t b_off =
                            (kBLayout == 1) ? (((kk >> 2) * (BNH * kBoxK * 2) + (kk & 3) * 32) >> 4) : kk * kBStep;
                        if (kInt8) {
                            tc_mma_i8_ss_pair(d_tmem, a_desc + static_cast<uint64_t>(a_off),
                                              b_desc + static_cast<uint64_t>(b_off), idesc, (kb | kk) != 0 ? 1u : 0u);
                        } else {
                            tc_mma_f16_ss_pair(d_tmem, a_desc + static_cast<uint64_t>(a_off),
                                               b_desc + static_cast<uint64_t>(b_off), idesc, (kb | kk) != 0 ? 1u : 0u);
                        }
                    }
                    // the stage is reusable in both blocks once these MMAs have read it
                    tc_commit_pair(empty_mine + stage * 8);
                    tc_commit_pair(empty_peer + stage * 8);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                tc_commit_pair(map_to_rank(&ctl->acc_full[acc], 0));
                tc_commit_pair(map_to_rank(&ctl->acc_full[acc], 1));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ TSTORE: epilogue warps (both blocks)
        const int quarter = warp & 3;
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = ((n & 3) == 0) && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0);
        uint8_t *slabs = staging + (warp - 2) * 2 * kSlabBytes;
        uint32_t slab = 0;
        for (int t = pair; t < num_tiles; t += pairs) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait_pair(&ctl->acc_full[acc], acc_phase, abort_flag, peer_abort)) {
                break;
            }
            tc_fence_after();
            const int row = tm * 2 * BM + static_cast<int>(rank) * BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            float *crow = c + static_cast<int64_t>(row) * n + static_cast<int64_t>(tn) * BN;
            if constexpr (kOut16 != 0) {
                uint16_t *crow16 = reinterpret_cast<uint16_t *>(c) + static_cast<int64_t>(row) * n + static_cast<int64_t>(tn) * BN;
#pragma unroll 1
                for (int cb = 0; cb < BN / 64; ++cb) {
                    uint32_t r0[32], r1[32], w[32]; // 64 columns -> 128 bytes of this row
                    tmem_ld_32x32(taddr + cb * 64, r0);
                    tmem_ld_32x32(taddr + cb * 64 + 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (kOut16 == 1) {
                            const __half2 p0 = __floats2half2_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                            const __half2 p1 = __floats2half2_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                            w[j] = *reinterpret_cast<const uint32_t *>(&p0);
                            w[16 + j] = *reinterpret_cast<const uint32_t *>(&p1);
                        } else {
                            const __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                            const __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                            w[j] = *reinterpret_cast<const uint32_t *>(&p0);
                            w[16 + j] = *reinterpret_cast<const uint32_t *>(&p1);
                        }
                    }
                    const int col0 = tn * BN + cb * 64;
                    if (c_by_tma) {
                        if (lane == 0) {
                            tma_store_wait_read<1>();
                        }
                        __syncwarp();
                        uint8_t *dst = slabs + slab * kSlabBytes + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            *reinterpret_cast<uint4 *>(dst + ((j ^ (lane & 7)) << 4)) =
                                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int slab_row0 = row - lane;
                            if (slab_row0 < m && col0 < n) {
                                PTO_GEMM2_STORE(&tmap_c, slabs + slab * kSlabBytes, col0, slab_row0);
                            }
                            tma_store_commit();
                        }
                        slab ^= 1u;
                    } else if (row < m) {
#pragma unroll
                        for (int j = 0; j < 64; ++j) {
                            if (col0 + j < n) {
                                crow16[cb * 64 + j] = static_cast<uint16_t>((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu));
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + cb * 32, r);
                tmem_ld_wait();
                const int col0 = tn * BN + cb * 32;
                if (kBias) {
                    // TMATMUL_BIAS: one bias value per column, the same for every row (uniform loads)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float bv = (col0 + j < n) ? __ldg(bias + col0 + j) : 0.0f;
                        r[j] = __float_as_uint(__uint_as_float(r[j]) + bv);
                    }
                }
                if (c_by_tma) {
                    // the store that last read this slab (two chunks ago) has finished reading it
                    if (lane == 0) {
                        tma_store_wait_read<1>();
                    }
                    __syncwarp();
                    uint8_t *dst = slabs + slab * kSlabBytes + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        *reinterpret_cast<uint4 *>(dst + ((j ^ (lane & 7)) << 4)) =
                            make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int slab_row0 = row - lane;
                        if (slab_row0 < m && col0 < n) {
                            PTO_GEMM2_STORE(&tmap_c, slabs + slab * kSlabBytes, col0, slab_row0);
                        }
                        tma_store_commit();
                    }
                    slab ^= 1u;
                } else if (row < m) {
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
            } // fp32 / int32 output
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                remote_arrive(map_to_rank(&ctl->acc_empty[acc], 0)); // the leader's MMA warp owns the accumulators
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (c_by_tma && lane == 0) {
            tma_store_wait_all<0>(); // the slabs are read, and C is written, before the block retires
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == kThreads - 1) {
        profile_stamp(status, 1);
    }
    if (ctl->abort_flag) {
        for (int i = 0; i < 1024; ++i) {
            __nanosleep(1000);
        }
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, kErrDeviceWaitTimeout) == 0) {
            status->block = blockIdx.x;
            status->where = 3;
        }
        __syncthreads();
    }
    cluster_sync(); // neither block leaves while the other may still signal it or read its shared memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

} // namespace

namespace {

// One launcher for every instance of the kernel.  kMode: bit 0 B stored n x k, bit 1 bias, bit 2 int8 operands (k
// counts 16-bit pairs), bits 3-4 output type (0 fp32 / int32, 1 fp16, 2 bf16), bit 5 bfloat16 operands.
template <int kMode, int kBN>
int launch_pair_bn(const void *a, const void *b, void *c, const float *bias, int m, int n, int k, cudaStream_t stream)
{
    constexpr int BN = Shape<kBN>::BN, BNH = Shape<kBN>::BNH, BK = Shape<kBN>::BK, kSmemBytes = Shape<kBN>::kSmemBytes;
    constexpr bool kBnk = (kMode & 1) != 0;
    constexpr int kOutBytes = ((kMode >> 3) & 3) == 0 ? 4 : 2;
    CUtensorMap tmap_a, tmap_b, tmap_c;
    int rc = make_tmap_2d(&tmap_a, a, 2, m, k, k, BM, kBoxK, true);
    if (rc != kOk) {
        return rc;
    }
    // C leaves through TMA stores when its rows are 16-byte aligned; otherwise the epilogue stores directly
    const int c_by_tma = ((n & (16 / kOutBytes - 1)) == 0 && (reinterpret_cast<uintptr_t>(c) & 15u) == 0) ? 1 : 0;
    if (c_by_tma) {
        if ((rc = make_tmap_2d(&tmap_c, c, kOutBytes, m, n, n, 32, kOutBytes == 4 ? 32 : 64, true)) != kOk) {
            return rc;
        }
    } else {
        tmap_c = tmap_a; // never dereferenced
    }
    rc = kBnk ? make_tmap_2d(&tmap_b, b, 2, n, k, k, BNH, kBoxK, true) : make_tmap_2d(&tmap_b, b, 2, k, n, n, BK, 64, true);
    if (rc != kOk) {
        return rc;
    }
    const int tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    int pairs = sm_count() / 2;
    if (tiles < pairs) {
        pairs = tiles;
    }
    DeviceStatus *status = device_status_ptr();
    if (status == nullptr) {
        return kErrCuda;
    }
    if ((rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&gemm2_f16f32_kernel<kMode, kBN>), kSmemBytes)) != kOk) {
        return rc;
    }
    gemm2_f16f32_kernel<kMode, kBN><<<2 * pairs, kThreads, kSmemBytes, stream>>>(tmap_a, tmap_b, tmap_c, c_by_tma,
                                                                                  static_cast<float *>(c), bias, m, n, k, status);
    return check_launch();
}

// The tile width follows the problem: 256 columns per block pair unless 128 finish sooner.  A pass over the tile list
// costs (tiles / pairs, rounded up) tile times, and a 128-wide tile takes half as long as a 256-wide one but pulls half
// as much again from L2 per FLOP, so the narrow tile is chosen only where it saves at least a tenth (in practice:
// problems with fewer 256-wide tiles than block pairs, such as 1536^3 with 36 tiles on 74 pairs).
// PTO_B200_GEMM2_BN=128 / 256 forces a width.
template <int kMode>
int launch_pair(const void *a, const void *b, void *c, const float *bias, int m, int n, int k, cudaStream_t stream)
{
    static const int forced = [] {
        const char *e = getenv("PTO_B200_GEMM2_BN");
        return e != nullptr ? atoi(e) : 0;
    }();
    const long long pairs = sm_count() / 2 > 0 ? sm_count() / 2 : 1;
    const long long rows = (m + 2 * BM - 1) / (2 * BM);
    const long long waves_wide = (rows * ((n + 255) / 256) + pairs - 1) / pairs;
    const long long waves_narrow = (rows * ((n + 127) / 128) + pairs - 1) / pairs;
    const bool narrow = forced == 128 || (forced != 256 && waves_narrow * 11 < waves_wide * 20);
    return narrow ? launch_pair_bn<kMode, 128>(a, b, c, bias, m, n, k, stream)
                  : launch_pair_bn<kMode, 256>(a, b, c, bias, m, n, k, stream);
}

} // namespace

int launch_gemm2_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                        cudaStream_t stream, const float *bias)
{
    if (bias == nullptr) {
        return b_layout == 1 ? launch_pair<1>(a, b, c, nullptr, m, n, k, stream)
                             : launch_pair<0>(a, b, c, nullptr, m, n, k, stream);
    }
    return b_layout == 1 ? launch_pair<3>(a, b, c, bias, m, n, k, stream) : launch_pair<2>(a, b, c, bias, m, n, k, stream);
}

// bfloat16 operands, fp32 accumulate and output: the other operand format in the instruction descriptor (kMode bit 5);
// arguments validated by the caller
int launch_gemm2_bf16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                         cudaStream_t stream)
{
    return b_layout == 1 ? launch_pair<33>(a, b, c, nullptr, m, n, k, stream)
                         : launch_pair<32>(a, b, c, nullptr, m, n, k, stream);
}

// C rounded to fp16 (out16 == 1) or bf16 (2): the converting epilogue (kMode bits 3-4)
int launch_gemm2_f16_out16(const uint16_t *a, const uint16_t *b, uint16_t *c, int m, int n, int k, int b_layout, int out16,
                           cudaStream_t stream)
{
    if (out16 == 1) {
        return b_layout == 1 ? launch_pair<9>(a, b, c, nullptr, m, n, k, stream)
                             : launch_pair<8>(a, b, c, nullptr, m, n, k, stream);
    }
    return b_layout == 1 ? launch_pair<17>(a, b, c, nullptr, m, n, k, stream)
                         : launch_pair<16>(a, b, c, nullptr, m, n, k, stream);
}

// C[m x n] int32 = A[m x k] int8 * B[n x k]^T int8 (kMode bit 2): rows are handed to TMA as 16-bit pairs
int launch_gemm2_i8i32(const int8_t *a, const int8_t *b, int32_t *c, int m, int n, int k, cudaStream_t stream)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0) {
        set_error_text("gemm_i8: bad argument");
        return kErrBadArgument;
    }
    if ((k % 16) != 0 || (reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u)) {
        set_error_text("gemm_i8: k must be a multiple of 16 and the operands 16-byte aligned");
        return kErrUnsupportedShape;
    }
    return launch_pair<5>(a, b, c, nullptr, m, n, k / 2, stream);
}

} // namespace pto_b200
