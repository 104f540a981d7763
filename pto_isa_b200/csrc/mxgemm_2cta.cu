// MX block-scaled GEMM for sm_100a on CTA pairs: C[m x n] (bf16 or fp32) = (scaleA (x) A) * (scaleB (x) B)^T with
// A [m x k] and B [n x k] in fp8 (e4m3 or e5m2) or packed fp4 (e2m1, two per byte), one e8m0 scale per 32 consecutive k
// of a row.  It stands for the reference's MxMatmul tile programs (kernels/manual/a5/matmul_mxfp8_performance and
// matmul_mxfp4_performance, mxmatmul_performance_kernel.cpp: TLOAD of data and scale tiles, TEXTRACT, TMATMUL_MX,
// TSTORE) and maps them to tcgen05.mma kind::mxf8f6f4 / kind::mxf4 with block scaling: the data tiles arrive by TMA
// in the 128-byte swizzle, the scale tiles arrive by TMA in the 32-row x 16-byte atoms the tensor core reads, are
// copied into tensor memory (tcgen05.cp) by the MMA thread and are consumed from there by the four MMAs of a
// 128-byte span of k.
//
// The block pair works on a 256 x 256 C tile as in gemm_2cta.cu (each block stages its own 128 rows of A and half of
// the B tile; full[] lives in the leader, empty[] in both blocks; one multicast commit per stage).  A stage is two
// spans.  Tensor memory holds two accumulators that share 64 columns, and the scale slots behind them: the epilogue
// drains the shared columns of a tile first and releases the accumulator then, so that the next tile's MMAs run under
// the rest of the epilogue.
#include "ptx.cuh"
#include "internal.h"

#include <cuda_bf16.h>

namespace pto_b200 {

namespace {

constexpr int BM = 128;  // rows of A / C per block (256 per pair)
constexpr int BN = 256;  // columns of C per pair
constexpr int BNH = 128; // rows of B staged per block
constexpr int kSpan = 128; // k extent of one 128-byte swizzle span of fp8: four MMAs, four scales per row
#ifndef PTO_B200_MX_SPANS
#define PTO_B200_MX_SPANS 2
#endif
constexpr int kSpans = PTO_B200_MX_SPANS; // spans per stage
constexpr int BK = kSpan * kSpans;        // k extent of a stage
constexpr int kStages = kSpans == 2 ? 3 : 6;
constexpr int kABytes = BM * BK;          // 16 KiB per span
constexpr int kBBytes = BNH * BK;         // 16 KiB per span
constexpr int kSfOff = kABytes + kBBytes; // per span: the A atoms, then the B atoms
// A scale atom holds the scales of 128 rows x 128 k (4 per row).  A 128-byte span is 128 k of fp8 = one atom per 128 rows,
// or 256 k of packed fp4 = two atoms: kAtoms below.
__host__ __device__ constexpr int sfa_bytes(int atoms) { return 512 * atoms; }        // this block's 128 rows of A
__host__ __device__ constexpr int sf_span_bytes(int atoms) { return 1536 * atoms; }
__host__ __device__ constexpr int stage_bytes(int atoms) { return ((kSfOff + kSpans * sf_span_bytes(atoms) + 1023) / 1024) * 1024; }
__host__ __device__ constexpr int tx_bytes(int atoms) { return kABytes + kBBytes + kSpans * sf_span_bytes(atoms); }
constexpr int kThreads = 192;             // warp 0 TMA, warp 1 MMA (leader only), warps 2..5 epilogue
constexpr int kTmemCols = 512;
// Tensor memory: two accumulators that share 64 columns, [0, 256) and [192, 448), then four scale slots of 16 columns
// (4 for A, 8 for B).  The epilogue drains the shared columns of a tile first and releases the accumulator to the MMA
// warp at that point, so the next tile's MMAs run under the rest of the epilogue.  The scale slots are reused every
// four spans: the copy into a slot is issued after the MMAs that read it, by the same thread, which the tensor pipe
// executes in issue order.
constexpr int kAccStride = 192;
constexpr int kAccShared = BN - kAccStride; // 64 columns belong to both accumulators
constexpr int kSfTmemBase = kAccStride + BN;
constexpr int kSfTmemCols = kTmemCols - kSfTmemBase; // 64: four 16-column slots (fp8) or two 32-column slots (fp4)

struct Control {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kSlabBytes = 32 * 128; // 32 rows x 128 bytes (64 bf16 or 32 fp32), 128-byte swizzle
constexpr int kSlabsPerWarp = 1;
constexpr int kStagingBytes = 4 * kSlabsPerWarp * kSlabBytes;
__host__ __device__ constexpr int smem_bytes(int atoms)
{
    // the fp4 layout (3 x 70 KiB of stages + 16 KiB of store staging + the barriers) ends 944 bytes under the 227 KiB
    // a block may have, so there is no room for the 1 KiB of slack that aligning by hand inside a larger allocation
    // takes: its buffer is declared 1024-byte aligned, and the kernel checks the address and reports instead of running
    // if the declaration was not honoured
    return kStages * stage_bytes(atoms) + kStagingBytes + static_cast<int>(sizeof(Control)) + (atoms == 1 ? 1024 : 0);
}

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

// one commit of the pair's MMAs and copies, delivered to the barrier at the same shared-memory offset in both blocks
__device__ __forceinline__ void tc_commit_both(uint32_t local_addr)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            local_addr),
        "h"(static_cast<uint16_t>(3))
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, uint32_t leader_bar, int c0,
                                                 int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory descriptor of a scale atom: 32 rows of 16 bytes, no swizzle; 8-row groups are 128 bytes apart
__device__ __forceinline__ uint64_t make_scale_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(128 >> 4) << 32; // stride between 8-row groups
    d |= 1ull << 46;                            // descriptor version for sm_100
    return d;
}

// 32 rows x 16 bytes of shared memory (in both blocks of the pair: each from its own) -> tensor memory columns
// [taddr, taddr + 4), the same 32 rows repeated in the four 32-lane quarters
__device__ __forceinline__ void tc_copy_scales_pair(uint32_t taddr, uint64_t desc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Instruction descriptor of kind::mxf8f6f4 with block scaling: fp32 accumulation, K-major operands, e8m0 scales.
// Formats: 0 = e4m3, 1 = e5m2.  The scale ids (which byte of the 4-byte scale column an MMA uses) are added per MMA.
__device__ __forceinline__ uint32_t make_idesc_mx(int m, int n, int a_fmt, int b_fmt)
{
    return (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
           (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <int kAtoms>
__device__ __forceinline__ void tc_mma_mx_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
    if (kAtoms == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
            "}\n"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
    }
}

// ---------------------------------------------------------------- scale packing
// scale[rows x kscales] (row-major e8m0 bytes) -> [row tile][k block][rows_per_tile / 128][32][4][4]: for every
// (tile of rows_per_tile rows, block of 128 k) the 512-byte atoms the tensor core reads, byte
// (r % 32) * 16 + ((r % 128) / 32) * 4 + j for row r and the j-th scale of the k block.  Rows and scales outside the
// matrix are written as 127 (2^0): the matching data are zero-filled by TMA, but an arbitrary byte could be the NaN
// code.  One thread per (row, k block).
__device__ __forceinline__ uint8_t *mx_atom_word(uint8_t *packed, int rows_per_tile, int kblocks, int r, int kb)
{
    const int tile = r / rows_per_tile, in_tile = r % rows_per_tile;
    const int64_t atom = (static_cast<int64_t>(tile) * kblocks + kb) * (rows_per_tile / 128) + in_tile / 128;
    return packed + atom * 512 + (in_tile % 32) * 16 + ((in_tile % 128) / 32) * 4;
}

// kQuad: one thread per (row, four k blocks) with one 16-byte load (kscales a multiple of 16, aligned sources, kblocks a
// multiple of 4); otherwise one thread per (row, k block) with byte loads.
template <bool kQuad>
__global__ void __launch_bounds__(256) mx_pack_scales_kernel(const uint8_t *__restrict__ sfa, const uint8_t *__restrict__ sfb,
                                                             uint8_t *__restrict__ packed_a, uint8_t *__restrict__ packed_b,
                                                             int m, int n, int kscales, int kblocks, int rows_a_padded,
                                                             int rows_b_padded)
{
    const int per_row = kQuad ? kblocks / 4 : kblocks;
    const int64_t total_a = static_cast<int64_t>(rows_a_padded) * per_row;
    const int64_t total = total_a + static_cast<int64_t>(rows_b_padded) * per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const bool is_a = i < total_a;
        const int64_t j = is_a ? i : i - total_a;
        const int r = static_cast<int>(j / per_row), q = static_cast<int>(j % per_row);
        const uint8_t *src = is_a ? sfa : sfb;
        uint8_t *packed = is_a ? packed_a : packed_b;
        const int rows = is_a ? m : n;
        const int rows_per_tile = is_a ? 128 : 256;
        if (kQuad) {
            uint4 v = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
            if (r < rows && q * 16 < kscales) {
                v = *reinterpret_cast<const uint4 *>(src + static_cast<int64_t>(r) * kscales + q * 16);
            }
            *reinterpret_cast<uint32_t *>(mx_atom_word(packed, rows_per_tile, kblocks, r, 4 * q + 0)) = v.x;
            *reinterpret_cast<uint32_t *>(mx_atom_word(packed, rows_per_tile, kblocks, r, 4 * q + 1)) = v.y;
            *reinterpret_cast<uint32_t *>(mx_atom_word(packed, rows_per_tile, kblocks, r, 4 * q + 2)) = v.z;
            *reinterpret_cast<uint32_t *>(mx_atom_word(packed, rows_per_tile, kblocks, r, 4 * q + 3)) = v.w;
        } else {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int ks = q * 4 + b;
                const uint32_t v = (r < rows && ks < kscales) ? src[static_cast<int64_t>(r) * kscales + ks] : 127u;
                word |= v << (8 * b);
            }
            *reinterpret_cast<uint32_t *>(mx_atom_word(packed, rows_per_tile, kblocks, r, q)) = word;
        }
    }
}

// kAtoms 1: fp8 operands (kind::mxf8f6f4, k = 32 per MMA, one scale per row and MMA); 2: packed fp4 e2m1 operands
// (kind::mxf4, k = 64 per MMA, two scales per row and MMA).  `k` is the row length of A and B in bytes.
template <bool kOutF32, int kAtoms>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
mxgemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                   const __grid_constant__ CUtensorMap tmap_c, int c_by_tma, void *__restrict__ c, int m, int n, int k,
                   int a_fmt, int b_fmt, DeviceStatus *status)
{
    constexpr int kStageBytes = stage_bytes(kAtoms);
    constexpr int kSfaBytes = sfa_bytes(kAtoms);
    constexpr int kSfSpanBytes = sf_span_bytes(kAtoms);
    constexpr int kSlotCols = 16 * kAtoms; // 4 columns per atom of A, 8 per atom of B
    constexpr int kSfSlots = kSfTmemCols / kSlotCols;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    if (kAtoms == 2 && smem != smem_raw) {
        // no room to realign: report instead of running over the end of the allocation
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, kErrCuda) == 0) {
            status->block = blockIdx.x;
            status->where = 6;
        }
        return;
    }
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
    const int katoms = kblocks * kSpans * kAtoms; // scale atoms along k (padded to whole stages by the packing kernel)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        mbar_init(&ctl->acc_full, 1);
        mbar_init(&ctl->acc_empty, 8); // four epilogue warps in each of the two blocks
        ctl->abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
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
                const int sfa_row0 = (tm * 2 + static_cast<int>(rank)) * katoms;
                const int sfb_row0 = tn * katoms;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_pair(&ctl->empty[stage], phase ^ 1u, abort_flag, peer_abort)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + stage * kStageBytes;
                    const uint32_t leader_full = map_to_rank(&ctl->full[stage], 0);
                    if (rank == 0) {
                        mbar_arrive_expect_tx(&ctl->full[stage], 2 * tx_bytes(kAtoms)); // bytes of both blocks
                    }
#pragma unroll
                    for (int sp = 0; sp < kSpans; ++sp) {
                        tma_load_2d_pair(sa + sp * (BM * kSpan), &tmap_a, leader_full, kb * BK + sp * kSpan, row0);
                        tma_load_2d_pair(sa + kABytes + sp * (BNH * kSpan), &tmap_b, leader_full, kb * BK + sp * kSpan,
                                         col0);
                        uint8_t *sf = sa + kSfOff + sp * kSfSpanBytes;
                        tma_load_2d_pair(sf, &tmap_sfa, leader_full, 0, sfa_row0 + (kb * kSpans + sp) * kAtoms);
                        tma_load_2d_pair(sf + kSfaBytes, &tmap_sfb, leader_full, 0, sfb_row0 + (kb * kSpans + sp) * kAtoms);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ TEXTRACT + TMATMUL_MX: MMA issuer (leader only)
        // The whole warp walks the loops (lane 0 waits and issues, the result of every wait is broadcast), so that the
        // control flow stays warp-uniform and the descriptors of the tcgen05 instructions can be kept in uniform
        // registers instead of being moved there one by one in front of every instruction.
        if (rank == 0) {
            const uint32_t idesc = kAtoms == 1 ? make_idesc_mx(2 * BM, BN, a_fmt, b_fmt) : make_idesc_mx(2 * BM, BN, 1, 1);
            uint32_t stage = 0, phase = 0, acc_phase = 0;
            const uint64_t a_desc0 = make_sw128_desc(smem_u32(smem), 16, 1024);
            const uint64_t b_desc0 = make_sw128_desc(smem_u32(smem) + kABytes, 16, 1024);
            const uint64_t sfa_desc0 = make_scale_desc(smem_u32(smem) + kSfOff);
            const uint64_t sfb_desc0 = make_scale_desc(smem_u32(smem) + kSfOff + kSfaBytes);
            const uint32_t empty_addr = smem_u32(&ctl->empty[0]);
            const uint32_t acc_full_addr = smem_u32(&ctl->acc_full);
            uint32_t local_tile = 0, span_ctr = 0;
            for (int t = pair; t < num_tiles; t += pairs) {
                // the epilogue warps of both blocks have drained the columns the previous tile shares with this one
                // (and all of the tile before that, which used this accumulator)
                int ok = 1;
                if (lane == 0) {
                    ok = mbar_wait_pair(&ctl->acc_empty, acc_phase ^ 1u, abort_flag, peer_abort) ? 1 : 0;
                }
                if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (local_tile & 1u) * kAccStride;
                ++local_tile;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (lane == 0) {
                        ok = mbar_wait_pair(&ctl->full[stage], phase, abort_flag, peer_abort) ? 1 : 0;
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok == 0) {
                        break;
                    }
                    tc_fence_after();
                    const uint64_t stage_off = static_cast<uint64_t>(stage * (kStageBytes >> 4));
                    if (lane == 0) {
#pragma unroll
                        for (int sp = 0; sp < kSpans; ++sp) {
                            const uint32_t sfa_tmem = tmem_base + kSfTmemBase + ((span_ctr + sp) % kSfSlots) * kSlotCols;
                            const uint32_t sfb_tmem = sfa_tmem + 4 * kAtoms;
                            const uint64_t sf_off = stage_off + static_cast<uint64_t>((sp * kSfSpanBytes) >> 4);
                            // the span's scales: per atom one copy for this block's 128 rows of A, two for the 256 rows
                            // of B
#pragma unroll
                            for (int at = 0; at < kAtoms; ++at) {
                                tc_copy_scales_pair(sfa_tmem + at * 4, sfa_desc0 + sf_off + static_cast<uint64_t>((at * 512) >> 4));
                                tc_copy_scales_pair(sfb_tmem + at * 8, sfb_desc0 + sf_off + static_cast<uint64_t>((at * 1024) >> 4));
                                tc_copy_scales_pair(sfb_tmem + at * 8 + 4,
                                                    sfb_desc0 + sf_off + static_cast<uint64_t>((at * 1024 + 512) >> 4));
                            }
#pragma unroll
                            for (int kk = 0; kk < kSpan / 32; ++kk) {
                                // 32 bytes of k per MMA inside the 128-byte span.  fp8: scale byte kk of the atom's
                                // columns; fp4: atom kk / 2, scale bytes {0, 1} or {2, 3}
                                const uint32_t sf_id = kAtoms == 1 ? static_cast<uint32_t>(kk) : static_cast<uint32_t>((kk & 1) * 2);
                                const uint32_t atom = kAtoms == 1 ? 0u : static_cast<uint32_t>(kk >> 1);
                                const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                                const uint64_t a_off = stage_off + static_cast<uint64_t>((sp * (BM * kSpan) + kk * 32) >> 4);
                                const uint64_t b_off = stage_off + static_cast<uint64_t>((sp * (BNH * kSpan) + kk * 32) >> 4);
                                tc_mma_mx_pair<kAtoms>(d_tmem, a_desc0 + a_off, b_desc0 + b_off, id, sfa_tmem + atom * 4,
                                                       sfb_tmem + atom * 8, (kb | sp | kk) != 0 ? 1u : 0u);
                            }
                        }
                        // the stage is reusable in both blocks once these MMAs have read it: one commit, delivered to
                        // the barrier at this offset in both blocks
                        tc_commit_both(empty_addr + stage * 8);
                    }
                    span_ctr += kSpans;
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok == 0) {
                    break;
                }
                if (lane == 0) {
                    tc_commit_both(acc_full_addr);
                }
                acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------------ TSTORE: epilogue warps (both blocks)
        const int quarter = warp & 3;
        uint32_t acc_phase = 0, local_tile = 0;
        constexpr int kSlabCols = kOutF32 ? 32 : 64; // 128 bytes of output per row and slab
        constexpr int kElem = kOutF32 ? 4 : 2;
        uint8_t *slabs = staging + (warp - 2) * kSlabsPerWarp * kSlabBytes;
        uint32_t slab = 0;
        const uint32_t acc_empty_leader = map_to_rank(&ctl->acc_empty, 0);
        for (int t = pair; t < num_tiles; t += pairs) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait_pair(&ctl->acc_full, acc_phase, abort_flag, peer_abort)) {
                break;
            }
            tc_fence_after();
            const int row = tm * 2 * BM + static_cast<int>(rank) * BM + quarter * 32 + lane;
            const uint32_t buf = local_tile & 1u;
            ++local_tile;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kAccStride;
            constexpr int kSlabs = BN / kSlabCols;
            constexpr int kEarly = kAccShared / kSlabCols; // slabs in the columns shared with the other accumulator
            uint8_t *crow = static_cast<uint8_t *>(c) + (static_cast<int64_t>(row) * n + static_cast<int64_t>(tn) * BN) * kElem;
#pragma unroll 1
            for (int i = 0; i < kSlabs; ++i) {
                // the shared columns first: the last ones of accumulator 0, the first ones of accumulator 1
                const int cb = (buf == 0) ? (i + kSlabs - kEarly) % kSlabs : i;
                uint32_t w[32]; // 128 bytes of this row's output
                if (kOutF32) {
                    tmem_ld_32x32(taddr + cb * 32, w);
                    tmem_ld_wait();
                } else {
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(taddr + cb * 64, r0);
                    tmem_ld_32x32(taddr + cb * 64 + 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
                        const __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
                        w[j] = *reinterpret_cast<const uint32_t *>(&p0);
                        w[16 + j] = *reinterpret_cast<const uint32_t *>(&p1);
                    }
                }
                if (i == kEarly - 1) {
                    // the shared columns are in registers: the next tile's MMAs may overwrite them
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        remote_arrive(acc_empty_leader); // the leader's MMA warp owns the accumulators
                    }
                }
                const int col0 = tn * BN + cb * kSlabCols;
                if (c_by_tma) {
                    if (lane == 0) {
                        tma_store_wait_read<kSlabsPerWarp - 1>(); // the store that last read this slab has finished reading it
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
                            tma_store_2d(&tmap_c, slabs + slab * kSlabBytes, col0, slab_row0);
                        }
                        tma_store_commit();
                    }
                    slab = (slab + 1) % kSlabsPerWarp;
                } else if (row < m) {
                    // unaligned C: element stores
#pragma unroll
                    for (int j = 0; j < kSlabCols; ++j) {
                        if (col0 + j < n) {
                            if (kOutF32) {
                                reinterpret_cast<uint32_t *>(crow)[cb * kSlabCols + j] = w[j];
                            } else {
                                reinterpret_cast<uint16_t *>(crow)[cb * kSlabCols + j] =
                                    static_cast<uint16_t>((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu));
                            }
                        }
                    }
                }
            }
            acc_phase ^= 1u;
        }
        if (c_by_tma && lane == 0) {
            tma_store_wait_all<0>(); // the slabs are read, and C is written, before the block retires
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ctl->abort_flag) {
        for (int i = 0; i < 1024; ++i) {
            __nanosleep(1000);
        }
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, kErrDeviceWaitTimeout) == 0) {
            status->block = blockIdx.x;
            status->where = 5;
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

// scale atoms (128 k each) along k, padded to whole stages; `fp4`: a stage is 512 k (two spans of 256), else 256 k
static int mx_atoms_along_k(int k, bool fp4)
{
    const int stage_k = fp4 ? 2 * BK : BK;
    return ((k + stage_k - 1) / stage_k) * (stage_k / 128);
}

size_t mxgemm_workspace_bytes(int m, int n, int k)
{
    // sized for the fp4 form, whose stages are longer (its padding along k is the larger one)
    const size_t atoms_k = static_cast<size_t>(mx_atoms_along_k(k, true));
    const size_t atoms_a = static_cast<size_t>((m + 127) / 128) * atoms_k;
    const size_t atoms_b = static_cast<size_t>((n + 255) / 256) * 2 * atoms_k;
    return (atoms_a + atoms_b) * 512;
}

template <bool kOutF32, int kAtoms>
static int launch_mx_kernel(int pairs, cudaStream_t stream, const CUtensorMap &tmap_a, const CUtensorMap &tmap_b,
                            const CUtensorMap &tmap_sfa, const CUtensorMap &tmap_sfb, const CUtensorMap &tmap_c,
                            int c_by_tma, void *c, int m, int n, int k_bytes, int a_fmt, int b_fmt, DeviceStatus *status)
{
    const int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&mxgemm2_kernel<kOutF32, kAtoms>), smem_bytes(kAtoms));
    if (rc != kOk) {
        return rc;
    }
    mxgemm2_kernel<kOutF32, kAtoms><<<2 * pairs, kThreads, smem_bytes(kAtoms), stream>>>(
        tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c, c_by_tma, c, m, n, k_bytes, a_fmt, b_fmt, status);
    return check_launch();
}

// `fp4`: A and B hold two e2m1 values per byte (the lower k index in the low nibble), k / 2 bytes per row
int launch_mxgemm(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, void *c, int m, int n, int k,
                  bool fp4, int a_fmt, int b_fmt, int out_f32, void *workspace, size_t workspace_bytes,
                  cudaStream_t stream)
{
    if (workspace == nullptr || workspace_bytes < mxgemm_workspace_bytes(m, n, k) ||
        (reinterpret_cast<uintptr_t>(workspace) & 127u) != 0) {
        set_error_text("mxgemm: the workspace must be 128-byte aligned and hold mxgemm_workspace_bytes(m, n, k) bytes");
        return kErrBadArgument;
    }
    const int kblocks = mx_atoms_along_k(k, fp4); // 128-k scale atoms along k, padded to whole stages
    const int k_bytes = fp4 ? k / 2 : k;
    const int atoms = fp4 ? 2 : 1;
    const int rows_a_padded = ((m + 127) / 128) * 128;
    const int rows_b_padded = ((n + 255) / 256) * 256;
    uint8_t *packed_a = static_cast<uint8_t *>(workspace);
    uint8_t *packed_b = packed_a + static_cast<size_t>(rows_a_padded / 128) * kblocks * 512;
    const int kscales = k / 32;
    const bool quad = (kscales % 16 == 0) && (kblocks % 4 == 0) && (reinterpret_cast<uintptr_t>(sfa) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(sfb) & 15u) == 0;
    const int64_t pack_items = static_cast<int64_t>(rows_a_padded + rows_b_padded) * (quad ? kblocks / 4 : kblocks);
    if (quad) {
        mx_pack_scales_kernel<true><<<grid_for(pack_items, 256), 256, 0, stream>>>(sfa, sfb, packed_a, packed_b, m, n, kscales,
                                                                                  kblocks, rows_a_padded, rows_b_padded);
    } else {
        mx_pack_scales_kernel<false><<<grid_for(pack_items, 256), 256, 0, stream>>>(sfa, sfb, packed_a, packed_b, m, n, kscales,
                                                                                   kblocks, rows_a_padded, rows_b_padded);
    }
    int rc = check_launch();
    if (rc != kOk) {
        return rc;
    }
    CUtensorMap tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c;
    // scales: one row of the map per atom (A: 512 bytes) or atom pair (B: 1024 bytes), `atoms` rows per copy
    if ((rc = make_tmap_2d(&tmap_a, a, 1, m, k_bytes, k_bytes, BM, kSpan, true)) != kOk ||
        (rc = make_tmap_2d(&tmap_b, b, 1, n, k_bytes, k_bytes, BNH, kSpan, true)) != kOk ||
        (rc = make_tmap_2d(&tmap_sfa, packed_a, 4, static_cast<uint64_t>(rows_a_padded / 128) * kblocks, 128, 128, atoms,
                           128, false)) != kOk ||
        (rc = make_tmap_2d(&tmap_sfb, packed_b, 4, static_cast<uint64_t>(rows_b_padded / 256) * kblocks, 256, 256, atoms,
                           256, false)) != kOk) {
        return rc;
    }
    const int elem = out_f32 ? 4 : 2;
    const int c_by_tma = ((n * elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(c) & 15u) == 0) ? 1 : 0;
    if (c_by_tma) {
        rc = make_tmap_2d(&tmap_c, c, elem, m, n, n, 32, out_f32 ? 32 : 64, true);
        if (rc != kOk) {
            return rc;
        }
    } else {
        tmap_c = tmap_a; // never dereferenced
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
    if (fp4) {
        return out_f32 ? launch_mx_kernel<true, 2>(pairs, stream, tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c, c_by_tma, c, m, n,
                                                   k_bytes, a_fmt, b_fmt, status)
                       : launch_mx_kernel<false, 2>(pairs, stream, tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c, c_by_tma, c, m,
                                                    n, k_bytes, a_fmt, b_fmt, status);
    }
    return out_f32 ? launch_mx_kernel<true, 1>(pairs, stream, tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c, c_by_tma, c, m, n,
                                               k_bytes, a_fmt, b_fmt, status)
                   : launch_mx_kernel<false, 1>(pairs, stream, tmap_a, tmap_b, tmap_sfa, tmap_sfb, tmap_c, c_by_tma, c, m, n,
                                                k_bytes, a_fmt, b_fmt, status);
}

int launch_mxgemm_fp8(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, void *c, int m, int n,
                      int k, int a_fmt, int b_fmt, int out_f32, void *workspace, size_t workspace_bytes,
                      cudaStream_t stream)
{
    return launch_mxgemm(a, b, sfa, sfb, c, m, n, k, false, a_fmt, b_fmt, out_f32, workspace, workspace_bytes, stream);
}

int launch_mxgemm_fp4(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, void *c, int m, int n,
                      int k, int out_f32, void *workspace, size_t workspace_bytes, cudaStream_t stream)
{
    return launch_mxgemm(a, b, sfa, sfb, c, m, n, k, true, 1, 1, out_f32, workspace, workspace_bytes, stream);
}

} // namespace pto_b200
