// Flash-attention forward for sm_100a (head size 128, fp16 Q/K/V, fp32 softmax, fp32 or fp16 O).
//
// The reference (kernels/manual/common/flash_atten/fa_performance_kernel.cpp:607-963, paths relative to the
// reference root) runs a cube core and two vector cores per 128 query rows and passes every QK tile, P tile
// and PV tile through global-memory FIFOs (TPUSH/TPOP, :782-821).  Here one CTA owns 256 query rows (two
// 128-row tiles) of one head and all of those hand-offs stay on chip:
//   compute_qk  (:280-352, TLOAD K + pto_macro_matmul)  -> TMA loads of K into swizzled shared memory,
//                                                          S = Q K^T by tcgen05.mma into tensor memory
//   compute_p   (:452-552, pto_macro_fa_softmax)        -> one thread per query row reads its S row from
//                                                          tensor memory, updates the running max and sum and
//                                                          writes P = exp(scale*(S - max)) as fp16 into shared
//                                                          memory in the tensor core's operand layout
//   compute_pv  (:357-447)                              -> O += P V by tcgen05.mma, P and V (MN-major) from
//                                                          shared memory
//   compute_gu  (:557-605, pto_macro_fa_gu)             -> O lives in tensor memory; it is rescaled there when
//                                                          a row's max grows, and divided by the row sum on
//                                                          the way out
// Because P does not live where S does, the product S(j+1) = Q K(j+1)^T is issued as soon as the softmax
// warps have *read* S(j), i.e. it runs on the tensor core while the exponentials of step j are computed;
// the reference's QK_PRELOAD look-ahead (fa_performance_kernel.h:18-26) plays the same role.
//
// Softmax conventions are the reference's (pto_macro_fa_softmax.hpp:81-97,141-184): the max is taken on
// the raw logits, p = exp(scale * (x - max)) in fp32, the row sum accumulates the fp32 p, p is rounded to
// fp16 for the second product, the causal mask hides keys beyond the query's own index, fully masked key
// tiles are skipped.  The running max is only moved when it grows by more than 8 in the log2 domain; the
// result O / l does not depend on which reference value is used (both carry the same factor).
//
// Warp roles (384 threads = 3 warpgroups): warps 0-3 softmax of query tile 0, warps 4-7 softmax of query tile 1
// (each thread owns one query row, so row reductions need no shuffles), warp 8 TMA producer, warps 9 and 10
// MMA issuers (one per query tile), warp 11 idle.  The softmax warpgroups raise their register budget with setmaxnreg and the third
// warpgroup lowers its own.
#include "ptx.cuh"
#include "internal.h"

#include <cuda_fp16.h>

#include <cstdlib>

namespace pto_b200 {

namespace {

constexpr int kD = 128;           // head size
constexpr int kTileQ = 128;       // query rows per tile (two tiles per CTA)
constexpr int kTileKV = 128;      // keys per step
constexpr int kRing = 3;          // K / V tiles in flight, in the order the tensor core consumes them
constexpr int kTileBytes = kTileQ * kD * 2; // 32 KiB: a 128 x 128 fp16 tile as two 64-column swizzled halves
constexpr int kHalfBytes = kTileBytes / 2;  // 16 KiB
constexpr int kThreads = 384;
constexpr int kRegsSoftmax = 224; // per-thread register budgets after the warpgroups rebalance (setmaxnreg):
constexpr int kRegsOther = 56;    // 256 * 224 + 128 * 56 = 64512 = 384 * 168, the pool the block was launched with
constexpr int kTmemCols = 512;
constexpr int kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;

struct Control {
    uint64_t q_full;
    uint64_t ring_full[kRing], ring_empty[kRing];
    uint64_t s_full[2];  // S tile complete in tensor memory
    uint64_t s_free[2];  // S tile copied to registers by all four softmax warps: S(j+1) may overwrite it
    uint64_t p_full[2];  // P tile written to shared memory (and O rescaled) by all four softmax warps
    uint64_t pv_done[2]; // PV product of the step complete: P buffer reusable, O consistent
    uint32_t tmem_base;
    int abort_flag;
};

// Q (2 tiles) + K/V ring (3 tiles) + P (2 tiles)
constexpr int kSmemBytes = (2 + kRing + 2) * kTileBytes + sizeof(Control) + 1024;

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// ---- packed fp32 pairs (two lanes per 64-bit register; one issue slot per pair of operations)
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x for a pair of arguments on the FMA pipe instead of the special-function unit (which bounds the
// exponential phase of the softmax): x is clamped to >= -126, split into round(x) + f with f in [-0.5, 0.5]
// by the 1.5 * 2^23 trick, 2^f is a degree-4 minimax polynomial (max relative error 2.7e-6, far below the
// fp16 rounding P undergoes), and round(x) is added to the exponent field.
__device__ __forceinline__ void exp2_poly_pair(float x0, float x1, float &p0, float &p1)
{
    const float kMagic = 12582912.0f; // 1.5 * 2^23
    x0 = fmaxf(x0, -126.0f);
    x1 = fmaxf(x1, -126.0f);
    const uint64_t x = pack2(x0, x1);
    const uint64_t t = add2(x, pack2(kMagic, kMagic));       // integer part lands in the low mantissa bits
    const uint64_t r = add2(t, pack2(-kMagic, -kMagic));     // round(x) as a float
    const uint64_t f = fma2(r, pack2(-1.0f, -1.0f), x);      // x - round(x)
    uint64_t p = pack2(0.009570101276040077f, 0.009570101276040077f);
    p = fma2(p, f, pack2(0.05591785907745361f, 0.05591785907745361f));
    p = fma2(p, f, pack2(0.240247443318367f, 0.240247443318367f));
    p = fma2(p, f, pack2(0.6931217908859253f, 0.6931217908859253f));
    p = fma2(p, f, pack2(0.9999992847442627f, 0.9999992847442627f));
    float t0, t1, q0, q1;
    unpack2(t, t0, t1);
    unpack2(p, q0, q1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// kPolyOf8: of every 8 pairs of probabilities, this many are exponentiated on the FMA pipe
template <bool kCausal, bool kOutF16, int kPolyOf8>
__global__ void __launch_bounds__(kThreads, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o, int sq, int sk,
                      float scale_log2, float defer_log2, DeviceStatus *status)
{
    if (threadIdx.x == 0) { // a softmax thread: it has nothing to do until the first logits arrive
        profile_stamp(status, 0);
    }
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_q = smem;                                // 2 tiles
    uint8_t *smem_ring = smem + 2 * kTileBytes;            // kRing tiles
    uint8_t *smem_p = smem_ring + kRing * kTileBytes;      // 2 tiles
    Control *ctl = reinterpret_cast<Control *>(smem_p + 2 * kTileBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // work assignment: consecutive CTAs share a head (K/V stay in L2); within a head the query blocks
    // with the most key tiles (causal) come first
    const int q_blocks = (sq + 2 * kTileQ - 1) / (2 * kTileQ);
    const int bh = blockIdx.x / q_blocks;
    const int qb = q_blocks - 1 - (blockIdx.x % q_blocks);
    const int kv_tiles = sk / kTileKV;
    int n_kv0, n_kv1;
    {
        int n[2];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int q0 = (2 * qb + t) * kTileQ;
            if (q0 >= sq) {
                n[t] = 0;
            } else if (kCausal) {
                const int lim = q0 / kTileKV + 1; // tiles that hold at least one key <= the tile's last query
                n[t] = lim < kv_tiles ? lim : kv_tiles;
            } else {
                n[t] = kv_tiles;
            }
        }
        n_kv0 = n[0];
        n_kv1 = n[1];
    }
    const int n_max = n_kv0 > n_kv1 ? n_kv0 : n_kv1;

    if (threadIdx.x == 0) {
        mbar_init(&ctl->q_full, 1);
        for (int s = 0; s < kRing; ++s) {
            mbar_init(&ctl->ring_full[s], 1);
            mbar_init(&ctl->ring_empty[s], 2); // both MMA issuers release a slot
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&ctl->s_full[t], 1);
            mbar_init(&ctl->s_free[t], kTileQ / 32); // one arrival per softmax warp
            mbar_init(&ctl->p_full[t], kTileQ / 32);
            mbar_init(&ctl->pv_done[t], 1);
        }
        ctl->abort_flag = 0;
        fence_mbar_init();
        // The first loads (both Q tiles and K(0), ring item 0) leave right here, before the tensor-memory allocation
        // and the block-wide barrier: their latency is the start-up cost of every block.
        {
            int q_bytes = 0;
            q_bytes += (n_kv0 > 0) ? kTileBytes : 0;
            q_bytes += (n_kv1 > 0) ? kTileBytes : 0;
            mbar_arrive_expect_tx(&ctl->q_full, q_bytes);
            for (int t = 0; t < 2; ++t) {
                if ((t == 0 ? n_kv0 : n_kv1) > 0) {
                    const int q0 = (2 * qb + t) * kTileQ;
                    tma_load_3d(smem_q + t * kTileBytes, &tmap_q, &ctl->q_full, 0, q0, bh);
                    tma_load_3d(smem_q + t * kTileBytes + kHalfBytes, &tmap_q, &ctl->q_full, 64, q0, bh);
                }
            }
            if (n_max > 0) {
                mbar_arrive_expect_tx(&ctl->ring_full[0], kTileBytes);
                tma_load_3d(smem_ring, &tmap_k, &ctl->ring_full[0], 0, 0, bh);
                tma_load_3d(smem_ring + kHalfBytes, &tmap_k, &ctl->ring_full[0], 64, 0, bh);
            }
        }
        tma_prefetch_desc(&tmap_v);
        tma_prefetch_desc(&tmap_o);
    }
    if (warp == 9) {
        tmem_alloc(&ctl->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int *abort_flag = &ctl->abort_flag;

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp == 8) {
            // -------------------------------------------------------- TMA producer (TLOAD of Q, K, V)
            // ring items in consumption order: K(0), then for every step j: K(j+1) (if any), V(j)
            if (lane == 0) {
                int item = 1; // item 0, K(0), was issued with the Q tiles before the block-wide barrier
                bool ok = true;
                auto load_item = [&](const CUtensorMap *map, int tile) {
                    const int s = item % kRing;
                    const uint32_t ph = (item / kRing) & 1;
                    if (!mbar_wait(&ctl->ring_empty[s], ph ^ 1u, abort_flag)) {
                        ok = false;
                        return;
                    }
                    uint8_t *dst = smem_ring + s * kTileBytes;
                    mbar_arrive_expect_tx(&ctl->ring_full[s], kTileBytes);
                    tma_load_3d(dst, map, &ctl->ring_full[s], 0, tile * kTileKV, bh);
                    tma_load_3d(dst + kHalfBytes, map, &ctl->ring_full[s], 64, tile * kTileKV, bh);
                    ++item;
                };
                for (int j = 0; j < n_max && ok; ++j) {
                    if (j + 1 < n_max) {
                        load_item(&tmap_k, j + 1);
                    }
                    if (ok) {
                        load_item(&tmap_v, j);
                    }
                }
            }
        } else if (warp == 9 || warp == 10) {
            // -------------------------------------------------------- MMA issuers: warp 9 for query tile 0,
            // warp 10 for query tile 1.  One thread sustains about one tcgen05.mma per 80 cycles, a 128 x 128 x 16
            // MMA takes 64: two issuing threads keep the tensor core fed.  Both walk the K/V ring in the same
            // order and both release every slot (the ring's empty barriers count two arrivals).
            if (lane == 0) {
                const int t = warp - 9;
                const int n_t = (t == 0) ? n_kv0 : n_kv1;
                constexpr uint32_t idesc_s = make_idesc_f16(kTileQ, kTileKV, 0, 0); // Q (K-major) x K (K-major)
                constexpr uint32_t idesc_o = make_idesc_f16(kTileQ, kD, 0, 1);      // P (K-major) x V (MN-major)
                const uint32_t ring_base = smem_u32(smem_ring);
                const uint32_t s_tmem = tmem_base + (t == 0 ? kColS0 : kColS1);
                const uint32_t o_tmem = tmem_base + (t == 0 ? kColO0 : kColO1);
                // descriptors of the operands that never move (Q_t, P_t): built once
                const uint64_t q_desc = make_sw128_desc(smem_u32(smem_q) + t * kTileBytes, 16, 1024);
                const uint64_t p_desc = make_sw128_desc(smem_u32(smem_p) + t * kTileBytes, 16, 1024);
                bool ok = mbar_wait(&ctl->q_full, 0, abort_flag);
                int item = 0;

                // a k step of 16 inside a K-major tile: +32 bytes, and +16 KiB when crossing into the second
                // 64-wide half; in descriptor units (16 bytes) that is +2 and +1024
                auto kmajor_step = [](int kk) -> uint64_t {
                    return static_cast<uint64_t>((kk >> 2) * (kHalfBytes >> 4) + (kk & 3) * 2);
                };
                auto issue_s = [&](uint32_t kb) {
                    const uint64_t k_desc = make_sw128_desc(kb, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < kD / 16; ++kk) {
                        tc_mma_f16_ss(s_tmem, q_desc + kmajor_step(kk), k_desc + kmajor_step(kk), idesc_s,
                                      kk != 0 ? 1u : 0u);
                    }
                    tc_commit(&ctl->s_full[t]);
                };
                auto issue_pv = [&](uint32_t vb, bool accumulate) {
                    const uint64_t v_desc = make_sw128_desc(vb, kHalfBytes, 1024); // MN-major: 16 keys = 2 KiB
#pragma unroll
                    for (int kk = 0; kk < kTileKV / 16; ++kk) {
                        tc_mma_f16_ss(o_tmem, p_desc + kmajor_step(kk), v_desc + static_cast<uint64_t>(kk * 128),
                                      idesc_o, (accumulate || kk != 0) ? 1u : 0u);
                    }
                    tc_commit(&ctl->pv_done[t]);
                };
                auto ring_wait = [&](uint32_t &addr, int &slot) {
                    slot = item % kRing;
                    const uint32_t ph = (item / kRing) & 1;
                    addr = ring_base + slot * kTileBytes;
                    ++item;
                    return mbar_wait(&ctl->ring_full[slot], ph, abort_flag);
                };

                uint32_t addr = 0;
                int slot = 0;
                if (ok && n_max > 0) {
                    ok = ring_wait(addr, slot); // K(0)
                    if (ok) {
                        if (n_t > 0) {
                            issue_s(addr);
                        }
                        tc_commit(&ctl->ring_empty[slot]);
                    }
                }
                for (int j = 0; j < n_max && ok; ++j) {
                    if (j + 1 < n_max) {
                        ok = ring_wait(addr, slot); // K(j+1)
                        if (ok && j + 1 < n_t) {
                            ok = mbar_wait(&ctl->s_free[t], j & 1, abort_flag); // S_t(j) has been read
                            if (ok) {
                                tc_fence_after();
                                issue_s(addr);
                            }
                        }
                        if (!ok) {
                            break;
                        }
                        tc_commit(&ctl->ring_empty[slot]);
                    }
                    ok = ring_wait(addr, slot); // V(j)
                    if (ok && j < n_t) {
                        ok = mbar_wait(&ctl->p_full[t], j & 1, abort_flag);
                        if (ok) {
                            tc_fence_after();
                            issue_pv(addr, j != 0);
                        }
                    }
                    if (!ok) {
                        break;
                    }
                    tc_commit(&ctl->ring_empty[slot]);
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ------------------------------------------------------------ softmax / rescale / output warps
        const int t = warp >> 2;               // query tile of this warpgroup
        const int quarter = warp & 3;          // TMEM lanes [32*quarter, +32)
        const int row_in_tile = quarter * 32 + lane;
        const int q_row = (2 * qb + t) * kTileQ + row_in_tile;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + (t == 0 ? kColS0 : kColS1);
        const uint32_t o_addr = lane_addr + (t == 0 ? kColO0 : kColO1);
        // this row of the P tile: two halves of 64 keys, 128 bytes per row and half, 16-byte chunks swizzled
        const uint32_t p_row = smem_u32(smem_p) + t * kTileBytes + row_in_tile * 128;
        const uint32_t swz = static_cast<uint32_t>(row_in_tile & 7);
        const int n = (t == 0) ? n_kv0 : n_kv1;
        float m_run = -INFINITY; // running reference max (raw logits)
        float l_run = 0.0f;      // running sum of p
        bool ok = true;

        for (int j = 0; j < n; ++j) {
            if (!mbar_wait(&ctl->s_full[t], j & 1, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                tmem_ld_32x32(s_addr + c * 32, sr[c]);
            }
            tmem_ld_wait();
            tc_fence_before();
            if (lane == 0) {
                mbar_arrive(&ctl->s_free[t]); // the tensor core may start S(j+1) into the same columns
            }

            const bool diag = kCausal && (j * kTileKV + kTileKV - 1 > (2 * qb + t) * kTileQ);
            if (diag) {
                const int kv0 = j * kTileKV;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (kv0 + c * 32 + i > q_row) {
                            sr[c][i] = 0xff800000u; // -inf
                        }
                    }
                }
            }
            // row maximum: eight independent chains of three-input maxima
            float mx8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                mx8[u] = fmaxf(__uint_as_float(sr[0][u]), __uint_as_float(sr[0][8 + u]));
            }
#pragma unroll
            for (int i = 16; i < 128; i += 16) {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    mx8[u] = max3(mx8[u], __uint_as_float(sr[i >> 5][(i & 31) + u]),
                                  __uint_as_float(sr[i >> 5][(i & 31) + 8 + u]));
                }
            }
            const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
            // The reference maximum follows the running maximum as soon as it grows by more than 2^defer_log2:
            // 0 = at every key tile where it grows at all, the reference's recurrence (pto_macro_fa_softmax.hpp:
            // 141-165 in the reference); 8 = only after it has grown 256-fold, which saves almost every rescale of O.
            const float m_new = fmaxf(m_run, mx);
            const bool grow = (m_new - m_run) * scale_log2 > defer_log2; // also true on the first tile (m_run = -inf)
            const bool rescale = __any_sync(0xffffffffu, grow);
            // The previous PV product must be complete before O is rescaled or P's buffer is rewritten.  The
            // rescale is rare, so normally this wait sits after the exponentials: they overlap that product.
            bool pv_waited = (j == 0);
            if (rescale) {
                if (j > 0) {
                    if (!mbar_wait(&ctl->pv_done[t], (j - 1) & 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    pv_waited = true;
                    tc_fence_after();
                    const float alpha = ex2_approx((m_run - m_new) * scale_log2);
                    l_run *= alpha;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t orow[32];
                        tmem_ld_32x32(o_addr + c * 32, orow);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                        }
                        tmem_st_32x32(o_addr + c * 32, orow);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                }
                m_run = m_new;
            }
            const float neg_m = -m_run * scale_log2;
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float a0 = fmaf(__uint_as_float(sr[c][i]), scale_log2, neg_m);
                    const float a1 = fmaf(__uint_as_float(sr[c][i + 1]), scale_log2, neg_m);
                    float p0, p1;
                    if (((i >> 1) & 7) < kPolyOf8) {
                        exp2_poly_pair(a0, a1, p0, p1);
                    } else {
                        p0 = ex2_approx(a0);
                        p1 = ex2_approx(a1);
                    }
                    sum4[(i >> 1) & 3] += p0 + p1;
                    pk[i >> 1] = pack_f16x2(p0, p1);
                }
                if (c == 0 && !pv_waited) {
                    // first store into P's buffer: the previous product must have finished reading it
                    if (!mbar_wait(&ctl->pv_done[t], (j - 1) & 1, abort_flag)) {
                        ok = false;
                    }
                }
                // 32 keys = four 16-byte chunks of this row; chunk index within the 64-key half: (c & 1) * 4 + q
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + q);
                    st_shared_v4(p_row + (c >> 1) * kHalfBytes + ((chunk ^ swz) << 4), pk[4 * q], pk[4 * q + 1],
                                 pk[4 * q + 2], pk[4 * q + 3]);
                }
            }
            if (!ok) {
                break;
            }
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            fence_proxy_async_smem(); // the tensor core reads P through the asynchronous proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->p_full[t]);
            }
        }

        // output: O / l.  The rows go through shared memory - the P tile's buffer (free once the last product is
        // complete) and, for fp32 output, the Q tile's buffer as well - in 128-byte-swizzled column groups, and each
        // warp hands its 32 rows to TMA stores: full 128-byte lines instead of one row-strided 16-byte store per lane.
        if (ok && n > 0) {
            if (mbar_wait(&ctl->pv_done[t], (n - 1) & 1, abort_flag)) {
                tc_fence_after();
                const float inv_l = 1.0f / l_run;
                const uint32_t q_row_smem = smem_u32(smem_q) + t * kTileBytes + row_in_tile * 128;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t orow[32];
                    tmem_ld_32x32(o_addr + c * 32, orow);
                    tmem_ld_wait();
                    if (kOutF16) {
                        // 32 columns = four 16-byte chunks of the 64-column group c >> 1
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + i);
                            st_shared_v4(p_row + (c >> 1) * kHalfBytes + ((chunk ^ swz) << 4),
                                         pack_f16x2(__uint_as_float(orow[8 * i + 0]) * inv_l, __uint_as_float(orow[8 * i + 1]) * inv_l),
                                         pack_f16x2(__uint_as_float(orow[8 * i + 2]) * inv_l, __uint_as_float(orow[8 * i + 3]) * inv_l),
                                         pack_f16x2(__uint_as_float(orow[8 * i + 4]) * inv_l, __uint_as_float(orow[8 * i + 5]) * inv_l),
                                         pack_f16x2(__uint_as_float(orow[8 * i + 6]) * inv_l, __uint_as_float(orow[8 * i + 7]) * inv_l));
                        }
                    } else {
                        // 32 columns = one 128-byte group: groups 0, 1 in P's buffer, 2, 3 in Q's
                        const uint32_t base = ((c < 2) ? p_row : q_row_smem) + (c & 1) * kHalfBytes;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            st_shared_v4(base + ((static_cast<uint32_t>(i) ^ swz) << 4),
                                         __float_as_uint(__uint_as_float(orow[4 * i + 0]) * inv_l),
                                         __float_as_uint(__uint_as_float(orow[4 * i + 1]) * inv_l),
                                         __float_as_uint(__uint_as_float(orow[4 * i + 2]) * inv_l),
                                         __float_as_uint(__uint_as_float(orow[4 * i + 3]) * inv_l));
                        }
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const int row0 = (2 * qb + t) * kTileQ + quarter * 32; // this warp's 32 rows
                    uint8_t *p_src = smem_p + t * kTileBytes + quarter * 32 * 128;
                    uint8_t *q_src = smem_q + t * kTileBytes + quarter * 32 * 128;
                    if (kOutF16) {
                        tma_store_3d(&tmap_o, p_src, 0, row0, bh);
                        tma_store_3d(&tmap_o, p_src + kHalfBytes, 64, row0, bh);
                    } else {
                        tma_store_3d(&tmap_o, p_src, 0, row0, bh);
                        tma_store_3d(&tmap_o, p_src + kHalfBytes, 32, row0, bh);
                        tma_store_3d(&tmap_o, q_src, 64, row0, bh);
                        tma_store_3d(&tmap_o, q_src + kHalfBytes, 96, row0, bh);
                    }
                    tma_store_commit();
                    tma_store_wait_all<0>(); // the buffers are read and O is written before the block retires
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        profile_stamp(status, 1);
    }
    if (ctl->abort_flag) {
        for (int i = 0; i < 1024; ++i) {
            __nanosleep(1000);
        }
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, kErrDeviceWaitTimeout) == 0) {
            status->block = blockIdx.x;
            status->where = 2;
        }
        __syncthreads();
    }
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <bool kCausal, bool kOutF16, int kPolyOf8>
int launch_variant(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const CUtensorMap &to, int bh, int sq, int sk,
                   float scale_log2, float defer_log2, DeviceStatus *status, cudaStream_t stream)
{
    const int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(&flash_attn_fwd_kernel<kCausal, kOutF16, kPolyOf8>),
                                       kSmemBytes);
    if (rc != kOk) {
        return rc;
    }
    const int q_blocks = (sq + 2 * kTileQ - 1) / (2 * kTileQ);
    flash_attn_fwd_kernel<kCausal, kOutF16, kPolyOf8>
        <<<bh * q_blocks, kThreads, kSmemBytes, stream>>>(tq, tk, tv, to, sq, sk, scale_log2, defer_log2, status);
    return check_launch();
}

template <int kPolyOf8>
int launch_mode(bool causal, bool out_f16, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const CUtensorMap &to,
                int bh, int sq, int sk, float scale_log2, float defer_log2, DeviceStatus *status, cudaStream_t stream)
{
    if (causal) {
        return out_f16 ? launch_variant<true, true, kPolyOf8>(tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream)
                       : launch_variant<true, false, kPolyOf8>(tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
    }
    return out_f16 ? launch_variant<false, true, kPolyOf8>(tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream)
                   : launch_variant<false, false, kPolyOf8>(tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
}

} // namespace

int launch_flash_attn_fwd(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int bh, int sq, int sk,
                          int d, int causal, float scale, int out_f16, cudaStream_t stream, int defer_rescale)
{
    if (defer_rescale < 0) {
        defer_rescale = out_f16; // fp32 O: the reference's recurrence; fp16 O (the benchmark's configuration): deferred
    }
    const float defer_log2 = defer_rescale ? 8.0f : 0.0f;
    if (d != kD) {
        set_error_text("flash attention: head size must be 128");
        return kErrUnsupportedShape;
    }
    if ((sq % kTileQ) != 0 || (sk % kTileKV) != 0) {
        set_error_text("flash attention: sequence lengths must be multiples of 128");
        return kErrUnsupportedShape;
    }
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(o)) & 15u) {
        set_error_text("flash attention: operands must be 16-byte aligned");
        return kErrUnsupportedShape;
    }
    CUtensorMap tq, tk, tv, to;
    int rc = make_tmap_3d(&tq, q, 2, bh, sq, d, d, static_cast<uint64_t>(sq) * d, kTileQ, 64, true);
    if (rc == kOk) {
        rc = make_tmap_3d(&tk, k, 2, bh, sk, d, d, static_cast<uint64_t>(sk) * d, kTileKV, 64, true);
    }
    if (rc == kOk) {
        rc = make_tmap_3d(&tv, v, 2, bh, sk, d, d, static_cast<uint64_t>(sk) * d, kTileKV, 64, true);
    }
    if (rc == kOk) {
        // O leaves in boxes of 32 rows x 128 bytes (64 fp16 or 32 fp32 columns), one set per softmax warp
        rc = make_tmap_3d(&to, o, out_f16 ? 2 : 4, bh, sq, d, d, static_cast<uint64_t>(sq) * d, 32, out_f16 ? 64 : 32, true);
    }
    if (rc != kOk) {
        return rc;
    }
    DeviceStatus *status = device_status_ptr();
    if (status == nullptr) {
        return kErrCuda;
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    // share of the exponentials moved from the special-function unit to the FMA pipe (pairs out of every 8);
    // PTO_B200_FA_POLY overrides the default for experiments
    static const int poly = [] {
        const char *e = getenv("PTO_B200_FA_POLY");
        return e != nullptr ? atoi(e) : 1;
    }();
    switch (poly) {
        case 0: return launch_mode<0>(causal != 0, out_f16 != 0, tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
        case 2: return launch_mode<2>(causal != 0, out_f16 != 0, tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
        case 3: return launch_mode<3>(causal != 0, out_f16 != 0, tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
        case 4: return launch_mode<4>(causal != 0, out_f16 != 0, tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
        default: return launch_mode<1>(causal != 0, out_f16 != 0, tq, tk, tv, to, bh, sq, sk, scale_log2, defer_log2, status, stream);
    }
}

} // namespace pto_b200
