// Host launcher templates of the reference, over the C ABI of libpto_b200.so (include/pto_b200.h).
//
// The reference's host programs forward-declare launcher templates and link against the kernel translation unit that
// instantiates them: LaunchGEMME2E<T> (kernels/manual/a2a3/gemm_performance/main.cpp:16-17, instantiated at
// gemm_performance_kernel.cpp:243-264), LaunchTFA<...> (kernels/manual/common/flash_atten/fa_performance_kernel.h:
// 26-39), the unit-test launchers launchTCVT<D,S,...> (tests/cpu/st/testcase/tcvt/tcvt_kernel.cpp:54-64),
// launchTGATHER1D_demo_* (tgather_kernel.cpp:291-316), LaunchTROWMAX / LaunchTROWSUM / LaunchTExp
// (trowmax_kernel.cpp:40-56, trowsum_kernel.cpp:36-46, texp_kernel.cpp:32-44) and LaunchTMATMUL<key> /
// LaunchTMATMULBIAS<key> (tmatmul_kernel.cpp:157-201).  A host written against those declarations links against
// libpto_b200_launchers.so instead and runs on a B200: same names, same argument order, pointers are device pointers,
// the call enqueues on `stream` and returns (the caller synchronises), as in the reference.
//
// Not reproduced: the Ascend runtime (acl*); hosts use the CUDA runtime for memory and streams.
#pragma once

#include <cstddef>
#include <cstdint>

using aclFloat16 = uint16_t; // the reference's host-side name for a half (bits)
using aclrtStream = void *;

// C[6144 x 6144] fp32 = A[6144 x 6144] fp16 * B, B stored n x k: the problem the reference's kernel TU is built for.
template <typename T>
void LaunchGEMME2E(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream);
// the same launcher for another problem size (the reference fixes the size at compile time in the kernel TU)
template <typename T>
void LaunchGEMME2E(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream, uint32_t m, uint32_t k, uint32_t n);

// Flash-attention forward for one head: q [S0 x HEAD], k, v [S1 x HEAD] fp16, o_out [S0 x HEAD] fp32.  The FIFO and
// partial-result workspaces of the reference's cube / vector pipeline are accepted and not touched: the hand-offs
// stay on chip.  global_sum_out / exp_max_out / o_parts_out are debug outputs of the reference and stay unwritten.
template <int S0, int HEAD_SIZE, int S1, int CUBE_S0, int CUBE_S1 = 128, int TILE_S1 = 256, int QK_PRELOAD = 4,
          int CV_FIFO_SIZE = 8, bool INTERMEDIATE_CHECK = false, bool CAUSAL_MASK = false,
          int CV_FIFO_CONS_SYNC_PERIOD = 4>
void LaunchTFA(uint16_t *ffts, aclFloat16 *q, aclFloat16 *k, aclFloat16 *v, aclFloat16 *p_tile_fifo,
               float *exp_max_ififo, float *global_sum_out, float *exp_max_out, float *o_out, float *o_parts_out,
               float *qk_tile_fifo, float *pv_tile_fifo, uint8_t *profile_data, aclrtStream stream,
               uint8_t *cv_comm_buf = nullptr);
template <int S0, int HEAD_SIZE, int S1, int CUBE_S0, int CUBE_S1, int TILE_S1, int QK_PRELOAD, int CV_FIFO_SIZE,
          bool INTERMEDIATE_CHECK, bool CAUSAL_MASK, int CV_FIFO_CONS_SYNC_PERIOD>
void LaunchTFA(uint16_t *ffts, aclFloat16 *q, aclFloat16 *k, aclFloat16 *v, aclFloat16 *p_tile_fifo,
               float *exp_max_ififo, float *global_sum_out, float *exp_max_out, float *o_out, float *o_parts_out,
               float *qk_tile_fifo, float *pv_tile_fifo, aclrtStream stream, uint8_t *cv_comm_buf = nullptr);

// unit-test launchers
template <typename D, typename S, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void launchTCVT(D *dst, S *src, void *stream);
void launchTGATHER1D_demo_float(float *out, float *src0, int32_t *src1, aclrtStream stream);
void launchTGATHER1D_demo_int32(int32_t *out, int32_t *src0, int32_t *src1, aclrtStream stream);
void launchTGATHER1D_demo_half(int16_t *out, int16_t *src0, int32_t *src1, aclrtStream stream);
void launchTGATHER1D_demo_int16(int16_t *out, int16_t *src0, int32_t *src1, aclrtStream stream);
template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTROWMAX(T *out, T *src, void *stream);
template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTROWSUM(T *out, T *src, void *stream);
template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTExp(T *out, T *src, void *stream);
// the flash-attention unit-test program, one 64 x 32 fp32 head (tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp:
// 110-114), the reference's own tile program compiled for B200
void LaunchTFLASHATTN(float *out, float *q, float *k, float *v, void *stream);
// keys as in the reference: 1 half 40 x 50 x 60, 2 int8 6 x 7 x 8, 3 five accumulated half 128 x 128 x 64 products,
// 4 float 120 x 110 x 50; bias keys 1 int8 8 x 7 x 6, 2 half 16 x 15 x 16, 5 float 127 x 128 x 63.  These run the
// reference's own tile programs compiled for B200 (libpto_b200_refkernels.so).
template <int32_t tilingKey>
void LaunchTMATMUL(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream);
template <int32_t tilingKey>
void LaunchTMATMULBIAS(uint8_t *out, uint8_t *src0, uint8_t *src1, uint8_t *src2, void *stream);

// status of the last launcher call on this thread (0 = enqueued); the reference's launchers return void
int pto_b200_launcher_status();
