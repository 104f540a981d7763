// Definitions and explicit instantiations of the reference's host launcher templates (include/pto_b200_launchers.hpp)
// over the C ABI.  Built into libpto_b200_launchers.so by pto_isa_b200/build.py.
#include "../../../include/pto_b200_launchers.hpp"

#include <cmath>

#include "../../../include/pto_b200.h"

// entry points of libpto_b200_refkernels.so (the reference's tile programs compiled for B200); resolved at link time
// when that library was built, otherwise LaunchTMATMUL reports PTO_B200_ERR_UNSUPPORTED_SHAPE
extern "C" {
int pto_refk_tmatmul(int key, uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream) __attribute__((weak));
int pto_refk_tmatmul_bias(int key, uint8_t *out, uint8_t *src0, uint8_t *src1, uint8_t *src2, void *stream)
    __attribute__((weak));
int pto_refk_tflashattn_64x32(float *out, float *q, float *k, float *v, void *stream, int *status_dev) __attribute__((weak));
}

namespace {
thread_local int g_status = 0;
}

int pto_b200_launcher_status()
{
    return g_status;
}

// ---------------------------------------------------------------- GEMM
template <typename T>
void LaunchGEMME2E(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream, uint32_t m, uint32_t k, uint32_t n)
{
    static_assert(sizeof(T) == 2, "LaunchGEMME2E: 16-bit (half) operands");
    g_status = pto_b200_gemm_f16f32(reinterpret_cast<const uint16_t *>(src0), reinterpret_cast<const uint16_t *>(src1),
                                    reinterpret_cast<float *>(out), static_cast<int>(m), static_cast<int>(n),
                                    static_cast<int>(k), /*b_layout: n x k*/ 1, stream);
}
template <typename T>
void LaunchGEMME2E(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream)
{
    LaunchGEMME2E<T>(out, src0, src1, stream, 6144, 6144, 6144);
}
template void LaunchGEMME2E<uint16_t>(uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchGEMME2E<uint16_t>(uint8_t *, uint8_t *, uint8_t *, void *, uint32_t, uint32_t, uint32_t);

// ---------------------------------------------------------------- flash attention
template <int S0, int HEAD_SIZE, int S1, int CUBE_S0, int CUBE_S1, int TILE_S1, int QK_PRELOAD, int CV_FIFO_SIZE,
          bool INTERMEDIATE_CHECK, bool CAUSAL_MASK, int CV_FIFO_CONS_SYNC_PERIOD>
void LaunchTFA(uint16_t *, aclFloat16 *q, aclFloat16 *k, aclFloat16 *v, aclFloat16 *, float *, float *, float *,
               float *o_out, float *, float *, float *, uint8_t *, aclrtStream stream, uint8_t *)
{
    // the reference applies 1 / sqrt(HEAD_SIZE) inside its softmax (pto_macro_fa_softmax.hpp:31-45)
    g_status = pto_b200_flash_attn_fwd_f16(q, k, v, o_out, 1, S0, S1, HEAD_SIZE, CAUSAL_MASK ? 1 : 0,
                                           1.0f / std::sqrt(static_cast<float>(HEAD_SIZE)), /*out_f16*/ 0, stream);
}
template <int S0, int HEAD_SIZE, int S1, int CUBE_S0, int CUBE_S1, int TILE_S1, int QK_PRELOAD, int CV_FIFO_SIZE,
          bool INTERMEDIATE_CHECK, bool CAUSAL_MASK, int CV_FIFO_CONS_SYNC_PERIOD>
void LaunchTFA(uint16_t *ffts, aclFloat16 *q, aclFloat16 *k, aclFloat16 *v, aclFloat16 *p_tile_fifo,
               float *exp_max_ififo, float *global_sum_out, float *exp_max_out, float *o_out, float *o_parts_out,
               float *qk_tile_fifo, float *pv_tile_fifo, aclrtStream stream, uint8_t *cv_comm_buf)
{
    LaunchTFA<S0, HEAD_SIZE, S1, CUBE_S0, CUBE_S1, TILE_S1, QK_PRELOAD, CV_FIFO_SIZE, INTERMEDIATE_CHECK, CAUSAL_MASK,
              CV_FIFO_CONS_SYNC_PERIOD>(ffts, q, k, v, p_tile_fifo, exp_max_ififo, global_sum_out, exp_max_out, o_out,
                                        o_parts_out, qk_tile_fifo, pv_tile_fifo, nullptr, stream, cv_comm_buf);
}
// the default case list of the reference's generator (kernels/manual/common/flash_atten/scripts/generate_cases.py:
// head 128, s0 in {128, 1024}, s1 in {1024 .. 8192}) plus causal squares
#define PTO_B200_TFA_CASE(S0, S1, CUBE_S0, CAUSAL)                                                                       \
    template void LaunchTFA<S0, 128, S1, CUBE_S0, 128, 256, 4, 8, false, CAUSAL, 4>(                                    \
        uint16_t *, aclFloat16 *, aclFloat16 *, aclFloat16 *, aclFloat16 *, float *, float *, float *, float *, float *, \
        float *, float *, uint8_t *, aclrtStream, uint8_t *);                                                           \
    template void LaunchTFA<S0, 128, S1, CUBE_S0, 128, 256, 4, 8, false, CAUSAL, 4>(                                    \
        uint16_t *, aclFloat16 *, aclFloat16 *, aclFloat16 *, aclFloat16 *, float *, float *, float *, float *, float *, \
        float *, float *, aclrtStream, uint8_t *);
PTO_B200_TFA_CASE(128, 1024, 128, false)
PTO_B200_TFA_CASE(128, 2048, 128, false)
PTO_B200_TFA_CASE(128, 4096, 128, false)
PTO_B200_TFA_CASE(128, 8192, 128, false)
PTO_B200_TFA_CASE(1024, 1024, 128, false)
PTO_B200_TFA_CASE(1024, 2048, 128, false)
PTO_B200_TFA_CASE(1024, 4096, 128, false)
PTO_B200_TFA_CASE(1024, 8192, 128, false)
PTO_B200_TFA_CASE(1024, 1024, 128, true)
PTO_B200_TFA_CASE(2048, 2048, 128, true)
#undef PTO_B200_TFA_CASE

// ---------------------------------------------------------------- unit-test launchers
template <typename D, typename S, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void launchTCVT(D *dst, S *src, void *stream)
{
    static_assert(sizeof(S) == 4, "launchTCVT: fp32 sources");
    const int64_t n = static_cast<int64_t>(kGRows_) * kGCols_;
    if constexpr (sizeof(D) == 2) {
        g_status = pto_b200_tcvt_f32_f16(reinterpret_cast<const float *>(src), reinterpret_cast<uint16_t *>(dst), n, stream);
    } else {
        g_status = pto_b200_tcvt_f32_i32(reinterpret_cast<const float *>(src), reinterpret_cast<int32_t *>(dst), n,
                                         /*CAST_RINT*/ 1, stream);
    }
}
template void launchTCVT<aclFloat16, float, 64, 64, 64, 64>(aclFloat16 *, float *, void *);
template void launchTCVT<int32_t, float, 128, 128, 128, 128>(int32_t *, float *, void *);
template void launchTCVT<int32_t, float, 32, 512, 32, 512>(int32_t *, float *, void *);
template void launchTCVT<int32_t, float, 4, 4096, 4, 4096>(int32_t *, float *, void *);

void launchTGATHER1D_demo_float(float *out, float *src0, int32_t *src1, aclrtStream stream)
{
    g_status = pto_b200_tgather(src0, 32 * 1024, src1, out, 16 * 64, 4, stream);
}
void launchTGATHER1D_demo_int32(int32_t *out, int32_t *src0, int32_t *src1, aclrtStream stream)
{
    g_status = pto_b200_tgather(src0, 32 * 512, src1, out, 16 * 256, 4, stream);
}
void launchTGATHER1D_demo_half(int16_t *out, int16_t *src0, int32_t *src1, aclrtStream stream)
{
    g_status = pto_b200_tgather(src0, 16 * 1024, src1, out, 16 * 128, 2, stream);
}
void launchTGATHER1D_demo_int16(int16_t *out, int16_t *src0, int32_t *src1, aclrtStream stream)
{
    g_status = pto_b200_tgather(src0, 32 * 256, src1, out, 32 * 64, 2, stream);
}

template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTROWMAX(T *out, T *src, void *stream)
{
    static_assert(sizeof(T) == 4, "LaunchTROWMAX: fp32");
    g_status = pto_b200_trowmax_f32(src, out, kTRows_, kTCols_, kTCols_, stream);
}
template void LaunchTROWMAX<float, 64, 64, 64, 64>(float *, float *, void *);
template void LaunchTROWMAX<float, 32, 32, 32, 16>(float *, float *, void *);

template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTROWSUM(T *out, T *src, void *stream)
{
    static_assert(sizeof(T) == 4, "LaunchTROWSUM: fp32");
    g_status = pto_b200_trowsum_f32(src, out, kTRows_, kTCols_, kTCols_, stream);
}
template void LaunchTROWSUM<float, 64, 64, 64, 64>(float *, float *, void *);

template <typename T, int kGRows_, int kGCols_, int kTRows_, int kTCols_>
void LaunchTExp(T *out, T *src, void *stream)
{
    static_assert(sizeof(T) == 4, "LaunchTExp: fp32");
    g_status = pto_b200_texp_f32(src, out, static_cast<int64_t>(kTRows_) * kTCols_, stream);
}
template void LaunchTExp<float, 64, 64, 64, 64>(float *, float *, void *);
template void LaunchTExp<float, 32, 32, 32, 32>(float *, float *, void *);

template <int32_t tilingKey>
void LaunchTMATMUL(uint8_t *out, uint8_t *src0, uint8_t *src1, void *stream)
{
    g_status = pto_refk_tmatmul != nullptr ? pto_refk_tmatmul(tilingKey, out, src0, src1, stream)
                                           : PTO_B200_ERR_UNSUPPORTED_SHAPE;
}
template void LaunchTMATMUL<1>(uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchTMATMUL<2>(uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchTMATMUL<3>(uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchTMATMUL<4>(uint8_t *, uint8_t *, uint8_t *, void *);

void LaunchTFLASHATTN(float *out, float *q, float *k, float *v, void *stream)
{
    g_status = pto_refk_tflashattn_64x32 != nullptr
                   ? pto_refk_tflashattn_64x32(out, q, k, v, stream, static_cast<int *>(pto_b200_status_record()))
                   : PTO_B200_ERR_UNSUPPORTED_SHAPE;
}

template <int32_t tilingKey>
void LaunchTMATMULBIAS(uint8_t *out, uint8_t *src0, uint8_t *src1, uint8_t *src2, void *stream)
{
    g_status = pto_refk_tmatmul_bias != nullptr ? pto_refk_tmatmul_bias(tilingKey, out, src0, src1, src2, stream)
                                                : PTO_B200_ERR_UNSUPPORTED_SHAPE;
}
template void LaunchTMATMULBIAS<1>(uint8_t *, uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchTMATMULBIAS<2>(uint8_t *, uint8_t *, uint8_t *, uint8_t *, void *);
template void LaunchTMATMULBIAS<5>(uint8_t *, uint8_t *, uint8_t *, uint8_t *, void *);
