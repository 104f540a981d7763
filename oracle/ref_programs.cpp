// TEST INFRASTRUCTURE ONLY - never linked into or called from the product library.
//
// Small PTO tile programs compiled against the *reference's own* CPU-simulation headers
// (`-D__CPU_SIM -I<reference>/include`); nothing from the reference is copied here, the headers
// are included from where they lie.  The resulting shared object (oracle/_ref/libpto_ref.so) is
// the ground truth the C restatement in pto_oracle.c is pinned against, and may serve as the
// timed CPU baseline ("kind": "reference").
//
// Each program mirrors the instruction sequence of the reference test kernel it cites:
//   TCVT     tests/cpu/st/testcase/tcvt/tcvt_kernel.cpp:17-52     (TLOAD -> TCVT(CAST_RINT) -> TSTORE)
//   TGATHER  tests/cpu/st/testcase/tgather/tgather_kernel.cpp:224-269 (index form), :158-198 (mask form)
//   TROWMAX / TROWSUM / TEXP   tests/cpu/st/testcase/{trowmax,trowsum,texp}/*_kernel.cpp
//   GEMM     kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:67-149
//            (TLOAD -> TEXTRACT -> TMATMUL / TMATMUL_ACC per 64-wide k step -> TSTORE, base tile 128x256)
//   attention  tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp:84-105 with fp16 operands
//
// All entry points take host pointers and return 0, or -1 for a shape that has no
// instantiation here (tile shapes are compile-time in the PTO surface).
#include <pto/pto-inst.hpp>
#include <pto/common/pto_tile.hpp>
#include <pto/common/constants.hpp>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdfloat>

using namespace pto;

namespace {

// ---------------------------------------------------------------- elementwise, chunked
// Elementwise ops are run over [1 x kChunk] tiles with a dynamic valid column count, so any
// length is covered by the same tile program.
constexpr int kChunk = 8192;

template <typename D, typename S, typename Fn>
void ForChunks(D *dst, const S *src, int64_t n, Fn fn)
{
    using GShape = Shape<1, 1, 1, 1, DYNAMIC>;
    using GStride = pto::Stride<1, 1, 1, DYNAMIC, 1>;
    using TileS = Tile<TileType::Vec, S, 1, kChunk, BLayout::RowMajor, 1, DYNAMIC>;
    using TileD = Tile<TileType::Vec, D, 1, kChunk, BLayout::RowMajor, 1, DYNAMIC>;
    for (int64_t off = 0; off < n; off += kChunk) {
        const int64_t len = (n - off < kChunk) ? (n - off) : kChunk;
        TileS s(static_cast<size_t>(len));
        TileD d(static_cast<size_t>(len));
        GlobalTensor<S, GShape, GStride> gs(const_cast<S *>(src) + off, GShape(len), GStride(len));
        GlobalTensor<D, GShape, GStride> gd(dst + off, GShape(len), GStride(len));
        TLOAD(s, gs);
        fn(d, s);
        TSTORE(gd, d);
    }
}

// ---------------------------------------------------------------- TGATHER index form
template <typename T, int SR, int SC>
void GatherIdx(T *dst, const T *src0, const int32_t *idx, int64_t n)
{
    using Src0Tile = Tile<TileType::Vec, T, SR, SC, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    using G0Shape = Shape<1, 1, 1, SR, SC>;
    using G0Stride = pto::Stride<1, 1, 1, SC, 1>;
    auto s0 = std::make_unique<Src0Tile>(static_cast<size_t>(SR), static_cast<size_t>(SC));
    GlobalTensor<T, G0Shape, G0Stride> g0(const_cast<T *>(src0));
    TLOAD(*s0, g0);

    using GShape = Shape<1, 1, 1, 1, DYNAMIC>;
    using GStride = pto::Stride<1, 1, 1, DYNAMIC, 1>;
    using IdxTile = Tile<TileType::Vec, int32_t, 1, kChunk, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    using DstTile = Tile<TileType::Vec, T, 1, kChunk, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    for (int64_t off = 0; off < n; off += kChunk) {
        const int64_t len = (n - off < kChunk) ? (n - off) : kChunk;
        IdxTile it(1, static_cast<size_t>(len));
        DstTile dt(1, static_cast<size_t>(len));
        GlobalTensor<int32_t, GShape, GStride> gi(const_cast<int32_t *>(idx) + off, GShape(len), GStride(len));
        GlobalTensor<T, GShape, GStride> gd(dst + off, GShape(len), GStride(len));
        TLOAD(it, gi);
        TGATHER(dt, *s0, it);
        TSTORE(gd, dt);
    }
}

// ---------------------------------------------------------------- TGATHER mask form
template <typename T, int R, int C, MaskPattern P>
void GatherMask(T *dst, const T *src)
{
    constexpr int kDiv = (P == MaskPattern::P1111) ? 1 : ((P == MaskPattern::P0101 || P == MaskPattern::P1010) ? 2 : 4);
    constexpr int DC = C / kDiv;
    using SrcTile = Tile<TileType::Vec, T, R, C, BLayout::RowMajor>;
    using DstTile = Tile<TileType::Vec, T, R, DC, BLayout::RowMajor>;
    auto s = std::make_unique<SrcTile>();
    auto d = std::make_unique<DstTile>();
    GlobalTensor<T, Shape<1, 1, 1, R, C>, pto::Stride<1, 1, 1, C, 1>> gs(const_cast<T *>(src));
    GlobalTensor<T, Shape<1, 1, 1, R, DC>, pto::Stride<1, 1, 1, DC, 1>> gd(dst);
    TLOAD(*s, gs);
    TGATHER<DstTile, SrcTile, P>(*d, *s);
    TSTORE(gd, *d);
}

template <typename T, int R, int C>
int GatherMaskDispatch(T *dst, const T *src, int pattern)
{
    switch (pattern) {
        case 1: GatherMask<T, R, C, MaskPattern::P0101>(dst, src); return 0;
        case 2: GatherMask<T, R, C, MaskPattern::P1010>(dst, src); return 0;
        case 3: GatherMask<T, R, C, MaskPattern::P0001>(dst, src); return 0;
        case 4: GatherMask<T, R, C, MaskPattern::P0010>(dst, src); return 0;
        case 5: GatherMask<T, R, C, MaskPattern::P0100>(dst, src); return 0;
        case 6: GatherMask<T, R, C, MaskPattern::P1000>(dst, src); return 0;
        case 7: GatherMask<T, R, C, MaskPattern::P1111>(dst, src); return 0;
        default: return -1;
    }
}

// ---------------------------------------------------------------- row reductions
constexpr int kRedRows = 8;
constexpr int kRedCols = 8192;

template <bool kIsMax>
int RowReduce(float *dst, const float *src, int rows, int cols)
{
    if (cols > kRedCols || cols <= 0) {
        return -1;
    }
    using SrcTile = Tile<TileType::Vec, float, kRedRows, kRedCols, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    using DstTile = Tile<TileType::Vec, float, kRedRows, 1, BLayout::ColMajor, DYNAMIC, 1>;
    using GShape = Shape<1, 1, 1, DYNAMIC, DYNAMIC>;
    using GStride = pto::Stride<1, 1, 1, DYNAMIC, 1>;
    auto s = std::make_unique<SrcTile>(1, 1);
    for (int r0 = 0; r0 < rows; r0 += kRedRows) {
        const int nr = (rows - r0 < kRedRows) ? (rows - r0) : kRedRows;
        s->RowMaskInternal = nr;
        s->ColMaskInternal = cols;
        DstTile d(static_cast<size_t>(nr));
        GlobalTensor<float, GShape, GStride> gs(const_cast<float *>(src) + static_cast<int64_t>(r0) * cols,
                                                GShape(nr, cols), GStride(cols));
        TLOAD(*s, gs);
        if constexpr (kIsMax) {
            TROWMAX(d, *s, *s);
        } else {
            TROWSUM(d, *s, *s);
        }
        for (int r = 0; r < nr; ++r) {
            dst[r0 + r] = d.data()[r];
        }
    }
    return 0;
}

// ---------------------------------------------------------------- GEMM tile program
// One C tile of 128x256 at a time; per 64-wide k step: TLOAD A[128x64], TLOAD B[64x256],
// TEXTRACT both at (0,0) into Left/Right tiles, TMATMUL (first step) or TMATMUL_ACC.
template <Layout kLayoutB>
int GemmTiles(float *c, const half *a, const half *b, int m, int n, int k, int tile_begin, int tile_end)
{
    constexpr int BM = 128, BN = 256, BK = 64;
    if (m % BM || n % BN || k % BK) {
        return -1;
    }
    using TileMatA = Tile<TileType::Mat, half, BM, BK, BLayout::ColMajor, BM, BK, SLayout::RowMajor>;
    using TileMatB = Tile<TileType::Mat, half, BK, BN, BLayout::RowMajor, BK, BN, SLayout::ColMajor>;
    using LeftT = TileLeft<half, BM, BK, BM, BK>;
    using RightT = TileRight<half, BK, BN, BK, BN>;
    using AccT = TileAcc<float, BM, BN, BM, BN>;
    using GA = GlobalTensor<half, TileShape2D<half, BM, BK, Layout::ND>, BaseShape2D<half, DYNAMIC, DYNAMIC, Layout::ND>,
                            Layout::ND>;
    using GB = GlobalTensor<half, TileShape2D<half, BK, BN, kLayoutB>, BaseShape2D<half, DYNAMIC, DYNAMIC, kLayoutB>,
                            kLayoutB>;
    using GC = GlobalTensor<float, TileShape2D<float, BM, BN, Layout::ND>,
                            BaseShape2D<float, DYNAMIC, DYNAMIC, Layout::ND>, Layout::ND>;
    auto aMat = std::make_unique<TileMatA>();
    auto bMat = std::make_unique<TileMatB>();
    auto aT = std::make_unique<LeftT>();
    auto bT = std::make_unique<RightT>();
    auto cT = std::make_unique<AccT>();
    const int tiles_n = n / BN;
    for (int t = tile_begin; t < tile_end; ++t) {
        const int ti = t / tiles_n, tj = t % tiles_n;
        for (int kk = 0; kk < k; kk += BK) {
            GA ga(const_cast<half *>(a) + static_cast<int64_t>(ti) * BM * k + kk, TileShape2D<half, BM, BK, Layout::ND>(),
                  BaseShape2D<half, DYNAMIC, DYNAMIC, Layout::ND>(m, k));
            const half *bp = (kLayoutB == Layout::ND) ? b + static_cast<int64_t>(kk) * n + static_cast<int64_t>(tj) * BN
                                                      : b + static_cast<int64_t>(tj) * BN * k + kk;
            GB gb(const_cast<half *>(bp), TileShape2D<half, BK, BN, kLayoutB>(),
                  BaseShape2D<half, DYNAMIC, DYNAMIC, kLayoutB>(k, n));
            TLOAD(*aMat, ga);
            TLOAD(*bMat, gb);
            TEXTRACT(*aT, *aMat, 0, 0);
            TEXTRACT(*bT, *bMat, 0, 0);
            if (kk == 0) {
                TMATMUL(*cT, *aT, *bT);
            } else {
                TMATMUL_ACC(*cT, *cT, *aT, *bT);
            }
        }
        GC gc(c + static_cast<int64_t>(ti) * BM * n + static_cast<int64_t>(tj) * BN,
              TileShape2D<float, BM, BN, Layout::ND>(), BaseShape2D<float, DYNAMIC, DYNAMIC, Layout::ND>(m, n));
        TSTORE(gc, *cT);
    }
    return 0;
}

// ---------------------------------------------------------------- small TMATMUL (one tile, any valid m,k,n)
template <typename CT, typename AT, int M, int K, int N>
void MatmulOne(CT *c, const AT *a, const AT *b)
{
    constexpr int A16 = 16;
    constexpr int MP = (M + A16 - 1) / A16 * A16, KP = (K + A16 - 1) / A16 * A16, NP = (N + A16 - 1) / A16 * A16;
    using MatA = Tile<TileType::Mat, AT, MP, KP, BLayout::ColMajor, M, K, SLayout::RowMajor, 512>;
    using MatB = Tile<TileType::Mat, AT, KP, NP, BLayout::ColMajor, K, N, SLayout::RowMajor, 512>;
    using LeftT = TileLeft<AT, MP, KP, M, K>;
    using RightT = TileRight<AT, KP, NP, K, N>;
    using AccT = TileAcc<CT, MP, NP, M, N>;
    auto aMat = std::make_unique<MatA>();
    auto bMat = std::make_unique<MatB>();
    auto aT = std::make_unique<LeftT>();
    auto bT = std::make_unique<RightT>();
    auto cT = std::make_unique<AccT>();
    GlobalTensor<AT, Shape<1, 1, 1, M, K>, pto::Stride<M * K, M * K, M * K, K, 1>> ga(const_cast<AT *>(a));
    GlobalTensor<AT, Shape<1, 1, 1, K, N>, pto::Stride<K * N, K * N, K * N, N, 1>> gb(const_cast<AT *>(b));
    GlobalTensor<CT, Shape<1, 1, 1, M, N>, pto::Stride<M * N, M * N, M * N, N, 1>> gc(c);
    TLOAD(*aMat, ga);
    TLOAD(*bMat, gb);
    TMOV(*aT, *aMat);
    TMOV(*bT, *bMat);
    TMATMUL(*cT, *aT, *bT);
    TSTORE(gc, *cT);
}

// ---------------------------------------------------------------- attention, one head
// The plain (untiled) instruction sequence of the reference flash-attention test, with fp16
// Q/K/V operands, fp32 scores/softmax and fp16 probabilities feeding the second product.
// scores = (Q K^T) * scale ; P = exp(scores - rowmax) ; O = (fp16(P) V) / rowsum(P)
template <int S0, int S1, int D>
void AttnHead(float *o, const half *q, const half *k, const half *v, float scale, int causal)
{
    using GQ = GlobalTensor<half, Shape<1, 1, 1, S0, D>, pto::Stride<S0 * D, S0 * D, S0 * D, D, 1>>;
    using GKT = GlobalTensor<half, Shape<1, 1, 1, D, S1>, pto::Stride<S1 * D, S1 * D, S1 * D, 1, D>, Layout::DN>;
    using GV = GlobalTensor<half, Shape<1, 1, 1, S1, D>, pto::Stride<S1 * D, S1 * D, S1 * D, D, 1>>;
    using GO = GlobalTensor<float, Shape<1, 1, 1, S0, D>, pto::Stride<S0 * D, S0 * D, S0 * D, D, 1>>;
    using QMat = Tile<TileType::Mat, half, S0, D, BLayout::ColMajor, S0, D, SLayout::RowMajor>;
    using KTMat = Tile<TileType::Mat, half, D, S1, BLayout::RowMajor, D, S1, SLayout::ColMajor>;
    using VMat = Tile<TileType::Mat, half, S1, D, BLayout::RowMajor, S1, D, SLayout::ColMajor>;
    using LeftQ = TileLeft<half, S0, D, S0, D>;
    using RightKT = TileRight<half, D, S1, D, S1>;
    using AccS = TileAcc<float, S0, S1, S0, S1>;
    using ScoresPlain = Tile<TileType::Vec, float, S0, S1, BLayout::RowMajor, S0, S1, SLayout::NoneBox>;
    using RowRed = Tile<TileType::Vec, float, S0, 1, BLayout::ColMajor, S0, 1, SLayout::NoneBox>;
    using ProbsHalf = Tile<TileType::Vec, half, S0, S1, BLayout::RowMajor, S0, S1, SLayout::NoneBox>;
    using LeftP = TileLeft<half, S0, S1, S0, S1>;
    using RightV = TileRight<half, S1, D, S1, D>;
    using AccO = TileAcc<float, S0, D, S0, D>;
    using OutPlain = Tile<TileType::Vec, float, S0, D, BLayout::RowMajor, S0, D, SLayout::NoneBox>;

    auto qMat = std::make_unique<QMat>();
    auto ktMat = std::make_unique<KTMat>();
    auto vMat = std::make_unique<VMat>();
    auto qL = std::make_unique<LeftQ>();
    auto kR = std::make_unique<RightKT>();
    auto sAcc = std::make_unique<AccS>();
    auto scores = std::make_unique<ScoresPlain>();
    auto rowMax = std::make_unique<RowRed>();
    auto rowSum = std::make_unique<RowRed>();
    auto pHalf = std::make_unique<ProbsHalf>();
    auto pL = std::make_unique<LeftP>();
    auto vR = std::make_unique<RightV>();
    auto oAcc = std::make_unique<AccO>();
    auto oPlain = std::make_unique<OutPlain>();

    GQ gq(const_cast<half *>(q));
    GKT gkt(const_cast<half *>(k));
    GV gv(const_cast<half *>(v));
    GO go(o);
    TLOAD(*qMat, gq);
    TLOAD(*ktMat, gkt);
    TLOAD(*vMat, gv);
    TMOV(*qL, *qMat);
    TMOV(*kR, *ktMat);
    TMATMUL(*sAcc, *qL, *kR);
    TMOV(*scores, *sAcc);
    if (causal) {
        // keys beyond the query's own position get the reference's "-inf" stand-in added
        // (kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:64-79: triu(1) * -3.40282e38)
        auto tri = std::make_unique<ScoresPlain>();
        TTRI<ScoresPlain, 1>(*tri, 1);
        TMULS(*tri, *tri, -3.40282e+38f);
        TADD(*scores, *scores, *tri);
    }
    TROWMAX(*rowMax, *scores, *scores);
    TROWEXPANDSUB(*scores, *scores, *rowMax);
    TMULS(*scores, *scores, scale);
    TEXP(*scores, *scores);
    TROWSUM(*rowSum, *scores, *scores);
    TCVT(*pHalf, *scores, RoundMode::CAST_ROUND);
    TMOV(*pL, *pHalf);
    TMOV(*vR, *vMat);
    TMATMUL(*oAcc, *pL, *vR);
    TMOV(*oPlain, *oAcc);
    TROWEXPANDDIV(*oPlain, *oPlain, *rowSum);
    TSTORE(go, *oPlain);
}

} // namespace

extern "C" {

int pto_ref_tcvt_f32_f16(const float *src, uint16_t *dst, int64_t n)
{
    ForChunks(reinterpret_cast<half *>(dst), src, n, [](auto &d, auto &s) { TCVT(d, s, RoundMode::CAST_RINT); });
    return 0;
}

// pto::bfloat16_t aliases _Float16 with this compiler (include/pto/common/type.hpp:257-268), so the
// bf16 destination tile is declared over std::bfloat16_t and runs through the same TCVT_IMPL.
int pto_ref_tcvt_f32_bf16(const float *src, uint16_t *dst, int64_t n)
{
    ForChunks(reinterpret_cast<std::bfloat16_t *>(dst), src, n,
              [](auto &d, auto &s) { TCVT(d, s, RoundMode::CAST_RINT); });
    return 0;
}

int pto_ref_tcvt_f32_i32(const float *src, int32_t *dst, int64_t n, int mode)
{
    ForChunks(dst, src, n, [mode](auto &d, auto &s) { TCVT(d, s, static_cast<RoundMode>(mode)); });
    return 0;
}

int pto_ref_texp_f32(const float *src, float *dst, int64_t n)
{
    ForChunks(dst, src, n, [](auto &d, auto &s) { TEXP(d, s); });
    return 0;
}

int pto_ref_tgather_f32(const float *src0, int src_rows, int src_cols, const int32_t *idx, float *dst, int64_t n)
{
    if (src_rows == 32 && src_cols == 1024) {
        GatherIdx<float, 32, 1024>(dst, src0, idx, n);
    } else if (src_rows == 64 && src_cols == 64) {
        GatherIdx<float, 64, 64>(dst, src0, idx, n);
    } else if (src_rows == 512 && src_cols == 2048) {
        GatherIdx<float, 512, 2048>(dst, src0, idx, n);
    } else if (src_rows == 4096 && src_cols == 4096) {
        GatherIdx<float, 4096, 4096>(dst, src0, idx, n);
    } else {
        return -1;
    }
    return 0;
}

int pto_ref_tgather_b16(const uint16_t *src0, int src_rows, int src_cols, const int32_t *idx, uint16_t *dst, int64_t n)
{
    auto *d = reinterpret_cast<int16_t *>(dst);
    auto *s = reinterpret_cast<const int16_t *>(src0);
    if (src_rows == 16 && src_cols == 1024) {
        GatherIdx<int16_t, 16, 1024>(d, s, idx, n);
    } else if (src_rows == 32 && src_cols == 256) {
        GatherIdx<int16_t, 32, 256>(d, s, idx, n);
    } else if (src_rows == 1024 && src_cols == 1024) {
        GatherIdx<int16_t, 1024, 1024>(d, s, idx, n);
    } else {
        return -1;
    }
    return 0;
}

int pto_ref_tgather_mask_f32(const float *src, float *dst, int rows, int cols, int pattern)
{
    if (rows == 16 && cols == 64) {
        return GatherMaskDispatch<float, 16, 64>(dst, src, pattern);
    }
    if (rows == 64 && cols == 256) {
        return GatherMaskDispatch<float, 64, 256>(dst, src, pattern);
    }
    if (rows == 256 && cols == 1024) {
        return GatherMaskDispatch<float, 256, 1024>(dst, src, pattern);
    }
    return -1;
}

int pto_ref_tgather_mask_b16(const uint16_t *src, uint16_t *dst, int rows, int cols, int pattern)
{
    auto *d = reinterpret_cast<int16_t *>(dst);
    auto *s = reinterpret_cast<const int16_t *>(src);
    if (rows == 16 && cols == 64) {
        return GatherMaskDispatch<int16_t, 16, 64>(d, s, pattern);
    }
    if (rows == 64 && cols == 256) {
        return GatherMaskDispatch<int16_t, 64, 256>(d, s, pattern);
    }
    return -1;
}

int pto_ref_trowmax_f32(const float *src, float *dst, int rows, int cols)
{
    return RowReduce<true>(dst, src, rows, cols);
}

int pto_ref_trowsum_f32(const float *src, float *dst, int rows, int cols)
{
    return RowReduce<false>(dst, src, rows, cols);
}

// b_layout 0: B is k x n row-major (Layout::ND); 1: B is stored n x k row-major, i.e. the
// column-major k x n view (Layout::DN) the reference GEMM kernel uses for its second operand.
// Tiles [tile_begin, tile_end) of the 128x256 C-tile grid (row-major tile order) are computed.
int pto_ref_gemm_f16f32_tiles(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                              int tile_begin, int tile_end)
{
    auto *ah = reinterpret_cast<const half *>(a);
    auto *bh = reinterpret_cast<const half *>(b);
    if (b_layout == 0) {
        return GemmTiles<Layout::ND>(c, ah, bh, m, n, k, tile_begin, tile_end);
    }
    return GemmTiles<Layout::DN>(c, ah, bh, m, n, k, tile_begin, tile_end);
}

int pto_ref_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout)
{
    if (m % 128 || n % 256) {
        return -1;
    }
    return pto_ref_gemm_f16f32_tiles(a, b, c, m, n, k, b_layout, 0, (m / 128) * (n / 256));
}

// Single-tile TMATMUL cases of the reference's own unit test
// (tests/cpu/st/testcase/tmatmul/main.cpp:97-170: 40x50x60 and 128x128x64 f16->f32, 120x110x50 f32).
int pto_ref_tmatmul_case(int which, const void *a, const void *b, void *c)
{
    switch (which) {
        case 1:
            MatmulOne<float, half, 40, 50, 60>(static_cast<float *>(c), static_cast<const half *>(a),
                                               static_cast<const half *>(b));
            return 0;
        case 2:
            MatmulOne<float, half, 128, 64, 128>(static_cast<float *>(c), static_cast<const half *>(a),
                                                 static_cast<const half *>(b));
            return 0;
        case 3:
            MatmulOne<float, float, 120, 50, 110>(static_cast<float *>(c), static_cast<const float *>(a),
                                                  static_cast<const float *>(b));
            return 0;
        default:
            return -1;
    }
}

int pto_ref_attn_head_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v, float *o, int s0, int s1, int d,
                          int causal, float scale)
{
    auto *qh = reinterpret_cast<const half *>(q);
    auto *kh = reinterpret_cast<const half *>(k);
    auto *vh = reinterpret_cast<const half *>(v);
    if (d == 128 && s0 == 128 && s1 == 128) {
        AttnHead<128, 128, 128>(o, qh, kh, vh, scale, causal);
    } else if (d == 128 && s0 == 128 && s1 == 512) {
        AttnHead<128, 512, 128>(o, qh, kh, vh, scale, causal);
    } else if (d == 128 && s0 == 256 && s1 == 256) {
        AttnHead<256, 256, 128>(o, qh, kh, vh, scale, causal);
    } else if (d == 128 && s0 == 512 && s1 == 512) {
        AttnHead<512, 512, 128>(o, qh, kh, vh, scale, causal);
    } else if (d == 128 && s0 == 1024 && s1 == 1024) {
        AttnHead<1024, 1024, 128>(o, qh, kh, vh, scale, causal);
    } else if (d == 64 && s0 == 128 && s1 == 256) {
        AttnHead<128, 256, 64>(o, qh, kh, vh, scale, causal);
    } else {
        return -1;
    }
    return 0;
}

int pto_ref_hardware_threads(void)
{
    return static_cast<int>(pto::cpu::get_thread_count());
}

} // extern "C"
