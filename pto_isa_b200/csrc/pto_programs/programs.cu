// Tile programs written against the PTO surface of this repository (include/pto/), in the style of the
// reference's unit-test kernels (tests/cpu/st/testcase/*/*_kernel.cpp in the reference): they exercise the
// instructions of the attention and vector path that the GEMM tile program does not - TGATHER (both forms),
// the softmax chain TROWMAX / TROWEXPANDSUB / TMULS / TEXP / TROWSUM / TROWEXPANDDIV, TCVT, TMOV between
// tensor memory, vector tiles and matrix operands, and both operand layouts of TMATMUL.
// Built into libpto_b200_programs.so; used by tests/test_pto_programs_gpu.py.
// Windows of the shared-memory arena for this translation unit: 116 KiB for Vec / Mat tiles (the attention
// program below needs 113 KiB), 32 KiB for Left tiles, the rest (73 KiB) for Right tiles.
#define PTO_B200_L0A_OFFSET (116 * 1024)
#define PTO_B200_L0B_OFFSET (148 * 1024)
#include <pto/pto-inst.hpp>

using namespace pto;

// ---------------------------------------------------------------- TGATHER, index form
template <typename T, int kSrcRows, int kSrcCols, int kDstRows, int kDstCols>
AICORE inline void ProgGatherIndex(__gm__ T *out, __gm__ T *src0, __gm__ int32_t *idx)
{
    using G0 = GlobalTensor<T, Shape<1, 1, 1, kSrcRows, kSrcCols>, Stride<1, 1, 1, kSrcCols, 1>>;
    using G1 = GlobalTensor<int32_t, Shape<1, 1, 1, kDstRows, kDstCols>, Stride<1, 1, 1, kDstCols, 1>>;
    using GD = GlobalTensor<T, Shape<1, 1, 1, kDstRows, kDstCols>, Stride<1, 1, 1, kDstCols, 1>>;
    using Src0Tile = Tile<TileType::Vec, T, kSrcRows, kSrcCols, BLayout::RowMajor, -1, -1>;
    using IdxTile = Tile<TileType::Vec, int32_t, kDstRows, kDstCols, BLayout::RowMajor, -1, -1>;
    using DstTile = Tile<TileType::Vec, T, kDstRows, kDstCols, BLayout::RowMajor, -1, -1>;
    Src0Tile s0(kSrcRows, kSrcCols);
    IdxTile it(kDstRows, kDstCols);
    DstTile dt(kDstRows, kDstCols);
    TASSIGN(s0, 0x0);
    TASSIGN(it, kSrcRows * kSrcCols * sizeof(T));
    TASSIGN(dt, kSrcRows * kSrcCols * sizeof(T) + kDstRows * kDstCols * sizeof(int32_t));
    G0 g0(src0);
    G1 g1(idx);
    GD gd(out);
    TLOAD(s0, g0);
    TLOAD(it, g1);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    TGATHER(dt, s0, it);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gd, dt);
}

// ---------------------------------------------------------------- TGATHER, mask form
template <typename T, int kRows, int kCols, MaskPattern kPattern, int kDiv>
AICORE inline void ProgGatherMask(__gm__ T *out, __gm__ T *src)
{
    using GS = GlobalTensor<T, Shape<1, 1, 1, kRows, kCols>, Stride<1, 1, 1, kCols, 1>>;
    using GD = GlobalTensor<T, Shape<1, 1, 1, kRows, kCols / kDiv>, Stride<1, 1, 1, kCols / kDiv, 1>>;
    using SrcTile = Tile<TileType::Vec, T, kRows, kCols, BLayout::RowMajor>;
    using DstTile = Tile<TileType::Vec, T, kRows, kCols / kDiv, BLayout::RowMajor>;
    SrcTile st;
    DstTile dt;
    TASSIGN(st, 0x0);
    TASSIGN(dt, kRows * kCols * sizeof(T));
    GS gs(src);
    GD gd(out);
    TLOAD(st, gs);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    TGATHER<DstTile, SrcTile, kPattern>(dt, st);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gd, dt);
}

// ---------------------------------------------------------------- row softmax of a fp32 tile
template <int kRows, int kCols>
AICORE inline void ProgRowSoftmax(__gm__ float *out, __gm__ float *rowmax_out, __gm__ float *rowsum_out,
                                  __gm__ float *in, float scale)
{
    using G = GlobalTensor<float, Shape<1, 1, 1, kRows, kCols>, Stride<1, 1, 1, kCols, 1>>;
    using GR = GlobalTensor<float, Shape<1, 1, 1, kRows, 1>, Stride<1, 1, 1, 1, kRows>, Layout::DN>;
    using X = Tile<TileType::Vec, float, kRows, kCols, BLayout::RowMajor>;
    using R = Tile<TileType::Vec, float, kRows, 1, BLayout::ColMajor>;
    X x, p;
    R mx, sm;
    TASSIGN(x, 0x0);
    TASSIGN(p, kRows * kCols * sizeof(float));
    TASSIGN(mx, 2 * kRows * kCols * sizeof(float));
    TASSIGN(sm, 2 * kRows * kCols * sizeof(float) + kRows * sizeof(float));
    G gin(in), gout(out);
    GR gmx(rowmax_out), gsm(rowsum_out);
    TLOAD(x, gin);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    TROWMAX(mx, x, p);
    TROWEXPANDSUB(p, x, mx);
    TMULS(p, p, scale);
    TEXP(p, p);
    TROWSUM(sm, p, x);
    TROWEXPANDDIV(p, p, sm);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gout, p);
    TSTORE(gmx, mx);
    TSTORE(gsm, sm);
}

// ---------------------------------------------------------------- one TMATMUL with B given k x n (Layout::ND)
template <int M, int K, int N>
AICORE inline void ProgMatmulND(__gm__ float *out, __gm__ half *a, __gm__ half *b)
{
    using GA = GlobalTensor<half, Shape<1, 1, 1, M, K>, Stride<M * K, M * K, M * K, K, 1>>;
    using GB = GlobalTensor<half, Shape<1, 1, 1, K, N>, Stride<K * N, K * N, K * N, N, 1>>;
    using GC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
    using MatA = Tile<TileType::Mat, half, M, K, BLayout::ColMajor, M, K, SLayout::RowMajor>;
    using MatB = Tile<TileType::Mat, half, K, N, BLayout::RowMajor, K, N, SLayout::ColMajor>;
    MatA am;
    MatB bm;
    TileLeft<half, M, K> al;
    TileRight<half, K, N> br;
    TileAcc<float, M, N> acc;
    TASSIGN(am, 0x0);
    TASSIGN(bm, M * K * sizeof(half));
    TASSIGN(al, 0x0);
    TASSIGN(br, 0x0);
    TASSIGN(acc, 0x0);
    GA ga(a);
    GB gb(b);
    GC gc(out);
    TLOAD(am, ga);
    TLOAD(bm, gb);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    TMOV(al, am);
    TMOV(br, bm);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    TMATMUL(acc, al, br);
    set_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    wait_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    TSTORE(gc, acc);
}

// ---------------------------------------------------------------- TMATMUL_BIAS
// The bias form of the reference's unit-test kernel (tests/cpu/st/testcase/tmatmul/tmatmul_kernel.cpp:26-98): the bias
// row is loaded into a TileType::Bias tile and added by the instruction.
template <int M, int K, int N>
AICORE inline void ProgMatmulBias(__gm__ float *out, __gm__ half *a, __gm__ half *b, __gm__ float *bias)
{
    using GA = GlobalTensor<half, Shape<1, 1, 1, M, K>, Stride<M * K, M * K, M * K, K, 1>>;
    using GB = GlobalTensor<half, Shape<1, 1, 1, K, N>, Stride<K * N, K * N, K * N, N, 1>>;
    using GBias = GlobalTensor<float, Shape<1, 1, 1, 1, N>, Stride<N, N, N, N, 1>>;
    using GC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
    using MatA = Tile<TileType::Mat, half, M, K, BLayout::ColMajor, M, K, SLayout::RowMajor>;
    using MatB = Tile<TileType::Mat, half, K, N, BLayout::RowMajor, K, N, SLayout::ColMajor>;
    using BiasTile = Tile<TileType::Bias, float, 1, N, BLayout::RowMajor, 1, N>;
    MatA am;
    MatB bm;
    TileLeft<half, M, K> al;
    TileRight<half, K, N> br;
    TileAcc<float, M, N> acc;
    BiasTile bias_tile;
    TASSIGN(am, 0x0);
    TASSIGN(bm, M * K * sizeof(half));
    TASSIGN(al, 0x0);
    TASSIGN(br, 0x0);
    TASSIGN(acc, 0x0);
    TASSIGN(bias_tile, 0x0);
    GA ga(a);
    GB gb(b);
    GBias gbias(bias);
    GC gc(out);
    TLOAD(am, ga);
    TLOAD(bm, gb);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    TMOV(al, am);
    TMOV(br, bm);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    TLOAD(bias_tile, gbias);
    TMATMUL_BIAS(acc, al, br, bias_tile);
    set_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    wait_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    TSTORE(gc, acc);
}

// ---------------------------------------------------------------- attention for one head, one key tile
// The instruction sequence of the reference's attention test (tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp:
// 84-105) with the flash-attention kernel's conventions: fp16 Q / K / V, max on the raw logits,
// p = exp(scale * (x - max)), fp32 row sum, fp16 P for the second product, division at the end.
// Q: S0 x D, K, V: S1 x D (row-major), O: S0 x D fp32.  S0 = 128, S1 = 128, D = 64.
template <int S0, int S1, int D>
AICORE inline void ProgAttentionHead(__gm__ float *o, __gm__ half *q, __gm__ half *k, __gm__ half *v, float scale)
{
    using GQ = GlobalTensor<half, Shape<1, 1, 1, S0, D>, Stride<S0 * D, S0 * D, S0 * D, D, 1>>;
    using GKT = GlobalTensor<half, Shape<1, 1, 1, D, S1>, Stride<S1 * D, S1 * D, S1 * D, 1, D>, Layout::DN>;
    using GV = GlobalTensor<half, Shape<1, 1, 1, S1, D>, Stride<S1 * D, S1 * D, S1 * D, D, 1>>;
    using GO = GlobalTensor<float, Shape<1, 1, 1, S0, D>, Stride<S0 * D, S0 * D, S0 * D, D, 1>>;
    using QMat = Tile<TileType::Mat, half, S0, D, BLayout::ColMajor, S0, D, SLayout::RowMajor>;
    using KTMat = Tile<TileType::Mat, half, D, S1, BLayout::RowMajor, D, S1, SLayout::ColMajor>;
    using VMat = Tile<TileType::Mat, half, S1, D, BLayout::RowMajor, S1, D, SLayout::ColMajor>;
    using Scores = Tile<TileType::Vec, float, S0, S1, BLayout::RowMajor>;
    using Probs = Tile<TileType::Vec, half, S0, S1, BLayout::RowMajor>;
    using RowRed = Tile<TileType::Vec, float, S0, 1, BLayout::ColMajor>;
    using OutVec = Tile<TileType::Vec, float, S0, D, BLayout::RowMajor>;

    QMat qm;
    KTMat km;
    VMat vm;
    TileLeft<half, S0, D> ql;
    TileRight<half, D, S1> kr;
    TileAcc<float, S0, S1> sacc;
    Scores x;
    Probs ph;
    RowRed mx, sm;
    TileLeft<half, S0, S1> pl;
    TileRight<half, S1, D> vr;
    TileAcc<float, S0, D> oacc;
    OutVec ov;

    // Vec / Mat window: [Q | K^T | V] staging, later reused by the fp16 P tile; [scores], later reused by O; row state
    constexpr uint32_t kQ = 0, kK = kQ + S0 * D * 2, kV = kK + D * S1 * 2, kX = kV + S1 * D * 2;
    constexpr uint32_t kP = 0, kMx = kX + S0 * S1 * 4, kSm = kMx + S0 * 4;
    static_assert(S0 * S1 * 2 <= kX, "the fp16 P tile must fit in the staging area it reuses");
    TASSIGN(qm, kQ);
    TASSIGN(km, kK);
    TASSIGN(vm, kV);
    TASSIGN(x, kX);
    TASSIGN(ph, kP);
    TASSIGN(mx, kMx);
    TASSIGN(sm, kSm);
    TASSIGN(ov, kX); // reuses the score tile's space once P has been written
    TASSIGN(ql, 0x0);
    TASSIGN(pl, 0x0);
    TASSIGN(kr, 0x0);
    TASSIGN(vr, 0x8000);
    TASSIGN(sacc, 0x0);
    TASSIGN(oacc, S1 * 512); // tensor-memory columns after the score accumulator

    GQ gq(q);
    GKT gk(k);
    GV gv(v);
    GO go(o);
    TLOAD(qm, gq);
    TLOAD(km, gk);
    TLOAD(vm, gv);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    TMOV(ql, qm);
    TMOV(kr, km);
    TMOV(vr, vm);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
    TMATMUL(sacc, ql, kr);
    set_flag(PIPE_M, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_M, PIPE_V, EVENT_ID0);
    TMOV(x, sacc);
    TROWMAX(mx, x, x);
    TROWEXPANDSUB(x, x, mx);
    TMULS(x, x, scale);
    TEXP(x, x);
    TROWSUM(sm, x, x);
    TCVT(ph, x, RoundMode::CAST_ROUND);
    TMOV(pl, ph);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID1);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID1);
    TMATMUL(oacc, pl, vr);
    set_flag(PIPE_M, PIPE_V, EVENT_ID1);
    wait_flag(PIPE_M, PIPE_V, EVENT_ID1);
    TMOV(ov, oacc);
    TROWEXPANDDIV(ov, ov, sm);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(go, ov);
}

// ---------------------------------------------------------------- the row-softmax tutorial and the second batch
// Row softmax in the decomposition of the reference's tutorial (docs/coding/tutorials/row-softmax.md:14-45):
// TROWMAX, TROWEXPAND + TSUB, TEXP, TROWSUM, TROWEXPAND + TDIV.
template <int M, int N>
AICORE inline void ProgRowSoftmaxTutorial(__gm__ float *out, __gm__ float *in)
{
    using GT = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<1, 1, 1, N, 1>>;
    using XTile = Tile<TileType::Vec, float, M, N, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    using Col1 = Tile<TileType::Vec, float, M, 1, BLayout::ColMajor, DYNAMIC, 1>;
    GT gin(in), gout(out);
    XTile x(M, N), tmp(M, N);
    Col1 row_max(M), row_sum(M);
    TASSIGN(x, 0x0);
    TASSIGN(tmp, M * N * sizeof(float));
    TASSIGN(row_max, 2 * M * N * sizeof(float));
    TASSIGN(row_sum, 2 * M * N * sizeof(float) + M * sizeof(float));
    TLOAD(x, gin);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    TROWMAX(row_max, x, tmp);
    TROWEXPAND(tmp, row_max);
    TSUB(x, x, tmp);
    TEXP(x, x);
    TROWSUM(row_sum, x, tmp);
    TROWEXPAND(tmp, row_sum);
    TDIV(x, x, tmp);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gout, x);
}

// TFILLPAD, TROWMIN, TCOLMAX / TCOLSUM / TCOLMIN, TTRANS, TCMPS + TSEL, TROWEXPAND{MAX,MIN,EXPDIF}, TROWEXPAND, TCMP
// on one 64 x 128 fp32 tile pair.  Every result goes to its own output array.
struct Vector2Out {
    float *fill, *rowmin, *colmax, *colsum, *colmin, *trans, *sel, *emax, *emin, *edif, *expand, *cmp;
    uint8_t *bits;
};

AICORE inline void ProgVector2(Vector2Out o, __gm__ float *a_in, __gm__ float *b_in, __gm__ float *s_in, int valid_rows,
                               int valid_cols)
{
    constexpr int R = 64, C = 128;
    using G = GlobalTensor<float, Shape<1, 1, 1, R, C>, Stride<1, 1, 1, C, 1>>;
    using GTr = GlobalTensor<float, Shape<1, 1, 1, C, R>, Stride<1, 1, 1, R, 1>>;
    using GCol = GlobalTensor<float, Shape<1, 1, 1, R, 1>, Stride<1, 1, 1, 1, R>, Layout::DN>;
    using GRow = GlobalTensor<float, Shape<1, 1, 1, 1, C>, Stride<1, 1, 1, C, 1>>;
    using GBits = GlobalTensor<uint8_t, Shape<1, 1, 1, R, C>, Stride<1, 1, 1, C, 1>>;
    using X = Tile<TileType::Vec, float, R, C, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    using XPad = Tile<TileType::Vec, float, R, C, BLayout::RowMajor, DYNAMIC, DYNAMIC, SLayout::NoneBox,
                      TileConfig::fractalABSize, PadValue::Max>;
    using XT = Tile<TileType::Vec, float, C, R, BLayout::RowMajor>;
    using XFull = Tile<TileType::Vec, float, R, C, BLayout::RowMajor>;
    using Col1 = Tile<TileType::Vec, float, R, 1, BLayout::ColMajor, DYNAMIC, 1>;
    using Row1 = Tile<TileType::Vec, float, 1, C, BLayout::RowMajor, 1, DYNAMIC>;
    using Bits = Tile<TileType::Vec, uint8_t, R, C, BLayout::RowMajor, DYNAMIC, DYNAMIC>;

    constexpr uint32_t kTile = R * C * sizeof(float);
    X a(R, C), b(R, C), w(R, C), part(valid_rows, valid_cols);
    XPad padded(R, C);
    XFull a_full, unused;
    XT tr;
    Col1 s(R), rmin(R);
    Row1 cred(C);
    Bits bits(R, C); // as in the reference's own test kernel the byte tile has the source's shape: the packed stream is contiguous
    TASSIGN(a, 0x0);
    TASSIGN(a_full, 0x0);
    TASSIGN(part, 0x0);
    TASSIGN(b, kTile);
    TASSIGN(w, 2 * kTile);
    TASSIGN(padded, 2 * kTile);
    TASSIGN(tr, 2 * kTile);
    TASSIGN(unused, 2 * kTile);
    TASSIGN(bits, 3 * kTile);
    TASSIGN(s, 3 * kTile + R * C);
    TASSIGN(rmin, 3 * kTile + R * C + R * sizeof(float));
    TASSIGN(cred, 3 * kTile + R * C + 2 * R * sizeof(float));

    G ga(a_in), gb(b_in);
    GCol gs(s_in);
    TLOAD(a, ga);
    TLOAD(b, gb);
    TLOAD(s, gs);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);

    auto store_w = [&](__gm__ float *dst) {
        G g(dst);
        set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        TSTORE(g, w);
        set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
        wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    };
    auto store_row = [&](__gm__ float *dst) {
        GRow g(dst);
        set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        TSTORE(g, cred);
        set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
        wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    };

    // pad everything outside the valid corner of `a` with +inf, then the row minima of the padded tile
    TFILLPAD(padded, part);
    TROWMIN(rmin, padded, unused);
    {
        G g(o.fill);
        GCol gm(o.rowmin);
        set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        TSTORE(g, padded);
        TSTORE(gm, rmin);
        set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
        wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    }
    TCOLMAX(cred, a);
    store_row(o.colmax);
    TCOLSUM(cred, a);
    store_row(o.colsum);
    TCOLMIN(cred, a);
    store_row(o.colmin);
    TTRANS(tr, a_full, unused);
    {
        GTr g(o.trans);
        set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
        TSTORE(g, tr);
        set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
        wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    }
    // relu-like selection: a where a > 0.25, else b
    TCMPS(bits, a, 0.25f, CmpMode::GT);
    TSEL(w, bits, a, b);
    store_w(o.sel);
    {
        GBits g(o.bits);
        Bits flat(R * C / 8 / C, C); // the packed stream sits at the start of the byte tile's storage
        TASSIGN(flat, 3 * kTile);
        TSTORE(g, flat);
    }
    TROWEXPANDMAX(w, a, s);
    store_w(o.emax);
    TROWEXPANDMIN(w, a, s);
    store_w(o.emin);
    TROWEXPANDEXPDIF(w, a, s);
    store_w(o.edif);
    TROWEXPAND(w, s);
    store_w(o.expand);
    TCMP(w, a, b, CmpMode::LT);
    store_w(o.cmp);
}

// ---------------------------------------------------------------- causal mask by TTRI, TRESHAPE
// The mask construction of the reference's streaming softmax (kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:
// 64-79: an upper-triangular tile of ones times the lowest float, added to the logits), a lower-triangular tile, and the
// masked tile seen as 128 x 64 by TRESHAPE with its row maxima.
AICORE inline void ProgTriReshape(__gm__ float *masked_out, __gm__ float *tril_out, __gm__ float *rowmax_out,
                                  __gm__ float *x_in, int diagonal)
{
    constexpr int R = 64, C = 128;
    using G = GlobalTensor<float, Shape<1, 1, 1, R, C>, Stride<1, 1, 1, C, 1>>;
    using GCol = GlobalTensor<float, Shape<1, 1, 1, 2 * R, 1>, Stride<1, 1, 1, 1, 2 * R>, Layout::DN>;
    using X = Tile<TileType::Vec, float, R, C, BLayout::RowMajor>;
    using XR = Tile<TileType::Vec, float, 2 * R, C / 2, BLayout::RowMajor>;
    using Col1 = Tile<TileType::Vec, float, 2 * R, 1, BLayout::ColMajor, DYNAMIC, 1>;
    constexpr uint32_t kTile = R * C * sizeof(float);
    X x, mask, w;
    XR reshaped, tmp;
    Col1 rmax(2 * R);
    TASSIGN(x, 0x0);
    TASSIGN(mask, kTile);
    TASSIGN(w, 2 * kTile);
    TASSIGN(reshaped, 3 * kTile);
    TASSIGN(tmp, kTile); // the mask tile's storage is free again when the row maxima are taken
    TASSIGN(rmax, 4 * kTile);
    G gx(x_in), gw(masked_out), gt(tril_out);
    GCol gm(rowmax_out);
    TLOAD(x, gx);
    set_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_V, EVENT_ID0);
    TTRI<X, 1>(mask, diagonal);
    TMULS(mask, mask, -3.40282e38f);
    TADD(w, x, mask);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gw, w);
    set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    TTRI<X, 0>(mask, -2);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gt, mask);
    set_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    wait_flag(PIPE_MTE3, PIPE_V, EVENT_ID0);
    TRESHAPE(reshaped, w);
    TROWMAX(rmax, reshaped, tmp);
    set_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    wait_flag(PIPE_V, PIPE_MTE3, EVENT_ID0);
    TSTORE(gm, rmax);
}

// ---------------------------------------------------------------- a multi-latent-attention head
// The instruction sequence of the reference's MLA demo (demos/cpu/mla_attention_demo/mla_attention_demo.cpp:326-376:
// latent projections, K_lat^T by TTRANS, scaled scores, row softmax, context, output projection) with fp16 matrix
// operands: every accumulator goes Acc -> Vec (fp32, TMOV) -> fp16 (TCVT) -> Left / Right (TMOV).
template <int S, int D, int R>
AICORE inline void ProgMlaHead(__gm__ float *out, __gm__ half *q, __gm__ half *k, __gm__ half *v, __gm__ half *wq,
                               __gm__ half *wk, __gm__ half *wv, __gm__ half *wo, float scale)
{
    using GSD = GlobalTensor<half, Shape<1, 1, 1, S, D>, Stride<S * D, S * D, S * D, D, 1>>;
    using GDR = GlobalTensor<half, Shape<1, 1, 1, D, R>, Stride<D * R, D * R, D * R, R, 1>>;
    using GRD = GlobalTensor<half, Shape<1, 1, 1, R, D>, Stride<R * D, R * D, R * D, D, 1>>;
    using GO = GlobalTensor<float, Shape<1, 1, 1, S, D>, Stride<S * D, S * D, S * D, D, 1>>;
    using SDh = Tile<TileType::Vec, half, S, D, BLayout::RowMajor>;
    using DRh = Tile<TileType::Vec, half, D, R, BLayout::RowMajor>;
    using RDh = Tile<TileType::Vec, half, R, D, BLayout::RowMajor>;
    using SRh = Tile<TileType::Vec, half, S, R, BLayout::RowMajor>;
    using RSh = Tile<TileType::Vec, half, R, S, BLayout::RowMajor>;
    using SRf = Tile<TileType::Vec, float, S, R, BLayout::RowMajor>;
    using SSf = Tile<TileType::Vec, float, S, S, BLayout::RowMajor>;
    using SSh = Tile<TileType::Vec, half, S, S, BLayout::RowMajor>;
    using RowRed = Tile<TileType::Vec, float, S, 1, BLayout::ColMajor>;
    static_assert(S == 128 && D == 64 && R == 64, "the arena plan below is for S 128, D 64, R 64");

    constexpr uint32_t K = 1024;
    SDh qv, kv, vv;
    DRh wqv, wkv, wvv;
    RDh wov;
    SRh qlat, klat, vlat, ctx16;
    RSh klat_t;
    SRf tmp32;
    SSf scores;
    SSh probs;
    RowRed mx, sm;
    TASSIGN(qv, 0);
    TASSIGN(kv, 16 * K);
    TASSIGN(vv, 32 * K);
    TASSIGN(wqv, 48 * K);
    TASSIGN(wkv, 56 * K);
    TASSIGN(wvv, 64 * K);
    TASSIGN(tmp32, 72 * K);   // 72..104 KiB
    TASSIGN(qlat, 0);         // over Q once it sits in the Left window
    TASSIGN(klat, 16 * K);    // over K
    TASSIGN(vlat, 32 * K);    // over V
    TASSIGN(klat_t, 48 * K);  // over Wq, Wk
    TASSIGN(scores, 48 * K);  // 48..112 KiB, over K_lat^T, Wv and the fp32 scratch, all consumed by then
    TASSIGN(probs, 0);        // 0..32 KiB, over Q_lat and K_lat
    TASSIGN(ctx16, 80 * K);
    TASSIGN(wov, 96 * K);
    TASSIGN(mx, 114 * K);
    TASSIGN(sm, 114 * K + S * 4);

    TileLeft<half, S, D> l_sd;
    TileLeft<half, S, R> l_sr;
    TileLeft<half, S, S> l_ss;
    TileRight<half, D, R> r_wq, r_wk, r_wv;
    TileRight<half, R, D> r_wo;
    TileRight<half, R, S> r_klat_t;
    TileRight<half, S, R> r_vlat;
    TileAcc<float, S, R> acc_sr;
    TileAcc<float, S, S> acc_ss;
    TileAcc<float, S, D> acc_sd;
    TASSIGN(l_sd, 0x0);
    TASSIGN(l_sr, 0x0);
    TASSIGN(l_ss, 0x0);
    TASSIGN(r_wq, 0);
    TASSIGN(r_wk, 8 * K);
    TASSIGN(r_wv, 16 * K);
    TASSIGN(r_wo, 24 * K);
    TASSIGN(r_klat_t, 32 * K);
    TASSIGN(r_vlat, 48 * K);
    TASSIGN(acc_sr, 0x0);
    TASSIGN(acc_ss, R * 512);         // tensor-memory columns after the S x R accumulator
    TASSIGN(acc_sd, (R + S) * 512);

    GSD gq(q), gk(k), gv(v);
    GDR gwq(wq), gwk(wk), gwv(wv);
    GRD gwo(wo);
    GO go(out);
    TLOAD(qv, gq);
    TLOAD(kv, gk);
    TLOAD(vv, gv);
    TLOAD(wqv, gwq);
    TLOAD(wkv, gwk);
    TLOAD(wvv, gwv);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    TMOV(r_wq, wqv);
    TMOV(r_wk, wkv);
    TMOV(r_wv, wvv);

    // latent projections (S x D) * (D x R) -> (S x R), each brought back as an fp16 Vec tile
    auto project = [&](SDh &x, TileRight<half, D, R> &w, SRh &dst, event_t ev) {
        TMOV(l_sd, x);
        set_flag(PIPE_MTE1, PIPE_M, ev);
        wait_flag(PIPE_MTE1, PIPE_M, ev);
        TMATMUL(acc_sr, l_sd, w);
        set_flag(PIPE_M, PIPE_V, ev);
        wait_flag(PIPE_M, PIPE_V, ev);
        TMOV(tmp32, acc_sr);
        TCVT(dst, tmp32, RoundMode::CAST_RINT);
    };
    project(qv, r_wq, qlat, EVENT_ID0);
    project(kv, r_wk, klat, EVENT_ID1);
    project(vv, r_wv, vlat, EVENT_ID2);

    // scores = Q_lat * K_lat^T, the transpose made by TTRANS
    TTRANS(klat_t, klat, klat);
    TMOV(r_klat_t, klat_t);
    TMOV(r_vlat, vlat);
    TMOV(l_sr, qlat);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID3);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID3);
    TMATMUL(acc_ss, l_sr, r_klat_t);
    set_flag(PIPE_M, PIPE_V, EVENT_ID3);
    wait_flag(PIPE_M, PIPE_V, EVENT_ID3);
    TMOV(scores, acc_ss);
    TMULS(scores, scores, scale);

    // row softmax
    TROWMAX(mx, scores, scores);
    TROWEXPANDSUB(scores, scores, mx);
    TEXP(scores, scores);
    TROWSUM(sm, scores, scores);
    TROWEXPANDDIV(scores, scores, sm);
    TCVT(probs, scores, RoundMode::CAST_RINT);

    // context = P * V_lat, output = context * Wo
    TMOV(l_ss, probs);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID4);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID4);
    TMATMUL(acc_sr, l_ss, r_vlat);
    set_flag(PIPE_M, PIPE_V, EVENT_ID4);
    wait_flag(PIPE_M, PIPE_V, EVENT_ID4);
    SRf ctx32;
    TASSIGN(ctx32, 48 * K); // the score tile is dead
    TMOV(ctx32, acc_sr);
    TCVT(ctx16, ctx32, RoundMode::CAST_RINT);
    TLOAD(wov, gwo);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID1);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID1);
    TMOV(r_wo, wov);
    TMOV(l_sr, ctx16);
    set_flag(PIPE_MTE1, PIPE_M, EVENT_ID5);
    wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID5);
    TMATMUL(acc_sd, l_sr, r_wo);
    set_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    wait_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    TSTORE(go, acc_sd);
}

// ---------------------------------------------------------------- MX block-scaled product, two k blocks
// The instruction sequence of the reference's MX kernels (kernels/manual/a5/matmul_mxfp8_performance/
// mxmatmul_performance_kernel.cpp:24-36,120-150: TLOAD of the data and scale tiles, TEXTRACT of the current k block of
// each, TMATMUL_MX for the first block and its accumulating form for the others, TSTORE with conversion to bfloat16).
// A [M x K] fp8, B stored [N x K] fp8 (the DN view), scale A [M x K/32], scale B stored [N x K/32], e8m0.
template <typename U, int M, int K, int N, int kBaseK>
AICORE inline void ProgMxMatmul(__gm__ bfloat16_t *out, __gm__ U *a, __gm__ U *b, __gm__ float8_e8m0_t *sa,
                                __gm__ float8_e8m0_t *sb)
{
    constexpr int S = K / 32, kBaseS = kBaseK / 32;
    using GA = GlobalTensor<U, Shape<1, 1, 1, M, K>, Stride<1, 1, 1, K, 1>>;
    using GB = GlobalTensor<U, Shape<1, 1, 1, K, N>, Stride<1, 1, 1, 1, K>, Layout::DN>;
    using GSA = GlobalTensor<float8_e8m0_t, Shape<1, 1, 1, M, S>, Stride<1, 1, 1, S, 1>>;
    using GSB = GlobalTensor<float8_e8m0_t, Shape<1, 1, 1, S, N>, Stride<1, 1, 1, 1, S>, Layout::DN>;
    using GC = GlobalTensor<bfloat16_t, Shape<1, 1, 1, M, N>, Stride<1, 1, 1, N, 1>>;
    using MatA = Tile<TileType::Mat, U, M, K, BLayout::ColMajor, M, K, SLayout::RowMajor>;
    using MatB = Tile<TileType::Mat, U, K, N, BLayout::RowMajor, K, N, SLayout::ColMajor>;
    using MatSA = Tile<TileType::Mat, float8_e8m0_t, M, S, BLayout::RowMajor, M, S, SLayout::RowMajor, 32>;
    using MatSB = Tile<TileType::Mat, float8_e8m0_t, S, N, BLayout::ColMajor, S, N, SLayout::ColMajor, 32>;
    MatA am;
    MatB bm;
    MatSA sam;
    MatSB sbm;
    TileLeft<U, M, kBaseK> al;
    TileRight<U, kBaseK, N> br;
    TileLeftScale<float8_e8m0_t, M, kBaseS> sal;
    TileRightScale<float8_e8m0_t, kBaseS, N> sbr;
    TileAcc<float, M, N> acc;
    TASSIGN(am, 0x0);
    TASSIGN(bm, M * K);
    TASSIGN(sam, M * K + K * N);
    TASSIGN(sbm, M * K + K * N + ((M * S + 1023) & ~1023));
    TASSIGN(al, 0x0);
    TASSIGN(br, 0x0);
    TASSIGN(sal, 0x0);
    TASSIGN(sbr, 0x0);
    TASSIGN(acc, 0x0);
    GA ga(a);
    GB gb(b);
    GSA gsa(sa);
    GSB gsb(sb);
    TLOAD(am, ga);
    TLOAD(bm, gb);
    TLOAD(sam, gsa);
    TLOAD(sbm, gsb);
    set_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    wait_flag(PIPE_MTE2, PIPE_MTE1, EVENT_ID0);
    for (int kb = 0; kb < K / kBaseK; ++kb) {
        if (kb > 0) {
            wait_flag(PIPE_M, PIPE_MTE1, EVENT_ID0); // the previous product has read the operand tiles
        }
        TEXTRACT(al, am, 0, kb * kBaseK);
        TEXTRACT(br, bm, kb * kBaseK, 0);
        TEXTRACT(sal, sam, 0, kb * kBaseS);
        TEXTRACT(sbr, sbm, kb * kBaseS, 0);
        set_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
        wait_flag(PIPE_MTE1, PIPE_M, EVENT_ID0);
        if (kb == 0) {
            TMATMUL_MX(acc, al, sal, br, sbr);
        } else {
            TMATMUL_MX(acc, acc, al, sal, br, sbr);
        }
        if (kb + 1 < K / kBaseK) {
            set_flag(PIPE_M, PIPE_MTE1, EVENT_ID0);
        }
    }
    set_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    wait_flag(PIPE_M, PIPE_FIX, EVENT_ID0);
    GC gc(out);
    TSTORE(gc, acc);
}

// ---------------------------------------------------------------- host entry points
#pragma GCC visibility push(default)
extern "C" {

int pto_prog_tgather_index_f32(float *out, const float *src0, const int32_t *idx, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgGatherIndex<float, 32, 1024, 16, 64>(out, const_cast<float *>(src0), const_cast<int32_t *>(idx));
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_tgather_index_b16(int16_t *out, const int16_t *src0, const int32_t *idx, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgGatherIndex<int16_t, 16, 1024, 16, 128>(out, const_cast<int16_t *>(src0),
                                                           const_cast<int32_t *>(idx));
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_tgather_mask_f32(float *out, const float *src, int pattern, void *stream)
{
    float *s = const_cast<float *>(src);
    cudaError_t e;
    switch (pattern) {
        case 1: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P0101, 2>(out, s); }); break;
        case 2: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P1010, 2>(out, s); }); break;
        case 3: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P0001, 4>(out, s); }); break;
        case 4: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P0010, 4>(out, s); }); break;
        case 5: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P0100, 4>(out, s); }); break;
        case 6: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P1000, 4>(out, s); }); break;
        case 7: e = pto::b200::launch(1, stream, [=] __device__() { ProgGatherMask<float, 64, 256, MaskPattern::P1111, 1>(out, s); }); break;
        default: return 1;
    }
    return e == cudaSuccess ? 0 : 3;
}

int pto_prog_row_softmax_64x256(float *out, float *rowmax, float *rowsum, const float *in, float scale, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgRowSoftmax<64, 256>(out, rowmax, rowsum, const_cast<float *>(in), scale);
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_matmul_nd_128x128x256(float *out, const __half *a, const __half *b, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgMatmulND<128, 128, 256>(out, const_cast<__half *>(a), const_cast<__half *>(b));
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_attention_head_128x128x64(float *o, const __half *q, const __half *k, const __half *v, float scale,
                                       void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgAttentionHead<128, 128, 64>(o, const_cast<__half *>(q), const_cast<__half *>(k),
                                               const_cast<__half *>(v), scale);
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_row_softmax_tutorial_64x256(float *out, const float *in, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgRowSoftmaxTutorial<64, 256>(out, const_cast<float *>(in));
           }) == cudaSuccess
               ? 0
               : 3;
}

// outs: 13 device pointers in the order of Vector2Out (the last one the packed comparison bits)
int pto_prog_vector2_64x128(void *const *outs, const float *a, const float *b, const float *s, int valid_rows,
                            int valid_cols, void *stream)
{
    Vector2Out o;
    float **f = reinterpret_cast<float **>(&o);
    for (int i = 0; i < 12; ++i) {
        f[i] = static_cast<float *>(outs[i]);
    }
    o.bits = static_cast<uint8_t *>(outs[12]);
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgVector2(o, const_cast<float *>(a), const_cast<float *>(b), const_cast<float *>(s), valid_rows,
                           valid_cols);
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_tmatmul_bias_128x64x256(float *out, const __half *a, const __half *b, const float *bias, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgMatmulBias<128, 64, 256>(out, const_cast<__half *>(a), const_cast<__half *>(b),
                                            const_cast<float *>(bias));
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_tri_reshape_64x128(float *masked, float *tril, float *rowmax, const float *x, int diagonal, void *stream)
{
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgTriReshape(masked, tril, rowmax, const_cast<float *>(x), diagonal);
           }) == cudaSuccess
               ? 0
               : 3;
}

int pto_prog_mla_head_128x64x64(float *out, const __half *q, const __half *k, const __half *v, const __half *wq,
                                const __half *wk, const __half *wv, const __half *wo, float scale, void *stream)
{
    auto c = [](const __half *p) { return const_cast<__half *>(p); };
    __half *q_ = c(q), *k_ = c(k), *v_ = c(v), *wq_ = c(wq), *wk_ = c(wk), *wv_ = c(wv), *wo_ = c(wo);
    return pto::b200::launch(1, stream, [=] __device__() {
               ProgMlaHead<128, 64, 64>(out, q_, k_, v_, wq_, wk_, wv_, wo_, scale);
           }) == cudaSuccess
               ? 0
               : 3;
}

// TMATMUL_MX: C[128 x 256] bf16 = (sa (x) A[128 x 256]) (sb (x) B[256 x 256])^T; fmt 0 = e4m3, 1 = e5m2; two k blocks of 128
int pto_prog_mx_matmul_128x256x256(void *out, const void *a, const void *b, const void *sa, const void *sb, int fmt,
                                   void *stream, int *status_dev)
{
    pto::b200::LaunchOptions opt;
    opt.status = status_dev;
    // matrix and scale tiles: 32 + 64 + 1 + 2 KiB; Left 16 KiB, Right 32 KiB
    opt.l0a_offset = 116 * 1024;
    opt.l0b_offset = 148 * 1024;
    bfloat16_t *o = static_cast<bfloat16_t *>(out);
    float8_e8m0_t *sa_ = static_cast<float8_e8m0_t *>(const_cast<void *>(sa));
    float8_e8m0_t *sb_ = static_cast<float8_e8m0_t *>(const_cast<void *>(sb));
    cudaError_t e;
    if (fmt == 1) {
        float8_e5m2_t *a_ = static_cast<float8_e5m2_t *>(const_cast<void *>(a));
        float8_e5m2_t *b_ = static_cast<float8_e5m2_t *>(const_cast<void *>(b));
        e = pto::b200::launch(1, stream, [=] __device__() { ProgMxMatmul<float8_e5m2_t, 128, 256, 256, 128>(o, a_, b_, sa_, sb_); }, opt);
    } else {
        float8_e4m3_t *a_ = static_cast<float8_e4m3_t *>(const_cast<void *>(a));
        float8_e4m3_t *b_ = static_cast<float8_e4m3_t *>(const_cast<void *>(b));
        e = pto::b200::launch(1, stream, [=] __device__() { ProgMxMatmul<float8_e4m3_t, 128, 256, 256, 128>(o, a_, b_, sa_, sb_); }, opt);
    }
    return e == cudaSuccess ? 0 : 3;
}

} // extern "C"
#pragma GCC visibility pop
