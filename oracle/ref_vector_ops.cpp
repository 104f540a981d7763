// TEST INFRASTRUCTURE ONLY.  Wrappers that run the reference's own CPU-simulation implementations of the row-expand
// family, TROWMIN, the column reductions, TFILLPAD, TTRANS, TSEL, TCMP and TCMPS on tiles, compiled against the
// reference headers where they lie (see Makefile).  They exist to pin oracle/pto_oracle.c; nothing in the product
// links or calls them.  Tile programs follow the reference's own test kernels (tests/cpu/st/testcase/<op>/*_kernel.cpp):
// TLOAD-free here, the operands are written into plain row-major tiles directly.
#include <pto/pto-inst.hpp>

#include <cstdint>
#include <cstring>
#include <memory>

using namespace pto;

namespace {

constexpr int kR = 64;   // tile rows
constexpr int kC = 256;  // tile columns (row pitch of every 2-D operand handed in)

using MatTile = Tile<TileType::Vec, float, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
using ColTile = Tile<TileType::Vec, float, kR, 1, BLayout::ColMajor, DYNAMIC, 1>;
using RowTile = Tile<TileType::Vec, float, 1, kC, BLayout::RowMajor, 1, DYNAMIC>;

bool fits(int rows, int cols)
{
    return rows >= 0 && rows <= kR && cols >= 0 && cols <= kC;
}

// dense rows x cols array <-> the valid corner of a kR x kC tile
void fill(MatTile &t, const float *src, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            t.data()[r * kC + c] = src[static_cast<int64_t>(r) * cols + c];
        }
    }
}
void drain(float *dst, MatTile &t, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            dst[static_cast<int64_t>(r) * cols + c] = t.data()[r * kC + c];
        }
    }
}

} // namespace

extern "C" {

// op codes of include/pto_b200.h: 0 add, 1 sub, 2 mul, 3 div, 4 max, 5 min, 6 expdif, 7 plain expand
int pto_ref_trowexpand_f32(const float *a, const float *s, float *dst, int rows, int cols, int op)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0) {
        return -1;
    }
    auto x = std::make_unique<MatTile>(rows, cols);
    auto y = std::make_unique<MatTile>(rows, cols);
    ColTile sc(static_cast<size_t>(rows));
    if (op != 7) {
        fill(*x, a, rows, cols);
    }
    for (int r = 0; r < rows; ++r) {
        sc.data()[r] = s[r];
    }
    switch (op) {
        case 0: TROWEXPANDADD(*y, *x, sc); break;
        case 1: TROWEXPANDSUB(*y, *x, sc); break;
        case 2: TROWEXPANDMUL(*y, *x, sc); break;
        case 3: TROWEXPANDDIV(*y, *x, sc); break;
        case 4: TROWEXPANDMAX(*y, *x, sc); break;
        case 5: TROWEXPANDMIN(*y, *x, sc); break;
        case 6: TROWEXPANDEXPDIF(*y, *x, sc); break;
        case 7: TROWEXPAND(*y, sc); break;
        default: return -1;
    }
    drain(dst, *y, rows, cols);
    return 0;
}

int pto_ref_trowmin_f32(const float *src, float *dst, int rows, int cols)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0) {
        return -1;
    }
    auto x = std::make_unique<MatTile>(rows, cols);
    ColTile d(static_cast<size_t>(rows));
    fill(*x, src, rows, cols);
    TROWMIN(d, *x, *x);
    for (int r = 0; r < rows; ++r) {
        dst[r] = d.data()[r];
    }
    return 0;
}

// op: 0 sum, 4 max, 5 min
int pto_ref_tcolreduce_f32(const float *src, float *dst, int rows, int cols, int op)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0) {
        return -1;
    }
    auto x = std::make_unique<MatTile>(rows, cols);
    RowTile d(static_cast<size_t>(cols));
    fill(*x, src, rows, cols);
    switch (op) {
        case 0: TCOLSUM(d, *x); break;
        case 4: TCOLMAX(d, *x); break;
        case 5: TCOLMIN(d, *x); break;
        default: return -1;
    }
    for (int c = 0; c < cols; ++c) {
        dst[c] = d.data()[c];
    }
    return 0;
}

// pad_kind: 1 zero, 2 max, 3 min (PadValue); src and dst are dense kR x kC here (the instruction works on whole tiles)
int pto_ref_tfillpad_f32(const float *src, float *dst, int valid_rows, int valid_cols, int pad_kind)
{
    if (!fits(valid_rows, valid_cols) || valid_rows == 0 || valid_cols == 0) {
        return -1;
    }
    auto x = std::make_unique<MatTile>(valid_rows, valid_cols);
    std::memcpy(x->data(), src, sizeof(float) * kR * kC);
    auto run = [&](auto &y) {
        TFILLPAD(y, *x);
        std::memcpy(dst, y.data(), sizeof(float) * kR * kC);
    };
    using Common = Tile<TileType::Vec, float, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC, SLayout::NoneBox,
                        TileConfig::fractalABSize, PadValue::Zero>;
    (void)sizeof(Common);
    if (pad_kind == 1) {
        auto y = std::make_unique<Tile<TileType::Vec, float, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC, SLayout::NoneBox,
                                       TileConfig::fractalABSize, PadValue::Zero>>(kR, kC);
        run(*y);
    } else if (pad_kind == 2) {
        auto y = std::make_unique<Tile<TileType::Vec, float, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC, SLayout::NoneBox,
                                       TileConfig::fractalABSize, PadValue::Max>>(kR, kC);
        run(*y);
    } else if (pad_kind == 3) {
        auto y = std::make_unique<Tile<TileType::Vec, float, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC, SLayout::NoneBox,
                                       TileConfig::fractalABSize, PadValue::Min>>(kR, kC);
        run(*y);
    } else {
        return -1;
    }
    return 0;
}

// src 64 x 128, dst 128 x 64, both dense (static valid extents: the instruction asserts them equal)
int pto_ref_ttrans_f32_64x128(const float *src, float *dst)
{
    using S = Tile<TileType::Vec, float, 64, 128, BLayout::RowMajor>;
    using D = Tile<TileType::Vec, float, 128, 64, BLayout::RowMajor>;
    auto s = std::make_unique<S>();
    auto d = std::make_unique<D>();
    std::memcpy(s->data(), src, sizeof(float) * 64 * 128);
    TTRANS(*d, *s, *s);
    std::memcpy(dst, d->data(), sizeof(float) * 64 * 128);
    return 0;
}

// mask: rows * cols / 8 bytes, flat
int pto_ref_tsel_f32(const uint8_t *mask, const float *a, const float *b, float *dst, int rows, int cols)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0 || cols != kC) {
        return -1; // a dense operand (cols == tile width) keeps the mask a flat bit array
    }
    using MaskTile = Tile<TileType::Vec, uint8_t, kR, kC / 8, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    auto x = std::make_unique<MatTile>(rows, cols);
    auto y = std::make_unique<MatTile>(rows, cols);
    auto z = std::make_unique<MatTile>(rows, cols);
    auto m = std::make_unique<MaskTile>(rows, cols / 8);
    fill(*x, a, rows, cols);
    fill(*y, b, rows, cols);
    std::memcpy(m->data(), mask, static_cast<size_t>(rows) * cols / 8);
    TSEL(*z, *m, *x, *y);
    drain(dst, *z, rows, cols);
    return 0;
}

// dense kR x kC source; dst: kR * kC / 8 bytes.  As in the reference's own test kernel
// (tests/cpu/st/testcase/tcmps/tcmps_kernel.cpp:24-35) the result tile is a byte tile of the source's shape; the
// simulation fills it row by row from the packed stream, so the stream sits contiguously at its start.
int pto_ref_tcmps_f32(const float *src, float scalar, uint8_t *dst, int mode)
{
    using BitTile = Tile<TileType::Vec, uint8_t, kR, kC, BLayout::RowMajor, DYNAMIC, DYNAMIC>;
    auto x = std::make_unique<MatTile>(kR, kC);
    auto d = std::make_unique<BitTile>(kR, kC);
    std::memcpy(x->data(), src, sizeof(float) * kR * kC);
    std::memset(d->data(), 0, kR * kC);
    TCMPS(*d, *x, scalar, static_cast<CmpMode>(mode));
    std::memcpy(dst, d->data(), kR * kC / 8);
    return 0;
}

int pto_ref_tcmp_f32(const float *a, const float *b, float *dst, int rows, int cols, int mode)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0) {
        return -1;
    }
    auto x = std::make_unique<MatTile>(rows, cols);
    auto y = std::make_unique<MatTile>(rows, cols);
    auto z = std::make_unique<MatTile>(rows, cols);
    fill(*x, a, rows, cols);
    fill(*y, b, rows, cols);
    TCMP(*z, *x, *y, static_cast<CmpMode>(mode));
    drain(dst, *z, rows, cols);
    return 0;
}

// TTRI on a rows x cols valid corner of the 64 x 256 float tile (tests/cpu/st/testcase/ttri/ttri_kernel.cpp pattern)
int pto_ref_ttri_f32(float *dst, int rows, int cols, int diagonal, int upper)
{
    if (!fits(rows, cols) || rows == 0 || cols == 0) {
        return -1;
    }
    auto z = std::make_unique<MatTile>(rows, cols);
    if (upper) {
        TTRI<MatTile, 1>(*z, diagonal);
    } else {
        TTRI<MatTile, 0>(*z, diagonal);
    }
    drain(dst, *z, rows, cols);
    return 0;
}

} // extern "C"
