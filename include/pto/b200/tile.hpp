// Tile and global-tensor descriptors of the PTO surface for the B200 backend.
// Template parameter lists and member names are those of the reference's descriptors
// (include/pto/common/pto_tile.hpp:26-442 Shape / Stride / GlobalTensor, :452-616 TileShape2D / BaseShape2D,
// :1201-1410 Tile, :1422-1459 TileLeft / TileRight / TileAcc; paths relative to the reference root).
// What differs is what a tile *is*: here it is a small value-type handle -
//   Vec / Mat / Left / Right : a byte offset into the block's shared-memory arena (bound by TASSIGN), plus, for
//               the matrix tiles, how the data lies there (block pitch, which dimension is contiguous),
//   Acc       : a column offset in tensor memory -
// so passing a tile by value copies the handle, as on the NPU, never the data.
#pragma once

#include "types.hpp"

namespace pto {

// ---------------------------------------------------------------- Shape / Stride (five dimensions, any of them dynamic)
namespace b200 {
template <int64_t... S>
struct DynCount {
    static constexpr int value = ((S == DYNAMIC ? 1 : 0) + ...);
};
} // namespace b200

template <int64_t N1 = DYNAMIC, int64_t N2 = DYNAMIC, int64_t N3 = DYNAMIC, int64_t N4 = DYNAMIC, int64_t N5 = DYNAMIC>
struct Shape {
    static constexpr int64_t staticShape[5] = {N1, N2, N3, N4, N5};
    // (device code cannot index a static constexpr array at run time)
    PTO_INTERNAL static constexpr int64_t static_at(int i) { return i == 0 ? N1 : i == 1 ? N2 : i == 2 ? N3 : i == 3 ? N4 : N5; }
    int64_t shape[5] = {N1 == DYNAMIC ? 1 : N1, N2 == DYNAMIC ? 1 : N2, N3 == DYNAMIC ? 1 : N3, N4 == DYNAMIC ? 1 : N4,
                        N5 == DYNAMIC ? 1 : N5};

    PTO_INTERNAL Shape() {}
    PTO_INTERNAL Shape(int64_t a, int64_t b, int64_t c, int64_t d, int64_t e)
    {
        const int64_t v[5] = {a, b, c, d, e};
        for (int i = 0; i < 5; ++i) {
            if (static_at(i) == DYNAMIC) {
                shape[i] = v[i];
            }
        }
    }
    // n values fill the n dynamic dimensions in order
    template <typename... Ts, std::enable_if_t<(sizeof...(Ts) >= 1 && sizeof...(Ts) <= 4), int> = 0>
    PTO_INTERNAL explicit Shape(Ts... vals)
    {
        static_assert(sizeof...(Ts) == b200::DynCount<N1, N2, N3, N4, N5>::value,
                      "the number of constructor arguments must equal the number of dynamic dimensions");
        const int64_t v[sizeof...(Ts)] = {static_cast<int64_t>(vals)...};
        int k = 0;
        for (int i = 0; i < 5; ++i) {
            if (static_at(i) == DYNAMIC) {
                shape[i] = v[k++];
            }
        }
    }
};

template <int64_t N1 = DYNAMIC, int64_t N2 = DYNAMIC, int64_t N3 = DYNAMIC, int64_t N4 = DYNAMIC, int64_t N5 = DYNAMIC>
struct Stride {
    static constexpr int64_t staticStride[5] = {N1, N2, N3, N4, N5};
    PTO_INTERNAL static constexpr int64_t static_at(int i) { return i == 0 ? N1 : i == 1 ? N2 : i == 2 ? N3 : i == 3 ? N4 : N5; }
    int64_t stride[5] = {N1 == DYNAMIC ? 1 : N1, N2 == DYNAMIC ? 1 : N2, N3 == DYNAMIC ? 1 : N3,
                         N4 == DYNAMIC ? 1 : N4, N5 == DYNAMIC ? 1 : N5};

    PTO_INTERNAL Stride() {}
    PTO_INTERNAL Stride(int64_t a, int64_t b, int64_t c, int64_t d, int64_t e)
    {
        const int64_t v[5] = {a, b, c, d, e};
        for (int i = 0; i < 5; ++i) {
            if (static_at(i) == DYNAMIC) {
                stride[i] = v[i];
            }
        }
    }
    template <typename... Ts, std::enable_if_t<(sizeof...(Ts) >= 1 && sizeof...(Ts) <= 4), int> = 0>
    PTO_INTERNAL explicit Stride(Ts... vals)
    {
        static_assert(sizeof...(Ts) == b200::DynCount<N1, N2, N3, N4, N5>::value,
                      "the number of constructor arguments must equal the number of dynamic dimensions");
        const int64_t v[sizeof...(Ts)] = {static_cast<int64_t>(vals)...};
        int k = 0;
        for (int i = 0; i < 5; ++i) {
            if (static_at(i) == DYNAMIC) {
                stride[i] = v[k++];
            }
        }
    }
};

// ---------------------------------------------------------------- 2-D conveniences
template <typename T, int64_t rows = DYNAMIC, int64_t cols = DYNAMIC, Layout L = Layout::ND>
struct TileShape2D : public Shape<1, 1, 1, rows, cols> {
    static_assert(L == Layout::ND || L == Layout::DN, "this backend loads from ND and DN global tensors");
    using Parent = Shape<1, 1, 1, rows, cols>;
    PTO_INTERNAL TileShape2D() : Parent() {}
    PTO_INTERNAL TileShape2D(int64_t r, int64_t c) : Parent(1, 1, 1, r, c) {}
};

namespace b200 {
constexpr int64_t mul_or_dyn(int64_t a, int64_t b)
{
    return (a == DYNAMIC || b == DYNAMIC) ? DYNAMIC : a * b;
}
} // namespace b200

template <typename T, int64_t rows = DYNAMIC, int64_t cols = DYNAMIC, Layout L = Layout::ND>
struct BaseShape2D;

// row-major parent matrix: element (r, c) at r * cols + c
template <typename T, int64_t rows, int64_t cols>
struct BaseShape2D<T, rows, cols, Layout::ND>
    : public Stride<b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), cols, 1> {
    using Parent =
        Stride<b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), cols, 1>;
    PTO_INTERNAL BaseShape2D() : Parent() {}
    PTO_INTERNAL BaseShape2D(int64_t r, int64_t c) : Parent(r * c, r * c, r * c, c, 1) {}
};

// column-major parent matrix: element (r, c) at r + c * rows
template <typename T, int64_t rows, int64_t cols>
struct BaseShape2D<T, rows, cols, Layout::DN>
    : public Stride<b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), 1, rows> {
    using Parent =
        Stride<b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), b200::mul_or_dyn(rows, cols), 1, rows>;
    PTO_INTERNAL BaseShape2D() : Parent() {}
    PTO_INTERNAL BaseShape2D(int64_t r, int64_t c) : Parent(r * c, r * c, r * c, 1, r) {}
};

// ---------------------------------------------------------------- GlobalTensor
template <typename Element_, typename Shape_, typename Stride_, Layout Layout_ = Layout::ND>
struct GlobalTensor {
    using Shape = Shape_;
    using Stride = Stride_;
    using RawDType = Element_;
    using DType = Element_;
    static constexpr Layout layout = Layout_;
    static constexpr int64_t staticShape[5] = {Shape::staticShape[0], Shape::staticShape[1], Shape::staticShape[2],
                                               Shape::staticShape[3], Shape::staticShape[4]};
    static constexpr int64_t staticStride[5] = {Stride::staticStride[0], Stride::staticStride[1],
                                                Stride::staticStride[2], Stride::staticStride[3],
                                                Stride::staticStride[4]};

    PTO_INTERNAL GlobalTensor() : data_(nullptr) {}
    PTO_INTERNAL GlobalTensor(DType *data) : data_(data) {}
    PTO_INTERNAL GlobalTensor(DType *data, const Shape &shape) : data_(data), shape_(shape) {}
    PTO_INTERNAL GlobalTensor(DType *data, const Shape &shape, const Stride &stride)
        : data_(data), shape_(shape), stride_(stride)
    {}

    PTO_INTERNAL int64_t GetShape(const int dim) const { return shape_.shape[dim]; }
    PTO_INTERNAL int64_t GetStride(const int dim) const { return stride_.stride[dim]; }
    template <int dim>
    PTO_INTERNAL static constexpr int64_t GetShape()
    {
        static_assert(staticShape[dim] != DYNAMIC, "this dimension is dynamic");
        return staticShape[dim];
    }
    template <int dim>
    PTO_INTERNAL static constexpr int64_t GetStride()
    {
        static_assert(staticStride[dim] != DYNAMIC, "this stride is dynamic");
        return staticStride[dim];
    }
    PTO_INTERNAL DType *data() const { return data_; }
    PTO_INTERNAL void SetAddr(DType *p) { data_ = p; }

private:
    DType *data_;
    Shape shape_;
    Stride stride_;
};

// ---------------------------------------------------------------- Tile
namespace b200 {
// how a staged Mat tile lies in shared memory (decided by TLOAD from the global tensor's contiguous dimension)
// kPlain: 8- and 32-bit matrix tiles, stored row-major Rows x Cols without swizzle (not read by the tensor core)
enum : uint8_t { kColsContiguous = 0, kRowsContiguous = 1, kPlain = 2 };
// bit of major_ on a Left / Right tile that is a view of a staged Mat tile: its address counts from the start of the
// arena, not from the operand window (TEXTRACT with LaunchOptions::extract_views)
enum : uint8_t { kView = 0x80 };

// A tile is constructed with storage of its own, as in the reference's CPU simulation where every tile object owns an
// array (include/pto/common/pto_tile.hpp, the `data_` member under __CPU_SIM): the constructor takes the next free
// stretch of its location's window (Vec and Mat tiles share one, Left, Right and Acc have their own) from a bump
// allocator of the block, and TASSIGN replaces that address as on the NPU.  Programs that assign every tile never
// see the difference; programs written for the simulation alone, which assign none, get distinct tiles.  Storage is
// not handed back: once a window is used up, further tiles are placed at its start (and must be assigned before use).
enum : int { kSpaceVec = 0, kSpaceLeft = 1, kSpaceRight = 2, kSpaceAcc = 3, kSpaceNone = 4 };
#if PTO_B200_DEVICE_CODE
__device__ __forceinline__ uint32_t tile_auto_place(int space, uint32_t amount);
#endif
constexpr int tile_space(TileType loc)
{
    return (loc == TileType::Vec || loc == TileType::Mat)
               ? kSpaceVec
               : (loc == TileType::Left ? kSpaceLeft
                                        : (loc == TileType::Right ? kSpaceRight : (loc == TileType::Acc ? kSpaceAcc : kSpaceNone)));
}
} // namespace b200

namespace b200 {
// the valid extents of a tile are members only where they are dynamic: a tile handle stays three words otherwise
// (arrays of handles indexed at run time live in local memory)
template <bool kDynamic, int kStatic>
struct RowMaskMember {
    static constexpr int RowMaskInternal = kStatic;
};
template <int kStatic>
struct RowMaskMember<true, kStatic> {
    int RowMaskInternal = 0;
};
template <bool kDynamic, int kStatic>
struct ColMaskMember {
    static constexpr int ColMaskInternal = kStatic;
};
template <int kStatic>
struct ColMaskMember<true, kStatic> {
    int ColMaskInternal = 0;
};
} // namespace b200

template <TileType Loc_, typename Element_, const int Rows_, const int Cols_,
          const BLayout BFractal_ = BLayout::RowMajor, const int RowValid_ = Rows_, const int ColValid_ = Cols_,
          const SLayout SFractal_ = SLayout::NoneBox, const int SFractalSize_ = TileConfig::fractalABSize,
          const PadValue PadVal_ = PadValue::Null, const CompactMode Compact_ = CompactMode::Null>
struct Tile : public b200::RowMaskMember<RowValid_ == DYNAMIC, RowValid_>, public b200::ColMaskMember<ColValid_ == DYNAMIC, ColValid_> {
    using DType = Element_;
    using TileDType = DType *;

    static constexpr TileType Loc = Loc_;
    static constexpr int Rows = Rows_;
    static constexpr int Cols = Cols_;
    static constexpr int RowStride = BFractal_ == BLayout::RowMajor ? Cols : 1;
    static constexpr int ColStride = BFractal_ == BLayout::RowMajor ? 1 : Rows;
    static constexpr int ValidRow = RowValid_;
    static constexpr int ValidCol = ColValid_;
    static constexpr BLayout BFractal = BFractal_;
    static constexpr SLayout SFractal = SFractal_;
    static constexpr int Numel = Rows * Cols;
    static constexpr bool isRowMajor = BFractal_ == BLayout::RowMajor;
    static constexpr int SFractalSize = SFractalSize_;
    static constexpr PadValue PadVal = PadVal_;
    static constexpr CompactMode Compact = Compact_;
    static constexpr bool isBoxedLayout = (SFractal != SLayout::NoneBox);
    static constexpr bool isInnerRowMajor = (SFractal == SLayout::RowMajor);
    static constexpr bool isInnerColMajor = (SFractal == SLayout::ColMajor);
    static constexpr int InnerRows =
        SFractalSize_ == TileConfig::fractalCSize
            ? TileConfig::fixedRowSize
            : (isBoxedLayout ? (isInnerRowMajor ? TileConfig::fixedRowSize : TileConfig::alignedSize / (int)sizeof(DType)) : 1);
    static constexpr int InnerCols =
        SFractalSize_ == TileConfig::fractalCSize
            ? TileConfig::fixedColSize
            : (isBoxedLayout ? (isInnerRowMajor ? TileConfig::alignedSize / (int)sizeof(DType) : TileConfig::fixedColSize) : 1);
    static constexpr int InnerNumel = InnerRows * InnerCols;

    static_assert(Rows > 0 && Cols > 0 && ValidRow <= Rows && ValidCol <= Cols, "invalid tile shape");

    PTO_INTERNAL Tile() { place(); }
    template <int RM = ValidRow, int CM = ValidCol>
    PTO_INTERNAL Tile(std::enable_if_t<RM == DYNAMIC && CM == DYNAMIC, size_t> vr,
                      std::enable_if_t<RM == DYNAMIC && CM == DYNAMIC, size_t> vc)
    {
        this->RowMaskInternal = static_cast<int>(vr);
        this->ColMaskInternal = static_cast<int>(vc);
        place();
    }
    template <int RM = ValidRow, int CM = ValidCol>
    PTO_INTERNAL Tile(std::enable_if_t<(RM == DYNAMIC) && (CM > 0), size_t> vr)
    {
        this->RowMaskInternal = static_cast<int>(vr);
        place();
    }
    template <int RM = ValidRow, int CM = ValidCol>
    PTO_INTERNAL Tile(std::enable_if_t<(RM > 0) && (CM == DYNAMIC), size_t> vc)
    {
        this->ColMaskInternal = static_cast<int>(vc);
        place();
    }
    Tile(const Tile &) = default;
    Tile &operator=(const Tile &) = default;

    PTO_INTERNAL int GetValidRow() const { return this->RowMaskInternal; }
    PTO_INTERNAL int GetValidCol() const { return this->ColMaskInternal; }

    // pointer to the tile's storage in the block's shared-memory arena (Vec and Mat tiles)
    PTO_INTERNAL TileDType data() const;
    PTO_INTERNAL void SetValue(const uint32_t offset, const DType val)
    {
        static_assert(Loc == TileType::Vec, "SetValue is for Vec tiles");
        data()[offset] = val;
    }
    PTO_INTERNAL DType GetValue(const uint32_t offset) const
    {
        static_assert(Loc == TileType::Vec, "GetValue is for Vec tiles");
        return data()[offset];
    }


    // storage of its own for a freshly constructed tile (see b200::tile_auto_place)
    PTO_INTERNAL void place()
    {
#if PTO_B200_DEVICE_CODE
        constexpr int space = b200::tile_space(Loc);
        if constexpr (space == b200::kSpaceAcc) {
            addr_ = b200::tile_auto_place(space, static_cast<uint32_t>(Cols)); // tensor-memory columns
        } else if constexpr (space != b200::kSpaceNone) {
            addr_ = b200::tile_auto_place(space, static_cast<uint32_t>(Numel * sizeof(DType)));
        }
#endif
    }

    // ---- backend handle
    uint32_t addr_ = 0;   // Vec / Mat / Left / Right: byte offset in the tile location's window of the arena;
                          // Acc: tensor-memory column offset
    uint32_t pitch_ = 0;  // Mat / Left / Right: bytes between consecutive 64-element blocks of the contiguous dimension
    uint8_t major_ = b200::kColsContiguous; // Mat / Left / Right: which logical dimension is contiguous in memory
};

template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileLeft = Tile<TileType::Left, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_, SLayout::RowMajor,
                      TileConfig::fractalABSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileRight = Tile<TileType::Right, Element_, Rows_, Cols_, BLayout::RowMajor, RowValid_, ColValid_,
                       SLayout::ColMajor, TileConfig::fractalABSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileAcc = Tile<TileType::Acc, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_, SLayout::RowMajor,
                     TileConfig::fractalCSize>;

template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileLeftScale = Tile<TileType::ScaleLeft, Element_, Rows_, Cols_, BLayout::RowMajor, RowValid_, ColValid_,
                           SLayout::RowMajor, TileConfig::fractalMxSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileRightScale = Tile<TileType::ScaleRight, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_,
                            SLayout::ColMajor, TileConfig::fractalMxSize>;

namespace b200 {
// element types the tensor core reads from shared memory: their matrix tiles are kept in the 128-byte swizzle
// (8- and 32-bit integers and fp32 are kept plain and multiplied on the CUDA cores)
template <typename T>
struct is_tc_elem : std::integral_constant<bool, std::is_same_v<T, __half> || std::is_same_v<T, __nv_bfloat16> ||
                                                     std::is_same_v<T, __nv_fp8_e4m3> || std::is_same_v<T, __nv_fp8_e5m2>> {};
} // namespace b200

template <typename T>
struct is_tile : std::false_type {};
template <TileType L, typename E, int R, int C, BLayout B, int RV, int CV, SLayout S, int SS, PadValue P, CompactMode CM>
struct is_tile<Tile<L, E, R, C, B, RV, CV, S, SS, P, CM>> : std::true_type {};
template <typename T>
struct is_global : std::false_type {};
template <typename E, typename S, typename St, Layout L>
struct is_global<GlobalTensor<E, S, St, L>> : std::true_type {};

} // namespace pto
