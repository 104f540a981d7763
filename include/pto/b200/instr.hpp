// PTO instructions on B200.  Call shapes follow the reference's instruction wrappers
// (include/pto/common/pto_instr.hpp, paths relative to the reference root): TASSIGN :24-41, TLOAD :127,
// TSTORE :159, TMATMUL :464, TMATMUL_ACC :481, TEXTRACT :624, TGATHER :800 / :824, TCVT :864, TMOV :882,
// TROWSUM :942, TROWMAX :990, TROWEXPAND{DIV,MUL,SUB} :1057-1073, TEXP :1129, TADDS :1161, TMULS :1188,
// TADD / TSUB / TMUL / TMAX :56-120; results follow the CPU simulation (include/pto/cpu/*.hpp).
//
// How each instruction runs on a thread block (see runtime.hpp for the block context):
//   TLOAD  -> Mat : every thread issues 16-byte asynchronous copies (cp.async) into the 128-byte-swizzled
//                   layout the tensor core reads; completion is observed through set_flag(PIPE_MTE2, ...)
//   TLOAD  -> Vec : cooperative copy into a plain row- or column-major tile in shared memory
//   TEXTRACT / TMOV (Mat -> Left / Right) : shared-memory staging: the window of the staged tile is copied,
//                   16 bytes per thread and step, into the operand tile in the swizzled layout the tensor core
//                   reads (so the Mat tile may be reloaded as soon as the copy is done, as on the NPU)
//   TMATMUL[_ACC] : one thread issues tcgen05.mma (M = 128, N = Right::Cols, K = 16 per instruction) with
//                   shared-memory descriptors built from the two views; the accumulator is an Acc tile in
//                   tensor memory; completion is observed through set_flag(PIPE_M, ...)
//   TSTORE <- Acc : tcgen05.ld, each thread owns one accumulator row, 16 columns at a time
//   vector instructions : the block sweeps the tile's valid region, one warp per row for reductions
#pragma once

#include <math.h>

#include <limits>

#include "event.hpp"

namespace pto {

// ---------------------------------------------------------------- helpers
namespace b200 {

template <typename TileT>
PTO_INTERNAL int vec_offset(int r, int c)
{
    static_assert(TileT::SFractal == SLayout::NoneBox, "vector instructions work on plain (NoneBox) tiles");
    return TileT::isRowMajor ? r * TileT::Cols + c : c * TileT::Rows + r;
}

#if PTO_B200_DEVICE_CODE
__device__ __forceinline__ void block_sync()
{
    b200::sync();
}

__device__ __forceinline__ uint64_t sw128_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16-byte asynchronous copy global -> shared; `valid_bytes` < 16 zero-fills the remainder
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc, int valid_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(valid_bytes)
                 : "memory");
}
#endif

// scalar conversions with the CPU simulation's semantics (include/pto/cpu/TCvt.hpp:28-92)
template <typename D, typename S>
PTO_INTERNAL D convert(S x, RoundMode mode)
{
#if PTO_B200_DEVICE_CODE
    if constexpr (std::is_same_v<D, S>) {
        return x;
    } else if constexpr (std::is_same_v<S, float> && std::is_same_v<D, __half>) {
        const uint32_t u = __float_as_uint(x);
        if ((u & 0x7fffffffu) > 0x7f800000u) { // NaN keeps sign and top payload bits, quiet bit set
            return __ushort_as_half(static_cast<unsigned short>(((u >> 16) & 0x8000u) | 0x7e00u | ((u >> 13) & 0x3ffu)));
        }
        return __float2half_rn(x);
    } else if constexpr (std::is_same_v<S, float> && std::is_same_v<D, __nv_bfloat16>) {
        const uint32_t u = __float_as_uint(x);
        if ((u & 0x7fffffffu) > 0x7f800000u) {
            return __ushort_as_bfloat16(static_cast<unsigned short>((u >> 16) | 0x40u));
        }
        return __float2bfloat16_rn(x);
    } else if constexpr (std::is_same_v<S, __half> && std::is_same_v<D, float>) {
        return __half2float(x);
    } else if constexpr (std::is_same_v<S, __nv_bfloat16> && std::is_same_v<D, float>) {
        return __bfloat162float(x);
    } else if constexpr ((std::is_same_v<S, float> || std::is_same_v<S, __half>)&&std::is_integral_v<D>) {
        double v;
        if constexpr (std::is_same_v<S, float>) {
            v = static_cast<double>(x);
        } else {
            v = static_cast<double>(__half2float(x));
        }
        double r;
        switch (mode) {
            case RoundMode::CAST_RINT: r = rint(v); break;
            case RoundMode::CAST_ROUND: r = round(v); break;
            case RoundMode::CAST_FLOOR: r = floor(v); break;
            case RoundMode::CAST_CEIL: r = ceil(v); break;
            case RoundMode::CAST_TRUNC: r = trunc(v); break;
            case RoundMode::CAST_ODD: {
                const double f = floor(v), frac = v - f;
                r = (frac > 0.5) ? f + 1 : ((frac < 0.5) ? f : ((static_cast<long long>(f) & 1) ? f : f + 1));
                break;
            }
            default: r = v; break;
        }
        return static_cast<D>(r);
    } else if constexpr (std::is_integral_v<S> && std::is_same_v<D, __half>) {
        return __float2half_rn(static_cast<float>(x));
    } else {
        return static_cast<D>(x);
    }
#else
    (void)mode;
    return D(x);
#endif
}

} // namespace b200

// ---------------------------------------------------------------- Tile::data
template <TileType L, typename E, const int R, const int C, const BLayout B, const int RV, const int CV, const SLayout S,
          const int SS, const PadValue P, const CompactMode CM>
PTO_INTERNAL typename Tile<L, E, R, C, B, RV, CV, S, SS, P, CM>::TileDType Tile<L, E, R, C, B, RV, CV, S, SS, P, CM>::data()
    const
{
#if PTO_B200_DEVICE_CODE
    return reinterpret_cast<E *>(b200::arena_of<L>() + addr_);
#else
    return nullptr;
#endif
}

// ---------------------------------------------------------------- TASSIGN
template <typename T, typename AddrType>
PTO_INST void TASSIGN(T &obj, AddrType addr)
{
    if constexpr (is_tile<T>::value) {
        if constexpr (std::is_pointer_v<AddrType>) {
#if PTO_B200_DEVICE_CODE
            obj.addr_ = static_cast<uint32_t>(reinterpret_cast<const uint8_t *>(addr) - b200::arena_of<T::Loc>());
#endif
        } else {
            if constexpr (T::Loc == TileType::Acc) {
                // an L0C byte address: one tensor-memory column holds 128 rows x 4 bytes
                obj.addr_ = static_cast<uint32_t>(addr) / 512u;
            } else {
                obj.addr_ = static_cast<uint32_t>(addr);
#if PTO_B200_DEVICE_CODE
                // `(uint64_t)tile.data() + bytes`, the reference's way of stepping a tile through its buffer, is a
                // generic address inside this block's arena: turn it back into the window's offset
                if constexpr (sizeof(AddrType) == 8) {
                    const uint64_t a = static_cast<uint64_t>(addr);
                    const uint64_t base = reinterpret_cast<uint64_t>(b200::arena_of<T::Loc>());
                    if (a >= base && a - base < static_cast<uint64_t>(b200::kDefaultSmemBytes)) {
                        obj.addr_ = static_cast<uint32_t>(a - base);
                    }
                }
#endif
            }
        }
    } else {
        obj.SetAddr(reinterpret_cast<typename T::DType *>(addr));
    }
}

// compile-time address form (include/pto/common/pto_instr.hpp:30-41 in the reference)
template <std::size_t Addr, typename T>
PTO_INST std::enable_if_t<is_tile<T>::value> TASSIGN(T &obj)
{
    static_assert(T::Loc == TileType::Acc || Addr % 32 == 0, "TASSIGN: tile addresses are 32-byte aligned");
    TASSIGN(obj, static_cast<std::size_t>(Addr));
}

// ---------------------------------------------------------------- TLOAD
// Results follow the CPU simulation (include/pto/cpu/TLoad.hpp:143-177 in the reference): the whole destination tile is
// the pad value of its type (PadValue::Null and Zero: 0; Max / Min: +-infinity, or the integer limits) except where the
// global tensor's elements land.  Row-major tiles: dimensions 0..3 of the global tensor fold into tile rows, dimension 4
// runs along the columns; column-major tiles: dimension 3 runs along the rows, dimensions 0..2 and 4 fold into columns.
namespace b200 {
template <typename T, PadValue P>
PTO_INTERNAL T pad_value();

// where element (i0, i1, i2, r, c) of a five-dimensional global tensor lies in a plain Vec tile
template <typename TileData>
PTO_INTERNAL int folded_offset(int64_t outer, int64_t r, int64_t c, int64_t n3, int64_t n4)
{
    if constexpr (TileData::isRowMajor) {
        return static_cast<int>((outer * n3 + r) * TileData::Cols + c);
    } else {
        return static_cast<int>((outer * n4 + c) * TileData::Rows + r);
    }
}
} // namespace b200

#if PTO_B200_DEVICE_CODE
namespace b200 {
// pipe_warps: a whole tile of a registered matrix is fetched by the copy engine.  The first thread of the loading team
// finds the matrix, turns the tile's address into coordinates and records the copy, which the set_flag that follows
// issues (runtime.hpp, PendingLoad).  Returns 0 when the tile has to go the cp.async way.  Plain arguments and out of
// line: the instruction stream of a tile program stays small and nothing of the caller's is forced into memory.
__device__ __noinline__ uint32_t tload_prepare_engine(unsigned long long addr, uint32_t es, unsigned long long line_stride_bytes,
                                                      uint32_t lines, uint32_t span_bytes, uint32_t dst_smem, PendingLoad *e)
{
    const RegionBounds *rb = region_bounds();
    const RegionShapes *rs = region_shapes();
    if ((span_bytes & 127u) != 0) {
        return 0;
    }
    {
        // the tile must lie inside the arena (a copy by the engine past the block's shared memory would fault)
        const uint32_t start = dst_smem - smem_u32(arena());
        const uint32_t bytes = lines * span_bytes;
        const uint32_t room = arena_bytes();
        if (start > room || bytes > room - start) {
            give_up(602);
            return 0;
        }
    }
    // which registered matrix holds the address (all bounds are read at once: one round trip to shared memory)
    const uint32_t count = rs->count;
    // (independent loads, eight bytes each: the flag words that hold them are eight-byte aligned)
    const ulonglong2 b01 = make_ulonglong2(rb->base[0], rb->base[1]), b23 = make_ulonglong2(rb->base[2], rb->base[3]);
    const ulonglong2 e01 = make_ulonglong2(rb->end[0], rb->end[1]), e23 = make_ulonglong2(rb->end[2], rb->end[3]);
    uint32_t r = kMaxTmaRegions;
    unsigned long long base = 0, end = 0;
    if (count > 0 && addr >= b01.x && addr < e01.x) {
        r = 0, base = b01.x, end = e01.x;
    } else if (count > 1 && addr >= b01.y && addr < e01.y) {
        r = 1, base = b01.y, end = e01.y;
    } else if (count > 2 && addr >= b23.x && addr < e23.x) {
        r = 2, base = b23.x, end = e23.x;
    } else if (count > 3 && addr >= b23.y && addr < e23.y) {
        r = 3, base = b23.y, end = e23.y;
    }
    if (r < kMaxTmaRegions) {
        const unsigned long long off = addr - base;
        const uint32_t pitch_bytes = rs->pitch_bytes[r], row_bytes = rs->row_bytes[r], box_rows = rs->box_rows[r];
        // (box_rows is a power of two and elements are one or two bytes: make_tma_table checks both; matrices of 4 GiB
        // and more go the cp.async way, so that everything below is 32-bit arithmetic)
        if (rs->elem_bytes[r] == es && pitch_bytes == line_stride_bytes && (lines & (box_rows - 1u)) == 0 && (off & 15u) == 0 &&
            end - base < (1ull << 32)) {
            const uint32_t o = static_cast<uint32_t>(off);
            uint32_t xb;
            const uint32_t y = divide_by_pitch(o, pitch_bytes, region_reciprocals()[r], xb);
            if (xb + span_bytes <= row_bytes && o + (lines - 1u) * pitch_bytes + span_bytes <= static_cast<uint32_t>(end - base)) {
                const uint32_t log2_rows = log2_pow2(box_rows);
                e->map = reinterpret_cast<unsigned long long>(&tma_table()->map[r]);
                e->dst = dst_smem;
                e->x = xb >> (es - 1u);
                e->y = y;
                e->shape = (span_bytes >> 7) | ((lines >> log2_rows) << 8) | (log2_rows << 16) | ((128u >> (es - 1u)) << 24);
                return 1;
            }
        }
    }
    return 0;
}
} // namespace b200
#endif

#if PTO_B200_DEVICE_CODE
namespace b200 {
template <typename TileData, typename GlobalData>
__device__ __forceinline__ void tload_impl(TileData &dst, GlobalData &src)
{
    using T = typename TileData::DType;
    const T *g = reinterpret_cast<const T *>(src.data());
    const int64_t s3 = src.GetStride(3), s4 = src.GetStride(4);
    if (b200::runs(PIPE_MTE2)) {
        b200::stamp(0x4000);
    }
    if constexpr (TileData::Loc == TileType::Mat && b200::is_tc_elem<T>::value) {
        // tiles the tensor core reads: the global tensor's unit-stride dimension decides the staged layout; a line is
        // 128 bytes of the contiguous dimension (64 16-bit or 128 8-bit elements), 16-byte chunks swizzled by the line
        constexpr int kCE = 16 / static_cast<int>(sizeof(T)); // elements per 16-byte chunk
        const bool cols_contig = (s4 == 1);
        const int vr = dst.GetValidRow(), vc = dst.GetValidCol();
        const int lines = cols_contig ? TileData::Rows : TileData::Cols;  // index of the strided dimension
        const int span = cols_contig ? TileData::Cols : TileData::Rows;   // extent of the contiguous dimension
        const int v_lines = cols_contig ? vr : vc, v_span = cols_contig ? vc : vr;
        const int64_t line_stride = cols_contig ? s3 : s4;
        const int chunks_per_line = span / kCE;
        const uint32_t base = b200::smem_u32(b200::arena() + dst.addr_);
        const uint32_t pitch = static_cast<uint32_t>(lines) * 128u;
        if (!b200::tile_in_arena<TileType::Mat>(dst.addr_, pitch * static_cast<uint32_t>((span * sizeof(T) + 127) / 128))) {
            b200::give_up(602); // the tile does not fit where it was assigned
            return;
        }
        // 16-byte asynchronous copies need 16-byte aligned sources; ragged rows are fetched element by element
        const bool aligned = ((reinterpret_cast<uintptr_t>(g) | static_cast<uintptr_t>(line_stride * sizeof(T))) & 15u) == 0 &&
                             !__isShared(g); // (a FIFO entry may lie in the block's own shared memory)
        const int team = b200::nthreads_l(), me = b200::tid_l();
        const int lines_per_step = team / chunks_per_line;
        if (aligned && v_lines == lines && v_span == span && lines_per_step * chunks_per_line == team &&
            (lines_per_step & 3) == 0) {
            // whole tile from aligned rows, the team a whole number of lines: a thread keeps its chunk column and walks
            // the lines, so source and destination advance by constants (the swizzle term depends on the line number's
            // low three bits only: constant for a step of eight lines, one flipped bit for a step of four)
            if (me < team) {
                const int ch = me % chunks_per_line, l0 = me / chunks_per_line;
                uint32_t off = base + (ch >> 3) * pitch + l0 * 128u + (((ch & 7) ^ (l0 & 7)) << 4);
                const uint32_t flip = (lines_per_step & 4) ? 64u : 0u;
                const uint32_t step = static_cast<uint32_t>(lines_per_step) * 128u;
                const T *gp = g + l0 * line_stride + ch * kCE;
                const int64_t gstep = lines_per_step * line_stride;
#pragma unroll 4
                for (int l = l0; l < lines; l += lines_per_step) {
                    b200::cp_async16(off, gp, 16);
                    gp += gstep;
                    off = (off + step) ^ flip;
                }
            }
            dst.pitch_ = pitch;
            dst.major_ = cols_contig ? b200::kColsContiguous : b200::kRowsContiguous;
            b200::complete_copies_if_in_order();
            if (b200::runs(PIPE_MTE2)) {
                b200::stamp(0x4001);
            }
            return;
        }
        for (int q = b200::tid_l(), q_step = b200::nthreads_l(); q < lines * chunks_per_line; q += q_step) {
            const int l = q / chunks_per_line, ch = q - l * chunks_per_line;
            const int e0 = ch * kCE; // first element of this 16-byte chunk along the contiguous dimension
            int valid = (l < v_lines) ? (v_span - e0) * static_cast<int>(sizeof(T)) : 0;
            valid = valid < 0 ? 0 : (valid > 16 ? 16 : valid);
            const uint32_t off = (ch >> 3) * pitch + l * 128u + (((ch & 7) ^ (l & 7)) << 4);
            if (aligned) {
                b200::cp_async16(base + off, valid > 0 ? g + l * line_stride + e0 : g, valid);
            } else {
                uint4 v = make_uint4(0, 0, 0, 0);
                unsigned char *h = reinterpret_cast<unsigned char *>(&v);
                const unsigned char *gb = reinterpret_cast<const unsigned char *>(g + l * line_stride + e0);
                for (int e = 0; e < valid; ++e) {
                    h[e] = gb[e];
                }
                *reinterpret_cast<uint4 *>(b200::arena() + dst.addr_ + off) = v;
            }
        }
        dst.pitch_ = pitch;
        dst.major_ = cols_contig ? b200::kColsContiguous : b200::kRowsContiguous;
        b200::complete_copies_if_in_order();
    } else if constexpr (TileData::Loc == TileType::Mat) {
        // matrix tiles of integers, fp32 and scale bytes are kept plain (row-major Rows x Cols, zero outside the valid
        // region); TMATMUL on int8 / fp32 runs on the CUDA cores with the simulation's arithmetic
        T *t = reinterpret_cast<T *>(b200::arena() + dst.addr_);
        const int vr = dst.GetValidRow(), vc = dst.GetValidCol();
        for (int i = b200::tid_l(), i_step = b200::nthreads_l(); i < TileData::Numel; i += i_step) {
            const int r = i / TileData::Cols, c = i - r * TileData::Cols;
            t[i] = (r < vr && c < vc) ? g[r * s3 + c * s4] : T(0);
        }
        dst.pitch_ = 0;
        dst.major_ = b200::kPlain;
        b200::sync_l();
    } else {
        static_assert(TileData::Loc == TileType::Vec || TileData::Loc == TileType::Bias,
                      "TLOAD: destination must be a Vec, Bias or Mat tile");
        static_assert(TileData::SFractal == SLayout::NoneBox, "TLOAD: plain (NoneBox) vector tiles");
        T *t = dst.data();
        const int64_t n0 = src.GetShape(0), n1 = src.GetShape(1), n2 = src.GetShape(2), n3 = src.GetShape(3),
                      n4 = src.GetShape(4);
        const int64_t outer = n0 * n1 * n2;
        // rows x cols of the tile that the global tensor covers; everything else becomes the pad value
        const int64_t cov_r = TileData::isRowMajor ? outer * n3 : n3;
        const int64_t cov_c = TileData::isRowMajor ? n4 : outer * n4;
        if (cov_r < TileData::Rows || cov_c < TileData::Cols) {
            const T pad = b200::pad_value<T, TileData::PadVal>();
            for (int i = b200::tid_l(), i_step = b200::nthreads_l(); i < TileData::Numel; i += i_step) {
                const int r = TileData::isRowMajor ? i / TileData::Cols : i % TileData::Rows;
                const int c = TileData::isRowMajor ? i % TileData::Cols : i / TileData::Rows;
                if (r >= cov_r || c >= cov_c) {
                    t[i] = pad;
                }
            }
        }
        const int64_t per = n3 * n4;
        for (int64_t i = b200::tid_l(), i_step = b200::nthreads_l(); i < outer * per; i += i_step) {
            const int64_t o = i / per, rc = i - o * per;
            // consecutive threads walk the global tensor's unit-stride dimension
            const int64_t r = (s4 == 1) ? rc / n4 : rc % n3, c = (s4 == 1) ? rc % n4 : rc / n3;
            const int64_t i2 = o % n2, i1 = (o / n2) % n1, i0 = o / (n2 * n1);
            t[b200::folded_offset<TileData>(o, r, c, n3, n4)] =
                g[i0 * src.GetStride(0) + i1 * src.GetStride(1) + i2 * src.GetStride(2) + r * s3 + c * s4];
        }
        b200::sync_l();
    }
}
} // namespace b200
#endif

template <typename TileData, typename GlobalData, typename... WaitEvents>
PTO_INST RecordEvent TLOAD(TileData &dst, GlobalData &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(sizeof(typename TileData::DType) == sizeof(typename GlobalData::DType),
                  "TLOAD: source and destination element sizes differ");
    static_assert(GlobalData::layout == Layout::ND || GlobalData::layout == Layout::DN,
                  "TLOAD: ND and DN global tensors are supported");
#if PTO_B200_DEVICE_CODE
    if constexpr (b200::kPipeWarps) {
        const bool helper = b200::helps_mte2();
        if (!helper && !b200::runs(PIPE_MTE1)) {
            return {}; // staged tiles are touched by the loading warps and by the thread of MTE1 / M only
        }
        volatile uint32_t *pend = b200::pending_count(); // [1]: the copy engine takes the tile
        if constexpr (TileData::Loc == TileType::Mat && b200::is_tc_elem<typename TileData::DType>::value) {
            using T = typename TileData::DType;
            const bool cols_contig = (src.GetStride(4) == 1);
            const int lines = cols_contig ? TileData::Rows : TileData::Cols;
            const int span = cols_contig ? TileData::Cols : TileData::Rows;
            const uint32_t pitch = static_cast<uint32_t>(lines) * 128u;
            dst.pitch_ = pitch;
            dst.major_ = cols_contig ? b200::kColsContiguous : b200::kRowsContiguous;
            if (!helper) {
                return {};
            }
            const int v_lines = cols_contig ? dst.GetValidRow() : dst.GetValidCol();
            const int v_span = cols_contig ? dst.GetValidCol() : dst.GetValidRow();
            if (b200::control()->mode & b200::kModeEngineLoads) {
                // the copy is prepared by the thread that runs ahead; the loading thread counts the TLOAD
                volatile uint32_t *c = b200::load_ring_counters();
                if (threadIdx.x == b200::kPrepareThread) {
                    const uint32_t head = c[0];
                    if (b200::wait_for_count(&c[2], head + 1u - b200::kLoadRing, 1537)) {
                        b200::PendingLoad *e = b200::load_ring() + (head & (b200::kLoadRing - 1));
                        uint32_t take = 0;
                        if (v_lines == lines && v_span == span) {
                            take = b200::tload_prepare_engine(
                                reinterpret_cast<unsigned long long>(src.data()), static_cast<uint32_t>(sizeof(T)),
                                static_cast<unsigned long long>(cols_contig ? src.GetStride(3) : src.GetStride(4)) * sizeof(T),
                                static_cast<uint32_t>(lines), static_cast<uint32_t>(span * sizeof(T)),
                                b200::smem_u32(b200::arena() + dst.addr_), e);
                        }
                        if (take == 0) {
                            e->shape = 0;
                        }
                        __threadfence_block();
                        c[0] = head + 1u;
                    }
                } else if (threadIdx.x == 0) {
                    b200::stamp(0x4000);
                    c[1] = c[1] + 1u;
                    b200::stamp(0x4001);
                }
                return {};
            }
            if (threadIdx.x == 0) {
                b200::stamp(0x4000);
                uint32_t take = 0;
                if (v_lines == lines && v_span == span && pend[0] < static_cast<uint32_t>(b200::kMaxPendingLoads)) {
                    take = b200::tload_prepare_engine(
                        reinterpret_cast<unsigned long long>(src.data()), static_cast<uint32_t>(sizeof(T)),
                        static_cast<unsigned long long>(cols_contig ? src.GetStride(3) : src.GetStride(4)) * sizeof(T),
                        static_cast<uint32_t>(lines), static_cast<uint32_t>(span * sizeof(T)),
                        b200::smem_u32(b200::arena() + dst.addr_), b200::pending_loads() + pend[0]);
                    if (take != 0) {
                        pend[0] = pend[0] + 1;
                    }
                }
                pend[1] = take;
            }
        } else {
            if constexpr (TileData::Loc == TileType::Mat) {
                dst.pitch_ = 0;
                dst.major_ = b200::kPlain;
            }
            if (!helper) {
                return {};
            }
            if (b200::control()->mode & b200::kModeEngineLoads) {
                if (threadIdx.x == 0) {
                    b200::give_up(601); // a TLOAD that the copy engine cannot do, in a launch that promised there are none
                }
                return {};
            }
            if (threadIdx.x == 0) {
                pend[1] = 0;
            }
        }
        // the helping threads learn here whether they copy (and, if so, that the loading thread is past its waits)
        b200::sync_l();
        const uint32_t take = pend[1];
        b200::sync_l();
        if (take != 0) {
            b200::stamp(0x4001);
            return {};
        }
        // copied by threads: complete when TLOAD returns, so that the loading thread alone can raise the flag
        b200::complete_loads();
        b200::tload_impl(dst, src);
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (threadIdx.x == 0) {
            b200::held_back()[14] = 1; // tiles written through the generic proxy from here on
        }
        b200::sync_l();
        return {};
    }
    b200::tload_impl(dst, src);
#endif
    return {};
}

// ---------------------------------------------------------------- TEXTRACT / TMOV into matrix operands
// Window of `src` starting at (indexRow, indexCol) with the destination's shape
// (docs/isa/TEXTRACT.md:14-18 in the reference).  Both tiles use the same kind of layout: "lines" along the
// strided dimension, 128 bytes (64 elements) of the contiguous dimension per line and block, 16-byte chunks
// XOR-swizzled with the line number inside each group of 8 lines.  The offset along the contiguous dimension
// must be a multiple of 8 elements.
#if PTO_B200_DEVICE_CODE
namespace b200 {
// LaunchOptions::extract_views: a window that is a whole number of swizzle atoms inside the staged tile is read by the
// tensor core in place: the operand tile becomes a view of it (address from the start of the arena, the staged tile's
// block pitch).  Returns false when the window has to be copied.
template <typename DstTileData, typename SrcTileData>
PTO_INTERNAL bool textract_view(DstTileData &dst, SrcTileData &src, int indexRow, int indexCol)
{
    using T = typename DstTileData::DType;
    constexpr uint32_t kCE = 16 / static_cast<uint32_t>(sizeof(T));
    constexpr uint32_t kChunksPerBlock = 8; // 128 bytes of the contiguous dimension
    if ((control()->mode & kModeViews) == 0) {
        return false;
    }
    // (one branch per staged layout, so that each works with the tiles' compile-time extents)
    const uint32_t src_addr = src.addr_, src_pitch = src.pitch_;
    uint32_t line0, chunk0;
    bool fits, k_major;
    if (src.major_ == kColsContiguous) {
        line0 = static_cast<uint32_t>(indexRow), chunk0 = static_cast<uint32_t>(indexCol) / kCE;
        fits = line0 + DstTileData::Rows <= SrcTileData::Rows && chunk0 + DstTileData::Cols / kCE <= SrcTileData::Cols / kCE;
        k_major = DstTileData::Loc == TileType::Left;
    } else {
        line0 = static_cast<uint32_t>(indexCol), chunk0 = static_cast<uint32_t>(indexRow) / kCE;
        fits = line0 + DstTileData::Cols <= SrcTileData::Cols && chunk0 + DstTileData::Rows / kCE <= SrcTileData::Rows / kCE;
        k_major = DstTileData::Loc != TileType::Left;
    }
    if (((line0 & 7u) | (chunk0 & (kChunksPerBlock - 1u))) != 0 || !fits) {
        return false;
    }
    dst.addr_ = src_addr + (chunk0 / kChunksPerBlock) * src_pitch + line0 * 128u;
    dst.pitch_ = src_pitch;
    dst.major_ = static_cast<uint8_t>((k_major ? 0 : 1) | kView);
    if (tid_b() == 0) {
        held_back()[15] = 1; // flags that free the staged tile wait for the products (runtime.hpp)
    }
    return true;
}

template <typename DstTileData, typename SrcTileData>
__device__ __forceinline__ void textract_impl(DstTileData &dst, SrcTileData &src, uint16_t indexRow, uint16_t indexCol)
{
    using T = typename DstTileData::DType;
    if constexpr (DstTileData::Loc == TileType::ScaleLeft || DstTileData::Loc == TileType::ScaleRight) {
        // e8m0 scales of an MX product, one per 32 k: the window of the plain scale tile is written as the atoms the
        // tensor core reads - for 128 rows (ScaleLeft) or 128 columns (ScaleRight) and four consecutive scales,
        // 512 bytes with byte (i % 32) * 16 + (i / 32) * 4 + j for row / column i and scale j.  Atoms are ordered
        // [group of 128][group of 4 scales]; positions outside the destination's valid region hold 2^0.
        static_assert(sizeof(T) == 1, "scale tiles hold one byte per scale");
        constexpr bool kLeftSide = DstTileData::Loc == TileType::ScaleLeft;
        constexpr int kLines = kLeftSide ? DstTileData::Rows : DstTileData::Cols;   // rows of A / columns of B
        constexpr int kScales = kLeftSide ? DstTileData::Cols : DstTileData::Rows;  // scales per line
        constexpr int kGroups = (kLines + 127) / 128, kAtoms = (kScales + 3) / 4;
        const unsigned char *sp = reinterpret_cast<const unsigned char *>(b200::arena_of<TileType::Mat>() + src.addr_);
        unsigned char *dp = reinterpret_cast<unsigned char *>(b200::arena_of<DstTileData::Loc>() + dst.addr_);
        for (int i = b200::tid_b(), i_step = b200::nthreads_b(); i < kGroups * kAtoms * 512; i += i_step) {
            const int atom = i >> 9, b = i & 511;
            const int grp = atom / kAtoms, a = atom - grp * kAtoms;
            const int line = grp * 128 + ((b >> 2) & 3) * 32 + (b >> 4), sc = a * 4 + (b & 3);
            unsigned char v = 127;
            if (line < kLines && sc < kScales) {
                const int r = kLeftSide ? line + indexRow : sc + indexRow, c = kLeftSide ? sc + indexCol : line + indexCol;
                if (r < SrcTileData::Rows && c < SrcTileData::Cols) {
                    v = sp[r * SrcTileData::Cols + c];
                }
            }
            dp[i] = v;
        }
        dst.pitch_ = 0;
        dst.major_ = b200::kPlain;
    } else if constexpr (!b200::is_tc_elem<T>::value) {
        // plain tiles (integers, fp32): the window, row by row; outside the source tile the operand is zero
        const T *s = reinterpret_cast<const T *>(b200::arena_of<TileType::Mat>() + src.addr_);
        T *d = reinterpret_cast<T *>(b200::arena_of<DstTileData::Loc>() + dst.addr_);
        for (int i = b200::tid_b(), i_step = b200::nthreads_b(); i < DstTileData::Numel; i += i_step) {
            const int r = i / DstTileData::Cols, c = i - r * DstTileData::Cols;
            const int sr = r + indexRow, sc = c + indexCol;
            d[i] = (sr < SrcTileData::Rows && sc < SrcTileData::Cols) ? s[sr * SrcTileData::Cols + sc] : T(0);
        }
        dst.pitch_ = 0;
        dst.major_ = b200::kPlain;
    } else {
        constexpr int kCE = 16 / static_cast<int>(sizeof(T));
        const bool cols_contig = (src.major_ == b200::kColsContiguous);
        const int line0 = cols_contig ? indexRow : indexCol;
        const int chunk0 = (cols_contig ? indexCol : indexRow) / kCE;
        const int lines = cols_contig ? DstTileData::Rows : DstTileData::Cols;
        const int chunks_per_line = (cols_contig ? DstTileData::Cols : DstTileData::Rows) / kCE;
        // lines and chunks of the source tile's own storage; a window that reaches past them reads zeros
        const int src_lines = cols_contig ? SrcTileData::Rows : SrcTileData::Cols;
        const int src_chunks = (cols_contig ? SrcTileData::Cols : SrcTileData::Rows) / kCE;
        const uint32_t dst_pitch = static_cast<uint32_t>(lines) * 128u;
        // Left [M x K] is a K-major operand when its columns are contiguous; Right [K x N] when its rows are
        const bool k_major = (DstTileData::Loc == TileType::Left) ? cols_contig : !cols_contig;
        if (b200::kPipeWarps && b200::tid_b() == 0) {
            b200::held_back()[14] = 1; // an operand tile written through the generic proxy
        }
        if (!b200::tile_in_arena<DstTileData::Loc>(dst.addr_, dst_pitch * static_cast<uint32_t>((chunks_per_line + 7) / 8))) {
            b200::give_up(602); // the operand tile does not fit where it was assigned
            return;
        }
        const uint8_t *s = b200::arena_of<TileType::Mat>() + src.addr_;
        uint8_t *d = b200::arena_of<DstTileData::Loc>() + dst.addr_;
        for (int q = b200::tid_b(), q_step = b200::nthreads_b(); q < lines * chunks_per_line; q += q_step) {
            const int l = q / chunks_per_line, ch = q - l * chunks_per_line;
            const int sl = line0 + l, sch = chunk0 + ch;
            const uint32_t s_off = (sch >> 3) * src.pitch_ + sl * 128u + (((sch & 7) ^ (sl & 7)) << 4);
            const uint32_t d_off = (ch >> 3) * dst_pitch + l * 128u + (((ch & 7) ^ (l & 7)) << 4);
            *reinterpret_cast<uint4 *>(d + d_off) = (sl < src_lines && sch < src_chunks)
                                                        ? *reinterpret_cast<const uint4 *>(s + s_off)
                                                        : make_uint4(0, 0, 0, 0);
        }
        dst.pitch_ = dst_pitch;
        dst.major_ = k_major ? 0 : 1;
    }
    if constexpr (DstTileData::ValidRow == DYNAMIC) {
        dst.RowMaskInternal = src.GetValidRow() - indexRow;
    }
    if constexpr (DstTileData::ValidCol == DYNAMIC) {
        dst.ColMaskInternal = src.GetValidCol() - indexCol;
    }
}
} // namespace b200
#endif

template <typename DstTileData, typename SrcTileData, typename... WaitEvents>
PTO_INST RecordEvent TEXTRACT(DstTileData &dst, SrcTileData &src, uint16_t indexRow = 0, uint16_t indexCol = 0,
                              WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(SrcTileData::Loc == TileType::Mat, "TEXTRACT: source must be a Mat tile");
    static_assert(DstTileData::Loc == TileType::Left || DstTileData::Loc == TileType::Right ||
                      DstTileData::Loc == TileType::ScaleLeft || DstTileData::Loc == TileType::ScaleRight,
                  "TEXTRACT: destination must be a Left, Right, ScaleLeft or ScaleRight tile");
    static_assert(sizeof(typename DstTileData::DType) == sizeof(typename SrcTileData::DType),
                  "TEXTRACT: element sizes differ");
#if PTO_B200_DEVICE_CODE
    if constexpr (b200::kPipeWarps) {
        if (!b200::runs(PIPE_MTE1)) {
            return {}; // operand tiles are only ever used by the thread of MTE1 and M
        }
        if constexpr ((DstTileData::Loc == TileType::Left || DstTileData::Loc == TileType::Right) &&
                      b200::is_tc_elem<typename DstTileData::DType>::value) {
            if (b200::textract_view(dst, src, indexRow, indexCol)) {
                if constexpr (DstTileData::ValidRow == DYNAMIC) {
                    dst.RowMaskInternal = src.GetValidRow() - indexRow;
                }
                if constexpr (DstTileData::ValidCol == DYNAMIC) {
                    dst.ColMaskInternal = src.GetValidCol() - indexCol;
                }
                return {};
            }
        }
    }
    b200::textract_impl(dst, src, indexRow, indexCol);
#endif
    return {};
}

// ---------------------------------------------------------------- TMATMUL / TMATMUL_ACC / TMATMUL_BIAS
// (half, half -> float) and (bfloat16, bfloat16 -> float) run on the tensor core; (float, float -> float) and
// (int8, int8 -> int32), the two other operand types of the reference (include/pto/cpu/TMatmul.hpp:46-51), are plain
// tiles multiplied on the CUDA cores in the simulation's order: one sum over k per output element, products and sums
// rounded separately, added to the accumulator (or the bias) at the end (TMatmul.hpp:22-37,99-116).
namespace b200 {
template <typename TileAccT, typename TileLeftT, typename TileRightT>
PTO_INTERNAL void matmul_check()
{
    using AT = typename TileLeftT::DType;
    using CT = typename TileAccT::DType;
    static_assert(std::is_same_v<AT, typename TileRightT::DType>, "TMATMUL: operand types differ");
    static_assert(((std::is_same_v<AT, __half> || std::is_same_v<AT, __nv_bfloat16> || std::is_same_v<AT, float>)&&std::is_same_v<CT, float>) ||
                      (std::is_same_v<AT, int8_t> && std::is_same_v<CT, int32_t>),
                  "TMATMUL: (half | bfloat16 | float -> float) or (int8 -> int32)");
    static_assert(TileLeftT::Loc == TileType::Left && TileRightT::Loc == TileType::Right &&
                      TileAccT::Loc == TileType::Acc,
                  "TMATMUL: expects (Acc, Left, Right)");
    static_assert(TileLeftT::Rows <= 128 && TileLeftT::Cols == TileRightT::Rows && TileLeftT::Rows == TileAccT::Rows,
                  "TMATMUL: m <= 128, inconsistent m / k");
    static_assert(TileRightT::Cols % 16 == 0 && TileRightT::Cols <= 256 && TileAccT::Cols == TileRightT::Cols,
                  "TMATMUL: n a multiple of 16, at most 256");
}

// tensor-core product; `accumulate` false: the accumulator is overwritten
template <typename TileAccT, typename TileLeftT, typename TileRightT>
PTO_INTERNAL void matmul_issue(TileAccT &c, TileLeftT &a, TileRightT &b, bool accumulate)
{
    using AT = typename TileLeftT::DType;
    static_assert(TileLeftT::Cols % 16 == 0, "TMATMUL: k a multiple of 16");
#if PTO_B200_DEVICE_CODE
    if (!kPipeWarps && (control()->mode & kModeInOrder)) { // (in-order launches are not pipe-warps launches)
        // no flags order the operands' staging before the product: every thread's writes are made visible to the
        // tensor core here (in a program with flags, set_flag(PIPE_MTE1, PIPE_M, ...) does this)
        fence_async_proxy();
        b200::sync();
    }
    if (b200::tid_b() == 0) {
        stamp(0x6000);
        constexpr uint32_t kBf16 = std::is_same_v<AT, __nv_bfloat16> ? 1u : 0u;
        const uint32_t a_major = a.major_ & 1u, b_major = b.major_ & 1u;
        const uint32_t idesc = (1u << 4) | (kBf16 << 7) | (kBf16 << 10) | (a_major << 15) | (b_major << 16) |
                               (static_cast<uint32_t>(TileRightT::Cols >> 3) << 17) | (8u << 24); // M = 128
        const uint32_t d_tmem = control()->tmem_base + c.addr_;
        // a view (TEXTRACT with extract_views) is addressed from the start of the arena
        const uint32_t a_addr = smem_u32(((a.major_ & kView) ? arena() : arena_of<TileType::Left>()) + a.addr_);
        const uint32_t b_addr = smem_u32(((b.major_ & kView) ? arena() : arena_of<TileType::Right>()) + b.addr_);
        tc_fence_after();
        // (the tiles' fields are read once: the products' "memory" clobbers would have them read again from the
        // handles, which live in local memory when a program indexes arrays of tiles at run time)
        const uint32_t a_pitch = a.pitch_, b_pitch = b.pitch_;
        // K-major view: 16 k-values are 32 bytes inside a 128-byte line, blocks of 64 k are `pitch` apart;
        // MN-major view: 16 k-values are 16 lines of 128 bytes, 64-element blocks of M/N are `pitch` apart.
        // The descriptor of step kk is the first one plus the step's byte offset (a multiple of 16) in its low field.
        const uint64_t a_desc0 = (a_major == 0) ? sw128_desc(a_addr, 16, 1024) : sw128_desc(a_addr, a_pitch, 1024);
        const uint64_t b_desc0 = (b_major == 0) ? sw128_desc(b_addr, 16, 1024) : sw128_desc(b_addr, b_pitch, 1024);
        if (a_major == 0 && b_major == 0) {
            // both operands K-major (the common case): the steps inside a 64-k block are constants apart
            const uint64_t a_block = a_pitch >> 4, b_block = b_pitch >> 4;
#pragma unroll
            for (int kk = 0; kk < TileLeftT::Cols / 16; ++kk) {
                const uint64_t in_block = static_cast<uint64_t>((kk & 3) * 2);
                mma_f16(d_tmem, a_desc0 + (kk >> 2) * a_block + in_block, b_desc0 + (kk >> 2) * b_block + in_block, idesc,
                        (accumulate || kk != 0) ? 1u : 0u);
            }
        } else {
#pragma unroll
            for (int kk = 0; kk < TileLeftT::Cols / 16; ++kk) {
                const uint32_t k0 = kk * 16;
                const uint32_t a_off = (a_major == 0) ? (k0 >> 6) * a_pitch + (k0 & 63u) * 2u : k0 * 128u;
                const uint32_t b_off = (b_major == 0) ? (k0 >> 6) * b_pitch + (k0 & 63u) * 2u : k0 * 128u;
                mma_f16(d_tmem, a_desc0 + (a_off >> 4), b_desc0 + (b_off >> 4), idesc, (accumulate || kk != 0) ? 1u : 0u);
            }
        }
        stamp(0x6001);
    }
    complete_matmul_if_in_order();
#endif
}

// CUDA-core product of plain tiles.  mode 0: C = A B, 1: C += A B, 2: C = A B + bias (one value per column).
// A thread owns one accumulator row (its tensor-memory lane), sixteen columns at a time.
template <typename TileAccT, typename TileLeftT, typename TileRightT>
PTO_INTERNAL void matmul_plain(TileAccT &c, TileLeftT &a, TileRightT &b, int mode, const typename TileAccT::DType *bias)
{
#if PTO_B200_DEVICE_CODE
    using AT = typename TileLeftT::DType;
    using CT = typename TileAccT::DType;
    constexpr int K = TileLeftT::Cols, N = TileRightT::Cols;
    if (not_with_pipe_warps(1)) {
        return; // a product on the CUDA cores needs four warps on the matrix pipe
    }
    const AT *pa = reinterpret_cast<const AT *>(arena_of<TileType::Left>() + a.addr_);
    const AT *pb = reinterpret_cast<const AT *>(arena_of<TileType::Right>() + b.addr_);
    const int m = a.GetValidRow(), kv = a.GetValidCol(), n = b.GetValidCol();
    const int warp = b200::tid() >> 5, lane = b200::tid() & 31;
    const int quarter = warp & 3, group = warp >> 2, groups = b200::nthreads() >> 7;
    const int row = quarter * 32 + lane;
    const uint32_t taddr = control()->tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c.addr_;
    b200::sync();
    tc_fence_after();
    for (int c0 = group * 16; c0 < N; c0 += groups * 16) {
        uint32_t r[16];
        if (mode == 1) {
            tmem_ld16(taddr + c0, r);
        }
#pragma unroll 1
        for (int j = 0; j < 16; ++j) {
            const int col = c0 + j;
            CT acc = CT(0);
            if (row < m && row < TileLeftT::Rows && col < n) {
                for (int k = 0; k < kv; ++k) {
                    if constexpr (std::is_same_v<CT, float>) {
                        acc = __fadd_rn(acc, __fmul_rn(pa[row * K + k], pb[k * N + col]));
                    } else {
                        acc += static_cast<CT>(pa[row * K + k]) * static_cast<CT>(pb[k * N + col]);
                    }
                }
                if (mode == 1) {
                    CT prev;
                    memcpy(&prev, &r[j], 4);
                    if constexpr (std::is_same_v<CT, float>) {
                        acc = __fadd_rn(prev, acc);
                    } else {
                        acc = prev + acc;
                    }
                } else if (mode == 2) {
                    if constexpr (std::is_same_v<CT, float>) {
                        acc = __fadd_rn(acc, bias[col]);
                    } else {
                        acc = acc + bias[col];
                    }
                }
            }
            memcpy(&r[j], &acc, 4);
        }
        tmem_st16(taddr + c0, r);
    }
    tc_fence_before();
    b200::sync();
    tc_fence_after();
#endif
}

template <typename TileAccT, typename TileLeftT, typename TileRightT>
PTO_INTERNAL void matmul_dispatch(TileAccT &c, TileLeftT &a, TileRightT &b, bool accumulate)
{
    matmul_check<TileAccT, TileLeftT, TileRightT>();
    if constexpr (is_tc_elem<typename TileLeftT::DType>::value) {
        matmul_issue(c, a, b, accumulate);
    } else {
        matmul_plain(c, a, b, accumulate ? 1 : 0, nullptr);
    }
}
} // namespace b200

// The AccPhase argument selects the NPU's unit-flag handshake between the matrix pipe and the store that follows
// (Partial: more products to come, Final: the accumulator is complete; include/pto/npu/a2a3/TMatmul.hpp:148-180 in the
// reference).  Here completion is observed through set_flag(PIPE_M, ...) in every case, so the phase changes nothing.
template <typename TileAccT, typename TileLeftT, typename TileRightT, typename... WaitEvents>
PTO_INST RecordEvent TMATMUL(TileAccT &cMatrix, TileLeftT &aMatrix, TileRightT &bMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::matmul_dispatch(cMatrix, aMatrix, bMatrix, false);
    return {};
}
template <AccPhase Phase, typename TileAccT, typename TileLeftT, typename TileRightT, typename... WaitEvents>
PTO_INST RecordEvent TMATMUL(TileAccT &cMatrix, TileLeftT &aMatrix, TileRightT &bMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::matmul_dispatch(cMatrix, aMatrix, bMatrix, false);
    return {};
}

// the accumulator is updated in place (the reference's kernels pass the same tile twice; a distinct input tile is
// copied into the output's tensor-memory columns first)
namespace b200 {
template <typename TileAccT>
PTO_INTERNAL void acc_copy(TileAccT &dst, TileAccT &src)
{
#if PTO_B200_DEVICE_CODE
    if (dst.addr_ != src.addr_) {
        if (not_with_pipe_warps(2)) {
            return;
        }
        const int warp = b200::tid() >> 5, quarter = warp & 3, group = warp >> 2, groups = b200::nthreads() >> 7;
        const uint32_t lane_base = control()->tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        b200::sync();
        tc_fence_after();
        for (int c0 = group * 16; c0 < TileAccT::Cols; c0 += groups * 16) {
            uint32_t r[16];
            tmem_ld16(lane_base + src.addr_ + c0, r);
            tmem_st16(lane_base + dst.addr_ + c0, r);
        }
        tc_fence_before();
        b200::sync();
        tc_fence_after();
    }
#endif
}
} // namespace b200

template <typename TileAccT, typename TileLeftT, typename TileRightT, typename... WaitEvents>
PTO_INST RecordEvent TMATMUL_ACC(TileAccT &cOutMatrix, TileAccT &cInMatrix, TileLeftT &aMatrix, TileRightT &bMatrix,
                                 WaitEvents &... events)
{
    TSYNC(events...);
    b200::acc_copy(cOutMatrix, cInMatrix);
    b200::matmul_dispatch(cOutMatrix, aMatrix, bMatrix, true);
    return {};
}
template <AccPhase Phase, typename TileAccT, typename TileLeftT, typename TileRightT, typename... WaitEvents>
PTO_INST RecordEvent TMATMUL_ACC(TileAccT &cOutMatrix, TileAccT &cInMatrix, TileLeftT &aMatrix, TileRightT &bMatrix,
                                 WaitEvents &... events)
{
    TSYNC(events...);
    b200::acc_copy(cOutMatrix, cInMatrix);
    b200::matmul_dispatch(cOutMatrix, aMatrix, bMatrix, true);
    return {};
}
// shared accumulator tile (include/pto/common/pto_instr.hpp:498-507 in the reference)
template <AccPhase Phase = AccPhase::Unspecified, typename TileAccT, typename TileLeftT, typename TileRightT,
          typename... WaitEvents,
          std::enable_if_t<TileLeftT::Loc == TileType::Left && TileRightT::Loc == TileType::Right, int> = 0>
PTO_INST RecordEvent TMATMUL_ACC(TileAccT &cMatrix, TileLeftT &aMatrix, TileRightT &bMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::matmul_dispatch(cMatrix, aMatrix, bMatrix, true);
    return {};
}

// TMATMUL_BIAS (include/pto/cpu/TMatmul.hpp:99-116): C = A * B + bias, one bias value per column.  On the tensor core
// the bias row is written into every lane of the accumulator's tensor-memory columns first, then the product is
// accumulated onto it.
template <typename TileAccT, typename TileLeftT, typename TileRightT, typename TileBiasT, typename... WaitEvents,
          std::enable_if_t<TileBiasT::Loc == TileType::Bias, int> = 0>
PTO_INST RecordEvent TMATMUL_BIAS(TileAccT &cMatrix, TileLeftT &aMatrix, TileRightT &bMatrix, TileBiasT &biasData,
                                  WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(TileBiasT::Loc == TileType::Bias && TileBiasT::Rows == 1 && TileBiasT::Cols == TileAccT::Cols,
                  "TMATMUL_BIAS: the bias is a 1 x N tile of TileType::Bias");
    static_assert(std::is_same_v<typename TileBiasT::DType, typename TileAccT::DType>,
                  "TMATMUL_BIAS: the bias has the accumulator's type");
    static_assert(TileAccT::Cols % 16 == 0, "TMATMUL_BIAS: accumulator width must be a multiple of 16");
    b200::matmul_check<TileAccT, TileLeftT, TileRightT>();
    if constexpr (!b200::is_tc_elem<typename TileLeftT::DType>::value) {
#if PTO_B200_DEVICE_CODE
        b200::matmul_plain(cMatrix, aMatrix, bMatrix, 2, biasData.data());
#endif
    } else {
#if PTO_B200_DEVICE_CODE
        if (b200::not_with_pipe_warps(3)) {
            return {};
        }
        const int warp = b200::tid() >> 5;
        const int quarter = warp & 3; // tensor-memory lanes [32 * quarter, +32) are writable by this warp
        const int group = warp >> 2, groups = b200::nthreads() >> 7;
        const uint32_t taddr = b200::control()->tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + cMatrix.addr_;
        const float *bias = biasData.data();
        const int vc = biasData.GetValidCol();
        for (int c0 = group * 16; c0 < TileAccT::Cols; c0 += groups * 16) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                r[j] = (c0 + j < vc) ? __float_as_uint(bias[c0 + j]) : 0u;
            }
            b200::tmem_st16(taddr + c0, r);
        }
        b200::tc_fence_before();
        b200::sync();
#endif
        b200::matmul_issue(cMatrix, aMatrix, bMatrix, true);
    }
    return {};
}
template <AccPhase Phase, typename TileAccT, typename TileLeftT, typename TileRightT, typename TileBiasT,
          typename... WaitEvents, std::enable_if_t<TileBiasT::Loc == TileType::Bias, int> = 0>
PTO_INST RecordEvent TMATMUL_BIAS(TileAccT &cMatrix, TileLeftT &aMatrix, TileRightT &bMatrix, TileBiasT &biasData,
                                  WaitEvents &... events)
{
    return TMATMUL_BIAS(cMatrix, aMatrix, bMatrix, biasData, events...);
}

// ---------------------------------------------------------------- TMATMUL_MX
// MX block-scaled product (include/pto/common/pto_instr.hpp:403-460 in the reference; its backends are the A5 / Kirin
// NPUs, there is no CPU simulation of it): C = (scaleA (x) A) * (scaleB (x) B), A [M x K] and B [K x N] in fp8 (e4m3 or
// e5m2), one e8m0 scale per 32 consecutive k of a row of A / a column of B, fp32 accumulation.  On B200 this is
// tcgen05.mma kind::mxf8f6f4 with block scaling: per 128 k the scale atoms (TEXTRACT writes ScaleLeft / ScaleRight
// tiles as atoms) are copied from shared memory into tensor-memory columns kept for them (tcgen05.cp), then four
// products of k = 32 each name their scale byte.  Both operands must be K-major (A loaded from an ND tensor, B from a
// DN one, as the reference's MX kernels do); K a multiple of 32, N at most 256.
namespace b200 {
#if PTO_B200_DEVICE_CODE
// shared-memory descriptor of a scale atom: 32 rows of 16 bytes, no swizzle; 8-row groups are 128 bytes apart
__device__ __forceinline__ uint64_t scale_atom_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= 1ull << 46;
    return d;
}
// 32 rows x 16 bytes of shared memory -> tensor-memory columns [taddr, taddr + 4), repeated in the four lane quarters
__device__ __forceinline__ void copy_scale_atom(uint32_t taddr, uint64_t desc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                         uint32_t sfb, uint32_t acc)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb)
        : "memory");
}
#endif

template <typename TileRes, typename TileLeftT, typename TileLeftScaleT, typename TileRightT, typename TileRightScaleT>
PTO_INTERNAL void matmul_mx_issue(TileRes &c, TileLeftT &a, TileLeftScaleT &sa, TileRightT &b, TileRightScaleT &sb,
                                  bool accumulate)
{
    using AT = typename TileLeftT::DType;
    using BT = typename TileRightT::DType;
    static_assert((std::is_same_v<AT, __nv_fp8_e4m3> || std::is_same_v<AT, __nv_fp8_e5m2>)&&(
                      std::is_same_v<BT, __nv_fp8_e4m3> || std::is_same_v<BT, __nv_fp8_e5m2>),
                  "TMATMUL_MX: fp8 (e4m3 or e5m2) operands");
    static_assert(std::is_same_v<typename TileRes::DType, float>, "TMATMUL_MX: fp32 accumulator");
    static_assert(TileLeftT::Loc == TileType::Left && TileRightT::Loc == TileType::Right && TileRes::Loc == TileType::Acc &&
                      TileLeftScaleT::Loc == TileType::ScaleLeft && TileRightScaleT::Loc == TileType::ScaleRight,
                  "TMATMUL_MX: expects (Acc, Left, ScaleLeft, Right, ScaleRight)");
    static_assert(TileLeftT::Rows <= 128 && TileLeftT::Cols == TileRightT::Rows && TileLeftT::Cols % 32 == 0,
                  "TMATMUL_MX: m <= 128, k a multiple of 32");
    static_assert(TileRightT::Cols % 16 == 0 && TileRightT::Cols <= 256 && TileRes::Cols == TileRightT::Cols,
                  "TMATMUL_MX: n a multiple of 16, at most 256");
    static_assert(TileLeftScaleT::Cols * 32 == TileLeftT::Cols && TileRightScaleT::Rows * 32 == TileRightT::Rows,
                  "TMATMUL_MX: one scale per 32 k");
#if PTO_B200_DEVICE_CODE
    constexpr int K = TileLeftT::Cols, N = TileRightT::Cols;
    constexpr int kSpans = (K + 127) / 128, kAtomsK = (K / 32 + 3) / 4, kGroupsN = (N + 127) / 128;
    if (!kPipeWarps && (control()->mode & kModeInOrder)) { // (in-order launches are not pipe-warps launches)
        fence_async_proxy();
        b200::sync();
    }
    if (b200::tid_b() == 0) {
        if ((a.major_ & 3u) != 0 || (b.major_ & 3u) != 0 || c.addr_ + N > kMxScaleTmemCol) {
            give_up(-2); // operand not K-major, or the accumulator reaches into the scale columns: reported, not run
        } else {
            constexpr uint32_t a_fmt = std::is_same_v<AT, __nv_fp8_e5m2> ? 1u : 0u;
            constexpr uint32_t b_fmt = std::is_same_v<BT, __nv_fp8_e5m2> ? 1u : 0u;
            const uint32_t idesc = (a_fmt << 7) | (b_fmt << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) | (8u << 24);
            const uint32_t d_tmem = control()->tmem_base + c.addr_;
            const uint32_t a_addr = smem_u32(((a.major_ & kView) ? arena() : arena_of<TileType::Left>()) + a.addr_);
            const uint32_t b_addr = smem_u32(((b.major_ & kView) ? arena() : arena_of<TileType::Right>()) + b.addr_);
            const uint32_t sa_addr = smem_u32(arena_of<TileType::ScaleLeft>() + sa.addr_);
            const uint32_t sb_addr = smem_u32(arena_of<TileType::ScaleRight>() + sb.addr_);
            tc_fence_after();
#pragma unroll
            for (int sp = 0; sp < kSpans; ++sp) {
                // two slots of 4 (A) + 8 (B) columns in turn: a slot is rewritten two spans later, after the products
                // that read it, by the same thread (the tensor pipe keeps issue order)
                const uint32_t sfa_tmem = control()->tmem_base + kMxScaleTmemCol + (sp & 1) * 16;
                const uint32_t sfb_tmem = sfa_tmem + 4;
                copy_scale_atom(sfa_tmem, scale_atom_desc(sa_addr + sp * 512));
#pragma unroll
                for (int gn = 0; gn < kGroupsN; ++gn) {
                    copy_scale_atom(sfb_tmem + gn * 4, scale_atom_desc(sb_addr + (gn * kAtomsK + sp) * 512));
                }
                const int kk_end = (K - sp * 128) >= 128 ? 4 : (K - sp * 128) / 32;
                for (int kk = 0; kk < kk_end; ++kk) {
                    const uint32_t kb = sp * 128 + kk * 32; // first k of this product, in bytes of a line
                    const uint64_t a_desc = sw128_desc(a_addr + (kb >> 7) * a.pitch_ + (kb & 127u), 16, 1024);
                    const uint64_t b_desc = sw128_desc(b_addr + (kb >> 7) * b.pitch_ + (kb & 127u), 16, 1024);
                    const uint32_t sf_id = static_cast<uint32_t>(kk);
                    mma_mxf8(d_tmem, a_desc, b_desc, idesc | (sf_id << 29) | (sf_id << 4), sfa_tmem, sfb_tmem,
                             (accumulate || sp != 0 || kk != 0) ? 1u : 0u);
                }
            }
        }
    }
    complete_matmul_if_in_order();
#endif
}
} // namespace b200

template <typename TileRes, typename TileLeftT, typename TileLeftScaleT, typename TileRightT, typename TileRightScaleT,
          typename... WaitEvents,
          std::enable_if_t<TileLeftScaleT::Loc == TileType::ScaleLeft && TileRightScaleT::Loc == TileType::ScaleRight, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes &cMatrix, TileLeftT &aMatrix, TileLeftScaleT &aScaleMatrix, TileRightT &bMatrix,
                                TileRightScaleT &bScaleMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::matmul_mx_issue(cMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix, false);
    return {};
}
template <AccPhase Phase, typename TileRes, typename TileLeftT, typename TileLeftScaleT, typename TileRightT,
          typename TileRightScaleT, typename... WaitEvents,
          std::enable_if_t<TileLeftScaleT::Loc == TileType::ScaleLeft && TileRightScaleT::Loc == TileType::ScaleRight, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes &cMatrix, TileLeftT &aMatrix, TileLeftScaleT &aScaleMatrix, TileRightT &bMatrix,
                                TileRightScaleT &bScaleMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::matmul_mx_issue(cMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix, false);
    return {};
}
// accumulating form: cOut = cIn + product (the accumulator is updated in place)
template <typename TileRes, typename TileLeftT, typename TileLeftScaleT, typename TileRightT, typename TileRightScaleT,
          typename... WaitEvents,
          std::enable_if_t<TileLeftT::Loc == TileType::Left && TileLeftScaleT::Loc == TileType::ScaleLeft, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes &cOutMatrix, TileRes &cInMatrix, TileLeftT &aMatrix, TileLeftScaleT &aScaleMatrix,
                                TileRightT &bMatrix, TileRightScaleT &bScaleMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::acc_copy(cOutMatrix, cInMatrix);
    b200::matmul_mx_issue(cOutMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix, true);
    return {};
}
template <AccPhase Phase, typename TileRes, typename TileLeftT, typename TileLeftScaleT, typename TileRightT,
          typename TileRightScaleT, typename... WaitEvents,
          std::enable_if_t<TileLeftT::Loc == TileType::Left && TileLeftScaleT::Loc == TileType::ScaleLeft, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes &cOutMatrix, TileRes &cInMatrix, TileLeftT &aMatrix, TileLeftScaleT &aScaleMatrix,
                                TileRightT &bMatrix, TileRightScaleT &bScaleMatrix, WaitEvents &... events)
{
    TSYNC(events...);
    b200::acc_copy(cOutMatrix, cInMatrix);
    b200::matmul_mx_issue(cOutMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix, true);
    return {};
}

// ---------------------------------------------------------------- TSTORE
// Vec -> GM follows include/pto/cpu/TStore.hpp:121-150 in the reference (the mirror image of TLOAD's folding of the five
// dimensions); Acc -> GM reads the accumulator out of tensor memory, converting fp32 to the global tensor's 16-bit type
// where that differs (docs/isa/TSTORE.md:67-72).  AtomicType::AtomicAdd adds into the destination; ReluPreMode::
// NormalRelu clamps negative accumulator values to zero before the store; the STPhase argument belongs to the NPU's
// unit-flag handshake and changes nothing here (completion is observed through set_flag).
namespace b200 {
template <typename GT, AtomicType kAtomic>
PTO_INTERNAL void store_elem(GT *p, GT v)
{
#if PTO_B200_DEVICE_CODE
    if constexpr (kAtomic == AtomicType::AtomicAdd) {
        static_assert(std::is_same_v<GT, float> || std::is_same_v<GT, int32_t> || std::is_same_v<GT, __half> ||
                          std::is_same_v<GT, __nv_bfloat16>,
                      "TSTORE<AtomicAdd>: float, int32, half or bfloat16 destinations");
        atomicAdd(p, v);
    } else {
        *p = v;
    }
#endif
}

#if PTO_B200_DEVICE_CODE
template <AtomicType kAtomic, ReluPreMode kRelu, typename GlobalData, typename TileData>
__device__ __forceinline__ void tstore_impl(GlobalData &dst, TileData &src)
{
    using GT = typename GlobalData::DType;
    GT *g = dst.data();
    const int64_t s3 = dst.GetStride(3), s4 = dst.GetStride(4);
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    if constexpr (TileData::Loc == TileType::Acc) {
        using CT = typename TileData::DType;
        static_assert(sizeof(CT) == 4, "TSTORE: 32-bit accumulator tiles");
        static_assert(TileData::Cols % 16 == 0, "TSTORE: accumulator width must be a multiple of 16");
        const int warp = b200::tid() >> 5, lane = b200::tid() & 31;
        const int quarter = warp & 3;   // tensor-memory lanes [32 * quarter, +32) are readable by this warp
        const int group = warp >> 2, groups = b200::nthreads() >> 7;
        const int row = quarter * 32 + lane;
        const uint32_t taddr = control()->tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + src.addr_;
        tc_fence_after();
        if (runs(PIPE_FIX)) {
            stamp(0x7000);
        }
        if constexpr (std::is_same_v<GT, CT> && kAtomic == AtomicType::AtomicNone && kRelu == ReluPreMode::NoRelu &&
                      TileData::Cols % 32 == 0) {
            const uint32_t staging = held_back()[13];
            if (staging != 0 && s4 == 1 && groups == 1 && vr == TileData::Rows && vc == TileData::Cols &&
                ((reinterpret_cast<uintptr_t>(g) | static_cast<uintptr_t>(s3 * 4)) & 15u) == 0) {
                // whole tile to aligned rows: 32 columns at a time, a thread stages the 128 bytes of its row (rows
                // 144 bytes apart, so that a warp's 16-byte stores spread over all banks) and hands them to a bulk
                // copy of its own; the staging row is rewritten once that copy has read it
                if (b200::tid() < TileData::Rows) {
                    uint8_t *mine = arena() + (staging - 1u) + static_cast<uint32_t>(b200::tid()) * kStoreStagingRowBytes;
                    const uint32_t mine_s = smem_u32(mine);
                    GT *grow = g + row * s3;
#pragma unroll 1
                    for (int c0 = 0; c0 < TileData::Cols; c0 += 32) {
                        uint32_t r0[16], r1[16];
                        tmem_ld16(taddr + c0, r0);
                        tmem_ld16(taddr + c0 + 16, r1);
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            *reinterpret_cast<uint4 *>(mine + j * 16) = make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
                            *reinterpret_cast<uint4 *>(mine + 64 + j * 16) = make_uint4(r1[4 * j], r1[4 * j + 1], r1[4 * j + 2], r1[4 * j + 3]);
                        }
                        fence_async_proxy();
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 128;" ::"l"(grow + c0), "r"(mine_s)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    if (!kPipeWarps && (control()->mode & kModeInOrder)) { // (in-order launches are not pipe-warps launches)
                        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    }
                }
                tc_fence_before();
                if (runs(PIPE_FIX)) {
                    stamp(0x7001);
                }
                return;
            }
        }
        for (int c0 = group * 16; c0 < TileData::Cols; c0 += groups * 16) {
            uint32_t r[16];
            tmem_ld16(taddr + c0, r);
            if (row < vr) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c0 + j < vc) {
                        CT v;
                        memcpy(&v, &r[j], 4);
                        if (kRelu == ReluPreMode::NormalRelu && v < CT(0)) {
                            v = CT(0);
                        }
                        if constexpr (std::is_same_v<GT, CT>) {
                            store_elem<GT, kAtomic>(&g[row * s3 + (c0 + j) * s4], v);
                        } else {
                            static_assert(std::is_same_v<CT, float>, "TSTORE: only fp32 accumulators are converted");
                            store_elem<GT, kAtomic>(&g[row * s3 + (c0 + j) * s4],
                                                    convert<GT, float>(v, RoundMode::CAST_RINT));
                        }
                    }
                }
            }
        }
        tc_fence_before();
    } else {
        static_assert(TileData::Loc == TileType::Vec, "TSTORE: source must be a Vec or Acc tile");
        static_assert(TileData::SFractal == SLayout::NoneBox, "TSTORE: plain (NoneBox) vector tiles");
        static_assert(sizeof(typename TileData::DType) == sizeof(GT), "TSTORE: element sizes differ");
        using T = typename TileData::DType;
        const T *t = src.data();
        T *gt = reinterpret_cast<T *>(g);
        const int64_t n0 = dst.GetShape(0), n1 = dst.GetShape(1), n2 = dst.GetShape(2), n3 = dst.GetShape(3),
                      n4 = dst.GetShape(4);
        const int64_t outer = n0 * n1 * n2, per = n3 * n4;
        for (int64_t i = b200::tid(), i_step = b200::nthreads(); i < outer * per; i += i_step) {
            const int64_t o = i / per, rc = i - o * per;
            const int64_t r = (s4 == 1) ? rc / n4 : rc % n3, c = (s4 == 1) ? rc % n4 : rc / n3;
            const int64_t i2 = o % n2, i1 = (o / n2) % n1, i0 = o / (n2 * n1);
            const int off = folded_offset<TileData>(o, r, c, n3, n4);
            const int tr = TileData::isRowMajor ? off / TileData::Cols : off % TileData::Rows;
            const int tc = TileData::isRowMajor ? off % TileData::Cols : off / TileData::Rows;
            if (tr < vr && tc < vc) {
                store_elem<T, kAtomic>(&gt[i0 * dst.GetStride(0) + i1 * dst.GetStride(1) + i2 * dst.GetStride(2) +
                                           r * s3 + c * s4],
                                       t[off]);
            }
        }
    }
}
#endif

template <AtomicType kAtomic, ReluPreMode kRelu, typename GlobalData, typename TileData>
PTO_INTERNAL void tstore(GlobalData &dst, TileData &src)
{
#if PTO_B200_DEVICE_CODE
    if (kPipeWarps && !runs(TileData::Loc == TileType::Acc ? PIPE_FIX : PIPE_MTE3)) {
        return;
    }
    tstore_impl<kAtomic, kRelu>(dst, src);
#endif
}
} // namespace b200

template <typename TileData, typename GlobalData, typename... WaitEvents,
          std::enable_if_t<is_global<GlobalData>::value && is_tile<TileData>::value, int> = 0>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<AtomicType::AtomicNone, ReluPreMode::NoRelu>(dst, src);
    return {};
}
template <STPhase Phase, typename TileData, typename GlobalData, typename... WaitEvents,
          std::enable_if_t<is_global<GlobalData>::value && is_tile<TileData>::value, int> = 0>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<AtomicType::AtomicNone, ReluPreMode::NoRelu>(dst, src);
    return {};
}
template <typename TileData, typename GlobalData, AtomicType atomicType, typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<atomicType, ReluPreMode::NoRelu>(dst, src);
    return {};
}
template <STPhase Phase, typename TileData, typename GlobalData, AtomicType atomicType, typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<atomicType, ReluPreMode::NoRelu>(dst, src);
    return {};
}
template <typename TileData, typename GlobalData, AtomicType atomicType, ReluPreMode reluPreMode, typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<atomicType, reluPreMode>(dst, src);
    return {};
}
template <STPhase Phase, typename TileData, typename GlobalData, AtomicType atomicType, ReluPreMode reluPreMode,
          typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::tstore<atomicType, reluPreMode>(dst, src);
    return {};
}

// the pre-quantisation scalar is accepted and, as in the simulation (include/pto/cpu/TStore.hpp:152-157), not applied
template <typename TileData, typename GlobalData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu, typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, uint64_t preQuantScalar, WaitEvents &... events)
{
    TSYNC(events...);
    (void)preQuantScalar;
    b200::tstore<atomicType, reluPreMode>(dst, src);
    return {};
}
template <STPhase Phase, typename TileData, typename GlobalData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu, typename... WaitEvents>
PTO_INST RecordEvent TSTORE(GlobalData &dst, TileData &src, uint64_t preQuantScalar, WaitEvents &... events)
{
    TSYNC(events...);
    (void)preQuantScalar;
    b200::tstore<atomicType, reluPreMode>(dst, src);
    return {};
}

// ---------------------------------------------------------------- TMOV
//   Mat -> Left / Right : the whole-tile form of TEXTRACT
//   Vec -> Left / Right : staging of a plain 16-bit tile into the swizzled operand layout
//   Acc -> Vec          : tensor memory to shared memory (with conversion to the destination type)
//   Vec -> Vec          : copy of the valid region
template <typename DstTileData, typename SrcTileData, typename... WaitEvents>
PTO_INST RecordEvent TMOV(DstTileData &dst, SrcTileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    if constexpr (SrcTileData::Loc == TileType::Mat) {
        return TEXTRACT(dst, src, 0, 0);
    } else {
#if PTO_B200_DEVICE_CODE
        if constexpr (SrcTileData::Loc == TileType::Acc) {
            static_assert(DstTileData::Loc == TileType::Vec, "TMOV from an Acc tile goes to a Vec tile");
            const int warp = b200::tid() >> 5, lane = b200::tid() & 31, quarter = warp & 3;
            const int group = warp >> 2, groups = b200::nthreads() >> 7;
            const int row = quarter * 32 + lane;
            const uint32_t taddr = b200::control()->tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + src.addr_;
            typename DstTileData::DType *t = dst.data();
            b200::tc_fence_after();
            for (int c0 = group * 16; c0 < SrcTileData::Cols; c0 += groups * 16) {
                uint32_t r[16];
                b200::tmem_ld16(taddr + c0, r);
                if (row < src.GetValidRow()) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j < src.GetValidCol()) {
                            if constexpr (std::is_same_v<typename DstTileData::DType, typename SrcTileData::DType>) {
                                memcpy(&t[b200::vec_offset<DstTileData>(row, c0 + j)], &r[j], 4);
                            } else {
                                t[b200::vec_offset<DstTileData>(row, c0 + j)] =
                                    b200::convert<typename DstTileData::DType, float>(__uint_as_float(r[j]),
                                                                                      RoundMode::CAST_RINT);
                            }
                        }
                    }
                }
            }
            b200::tc_fence_before();
        } else if constexpr (DstTileData::Loc == TileType::Left || DstTileData::Loc == TileType::Right) {
            static_assert(SrcTileData::Loc == TileType::Vec && SrcTileData::SFractal == SLayout::NoneBox,
                          "TMOV into a matrix operand: from a Mat tile or a plain Vec tile");
            static_assert(SrcTileData::Rows == DstTileData::Rows && SrcTileData::Cols == DstTileData::Cols,
                          "TMOV: shapes differ");
            if constexpr (!b200::is_tc_elem<typename SrcTileData::DType>::value) {
                // 8- and 32-bit operands are multiplied on the CUDA cores from plain row-major tiles
                static_assert(sizeof(typename SrcTileData::DType) == sizeof(typename DstTileData::DType), "TMOV: element sizes differ");
                const typename SrcTileData::DType *s = src.data();
                auto *d = reinterpret_cast<typename SrcTileData::DType *>(b200::arena_of<DstTileData::Loc>() + dst.addr_);
                for (int i = b200::tid_b(), i_step = b200::nthreads_b(); i < DstTileData::Rows * DstTileData::Cols; i += i_step) {
                    const int r = i / DstTileData::Cols, c = i - r * DstTileData::Cols;
                    d[i] = s[b200::vec_offset<SrcTileData>(r, c)];
                }
                dst.pitch_ = 0;
                dst.major_ = b200::kPlain;
                b200::sync_b();
                return {};
            }
            constexpr bool cols_contig = SrcTileData::isRowMajor;
            constexpr int lines = cols_contig ? DstTileData::Rows : DstTileData::Cols;
            constexpr int span = cols_contig ? DstTileData::Cols : DstTileData::Rows;
            constexpr int kCE = 16 / static_cast<int>(sizeof(typename SrcTileData::DType));
            static_assert(span % kCE == 0, "TMOV: the contiguous extent must be a multiple of 16 bytes");
            constexpr int chunks_per_line = span / kCE;
            constexpr uint32_t dst_pitch = static_cast<uint32_t>(lines) * 128u;
            const uint8_t *s = reinterpret_cast<const uint8_t *>(src.data());
            uint8_t *d = b200::arena_of<DstTileData::Loc>() + dst.addr_;
            if (b200::kPipeWarps && b200::tid_b() == 0) {
                b200::held_back()[14] = 1; // an operand tile written through the generic proxy
            }
            for (int q = b200::tid_b(), q_step = b200::nthreads_b(); q < lines * chunks_per_line; q += q_step) {
                const int l = q / chunks_per_line, ch = q - l * chunks_per_line;
                const uint32_t d_off = (ch >> 3) * dst_pitch + l * 128u + (((ch & 7) ^ (l & 7)) << 4);
                *reinterpret_cast<uint4 *>(d + d_off) =
                    *reinterpret_cast<const uint4 *>(s + (static_cast<uint32_t>(l) * span + ch * kCE) * sizeof(typename SrcTileData::DType));
            }
            dst.pitch_ = dst_pitch;
            const bool k_major = (DstTileData::Loc == TileType::Left) ? cols_contig : !cols_contig;
            dst.major_ = k_major ? 0 : 1;
            b200::sync_b();
            return {};
        } else {
            const int vr = src.GetValidRow(), vc = src.GetValidCol();
            for (int i = b200::tid(), i_step = b200::nthreads(); i < vr * vc; i += i_step) {
                const int r = i / vc, c = i - r * vc;
                dst.data()[b200::vec_offset<DstTileData>(r, c)] = src.data()[b200::vec_offset<SrcTileData>(r, c)];
            }
        }
        b200::sync();
#endif
        return {};
    }
}

// ---------------------------------------------------------------- elementwise vector instructions
namespace b200 {
template <typename DstT, typename SrcT, typename F>
PTO_INTERNAL void for_each_valid(DstT &dst, SrcT &src, F f)
{
#if PTO_B200_DEVICE_CODE
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    for (int i = b200::tid(), i_step = b200::nthreads(); i < vr * vc; i += i_step) {
        const int r = i / vc, c = i - r * vc;
        f(dst.data()[vec_offset<DstT>(r, c)], r, c);
    }
    b200::sync();
#endif
}
} // namespace b200

template <typename TileDataD, typename TileDataS, typename... WaitEvents>
PTO_INST RecordEvent TCVT(TileDataD &dst, TileDataS &src, RoundMode mode, WaitEvents &... events)
{
    TSYNC(events...);
    b200::for_each_valid(dst, src, [&](typename TileDataD::DType &d, int r, int c) {
        d = b200::convert<typename TileDataD::DType, typename TileDataS::DType>(
            src.data()[b200::vec_offset<TileDataS>(r, c)], mode);
    });
    return {};
}

template <typename TileDataD, typename TileDataS, typename... WaitEvents>
PTO_INST RecordEvent TCVT(TileDataD &dst, TileDataS &src, RoundMode mode, SaturationMode, WaitEvents &... events)
{
    TSYNC(events...);
    return TCVT(dst, src, mode);
}

template <typename TileData, typename... WaitEvents>
PTO_INST RecordEvent TEXP(TileData &dst, TileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::for_each_valid(dst, dst, [&](typename TileData::DType &d, int r, int c) {
#if PTO_B200_DEVICE_CODE
        d = b200::convert<typename TileData::DType, float>(
            expf(b200::convert<float, typename TileData::DType>(src.data()[b200::vec_offset<TileData>(r, c)],
                                                                RoundMode::CAST_RINT)),
            RoundMode::CAST_RINT);
#endif
    });
    return {};
}

#define PTO_B200_BINARY(NAME, EXPR)                                                                              \
    template <typename TileData, typename TileSrc0, typename TileSrc1, typename... WaitEvents,                   \
              std::enable_if_t<is_tile<TileSrc0>::value && is_tile<TileSrc1>::value, int> = 0>                   \
    PTO_INST RecordEvent NAME(TileData &dst, TileSrc0 &src0, TileSrc1 &src1, WaitEvents &... events)             \
    {                                                                                                            \
        TSYNC(events...);                                                                                        \
        b200::for_each_valid(dst, dst, [&](typename TileData::DType &d, int r, int c) {                          \
            const typename TileData::DType a = src0.data()[b200::vec_offset<TileSrc0>(r, c)];                    \
            const typename TileData::DType b = src1.data()[b200::vec_offset<TileSrc1>(r, c)];                    \
            d = (EXPR);                                                                                          \
        });                                                                                                      \
        return {};                                                                                               \
    }
PTO_B200_BINARY(TADD, a + b)
PTO_B200_BINARY(TSUB, a - b)
PTO_B200_BINARY(TMUL, a *b)
PTO_B200_BINARY(TDIV, a / b)
PTO_B200_BINARY(TMAX, (a < b) ? b : a)
PTO_B200_BINARY(TMIN, (b < a) ? b : a)
#undef PTO_B200_BINARY

#define PTO_B200_SCALAR(NAME, EXPR)                                                                              \
    template <typename TileData, typename... WaitEvents>                                                         \
    PTO_INST RecordEvent NAME(TileData &dst, TileData &src0, typename TileData::DType s, WaitEvents &... events)  \
    {                                                                                                            \
        TSYNC(events...);          \
        b200::for_each_valid(dst, dst, [&](typename TileData::DType &d, int r, int c) {                          \
            const auto a = src0.data()[b200::vec_offset<TileData>(r, c)];                                        \
            d = (EXPR);                                                                                          \
        });                                                                                                      \
        return {};                                                                                               \
    }
PTO_B200_SCALAR(TADDS, a + s)
PTO_B200_SCALAR(TMULS, a *s)
#undef PTO_B200_SCALAR

// dst[r, c] = src0[r, c] op s(r), s(r) read from src1 as the reference's load_row_scalar does: a 1 x R row tile, an
// R x 1 column tile, or element r of the storage otherwise (include/pto/cpu/TRowExpandOp.hpp:21-57)
namespace b200 {
template <typename TileVec>
PTO_INTERNAL typename TileVec::DType row_scalar(TileVec &src1, int r)
{
    const int vr = src1.GetValidRow(), vc = src1.GetValidCol();
    if (vr == 1 && r < vc) {
        return src1.data()[vec_offset<TileVec>(0, r)];
    }
    if (vc == 1 && r < vr) {
        return src1.data()[vec_offset<TileVec>(r, 0)];
    }
    return src1.data()[r % TileVec::Numel];
}
} // namespace b200

#define PTO_B200_ROWEXPAND(NAME, EXPR)                                                                           \
    template <typename TileDst, typename TileSrc1, typename... WaitEvents>                                       \
    PTO_INST RecordEvent NAME(TileDst &dst, TileDst &src0, TileSrc1 &src1, WaitEvents &... events)               \
    {                                                                                                            \
        TSYNC(events...);          \
        b200::for_each_valid(dst, dst, [&](typename TileDst::DType &d, int r, int c) {                           \
            const auto a = src0.data()[b200::vec_offset<TileDst>(r, c)];                                         \
            const auto s = static_cast<typename TileDst::DType>(b200::row_scalar(src1, r));                      \
            d = (EXPR);                                                                                          \
        });                                                                                                      \
        return {};                                                                                               \
    }
PTO_B200_ROWEXPAND(TROWEXPANDSUB, a - s)
PTO_B200_ROWEXPAND(TROWEXPANDMUL, a *s)
PTO_B200_ROWEXPAND(TROWEXPANDDIV, a / s)
PTO_B200_ROWEXPAND(TROWEXPANDADD, a + s)
PTO_B200_ROWEXPAND(TROWEXPANDMAX, (a < s) ? s : a)
PTO_B200_ROWEXPAND(TROWEXPANDMIN, (s < a) ? s : a)
PTO_B200_ROWEXPAND(TROWEXPANDEXPDIF, static_cast<typename TileDst::DType>(exp(static_cast<double>(a - s))))
#undef PTO_B200_ROWEXPAND

// dst[r, c] = src[r, 0]  (include/pto/cpu/TRowExpand.hpp:22-37)
template <typename TileDataDst, typename TileDataSrc, typename... WaitEvents>
PTO_INST RecordEvent TROWEXPAND(TileDataDst &dst, TileDataSrc &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::for_each_valid(dst, dst, [&](typename TileDataDst::DType &d, int r, int) {
        d = static_cast<typename TileDataDst::DType>(src.data()[b200::vec_offset<TileDataSrc>(r, 0)]);
    });
    return {};
}

// ---------------------------------------------------------------- row reductions (one warp per row)
namespace b200 {
template <int kMode, typename TileOut, typename TileIn> // 0 sum, 1 max, 2 min
PTO_INTERNAL void row_reduce(TileOut &dst, TileIn &src)
{
#if PTO_B200_DEVICE_CODE
    using AccT = float;
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    const int warp = b200::tid() >> 5, lane = b200::tid() & 31, warps = b200::nthreads() >> 5;
    for (int r = warp; r < vr; r += warps) {
        AccT acc = kMode == 1 ? -INFINITY : (kMode == 2 ? INFINITY : 0.0f);
        for (int c = lane; c < vc; c += 32) {
            const AccT v = convert<float, typename TileIn::DType>(src.data()[vec_offset<TileIn>(r, c)],
                                                                  RoundMode::CAST_RINT);
            acc = kMode == 1 ? fmaxf(acc, v) : (kMode == 2 ? fminf(acc, v) : acc + v);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const AccT other = __shfl_xor_sync(0xffffffffu, acc, o);
            acc = kMode == 1 ? fmaxf(acc, other) : (kMode == 2 ? fminf(acc, other) : acc + other);
        }
        if (lane == 0) {
            dst.data()[vec_offset<TileOut>(r, 0)] = convert<typename TileOut::DType, float>(acc, RoundMode::CAST_RINT);
        }
    }
    b200::sync();
#endif
}
} // namespace b200

template <typename TileOut, typename TileIn, typename TileTmp, typename... WaitEvents>
PTO_INST RecordEvent TROWMAX(TileOut &dst, TileIn &src, TileTmp &tmp, WaitEvents &... events)
{
    TSYNC(events...);
    b200::row_reduce<1>(dst, src);
    return {};
}

template <typename TileOut, typename TileIn, typename TileTmp, typename... WaitEvents>
PTO_INST RecordEvent TROWSUM(TileOut &dst, TileIn &src, TileTmp &tmp, WaitEvents &... events)
{
    TSYNC(events...);
    b200::row_reduce<0>(dst, src);
    return {};
}

template <typename TileOut, typename TileIn, typename TileTmp, typename... WaitEvents>
PTO_INST RecordEvent TROWMIN(TileOut &dst, TileIn &src, TileTmp &tmp, WaitEvents &... events)
{
    TSYNC(events...);
    b200::row_reduce<2>(dst, src);
    return {};
}

// ---------------------------------------------------------------- column reductions (one thread per column)
// Rows are visited top to bottom, so TCOLSUM adds in the reference's order (include/pto/cpu/TColSum.hpp:19-30,
// TColMax.hpp:19-33, TColMin.hpp); the result goes to row 0 of dst.
namespace b200 {
template <int kMode, typename TileOut, typename TileIn> // 0 sum, 1 max, 2 min
PTO_INTERNAL void col_reduce(TileOut &dst, TileIn &src)
{
#if PTO_B200_DEVICE_CODE
    using T = typename TileOut::DType;
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    for (int c = b200::tid(), c_step = b200::nthreads(); c < vc; c += c_step) {
        T acc = kMode == 0 ? T(0) : static_cast<T>(src.data()[vec_offset<TileIn>(0, c)]);
        for (int r = (kMode == 0 ? 0 : 1); r < vr; ++r) {
            const T v = static_cast<T>(src.data()[vec_offset<TileIn>(r, c)]);
            if (kMode == 0) {
                acc += v;
            } else if (kMode == 1) {
                acc = (v > acc) ? v : acc;
            } else {
                acc = (v < acc) ? v : acc;
            }
        }
        dst.data()[vec_offset<TileOut>(0, c)] = acc;
    }
    b200::sync();
#endif
}
} // namespace b200

template <typename TileOut, typename TileIn, typename... WaitEvents>
PTO_INST RecordEvent TCOLSUM(TileOut &dst, TileIn &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::col_reduce<0>(dst, src);
    return {};
}
template <typename TileOut, typename TileIn, typename TileTmp, typename... WaitEvents>
PTO_INST RecordEvent TCOLSUM(TileOut &dst, TileIn &src, TileTmp &tmp, bool isBinary, WaitEvents &... events)
{
    TSYNC(events...);
    b200::col_reduce<0>(dst, src);
    return {};
}
template <typename TileOut, typename TileIn, typename... WaitEvents>
PTO_INST RecordEvent TCOLMAX(TileOut &dst, TileIn &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::col_reduce<1>(dst, src);
    return {};
}
template <typename TileOut, typename TileIn, typename... WaitEvents>
PTO_INST RecordEvent TCOLMIN(TileOut &dst, TileIn &src, WaitEvents &... events)
{
    TSYNC(events...);
    b200::col_reduce<2>(dst, src);
    return {};
}

// ---------------------------------------------------------------- TFILLPAD (include/pto/cpu/TFillPad.hpp:19-104)
// every element of dst: the source's valid corner is copied, the rest becomes the pad value of dst's type
namespace b200 {
template <typename T, PadValue P>
PTO_INTERNAL T pad_value()
{
    if constexpr (std::is_floating_point_v<T> || std::is_same_v<T, half> || std::is_same_v<T, bfloat16_t>) {
        if constexpr (P == PadValue::Max) {
            return convert<T, float>(INFINITY, RoundMode::CAST_RINT);
        } else if constexpr (P == PadValue::Min) {
            return convert<T, float>(-INFINITY, RoundMode::CAST_RINT);
        } else {
            return convert<T, float>(0.0f, RoundMode::CAST_RINT);
        }
    } else {
        if constexpr (P == PadValue::Max) {
            return std::numeric_limits<T>::max();
        } else if constexpr (P == PadValue::Min) {
            return std::numeric_limits<T>::min();
        } else {
            return T(0);
        }
    }
}
template <typename TileDataDst, typename TileDataSrc>
PTO_INTERNAL void fill_pad(TileDataDst &dst, TileDataSrc &src)
{
    static_assert(TileDataDst::PadVal != PadValue::Null, "TFILLPAD: the destination tile needs a pad value");
    static_assert(sizeof(typename TileDataDst::DType) == sizeof(typename TileDataSrc::DType), "TFILLPAD: element sizes");
#if PTO_B200_DEVICE_CODE
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    const auto pad = pad_value<typename TileDataDst::DType, TileDataDst::PadVal>();
    if (dst.GetValidRow() != 0 && dst.GetValidCol() != 0) {
        for (int i = b200::tid(), i_step = b200::nthreads(); i < TileDataDst::Rows * TileDataDst::Cols; i += i_step) {
            const int r = i / TileDataDst::Cols, c = i - r * TileDataDst::Cols;
            dst.data()[vec_offset<TileDataDst>(r, c)] =
                (r < vr && c < vc) ? static_cast<typename TileDataDst::DType>(src.data()[vec_offset<TileDataSrc>(r, c)]) : pad;
        }
    }
    b200::sync();
#endif
}
} // namespace b200

template <typename DstTileData, typename SrcTileData, typename... WaitEvents>
PTO_INST RecordEvent TFILLPAD(DstTileData &dst, SrcTileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(DstTileData::Cols == SrcTileData::Cols && DstTileData::Rows == SrcTileData::Rows,
                  "TFILLPAD: dst and src have the same rows and columns");
    b200::fill_pad(dst, src);
    return {};
}
template <typename DstTileData, typename SrcTileData, typename... WaitEvents>
PTO_INST RecordEvent TFILLPAD_INPLACE(DstTileData &dst, SrcTileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(DstTileData::Cols == SrcTileData::Cols && DstTileData::Rows == SrcTileData::Rows,
                  "TFILLPAD_INPLACE: dst and src have the same rows and columns");
    b200::fill_pad(dst, src);
    return {};
}
template <typename DstTileData, typename SrcTileData, typename... WaitEvents>
PTO_INST RecordEvent TFILLPAD_EXPAND(DstTileData &dst, SrcTileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(DstTileData::Cols >= SrcTileData::Cols && DstTileData::Rows >= SrcTileData::Rows,
                  "TFILLPAD_EXPAND: dst is at least as large as src");
    b200::fill_pad(dst, src);
    return {};
}

// ---------------------------------------------------------------- TTRANS (include/pto/cpu/TTrans.hpp:17-58)
template <typename TileDataDst, typename TileDataSrc, typename TileDataTmp, typename... WaitEvents>
PTO_INST RecordEvent TTRANS(TileDataDst &dst, TileDataSrc &src, TileDataTmp &tmp, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(TileDataSrc::ValidRow == TileDataDst::ValidCol && TileDataSrc::ValidCol == TileDataDst::ValidRow,
                  "TTRANS: the valid extents of dst are those of src exchanged");
#if PTO_B200_DEVICE_CODE
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    for (int i = b200::tid(), i_step = b200::nthreads(); i < vr * vc; i += i_step) {
        const int c = i / vr, r = i - c * vr; // consecutive threads write consecutive elements of a dst row
        dst.data()[b200::vec_offset<TileDataDst>(c, r)] = src.data()[b200::vec_offset<TileDataSrc>(r, c)];
    }
    b200::sync();
#endif
    return {};
}

// ---------------------------------------------------------------- TTRI (include/pto/cpu/TTRI.hpp:30-77)
// isUpperOrLower 0: one where c <= r + diagonal; 1: one where c >= r + diagonal; zero elsewhere in the valid region
template <typename TileData, int isUpperOrLower, typename... WaitEvents>
PTO_INST RecordEvent TTRI(TileData &dst, int diagonal, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(isUpperOrLower == 0 || isUpperOrLower == 1, "TTRI: isUpperOrLower must be 0 or 1");
    static_assert(TileData::isRowMajor, "TTRI: row-major tiles only");
#if PTO_B200_DEVICE_CODE
    using T = typename TileData::DType;
    const int vr = dst.GetValidRow(), vc = dst.GetValidCol();
    for (int i = b200::tid(), i_step = b200::nthreads(); i < vr * vc; i += i_step) {
        const int r = i / vc, c = i - r * vc;
        const bool in = isUpperOrLower ? (c >= r + diagonal) : (c <= r + diagonal);
        dst.data()[b200::vec_offset<TileData>(r, c)] = in ? b200::convert<T, float>(1.0f, RoundMode::CAST_RINT)
                                                          : b200::convert<T, float>(0.0f, RoundMode::CAST_RINT);
    }
    b200::sync();
#endif
    return {};
}

// ---------------------------------------------------------------- TRESHAPE
// The same bytes under another tile type of the same location and total size.  As on the NPU
// (include/pto/npu/a2a3/TReshape.hpp:21-51 in the reference) the destination is re-bound to the source's storage, so
// that writes through either tile are seen through the other: the reference's streaming softmax relies on this
// (kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:141-165).  The CPU simulation copies the bytes instead
// (include/pto/cpu/TReshape.hpp:18-56); a program that only reads the reshaped tile sees the same values either way.
template <typename TileDataOut, typename TileDataIn, typename... WaitEvents>
PTO_INST RecordEvent TRESHAPE(TileDataOut &dst, TileDataIn &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(TileDataOut::Loc == TileDataIn::Loc, "TRESHAPE: source and target TileType must be the same");
    static_assert(sizeof(typename TileDataOut::DType) * TileDataOut::Rows * TileDataOut::Cols ==
                      sizeof(typename TileDataIn::DType) * TileDataIn::Rows * TileDataIn::Cols,
                  "TRESHAPE: total byte size must match");
    static_assert((TileDataOut::SFractal == SLayout::NoneBox) == (TileDataIn::SFractal == SLayout::NoneBox),
                  "TRESHAPE: cannot reshape between boxed and non-boxed layouts");
    dst.addr_ = src.addr_;
    dst.pitch_ = src.pitch_;
    dst.major_ = src.major_;
    return {};
}

// ---------------------------------------------------------------- TSEL (include/pto/cpu/TSel.hpp:22-57)
// the mask tile's bytes are consumed bit by bit, least significant first, row-major over dst's valid region; the
// mask bytes themselves are walked row by row over the mask tile's valid columns
template <typename TileData, typename MaskTile, typename... WaitEvents>
PTO_INST RecordEvent TSEL(TileData &dst, MaskTile &selMask, TileData &src0, TileData &src1, WaitEvents &... events)
{
    TSYNC(events...);
    const int mask_cols = selMask.GetValidCol();
    const int vc = dst.GetValidCol();
    b200::for_each_valid(dst, dst, [&](typename TileData::DType &d, int r, int c) {
        const int bit_index = r * vc + c;
        const int byte_index = bit_index >> 3;
        const auto byte = static_cast<uint8_t>(
            selMask.data()[b200::vec_offset<MaskTile>(byte_index / mask_cols, byte_index % mask_cols)]);
        const auto off = b200::vec_offset<TileData>(r, c);
        d = ((byte >> (bit_index & 7)) & 1) ? src0.data()[off] : src1.data()[off];
    });
    return {};
}

// ---------------------------------------------------------------- TCMPS / TCMP
namespace b200 {
// include/pto/cpu/TCmps.hpp:23-52: EQ / NE look at |a - b| in double against 1e-9
template <typename T>
PTO_INTERNAL uint8_t cmps_call(T a, T b, CmpMode mode)
{
    const double diff = static_cast<double>(convert<float, T>(a, RoundMode::CAST_RINT)) -
                        static_cast<double>(convert<float, T>(b, RoundMode::CAST_RINT));
    const double mag = diff < 0 ? -diff : diff;
    switch (mode) {
        case CmpMode::NE: return mag > 1e-9;
        case CmpMode::LT: return a < b;
        case CmpMode::GT: return a > b;
        case CmpMode::GE: return a >= b;
        case CmpMode::LE: return a <= b;
        default: return mag < 1e-9;
    }
}
} // namespace b200

// One bit per element of src0's whole tile (zero outside its valid region), eight to a byte, least significant first,
// Cols / 8 bytes per tile row; byte number i * dstValidCol + j of that stream lands at element offset
// i * SrcCols + j of dst's storage, exactly as the simulation writes it (include/pto/cpu/TCmps.hpp:54-91).
template <typename TileDataDst, typename TileDataSrc, typename T, typename... WaitEvents>
PTO_INST RecordEvent TCMPS(TileDataDst &dst, TileDataSrc &src0, T src1, CmpMode cmpMode, WaitEvents &... events)
{
    TSYNC(events...);
#if PTO_B200_DEVICE_CODE
    constexpr int H = TileDataSrc::Rows, W = TileDataSrc::Cols;
    constexpr int bytes_per_row = W / 8;
    const int svr = src0.GetValidRow(), svc = src0.GetValidCol();
    const int dvr = dst.GetValidRow(), dvc = dst.GetValidCol();
    const auto scalar = static_cast<typename TileDataSrc::DType>(src1);
    for (int n = b200::tid(), n_step = b200::nthreads(); n < dvr * dvc; n += n_step) {
        if (n >= H * bytes_per_row) {
            break;
        }
        const int h = n / bytes_per_row, k = n - h * bytes_per_row;
        uint32_t byte = 0;
        for (int bit = 0; bit < 8; ++bit) {
            const int c = k * 8 + bit;
            if (h < svr && c < svc) {
                byte |= static_cast<uint32_t>(b200::cmps_call(src0.data()[h * TileDataSrc::RowStride + c], scalar, cmpMode))
                        << bit;
            }
        }
        const int i = n / dvc, j = n - i * dvc;
        dst.data()[i * W + j] = static_cast<typename TileDataDst::DType>(byte);
    }
    b200::sync();
#endif
    return {};
}

// the simulation's TCMP: 1 or 0 in the operands' type (include/pto/cpu/ElementTileOp.h:177-184, ElementOp.h:227-254)
template <typename TileDataDst, typename TileDataSrc, typename... WaitEvents>
PTO_INST RecordEvent TCMP(TileDataDst &dst, TileDataSrc &src0, TileDataSrc &src1, CmpMode cmpMode, WaitEvents &... events)
{
    TSYNC(events...);
    b200::for_each_valid(dst, dst, [&](typename TileDataDst::DType &d, int r, int c) {
        const auto a = src0.data()[b200::vec_offset<TileDataSrc>(r, c)];
        const auto b = src1.data()[b200::vec_offset<TileDataSrc>(r, c)];
        bool res;
        switch (cmpMode) {
            case CmpMode::NE: res = a != b; break;
            case CmpMode::GT: res = a > b; break;
            case CmpMode::LT: res = a < b; break;
            case CmpMode::GE: res = a >= b; break;
            case CmpMode::LE: res = a <= b; break;
            default: res = a == b; break;
        }
        d = static_cast<typename TileDataDst::DType>(res ? 1 : 0);
    });
    return {};
}

// ---------------------------------------------------------------- TGATHER
// index form (include/pto/cpu/TGather.hpp:68-100): out-of-range and negative indices give 0
template <typename TileDataD, typename TileDataS0, typename TileDataS1, typename... WaitEvents>
PTO_INST RecordEvent TGATHER(TileDataD &dst, TileDataS0 &src0, TileDataS1 &src1, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(sizeof(typename TileDataS1::DType) == 4, "TGATHER: 32-bit indices");
    static_assert(std::is_same_v<typename TileDataD::DType, typename TileDataS0::DType>, "TGATHER: types differ");
    b200::for_each_valid(dst, dst, [&](typename TileDataD::DType &d, int r, int c) {
        const int64_t raw = static_cast<int64_t>(src1.data()[b200::vec_offset<TileDataS1>(r, c)]);
        if (raw < 0 || raw >= static_cast<int64_t>(TileDataS0::Numel)) {
            d = typename TileDataD::DType(0);
        } else {
            const int sr = static_cast<int>(raw / TileDataS0::Cols), sc = static_cast<int>(raw % TileDataS0::Cols);
            d = src0.data()[b200::vec_offset<TileDataS0>(sr, sc)];
        }
    });
    return {};
}

// mask form (include/pto/cpu/TGather.hpp:102-129): selected columns of every row, packed contiguously
template <typename DstTileData, typename SrcTileData, MaskPattern maskPattern, typename... WaitEvents>
PTO_INST RecordEvent TGATHER(DstTileData &dst, SrcTileData &src, WaitEvents &... events)
{
    TSYNC(events...);
    static_assert(DstTileData::isRowMajor && SrcTileData::isRowMajor, "TGATHER (mask): row-major tiles");
#if PTO_B200_DEVICE_CODE
    constexpr int div = (maskPattern == MaskPattern::P1111) ? 1
                        : ((maskPattern == MaskPattern::P0101 || maskPattern == MaskPattern::P1010) ? 2 : 4);
    constexpr int off = (maskPattern == MaskPattern::P1010 || maskPattern == MaskPattern::P0010)   ? 1
                        : (maskPattern == MaskPattern::P0100)                                      ? 2
                        : (maskPattern == MaskPattern::P1000)                                      ? 3
                                                                                                   : 0;
    const int vr = src.GetValidRow(), vc = src.GetValidCol();
    const int per_row = (vc - off + div - 1) / div;
    for (int i = b200::tid(), i_step = b200::nthreads(); i < vr * per_row; i += i_step) {
        const int r = i / per_row, k = i - r * per_row;
        dst.data()[i] = src.data()[b200::vec_offset<SrcTileData>(r, k * div + off)];
    }
    b200::sync();
#endif
    return {};
}

} // namespace pto
