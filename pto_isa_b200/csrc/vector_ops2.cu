// Second batch of vector tile ops as HBM-streaming kernels for sm_100a: the row-expand family, TROWMIN, the column
// reductions, TFILLPAD, TTRANS, TSEL, TCMPS and TCMP.  All are memory bound: 128-bit accesses where the shape
// allows, grids sized from the element count, enough bytes in flight per SM to cover the HBM latency.
// Semantics follow the reference's CPU simulation (paths relative to the reference root):
//   TROWEXPAND*   include/pto/cpu/TRowExpandOp.hpp:38-57, TRowExpand.hpp:22-37, ElementOp.h:85-270
//                 (max / min are std::max / std::min, EXPDIF is float(exp(double(a - b))))
//   TROWMIN       include/pto/cpu/TRowMin.hpp:21-41
//   TCOLSUM/MAX/MIN  include/pto/cpu/TColSum.hpp:19-30, TColMax.hpp:19-33, TColMin.hpp
//   TFILLPAD      include/pto/cpu/TFillPad.hpp:19-49
//   TTRANS        include/pto/cpu/TTrans.hpp:17-45 (plain layouts)
//   TSEL          include/pto/cpu/TSel.hpp:22-46 (mask bits consumed least significant first, row-major)
//   TCMPS / TCMP  include/pto/cpu/TCmps.hpp:23-91, ElementOp.h:227-254
#include "ptx.cuh"
#include "internal.h"

namespace pto_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kRowWarps = 4; // rows (one warp each) per block of the row reductions

bool aligned16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// 0 add, 1 sub, 2 mul, 3 div, 4 max, 5 min, 6 expdif, 7 second operand (plain expand)
__device__ __forceinline__ float elem_op(int op, float a, float b)
{
    switch (op) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return (a < b) ? b : a;
        case 5: return (b < a) ? b : a;
        case 6: return static_cast<float>(exp(static_cast<double>(a - b)));
        default: return b;
    }
}

// ---------------------------------------------------------------- row-expand family
// dst[r, c] = a[r, c] op s[r]; four columns per thread when the rows are 16-byte multiples
template <bool kVec>
__global__ void __launch_bounds__(kThreads) trowexpand_kernel(const float *__restrict__ a, const float *__restrict__ s,
                                                              float *__restrict__ dst, int rows, int cols, int op)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (kVec) {
        const int vcols = cols >> 2;
        const int64_t nvec = static_cast<int64_t>(rows) * vcols;
        // two independent 16-byte loads in flight per thread
        for (int64_t i = tid; i < nvec; i += 2 * stride) {
            const int64_t j = i + stride;
            const bool two = j < nvec;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f), w = v;
            if (op != 7) {
                v = ld_stream_f4(reinterpret_cast<const float4 *>(a) + i);
                if (two) {
                    w = ld_stream_f4(reinterpret_cast<const float4 *>(a) + j);
                }
            }
            const float sv = __ldg(s + i / vcols);
            const float sw = two ? __ldg(s + j / vcols) : 0.0f;
            v.x = elem_op(op, v.x, sv);
            v.y = elem_op(op, v.y, sv);
            v.z = elem_op(op, v.z, sv);
            v.w = elem_op(op, v.w, sv);
            st_stream_f4(reinterpret_cast<float4 *>(dst) + i, v);
            if (two) {
                w.x = elem_op(op, w.x, sw);
                w.y = elem_op(op, w.y, sw);
                w.z = elem_op(op, w.z, sw);
                w.w = elem_op(op, w.w, sw);
                st_stream_f4(reinterpret_cast<float4 *>(dst) + j, w);
            }
        }
    } else {
        const int64_t n = static_cast<int64_t>(rows) * cols;
        for (int64_t i = tid; i < n; i += stride) {
            dst[i] = elem_op(op, op != 7 ? a[i] : 0.0f, s[i / cols]);
        }
    }
}

// ---------------------------------------------------------------- TROWMIN: one warp per row
__global__ void __launch_bounds__(kThreads) trowmin_kernel(const float *__restrict__ src, float *__restrict__ dst, int rows,
                                                           int cols, int64_t row_stride)
{
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
        const float *p = src + static_cast<int64_t>(row) * row_stride;
        float acc = INFINITY;
        int c = 0;
        if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
            const int nvec = cols >> 2;
            int i = lane;
            for (; i + 96 < nvec; i += 128) { // four 16-byte loads in flight per lane
                const float4 v0 = ld_stream_f4(reinterpret_cast<const float4 *>(p) + i);
                const float4 v1 = ld_stream_f4(reinterpret_cast<const float4 *>(p) + i + 32);
                const float4 v2 = ld_stream_f4(reinterpret_cast<const float4 *>(p) + i + 64);
                const float4 v3 = ld_stream_f4(reinterpret_cast<const float4 *>(p) + i + 96);
                acc = fminf(acc, fminf(fminf(fminf(v0.x, v0.y), fminf(v0.z, v0.w)), fminf(fminf(v1.x, v1.y), fminf(v1.z, v1.w))));
                acc = fminf(acc, fminf(fminf(fminf(v2.x, v2.y), fminf(v2.z, v2.w)), fminf(fminf(v3.x, v3.y), fminf(v3.z, v3.w))));
            }
            for (; i < nvec; i += 32) {
                const float4 v = ld_stream_f4(reinterpret_cast<const float4 *>(p) + i);
                acc = fminf(acc, fminf(fminf(v.x, v.y), fminf(v.z, v.w)));
            }
            c = nvec << 2;
        }
        for (int i = c + lane; i < cols; i += 32) {
            acc = fminf(acc, p[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc = fminf(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        }
        if (lane == 0) {
            dst[row] = acc;
        }
    }
}

// ---------------------------------------------------------------- column reductions
// A block of 32 warps owns a strip of 32 columns: a warp reads one 128-byte row segment per load, eight rows in
// flight (32 KiB per block, enough to cover the HBM latency), then the 32 warps' partial results are combined in
// a fixed order (deterministic; for the sum not the reference's top-to-bottom order).
constexpr int kColWarps = 32;
constexpr int kColUnroll = 8;

template <int kOp> // 0 sum, 4 max, 5 min
__device__ __forceinline__ float col_op(float a, float b)
{
    return kOp == 0 ? a + b : (kOp == 4 ? fmaxf(a, b) : fminf(a, b));
}

template <int kOp>
__global__ void __launch_bounds__(kColWarps * 32) tcolreduce_kernel(const float *__restrict__ src, float *__restrict__ dst,
                                                                    int rows, int cols, int64_t row_stride)
{
    __shared__ float part[kColWarps][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float ident = kOp == 0 ? 0.0f : (kOp == 4 ? -INFINITY : INFINITY);
    for (int c0 = blockIdx.x * 32; c0 < cols; c0 += gridDim.x * 32) {
        const int c = c0 + lane;
        float acc[kColUnroll];
#pragma unroll
        for (int u = 0; u < kColUnroll; ++u) {
            acc[u] = ident;
        }
        if (c < cols) {
            const float *p = src + c;
            for (int r = warp; r < rows; r += kColWarps * kColUnroll) {
#pragma unroll
                for (int u = 0; u < kColUnroll; ++u) {
                    const int rr = r + u * kColWarps;
                    if (rr < rows) {
                        acc[u] = col_op<kOp>(acc[u], __ldg(p + static_cast<int64_t>(rr) * row_stride));
                    }
                }
            }
        }
        float v = acc[0];
#pragma unroll
        for (int u = 1; u < kColUnroll; ++u) {
            v = col_op<kOp>(v, acc[u]);
        }
        part[warp][lane] = v;
        __syncthreads();
        if (warp == 0 && c < cols) {
            float t = part[0][lane];
#pragma unroll
            for (int w = 1; w < kColWarps; ++w) {
                t = col_op<kOp>(t, part[w][lane]);
            }
            dst[c] = t;
        }
        __syncthreads();
    }
}

// Two-pass form for large tiles (needs a caller-provided workspace of segments * cols floats): the rows are cut
// into segments so that strips x segments blocks fill the GPU in one wave; a block of 8 warps reduces 128 columns (one 512-byte
// row piece per warp load, four in flight) of one segment and writes a partial row, the second pass combines the
// segments top to bottom.  Deterministic; the sum's order is fixed but not the reference's.
constexpr int kSegWarps = 8;
constexpr int kSegUnroll = 4;
constexpr int kSegBlocksPerSm = 6; // 40 registers x 256 threads: six blocks fit the register file, not eight

template <int kOp>
__device__ __forceinline__ float4 col_op4(float4 a, float4 b)
{
    return make_float4(col_op<kOp>(a.x, b.x), col_op<kOp>(a.y, b.y), col_op<kOp>(a.z, b.z), col_op<kOp>(a.w, b.w));
}

template <int kOp>
__global__ void __launch_bounds__(kSegWarps * 32, kSegBlocksPerSm) tcolreduce_seg_kernel(const float *__restrict__ src,
                                                                         float *__restrict__ partial, int rows, int cols,
                                                                         int64_t row_stride, int rows_per_seg)
{
    __shared__ float4 part[kSegWarps][32];
    // the second pass may be scheduled as soon as this grid's blocks are all resident; it waits for this grid's
    // completion (and its writes) before it reads a partial
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float id1 = kOp == 0 ? 0.0f : (kOp == 4 ? -INFINITY : INFINITY);
    const float4 ident = make_float4(id1, id1, id1, id1);
    const int c = (blockIdx.x * 32 + lane) * 4; // cols is a multiple of 4
    const int r_begin = blockIdx.y * rows_per_seg;
    const int r_end = min(rows, r_begin + rows_per_seg);
    float4 acc[kSegUnroll];
#pragma unroll
    for (int u = 0; u < kSegUnroll; ++u) {
        acc[u] = ident;
    }
    if (c < cols) {
        const float *p = src + c;
        for (int r = r_begin + warp; r < r_end; r += kSegWarps * kSegUnroll) {
#pragma unroll
            for (int u = 0; u < kSegUnroll; ++u) {
                const int rr = r + u * kSegWarps;
                if (rr < r_end) {
                    acc[u] = col_op4<kOp>(acc[u], ld_stream_f4(reinterpret_cast<const float4 *>(
                                                      p + static_cast<int64_t>(rr) * row_stride)));
                }
            }
        }
    }
    float4 v = col_op4<kOp>(col_op4<kOp>(acc[0], acc[1]), col_op4<kOp>(acc[2], acc[3]));
    part[warp][lane] = v;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float4 t = part[0][lane];
#pragma unroll
        for (int w = 1; w < kSegWarps; ++w) {
            t = col_op4<kOp>(t, part[w][lane]);
        }
        *reinterpret_cast<float4 *>(partial + static_cast<int64_t>(blockIdx.y) * cols + c) = t;
    }
}

// second pass: a block per 32 columns, warp w folds segments w, w + 8, ... (independent loads), then the eight
// warps' values are folded in warp order: a fixed order for every column
template <int kOp>
__global__ void __launch_bounds__(kThreads) tcolreduce_final_kernel(const float *__restrict__ partial,
                                                                    float *__restrict__ dst, int cols, int segments)
{
    __shared__ float part[kThreads / 32][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 32 + lane;
    float t = kOp == 0 ? 0.0f : (kOp == 4 ? -INFINITY : INFINITY);
    asm volatile("griddepcontrol.wait;" ::: "memory"); // first pass complete and visible (no-op in a plain launch)
    if (c < cols) {
#pragma unroll 4
        for (int sgm = warp; sgm < segments; sgm += kThreads / 32) {
            t = col_op<kOp>(t, __ldg(partial + static_cast<int64_t>(sgm) * cols + c));
        }
    }
    part[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float v = part[0][lane];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) {
            v = col_op<kOp>(v, part[w][lane]);
        }
        dst[c] = v;
    }
}

// ---------------------------------------------------------------- TFILLPAD
// dst[r, c] = (r < valid_rows && c < valid_cols) ? src[r, c] : pad; the source is only read inside the valid corner
template <typename T, int kVec> // kVec elements (16 bytes) per thread, or 1
__global__ void __launch_bounds__(kThreads) tfillpad_kernel(const T *__restrict__ src, T *__restrict__ dst, int rows,
                                                            int cols, int valid_rows, int valid_cols, T pad)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int vcols = cols / kVec;
    const int64_t n = static_cast<int64_t>(rows) * vcols;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int r = static_cast<int>(i / vcols);
        const int c = static_cast<int>(i - static_cast<int64_t>(r) * vcols) * kVec;
        if (kVec == 1) {
            dst[i] = (r < valid_rows && c < valid_cols) ? src[i] : pad;
        } else {
            union {
                uint4 v;
                T e[kVec];
            } u;
            if (r < valid_rows && c < valid_cols) {
                u.v = *reinterpret_cast<const uint4 *>(src + static_cast<int64_t>(r) * cols + c);
#pragma unroll
                for (int j = 0; j < kVec; ++j) {
                    if (c + j >= valid_cols) {
                        u.e[j] = pad;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < kVec; ++j) {
                    u.e[j] = pad;
                }
            }
            st_stream_u4(reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(r) * cols + c), u.v);
        }
    }
}

// ---------------------------------------------------------------- TTRANS
// 32 x 32 (4-byte) or 64 x 64 (2-byte) element tiles through padded shared memory; both the reads and the writes
// are 128-byte row segments
template <typename T>
__global__ void __launch_bounds__(256) ttrans_kernel(const T *__restrict__ src, T *__restrict__ dst, int rows, int cols)
{
    constexpr int kTile = 128 / sizeof(T); // 32 or 64 elements = 128 bytes
    __shared__ T tile[kTile][kTile + (sizeof(T) == 4 ? 1 : 2)];
    const int tx = threadIdx.x % kTile, ty = threadIdx.x / kTile; // ty in [0, 256 / kTile)
    constexpr int kRowsPerPass = 256 / kTile;
    const int tiles_c = (cols + kTile - 1) / kTile;
    const int tiles_r = (rows + kTile - 1) / kTile;
    for (int64_t t = blockIdx.x; t < static_cast<int64_t>(tiles_r) * tiles_c; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_c) * kTile, c0 = static_cast<int>(t % tiles_c) * kTile;
#pragma unroll 4
        for (int j = ty; j < kTile; j += kRowsPerPass) {
            const int r = r0 + j, c = c0 + tx;
            if (r < rows && c < cols) {
                tile[j][tx] = src[static_cast<int64_t>(r) * cols + c];
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int j = ty; j < kTile; j += kRowsPerPass) {
            const int c = c0 + j, r = r0 + tx; // dst[c, r]
            if (c < cols && r < rows) {
                dst[static_cast<int64_t>(c) * rows + r] = tile[tx][j];
            }
        }
        __syncthreads();
    }
}

// 4-byte elements, rows and cols multiples of 4, 16-byte aligned operands: 64 x 64 tiles, every thread moves a 4 x 4
// block.  It loads four 16-byte row pieces (256-byte row segments per half warp, 16 KB in flight per block),
// transposes the block in registers, writes the four transposed pieces into shared memory whose 16-byte chunks are
// XOR-swizzled by (row / 4) % 8 - the stores of a quarter warp go to rows 4 apart, the loads to one row, both hit eight
// different bank groups - and stores 16-byte pieces of the transposed rows, again 256-byte segments.
__global__ void __launch_bounds__(256) ttrans4_vec_kernel(const float *__restrict__ src, float *__restrict__ dst,
                                                          int rows, int cols)
{
    __shared__ float4 tile[64][16]; // [transposed row][swizzled chunk]
    const int cg = threadIdx.x & 15, rg = threadIdx.x >> 4; // column group / row group of the 4 x 4 block
    const int tiles_c = (cols + 63) / 64;
    const int tiles_r = (rows + 63) / 64;
    for (int64_t t = blockIdx.x; t < static_cast<int64_t>(tiles_r) * tiles_c; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_c) * 64, c0 = static_cast<int>(t % tiles_c) * 64;
        const int r = r0 + 4 * rg, c = c0 + 4 * cg;
        float4 in[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            in[j] = (r + j < rows && c < cols)
                        ? ld_stream_f4(reinterpret_cast<const float4 *>(src + static_cast<int64_t>(r + j) * cols + c))
                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        tile[4 * cg + 0][rg ^ (cg & 7)] = make_float4(in[0].x, in[1].x, in[2].x, in[3].x);
        tile[4 * cg + 1][rg ^ (cg & 7)] = make_float4(in[0].y, in[1].y, in[2].y, in[3].y);
        tile[4 * cg + 2][rg ^ (cg & 7)] = make_float4(in[0].z, in[1].z, in[2].z, in[3].z);
        tile[4 * cg + 3][rg ^ (cg & 7)] = make_float4(in[0].w, in[1].w, in[2].w, in[3].w);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tr = rg + 16 * j;                   // transposed row inside the tile = source column
            const int out_r = c0 + tr, out_c = r0 + 4 * cg; // dst[out_r, out_c .. out_c + 3]
            if (out_r < cols && out_c < rows) {
                st_stream_f4(reinterpret_cast<float4 *>(dst + static_cast<int64_t>(out_r) * rows + out_c),
                             tile[tr][cg ^ ((tr >> 2) & 7)]);
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------- TTRI: triangular 0 / 1 tile
// lower: one for c <= r + diagonal; upper: one for c >= r + diagonal (include/pto/cpu/TTRI.hpp:30-77)
template <typename T>
__global__ void __launch_bounds__(kThreads) ttri_kernel(T *__restrict__ dst, int rows, int cols, int diagonal, int upper,
                                                        T one)
{
    const int64_t n = static_cast<int64_t>(rows) * cols;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int r = static_cast<int>(i / cols), c = static_cast<int>(i - static_cast<int64_t>(r) * cols);
        const bool in = upper ? (c >= r + diagonal) : (c <= r + diagonal);
        dst[i] = in ? one : T(0);
    }
}

// ---------------------------------------------------------------- TSEL: one mask byte (8 elements) per thread
template <typename T>
__global__ void __launch_bounds__(kThreads) tsel_kernel(const uint8_t *__restrict__ mask, const T *__restrict__ a,
                                                        const T *__restrict__ b, T *__restrict__ dst, int64_t n,
                                                        bool vec_ok)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t nbytes = (n + 7) >> 3;
    constexpr int kVecs = 8 * sizeof(T) / 16; // uint4 per 8 elements: 2 (4-byte) or 1 (2-byte)
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        const uint32_t m = mask[i];
        const int64_t e0 = i << 3;
        if (vec_ok && e0 + 8 <= n) {
            union {
                uint4 v[kVecs];
                T e[8];
            } ua, ub;
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                ua.v[q] = *(reinterpret_cast<const uint4 *>(a + e0) + q);
                ub.v[q] = *(reinterpret_cast<const uint4 *>(b + e0) + q);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ua.e[j] = ((m >> j) & 1u) ? ua.e[j] : ub.e[j];
            }
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
                st_stream_u4(reinterpret_cast<uint4 *>(dst + e0) + q, ua.v[q]);
            }
        } else {
            for (int j = 0; j < 8 && e0 + j < n; ++j) {
                dst[e0 + j] = ((m >> j) & 1u) ? a[e0 + j] : b[e0 + j];
            }
        }
    }
}

// ---------------------------------------------------------------- TCMPS / TCMP
// EQ 0, NE 1, LT 2, LE 3, GT 4, GE 5
__device__ __forceinline__ uint32_t cmps_call(float a, float b, int mode)
{
    switch (mode) {
        case 1: return fabs(static_cast<double>(a) - static_cast<double>(b)) > 1e-9;
        case 2: return a < b;
        case 3: return a <= b;
        case 4: return a > b;
        case 5: return a >= b;
        default: return fabs(static_cast<double>(a) - static_cast<double>(b)) < 1e-9;
    }
}

// one output byte (8 elements, least significant bit first) per thread
__global__ void __launch_bounds__(kThreads) tcmps_kernel(const float *__restrict__ src, float scalar,
                                                         uint8_t *__restrict__ dst, int64_t nbytes, int mode, bool vec_ok)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        float e[8];
        if (vec_ok) {
            const float4 v0 = ld_stream_f4(reinterpret_cast<const float4 *>(src) + 2 * i);
            const float4 v1 = ld_stream_f4(reinterpret_cast<const float4 *>(src) + 2 * i + 1);
            e[0] = v0.x, e[1] = v0.y, e[2] = v0.z, e[3] = v0.w, e[4] = v1.x, e[5] = v1.y, e[6] = v1.z, e[7] = v1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                e[j] = src[8 * i + j];
            }
        }
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            byte |= cmps_call(e[j], scalar, mode) << j;
        }
        dst[i] = static_cast<uint8_t>(byte);
    }
}

__device__ __forceinline__ float cmp_call(float a, float b, int mode)
{
    bool r;
    switch (mode) {
        case 1: r = a != b; break;
        case 2: r = a < b; break;
        case 3: r = a <= b; break;
        case 4: r = a > b; break;
        case 5: r = a >= b; break;
        default: r = a == b; break;
    }
    return r ? 1.0f : 0.0f;
}

__global__ void __launch_bounds__(kThreads) tcmp_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                                        float *__restrict__ dst, int64_t n, int mode, bool vec_ok)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = n >> 2;
        for (int64_t i = tid; i < nvec; i += stride) {
            const float4 x = ld_stream_f4(reinterpret_cast<const float4 *>(a) + i);
            const float4 y = ld_stream_f4(reinterpret_cast<const float4 *>(b) + i);
            st_stream_f4(reinterpret_cast<float4 *>(dst) + i,
                         make_float4(cmp_call(x.x, y.x, mode), cmp_call(x.y, y.y, mode), cmp_call(x.z, y.z, mode),
                                     cmp_call(x.w, y.w, mode)));
        }
        done = nvec << 2;
    }
    for (int64_t i = done + tid; i < n; i += stride) {
        dst[i] = cmp_call(a[i], b[i], mode);
    }
}

} // namespace

// ---------------------------------------------------------------- launchers (called from the C ABI)

int launch_trowexpand(const float *a, const float *row_scalar, float *dst, int rows, int cols, int op,
                      cudaStream_t stream)
{
    if (rows == 0 || cols == 0) {
        return kOk;
    }
    const bool vec = (cols % 4 == 0) && aligned16(dst) && (op == 7 || aligned16(a));
    if (vec) {
        trowexpand_kernel<true><<<grid_for(static_cast<int64_t>(rows) * (cols >> 3) + 1, kThreads), kThreads, 0, stream>>>(
            a, row_scalar, dst, rows, cols, op);
    } else {
        trowexpand_kernel<false><<<grid_for(static_cast<int64_t>(rows) * cols, kThreads), kThreads, 0, stream>>>(
            a, row_scalar, dst, rows, cols, op);
    }
    return check_launch();
}

int launch_trowmin(const float *src, float *dst, int rows, int cols, int64_t row_stride, cudaStream_t stream)
{
    if (rows == 0) {
        return kOk;
    }
    trowmin_kernel<<<grid_for(rows, kRowWarps), kRowWarps * 32, 0, stream>>>(src, dst, rows, cols, row_stride);
    return check_launch();
}

// segments the two-pass form cuts `rows` into (1: the single-pass kernel is used)
int tcolreduce_segments(int rows, int cols)
{
    if ((cols & 3) != 0 || rows < 256) {
        return 1;
    }
    const int strips = (cols + 127) / 128;
    int segs = kSegBlocksPerSm * sm_count() / strips; // rounded down: all blocks resident at once, no second wave
    const int max_segs = rows / 64; // at least 64 rows per segment
    if (segs > max_segs) {
        segs = max_segs;
    }
    return segs < 2 ? 1 : segs;
}

int launch_tcolreduce(const float *src, float *dst, int rows, int cols, int64_t row_stride, int op, float *workspace,
                      size_t workspace_bytes, cudaStream_t stream)
{
    if (cols == 0) {
        return kOk;
    }
    const int segs = tcolreduce_segments(rows, cols);
    const bool two_pass = segs > 1 && workspace != nullptr &&
                          workspace_bytes >= static_cast<size_t>(segs) * cols * sizeof(float) && aligned16(src) &&
                          aligned16(workspace) && (row_stride & 3) == 0;
    if (two_pass) {
        const int rows_per_seg = (rows + segs - 1) / segs;
        const dim3 grid((cols + 127) / 128, segs);
        const int fgrid = (cols + 31) / 32;
        // the second pass is launched with programmatic stream serialization: its blocks are scheduled while the
        // first pass drains and wait on the device for its completion, which hides the launch latency between the two
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(fgrid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        const float *partial = workspace;
        cudaError_t err = cudaSuccess;
        switch (op) {
            case 0:
                tcolreduce_seg_kernel<0><<<grid, kSegWarps * 32, 0, stream>>>(src, workspace, rows, cols, row_stride, rows_per_seg);
                err = cudaLaunchKernelEx(&cfg, tcolreduce_final_kernel<0>, partial, dst, cols, segs);
                break;
            case 4:
                tcolreduce_seg_kernel<4><<<grid, kSegWarps * 32, 0, stream>>>(src, workspace, rows, cols, row_stride, rows_per_seg);
                err = cudaLaunchKernelEx(&cfg, tcolreduce_final_kernel<4>, partial, dst, cols, segs);
                break;
            case 5:
                tcolreduce_seg_kernel<5><<<grid, kSegWarps * 32, 0, stream>>>(src, workspace, rows, cols, row_stride, rows_per_seg);
                err = cudaLaunchKernelEx(&cfg, tcolreduce_final_kernel<5>, partial, dst, cols, segs);
                break;
            default: return kErrBadArgument;
        }
        if (err != cudaSuccess) {
            return check_cuda(err, "cudaLaunchKernelEx");
        }
        return check_launch();
    }
    const int strips = (cols + 31) / 32;
    const int grid = strips < 4 * sm_count() ? strips : 4 * sm_count();
    switch (op) {
        case 0: tcolreduce_kernel<0><<<grid, kColWarps * 32, 0, stream>>>(src, dst, rows, cols, row_stride); break;
        case 4: tcolreduce_kernel<4><<<grid, kColWarps * 32, 0, stream>>>(src, dst, rows, cols, row_stride); break;
        case 5: tcolreduce_kernel<5><<<grid, kColWarps * 32, 0, stream>>>(src, dst, rows, cols, row_stride); break;
        default: return kErrBadArgument;
    }
    return check_launch();
}

int launch_tfillpad(const void *src, void *dst, int rows, int cols, int valid_rows, int valid_cols, uint32_t pad,
                    int elem_bytes, cudaStream_t stream)
{
    if (rows == 0 || cols == 0) {
        return kOk;
    }
    const int vec = 16 / elem_bytes;
    const bool vec_ok = (cols % vec == 0) && aligned16(src) && aligned16(dst);
    const int64_t items = static_cast<int64_t>(rows) * (vec_ok ? cols / vec : cols);
    const int grid = grid_for(items, kThreads);
    if (elem_bytes == 4) {
        if (vec_ok) {
            tfillpad_kernel<uint32_t, 4><<<grid, kThreads, 0, stream>>>(static_cast<const uint32_t *>(src),
                                                                        static_cast<uint32_t *>(dst), rows, cols,
                                                                        valid_rows, valid_cols, pad);
        } else {
            tfillpad_kernel<uint32_t, 1><<<grid, kThreads, 0, stream>>>(static_cast<const uint32_t *>(src),
                                                                        static_cast<uint32_t *>(dst), rows, cols,
                                                                        valid_rows, valid_cols, pad);
        }
    } else {
        const uint16_t p16 = static_cast<uint16_t>(pad);
        if (vec_ok) {
            tfillpad_kernel<uint16_t, 8><<<grid, kThreads, 0, stream>>>(static_cast<const uint16_t *>(src),
                                                                        static_cast<uint16_t *>(dst), rows, cols,
                                                                        valid_rows, valid_cols, p16);
        } else {
            tfillpad_kernel<uint16_t, 1><<<grid, kThreads, 0, stream>>>(static_cast<const uint16_t *>(src),
                                                                        static_cast<uint16_t *>(dst), rows, cols,
                                                                        valid_rows, valid_cols, p16);
        }
    }
    return check_launch();
}

int launch_ttrans(const void *src, void *dst, int rows, int cols, int elem_bytes, cudaStream_t stream)
{
    if (rows == 0 || cols == 0) {
        return kOk;
    }
    const int tile = 128 / elem_bytes;
    const int64_t tiles = static_cast<int64_t>((rows + tile - 1) / tile) * ((cols + tile - 1) / tile);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const int grid = static_cast<int>(tiles < cap ? tiles : cap);
    if (elem_bytes == 4 && (rows & 3) == 0 && (cols & 3) == 0 && aligned16(src) && aligned16(dst)) {
        const int64_t tiles64 = static_cast<int64_t>((rows + 63) / 64) * ((cols + 63) / 64);
        const int64_t cap64 = static_cast<int64_t>(sm_count()) * 8;
        ttrans4_vec_kernel<<<static_cast<int>(tiles64 < cap64 ? tiles64 : cap64), 256, 0, stream>>>(
            static_cast<const float *>(src), static_cast<float *>(dst), rows, cols);
    } else if (elem_bytes == 4) {
        ttrans_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t *>(src), static_cast<uint32_t *>(dst),
                                                          rows, cols);
    } else {
        ttrans_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t *>(src), static_cast<uint16_t *>(dst),
                                                          rows, cols);
    }
    return check_launch();
}

int launch_ttri(void *dst, int rows, int cols, int diagonal, int upper, uint32_t one_bits, int elem_bytes,
                cudaStream_t stream)
{
    if (rows == 0 || cols == 0) {
        return kOk;
    }
    const int grid = grid_for(static_cast<int64_t>(rows) * cols, kThreads);
    if (elem_bytes == 4) {
        ttri_kernel<uint32_t><<<grid, kThreads, 0, stream>>>(static_cast<uint32_t *>(dst), rows, cols, diagonal, upper, one_bits);
    } else {
        ttri_kernel<uint16_t><<<grid, kThreads, 0, stream>>>(static_cast<uint16_t *>(dst), rows, cols, diagonal, upper,
                                                             static_cast<uint16_t>(one_bits));
    }
    return check_launch();
}

int launch_tsel(const uint8_t *mask, const void *src0, const void *src1, void *dst, int64_t n, int elem_bytes,
                cudaStream_t stream)
{
    if (n == 0) {
        return kOk;
    }
    const bool vec_ok = aligned16(src0) && aligned16(src1) && aligned16(dst);
    const int grid = grid_for((n + 7) >> 3, kThreads);
    if (elem_bytes == 4) {
        tsel_kernel<uint32_t><<<grid, kThreads, 0, stream>>>(mask, static_cast<const uint32_t *>(src0),
                                                             static_cast<const uint32_t *>(src1),
                                                             static_cast<uint32_t *>(dst), n, vec_ok);
    } else {
        tsel_kernel<uint16_t><<<grid, kThreads, 0, stream>>>(mask, static_cast<const uint16_t *>(src0),
                                                             static_cast<const uint16_t *>(src1),
                                                             static_cast<uint16_t *>(dst), n, vec_ok);
    }
    return check_launch();
}

int launch_tcmps(const float *src, float scalar, uint8_t *dst, int64_t n, int mode, cudaStream_t stream)
{
    if (n == 0) {
        return kOk;
    }
    tcmps_kernel<<<grid_for(n >> 3, kThreads), kThreads, 0, stream>>>(src, scalar, dst, n >> 3, mode, aligned16(src));
    return check_launch();
}

int launch_tcmp(const float *a, const float *b, float *dst, int64_t n, int mode, cudaStream_t stream)
{
    if (n == 0) {
        return kOk;
    }
    const bool vec_ok = aligned16(a) && aligned16(b) && aligned16(dst);
    tcmp_kernel<<<grid_for(vec_ok ? (n >> 2) + 1 : n, kThreads), kThreads, 0, stream>>>(a, b, dst, n, mode, vec_ok);
    return check_launch();
}

} // namespace pto_b200
