// The C ABI of libpto_b200.so (declared in include/pto_b200.h): argument checks, stream handling and the
// host-buffer variants around the kernel launchers.  No torch types, no allocation of caller-visible
// buffers, no CPU fallback: a call without a usable CUDA device fails with PTO_B200_ERR_CUDA.
#include "../../include/pto_b200.h"
#include "internal.h"
#include "ptx.cuh"

#include <mutex>

using namespace pto_b200;

namespace {

inline cudaStream_t as_stream(void *s)
{
    return static_cast<cudaStream_t>(s);
}

int bad(const char *what)
{
    set_error_text("%s", what);
    return kErrBadArgument;
}

// Device scratch for the *_host entry points: grown on demand, kept for reuse, one set per device.  A *_host call
// holds g_host_mutex from its first use of the set to its last synchronisation, so concurrent callers take turns.
struct HostArena {
    void *ptr[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t cap[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaStream_t stream = nullptr;
    // the batched host GEMM pipelines copies in, kernels and copies out on three streams over two staging sets
    cudaStream_t pipe[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t h2d_done[2] = {nullptr, nullptr}, comp_done[2] = {nullptr, nullptr}, d2h_done[2] = {nullptr, nullptr};
};
constexpr int kMaxHostDevices = 64;
HostArena g_arenas[kMaxHostDevices];
std::mutex g_host_mutex;

// the current device's set (nullptr, with the error text set, when there is no usable device)
HostArena *arena_of_current_device()
{
    const int dev = current_device_ordinal();
    if (dev < 0 || dev >= kMaxHostDevices) {
        set_error_text("no current CUDA device");
        return nullptr;
    }
    return &g_arenas[dev];
}

int arena_get(HostArena &ar, int slot, size_t bytes, void **out)
{
    if (ar.cap[slot] < bytes) {
        if (ar.ptr[slot] != nullptr) {
            cudaFree(ar.ptr[slot]);
            ar.ptr[slot] = nullptr;
            ar.cap[slot] = 0;
        }
        int rc = check_cuda(cudaMalloc(&ar.ptr[slot], bytes), "cudaMalloc(host-variant staging)");
        if (rc != kOk) {
            return rc;
        }
        ar.cap[slot] = bytes;
    }
    *out = ar.ptr[slot];
    return kOk;
}

int arena_stream(HostArena &ar, cudaStream_t *s)
{
    if (ar.stream == nullptr) {
        int rc = check_cuda(cudaStreamCreateWithFlags(&ar.stream, cudaStreamNonBlocking), "cudaStreamCreate");
        if (rc != kOk) {
            return rc;
        }
    }
    *s = ar.stream;
    return kOk;
}

int arena_pipeline(HostArena &ar)
{
    for (int i = 0; i < 3; ++i) {
        if (ar.pipe[i] == nullptr) {
            int rc = check_cuda(cudaStreamCreateWithFlags(&ar.pipe[i], cudaStreamNonBlocking), "cudaStreamCreate");
            if (rc != kOk) {
                return rc;
            }
        }
    }
    for (int i = 0; i < 2; ++i) {
        cudaEvent_t *evs[3] = {&ar.h2d_done[i], &ar.comp_done[i], &ar.d2h_done[i]};
        for (cudaEvent_t *e : evs) {
            if (*e == nullptr) {
                int rc = check_cuda(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "cudaEventCreate");
                if (rc != kOk) {
                    return rc;
                }
            }
        }
    }
    return kOk;
}

// end of a *_host call: wait for the stream (also after an error, so that no copy stays in flight on the caller's
// buffers), then read the device status record: a kernel that gave up on a wait must not look like success
int finish_host_call(int rc, cudaStream_t s)
{
    const int sync_rc = check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    if (rc != kOk) {
        return rc;
    }
    if (sync_rc != kOk) {
        return sync_rc;
    }
    return fetch_device_status(s);
}

} // namespace

#pragma GCC visibility push(default)
extern "C" {

int pto_b200_version(void)
{
    return PTO_B200_ABI_VERSION;
}

const char *pto_b200_last_error(void)
{
    return error_text();
}

int pto_b200_last_status(void)
{
    return last_status();
}

int pto_b200_device_status(void *stream)
{
    return fetch_device_status(as_stream(stream));
}

int pto_b200_device_status_ex(void *stream, int record[4])
{
    return fetch_device_status(as_stream(stream), record);
}

void *pto_b200_status_record(void)
{
    return device_status_ptr();
}

int pto_b200_set_profile_buffer(uint64_t *stamps, int64_t capacity_blocks, void *stream)
{
    if (stamps != nullptr && capacity_blocks <= 0) {
        return bad("set_profile_buffer: capacity_blocks must be positive");
    }
    return set_profile_buffer(reinterpret_cast<unsigned long long *>(stamps), capacity_blocks, as_stream(stream));
}

// ------------------------------------------------------------------ vector ops

int pto_b200_tcvt_f32_f16(const float *src, uint16_t *dst, int64_t n, void *stream)
{
    if (n < 0 || (n > 0 && (src == nullptr || dst == nullptr))) {
        return bad("tcvt_f32_f16: null pointer or negative length");
    }
    return launch_tcvt_f32_16(src, dst, n, false, as_stream(stream));
}

int pto_b200_tcvt_f32_bf16(const float *src, uint16_t *dst, int64_t n, void *stream)
{
    if (n < 0 || (n > 0 && (src == nullptr || dst == nullptr))) {
        return bad("tcvt_f32_bf16: null pointer or negative length");
    }
    return launch_tcvt_f32_16(src, dst, n, true, as_stream(stream));
}

int pto_b200_tcvt_f32_i32(const float *src, int32_t *dst, int64_t n, int round_mode, void *stream)
{
    if (n < 0 || (n > 0 && (src == nullptr || dst == nullptr))) {
        return bad("tcvt_f32_i32: null pointer or negative length");
    }
    if (round_mode < 0 || round_mode > 6) {
        return bad("tcvt_f32_i32: unknown round mode");
    }
    return launch_tcvt_f32_i32(src, dst, n, round_mode, as_stream(stream));
}

int pto_b200_tgather(const void *src0, int64_t src_numel, const int32_t *idx, void *dst, int64_t n, int elem_bytes,
                     void *stream)
{
    if (n < 0 || src_numel < 0 || (n > 0 && (idx == nullptr || dst == nullptr)) || (src_numel > 0 && src0 == nullptr)) {
        return bad("tgather: null pointer or negative length");
    }
    if (elem_bytes != 2 && elem_bytes != 4) {
        return bad("tgather: element size must be 2 or 4 bytes");
    }
    if (src_numel > 0x7fffffffLL) {
        set_error_text("tgather: source larger than the 32-bit index range");
        return kErrTooLarge;
    }
    return launch_tgather(src0, src_numel, idx, dst, n, elem_bytes, as_stream(stream));
}

int pto_b200_tgather_mask(const void *src, void *dst, int rows, int cols, int pattern, int elem_bytes, void *stream)
{
    if (rows < 0 || cols < 0 || (rows > 0 && cols > 0 && (src == nullptr || dst == nullptr))) {
        return bad("tgather_mask: null pointer or negative shape");
    }
    if (elem_bytes != 2 && elem_bytes != 4) {
        return bad("tgather_mask: element size must be 2 or 4 bytes");
    }
    if (pattern < 1 || pattern > 7) {
        return bad("tgather_mask: unknown mask pattern");
    }
    return launch_tgather_mask(src, dst, rows, cols, pattern, elem_bytes, as_stream(stream));
}

int pto_b200_trowmax_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream)
{
    if (rows < 0 || cols <= 0 || row_stride < cols || (rows > 0 && (src == nullptr || dst == nullptr))) {
        return bad("trowmax: bad shape or null pointer");
    }
    return launch_trow_reduce(src, dst, rows, cols, row_stride, true, as_stream(stream));
}

int pto_b200_trowsum_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream)
{
    if (rows < 0 || cols <= 0 || row_stride < cols || (rows > 0 && (src == nullptr || dst == nullptr))) {
        return bad("trowsum: bad shape or null pointer");
    }
    return launch_trow_reduce(src, dst, rows, cols, row_stride, false, as_stream(stream));
}

int pto_b200_texp_f32(const float *src, float *dst, int64_t n, void *stream)
{
    if (n < 0 || (n > 0 && (src == nullptr || dst == nullptr))) {
        return bad("texp: null pointer or negative length");
    }
    return launch_texp(src, dst, n, as_stream(stream));
}

int pto_b200_tbinary_f32(const float *a, const float *b, float *dst, int64_t n, int op, void *stream)
{
    if (n < 0 || (n > 0 && (a == nullptr || b == nullptr || dst == nullptr)) || op < 0 || op > 5) {
        return bad("tbinary: bad argument");
    }
    return launch_tbinary(a, b, dst, n, op, as_stream(stream));
}

int pto_b200_tscalar_f32(const float *a, float scalar, float *dst, int64_t n, int op, void *stream)
{
    if (n < 0 || (n > 0 && (a == nullptr || dst == nullptr)) || op < 0 || op > 5) {
        return bad("tscalar: bad argument");
    }
    return launch_tscalar(a, scalar, dst, n, op, as_stream(stream));
}

int pto_b200_trowexpand_f32(const float *a, const float *row_scalar, float *dst, int rows, int cols, int op,
                            void *stream)
{
    if (rows < 0 || cols < 0 || op < 0 || op > 7 ||
        (rows > 0 && cols > 0 && ((a == nullptr && op != 7) || row_scalar == nullptr || dst == nullptr))) {
        return bad("trowexpand: bad argument");
    }
    return launch_trowexpand(a, row_scalar, dst, rows, cols, op, as_stream(stream));
}

int pto_b200_trowmin_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream)
{
    if (rows < 0 || cols <= 0 || row_stride < cols || (rows > 0 && (src == nullptr || dst == nullptr))) {
        return bad("trowmin: bad argument");
    }
    return launch_trowmin(src, dst, rows, cols, row_stride, as_stream(stream));
}

int64_t pto_b200_tcolreduce_workspace_bytes(int rows, int cols)
{
    if (rows <= 0 || cols <= 0) {
        return 0;
    }
    const int segs = tcolreduce_segments(rows, cols);
    return segs > 1 ? static_cast<int64_t>(segs) * cols * static_cast<int64_t>(sizeof(float)) : 0;
}

int pto_b200_tcolreduce_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, int op, void *workspace,
                            int64_t workspace_bytes, void *stream)
{
    if (rows <= 0 || cols < 0 || row_stride < cols || (op != 0 && op != 4 && op != 5) || workspace_bytes < 0 ||
        (cols > 0 && (src == nullptr || dst == nullptr))) {
        return bad("tcolreduce: bad argument (op must be PTO_B200_OP_ADD, _MAX or _MIN; at least one row)");
    }
    return launch_tcolreduce(src, dst, rows, cols, row_stride, op, static_cast<float *>(workspace),
                             static_cast<size_t>(workspace_bytes), as_stream(stream));
}

int pto_b200_tfillpad(const void *src, void *dst, int rows, int cols, int valid_rows, int valid_cols, uint32_t pad_bits,
                      int elem_bytes, void *stream)
{
    if (rows < 0 || cols < 0 || valid_rows < 0 || valid_cols < 0 || valid_rows > rows || valid_cols > cols ||
        (elem_bytes != 4 && elem_bytes != 2) || (rows > 0 && cols > 0 && dst == nullptr) ||
        (valid_rows > 0 && valid_cols > 0 && src == nullptr)) {
        return bad("tfillpad: bad argument");
    }
    return launch_tfillpad(src, dst, rows, cols, valid_rows, valid_cols, pad_bits, elem_bytes, as_stream(stream));
}

int pto_b200_ttrans(const void *src, void *dst, int rows, int cols, int elem_bytes, void *stream)
{
    if (rows < 0 || cols < 0 || (elem_bytes != 4 && elem_bytes != 2) ||
        (rows > 0 && cols > 0 && (src == nullptr || dst == nullptr)) || src == dst) {
        if (!(rows == 0 || cols == 0)) {
            return bad("ttrans: bad argument (in-place transposition is not supported)");
        }
    }
    return launch_ttrans(src, dst, rows, cols, elem_bytes, as_stream(stream));
}

int pto_b200_tsel(const uint8_t *mask, const void *src0, const void *src1, void *dst, int64_t n, int elem_bytes,
                  void *stream)
{
    if (n < 0 || (elem_bytes != 4 && elem_bytes != 2) ||
        (n > 0 && (mask == nullptr || src0 == nullptr || src1 == nullptr || dst == nullptr))) {
        return bad("tsel: bad argument");
    }
    return launch_tsel(mask, src0, src1, dst, n, elem_bytes, as_stream(stream));
}

int pto_b200_tcmps_f32(const float *src, float scalar, uint8_t *dst_bits, int64_t n, int mode, void *stream)
{
    if (n < 0 || (n & 7) != 0 || mode < 0 || mode > 5 || (n > 0 && (src == nullptr || dst_bits == nullptr))) {
        return bad("tcmps: bad argument (n must be a multiple of 8)");
    }
    return launch_tcmps(src, scalar, dst_bits, n, mode, as_stream(stream));
}

int pto_b200_tcmp_f32(const float *a, const float *b, float *dst, int64_t n, int mode, void *stream)
{
    if (n < 0 || mode < 0 || mode > 5 || (n > 0 && (a == nullptr || b == nullptr || dst == nullptr))) {
        return bad("tcmp: bad argument");
    }
    return launch_tcmp(a, b, dst, n, mode, as_stream(stream));
}

// ------------------------------------------------------------------ GEMM

int pto_b200_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                         void *stream)
{
    return launch_gemm_f16f32(a, b, c, m, n, k, b_layout, as_stream(stream));
}

int64_t pto_b200_mxgemm_workspace_bytes(int m, int n, int k)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return 0;
    }
    return static_cast<int64_t>(mxgemm_workspace_bytes(m, n, k));
}

int pto_b200_mxgemm_fp8(const uint8_t *a, const uint8_t *b, const uint8_t *scale_a, const uint8_t *scale_b, void *c, int m,
                        int n, int k, int a_format, int b_format, int out_f32, void *workspace, int64_t workspace_bytes,
                        void *stream)
{
    if (a == nullptr || b == nullptr || scale_a == nullptr || scale_b == nullptr || c == nullptr || m <= 0 || n <= 0 ||
        k <= 0) {
        return bad("mxgemm: bad argument");
    }
    if ((k % 32) != 0) {
        return bad("mxgemm: k must be a multiple of the 32-element scale block");
    }
    if (a_format < 0 || a_format > 1 || b_format < 0 || b_format > 1) {
        return bad("mxgemm: formats are 0 (e4m3) or 1 (e5m2)");
    }
    if ((reinterpret_cast<uintptr_t>(a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(b) & 15u) != 0) {
        return bad("mxgemm: A and B must be 16-byte aligned");
    }
    return launch_mxgemm_fp8(a, b, scale_a, scale_b, c, m, n, k, a_format, b_format, out_f32 ? 1 : 0, workspace,
                             workspace_bytes < 0 ? 0 : static_cast<size_t>(workspace_bytes), as_stream(stream));
}

int pto_b200_ttri(void *dst, int rows, int cols, int diagonal, int upper, int dtype, void *stream)
{
    if (dst == nullptr || rows < 0 || cols < 0 || (upper != 0 && upper != 1)) {
        return bad("ttri: bad argument");
    }
    uint32_t one;
    int bytes;
    switch (dtype) {
        case PTO_B200_DTYPE_F32: one = 0x3f800000u; bytes = 4; break;
        case PTO_B200_DTYPE_I32: one = 1u; bytes = 4; break;
        case PTO_B200_DTYPE_F16: one = 0x3c00u; bytes = 2; break;
        case PTO_B200_DTYPE_I16: one = 1u; bytes = 2; break;
        default: return bad("ttri: dtype is one of PTO_B200_DTYPE_F32 / I32 / F16 / I16");
    }
    return launch_ttri(dst, rows, cols, diagonal, upper, one, bytes, as_stream(stream));
}

int pto_b200_mxgemm_fp4(const uint8_t *a, const uint8_t *b, const uint8_t *scale_a, const uint8_t *scale_b, void *c, int m,
                        int n, int k, int out_f32, void *workspace, int64_t workspace_bytes, void *stream)
{
    if (a == nullptr || b == nullptr || scale_a == nullptr || scale_b == nullptr || c == nullptr || m <= 0 || n <= 0 ||
        k <= 0) {
        return bad("mxgemm_fp4: bad argument");
    }
    if ((k % 32) != 0) {
        return bad("mxgemm_fp4: k must be a multiple of the 32-element scale block");
    }
    if ((reinterpret_cast<uintptr_t>(a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(b) & 15u) != 0) {
        return bad("mxgemm_fp4: A and B must be 16-byte aligned");
    }
    return launch_mxgemm_fp4(a, b, scale_a, scale_b, c, m, n, k, out_f32 ? 1 : 0, workspace,
                             workspace_bytes < 0 ? 0 : static_cast<size_t>(workspace_bytes), as_stream(stream));
}

int pto_b200_gemm_bf16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout, void *stream)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0 || (b_layout != 0 && b_layout != 1)) {
        return bad("gemm_bf16: bad argument");
    }
    if ((k % 8) != 0 || (b_layout == 0 && (n % 8) != 0) || (reinterpret_cast<uintptr_t>(a) & 15u) ||
        (reinterpret_cast<uintptr_t>(b) & 15u)) {
        set_error_text("gemm_bf16: k (and n for a k x n B) must be multiples of 8 and operands 16-byte aligned");
        return kErrUnsupportedShape;
    }
    return launch_gemm2_bf16f32(a, b, c, m, n, k, b_layout, as_stream(stream));
}

int pto_b200_gemm_f16_out16(const uint16_t *a, const uint16_t *b, uint16_t *c, int m, int n, int k, int b_layout,
                            int out_dtype, void *stream)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0 || (b_layout != 0 && b_layout != 1)) {
        return bad("gemm_out16: bad argument");
    }
    if (out_dtype != PTO_B200_DTYPE_F16 && out_dtype != PTO_B200_DTYPE_BF16) {
        return bad("gemm_out16: out_dtype is PTO_B200_DTYPE_F16 or PTO_B200_DTYPE_BF16");
    }
    if ((k % 8) != 0 || (b_layout == 0 && (n % 8) != 0) || (reinterpret_cast<uintptr_t>(a) & 15u) ||
        (reinterpret_cast<uintptr_t>(b) & 15u)) {
        set_error_text("gemm_out16: k (and n for a k x n B) must be multiples of 8 and operands 16-byte aligned");
        return kErrUnsupportedShape;
    }
    return launch_gemm2_f16_out16(a, b, c, m, n, k, b_layout, out_dtype == PTO_B200_DTYPE_F16 ? 1 : 2, as_stream(stream));
}

int pto_b200_gemm_i8i32(const int8_t *a, const int8_t *b, int32_t *c, int m, int n, int k, void *stream)
{
    return launch_gemm2_i8i32(a, b, c, m, n, k, as_stream(stream));
}

int pto_b200_gemm_f16f32_bias(const uint16_t *a, const uint16_t *b, const float *bias, float *c, int m, int n, int k,
                              int b_layout, void *stream)
{
    if (bias == nullptr) {
        return bad("gemm_bias: bias is null");
    }
    return launch_gemm_f16f32(a, b, c, m, n, k, b_layout, as_stream(stream), bias);
}

int pto_b200_gemm_f16f32_batched(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                                 int batch, int64_t a_stride, int64_t b_stride, int64_t c_stride, void *stream)
{
    if (batch < 0) {
        return bad("gemm_batched: negative batch");
    }
    for (int i = 0; i < batch; ++i) {
        const int rc = launch_gemm_f16f32(a + i * a_stride, b + i * b_stride, c + i * c_stride, m, n, k, b_layout,
                                          as_stream(stream));
        if (rc != kOk) {
            return rc;
        }
    }
    return kOk;
}

int pto_b200_gemm_f16f32_host(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0) {
        return bad("gemm_host: bad argument");
    }
    const size_t a_bytes = static_cast<size_t>(m) * k * 2, b_bytes = static_cast<size_t>(n) * k * 2,
                 c_bytes = static_cast<size_t>(m) * n * 4;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostArena *ar = arena_of_current_device();
    if (ar == nullptr) {
        return kErrCuda;
    }
    void *da, *db, *dc;
    cudaStream_t s;
    int rc;
    if ((rc = arena_stream(*ar, &s)) != kOk || (rc = arena_get(*ar, 0, a_bytes, &da)) != kOk ||
        (rc = arena_get(*ar, 1, b_bytes, &db)) != kOk || (rc = arena_get(*ar, 2, c_bytes, &dc)) != kOk) {
        return rc;
    }
    if ((rc = check_cuda(cudaMemcpyAsync(da, a, a_bytes, cudaMemcpyHostToDevice, s), "H2D A")) == kOk &&
        (rc = check_cuda(cudaMemcpyAsync(db, b, b_bytes, cudaMemcpyHostToDevice, s), "H2D B")) == kOk &&
        (rc = launch_gemm_f16f32(static_cast<const uint16_t *>(da), static_cast<const uint16_t *>(db),
                                 static_cast<float *>(dc), m, n, k, b_layout, s)) == kOk) {
        rc = check_cuda(cudaMemcpyAsync(c, dc, c_bytes, cudaMemcpyDeviceToHost, s), "D2H C");
    }
    return finish_host_call(rc, s);
}

int pto_b200_gemm_f16f32_host_batched(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                                      int batch, int64_t a_stride, int64_t b_stride, int64_t c_stride)
{
    if (m <= 0 || n <= 0 || k <= 0 || batch < 0 || a_stride < 0 || b_stride < 0 || c_stride < 0 ||
        (batch > 0 && (a == nullptr || b == nullptr || c == nullptr))) {
        return bad("gemm_host_batched: bad argument");
    }
    if (batch == 0) {
        return kOk;
    }
    const size_t a_bytes = static_cast<size_t>(m) * k * 2, b_bytes = static_cast<size_t>(n) * k * 2,
                 c_bytes = static_cast<size_t>(m) * n * 4;
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostArena *arp = arena_of_current_device();
    if (arp == nullptr) {
        return kErrCuda;
    }
    HostArena &ar = *arp;
    void *da[2], *db[2], *dc[2];
    int rc = arena_pipeline(ar);
    for (int s = 0; s < 2 && rc == kOk; ++s) {
        if ((rc = arena_get(ar, 2 + 3 * s, a_bytes, &da[s])) == kOk &&
            (rc = arena_get(ar, 3 + 3 * s, b_bytes, &db[s])) == kOk) {
            rc = arena_get(ar, 4 + 3 * s, c_bytes, &dc[s]);
        }
    }
    if (rc != kOk) {
        return rc;
    }
    cudaStream_t in = ar.pipe[0], run = ar.pipe[1], out = ar.pipe[2];
    for (int i = 0; i < batch && rc == kOk; ++i) {
        const int s = i & 1;
        const uint16_t *ha = a + static_cast<int64_t>(i) * a_stride, *hb = b + static_cast<int64_t>(i) * b_stride;
        float *hc = c + static_cast<int64_t>(i) * c_stride;
        // copies in: the kernel of problem i - 2 has consumed this set's A and B
        if (i >= 2) {
            rc = check_cuda(cudaStreamWaitEvent(in, ar.comp_done[s], 0), "cudaStreamWaitEvent");
        }
        if (rc == kOk) rc = check_cuda(cudaMemcpyAsync(da[s], ha, a_bytes, cudaMemcpyHostToDevice, in), "H2D A");
        if (rc == kOk) rc = check_cuda(cudaMemcpyAsync(db[s], hb, b_bytes, cudaMemcpyHostToDevice, in), "H2D B");
        if (rc == kOk) rc = check_cuda(cudaEventRecord(ar.h2d_done[s], in), "cudaEventRecord");
        // kernel: operands are in, and the copy out of problem i - 2 has read this set's C
        if (rc == kOk) rc = check_cuda(cudaStreamWaitEvent(run, ar.h2d_done[s], 0), "cudaStreamWaitEvent");
        if (rc == kOk && i >= 2) rc = check_cuda(cudaStreamWaitEvent(run, ar.d2h_done[s], 0), "cudaStreamWaitEvent");
        if (rc == kOk) {
            rc = launch_gemm_f16f32(static_cast<const uint16_t *>(da[s]), static_cast<const uint16_t *>(db[s]),
                                    static_cast<float *>(dc[s]), m, n, k, b_layout, run);
        }
        if (rc == kOk) rc = check_cuda(cudaEventRecord(ar.comp_done[s], run), "cudaEventRecord");
        // copy out
        if (rc == kOk) rc = check_cuda(cudaStreamWaitEvent(out, ar.comp_done[s], 0), "cudaStreamWaitEvent");
        if (rc == kOk) rc = check_cuda(cudaMemcpyAsync(hc, dc[s], c_bytes, cudaMemcpyDeviceToHost, out), "D2H C");
        if (rc == kOk) rc = check_cuda(cudaEventRecord(ar.d2h_done[s], out), "cudaEventRecord");
    }
    // drain all three streams even after an error so that no copy is left in flight on the caller's buffers
    const int r0 = check_cuda(cudaStreamSynchronize(in), "cudaStreamSynchronize");
    const int r1 = check_cuda(cudaStreamSynchronize(run), "cudaStreamSynchronize");
    const int r2 = check_cuda(cudaStreamSynchronize(out), "cudaStreamSynchronize");
    if (rc != kOk || r0 != kOk || r1 != kOk || r2 != kOk) {
        return rc != kOk ? rc : (r0 != kOk ? r0 : (r1 != kOk ? r1 : r2));
    }
    return fetch_device_status(run); // a kernel that gave up on a wait must not look like success
}

int pto_b200_gemm_f16f32_host_static(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout)
{
    return gemm_f16f32_host_static(a, b, c, m, n, k, b_layout);
}

// ------------------------------------------------------------------ measurement helpers

int pto_b200_probe_random_reads(const uint32_t *table, int64_t table_bytes, int64_t reads, uint32_t *sink, void *stream)
{
    if (table == nullptr || sink == nullptr || reads <= 0 || table_bytes < 1024 || (table_bytes & (table_bytes - 1)) != 0 ||
        table_bytes > (static_cast<int64_t>(1) << 34)) {
        return bad("probe_random_reads: the table size must be a power of two between 1 KiB and 16 GiB, reads > 0");
    }
    return launch_random_read_probe(table, table_bytes, reads, sink, as_stream(stream));
}

// ------------------------------------------------------------------ flash attention

int pto_b200_flash_attn_fwd_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int batch_heads,
                                int sq, int sk, int d, int causal, float scale, int out_f16, void *stream)
{
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || batch_heads <= 0 || sq <= 0 || sk <= 0) {
        return bad("flash_attn_fwd: bad argument");
    }
    return launch_flash_attn_fwd(q, k, v, o, batch_heads, sq, sk, d, causal, scale, out_f16, as_stream(stream));
}

int pto_b200_flash_attn_fwd_f16_ex(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int batch_heads,
                                   int sq, int sk, int d, int causal, float scale, int out_f16, int defer_rescale,
                                   void *stream)
{
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || batch_heads <= 0 || sq <= 0 || sk <= 0 ||
        (defer_rescale != 0 && defer_rescale != 1)) {
        return bad("flash_attn_fwd_ex: bad argument");
    }
    return launch_flash_attn_fwd(q, k, v, o, batch_heads, sq, sk, d, causal, scale, out_f16, as_stream(stream),
                                 defer_rescale);
}

int pto_b200_flash_attn_fwd_f16_host(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o,
                                     int batch_heads, int sq, int sk, int d, int causal, float scale, int out_f16)
{
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || batch_heads <= 0 || sq <= 0 || sk <= 0 ||
        d <= 0) {
        return bad("flash_attn_fwd_host: bad argument");
    }
    const size_t q_bytes = static_cast<size_t>(batch_heads) * sq * d * 2;
    const size_t kv_bytes = static_cast<size_t>(batch_heads) * sk * d * 2;
    const size_t o_bytes = static_cast<size_t>(batch_heads) * sq * d * (out_f16 ? 2 : 4);
    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostArena *ar = arena_of_current_device();
    if (ar == nullptr) {
        return kErrCuda;
    }
    void *dq, *dk, *dv, *dout;
    cudaStream_t s;
    int rc;
    if ((rc = arena_stream(*ar, &s)) != kOk || (rc = arena_get(*ar, 0, q_bytes, &dq)) != kOk ||
        (rc = arena_get(*ar, 1, kv_bytes, &dk)) != kOk || (rc = arena_get(*ar, 2, kv_bytes, &dv)) != kOk ||
        (rc = arena_get(*ar, 3, o_bytes, &dout)) != kOk) {
        return rc;
    }
    if ((rc = check_cuda(cudaMemcpyAsync(dq, q, q_bytes, cudaMemcpyHostToDevice, s), "H2D Q")) == kOk &&
        (rc = check_cuda(cudaMemcpyAsync(dk, k, kv_bytes, cudaMemcpyHostToDevice, s), "H2D K")) == kOk &&
        (rc = check_cuda(cudaMemcpyAsync(dv, v, kv_bytes, cudaMemcpyHostToDevice, s), "H2D V")) == kOk &&
        (rc = launch_flash_attn_fwd(static_cast<const uint16_t *>(dq), static_cast<const uint16_t *>(dk),
                                    static_cast<const uint16_t *>(dv), dout, batch_heads, sq, sk, d, causal, scale,
                                    out_f16, s)) == kOk) {
        rc = check_cuda(cudaMemcpyAsync(o, dout, o_bytes, cudaMemcpyDeviceToHost, s), "D2H O");
    }
    return finish_host_call(rc, s);
}

// ------------------------------------------------------------------ reference-shaped shims

void pto_b200_gemm_call_kernel(uint32_t blockDim, void *stream, uint8_t *out, uint8_t *src0, uint8_t *src1)
{
    (void)blockDim;
    set_last_status(launch_gemm_f16f32(reinterpret_cast<const uint16_t *>(src0),
                                       reinterpret_cast<const uint16_t *>(src1), reinterpret_cast<float *>(out), 6144,
                                       6144, 6144, 1, as_stream(stream)));
}

void pto_b200_fa_call_kernel(void *stream, int headSize, int s0, int s1, bool is_causal, uint8_t *q, uint8_t *k,
                             uint8_t *v, uint8_t *o_out, float *qk_ws, uint16_t *p_ws, float *pmax_ws, float *pv_ws,
                             float *gsum, float *expmax, float *o_parts)
{
    (void)qk_ws;
    (void)p_ws;
    (void)pmax_ws;
    (void)pv_ws;
    (void)gsum;
    (void)expmax;
    (void)o_parts;
    if (headSize != 128 || (s0 % 128) != 0) {
        // the reference returns silently for these (fa_kernel.cpp:1051-1059); the status says why
        set_error_text("fa call_kernel: headSize must be 128 and s0 a multiple of 128");
        set_last_status(kErrUnsupportedShape);
        return;
    }
    set_last_status(launch_flash_attn_fwd(reinterpret_cast<const uint16_t *>(q), reinterpret_cast<const uint16_t *>(k),
                                          reinterpret_cast<const uint16_t *>(v), o_out, 1, s0, s1, headSize,
                                          is_causal ? 1 : 0, 0.08838834764831845f, 0, as_stream(stream)));
}

} // extern "C"
#pragma GCC visibility pop
