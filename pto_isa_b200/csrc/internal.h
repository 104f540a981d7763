// Declarations shared by the translation units of libpto_b200.so (not part of the public ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pto_b200 {

struct DeviceStatus;

// number of SMs of the current device (cached per device)
int sm_count();
// raises the dynamic shared-memory limit of a kernel on the current device, once per (kernel, device): the attribute is
// kept per device, so a process that drives several GPUs needs it set on each of them
int ensure_dynamic_smem(const void *kernel, int bytes);
// ordinal of the current device, -1 when there is none (or more than the library's tables hold)
int current_device_ordinal();
// cudaGetLastError() mapped to a status code; records the CUDA error text for pto_b200_last_error()
int check_launch();
int check_cuda(cudaError_t e, const char *what);
void set_error_text(const char *fmt, ...);
const char *error_text();
void set_last_status(int code);
int last_status();
// per-device status record in global memory that kernels with bounded waits report into;
// allocated on first use for the current device
DeviceStatus *device_status_ptr();
// reads the status record back (synchronises `stream`) and clears it; returns its code
int fetch_device_status(cudaStream_t stream, int *record = nullptr); // record: {code, block, where, detail}

// per-block profile stamps of the current device's kernels: on with a buffer of 4 * capacity_blocks words, off with null
int set_profile_buffer(unsigned long long *stamps, long long capacity_blocks, cudaStream_t stream);

// cuTensorMapEncodeTiled resolved through the runtime (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// Encodes a tiled tensor map over a row-major 2-D (rows x cols) or 3-D (outer x rows x cols) array of
// 16-bit (or 32-bit) elements with a (box_rows x box_cols) box and 128-byte swizzle.  Returns a status code.
int make_tmap_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols, bool swizzle128);
int make_tmap_3d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t outer, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_elems, uint64_t outer_stride_elems, uint32_t box_rows, uint32_t box_cols,
                 bool swizzle128);

// vector ops
int launch_tcvt_f32_16(const float *src, uint16_t *dst, int64_t n, bool bf16, cudaStream_t stream);
int launch_tcvt_f32_i32(const float *src, int32_t *dst, int64_t n, int mode, cudaStream_t stream);
int launch_tgather(const void *src0, int64_t numel, const int32_t *idx, void *dst, int64_t n, int elem_bytes,
                   cudaStream_t stream);
int launch_random_read_probe(const uint32_t *table, int64_t table_bytes, int64_t reads, uint32_t *sink,
                             cudaStream_t stream);
int launch_tgather_mask(const void *src, void *dst, int rows, int cols, int pattern, int elem_bytes,
                        cudaStream_t stream);
int launch_trow_reduce(const float *src, float *dst, int rows, int cols, int64_t row_stride, bool is_max,
                       cudaStream_t stream);
int launch_texp(const float *src, float *dst, int64_t n, cudaStream_t stream);
int launch_tbinary(const float *a, const float *b, float *dst, int64_t n, int op, cudaStream_t stream);
int launch_tscalar(const float *a, float s, float *dst, int64_t n, int op, cudaStream_t stream);
int launch_trowexpand(const float *a, const float *row_scalar, float *dst, int rows, int cols, int op,
                      cudaStream_t stream);
int launch_trowmin(const float *src, float *dst, int rows, int cols, int64_t row_stride, cudaStream_t stream);
int launch_tcolreduce(const float *src, float *dst, int rows, int cols, int64_t row_stride, int op, float *workspace,
                      size_t workspace_bytes, cudaStream_t stream);
int tcolreduce_segments(int rows, int cols);
int launch_tfillpad(const void *src, void *dst, int rows, int cols, int valid_rows, int valid_cols, uint32_t pad,
                    int elem_bytes, cudaStream_t stream);
int launch_ttrans(const void *src, void *dst, int rows, int cols, int elem_bytes, cudaStream_t stream);
int launch_tsel(const uint8_t *mask, const void *src0, const void *src1, void *dst, int64_t n, int elem_bytes,
                cudaStream_t stream);
int launch_tcmps(const float *src, float scalar, uint8_t *dst, int64_t n, int mode, cudaStream_t stream);
int launch_tcmp(const float *a, const float *b, float *dst, int64_t n, int mode, cudaStream_t stream);
// blocks for a grid-stride kernel over `work_items` items, `items_per_block` per block per pass (capped at 32 per SM)
int grid_for(int64_t work_items, int items_per_block);

// GEMM: C[m x n] fp32 = A[m x k] fp16 * B, B given k x n row-major (b_layout 0) or n x k row-major (1)
// `bias` (optional): n floats added to every row of C (TMATMUL_BIAS)
int launch_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                       cudaStream_t stream, const float *bias = nullptr);

// the same product on pairs of thread blocks (cta_group::2); arguments already validated by the caller
int launch_gemm2_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                        cudaStream_t stream, const float *bias = nullptr);
// TTRI: rows x cols tile of `one_bits` (the element type's one) inside the lower / upper triangle, zero outside
int launch_ttri(void *dst, int rows, int cols, int diagonal, int upper, uint32_t one_bits, int elem_bytes,
                cudaStream_t stream);

// MX block-scaled fp8 GEMM (kind::mxf8f6f4): C[m x n] bf16 (or fp32) = (sfa (x) A[m x k]) * (sfb (x) B[n x k])^T, one e8m0
// scale per 32 k; a_fmt / b_fmt 0 = e4m3, 1 = e5m2.  The workspace receives the scales in the tensor core's atoms.
size_t mxgemm_workspace_bytes(int m, int n, int k);
int launch_mxgemm_fp8(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, void *c, int m, int n,
                      int k, int a_fmt, int b_fmt, int out_f32, void *workspace, size_t workspace_bytes,
                      cudaStream_t stream);
// the same with packed fp4 (e2m1) operands, two per byte, the lower k index in the low nibble (kind::mxf4, block 32)
int launch_mxgemm_fp4(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, void *c, int m, int n,
                      int k, int out_f32, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// bfloat16 operands, fp32 accumulate and output; arguments validated by the caller
int launch_gemm2_bf16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                         cudaStream_t stream);
// the fp16 product with C rounded to fp16 (out16 1) or bf16 (2) in the epilogue; arguments validated by the caller
int launch_gemm2_f16_out16(const uint16_t *a, const uint16_t *b, uint16_t *c, int m, int n, int k, int b_layout, int out16,
                           cudaStream_t stream);
// C[m x n] int32 = A[m x k] int8 * B[n x k]^T int8 (kind::i8 on the CTA-pair kernel); k a multiple of 16
int launch_gemm2_i8i32(const int8_t *a, const int8_t *b, int32_t *c, int m, int n, int k, cudaStream_t stream);
// host-buffer GEMM whose device staging and status record live in a built-in static device array (no allocation)
int gemm_f16f32_host_static(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout);
size_t gemm_static_scratch_bytes();

// flash attention forward; q/k/v/o are [batch*heads, seq, d] contiguous; out_f16 selects the output type
int launch_flash_attn_fwd(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int bh, int sq, int sk,
                          int d, int causal, float scale, int out_f16, cudaStream_t stream, int defer_rescale = -1);

} // namespace pto_b200
