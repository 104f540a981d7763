/*
 * pto_b200.h - C ABI of libpto_b200.so, the B200 (sm_100a) backend for the PTO tile-ISA hot path:
 * fp16 GEMM, flash-attention forward and the vector tile ops (TCVT, TGATHER, TROWMAX, TROWSUM, TEXP, ...).
 *
 * Conventions (the same as the reference's only FFI, `call_kernel`, demos/torch_jit/gemm/gemm_kernel.cpp:259-262
 * and demos/torch_jit/flash_atten/fa_kernel.cpp:1017-1037; paths are relative to the reference root):
 *   - plain pointers and sizes only; pointers are DEVICE pointers unless the function name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream); work is enqueued
 *     asynchronously and the caller synchronises, exactly like the reference launchers
 *     (kernels/manual/a2a3/gemm_performance/main.cpp:49-52);
 *   - no allocation of caller-visible buffers: outputs and workspaces are caller-provided;
 *   - every function returns an int status (0 = ok); `pto_b200_last_error()` gives the text of the
 *     last failure on the calling thread.  The `call_kernel`-shaped shims return void like the
 *     reference's and leave their status in `pto_b200_last_status()`.
 * The library never falls back to a CPU path: without a usable sm_100 device every call fails.
 */
#ifndef PTO_B200_H
#define PTO_B200_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTO_B200_OK 0
#define PTO_B200_ERR_BAD_ARGUMENT 1
#define PTO_B200_ERR_UNSUPPORTED_SHAPE 2
#define PTO_B200_ERR_CUDA 3
#define PTO_B200_ERR_DEVICE_WAIT_TIMEOUT 4
#define PTO_B200_ERR_TOO_LARGE 5

/* RoundMode values of the reference (include/pto/common/type.hpp:167-176). */
#define PTO_B200_CAST_RINT 1
#define PTO_B200_CAST_ROUND 2
#define PTO_B200_CAST_FLOOR 3
#define PTO_B200_CAST_CEIL 4
#define PTO_B200_CAST_TRUNC 5
#define PTO_B200_CAST_ODD 6

/* MaskPattern values of the reference (include/pto/common/type.hpp:95-106). */
#define PTO_B200_P0101 1
#define PTO_B200_P1010 2
#define PTO_B200_P0001 3
#define PTO_B200_P0010 4
#define PTO_B200_P0100 5
#define PTO_B200_P1000 6
#define PTO_B200_P1111 7

/* Elementwise operators for pto_b200_tbinary_f32 / pto_b200_tscalar_f32 / pto_b200_trowexpand_f32. */
#define PTO_B200_OP_ADD 0
#define PTO_B200_OP_SUB 1
#define PTO_B200_OP_MUL 2
#define PTO_B200_OP_DIV 3
#define PTO_B200_OP_MAX 4
#define PTO_B200_OP_MIN 5
#define PTO_B200_OP_EXPDIF 6 /* exp(a - b); pto_b200_trowexpand_f32 only */
#define PTO_B200_OP_EXPAND 7 /* the row scalar itself (plain TROWEXPAND); pto_b200_trowexpand_f32 only */

/* CmpMode values of the reference (include/pto/common/type.hpp:131-139). */
#define PTO_B200_CMP_EQ 0
#define PTO_B200_CMP_NE 1
#define PTO_B200_CMP_LT 2
#define PTO_B200_CMP_LE 3
#define PTO_B200_CMP_GT 4
#define PTO_B200_CMP_GE 5

/* ---- library state ------------------------------------------------------------------------------ */

/* ABI version of this header (2: second batch of vector ops; 3: MX block-scaled GEMM, TMATMUL_BIAS form, TTRI;
 * 4: status record exports, per-block profile stamps, the random-read probe);
 * pto_b200_version() returns the version the library was built from. */
#define PTO_B200_ABI_VERSION 4
int pto_b200_version(void);
/* Text of the last error raised on the calling thread ("" if none). */
const char *pto_b200_last_error(void);
/* Status left by the last void-returning `call_kernel`-shaped shim on the calling thread. */
int pto_b200_last_status(void);
/* Reads (and clears) the device-side status record that kernels with bounded waits report into.
 * Synchronises `stream`.  Returns 0, or PTO_B200_ERR_DEVICE_WAIT_TIMEOUT if a kernel gave up on a wait. */
int pto_b200_device_status(void *stream);
/* The same, and copies the record out: record[0] the code, [1] the block that reported, [2] which wait gave up (for a
 * tile program: the flag's index ((source pipe * 8 + destination pipe) * 8 + event id), 512 + id for a cross-core
 * flag), [3] detail (for a tile program: source pipe * 16 + destination pipe).  The reference's waits are unbounded
 * (include/pto/npu/a2a3/TPush.hpp:141-146, wait_flag / wait_flag_dev); every wait here carries a limit. */
int pto_b200_device_status_ex(void *stream, int record[4]);
/* Device address of the current device's status record (four ints), so that tile programs launched through
 * pto::b200::launch (include/pto/b200/runtime.hpp) can report into the record pto_b200_device_status reads. */
void *pto_b200_status_record(void);

/* ---- vector tile ops ---------------------------------------------------------------------------- */

/* TCVT fp32 -> fp16 / bf16 over n contiguous elements: IEEE round-to-nearest-even, overflow to infinity,
 * NaN quieted.  Replaces TCVT(dst, src, RoundMode) of include/pto/common/pto_instr.hpp:864-879 for
 * float->float pairs (CPU semantics: include/pto/cpu/TCvt.hpp:76-81, where the round mode is ignored). */
int pto_b200_tcvt_f32_f16(const float *src, uint16_t *dst, int64_t n, void *stream);
int pto_b200_tcvt_f32_bf16(const float *src, uint16_t *dst, int64_t n, void *stream);
/* TCVT fp32 -> int32 with a round mode (include/pto/cpu/TCvt.hpp:28-63, :72-75). */
int pto_b200_tcvt_f32_i32(const float *src, int32_t *dst, int64_t n, int round_mode, void *stream);

/* TGATHER index form, dst[i] = src0_flat[idx[i]], an index < 0 or >= src_numel gives 0.
 * Replaces TGATHER(dst, src0, idx) of include/pto/common/pto_instr.hpp:800-806
 * (include/pto/cpu/TGather.hpp:68-100).  `elem_bytes` is 4 or 2 (bit copy). */
int pto_b200_tgather(const void *src0, int64_t src_numel, const int32_t *idx, void *dst, int64_t n, int elem_bytes,
                     void *stream);
/* TGATHER mask form: keeps the columns selected by a MaskPattern, packed contiguously
 * (include/pto/common/pto_instr.hpp:824-830, include/pto/cpu/TGather.hpp:102-129). */
int pto_b200_tgather_mask(const void *src, void *dst, int rows, int cols, int pattern, int elem_bytes, void *stream);

/* TROWMAX / TROWSUM: dst[r] = max / sum over the `cols` valid columns of row r; rows are `row_stride`
 * elements apart (include/pto/common/pto_instr.hpp:990, :942; include/pto/cpu/TRowMax.hpp:20-59,
 * TRowSum.hpp:17-63).  The sum is a tree reduction in fp32 (the reference sums sequentially). */
int pto_b200_trowmax_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream);
int pto_b200_trowsum_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream);
/* TEXP (include/pto/common/pto_instr.hpp:1129, include/pto/cpu/TExp.hpp:22-60). */
int pto_b200_texp_f32(const float *src, float *dst, int64_t n, void *stream);
/* TADD / TSUB / TMUL / TDIV / TMAX / TMIN: dst = a op b (include/pto/common/pto_instr.hpp:56-120). */
int pto_b200_tbinary_f32(const float *a, const float *b, float *dst, int64_t n, int op, void *stream);
/* TADDS / TMULS / ...: dst = a op scalar (include/pto/common/pto_instr.hpp:1161, :1188). */
int pto_b200_tscalar_f32(const float *a, float scalar, float *dst, int64_t n, int op, void *stream);
/* TROWEXPANDSUB / MUL / DIV / ADD / MAX / MIN / EXPDIF: dst[r, c] = a[r, c] op row_scalar[r], and with
 * PTO_B200_OP_EXPAND the plain TROWEXPAND dst[r, c] = row_scalar[r] (`a` is not read and may be NULL)
 * (include/pto/common/pto_instr.hpp:1049-1108; include/pto/cpu/TRowExpandOp.hpp:38-98, TRowExpand.hpp:22-37).
 * max / min are std::max / std::min; EXPDIF is exp evaluated in double and rounded to float. */
int pto_b200_trowexpand_f32(const float *a, const float *row_scalar, float *dst, int rows, int cols, int op,
                            void *stream);
/* TROWMIN: dst[r] = min over the `cols` valid columns of row r (include/pto/common/pto_instr.hpp:1007-1012,
 * include/pto/cpu/TRowMin.hpp:21-41). */
int pto_b200_trowmin_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, void *stream);
/* TCOLSUM / TCOLMAX / TCOLMIN: dst[c] = sum / max / min over the `rows` valid rows of column c; `op` is
 * PTO_B200_OP_ADD, _MAX or _MIN (include/pto/common/pto_instr.hpp:959-988, :1305-1310; include/pto/cpu/TColSum.hpp:19-30,
 * TColMax.hpp:19-33, TColMin.hpp).  The sum is a fixed-order tree in fp32 (the reference sums top to bottom).
 * `workspace` is optional scratch in device memory: with at least pto_b200_tcolreduce_workspace_bytes(rows, cols)
 * bytes of it (16-byte aligned) a large tile is reduced in two passes that use the whole GPU; with NULL, or for small
 * tiles (the query returns 0), one block per strip of 32 columns does the whole column.  The result does not depend
 * on which form ran for max / min; for the sum both orders are fixed but differ in the last bits. */
int64_t pto_b200_tcolreduce_workspace_bytes(int rows, int cols);
int pto_b200_tcolreduce_f32(const float *src, float *dst, int rows, int cols, int64_t row_stride, int op, void *workspace,
                            int64_t workspace_bytes, void *stream);
/* TFILLPAD: dst is rows x cols; its valid_rows x valid_cols corner is copied from src (same shape and pitch, read
 * only inside that corner), every other element becomes `pad_bits` (the low 16 bits for 2-byte elements): the
 * caller passes the pattern PadValue::Zero / Max / Min mean for its element type, e.g. 0x7f800000 / 0xff800000 for
 * float Max / Min (include/pto/common/pto_instr.hpp:754-782, include/pto/cpu/TFillPad.hpp:19-49). */
int pto_b200_tfillpad(const void *src, void *dst, int rows, int cols, int valid_rows, int valid_cols, uint32_t pad_bits,
                      int elem_bytes, void *stream);
/* TTRANS: dst[c, r] = src[r, c]; src is rows x cols, dst cols x rows, both dense; elem_bytes 4 or 2
 * (include/pto/common/pto_instr.hpp:1032-1037, include/pto/cpu/TTrans.hpp:17-45). */
int pto_b200_ttrans(const void *src, void *dst, int rows, int cols, int elem_bytes, void *stream);
/* TSEL: dst[i] = bit i of `mask` ? src0[i] : src1[i] over n elements of a dense row-major tile; the mask is read
 * one bit per element, least significant bit of byte 0 first, (n + 7) / 8 bytes; elem_bytes 4 or 2
 * (include/pto/common/pto_instr.hpp:1024-1029, include/pto/cpu/TSel.hpp:22-46). */
int pto_b200_tsel(const uint8_t *mask, const void *src0, const void *src1, void *dst, int64_t n, int elem_bytes,
                  void *stream);
/* TCMPS: one result bit per element of src compared with `scalar`, packed least significant bit first into n / 8
 * bytes (n a multiple of 8).  EQ / NE compare |a - b| in double against 1e-9 like the reference
 * (include/pto/common/pto_instr.hpp:143-148, include/pto/cpu/TCmps.hpp:23-91). */
int pto_b200_tcmps_f32(const float *src, float scalar, uint8_t *dst_bits, int64_t n, int mode, void *stream);
/* TCMP as the CPU simulation defines it: dst[i] = 1.0f or 0.0f from the plain comparison of a[i] and b[i]
 * (include/pto/common/pto_instr.hpp:151-157, include/pto/cpu/ElementTileOp.h:177-184, ElementOp.h:227-254). */
int pto_b200_tcmp_f32(const float *a, const float *b, float *dst, int64_t n, int mode, void *stream);

/* TTRI<Tile, isUpperOrLower>(dst, diagonal) (include/pto/common/pto_instr.hpp:817-823, include/pto/cpu/TTRI.hpp:30-77):
 * a rows x cols row-major tile of ones and zeros; lower (upper 0): one where c <= r + diagonal; upper (1): one where
 * c >= r + diagonal.  dtype: the element type whose "one" is written.  (TRESHAPE, pto_instr.hpp:999-1004, moves no data:
 * it is the same bytes under another tile shape, i.e. the same device pointer.) */
#define PTO_B200_DTYPE_F32 0
#define PTO_B200_DTYPE_I32 1
#define PTO_B200_DTYPE_F16 2
#define PTO_B200_DTYPE_I16 3
#define PTO_B200_DTYPE_BF16 4
int pto_b200_ttri(void *dst, int rows, int cols, int diagonal, int upper, int dtype, void *stream);

/* ---- GEMM --------------------------------------------------------------------------------------- */

/* C[m x n] fp32 = A[m x k] fp16 * B, fp32 accumulation.  b_layout 0: B is k x n row-major (Layout::ND);
 * 1: B is stored n x k row-major, the Layout::DN view the reference kernel uses for its second operand.
 * Replaces LaunchGEMME2E<T>(out, src0, src1, stream) of
 * kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:243-264 for any m, n, k
 * (k a multiple of 8; n a multiple of 8 when b_layout is 0). */
int pto_b200_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                         void *stream);
/* MX block-scaled fp8 GEMM: C[m x n] = (scale_a (x) A) * (scale_b (x) B)^T, the MxMatmul of
 * kernels/manual/a5/matmul_mxfp8_performance (README.md "C = (scaleA (x) A) * (scaleB (x) B)"; kernel entry
 * LaunchMxMatmul, mxmatmul_performance_kernel.cpp; instruction TMATMUL_MX, include/pto/common/pto_instr.hpp:403-460).
 * A is m x k and B is n x k (the reference's transposed second operand), both fp8: format 0 = float8_e4m3fn,
 * 1 = float8_e5m2.  scale_a is m x (k / 32) and scale_b is n x (k / 32) float8_e8m0 bytes (value 2^(byte - 127)), one
 * per 32 consecutive k of a row, row-major - the files x1_scale_gm.bin / x2_scale_gm.bin of scripts/gen_data.py:56-64.
 * C is bfloat16 (out_f32 0, the reference's output type) or float (1); products are accumulated in fp32.
 * k must be a multiple of 32.  `workspace` (device memory, 128-byte aligned, pto_b200_mxgemm_workspace_bytes(m, n, k)
 * bytes) receives the scales rearranged for the tensor core; it can be reused by the next call on the same stream. */
int64_t pto_b200_mxgemm_workspace_bytes(int m, int n, int k);
int pto_b200_mxgemm_fp8(const uint8_t *a, const uint8_t *b, const uint8_t *scale_a, const uint8_t *scale_b, void *c, int m,
                        int n, int k, int a_format, int b_format, int out_f32, void *workspace, int64_t workspace_bytes,
                        void *stream);
/* The same product with packed fp4 operands, the MxMatmul of kernels/manual/a5/matmul_mxfp4_performance: A is m x k and
 * B is n x k float4_e2m1 values, two per byte with the lower k index in the low nibble (pack_two_fp4,
 * scripts/gen_data.py:24-34), k / 2 bytes per row; scales, output, workspace and k % 32 == 0 as for the fp8 form. */
int pto_b200_mxgemm_fp4(const uint8_t *a, const uint8_t *b, const uint8_t *scale_a, const uint8_t *scale_b, void *c, int m,
                        int n, int k, int out_f32, void *workspace, int64_t workspace_bytes, void *stream);
/* The same product on bfloat16 operands (TMATMUL's bfloat16 form on the NPU back ends, include/pto/npu/a2a3/TMatmul.hpp),
 * fp32 accumulate and output. */
int pto_b200_gemm_bf16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout, void *stream);
/* The fp16 product with C rounded to fp16 or bfloat16 (nearest even) on the way out of the accumulator: the conversion
 * TSTORE offers for accumulator tiles (include/pto/common/pto_instr.hpp:159-226, docs/isa/TSTORE.md:67-72).
 * out_dtype: PTO_B200_DTYPE_F16 or PTO_B200_DTYPE_BF16.  Shapes as pto_b200_gemm_f16f32. */
int pto_b200_gemm_f16_out16(const uint16_t *a, const uint16_t *b, uint16_t *c, int m, int n, int k, int b_layout,
                            int out_dtype, void *stream);
/* TMATMUL's (int8, int8 -> int32) form (include/pto/cpu/TMatmul.hpp:46-51; tests/cpu/st/testcase/tmatmul case2):
 * C[m x n] int32 = A[m x k] int8 * B^T with B stored n x k; exact integer arithmetic.  k a multiple of 16. */
int pto_b200_gemm_i8i32(const int8_t *a, const int8_t *b, int32_t *c, int m, int n, int k, void *stream);
/* TMATMUL_BIAS (include/pto/common/pto_instr.hpp:509-527, include/pto/cpu/TMatmul.hpp:99-116): the same product with
 * bias[j] (n floats) added to every element of column j. */
int pto_b200_gemm_f16f32_bias(const uint16_t *a, const uint16_t *b, const float *bias, float *c, int m, int n, int k,
                              int b_layout, void *stream);
/* `batch` independent problems of the same shape, operands `*_stride` elements apart. */
int pto_b200_gemm_f16f32_batched(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                                 int batch, int64_t a_stride, int64_t b_stride, int64_t c_stride, void *stream);
/* Same product with HOST buffers: copies A and B in, runs the kernel, copies C out, synchronises. */
int pto_b200_gemm_f16f32_host(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout);
/* `batch` problems from HOST buffers, operands `*_stride` elements apart: the copy in of problem i + 1, the kernel of
 * problem i and the copy out of problem i - 1 overlap (three streams over two staging sets; pinned host buffers are
 * needed for the copies to overlap).  Returns after the last C has arrived. */
int pto_b200_gemm_f16f32_host_batched(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                                      int batch, int64_t a_stride, int64_t b_stride, int64_t c_stride);

/* Host-buffer GEMM for callers that must not allocate device memory at call time: processes whose device memory
 * is wholly owned by another allocator, plugins barred from allocation calls after start-up, or paths that cannot
 * afford an allocation's implicit synchronisation.  It has no counterpart in the reference.  It calls no
 * cudaMalloc / cudaFree or other allocating routine: the device copies of A, B and C and the kernel's status record
 * live in a 36 MiB array built into the library, held by every GPU that loads it until the process exits.
 * Problems whose operands need more than that (about m = n = k = 2048) return PTO_B200_ERR_TOO_LARGE.
 * The first call on a device also looks up the array's device address, and it is then that CUDA, which loads a
 * library's device code and data on first use, takes the 36 MiB from that device: make one warm-up call per device
 * at start-up, while the memory is still there to take and before any stream capture starts.  Calls run on the
 * legacy default stream and return after C has been copied out; all calls share the array (it keeps the previous
 * call's contents, the status record is cleared per call), so calls that overlap on the GPU would race - do not
 * issue them concurrently. */
int pto_b200_gemm_f16f32_host_static(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k,
                                     int b_layout);

/* ---- measurement helpers ------------------------------------------------------------------------ */

/* Per-block profile stamps, the counterpart of the reference kernel's get_sys_cnt() stamps per block
 * (kernels/manual/common/flash_atten/fa_performance_kernel.cpp:615,728-738,950-953, reduced on the host to duration and
 * TFLOPS in flash_atten/main.cpp:616-660).  With a buffer of 4 * capacity_blocks 64-bit words set for the current
 * device, every block b < capacity_blocks of the GEMM pair kernel and of the attention kernel writes
 * stamps[4 b + 0 / 1] = the global nanosecond timer at its start / end and stamps[4 b + 2 / 3] = its SM's cycle counter
 * at its start / end (cycles / nanoseconds = the clock the block really ran at).  A null pointer switches the stamps
 * off (the default).  Synchronises `stream`; kernels launched afterwards see the setting. */
int pto_b200_set_profile_buffer(uint64_t *stamps, int64_t capacity_blocks, void *stream);

/* `reads` random 4-byte reads spread over the first `table_bytes` (a power of two) of `table`, indices from a hash, no
 * index or output stream: the rate at which this GPU serves random 32-byte sectors of a table of that size, which is
 * what bounds TGATHER (include/pto/cpu/TGather.hpp:68-100) beside its two streams.  `sink` receives one word. */
int pto_b200_probe_random_reads(const uint32_t *table, int64_t table_bytes, int64_t reads, uint32_t *sink, void *stream);

/* ---- flash attention forward -------------------------------------------------------------------- */

/* O = softmax(scale * Q K^T [+ causal mask]) V for batch*heads independent heads.
 * q: [batch*heads, sq, d], k, v: [batch*heads, sk, d] fp16 contiguous; o: same shape as q, fp32
 * (out_f16 = 0, the reference's o_out type) or fp16 (out_f16 = 1).  Row max is taken on the raw logits,
 * p = exp(scale * (x - max)) in fp32, p is rounded to fp16 for the second product, O is normalised by
 * the fp32 row sum at the end; the causal mask hides keys beyond the query's own index.
 * Replaces LaunchTFA<...>(...) of kernels/manual/common/flash_atten/fa_performance_kernel.cpp:970-1004,
 * one launch per head there; d must be 128 (the reference's only head size), sq and sk multiples of 128. */
int pto_b200_flash_attn_fwd_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int batch_heads,
                                int sq, int sk, int d, int causal, float scale, int out_f16, void *stream);
/* The same with the handling of the running row maximum stated explicitly.  defer_rescale = 0: the maximum that P is
 * taken relative to follows the running maximum at every key tile (of 128 keys) where it grows, and O is rescaled each
 * time - the reference's recurrence (kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:100-184,
 * pto_macro_fa_gu.hpp:33-49).  defer_rescale = 1: it follows only once the running maximum has grown 256-fold, which
 * saves almost every rescale of O; the result is the same up to which fp16 roundings of P occur.
 * pto_b200_flash_attn_fwd_f16 uses 0 for fp32 output (the reference's output type) and 1 for fp16 output. */
int pto_b200_flash_attn_fwd_f16_ex(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o, int batch_heads,
                                   int sq, int sk, int d, int causal, float scale, int out_f16, int defer_rescale,
                                   void *stream);
/* HOST-buffer variant (copies in, runs, copies out, synchronises). */
int pto_b200_flash_attn_fwd_f16_host(const uint16_t *q, const uint16_t *k, const uint16_t *v, void *o,
                                     int batch_heads, int sq, int sk, int d, int causal, float scale, int out_f16);

/* ---- drop-in shims with the reference's FFI signatures ------------------------------------------ */

/* demos/torch_jit/gemm/gemm_kernel.cpp:259-262 `call_kernel(blockDim, stream, out, src0, src1)`: the 6144^3
 * fp16 -> fp32 GEMM with src1 stored n x k.  blockDim is accepted and ignored (the grid is sized here). */
void pto_b200_gemm_call_kernel(uint32_t blockDim, void *stream, uint8_t *out, uint8_t *src0, uint8_t *src1);
/* demos/torch_jit/flash_atten/fa_kernel.cpp:1017-1037 `call_kernel(stream, headSize, s0, s1, is_causal, q, k, v,
 * o_out, <seven workspace pointers>)`: one head, fp32 o_out.  The workspaces hold the reference's global-memory
 * FIFOs between its cube and vector cores; here those hand-offs stay on chip, so they are accepted and unused. */
void pto_b200_fa_call_kernel(void *stream, int headSize, int s0, int s1, bool is_causal, uint8_t *q, uint8_t *k,
                             uint8_t *v, uint8_t *o_out, float *qk_ws, uint16_t *p_ws, float *pmax_ws, float *pv_ws,
                             float *gsum, float *expmax, float *o_parts);

#ifdef __cplusplus
}
#endif

#endif /* PTO_B200_H */
