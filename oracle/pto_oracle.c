/*
 * TEST INFRASTRUCTURE ONLY - a CPU restatement of the reference's CPU-simulation arithmetic for
 * the tile ops on the GEMM / flash-attention / vector hot path.  It exists to check the CUDA
 * kernels; it is never linked into, imported by, or called from the product library.
 * Only the tests, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Parity pin: every function below is compared bit-for-bit (GEMM, attention: bit-for-bit too,
 * because the summation order is kept) against the reference's own headers compiled as
 * oracle/_ref/libpto_ref.so, and against the golden vectors under tests/golden/ that were
 * produced by the reference's own generator scripts.  bf16 conversion has no case in the
 * reference's tests; its pin is the reference TCVT_IMPL instantiated over std::bfloat16_t.
 *
 * Paths are relative to the reference project root.  Plain C11, no dependencies beyond libm and
 * pthreads.  Compile with -ffp-contract=off so that a*b+c is rounded twice like the reference
 * build (x86-64 -O2 without FMA).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------ scalar conversions */

static inline uint32_t f32_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
static inline float bits_f32(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* IEEE binary16 -> binary32, exact. */
static inline float half_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) {
            return bits_f32(sign);
        }
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return bits_f32(f32_bits(v) | sign);
    }
    if (exp == 31) {
        return bits_f32(sign | 0x7f800000u | (man << 13));
    }
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round-to-nearest-even, overflow to infinity (no saturation), NaN keeps
 * its sign and top payload bits with the quiet bit set: what `static_cast<_Float16>(float)` does
 * in include/pto/cpu/TCvt.hpp:80. */
static inline uint16_t f32_to_half(float f)
{
    uint32_t u = f32_bits(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) {
        return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x3ffu));
    }
    if (a >= 0x47800000u) { /* |f| >= 65536 or inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a >= 0x38800000u) { /* normal half range: |f| >= 2^-14 */
        uint32_t r = a - 0x38000000u; /* rebias exponent by 112 */
        uint32_t lsb = (r >> 13) & 1u;
        r += 0xfffu + lsb;
        return (uint16_t)(sign | (r >> 13)); /* a carry into the exponent is the right answer, up to inf */
    }
    if (a < 0x33000000u) { /* |f| < 2^-25 rounds to zero (2^-25 itself ties to even = 0) */
        return sign;
    }
    /* subnormal half: shift the 24-bit significand right, RNE */
    {
        uint32_t e = a >> 23;                       /* biased exponent, 102..112 */
        uint32_t m = (a & 0x7fffffu) | 0x800000u;   /* 24-bit significand */
        uint32_t shift = 126u - e;                  /* 14..24 */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1u);
        if (rem > halfway || (rem == halfway && (q & 1u))) {
            q++;
        }
        return (uint16_t)(sign | q);
    }
}

/* binary32 -> bfloat16, round-to-nearest-even; NaN is quieted and keeps sign + top payload. */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* ------------------------------------------------------------------ tiny parallel-for */

typedef void (*range_fn)(int64_t begin, int64_t end, void *ctx);
typedef struct {
    range_fn fn;
    void *ctx;
    int64_t begin, end;
} worker_arg;

static void *worker_main(void *p)
{
    worker_arg *w = (worker_arg *)p;
    w->fn(w->begin, w->end, w->ctx);
    return NULL;
}

static int g_threads = 0;

int pto_oracle_set_threads(int n)
{
    g_threads = n;
    return 0;
}

int pto_oracle_threads(void)
{
    if (g_threads > 0) {
        return g_threads;
    }
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

static void parallel_range(int64_t begin, int64_t end, range_fn fn, void *ctx)
{
    int64_t count = end - begin;
    int nt = pto_oracle_threads();
    if (count <= 0) {
        return;
    }
    if (nt > count) {
        nt = (int)count;
    }
    if (nt <= 1) {
        fn(begin, end, ctx);
        return;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
    worker_arg *args = (worker_arg *)malloc(sizeof(worker_arg) * (size_t)nt);
    int64_t chunk = (count + nt - 1) / nt;
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        int64_t b = begin + chunk * t;
        int64_t e = b + chunk < end ? b + chunk : end;
        if (b >= e) {
            break;
        }
        args[t].fn = fn;
        args[t].ctx = ctx;
        args[t].begin = b;
        args[t].end = e;
        pthread_create(&th[t], NULL, worker_main, &args[t]);
        started++;
    }
    for (int t = 0; t < started; ++t) {
        pthread_join(th[t], NULL);
    }
    free(th);
    free(args);
}

/* ------------------------------------------------------------------ TCVT
 * include/pto/cpu/TCvt.hpp:65-92: float->float pairs are a static_cast (IEEE round-to-nearest-even,
 * the RoundMode argument is ignored, no saturation); float->integer applies the round mode in
 * double and then casts (:28-63). */

int pto_oracle_tcvt_f32_f16(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = f32_to_half(src[i]);
    }
    return 0;
}

int pto_oracle_tcvt_f32_bf16(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = f32_to_bf16(src[i]);
    }
    return 0;
}

/* RoundMode numbering of include/pto/common/type.hpp:167-176:
 * 0 NONE, 1 RINT, 2 ROUND, 3 FLOOR, 4 CEIL, 5 TRUNC, 6 ODD. */
static double round_integral(double v, int mode)
{
    switch (mode) {
        case 1: return rint(v);
        case 2: return round(v);
        case 3: return floor(v);
        case 4: return ceil(v);
        case 5: return trunc(v);
        case 6: {
            double f = floor(v), frac = v - f;
            if (frac > 0.5) return f + 1;
            if (frac < 0.5) return f;
            return (((long long)f) & 1) ? f : f + 1;
        }
        default: return v;
    }
}

int pto_oracle_tcvt_f32_i32(const float *src, int32_t *dst, int64_t n, int mode)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = (int32_t)round_integral((double)src[i], mode);
    }
    return 0;
}

/* ------------------------------------------------------------------ TGATHER
 * Index form, include/pto/cpu/TGather.hpp:68-100: dst[i] = src0.flat[idx[i]] with the flat index
 * taken over the full (rows x cols) source tile; an index that is negative or >= rows*cols
 * yields 0.  Mask form, :102-129: keep the columns a pattern selects, packed contiguously in
 * row-major order over the whole tile (:18-44 for the patterns). */

int pto_oracle_tgather_f32(const float *src0, int src_rows, int src_cols, const int32_t *idx, float *dst, int64_t n)
{
    const int64_t numel = (int64_t)src_rows * src_cols;
    for (int64_t i = 0; i < n; ++i) {
        int32_t r = idx[i];
        dst[i] = (r < 0 || (int64_t)r >= numel) ? 0.0f : src0[r];
    }
    return 0;
}

int pto_oracle_tgather_b16(const uint16_t *src0, int src_rows, int src_cols, const int32_t *idx, uint16_t *dst,
                           int64_t n)
{
    const int64_t numel = (int64_t)src_rows * src_cols;
    for (int64_t i = 0; i < n; ++i) {
        int32_t r = idx[i];
        dst[i] = (r < 0 || (int64_t)r >= numel) ? (uint16_t)0 : src0[r];
    }
    return 0;
}

/* pattern: 1 P0101, 2 P1010, 3 P0001, 4 P0010, 5 P0100, 6 P1000, 7 P1111 (type.hpp:96-106) */
static int mask_select(int pattern, unsigned c)
{
    switch (pattern) {
        case 1: return (c % 2u) == 0;
        case 2: return (c % 2u) == 1;
        case 3: return (c % 4u) == 0;
        case 4: return (c % 4u) == 1;
        case 5: return (c % 4u) == 2;
        case 6: return (c % 4u) == 3;
        default: return 1;
    }
}

int pto_oracle_tgather_mask_f32(const float *src, float *dst, int rows, int cols, int pattern)
{
    int64_t d = 0;
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            if (mask_select(pattern, (unsigned)c)) {
                dst[d++] = src[(int64_t)r * cols + c];
            }
        }
    }
    return 0;
}

int pto_oracle_tgather_mask_b16(const uint16_t *src, uint16_t *dst, int rows, int cols, int pattern)
{
    int64_t d = 0;
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            if (mask_select(pattern, (unsigned)c)) {
                dst[d++] = src[(int64_t)r * cols + c];
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ row reductions and TEXP
 * include/pto/cpu/TRowMax.hpp:20-48 (std::max fold from column 0), TRowSum.hpp:17-40 (sequential
 * fp32 sum from 0), TExp.hpp:22-45 (float(exp(double(x)))). */

int pto_oracle_trowmax_f32(const float *src, float *dst, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        const float *p = src + (int64_t)r * cols;
        float m = p[0];
        for (int c = 1; c < cols; ++c) {
            m = (m < p[c]) ? p[c] : m; /* std::max(m, x) */
        }
        dst[r] = m;
    }
    return 0;
}

int pto_oracle_trowsum_f32(const float *src, float *dst, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        const float *p = src + (int64_t)r * cols;
        float s = 0.0f;
        for (int c = 0; c < cols; ++c) {
            s += p[c];
        }
        dst[r] = s;
    }
    return 0;
}

int pto_oracle_texp_f32(const float *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = (float)exp((double)src[i]);
    }
    return 0;
}

/* ------------------------------------------------------------------ GEMM
 * The tile program of kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:67-149 with a
 * 64-wide k step: for every C element, each k step contributes a dot product summed sequentially
 * in fp32 from 0 (include/pto/cpu/TMatmul.hpp:22-37), and the steps are added to the accumulator in
 * order (first step assigns).  b_layout 0: B is k x n row-major; 1: B is stored n x k row-major
 * (Layout::DN view).  Loops are ordered so that the innermost runs over n for SIMD; the value of
 * every output is unchanged by that because each (i, j) keeps its own k order. */

typedef struct {
    const uint16_t *a, *b;
    float *c;
    int m, n, k, b_layout;
    int r0, r1, c0, c1; /* optional output window (rows [r0,r1), cols [c0,c1)) */
} gemm_ctx;

#define GEMM_KSTEP 64

static void gemm_rows(int64_t begin, int64_t end, void *p)
{
    const gemm_ctx *g = (const gemm_ctx *)p;
    const int ncols = g->c1 - g->c0;
    const int k = g->k;
    float *bt = (float *)malloc(sizeof(float) * (size_t)GEMM_KSTEP * (size_t)ncols); /* B step, [kk][j] */
    float *part = (float *)malloc(sizeof(float) * (size_t)ncols);
    float arow[GEMM_KSTEP];
    /* walk k steps outermost so the converted B step is reused by all rows of this range */
    for (int ks = 0; ks < k; ks += GEMM_KSTEP) {
        for (int kk = 0; kk < GEMM_KSTEP; ++kk) {
            for (int j = 0; j < ncols; ++j) {
                uint16_t h = (g->b_layout == 0) ? g->b[(int64_t)(ks + kk) * g->n + (g->c0 + j)]
                                                : g->b[(int64_t)(g->c0 + j) * k + (ks + kk)];
                bt[(int64_t)kk * ncols + j] = half_to_f32(h);
            }
        }
        for (int64_t i = begin; i < end; ++i) {
            const uint16_t *ar = g->a + i * k + ks;
            for (int kk = 0; kk < GEMM_KSTEP; ++kk) {
                arow[kk] = half_to_f32(ar[kk]);
            }
            for (int j = 0; j < ncols; ++j) {
                part[j] = 0.0f;
            }
            for (int kk = 0; kk < GEMM_KSTEP; ++kk) {
                const float av = arow[kk];
                const float *brow = bt + (int64_t)kk * ncols;
                for (int j = 0; j < ncols; ++j) {
                    part[j] += av * brow[j];
                }
            }
            float *crow = g->c + i * g->n + g->c0;
            if (ks == 0) {
                for (int j = 0; j < ncols; ++j) {
                    crow[j] = part[j];
                }
            } else {
                for (int j = 0; j < ncols; ++j) {
                    crow[j] = crow[j] + part[j];
                }
            }
        }
    }
    free(bt);
    free(part);
}

int pto_oracle_gemm_f16f32_window(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout,
                                  int r0, int r1, int c0, int c1)
{
    if (k % GEMM_KSTEP || r0 < 0 || r1 > m || c0 < 0 || c1 > n) {
        return -1;
    }
    gemm_ctx g = {a, b, c, m, n, k, b_layout, r0, r1, c0, c1};
    parallel_range(r0, r1, gemm_rows, &g);
    return 0;
}

int pto_oracle_gemm_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int n, int k, int b_layout)
{
    return pto_oracle_gemm_f16f32_window(a, b, c, m, n, k, b_layout, 0, m, 0, n);
}

/* ------------------------------------------------------------------ TTRI
 * include/pto/cpu/TTRI.hpp:30-77: lower (upper == 0): dst[r, c] = 1 for c <= r + diagonal, else 0; upper: dst[r, c] = 1
 * for c >= r + diagonal, else 0.  "1" is the element type's one: 32-bit words (float 1.0f or integer 1) are passed in. */
int pto_oracle_ttri_b32(uint32_t *dst, int rows, int cols, int diagonal, int upper, uint32_t one)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            int in = upper ? (c >= r + diagonal) : (c <= r + diagonal);
            dst[(int64_t)r * cols + c] = in ? one : 0u;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ MX block-scaled fp8 GEMM
 * C = (scaleA (x) A) * (scaleB (x) B)^T as kernels/manual/a5/matmul_mxfp8_performance/scripts/gen_data.py:27-52
 * computes its golden: every fp8 element is multiplied by 2^(scale byte - 127) of its 32-element k block, the
 * products are summed (here exactly, in double) and the sum is returned as float; the caller rounds to bfloat16.
 * a: m x k, b: n x k fp8 bytes (format 0 = float8_e4m3fn, 1 = float8_e5m2); sfa: m x k/32, sfb: n x k/32 e8m0. */
static double fp8_value(uint8_t v, int fmt)
{
    int sign = v >> 7;
    double r;
    if (fmt == 1) { /* e5m2: the upper byte of an IEEE half */
        r = (double)half_to_f32((uint16_t)((uint16_t)v << 8));
        return r;
    }
    int e = (v >> 3) & 15, mnt = v & 7;
    if (e == 15 && mnt == 7) {
        return NAN; /* e4m3fn: the only non-finite code */
    }
    r = e == 0 ? ldexp((double)mnt, -9) : ldexp((double)(8 + mnt), e - 10);
    return sign ? -r : r;
}

typedef struct {
    const uint8_t *a, *b, *sfa, *sfb;
    float *c;
    int m, n, k, c0, c1;
    const double *lut_a, *lut_b;
} mx_ctx;

static void mx_rows(int64_t begin, int64_t end, void *ctx)
{
    const mx_ctx *g = (const mx_ctx *)ctx;
    int ks = g->k / 32;
    for (int64_t i = begin; i < end; ++i) {
        for (int j = g->c0; j < g->c1; ++j) {
            double sum = 0.0;
            for (int blk = 0; blk < ks; ++blk) {
                double part = 0.0;
                const uint8_t *pa = g->a + i * g->k + blk * 32, *pb = g->b + (int64_t)j * g->k + blk * 32;
                for (int t = 0; t < 32; ++t) {
                    part += g->lut_a[pa[t]] * g->lut_b[pb[t]];
                }
                int ea = g->sfa[i * ks + blk], eb = g->sfb[(int64_t)j * ks + blk];
                sum += (ea == 255 || eb == 255) ? NAN : ldexp(part, ea + eb - 254);
            }
            g->c[i * g->n + j] = (float)sum;
        }
    }
}

int pto_oracle_mxgemm_fp8_window(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, float *c, int m,
                                 int n, int k, int a_fmt, int b_fmt, int r0, int r1, int c0, int c1)
{
    if (k % 32 || a_fmt < 0 || a_fmt > 1 || b_fmt < 0 || b_fmt > 1 || r0 < 0 || r1 > m || c0 < 0 || c1 > n) {
        return -1;
    }
    double lut[2][256];
    for (int f = 0; f < 2; ++f) {
        for (int v = 0; v < 256; ++v) {
            lut[f][v] = fp8_value((uint8_t)v, f);
        }
    }
    mx_ctx g = {a, b, sfa, sfb, c, m, n, k, c0, c1, lut[a_fmt], lut[b_fmt]};
    parallel_range(r0, r1, mx_rows, &g);
    return 0;
}

/* Packed fp4 form (kernels/manual/a5/matmul_mxfp4_performance/scripts/gen_data.py:24-34,37-66): two float4_e2m1 values per
 * byte, element 2i in the low nibble and element 2i + 1 in the high nibble; a: m x k/2, b: n x k/2 bytes.
 * e2m1 codes 0..7 are 0, 0.5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign. */
int pto_oracle_mxgemm_fp4_window(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, float *c, int m,
                                 int n, int k, int r0, int r1, int c0, int c1)
{
    static const double mag[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
    if (k % 32 || r0 < 0 || r1 > m || c0 < 0 || c1 > n) {
        return -1;
    }
    int ks = k / 32, kb = k / 2;
    for (int i = r0; i < r1; ++i) {
        for (int j = c0; j < c1; ++j) {
            double sum = 0.0;
            for (int blk = 0; blk < ks; ++blk) {
                double part = 0.0;
                for (int t = 0; t < 32; ++t) {
                    int e = blk * 32 + t;
                    uint8_t ba = a[(int64_t)i * kb + e / 2], bb = b[(int64_t)j * kb + e / 2];
                    int va = (e & 1) ? (ba >> 4) : (ba & 15), vb = (e & 1) ? (bb >> 4) : (bb & 15);
                    double x = (va & 8) ? -mag[va & 7] : mag[va & 7], y = (vb & 8) ? -mag[vb & 7] : mag[vb & 7];
                    part += x * y;
                }
                int ea = sfa[(int64_t)i * ks + blk], eb = sfb[(int64_t)j * ks + blk];
                sum += (ea == 255 || eb == 255) ? NAN : ldexp(part, ea + eb - 254);
            }
            c[(int64_t)i * n + j] = (float)sum;
        }
    }
    return 0;
}

int pto_oracle_mxgemm_fp8(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb, float *c, int m, int n,
                          int k, int a_fmt, int b_fmt)
{
    return pto_oracle_mxgemm_fp8_window(a, b, sfa, sfb, c, m, n, k, a_fmt, b_fmt, 0, m, 0, n);
}

/* Single TMATMUL over the whole k extent (no k stepping): tests/cpu/st/testcase/tmatmul cases. */
int pto_oracle_tmatmul_f16f32(const uint16_t *a, const uint16_t *b, float *c, int m, int k, int n)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float s = 0.0f;
            for (int kk = 0; kk < k; ++kk) {
                s += half_to_f32(a[(int64_t)i * k + kk]) * half_to_f32(b[(int64_t)kk * n + j]);
            }
            c[(int64_t)i * n + j] = s;
        }
    }
    return 0;
}

/* (int8, int8 -> int32) form of the same instruction (include/pto/cpu/TMatmul.hpp:22-37,46-51): exact integer sums.
 * a: m x k, b: k x n, row-major. */
int pto_oracle_tmatmul_i8i32(const int8_t *a, const int8_t *b, int32_t *c, int m, int k, int n)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            int32_t s = 0;
            for (int kk = 0; kk < k; ++kk) {
                s += (int32_t)a[(int64_t)i * k + kk] * (int32_t)b[(int64_t)kk * n + j];
            }
            c[(int64_t)i * n + j] = s;
        }
    }
    return 0;
}

int pto_oracle_tmatmul_f32(const float *a, const float *b, float *c, int m, int k, int n)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float s = 0.0f;
            for (int kk = 0; kk < k; ++kk) {
                s += a[(int64_t)i * k + kk] * b[(int64_t)kk * n + j];
            }
            c[(int64_t)i * n + j] = s;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ attention, one head
 * Plain (untiled) sequence of tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp:84-105 with the
 * flash-attention kernel's conventions (kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:
 * 81-97): row max over the raw logits, p = exp(scale * (x - max)), row sum of the fp32 p, p rounded
 * to fp16 before the second product, O = (p16 V) / sum.  Causal adds -3.40282e38 to keys beyond the
 * query position (:64-79). q: s0 x d, k/v: s1 x d (row-major fp16), o: s0 x d fp32. */

typedef struct {
    const uint16_t *q, *k, *v;
    float *o;
    int s0, s1, d, causal, tile_s1;
    float scale;
} attn_ctx;

static void attn_rows_plain(int64_t begin, int64_t end, void *p)
{
    const attn_ctx *a = (const attn_ctx *)p;
    const int s1 = a->s1, d = a->d;
    float *x = (float *)malloc(sizeof(float) * (size_t)s1);
    float *qf = (float *)malloc(sizeof(float) * (size_t)d);
    float *acc = (float *)malloc(sizeof(float) * (size_t)d);
    for (int64_t i = begin; i < end; ++i) {
        for (int t = 0; t < d; ++t) {
            qf[t] = half_to_f32(a->q[i * d + t]);
        }
        for (int j = 0; j < s1; ++j) {
            float s = 0.0f;
            const uint16_t *kr = a->k + (int64_t)j * d;
            for (int t = 0; t < d; ++t) {
                s += qf[t] * half_to_f32(kr[t]);
            }
            if (a->causal) {
                s = s + ((j > i) ? -3.40282e+38f : -0.0f);
            }
            x[j] = s;
        }
        float mx = x[0];
        for (int j = 1; j < s1; ++j) {
            mx = (mx < x[j]) ? x[j] : mx;
        }
        float sum = 0.0f;
        for (int j = 0; j < s1; ++j) {
            float e = (float)exp((double)((x[j] - mx) * a->scale));
            sum += e;
            x[j] = e;
        }
        for (int t = 0; t < d; ++t) {
            acc[t] = 0.0f;
        }
        for (int j = 0; j < s1; ++j) {
            const float pj = half_to_f32(f32_to_half(x[j]));
            const uint16_t *vr = a->v + (int64_t)j * d;
            for (int t = 0; t < d; ++t) {
                acc[t] += pj * half_to_f32(vr[t]);
            }
        }
        for (int t = 0; t < d; ++t) {
            a->o[i * d + t] = acc[t] / sum;
        }
    }
    free(x);
    free(qf);
    free(acc);
}

int pto_oracle_attn_head_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v, float *o, int s0, int s1, int d,
                             int causal, float scale)
{
    attn_ctx a = {q, k, v, o, s0, s1, d, causal, 0, scale};
    parallel_range(0, s0, attn_rows_plain, &a);
    return 0;
}

/* Streaming (tiled) recurrence of the flash-attention kernel, one head:
 * kernels/manual/common/flash_atten/pto_macro_fa_softmax.hpp:47-215, pto_macro_fa_gu.hpp:33-56 and the
 * NumPy model scripts/gen_data.py:32-149.  Keys are consumed in tiles of tile_s1 (256 in the
 * reference); per tile: m_new = max(m_old, rowmax(X)); alpha = exp(scale*(m_old-m_new));
 * p = exp(scale*(X-m_new)); l = alpha*l + rowsum(p); O = O*alpha + fp16(p) V; after the last
 * tile O /= l.  Causal (query block of 128 rows): tiles that start beyond the block's first row are
 * skipped; the tile holding the diagonal gets the -3.40282e38 mask. */
static void attn_rows_tiled(int64_t begin, int64_t end, void *p)
{
    const attn_ctx *a = (const attn_ctx *)p;
    const int s1 = a->s1, d = a->d, ts = a->tile_s1;
    float *x = (float *)malloc(sizeof(float) * (size_t)ts);
    float *qf = (float *)malloc(sizeof(float) * (size_t)d);
    float *acc = (float *)malloc(sizeof(float) * (size_t)d);
    float *pv = (float *)malloc(sizeof(float) * (size_t)d);
    for (int64_t i = begin; i < end; ++i) {
        const int64_t blk0 = (i / 128) * 128; /* first row of this query block (CUBE_S0 = 128) */
        float m_run = 0.0f, l_run = 0.0f;
        int first = 1;
        for (int t = 0; t < d; ++t) {
            qf[t] = half_to_f32(a->q[i * d + t]);
            acc[t] = 0.0f;
        }
        for (int j0 = 0; j0 < s1; j0 += ts) {
            if (a->causal && j0 > blk0) {
                continue; /* fully masked tile: x_exp = 0, exp_max = 1 */
            }
            const int diag = a->causal && (blk0 / ts == j0 / ts);
            for (int jj = 0; jj < ts; ++jj) {
                const int j = j0 + jj;
                float s = 0.0f;
                const uint16_t *kr = a->k + (int64_t)j * d;
                for (int t = 0; t < d; ++t) {
                    s += qf[t] * half_to_f32(kr[t]);
                }
                if (diag) {
                    s = s + ((j > i) ? -3.40282e+38f : -0.0f);
                }
                x[jj] = s;
            }
            float mx = x[0];
            for (int jj = 1; jj < ts; ++jj) {
                mx = (mx < x[jj]) ? x[jj] : mx;
            }
            float alpha = 1.0f;
            if (!first) {
                mx = (mx < m_run) ? m_run : mx;
                alpha = (float)exp((double)((m_run - mx) * a->scale));
            }
            float sum = 0.0f;
            for (int jj = 0; jj < ts; ++jj) {
                float e = (float)exp((double)((x[jj] - mx) * a->scale));
                sum += e;
                x[jj] = e;
            }
            for (int t = 0; t < d; ++t) {
                pv[t] = 0.0f;
            }
            for (int jj = 0; jj < ts; ++jj) {
                const float pj = half_to_f32(f32_to_half(x[jj]));
                const uint16_t *vr = a->v + (int64_t)(j0 + jj) * d;
                for (int t = 0; t < d; ++t) {
                    pv[t] += pj * half_to_f32(vr[t]);
                }
            }
            if (first) {
                l_run = sum;
                for (int t = 0; t < d; ++t) {
                    acc[t] = pv[t];
                }
                first = 0;
            } else {
                l_run = alpha * l_run + sum;
                for (int t = 0; t < d; ++t) {
                    acc[t] = acc[t] * alpha + pv[t];
                }
            }
            m_run = mx;
        }
        for (int t = 0; t < d; ++t) {
            a->o[i * d + t] = acc[t] / l_run;
        }
    }
    free(x);
    free(qf);
    free(acc);
    free(pv);
}

int pto_oracle_fa_tiled_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v, float *o, int s0, int s1, int d,
                            int causal, float scale, int tile_s1)
{
    if (tile_s1 <= 0 || s1 % tile_s1) {
        return -1;
    }
    attn_ctx a = {q, k, v, o, s0, s1, d, causal, tile_s1, scale};
    parallel_range(0, s0, attn_rows_tiled, &a);
    return 0;
}

/* fp32 -> fp16 of a finished output, for checking a half-precision O against fp16(oracle O). */
int pto_oracle_f32_to_f16(const float *src, uint16_t *dst, int64_t n)
{
    return pto_oracle_tcvt_f32_f16(src, dst, n);
}

int pto_oracle_f16_to_f32(const uint16_t *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = half_to_f32(src[i]);
    }
    return 0;
}

/* The reference's own attention unit test in fp32 (tests/cpu/st/testcase/tflashattn/tflashattn_kernel.cpp:
 * 84-105): scores = (Q K^T) * scale; p = exp(scores - rowmax) / rowsum; O = p V, all fp32. */
int pto_oracle_attn_head_f32_plain(const float *q, const float *k, const float *v, float *o, int s, int d)
{
    const float scale = 1.0f / sqrtf((float)d);
    float *x = (float *)malloc(sizeof(float) * (size_t)s);
    for (int i = 0; i < s; ++i) {
        for (int j = 0; j < s; ++j) {
            float acc = 0.0f;
            for (int t = 0; t < d; ++t) {
                acc += q[(int64_t)i * d + t] * k[(int64_t)j * d + t];
            }
            x[j] = acc * scale;
        }
        float mx = x[0];
        for (int j = 1; j < s; ++j) {
            mx = (mx < x[j]) ? x[j] : mx;
        }
        float sum = 0.0f;
        for (int j = 0; j < s; ++j) {
            x[j] = (float)exp((double)(x[j] - mx));
            sum += x[j];
        }
        for (int j = 0; j < s; ++j) {
            x[j] = x[j] / sum;
        }
        for (int t = 0; t < d; ++t) {
            float acc = 0.0f;
            for (int j = 0; j < s; ++j) {
                acc += x[j] * v[(int64_t)j * d + t];
            }
            o[(int64_t)i * d + t] = acc;
        }
    }
    free(x);
    return 0;
}

/* ------------------------------------------------------------------ FA-adjacent vector ops (second batch)
 * Row-expand family, column reductions, TROWMIN, TFILLPAD, TTRANS, TSEL, TCMP / TCMPS.
 * All tensors are dense row-major; `cols` is both the valid width and the row pitch. */

/* ElementOpCal of include/pto/cpu/ElementOp.h: ADD :85-95, SUB :98-108, MUL, DIV, MAX :201-211 (std::max),
 * MIN :214-224 (std::min), EXPDIF :265-270 (float(exp(double(a - b)))).  Codes as in include/pto_b200.h. */
static inline float elem_op(int op, float a, float b)
{
    switch (op) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return (a < b) ? b : a; /* std::max(a, b) */
        case 5: return (b < a) ? b : a; /* std::min(a, b) */
        case 6: return (float)exp((double)(a - b));
        default: return b;              /* 7: plain TROWEXPAND, include/pto/cpu/TRowExpand.hpp:22-37 */
    }
}

/* TROWEXPAND{ADD,SUB,MUL,DIV,MAX,MIN,EXPDIF} and TROWEXPAND: dst[r, c] = a[r, c] op s[r]
 * (include/pto/cpu/TRowExpandOp.hpp:38-57; s read from column 0 of an R x 1 tile, :22-33). */
int pto_oracle_trowexpand_f32(const float *a, const float *s, float *dst, int rows, int cols, int op)
{
    if (op < 0 || op > 7) {
        return -1;
    }
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            const int64_t i = (int64_t)r * cols + c;
            dst[i] = elem_op(op, op == 7 ? 0.0f : a[i], s[r]);
        }
    }
    return 0;
}

/* TROWMIN (include/pto/cpu/TRowMin.hpp:21-41): first element, then std::min left to right. */
int pto_oracle_trowmin_f32(const float *src, float *dst, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        float m = src[(int64_t)r * cols];
        for (int c = 1; c < cols; ++c) {
            const float x = src[(int64_t)r * cols + c];
            m = (x < m) ? x : m;
        }
        dst[r] = m;
    }
    return 0;
}

/* TCOLSUM / TCOLMAX / TCOLMIN: dst[c] over the rows, top to bottom (include/pto/cpu/TColSum.hpp:19-30 sequential
 * fp32 sum from 0; TColMax.hpp:19-33 and TColMin.hpp start from row 0 and replace on strict > / <).
 * op: 0 = sum, 4 = max, 5 = min. */
int pto_oracle_tcolreduce_f32(const float *src, float *dst, int rows, int cols, int op)
{
    if (op != 0 && op != 4 && op != 5) {
        return -1;
    }
    for (int c = 0; c < cols; ++c) {
        float acc = (op == 0) ? 0.0f : src[c];
        for (int r = (op == 0) ? 0 : 1; r < rows; ++r) {
            const float x = src[(int64_t)r * cols + c];
            if (op == 0) {
                acc += x;
            } else if (op == 4) {
                acc = (x > acc) ? x : acc;
            } else {
                acc = (x < acc) ? x : acc;
            }
        }
        dst[c] = acc;
    }
    return 0;
}

/* TFILLPAD (include/pto/cpu/TFillPad.hpp:19-49): dst is rows x cols; the valid_rows x valid_cols corner is copied
 * from src (same pitch), everything else becomes the pad value.  Elements are 32-bit patterns; the caller picks
 * the pattern that PadValue::Zero / Max / Min mean for its type (:24-36: +inf / -inf for floating types). */
int pto_oracle_tfillpad_b32(const uint32_t *src, uint32_t *dst, int rows, int cols, int valid_rows, int valid_cols,
                            uint32_t pad)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            const int64_t i = (int64_t)r * cols + c;
            dst[i] = (r < valid_rows && c < valid_cols) ? src[i] : pad;
        }
    }
    return 0;
}

/* TTRANS (include/pto/cpu/TTrans.hpp:17-45, plain layouts): dst[c, r] = src[r, c]; src rows x cols, dst cols x rows. */
int pto_oracle_ttrans_b32(const uint32_t *src, uint32_t *dst, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            dst[(int64_t)c * rows + r] = src[(int64_t)r * cols + c];
        }
    }
    return 0;
}
int pto_oracle_ttrans_b16(const uint16_t *src, uint16_t *dst, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            dst[(int64_t)c * rows + r] = src[(int64_t)r * cols + c];
        }
    }
    return 0;
}

/* TSEL (include/pto/cpu/TSel.hpp:22-46): the mask bytes are consumed bit by bit, least significant first, in
 * row-major order over the valid region: element i = r * cols + c takes src0 when bit (i & 7) of byte (i >> 3)
 * is set, else src1. */
int pto_oracle_tsel_b32(const uint8_t *mask, const uint32_t *src0, const uint32_t *src1, uint32_t *dst, int rows,
                        int cols)
{
    const int64_t n = (int64_t)rows * cols;
    for (int64_t i = 0; i < n; ++i) {
        dst[i] = ((mask[i >> 3] >> (i & 7)) & 1) ? src0[i] : src1[i];
    }
    return 0;
}

/* CmpCall of include/pto/cpu/TCmps.hpp:23-52: EQ / NE compare |a - b| in double against 1e-9, the others are the
 * plain operators.  Modes: EQ 0, NE 1, LT 2, LE 3, GT 4, GE 5 (include/pto/common/type.hpp:131-139). */
static inline int cmp_call(float a, float b, int mode)
{
    const double diff = (double)a - (double)b;
    switch (mode) {
        case 0: return fabs(diff) < 1e-9;
        case 1: return fabs(diff) > 1e-9;
        case 2: return a < b;
        case 3: return a <= b;
        case 4: return a > b;
        case 5: return a >= b;
        default: return fabs(diff) < 1e-9;
    }
}

/* TCMPS (include/pto/cpu/TCmps.hpp:54-91): one result bit per element, packed least significant bit first,
 * cols / 8 bytes per row, rows back to back.  cols must be a multiple of 8. */
int pto_oracle_tcmps_f32(const float *src, float scalar, uint8_t *dst, int rows, int cols, int mode)
{
    if (cols % 8 != 0) {
        return -1;
    }
    const int64_t n = (int64_t)rows * cols;
    for (int64_t b = 0; b < n / 8; ++b) {
        uint8_t v = 0;
        for (int bit = 0; bit < 8; ++bit) {
            v |= (uint8_t)(cmp_call(src[b * 8 + bit], scalar, mode) << bit);
        }
        dst[b] = v;
    }
    return 0;
}

/* TCMP in the CPU simulation (include/pto/cpu/ElementTileOp.h:177-184, ElementOp.h:227-254): the result tile has
 * the operands' type and holds 1 or 0 from the plain C++ operators. */
int pto_oracle_tcmp_f32(const float *a, const float *b, float *dst, int64_t n, int mode)
{
    for (int64_t i = 0; i < n; ++i) {
        int r;
        switch (mode) {
            case 0: r = a[i] == b[i]; break;
            case 1: r = a[i] != b[i]; break;
            case 2: r = a[i] < b[i]; break;
            case 3: r = a[i] <= b[i]; break;
            case 4: r = a[i] > b[i]; break;
            case 5: r = a[i] >= b[i]; break;
            default: r = a[i] == b[i]; break;
        }
        dst[i] = (float)r;
    }
    return 0;
}
