// C++ host in the shape of the reference's kernel hosts (kernels/manual/a2a3/gemm_performance/main.cpp:22-98,
// kernels/manual/common/flash_atten/main.cpp:124-614): read the case's .bin inputs, copy them to the device, call the
// launcher template the reference's host calls (include/pto_b200_launchers.hpp), synchronise, copy the result back,
// write it next to the golden and compare with the reference's ResultCmp rule (tests/common/test_common.h:211-300:
// an element is wrong when |diff| > eps and |diff / expected| > eps; the case passes while the wrong elements number
// at most size * eps and fewer than 1000 outputs are zero where the golden is not).
//
//   pto_b200_host gemm <case_dir> [m k n]        input/x1_gm.bin (m x k half), input/x2_gm.bin (n x k half),
//                                                output/golden.bin (m x n float) -> output/output_z.bin; default 6144^3
//   pto_b200_host fa <case_dir> <s0> <s1> <causal>   q.bin, kt.bin (K rows: s1 x 128 half), v.bin, o.bin (golden, float)
//                                                -> o_out.bin; head size 128
//   pto_b200_host tmatmul <case_dir> <key>       the reference's TMATMUL unit-test cases (tests/cpu/st/testcase/tmatmul/
//                                                main.cpp:97-170): x1_gm.bin, x2_gm.bin, golden.bin -> output.bin;
//                                                key 1 half 40x50x60, 3 five half 128x128x64 products, 4 float 120x110x50
// Exit code 0 and "test success" when the comparison passes.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/pto_b200_launchers.hpp"

namespace {

bool read_file(const std::string &path, void *dst, size_t bytes)
{
    FILE *f = std::fopen(path.c_str(), "rb");
    if (f == nullptr) {
        std::fprintf(stderr, "cannot open %s\n", path.c_str());
        return false;
    }
    const size_t got = std::fread(dst, 1, bytes, f);
    std::fclose(f);
    if (got != bytes) {
        std::fprintf(stderr, "%s: expected %zu bytes, read %zu\n", path.c_str(), bytes, got);
        return false;
    }
    return true;
}

bool write_file(const std::string &path, const void *src, size_t bytes)
{
    FILE *f = std::fopen(path.c_str(), "wb");
    if (f == nullptr) {
        std::fprintf(stderr, "cannot create %s\n", path.c_str());
        return false;
    }
    const size_t put = std::fwrite(src, 1, bytes, f);
    std::fclose(f);
    return put == bytes;
}

bool result_cmp(const std::vector<float> &golden, const std::vector<float> &actual, float eps)
{
    size_t wrong = 0, zeros = 0;
    float max_diff = 0.f, max_ratio = 0.f;
    for (size_t i = 0; i < golden.size(); ++i) {
        const float diff = std::fabs(golden[i] - actual[i]);
        const float ratio = std::fabs(diff / golden[i]);
        max_diff = std::fmax(max_diff, diff);
        if (std::isfinite(ratio)) {
            max_ratio = std::fmax(max_ratio, ratio);
        }
        zeros += (std::fabs(actual[i]) <= 1e-6f && std::fabs(golden[i]) > 1e-6f) ? 1 : 0;
        wrong += (diff > eps && ratio > eps) ? 1 : 0;
        if (std::isnan(golden[i]) != std::isnan(actual[i])) {
            ++wrong;
        }
    }
    const size_t allowed = static_cast<size_t>(golden.size() * eps);
    std::printf("max diff: %g, diff threshold: %g, max diff ratio: %g, err count: %zu, err threshold: %zu, act zero count: %zu\n",
                max_diff, eps, max_ratio, wrong, allowed, zeros);
    return wrong <= allowed && zeros <= 1000;
}

#define CUDA_OK(x)                                                                       \
    do {                                                                                 \
        cudaError_t e_ = (x);                                                            \
        if (e_ != cudaSuccess) {                                                         \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));               \
            return 2;                                                                    \
        }                                                                                \
    } while (0)

int run_gemm(const std::string &dir, uint32_t m, uint32_t k, uint32_t n)
{
    const size_t a_bytes = size_t(m) * k * 2, b_bytes = size_t(n) * k * 2, c_bytes = size_t(m) * n * 4;
    std::vector<uint8_t> a(a_bytes), b(b_bytes);
    std::vector<float> c(size_t(m) * n), golden(size_t(m) * n);
    if (!read_file(dir + "/input/x1_gm.bin", a.data(), a_bytes) || !read_file(dir + "/input/x2_gm.bin", b.data(), b_bytes)) {
        return 2;
    }
    CUDA_OK(cudaSetDevice(0));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    uint8_t *da, *db, *dc;
    CUDA_OK(cudaMalloc(&da, a_bytes));
    CUDA_OK(cudaMalloc(&db, b_bytes));
    CUDA_OK(cudaMalloc(&dc, c_bytes));
    CUDA_OK(cudaMemcpyAsync(da, a.data(), a_bytes, cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(db, b.data(), b_bytes, cudaMemcpyHostToDevice, stream));
    if (m == 6144 && k == 6144 && n == 6144) {
        LaunchGEMME2E<uint16_t>(dc, da, db, stream);
    } else {
        LaunchGEMME2E<uint16_t>(dc, da, db, stream, m, k, n);
    }
    if (pto_b200_launcher_status() != 0) {
        std::fprintf(stderr, "LaunchGEMME2E failed with status %d\n", pto_b200_launcher_status());
        return 2;
    }
    CUDA_OK(cudaStreamSynchronize(stream));
    CUDA_OK(cudaMemcpy(c.data(), dc, c_bytes, cudaMemcpyDeviceToHost));
    cudaFree(da);
    cudaFree(db);
    cudaFree(dc);
    cudaStreamDestroy(stream);
    if (!write_file(dir + "/output/output_z.bin", c.data(), c_bytes) ||
        !read_file(dir + "/output/golden.bin", golden.data(), c_bytes)) {
        return 2;
    }
    const bool ok = result_cmp(golden, c, 0.001f);
    std::printf(ok ? "test success\n" : "test failed\n");
    return ok ? 0 : 1;
}

template <int S0, int S1, bool CAUSAL>
void launch_fa(aclFloat16 *q, aclFloat16 *k, aclFloat16 *v, float *o, cudaStream_t stream)
{
    LaunchTFA<S0, 128, S1, 128, 128, 256, 4, 8, false, CAUSAL, 4>(nullptr, q, k, v, nullptr, nullptr, nullptr, nullptr, o,
                                                                  nullptr, nullptr, nullptr, stream, nullptr);
}

int run_fa(const std::string &dir, int s0, int s1, int causal)
{
    const size_t q_bytes = size_t(s0) * 128 * 2, kv_bytes = size_t(s1) * 128 * 2, o_bytes = size_t(s0) * 128 * 4;
    std::vector<uint8_t> q(q_bytes), k(kv_bytes), v(kv_bytes);
    std::vector<float> o(size_t(s0) * 128), golden(size_t(s0) * 128);
    if (!read_file(dir + "/q.bin", q.data(), q_bytes) || !read_file(dir + "/kt.bin", k.data(), kv_bytes) ||
        !read_file(dir + "/v.bin", v.data(), kv_bytes)) {
        return 2;
    }
    CUDA_OK(cudaSetDevice(0));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    aclFloat16 *dq, *dk, *dv;
    float *dout;
    CUDA_OK(cudaMalloc(&dq, q_bytes));
    CUDA_OK(cudaMalloc(&dk, kv_bytes));
    CUDA_OK(cudaMalloc(&dv, kv_bytes));
    CUDA_OK(cudaMalloc(&dout, o_bytes));
    CUDA_OK(cudaMemcpyAsync(dq, q.data(), q_bytes, cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(dk, k.data(), kv_bytes, cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(dv, v.data(), kv_bytes, cudaMemcpyHostToDevice, stream));
    if (s0 == 128 && s1 == 1024 && !causal) {
        launch_fa<128, 1024, false>(dq, dk, dv, dout, stream);
    } else if (s0 == 1024 && s1 == 1024 && !causal) {
        launch_fa<1024, 1024, false>(dq, dk, dv, dout, stream);
    } else if (s0 == 1024 && s1 == 1024 && causal) {
        launch_fa<1024, 1024, true>(dq, dk, dv, dout, stream);
    } else if (s0 == 128 && s1 == 2048 && !causal) {
        launch_fa<128, 2048, false>(dq, dk, dv, dout, stream);
    } else {
        std::fprintf(stderr, "fa: no LaunchTFA instance for s0 %d s1 %d causal %d in this host\n", s0, s1, causal);
        return 2;
    }
    if (pto_b200_launcher_status() != 0) {
        std::fprintf(stderr, "LaunchTFA failed with status %d\n", pto_b200_launcher_status());
        return 2;
    }
    CUDA_OK(cudaStreamSynchronize(stream));
    CUDA_OK(cudaMemcpy(o.data(), dout, o_bytes, cudaMemcpyDeviceToHost));
    cudaFree(dq);
    cudaFree(dk);
    cudaFree(dv);
    cudaFree(dout);
    cudaStreamDestroy(stream);
    if (!write_file(dir + "/o_out.bin", o.data(), o_bytes) || !read_file(dir + "/o.bin", golden.data(), o_bytes)) {
        return 2;
    }
    std::printf("[CHECK] O running output compare\n");
    const bool ok = result_cmp(golden, o, 0.001f);
    std::printf(ok ? "test success\n" : "test failed\n");
    return ok ? 0 : 1;
}

int run_tmatmul(const std::string &dir, int key)
{
    size_t a_bytes, b_bytes, m, n;
    switch (key) {
        case 1: a_bytes = 40 * 50 * 2; b_bytes = 50 * 60 * 2; m = 40; n = 60; break;
        case 3: a_bytes = 5 * 128 * 128 * 2; b_bytes = 5 * 128 * 64 * 2; m = 128; n = 64; break;
        case 4: a_bytes = 120 * 110 * 4; b_bytes = 110 * 50 * 4; m = 120; n = 50; break;
        default: std::fprintf(stderr, "tmatmul: key 1, 3 or 4\n"); return 2;
    }
    const size_t c_bytes = m * n * 4;
    std::vector<uint8_t> a(a_bytes), b(b_bytes);
    std::vector<float> c(m * n), golden(m * n);
    if (!read_file(dir + "/x1_gm.bin", a.data(), a_bytes) || !read_file(dir + "/x2_gm.bin", b.data(), b_bytes) ||
        !read_file(dir + "/golden.bin", golden.data(), c_bytes)) {
        return 2;
    }
    CUDA_OK(cudaSetDevice(0));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    uint8_t *da, *db, *dc;
    CUDA_OK(cudaMalloc(&da, a_bytes));
    CUDA_OK(cudaMalloc(&db, b_bytes));
    CUDA_OK(cudaMalloc(&dc, c_bytes));
    CUDA_OK(cudaMemcpyAsync(da, a.data(), a_bytes, cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(db, b.data(), b_bytes, cudaMemcpyHostToDevice, stream));
    if (key == 1) {
        LaunchTMATMUL<1>(dc, da, db, stream);
    } else if (key == 3) {
        LaunchTMATMUL<3>(dc, da, db, stream);
    } else {
        LaunchTMATMUL<4>(dc, da, db, stream);
    }
    if (pto_b200_launcher_status() != 0) {
        std::fprintf(stderr, "LaunchTMATMUL failed with status %d\n", pto_b200_launcher_status());
        return 2;
    }
    CUDA_OK(cudaStreamSynchronize(stream));
    CUDA_OK(cudaMemcpy(c.data(), dc, c_bytes, cudaMemcpyDeviceToHost));
    cudaFree(da);
    cudaFree(db);
    cudaFree(dc);
    cudaStreamDestroy(stream);
    if (!write_file(dir + "/output.bin", c.data(), c_bytes)) {
        return 2;
    }
    const bool ok = result_cmp(golden, c, 0.001f);
    std::printf(ok ? "test success\n" : "test failed\n");
    return ok ? 0 : 1;
}

} // namespace

int main(int argc, char **argv)
{
    if (argc >= 3 && std::strcmp(argv[1], "gemm") == 0) {
        uint32_t m = 6144, k = 6144, n = 6144;
        if (argc >= 6) {
            m = static_cast<uint32_t>(std::atoi(argv[3]));
            k = static_cast<uint32_t>(std::atoi(argv[4]));
            n = static_cast<uint32_t>(std::atoi(argv[5]));
        }
        return run_gemm(argv[2], m, k, n);
    }
    if (argc >= 6 && std::strcmp(argv[1], "fa") == 0) {
        return run_fa(argv[2], std::atoi(argv[3]), std::atoi(argv[4]), std::atoi(argv[5]));
    }
    if (argc >= 4 && std::strcmp(argv[1], "tmatmul") == 0) {
        return run_tmatmul(argv[2], std::atoi(argv[3]));
    }
    std::fprintf(stderr, "usage: %s gemm <case_dir> [m k n] | fa <case_dir> <s0> <s1> <causal> | tmatmul <case_dir> <key>\n",
                 argv[0]);
    return 2;
}
