// Host-side support shared by the kernels: device queries, error text, the device status record that
// bounded waits report into, and TMA tensor-map encoding (driver entry point resolved at run time so the
// library has no link-time dependency on libcuda).
#include "ptx.cuh"
#include "internal.h"

#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

namespace pto_b200 {

namespace {

constexpr int kMaxDevices = 64;
thread_local char g_error_text[512] = "";
thread_local int g_last_status = 0;
int g_sm_count[kMaxDevices] = {0};
DeviceStatus *g_status[kMaxDevices] = {nullptr};
std::mutex g_mutex;

int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        return -1;
    }
    return dev;
}

} // namespace

void set_error_text(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error_text, sizeof(g_error_text), fmt, ap);
    va_end(ap);
}

const char *error_text()
{
    return g_error_text;
}

void set_last_status(int code)
{
    g_last_status = code;
}

int last_status()
{
    return g_last_status;
}

int check_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) {
        return kOk;
    }
    set_error_text("%s: %s", what, cudaGetErrorString(e));
    return kErrCuda;
}

int check_launch()
{
    return check_cuda(cudaGetLastError(), "kernel launch");
}

int current_device_ordinal()
{
    return current_device();
}

int ensure_dynamic_smem(const void *kernel, int bytes)
{
    // (kernel, device) pairs already raised; a handful of kernels times a handful of devices
    static std::vector<std::pair<const void *, int>> done;
    const int dev = current_device();
    if (dev < 0) {
        set_error_text("no current CUDA device");
        return kErrCuda;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    for (const auto &e : done) {
        if (e.first == kernel && e.second == dev) {
            return kOk;
        }
    }
    const int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
                              "cudaFuncSetAttribute(max dynamic shared memory)");
    if (rc == kOk) {
        done.emplace_back(kernel, dev);
    }
    return rc;
}

int sm_count()
{
    const int dev = current_device();
    if (dev < 0) {
        return 1;
    }
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            n = 1;
        }
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

DeviceStatus *device_status_ptr()
{
    const int dev = current_device();
    if (dev < 0) {
        set_error_text("no current CUDA device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status[dev] == nullptr) {
        DeviceStatus *p = nullptr;
        if (check_cuda(cudaMalloc(&p, sizeof(DeviceStatus)), "cudaMalloc(status)") != kOk) {
            return nullptr;
        }
        if (check_cuda(cudaMemset(p, 0, sizeof(DeviceStatus)), "cudaMemset(status)") != kOk) {
            cudaFree(p);
            return nullptr;
        }
        g_status[dev] = p;
    }
    return g_status[dev];
}

int fetch_device_status(cudaStream_t stream, int *record)
{
    DeviceStatus *p = device_status_ptr();
    if (p == nullptr) {
        return kErrCuda;
    }
    DeviceStatus h;
    int rc = check_cuda(cudaMemcpyAsync(&h, p, sizeof(h), cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync(status)");
    if (rc != kOk) {
        return rc;
    }
    rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (rc != kOk) {
        return rc;
    }
    if (record != nullptr) {
        record[0] = h.code;
        record[1] = h.block;
        record[2] = h.where;
        record[3] = h.detail;
    }
    if (h.code != 0) {
        set_error_text("device-side wait gave up: code %d, block %d, where %d, detail %d", h.code, h.block, h.where,
                       h.detail);
        cudaMemsetAsync(p, 0, 4 * sizeof(int), stream); // the four status words; the profile settings stay
    }
    return h.code;
}

int set_profile_buffer(unsigned long long *stamps, long long capacity_blocks, cudaStream_t stream)
{
    DeviceStatus *p = device_status_ptr();
    if (p == nullptr) {
        return kErrCuda;
    }
    struct {
        unsigned long long *stamps;
        long long cap;
    } v = {stamps, stamps == nullptr ? 0 : capacity_blocks};
    int rc = check_cuda(cudaMemcpyAsync(reinterpret_cast<char *>(p) + offsetof(DeviceStatus, stamps), &v, sizeof(v),
                                        cudaMemcpyHostToDevice, stream),
                        "cudaMemcpyAsync(profile settings)");
    if (rc == kOk) {
        rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    }
    return rc;
}

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes)
{
    return elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : (elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32);
}

int make_tmap_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols, bool swizzle128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_error_text("cuTensorMapEncodeTiled is not available from this driver");
        return kErrCuda;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_elems * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(map, dtype_of(elem_bytes), 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error_text("cuTensorMapEncodeTiled(2d) failed with CUresult %d (rows %llu cols %llu pitch %llu box %ux%u)",
                       static_cast<int>(r), static_cast<unsigned long long>(rows),
                       static_cast<unsigned long long>(cols), static_cast<unsigned long long>(strides[0]), box_rows,
                       box_cols);
        return kErrCuda;
    }
    return kOk;
}

int make_tmap_3d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t outer, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_elems, uint64_t outer_stride_elems, uint32_t box_rows, uint32_t box_cols,
                 bool swizzle128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        set_error_text("cuTensorMapEncodeTiled is not available from this driver");
        return kErrCuda;
    }
    const cuuint64_t dims[3] = {cols, rows, outer};
    const cuuint64_t strides[2] = {row_stride_elems * static_cast<uint64_t>(elem_bytes),
                                   outer_stride_elems * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[3] = {box_cols, box_rows, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    const CUresult r = fn(map, dtype_of(elem_bytes), 3, const_cast<void *>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error_text("cuTensorMapEncodeTiled(3d) failed with CUresult %d", static_cast<int>(r));
        return kErrCuda;
    }
    return kOk;
}

int grid_for(int64_t work_items, int items_per_block)
{
    int64_t blocks = (work_items + items_per_block - 1) / items_per_block;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32; // grid-stride beyond this
    if (blocks > cap) {
        // every block makes the same number of passes (the last one possibly short): a grid of exactly `cap` blocks
        // would leave some blocks with one pass more than others and a tail in which most of the GPU idles
        const int64_t passes = (blocks + cap - 1) / cap;
        blocks = (blocks + passes - 1) / passes;
    }
    if (blocks < 1) {
        blocks = 1;
    }
    return static_cast<int>(blocks);
}

} // namespace pto_b200
