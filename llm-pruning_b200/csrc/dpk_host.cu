// Host-side plumbing of the C ABI: error text, tensor-map encoding through the
// driver entry point, cached device properties, the device status word.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "dpk_host.h"

namespace dpk {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

static int make_tmap(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                     uint64_t row_stride_elems, uint32_t box_cols, uint32_t box_rows,
                     CUtensorMapSwizzle swz)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(DPK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (!aligned16(base) || (row_stride_elems * 2) % 16 != 0)
        return fail(DPK_ERR_INVALID, "tensor base and row stride must be 16-byte aligned");
    if (box_rows == 0 || box_rows > 256 || box_cols == 0 || box_cols > 256)
        return fail(DPK_ERR_INVALID, "tensor-map box %ux%u out of range", box_cols, box_rows);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    // fp16 and bf16 are both plain 16-bit payloads to the copy engine
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DPK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (cols=%llu rows=%llu)",
                    (int)r, (unsigned long long)cols, (unsigned long long)rows);
    return DPK_OK;
}

int make_tmap_3d_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t batches, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                       uint32_t box_cols, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(DPK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (box_cols != 64) return fail(DPK_ERR_INVALID, "128-byte swizzle needs a 64-element box row");
    if (!aligned16(base) || (row_stride_elems * 2) % 16 != 0 || (batch_stride_elems * 2) % 16 != 0)
        return fail(DPK_ERR_INVALID, "tensor base, row stride and batch stride must be 16-byte aligned");
    if (box_rows == 0 || box_rows > 256)
        return fail(DPK_ERR_INVALID, "tensor-map box %ux%u out of range", box_cols, box_rows);
    if (batches == 0) batches = 1;
    if (batches == 1) batch_stride_elems = rows * row_stride_elems;    // unused, but must be valid
    cuuint64_t dims[3] = {cols, rows, batches};
    cuuint64_t strides[2] = {row_stride_elems * 2, batch_stride_elems * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DPK_ERR_CUDA,
                    "cuTensorMapEncodeTiled (3-D) failed with code %d (cols=%llu rows=%llu batches=%llu)",
                    (int)r, (unsigned long long)cols, (unsigned long long)rows,
                    (unsigned long long)batches);
    return DPK_OK;
}

int make_tmap_2d_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t row_stride_elems, uint32_t box_cols, uint32_t box_rows)
{
    if (box_cols != 64) return fail(DPK_ERR_INVALID, "128-byte swizzle needs a 64-element box row");
    return make_tmap(map, base, cols, rows, row_stride_elems, box_cols, box_rows,
                     CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tmap_2d_plain(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t row_stride_elems, uint32_t box_cols, uint32_t box_rows)
{
    return make_tmap(map, base, cols, rows, row_stride_elems, box_cols, box_rows,
                     CU_TENSOR_MAP_SWIZZLE_NONE);
}

static const int kMaxDev = 64;
static int g_sm_margin = 0;

int sm_count()
{
    static int cached[kMaxDev] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    const int usable = cached[dev] - g_sm_margin;
    return usable < 1 ? 1 : usable;
}

__device__ int g_dpk_status = 0;

int* device_status_ptr()
{
    static int* cached[kMaxDev] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dpk_status) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int*>(p);
    }
    return cached[dev];
}

}  // namespace dpk

extern "C" {

int dpk_version(void) { return 100; }

int dpk_set_sm_margin(int sms)
{
    DPK_REQUIRE(sms >= 0 && sms < 128, "margin %d outside [0,128)", sms);
    dpk::g_sm_margin = sms;
    return DPK_OK;
}

const char* dpk_last_error(void) { return dpk::g_err; }

int dpk_device_status(int* status, void* stream)
{
    DPK_REQUIRE(status != nullptr, "status must not be NULL");
    int* dptr = dpk::device_status_ptr();
    if (!dptr) return dpk::fail(DPK_ERR_CUDA, "no status word on this device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DPK_CUDA(cudaMemcpyAsync(status, dptr, sizeof(int), cudaMemcpyDeviceToHost, s));
    DPK_CUDA(cudaStreamSynchronize(s));
    if (*status != 0) DPK_CUDA(cudaMemsetAsync(dptr, 0, sizeof(int), s));
    return DPK_OK;
}

}  // extern "C"
