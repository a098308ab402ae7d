// Host-side helpers shared by the C-ABI entry points: error reporting, argument
// checks, tensor-map encoding through the driver entry point (no link-time libcuda
// dependency, so the library loads on a machine without a GPU), device properties.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/dpk_b200.h"

namespace dpk {

// Stores a printf-style message for dpk_last_error() (thread local) and returns `code`.
int fail(int code, const char* fmt, ...);

#define DPK_REQUIRE(cond, ...)                                      \
    do {                                                            \
        if (!(cond)) return ::dpk::fail(DPK_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define DPK_CUDA(expr)                                                                   \
    do {                                                                                 \
        cudaError_t e__ = (expr);                                                        \
        if (e__ != cudaSuccess)                                                          \
            return ::dpk::fail(DPK_ERR_CUDA, "%s failed at %s:%d: %s", #expr, __FILE__,  \
                               __LINE__, cudaGetErrorString(e__));                       \
    } while (0)

// Row-major 2-D tensor of 16-bit elements: `cols` contiguous elements per row, rows
// `row_stride_elems` apart.  The box is `box_cols` x `box_rows` and lands in shared
// memory under the 128-byte swizzle (box_cols must be 64).
int make_tmap_2d_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t row_stride_elems, uint32_t box_cols, uint32_t box_rows);

// Batched form: `batches` such 2-D tensors `batch_stride_elems` apart, as a 3-D map whose box is
// `box_cols` x `box_rows` x 1, so that rows past the end of one batch entry are zero-filled
// instead of running into the next entry (or into unused capacity of a cache).
int make_tmap_3d_sw128(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t batches, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                       uint32_t box_cols, uint32_t box_rows);

// Same, without swizzle (rows of the box stored back to back).
int make_tmap_2d_plain(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                       uint64_t row_stride_elems, uint32_t box_cols, uint32_t box_rows);

// Number of SMs of the current device (cached per device).
int sm_count();

// Address of the per-device status word kernels report into.
int* device_status_ptr();

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace dpk
