// Routing kernels: top-k mask, routing layout (stable active-first compaction per
// group column), per-column counts of a given layout, packed row / window bits.
//
// All of this is integer work bounded by HBM traffic: the byte mask is read twice
// (M*NG bytes each) and sorted_indices + sorted_mask are written once (9*M*NG
// bytes).  Reads go through a shared-memory tile so that global accesses are
// row-contiguous; writes of sorted_indices are 8-byte scatters by construction of
// the [M,NG] layout the operator API returns.
#define DPK_KERNEL_ID 7   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kRouteRows = 256;   // rows per CTA tile
constexpr int kRouteCols = 32;    // group columns per CTA tile
constexpr int kRouteThreads = 256;

// Loads the [256 x 32] byte tile of `mask` at (r0, c0) into shared memory as 0/1.
__device__ __forceinline__ void route_load_tile(const uint8_t* __restrict__ mask, int64_t M, int NG,
                                                int64_t r0, int c0,
                                                uint8_t (*tile)[kRouteCols + 4])
{
    for (int i = threadIdx.x; i < kRouteRows * kRouteCols; i += kRouteThreads) {
        int row = i / kRouteCols, col = i % kRouteCols;
        int64_t r = r0 + row;
        int c = c0 + col;
        uint8_t v = 0;
        if (r < M && c < NG) v = mask[r * NG + c] != 0;
        tile[row][col] = v;
    }
}

// pass 1: active rows of every (row block, column); optionally also the packed routing
// bits of the reduction-width GEMM (row_bits / win_bits, see mask_pack_kernel), which come
// for free from the tile that is already in shared memory
__global__ void __launch_bounds__(kRouteThreads)
route_count_kernel(const uint8_t* __restrict__ mask, int64_t M, int NG, int nrb,
                   int32_t* __restrict__ block_cnt, uint32_t* __restrict__ row_bits,
                   uint32_t* __restrict__ win_bits, int words)
{
    __shared__ uint8_t tile[kRouteRows][kRouteCols + 4];
    __shared__ uint32_t win_or[kRouteThreads / 32];
    const int b = blockIdx.z;
    const int rb = blockIdx.x;
    const int c0 = blockIdx.y * kRouteCols;
    const int64_t r0 = static_cast<int64_t>(rb) * kRouteRows;
    mask += static_cast<int64_t>(b) * M * NG;
    route_load_tile(mask, M, NG, r0, c0, tile);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int col = warp; col < kRouteCols; col += kRouteThreads / 32) {
        int c = c0 + col;
        if (c >= NG) break;
        int total = 0;
        for (int chunk = 0; chunk < kRouteRows / 32; ++chunk) {
            unsigned bal = __ballot_sync(0xffffffffu, tile[chunk * 32 + lane][col] != 0);
            total += __popc(bal);
        }
        if (lane == 0) block_cnt[(static_cast<int64_t>(b) * nrb + rb) * NG + c] = total;
    }
    if (row_bits != nullptr) {
        // warp w packs rows [32w, 32w+32) of the tile: one word (this column block) per row
        uint32_t acc = 0;
        for (int i = 0; i < 32; ++i) {
            const int row = warp * 32 + i;
            const uint32_t bits = __ballot_sync(0xffffffffu, tile[row][lane] != 0);
            acc |= bits;
            const int64_t r = r0 + row;
            if (lane == 0 && r < M) row_bits[r * words + blockIdx.y] = bits;
        }
        if (lane == 0) win_or[warp] = acc;
        __syncthreads();
        // the tile covers two 128-row windows: warps 0-3 and warps 4-7
        if (threadIdx.x < 2) {
            const int64_t win = static_cast<int64_t>(rb) * 2 + threadIdx.x;
            if (win * 128 < M) {
                const int w0 = threadIdx.x * 4;
                win_bits[win * words + blockIdx.y] =
                    win_or[w0] | win_or[w0 + 1] | win_or[w0 + 2] | win_or[w0 + 3];
            }
        }
    }
}

// pass 2: exclusive scan over row blocks per column (in place), totals into counts.
// The counters of 16 row blocks are fetched with independent loads before any is
// rewritten, so the latency of the column walk is paid once per 16 blocks.
__global__ void route_scan_kernel(int32_t* __restrict__ block_cnt, int nrb, int NG, int batches,
                                  int32_t* __restrict__ counts)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batches * NG) return;
    int b = i / NG, c = i % NG;
    int32_t run = 0;
    int32_t* p = block_cnt + static_cast<int64_t>(b) * nrb * NG + c;
    for (int rb0 = 0; rb0 < nrb; rb0 += 16) {
        int32_t v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            v[k] = rb0 + k < nrb ? p[static_cast<int64_t>(rb0 + k) * NG] : 0;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (rb0 + k < nrb) p[static_cast<int64_t>(rb0 + k) * NG] = run;
            run += v[k];
        }
    }
    counts[i] = run;
}

// pass 3: write the layout
__global__ void __launch_bounds__(kRouteThreads)
route_scatter_kernel(const uint8_t* __restrict__ mask, int64_t M, int NG, int nrb,
                     const int32_t* __restrict__ block_off, const int32_t* __restrict__ counts,
                     uint8_t* __restrict__ sorted_mask, int64_t* __restrict__ sorted_indices)
{
    __shared__ uint8_t tile[kRouteRows][kRouteCols + 4];
    const int b = blockIdx.z;
    const int rb = blockIdx.x;
    const int c0 = blockIdx.y * kRouteCols;
    const int64_t r0 = static_cast<int64_t>(rb) * kRouteRows;
    const int64_t boff = static_cast<int64_t>(b) * M * NG;
    mask += boff;
    sorted_mask += boff;
    sorted_indices += boff;
    counts += static_cast<int64_t>(b) * NG;
    route_load_tile(mask, M, NG, r0, c0, tile);
    __syncthreads();

    // sorted_mask: row r of column c is active iff r < counts[c]
    for (int i = threadIdx.x; i < kRouteRows * kRouteCols; i += kRouteThreads) {
        int row = i / kRouteCols, col = i % kRouteCols;
        int64_t r = r0 + row;
        int c = c0 + col;
        if (r < M && c < NG) sorted_mask[r * NG + c] = r < counts[c] ? 1 : 0;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned lt = (1u << lane) - 1u;
    for (int col = warp; col < kRouteCols; col += kRouteThreads / 32) {
        int c = c0 + col;
        if (c >= NG) break;
        int64_t act_base = block_off[(static_cast<int64_t>(b) * nrb + rb) * NG + c];
        int64_t ina_base = static_cast<int64_t>(counts[c]) + (r0 - act_base);
        for (int chunk = 0; chunk < kRouteRows / 32; ++chunk) {
            int64_t r = r0 + chunk * 32 + lane;
            bool valid = r < M;
            bool on = tile[chunk * 32 + lane][col] != 0;
            unsigned bal = __ballot_sync(0xffffffffu, on);
            unsigned val = __ballot_sync(0xffffffffu, valid);
            unsigned off = val & ~bal;
            if (valid) {
                int64_t pos = on ? act_base + __popc(bal & lt) : ina_base + __popc(off & lt);
                sorted_indices[pos * NG + c] = r;
            }
            act_base += __popc(bal);
            ina_base += __popc(off);
        }
    }
}

// All three passes in one launch when the tokens fit one row block (M <= 256: decode batches):
// the only row block's offsets are zero, so no scan is needed -- count, write counts and the
// packed bits, then write the layout from the same shared-memory tile.
__global__ void __launch_bounds__(kRouteThreads)
route_one_block_kernel(const uint8_t* __restrict__ mask, int64_t M, int NG,
                       int32_t* __restrict__ counts, uint8_t* __restrict__ sorted_mask,
                       int64_t* __restrict__ sorted_indices, uint32_t* __restrict__ row_bits,
                       uint32_t* __restrict__ win_bits, int words)
{
    __shared__ uint8_t tile[kRouteRows][kRouteCols + 4];
    __shared__ uint32_t win_or[kRouteThreads / 32];
    __shared__ int32_t col_cnt[kRouteCols];
    const int b = blockIdx.z;
    const int c0 = blockIdx.y * kRouteCols;
    const int64_t boff = static_cast<int64_t>(b) * M * NG;
    mask += boff;
    sorted_mask += boff;
    sorted_indices += boff;
    counts += static_cast<int64_t>(b) * NG;
    route_load_tile(mask, M, NG, 0, c0, tile);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int col = warp; col < kRouteCols; col += kRouteThreads / 32) {
        int total = 0;
        for (int chunk = 0; chunk < kRouteRows / 32; ++chunk)
            total += __popc(__ballot_sync(0xffffffffu, tile[chunk * 32 + lane][col] != 0));
        if (lane == 0) {
            col_cnt[col] = total;
            if (c0 + col < NG) counts[c0 + col] = total;
        }
    }
    if (row_bits != nullptr) {
        uint32_t acc = 0;
        for (int i = 0; i < 32; ++i) {
            const int row = warp * 32 + i;
            const uint32_t bits = __ballot_sync(0xffffffffu, tile[row][lane] != 0);
            acc |= bits;
            if (lane == 0 && row < M) row_bits[static_cast<int64_t>(row) * words + blockIdx.y] = bits;
        }
        if (lane == 0) win_or[warp] = acc;
    }
    __syncthreads();
    if (row_bits != nullptr && threadIdx.x < 2 && threadIdx.x * 128 < M) {
        const int w0 = threadIdx.x * 4;
        win_bits[static_cast<int64_t>(threadIdx.x) * words + blockIdx.y] =
            win_or[w0] | win_or[w0 + 1] | win_or[w0 + 2] | win_or[w0 + 3];
    }
    for (int i = threadIdx.x; i < kRouteRows * kRouteCols; i += kRouteThreads) {
        const int row = i / kRouteCols, col = i % kRouteCols;
        if (row < M && c0 + col < NG)
            sorted_mask[static_cast<int64_t>(row) * NG + c0 + col] = row < col_cnt[col] ? 1 : 0;
    }
    const unsigned lt = (1u << lane) - 1u;
    for (int col = warp; col < kRouteCols; col += kRouteThreads / 32) {
        const int c = c0 + col;
        if (c >= NG) break;
        int act_base = 0, ina_base = col_cnt[col];
        for (int chunk = 0; chunk < kRouteRows / 32; ++chunk) {
            const int r = chunk * 32 + lane;
            const bool valid = r < M;
            const bool on = tile[r][col] != 0;
            const unsigned bal = __ballot_sync(0xffffffffu, on);
            const unsigned off = __ballot_sync(0xffffffffu, valid) & ~bal;
            if (valid) {
                const int pos = on ? act_base + __popc(bal & lt) : ina_base + __popc(off & lt);
                sorted_indices[static_cast<int64_t>(pos) * NG + c] = r;
            }
            act_base += __popc(bal);
            ina_base += __popc(off);
        }
    }
}

// counts of a caller-supplied sorted_mask.  The layout puts every active row of a column
// before every inactive one (the invariant the reference's kernels rely on as well,
// include/gemm_mn/v1/sm12x.cuh:272-311), so the count is the position of the first zero:
// one thread per column, a binary search of log2(M) loads.
__global__ void __launch_bounds__(128)
route_counts_kernel(const uint8_t* __restrict__ sorted_mask, int64_t M, int NG,
                    int32_t* __restrict__ counts)
{
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= NG) return;
    sorted_mask += static_cast<int64_t>(b) * M * NG;
    int64_t lo = 0, hi = M;              // invariant: rows < lo are active, rows >= hi are not
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (sorted_mask[mid * NG + c] != 0) lo = mid + 1; else hi = mid;
    }
    counts[static_cast<int64_t>(b) * NG + c] = static_cast<int32_t>(lo);
}

// packed bits: one CTA per 128-row window
__global__ void __launch_bounds__(128)
mask_pack_kernel(const uint8_t* __restrict__ mask, int64_t M, int NG, int words,
                 uint32_t* __restrict__ row_bits, uint32_t* __restrict__ win_bits)
{
    extern __shared__ uint32_t s_or[];   // [4][words]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * 128;
    for (int w = 0; w < words; ++w) {
        int g = w * 32 + lane;
        uint32_t acc = 0;
        for (int i = warp; i < 128; i += 4) {
            int64_t r = r0 + i;
            bool on = (r < M && g < NG) ? (mask[r * NG + g] != 0) : false;
            uint32_t bits = __ballot_sync(0xffffffffu, on);
            if (lane == 0 && r < M) row_bits[r * words + w] = bits;
            acc |= bits;
        }
        if (lane == 0) s_or[warp * words + w] = acc;
    }
    __syncthreads();
    for (int w = threadIdx.x; w < words; w += 128)
        win_bits[static_cast<int64_t>(blockIdx.x) * words + w] =
            s_or[w] | s_or[words + w] | s_or[2 * words + w] | s_or[3 * words + w];
}

// top-k mask: one warp per token row.  The k-th largest logit is found by a bitwise binary
// search over order-preserving integer keys (32 steps of count-and-compare), then
// everything above it is kept and ties with it are kept in index order, so that ties go to
// the lower group index.
__device__ __forceinline__ uint32_t topk_key(float f)
{
    // monotone map float -> uint32 (larger float = larger key); -0 and +0 coincide
    uint32_t u = __float_as_uint(f + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kTopkPerLane = 8;    // covers NG <= 256 in registers

__global__ void __launch_bounds__(128)
topk_mask_kernel(const float* __restrict__ logits, int64_t M, int NG, int keep,
                 uint8_t* __restrict__ mask)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * 4 + warp;
    if (r >= M) return;
    uint32_t key[kTopkPerLane];
#pragma unroll
    for (int i = 0; i < kTopkPerLane; ++i) {
        const int g = i * 32 + lane;
        key[i] = g < NG ? topk_key(logits[r * NG + g]) : 0u;   // real keys are never 0
    }
    if (keep <= 0 || keep >= NG) {
#pragma unroll
        for (int i = 0; i < kTopkPerLane; ++i) {
            const int g = i * 32 + lane;
            if (g < NG) mask[r * NG + g] = keep > 0 ? 1 : 0;
        }
        return;
    }
    // largest T with count(key >= T) >= keep  ==  the keep-th largest key
    uint32_t thr = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const uint32_t cand = thr | (1u << bit);
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < kTopkPerLane; ++i) cnt += key[i] >= cand;
        cnt = __reduce_add_sync(0xffffffffu, cnt);
        if (cnt >= keep) thr = cand;
    }
    int above = 0;
#pragma unroll
    for (int i = 0; i < kTopkPerLane; ++i) above += key[i] > thr;
    above = __reduce_add_sync(0xffffffffu, above);
    int ties_left = keep - above;                     // ties to keep, lowest indices first
    const unsigned lt = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < kTopkPerLane; ++i) {
        const int g = i * 32 + lane;
        const bool tie = g < NG && key[i] == thr;
        const unsigned bal = __ballot_sync(0xffffffffu, tie);
        const bool on = g < NG && (key[i] > thr || (tie && __popc(bal & lt) < ties_left));
        if (g < NG) mask[r * NG + g] = on ? 1 : 0;
        ties_left -= __popc(bal);
    }
}

// same result for any NG (rank by counting through shared memory); used beyond 256 groups
__global__ void __launch_bounds__(128)
topk_mask_rank_kernel(const float* __restrict__ logits, int64_t M, int NG, int keep,
                      uint8_t* __restrict__ mask)
{
    extern __shared__ float s_l[];   // [4][NG]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * 4 + warp;
    if (r >= M) return;
    float* l = s_l + warp * NG;
    for (int g = lane; g < NG; g += 32) l[g] = logits[r * NG + g];
    __syncwarp();
    for (int g = lane; g < NG; g += 32) {
        float v = l[g];
        int rank = 0;
        for (int h = 0; h < NG; ++h) {
            float u = l[h];
            rank += (u > v) || (u == v && h < g);
        }
        mask[r * NG + g] = rank < keep ? 1 : 0;
    }
}

// ---- scratch for dpk_route_compact_static --------------------------------------------
// Fixed-size per-(row block, group) counters for callers that cannot hand in a workspace.
// The array is part of the library image: every GPU that loads the library keeps these
// 256 KiB until the process exits.
constexpr size_t kStaticRouteInts = 65536;
static __device__ __align__(256) int32_t g_route_static_scratch[kStaticRouteInts];

// Device address of the array above for the current device.  The array's name is only a
// host-side handle in host code, so the address is asked from the runtime once per
// device (with that device current) and remembered.
static int route_static_scratch_ptr(int32_t** out)
{
    constexpr int kMaxDev = 64;
    static int32_t* cached[kMaxDev] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return fail(DPK_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDev) return fail(DPK_ERR_UNSUPPORTED, "device index %d too large", dev);
    if (!cached[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_route_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(DPK_ERR_CUDA, "cudaGetSymbolAddress(route scratch) failed: %s",
                        cudaGetErrorString(e));
        cached[dev] = static_cast<int32_t*>(p);
    }
    *out = cached[dev];
    return DPK_OK;
}

}  // namespace dpk

using namespace dpk;

extern "C" {

int dpk_topk_mask(const float* logits, int64_t M, int NG, int keep, uint8_t* mask, void* stream)
{
    DPK_REQUIRE(logits && mask, "logits and mask must not be NULL");
    DPK_REQUIRE(M >= 0 && NG >= 1 && NG <= 4096, "bad shape M=%lld NG=%d", (long long)M, NG);
    DPK_REQUIRE(keep >= 0 && keep <= NG, "keep=%d outside [0,%d]", keep, NG);
    if (M == 0) return DPK_OK;
    unsigned blocks = static_cast<unsigned>((M + 3) / 4);
    if (NG <= 32 * kTopkPerLane)
        topk_mask_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, M, NG, keep,
                                                                               mask);
    else
        topk_mask_rank_kernel<<<blocks, 128, 4 * NG * sizeof(float),
                                static_cast<cudaStream_t>(stream)>>>(logits, M, NG, keep, mask);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

size_t dpk_route_workspace_bytes(int batches, int64_t M, int NG)
{
    if (batches < 1 || M < 0 || NG < 1) return 0;
    int64_t nrb = (M + kRouteRows - 1) / kRouteRows;
    if (nrb < 1) nrb = 1;
    return static_cast<size_t>(batches) * nrb * NG * sizeof(int32_t);
}

int dpk_route_compact(const uint8_t* mask, int batches, int64_t M, int NG, uint8_t* sorted_mask,
                      int64_t* sorted_indices, int32_t* counts, void* workspace,
                      size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(mask && sorted_mask && sorted_indices && counts, "NULL tensor");
    DPK_REQUIRE(batches >= 1 && batches <= 65535 && M >= 0 && NG >= 1,
                "bad shape batches=%d M=%lld NG=%d", batches, (long long)M, NG);
    DPK_REQUIRE(M < (1ll << 31), "M=%lld too large", (long long)M);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M == 0) {
        DPK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * batches * NG, s));
        return DPK_OK;
    }
    size_t need = dpk_route_workspace_bytes(batches, M, NG);
    DPK_REQUIRE(workspace && workspace_bytes >= need, "workspace of %zu bytes needed, %zu given",
                need, workspace_bytes);
    int nrb = static_cast<int>((M + kRouteRows - 1) / kRouteRows);
    int ncb = (NG + kRouteCols - 1) / kRouteCols;
    DPK_REQUIRE(ncb <= 65535, "NG=%d too large", NG);
    int32_t* block_cnt = static_cast<int32_t*>(workspace);
    dim3 grid(nrb, ncb, batches);
    if (nrb == 1) {
        route_one_block_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, counts, sorted_mask,
                                                               sorted_indices, nullptr, nullptr, 0);
        DPK_CUDA(cudaGetLastError());
        return DPK_OK;
    }
    route_count_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, nullptr, nullptr, 0);
    int total = batches * NG;
    route_scan_kernel<<<(total + 127) / 128, 128, 0, s>>>(block_cnt, nrb, NG, batches, counts);
    route_scatter_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, counts,
                                                         sorted_mask, sorted_indices);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

int dpk_route_counts(const uint8_t* sorted_mask, int batches, int64_t M, int NG, int32_t* counts,
                     void* stream)
{
    DPK_REQUIRE(sorted_mask && counts, "NULL tensor");
    DPK_REQUIRE(batches >= 1 && batches <= 65535 && M >= 0 && NG >= 1, "bad shape");
    dim3 grid((NG + 127) / 128, batches);
    route_counts_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(sorted_mask, M, NG,
                                                                              counts);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

int dpk_mask_pack(const uint8_t* mask, int64_t M, int NG, uint32_t* row_bits, uint32_t* win_bits,
                  void* stream)
{
    DPK_REQUIRE(mask && row_bits && win_bits, "NULL tensor");
    DPK_REQUIRE(M >= 0 && NG >= 1 && NG <= 8192, "bad shape M=%lld NG=%d", (long long)M, NG);
    if (M == 0) return DPK_OK;
    int words = (NG + 31) / 32;
    unsigned nwin = static_cast<unsigned>((M + 127) / 128);
    mask_pack_kernel<<<nwin, 128, 4 * words * sizeof(uint32_t), static_cast<cudaStream_t>(stream)>>>(
        mask, M, NG, words, row_bits, win_bits);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

int dpk_route_compact_static(const uint8_t* mask, int batches, int64_t M, int NG,
                             uint8_t* sorted_mask, int64_t* sorted_indices, int32_t* counts,
                             void* stream)
{
    DPK_REQUIRE(mask && sorted_mask && sorted_indices && counts, "NULL tensor");
    DPK_REQUIRE(batches >= 1 && batches <= 65535 && M >= 0 && NG >= 1,
                "bad shape batches=%d M=%lld NG=%d", batches, (long long)M, NG);
    DPK_REQUIRE(M < (1ll << 31), "M=%lld too large", (long long)M);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M == 0) {
        DPK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * batches * NG, s));
        return DPK_OK;
    }
    const size_t need = dpk_route_workspace_bytes(batches, M, NG);
    DPK_REQUIRE(need <= kStaticRouteInts * sizeof(int32_t),
                "routing problem needs %zu bytes of scratch but the built-in scratch holds %zu "
                "(batches * ceil(M/256) * NG must not exceed %zu); use dpk_route_compact with a "
                "caller workspace instead",
                need, kStaticRouteInts * sizeof(int32_t), kStaticRouteInts);
    int32_t* block_cnt = nullptr;
    int rc = route_static_scratch_ptr(&block_cnt);
    if (rc) return rc;
    int nrb = static_cast<int>((M + kRouteRows - 1) / kRouteRows);
    int ncb = (NG + kRouteCols - 1) / kRouteCols;
    DPK_REQUIRE(ncb <= 65535, "NG=%d too large", NG);
    dim3 grid(nrb, ncb, batches);
    // every counter this call reads is written by the first kernel, so nothing left by an
    // earlier call needs clearing
    route_count_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, nullptr, nullptr, 0);
    int total = batches * NG;
    route_scan_kernel<<<(total + 127) / 128, 128, 0, s>>>(block_cnt, nrb, NG, batches, counts);
    route_scatter_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, counts,
                                                         sorted_mask, sorted_indices);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

int dpk_route_plan(const uint8_t* mask, int64_t M, int NG, uint8_t* sorted_mask,
                   int64_t* sorted_indices, int32_t* counts, uint32_t* row_bits, uint32_t* win_bits,
                   void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(mask && sorted_mask && sorted_indices && counts && row_bits && win_bits, "NULL tensor");
    DPK_REQUIRE(M >= 0 && M < (1ll << 31) && NG >= 1 && NG <= 8192, "bad shape M=%lld NG=%d",
                (long long)M, NG);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M == 0) {
        DPK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * NG, s));
        return DPK_OK;
    }
    size_t need = dpk_route_workspace_bytes(1, M, NG);
    DPK_REQUIRE(workspace && workspace_bytes >= need, "workspace of %zu bytes needed, %zu given",
                need, workspace_bytes);
    int nrb = static_cast<int>((M + kRouteRows - 1) / kRouteRows);
    int ncb = (NG + kRouteCols - 1) / kRouteCols;     // == words of the packed bits
    int32_t* block_cnt = static_cast<int32_t*>(workspace);
    dim3 grid(nrb, ncb, 1);
    if (nrb == 1) {
        route_one_block_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, counts, sorted_mask,
                                                               sorted_indices, row_bits, win_bits, ncb);
        DPK_CUDA(cudaGetLastError());
        return DPK_OK;
    }
    route_count_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, row_bits, win_bits,
                                                       ncb);
    route_scan_kernel<<<(NG + 127) / 128, 128, 0, s>>>(block_cnt, nrb, NG, 1, counts);
    route_scatter_kernel<<<grid, kRouteThreads, 0, s>>>(mask, M, NG, nrb, block_cnt, counts,
                                                         sorted_mask, sorted_indices);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // extern "C"
