// Tensor-parallel plumbing that lives next to the kernels: buffers another process of the
// node can map (CUDA IPC), and the second half of the fused row-parallel sum.
//
// The first half is the epilogue of the reduction-width projection (dpk_gemm_k_scatter):
// every rank stores its partial sums of a token window straight into the staging buffer
// of the rank that owns the window.  After all ranks have finished that kernel (the
// caller's barrier), dpk_reduce_gather on owner o adds the `world` slabs of its rows in
// fp32, optionally adds a residual, rounds once and stores the rows into every rank's
// output -- again plain stores into peer memory, 16 bytes per thread and 512 contiguous
// bytes per warp.  No kernel here waits for another GPU.
#define DPK_KERNEL_ID 8   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kMaxPeersRG = 8;

struct ReduceGatherParams {
    const uint8_t* stage;            // [world, rows_per_owner, ld] halves (this rank's staging)
    const uint8_t* residual;         // [M, ld] halves or NULL (local)
    uint8_t* out[kMaxPeersRG];       // every rank's [M, ld] output, starting with rank + 1
    int world, rank;
    int64_t rows_per_owner, rows;    // rows = owned rows inside the token range
    int64_t ld;
    int N;
};

template <bool kBf16>
__device__ __forceinline__ void accumulate8(float (&acc)[8], const uint4& v)
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo, hi;
        unpack_half2<kBf16>(w[j], lo, hi);
        acc[2 * j] += lo;
        acc[2 * j + 1] += hi;
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) reduce_gather_kernel(const ReduceGatherParams p)
{
    const int64_t chunks_per_row = p.N / 8;
    const int64_t total = p.rows * chunks_per_row;
    const int64_t slab = p.rows_per_owner * p.ld * 2;                 // bytes
    const int64_t first_row = int64_t(p.rank) * p.rows_per_owner;     // in the full matrix
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / chunks_per_row;
        const int64_t c = i - r * chunks_per_row;
        const int64_t off = (r * p.ld + c * 8) * 2;
        // all slabs are requested before the first is used
        uint4 v[kMaxPeersRG];
#pragma unroll
        for (int j = 0; j < kMaxPeersRG; ++j)
            if (j < p.world) v[j] = *reinterpret_cast<const uint4*>(p.stage + j * slab + off);
        const int64_t goff = ((first_row + r) * p.ld + c * 8) * 2;
        uint4 res = make_uint4(0, 0, 0, 0);
        if (p.residual) res = *reinterpret_cast<const uint4*>(p.residual + goff);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // the slabs are summed in rank order on every owner: the result does not depend on
        // which rank computes it
#pragma unroll
        for (int j = 0; j < kMaxPeersRG; ++j)
            if (j < p.world) accumulate8<kBf16>(acc, v[j]);
        if (p.residual) accumulate8<kBf16>(acc, res);
        uint4 o;
        o.x = pack_half2<kBf16>(acc[0], acc[1]);
        o.y = pack_half2<kBf16>(acc[2], acc[3]);
        o.z = pack_half2<kBf16>(acc[4], acc[5]);
        o.w = pack_half2<kBf16>(acc[6], acc[7]);
        // out[] starts with the next rank (rotated on the host), so that the ranks do not all
        // store to the same peer at once
#pragma unroll
        for (int j = 0; j < kMaxPeersRG; ++j)
            if (j < p.world) *reinterpret_cast<uint4*>(p.out[j] + goff) = o;
    }
}

// Barrier between the ranks of one node through flags in peer-mapped memory.  Every rank owns
// an array of `world` 32-bit slots; slot s of rank o's array is written only by rank s.  Thread j
// of the single block publishes this rank's arrival to rank j (a system-scope release store of
// the epoch number into slot `rank` of j's array, after the peer stores of the kernels before
// this one in the stream) and then waits until slot j of its OWN array has reached the epoch.  The
// wait is bounded: after `limit_cycles` it records a status code and the kernel returns, so the
// context stays usable; the caller must treat the step's result as invalid then.  Epochs only
// grow, so a rank that is one barrier ahead cannot be mistaken for one that has arrived at this
// one, and no slot is ever reset.  Every rank runs this kernel on its own GPU.
struct PeerFlagTable {
    uint32_t* p[kMaxPeersRG];
};

__global__ void __launch_bounds__(32) peer_barrier_table_kernel(const PeerFlagTable peer_flags,
                                                                uint32_t* my_flags, int world, int rank,
                                                                uint32_t epoch, long long limit_cycles,
                                                                int* status)
{
    const int j = threadIdx.x;
    if (j >= world) return;
    __threadfence_system();
    uint32_t* remote = peer_flags.p[j] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    // poll with plain (relaxed, uncached) loads and fence once at the end
    const volatile uint32_t* mine = my_flags + j;
    const long long t0 = clock64();
    while (true) {
        const uint32_t seen = *mine;
        if (static_cast<int32_t>(seen - epoch) >= 0) break;
        if (clock64() - t0 > limit_cycles) {
            atomicCAS(status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_TIMEOUT_PEER);
            break;
        }
        __nanosleep(1000);
    }
    __threadfence_system();       // what the peers wrote before their arrival is visible after this
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_peer_barrier(void* const* peer_flags, void* my_flags, int world, int rank,
                                uint32_t epoch, int timeout_ms, void* stream)
{
    DPK_REQUIRE(peer_flags && my_flags, "NULL flags");
    DPK_REQUIRE(world >= 1 && world <= kMaxPeersRG && rank >= 0 && rank < world, "bad world / rank");
    DPK_REQUIRE(timeout_ms > 0 && timeout_ms <= 10000, "timeout_ms must be 1..10000");
    DPK_REQUIRE((reinterpret_cast<uintptr_t>(my_flags) & 3u) == 0, "flags must be 4-byte aligned");
    int* status = device_status_ptr();
    if (!status) return fail(DPK_ERR_CUDA, "no status word on this device");
    // the table of peer pointers travels as a kernel argument: no device allocation
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PeerFlagTable t;
    for (int i = 0; i < kMaxPeersRG; ++i) t.p[i] = nullptr;
    for (int i = 0; i < world; ++i) {
        DPK_REQUIRE(peer_flags[i] && (reinterpret_cast<uintptr_t>(peer_flags[i]) & 3u) == 0, "flag array %d", i);
        t.p[i] = static_cast<uint32_t*>(peer_flags[i]);
    }
    int dev = 0, khz = 0;
    DPK_CUDA(cudaGetDevice(&dev));
    DPK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    const long long limit = static_cast<long long>(khz > 0 ? khz : 2000000) * timeout_ms;
    peer_barrier_table_kernel<<<1, 32, 0, s>>>(t, static_cast<uint32_t*>(my_flags), world, rank, epoch,
                                              limit, status);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

extern "C" int dpk_peer_alloc(size_t bytes, void** ptr, void* handle)
{
    DPK_REQUIRE(ptr && handle && bytes > 0, "bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void* p = nullptr;
    DPK_CUDA(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(DPK_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return DPK_OK;
}

extern "C" int dpk_peer_open(const void* handle, void** ptr)
{
    DPK_REQUIRE(ptr && handle, "bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    DPK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return DPK_OK;
}

extern "C" int dpk_peer_close(void* ptr)
{
    DPK_REQUIRE(ptr, "NULL pointer");
    DPK_CUDA(cudaIpcCloseMemHandle(ptr));
    return DPK_OK;
}

extern "C" int dpk_peer_free(void* ptr)
{
    DPK_REQUIRE(ptr, "NULL pointer");
    DPK_CUDA(cudaFree(ptr));
    return DPK_OK;
}

extern "C" int dpk_reduce_gather(const void* stage, void* const* out, const void* residual, int world,
                                 int rank, int64_t rows_per_owner, int64_t M, int N, int64_t ld,
                                 int dtype, int max_blocks, void* stream)
{
    DPK_REQUIRE(stage && out, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(world >= 1 && world <= kMaxPeersRG, "world must be 1..%d", kMaxPeersRG);
    DPK_REQUIRE(rank >= 0 && rank < world, "rank outside the world");
    DPK_REQUIRE(rows_per_owner > 0 && M >= 0 && M <= rows_per_owner * world, "bad row split");
    DPK_REQUIRE(N > 0 && N % 8 == 0 && ld >= N && ld % 8 == 0, "N and ld must be multiples of 8");
    DPK_REQUIRE(aligned16(stage) && aligned16(residual), "tensors must be 16-byte aligned");
    ReduceGatherParams p;
    p.stage = static_cast<const uint8_t*>(stage);
    p.residual = static_cast<const uint8_t*>(residual);
    for (int i = 0; i < kMaxPeersRG; ++i) p.out[i] = nullptr;
    for (int i = 0; i < world; ++i) {
        DPK_REQUIRE(out[i] && aligned16(out[i]), "output %d", i);
        p.out[(i - rank - 1 + 2 * world) % world] = static_cast<uint8_t*>(out[i]);
    }
    p.world = world;
    p.rank = rank;
    p.rows_per_owner = rows_per_owner;
    const int64_t first = int64_t(rank) * rows_per_owner;
    p.rows = M - first < 0 ? 0 : (M - first > rows_per_owner ? rows_per_owner : M - first);
    p.ld = ld;
    p.N = N;
    if (p.rows == 0) return DPK_OK;
    const int64_t total = p.rows * (N / 8);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = max_blocks > 0 ? max_blocks : int64_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // capped grid: small blocks, so that one of them fits on an SM beside a projection CTA
    const int threads = max_blocks > 0 ? 128 : 256;
    if (dtype == DPK_BF16)
        reduce_gather_kernel<true><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
    else
        reduce_gather_kernel<false><<<static_cast<unsigned>(blocks), threads, 0, s>>>(p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
