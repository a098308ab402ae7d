// Token router fused with the RMSNorm that reads the same hidden state (sm_100a).
//
// What it computes, per token row x[H] (reference: TokenRouter, WIDE/wrapper/base_layer.py:
// 89-114, the same arithmetic as BottleneckRouter, PruningInferSim/ops/router.py:85-126; the
// evaluation-time decision of base_layer.py:204-207; call sites attn_group_ffn_block.py:
// 170-176 and 195-200, where the router reads the un-normalised state and the norm output
// feeds the projections):
//
//     c      = x . w_down^T + b_down                     [R]      (R <= 16)
//     logits = c . w_route^T + b_route                   [NG, 2]
//     execute[g] = logits[g,0] >= logits[g,1]                     (argmax; ties execute)
//     xn     = weight * dtype(x * rsqrt(mean(x^2) + eps))         (optional)
//
// The hidden state is read from HBM exactly once: a CTA brings 8 rows into shared memory with
// bulk copies (one per row, one mbarrier), and every element is then loaded from shared memory
// by exactly one thread, which uses it twice -- as an operand of the [8 x H] x [H x 16]
// contraction (mma.sync m16n8k16, rows 8-15 of the tile are zero; the contraction is 0.3 % of
// the time, the kernel is HBM-bound) and for the row's sum of squares.  The k index of the MMA
// is permuted so that a thread's 16 contiguous bytes of x and of w_down are its fragments of
// two consecutive k-steps; the same permutation on both operands leaves the dot products
// unchanged.  The eight warps split H; partial sums meet in shared memory.  The normalised
// rows are written from shared memory with 16-byte stores.
#define DPK_KERNEL_ID 9   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kRnRows = 8;
constexpr int kRnThreads = 512;      // at most; narrow rows run two CTAs of 256 threads per SM
constexpr int kRnWarps = kRnThreads / 32;
constexpr int kRnRank = 16;          // padded router rank
constexpr int kRnBatch = 4;         // k-blocks whose loads a warp issues together
constexpr int kRnSkew = 64;          // bytes between rows beyond H*2: spreads the rows over the banks

struct RouterNormParams {
    const uint8_t* x;        // [M, ldx] halves
    const uint8_t* gamma;    // [H] halves or NULL
    const uint8_t* w_down;   // [R, H] halves
    const uint8_t* b_down;   // [R] halves or NULL
    const uint8_t* w_route;  // [2*NG, R] halves
    const uint8_t* b_route;  // [2*NG] halves or NULL
    uint8_t* xn;             // [M, ldxn] halves or NULL
    uint8_t* execute;        // [M, NG] bytes
    float* logits;           // [M, NG, 2] or NULL
    int64_t ldx, ldxn, M;
    int H, R, NG;
    int round_like_module;
    float eps;
    int* status;
};

template <bool kBf16>
__device__ __forceinline__ float half_at(const uint8_t* p, int64_t i)
{
    if constexpr (kBf16)
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    else
        return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

template <bool kBf16>
__device__ __forceinline__ float round_half(float v)
{
    if constexpr (kBf16)
        return __bfloat162float(__float2bfloat16_rn(v));
    else
        return __half2float(__float2half_rn(v));
}

// packed product of two half pairs, rounded to the same dtype
template <bool kBf16>
__device__ __forceinline__ uint32_t mul_half2(uint32_t a, uint32_t b)
{
    if constexpr (kBf16) {
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                         *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    } else {
        const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a),
                                  *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
}

template <bool kBf16>
__device__ __forceinline__ void rn_mma(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1)
{
    // rows 8-15 of the A tile (a1, a3) are zero
    if constexpr (kBf16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ void bulk_load_row(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

template <bool kBf16>
__global__ void __launch_bounds__(kRnThreads, 1) router_norm_kernel(const RouterNormParams p)
{
    extern __shared__ __align__(128) uint8_t rn_smem[];
    const int pitch = p.H * 2 + kRnSkew;
    uint8_t* rows = rn_smem;
    float* cpart = reinterpret_cast<float*>(rn_smem + size_t(kRnRows) * pitch);   // [warps][rows][16]
    float* sspart = cpart + kRnWarps * kRnRows * kRnRank;                         // [warps][rows]
    float* cfin = sspart + kRnWarps * kRnRows;                                    // [rows][16]
    float* rs = cfin + kRnRows * kRnRank;                                         // [rows]
    uint64_t* bar = reinterpret_cast<uint64_t*>(rs + kRnRows);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int frow = lane >> 2;           // fragment row (A) / column (B), 0..7
    const int fk = (lane & 3) * 8;        // this thread's 8 consecutive k inside a 32-wide block
    if (tid == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // second-stage weights of this thread's first group stay in registers for all tiles
    float wa0[kRnRank], wb0[kRnRank], ba0 = 0.f, bb0 = 0.f;
#pragma unroll
    for (int j = 0; j < kRnRank; ++j) {
        const bool in = tid < p.NG && j < p.R;
        wa0[j] = in ? half_at<kBf16>(p.w_route, int64_t(2 * tid) * p.R + j) : 0.f;
        wb0[j] = in ? half_at<kBf16>(p.w_route, int64_t(2 * tid + 1) * p.R + j) : 0.f;
    }
    if (tid < p.NG && p.b_route) {
        ba0 = half_at<kBf16>(p.b_route, 2 * tid);
        bb0 = half_at<kBf16>(p.b_route, 2 * tid + 1);
    }

    const int64_t ntiles = (p.M + kRnRows - 1) / kRnRows;
    const int kblocks = p.H / 32;
    uint32_t phase = 0;
    auto rows_of = [&](int64_t t) -> int {
        const int64_t left = p.M - t * kRnRows;
        return left < kRnRows ? static_cast<int>(left) : kRnRows;
    };
    if (tid == 0 && blockIdx.x < ntiles) {          // first tile: all rows at once
        const int n = rows_of(blockIdx.x);
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(n) * p.H * 2);
        for (int r = 0; r < n; ++r)
            bulk_load_row(rows + size_t(r) * pitch, p.x + (int64_t(blockIdx.x) * kRnRows + r) * p.ldx * 2,
                          p.H * 2, bar);
    }
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t row0 = tile * kRnRows;
        const int nrows = rows_of(tile);
        const bool landed = mbar_wait(bar, phase, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL);
        phase ^= 1;
        if (!__syncthreads_and(landed)) break;

        // ---- contraction with w_down and the sum of squares: the warps split H ----------
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
        float ss = 0.f;
        const bool row_ok = frow < nrows;
        const uint8_t* xrow = rows + size_t(frow) * pitch;
        const uint8_t* w0 = p.w_down + size_t(frow) * p.H * 2;
        const uint8_t* w1 = p.w_down + size_t(frow + 8) * p.H * 2;
        const bool w0_ok = frow < p.R, w1_ok = frow + 8 < p.R;
        // kRnBatch k-blocks per step: all loads (the weights come from L2) are issued before
        // the first use, so that a warp keeps 12 16-byte requests in flight
        for (int kb0 = warp; kb0 < kblocks; kb0 += nwarps * kRnBatch) {
            uint4 xa[kRnBatch], b0[kRnBatch], b1[kRnBatch];
#pragma unroll
            for (int u = 0; u < kRnBatch; ++u) {
                const int kb = kb0 + u * nwarps;
                const int k = kb * 32 + fk;
                const bool in = kb < kblocks;
                xa[u] = b0[u] = b1[u] = make_uint4(0, 0, 0, 0);
                if (in && row_ok) xa[u] = *reinterpret_cast<const uint4*>(xrow + k * 2);
                if (in && w0_ok) b0[u] = __ldg(reinterpret_cast<const uint4*>(w0 + k * 2));
                if (in && w1_ok) b1[u] = __ldg(reinterpret_cast<const uint4*>(w1 + k * 2));
            }
#pragma unroll
            for (int u = 0; u < kRnBatch; ++u) {
                const uint32_t xv[4] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo, hi;
                    unpack_half2<kBf16>(xv[j], lo, hi);
                    ss = fmaf(lo, lo, ss);
                    ss = fmaf(hi, hi, ss);
                }
                rn_mma<kBf16>(acc0, xa[u].x, xa[u].y, b0[u].x, b0[u].y);
                rn_mma<kBf16>(acc0, xa[u].z, xa[u].w, b0[u].z, b0[u].w);
                rn_mma<kBf16>(acc1, xa[u].x, xa[u].y, b1[u].x, b1[u].y);
                rn_mma<kBf16>(acc1, xa[u].z, xa[u].w, b1[u].z, b1[u].w);
            }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        {
            float* cp = cpart + (warp * kRnRows + frow) * kRnRank + (lane & 3) * 2;
            cp[0] = acc0[0];
            cp[1] = acc0[1];
            cp[8] = acc1[0];
            cp[9] = acc1[1];
            if ((lane & 3) == 0) sspart[warp * kRnRows + frow] = ss;
        }
        __syncthreads();
        if (tid < kRnRows * kRnRank) {
            const int r = tid / kRnRank, j = tid % kRnRank;
            float c = 0.f;
            for (int w = 0; w < nwarps; ++w) c += cpart[(w * kRnRows + r) * kRnRank + j];
            if (j < p.R && p.b_down) c += half_at<kBf16>(p.b_down, j);
            if (p.round_like_module) c = round_half<kBf16>(c);
            cfin[r * kRnRank + j] = j < p.R ? c : 0.f;
        } else if (tid < kRnRows * kRnRank + kRnRows) {
            const int r = tid - kRnRows * kRnRank;
            float s = 0.f;
            for (int w = 0; w < nwarps; ++w) s += sspart[w * kRnRows + r];
            rs[r] = rsqrtf(s / static_cast<float>(p.H) + p.eps);
        }
        __syncthreads();

        // ---- second stage and the decision: one thread per group, all rows ----------------
        for (int g = tid; g < p.NG; g += nthreads) {
            float wa[kRnRank], wb[kRnRank], ba = ba0, bb = bb0;
#pragma unroll
            for (int j = 0; j < kRnRank; ++j) {
                wa[j] = wa0[j];
                wb[j] = wb0[j];
            }
            if (g != tid) {          // more groups than threads: reload
#pragma unroll
                for (int j = 0; j < kRnRank; ++j) {
                    wa[j] = j < p.R ? half_at<kBf16>(p.w_route, int64_t(2 * g) * p.R + j) : 0.f;
                    wb[j] = j < p.R ? half_at<kBf16>(p.w_route, int64_t(2 * g + 1) * p.R + j) : 0.f;
                }
                ba = p.b_route ? half_at<kBf16>(p.b_route, 2 * g) : 0.f;
                bb = p.b_route ? half_at<kBf16>(p.b_route, 2 * g + 1) : 0.f;
            }
            for (int r = 0; r < nrows; ++r) {
                float la = 0.f, lb = 0.f;
#pragma unroll
                for (int j = 0; j < kRnRank; ++j) {
                    const float c = cfin[r * kRnRank + j];
                    la = fmaf(c, wa[j], la);
                    lb = fmaf(c, wb[j], lb);
                }
                la += ba;
                lb += bb;
                if (p.round_like_module) {
                    la = round_half<kBf16>(la);
                    lb = round_half<kBf16>(lb);
                }
                p.execute[(row0 + r) * p.NG + g] = la >= lb ? 1 : 0;
                if (p.logits) {
                    float2* out = reinterpret_cast<float2*>(p.logits + ((row0 + r) * p.NG + g) * 2);
                    *out = make_float2(la, lb);
                }
            }
        }

        // ---- normalised rows ----------------------------------------------------------------
        // ---- normalised rows, written row by row; a row that has been written is refilled
        //      with the same row of this CTA's next tile, so the load runs under the stores ----
        const int64_t next = tile + gridDim.x;
        const int next_rows = next < ntiles ? rows_of(next) : 0;
        if (tid == 0 && next_rows > 0)
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(next_rows) * p.H * 2);
        const int chunks = p.H / 8;
        for (int r = 0; r < kRnRows; ++r) {
            if (p.xn && r < nrows) {
                // the product dtype(x * scale) * weight is a packed multiply in the tensor dtype,
                // which rounds exactly as the module's elementwise multiply does
                const float scale = rs[r];
                const uint8_t* src = rows + size_t(r) * pitch;
                uint8_t* dst = p.xn + (row0 + r) * p.ldxn * 2;
                for (int c = tid; c < chunks; c += nthreads) {
                    const uint4 xa = *reinterpret_cast<const uint4*>(src + c * 16);
                    const uint4 ga = __ldg(reinterpret_cast<const uint4*>(p.gamma + c * 16));
                    const uint32_t xv[4] = {xa.x, xa.y, xa.z, xa.w}, gv[4] = {ga.x, ga.y, ga.z, ga.w};
                    uint32_t ov[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float lo, hi;
                        unpack_half2<kBf16>(xv[j], lo, hi);
                        ov[j] = mul_half2<kBf16>(pack_half2<kBf16>(lo * scale, hi * scale), gv[j]);
                    }
                    *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
                }
            }
            __syncthreads();      // row r has been read by everyone
            if (tid == 0 && r < next_rows)
                bulk_load_row(rows + size_t(r) * pitch, p.x + (next * kRnRows + r) * p.ldx * 2, p.H * 2, bar);
        }
    }
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_router_norm(const void* x, int64_t ldx, const void* gamma, float eps,
                               const void* w_down, const void* b_down, const void* w_route,
                               const void* b_route, void* xn, int64_t ldxn, uint8_t* execute,
                               float* logits, int64_t M, int H, int R, int NG, int dtype,
                               int round_like_module, void* stream)
{
    DPK_REQUIRE(x && w_down && w_route && execute, "NULL tensor");
    DPK_REQUIRE((gamma == nullptr) == (xn == nullptr), "gamma and xn go together");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(M >= 0 && H > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(R >= 1 && R <= kRnRank, "router rank R=%d must be 1..%d", R, kRnRank);
    DPK_REQUIRE(H % 32 == 0, "H=%d must be a multiple of 32", H);
    DPK_REQUIRE(ldx >= H && ldx % 8 == 0 && (!xn || (ldxn >= H && ldxn % 8 == 0)),
                "row strides must be multiples of 8 and at least H");
    DPK_REQUIRE(aligned16(x) && aligned16(w_down) && aligned16(gamma) && aligned16(xn),
                "tensors must be 16-byte aligned");
    DPK_REQUIRE(!logits || (reinterpret_cast<uintptr_t>(logits) & 7u) == 0, "logits must be 8-byte aligned");
    if (M == 0) return DPK_OK;
    const size_t smem = size_t(kRnRows) * (size_t(H) * 2 + kRnSkew) +
                        sizeof(float) * (kRnWarps * kRnRows * kRnRank + kRnWarps * kRnRows +
                                         kRnRows * kRnRank + kRnRows) + 32;
    DPK_REQUIRE(smem <= 227 * 1024, "H=%d is too wide for the %d-row tile in shared memory", H, kRnRows);

    RouterNormParams p;
    p.x = static_cast<const uint8_t*>(x);
    p.gamma = static_cast<const uint8_t*>(gamma);
    p.w_down = static_cast<const uint8_t*>(w_down);
    p.b_down = static_cast<const uint8_t*>(b_down);
    p.w_route = static_cast<const uint8_t*>(w_route);
    p.b_route = static_cast<const uint8_t*>(b_route);
    p.xn = static_cast<uint8_t*>(xn);
    p.execute = execute;
    p.logits = logits;
    p.ldx = ldx;
    p.ldxn = ldxn;
    p.M = M;
    p.H = H;
    p.R = R;
    p.NG = NG;
    p.round_like_module = round_like_module;
    p.eps = eps;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");

    const int64_t ntiles = (M + kRnRows - 1) / kRnRows;
    // rows up to ~6000 wide: two CTAs of 256 threads share an SM and overlap each other's
    // phases; wider rows leave room for one CTA, which then runs 512 threads
    const int per_sm = 2 * smem <= 227 * 1024 ? 2 : 1;
    const int threads = per_sm == 2 ? 256 : kRnThreads;
    int64_t grid = int64_t(sm_count()) * per_sm;
    if (grid > ntiles) grid = ntiles;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(router_norm_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        router_norm_kernel<true><<<static_cast<unsigned>(grid), threads, smem, s>>>(p);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(router_norm_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        router_norm_kernel<false><<<static_cast<unsigned>(grid), threads, smem, s>>>(p);
    }
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
