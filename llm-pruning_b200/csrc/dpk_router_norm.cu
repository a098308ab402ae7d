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
#include <map>
#include <mutex>
#include <tuple>

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


// ---------------------------------------------------------------------------------------------
// Column-split variant: a cluster of C CTAs shares a 16-row tile, each CTA owning H / C columns.
//
// What bounds the kernel above is not memory.  One CTA per SM at H = 8192, every phase behind a
// CTA-wide barrier, the first-stage weights (16 x H halves) streamed from L2 again for every
// 8 rows, and a second stage whose scalar arithmetic sits on a few warps: the loads run out
// while the arithmetic runs, and the other way round.  Here
//   * the CTA is split into two groups of eight warps that work on different tiles at the same
//     time: the CONTRACTING warps (first stage, exchange, second stage, decisions) and the
//     NORMALISING warps (scaling in place in shared memory; their first warp also issues all
//     bulk copies).  Row slices go through a ring of 3-4 stages: one being normalised and
//     drained, one being contracted, the rest in flight;
//   * the normalised rows leave through bulk stores from shared memory;
//   * a contracting thread keeps its fragments of the [16 x H/C] weight slice in registers for
//     the whole launch (64 registers), so the slice occupies no shared memory or bandwidth;
//   * both row halves of the m16n8k16 tile carry tokens;
//   * the C partial contractions and sums of squares of a tile meet through distributed shared
//     memory without a cluster barrier: every CTA pushes its 16 x 17 partials into every rank's
//     receive slot with st.async, which counts the bytes on an mbarrier of the receiver; the
//     slots are summed in rank order, so all ranks hold the same contraction and normalise with
//     the same scales;
//   * the second stage [16 x 16] x [16 x 2*NG] is split by groups: rank q computes the logits
//     and decisions of groups q*NG/C ... for all 16 rows, a few full MMAs per warp (when the
//     contraction is rounded to the tensor dtype, as a module in that dtype does; the fp32
//     variant keeps scalar arithmetic), with its share of the second-stage weights staged in
//     shared memory; the decisions are collected there too and leave as 4-byte stores.
// Measured on the 70B-shaped layer's router (M = 16384, H = 8192, 224 groups): every variant that
// kept one CTA-wide sequence of phases took 0.16-0.20 ms whatever the data path; with the
// second stage split by rows instead of groups (a quarter-filled MMA tile per rank, four times
// the MMAs and their epilogues) 0.158 ms; this layout 0.127 ms.  The same loads, barriers and
// stores without any arithmetic take 0.099 ms.
// Two receive slots alternate.  A CTA can only push for tile i+2 after it has seen every peer's
// push for tile i+1, which a peer issues after reading its slot of tile i, so a slot is never
// overwritten before it has been read.  Every wait is bounded; a group that gives up raises the
// CTA's abort flag, which ends the other group's waits, and all CTAs meet at the final cluster
// barrier.
constexpr int kRcRows = 16;
constexpr int kRcGroup = 256;                         // threads of one warp group
constexpr int kRcThreads = 2 * kRcGroup;
constexpr int kRcGWarps = kRcGroup / 32;
constexpr int kRcMaxStages = 4;
constexpr int kRcMaxSlice = 2048;                     // columns per CTA
constexpr int kRcKPerWarp = kRcMaxSlice / 32 / kRcGWarps;   // 32-wide k-blocks of a contracting warp: 8
constexpr int kRcMaxCluster = 8;
constexpr int kRcPart = kRcRows * (kRnRank + 1);      // partials of one tile: 16 x 16 contraction + 16 sums of squares
constexpr int kRcExBytes = 2048;                      // decisions of one tile collected in shared memory, at most

__device__ __forceinline__ uint32_t cluster_nctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_count_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_addr(const void* own, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(own)), "r"(rank));
    return remote;
}
// one float into a peer's shared memory; the peer's mbarrier counts its four bytes
__device__ __forceinline__ void st_async_f32(uint32_t remote_dst, float v, uint32_t remote_bar)
{
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_dst), "r"(__float_as_uint(v)), "r"(remote_bar)
                 : "memory");
}
// barrier of one warp group (id 1 or 2, kRcGroup threads)
__device__ __forceinline__ void group_sync(int id)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(kRcGroup) : "memory");
}
// the same barrier, returning whether `ok` held for every thread of the group
__device__ __forceinline__ bool group_all(int id, bool ok)
{
    uint32_t r;
    asm volatile("{\n"
                 ".reg .pred p, q;\n"
                 "setp.ne.u32 q, %1, 0;\n"
                 "bar.red.and.pred p, %2, %3, q;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(r)
                 : "r"(static_cast<uint32_t>(ok)), "r"(id), "r"(kRcGroup)
                 : "memory");
    return r != 0;
}
// acc += {lo*lo, hi*hi} as one packed fp32 instruction (each lane rounds like a scalar fma)
__device__ __forceinline__ void fma_sq2(float2& acc, float lo, float hi)
{
    asm("{\n"
        ".reg .b64 v, a;\n"
        "mov.b64 v, {%2, %3};\n"
        "mov.b64 a, {%0, %1};\n"
        "fma.rn.f32x2 a, v, v, a;\n"
        "mov.b64 {%0, %1}, a;\n"
        "}\n"
        : "+f"(acc.x), "+f"(acc.y)
        : "f"(lo), "f"(hi));
}
// {lo, hi} * s as one packed fp32 instruction
__device__ __forceinline__ void mul_s2(float& lo, float& hi, float s)
{
    asm("{\n"
        ".reg .b64 v, w;\n"
        "mov.b64 v, {%0, %1};\n"
        "mov.b64 w, {%2, %2};\n"
        "mul.rn.f32x2 v, v, w;\n"
        "mov.b64 {%0, %1}, v;\n"
        "}\n"
        : "+f"(lo), "+f"(hi)
        : "f"(s));
}
// shared memory -> global bulk copy, tracked by the issuing thread's bulk group
__device__ __forceinline__ void bulk_store_row(void* gdst, const void* ssrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but this thread's newest bulk store have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// this thread's bulk stores are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <bool kBf16>
__device__ __forceinline__ void rc_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1)
{
    if constexpr (kBf16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// two consecutive halves of row n of w_route as one 32-bit MMA operand; zero beyond the rank
template <bool kBf16>
__device__ __forceinline__ uint32_t route_pair(const RouterNormParams& p, int n, int k, bool n_ok)
{
    if (!n_ok) return 0u;
    if (p.R == kRnRank) return __ldg(reinterpret_cast<const uint32_t*>(p.w_route + (int64_t(n) * kRnRank + k) * 2));
    const uint16_t* w = reinterpret_cast<const uint16_t*>(p.w_route) + int64_t(n) * p.R;
    const uint32_t lo = k < p.R ? w[k] : 0u, hi = k + 1 < p.R ? w[k + 1] : 0u;
    return lo | (hi << 16);
}

template <bool kBf16>
__global__ void __launch_bounds__(kRcThreads, 1)
router_norm_cluster_kernel(const RouterNormParams p, const int hc, const int stages, const int wr_staged)
{
    extern __shared__ __align__(128) uint8_t rn_smem[];
    const int pitch = hc * 2 + kRnSkew;
    uint8_t* ring = rn_smem;                                            // [stages][16][pitch]
    float* cpart = reinterpret_cast<float*>(ring + size_t(stages) * kRcRows * pitch);   // [warps][rows][16]
    float* sspart = cpart + kRcGWarps * kRcRows * kRnRank;              // [warps][rows]
    float* slot = sspart + kRcGWarps * kRcRows;                         // [2][csize][kRcPart], written by the cluster
    float* cfin = slot + 2 * cluster_nctarank() * kRcPart;              // [rows][16]
    float* rs = cfin + kRcRows * kRnRank;                               // [kRcMaxStages][rows]
    uint8_t* exbuf = reinterpret_cast<uint8_t*>(rs + kRcMaxStages * kRcRows);     // [kRcExBytes]
    uint64_t* full = reinterpret_cast<uint64_t*>(exbuf + kRcExBytes);   // [kRcMaxStages] rows landed
    uint64_t* ready = full + kRcMaxStages;                              // [kRcMaxStages] scales of the stage written
    uint64_t* xbar = ready + kRcMaxStages;                              // [2] partials of a tile received
    volatile int* abort_flag = reinterpret_cast<volatile int*>(xbar + 2);
    // this rank's groups of the second stage: weights [2*ng][16] halves, zero beyond the router's
    // rank, then the biases [2*ng] halves (only when wr_staged: they fit behind the rest)
    uint8_t* wr = reinterpret_cast<uint8_t*>(xbar + 2) + 16;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
    // the groups whose logits and decisions this rank computes, for all 16 rows of a tile
    const int g0 = static_cast<int>(int64_t(p.NG) * rank / csize);
    const int ng = static_cast<int>(int64_t(p.NG) * (rank + 1) / csize) - g0;
    uint8_t* wrb = wr + size_t(2 * ng) * kRnRank * 2;
    const int64_t col0 = int64_t(rank) * hc;
    const int64_t ntiles = (p.M + kRcRows - 1) / kRcRows;
    const int64_t first = cluster_id_x(), step = cluster_count_x();
    auto rows_of = [&](int64_t t) -> int {
        const int64_t left = p.M - t * kRcRows;
        return left < kRcRows ? static_cast<int>(left) : kRcRows;
    };

    if (tid == 0) {
        for (int s = 0; s < kRcMaxStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&ready[s], 1);
        }
        mbar_init(&xbar[0], 1);
        mbar_init(&xbar[1], 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (wr_staged) {
        uint16_t* w16 = reinterpret_cast<uint16_t*>(wr);
        const uint16_t* src = reinterpret_cast<const uint16_t*>(p.w_route) + int64_t(2 * g0) * p.R;
        for (int i = tid; i < 2 * ng * kRnRank; i += kRcThreads) {
            const int n = i / kRnRank, k = i % kRnRank;
            w16[i] = k < p.R ? src[int64_t(n) * p.R + k] : uint16_t(0);
        }
        uint16_t* b16 = reinterpret_cast<uint16_t*>(wrb);
        for (int i = tid; i < 2 * ng; i += kRcThreads)
            b16[i] = p.b_route ? reinterpret_cast<const uint16_t*>(p.b_route)[2 * g0 + i] : uint16_t(0);
    }
    __syncthreads();
    cluster_sync_all();       // every CTA's barriers exist before a peer pushes to them

    if (warp < kRcGWarps) {
        // =============================== contracting warps ===============================
        const int frow = lane >> 2;           // fragment row (A: rows frow and frow + 8) / column (B)
        const int fq = lane & 3;
        const int fk = fq * 8;                // this thread's 8 consecutive k inside a 32-wide block
        const int kblocks = hc / 32;
        const uint32_t xbytes = csize * static_cast<uint32_t>(kRcPart) * 4u;
        const int ntile8 = (2 * ng + 7) / 8;            // 8-column tiles of this rank's share of the second stage
        // this rank's decisions of a tile are collected in shared memory and leave as 4-byte stores
        // where every row's run of ng bytes starts and ends on a 4-byte boundary
        const bool ex_staged = kRcRows * ng <= kRcExBytes && ng % 4 == 0 && g0 % 4 == 0 && p.NG % 4 == 0 &&
                               (reinterpret_cast<uintptr_t>(p.execute) & 3u) == 0;

        // this thread's fragments of the weight slice, for the whole launch
        uint4 wf0[kRcKPerWarp], wf1[kRcKPerWarp];
#pragma unroll
        for (int i = 0; i < kRcKPerWarp; ++i) {
            const int kb = warp + i * kRcGWarps;
            wf0[i] = wf1[i] = make_uint4(0, 0, 0, 0);
            if (kb < kblocks) {
                const int64_t k = col0 + kb * 32 + fk;
                if (frow < p.R) wf0[i] = __ldg(reinterpret_cast<const uint4*>(p.w_down + (int64_t(frow) * p.H + k) * 2));
                if (frow + 8 < p.R)
                    wf1[i] = __ldg(reinterpret_cast<const uint4*>(p.w_down + (int64_t(frow + 8) * p.H + k) * 2));
            }
        }
        // first-stage bias of the column this thread finishes (a global load inside the loop would
        // put a round trip to L2 on every tile's critical path)
        const float bias_down = (tid % kRnRank < p.R && p.b_down) ? half_at<kBf16>(p.b_down, tid % kRnRank) : 0.f;
        int64_t it = 0;
        for (int64_t tile = first; tile < ntiles; tile += step, ++it) {
            const int s = static_cast<int>(it % stages);
            const uint32_t phase = static_cast<uint32_t>(it / stages) & 1u;
            const int par = static_cast<int>(it & 1);
            const uint32_t xphase = static_cast<uint32_t>(it >> 1) & 1u;
            const int64_t row0 = tile * kRcRows;
            const uint8_t* rows = ring + size_t(s) * kRcRows * pitch;
            if (tid == 0) mbar_arrive_expect_tx(&xbar[par], xbytes);
            if (!group_all(1, mbar_wait(&full[s], phase, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL))) break;

            // ---- first stage against the weight fragments, and the sums of squares -------------
            {
                float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
                float acc2[4] = {0.f, 0.f, 0.f, 0.f}, acc3[4] = {0.f, 0.f, 0.f, 0.f};
                float2 ssa = make_float2(0.f, 0.f), ssb = make_float2(0.f, 0.f);
                const uint8_t* xra = rows + size_t(frow) * pitch + fk * 2;
                const uint8_t* xrb = xra + size_t(8) * pitch;
#pragma unroll
                for (int i = 0; i < kRcKPerWarp; ++i) {
                    const int kb = warp + i * kRcGWarps;
                    if (kb < kblocks) {
                        // rows beyond a ragged last tile hold stale bytes: each row of the tile is
                        // independent in the MMA and in the sums, and nothing of those rows is stored
                        const uint4 xa = *reinterpret_cast<const uint4*>(xra + kb * 64);
                        const uint4 xb = *reinterpret_cast<const uint4*>(xrb + kb * 64);
                        const uint32_t xav[4] = {xa.x, xa.y, xa.z, xa.w}, xbv[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float lo, hi;
                            unpack_half2<kBf16>(xav[j], lo, hi);
                            fma_sq2(ssa, lo, hi);
                            unpack_half2<kBf16>(xbv[j], lo, hi);
                            fma_sq2(ssb, lo, hi);
                        }
                        // two accumulator sets per output half: shorter dependent chains
                        rc_mma<kBf16>(acc0, xa.x, xb.x, xa.y, xb.y, wf0[i].x, wf0[i].y);
                        rc_mma<kBf16>(acc1, xa.x, xb.x, xa.y, xb.y, wf1[i].x, wf1[i].y);
                        rc_mma<kBf16>(acc2, xa.z, xb.z, xa.w, xb.w, wf0[i].z, wf0[i].w);
                        rc_mma<kBf16>(acc3, xa.z, xb.z, xa.w, xb.w, wf1[i].z, wf1[i].w);
                    }
                }
                float sa = ssa.x + ssa.y, sb = ssb.x + ssb.y;
                sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                sb += __shfl_xor_sync(0xffffffffu, sb, 1);
                sb += __shfl_xor_sync(0xffffffffu, sb, 2);
                float* cpa = cpart + (warp * kRcRows + frow) * kRnRank + fq * 2;
                float* cpb = cpa + 8 * kRnRank;
                cpa[0] = acc0[0] + acc2[0];
                cpa[1] = acc0[1] + acc2[1];
                cpa[8] = acc1[0] + acc3[0];
                cpa[9] = acc1[1] + acc3[1];
                cpb[0] = acc0[2] + acc2[2];
                cpb[1] = acc0[3] + acc2[3];
                cpb[8] = acc1[2] + acc3[2];
                cpb[9] = acc1[3] + acc3[3];
                if (fq == 0) {
                    sspart[warp * kRcRows + frow] = sa;
                    sspart[warp * kRcRows + frow + 8] = sb;
                }
            }
            group_sync(1);

            // ---- this CTA's partials go to every rank of the cluster ------------------------------------
            for (int e = tid; e < kRcPart; e += kRcGroup) {
                float v = 0.f;
                if (e < kRcRows * kRnRank) {
#pragma unroll
                    for (int w = 0; w < kRcGWarps; ++w) v += cpart[w * kRcRows * kRnRank + e];
                } else {
#pragma unroll
                    for (int w = 0; w < kRcGWarps; ++w) v += sspart[w * kRcRows + e - kRcRows * kRnRank];
                }
                const float* own = slot + (par * static_cast<int>(csize) + static_cast<int>(rank)) * kRcPart + e;
                for (uint32_t dst = 0; dst < csize; ++dst)
                    st_async_f32(cluster_addr(own, dst), v, cluster_addr(&xbar[par], dst));
            }
            if (!group_all(1, mbar_wait(&xbar[par], xphase, abort_flag, p.status, DPK_DEV_TIMEOUT_PEER))) break;
            for (int e = tid; e < kRcPart; e += kRcGroup) {
                const float* src = slot + par * static_cast<int>(csize) * kRcPart + e;
                float v = 0.f;
                for (uint32_t c = 0; c < csize; ++c) v += src[c * kRcPart];
                if (e < kRcRows * kRnRank) {
                    const int j = e % kRnRank;          // == tid % kRnRank
                    v += bias_down;
                    if (p.round_like_module) v = round_half<kBf16>(v);
                    cfin[e] = j < p.R ? v : 0.f;
                } else {
                    rs[s * kRcRows + e - kRcRows * kRnRank] = rsqrtf(v / static_cast<float>(p.H) + p.eps);
                }
            }
            group_sync(1);
            if (tid == 0) mbar_arrive(&ready[s]);      // the normalising warps may take the stage

            // ---- second stage and the decisions: all 16 rows, this rank's groups ------------------------
            const int nrows = rows_of(tile);
            auto record = [&](int r, int gl, float la, float lb) {      // row of the tile, group of this rank
                const uint8_t e = la >= lb ? 1 : 0;
                if (ex_staged)
                    exbuf[r * ng + gl] = e;
                else
                    p.execute[(row0 + r) * p.NG + g0 + gl] = e;
                if (p.logits)
                    *reinterpret_cast<float2*>(p.logits + ((row0 + r) * p.NG + g0 + gl) * 2) = make_float2(la, lb);
            };
            if (p.round_like_module) {
                // A = the finished contraction of the 16 rows (exact in the tensor dtype)
                const float* ca = cfin + frow * kRnRank + fq * 2;
                const float* cb = ca + 8 * kRnRank;
                const uint32_t a0 = pack_half2<kBf16>(ca[0], ca[1]), a2 = pack_half2<kBf16>(ca[8], ca[9]);
                const uint32_t a1 = pack_half2<kBf16>(cb[0], cb[1]), a3 = pack_half2<kBf16>(cb[8], cb[9]);
                for (int nt = warp; nt < ntile8; nt += kRcGWarps) {
                    const int nb = nt * 8 + frow, gl = nt * 4 + fq;      // columns 2 gl, 2 gl + 1 are this thread's
                    const bool nb_ok = nb < 2 * ng, g_ok = gl < ng;
                    uint32_t b0, b1;
                    float ba = 0.f, bb = 0.f;
                    if (wr_staged) {
                        const uint32_t* wrow = reinterpret_cast<const uint32_t*>(wr + size_t(nb) * kRnRank * 2);
                        b0 = nb_ok ? wrow[fq] : 0u;
                        b1 = nb_ok ? wrow[fq + 4] : 0u;
                        if (g_ok) unpack_half2<kBf16>(reinterpret_cast<const uint32_t*>(wrb)[gl], ba, bb);
                    } else {
                        b0 = route_pair<kBf16>(p, 2 * g0 + nb, fq * 2, nb_ok);
                        b1 = route_pair<kBf16>(p, 2 * g0 + nb, fq * 2 + 8, nb_ok);
                        if (g_ok && p.b_route) {
                            ba = half_at<kBf16>(p.b_route, 2 * (g0 + gl));
                            bb = half_at<kBf16>(p.b_route, 2 * (g0 + gl) + 1);
                        }
                    }
                    float l[4] = {0.f, 0.f, 0.f, 0.f};
                    rc_mma<kBf16>(l, a0, a1, a2, a3, b0, b1);
                    if (g_ok) {
                        if (frow < nrows) record(frow, gl, round_half<kBf16>(l[0] + ba), round_half<kBf16>(l[1] + bb));
                        if (frow + 8 < nrows)
                            record(frow + 8, gl, round_half<kBf16>(l[2] + ba), round_half<kBf16>(l[3] + bb));
                    }
                }
            } else {
                for (int item = tid; item < nrows * ng; item += kRcGroup) {
                    const int r = item / ng, gl = item % ng, g = g0 + gl;
                    float la = 0.f, lb = 0.f;
                    for (int j = 0; j < p.R; ++j) {
                        const float c = cfin[r * kRnRank + j];
                        la = fmaf(c, half_at<kBf16>(p.w_route, int64_t(2 * g) * p.R + j), la);
                        lb = fmaf(c, half_at<kBf16>(p.w_route, int64_t(2 * g + 1) * p.R + j), lb);
                    }
                    if (p.b_route) {
                        la += half_at<kBf16>(p.b_route, 2 * g);
                        lb += half_at<kBf16>(p.b_route, 2 * g + 1);
                    }
                    record(r, gl, la, lb);
                }
            }
            if (ex_staged) {
                group_sync(1);
                const int wpr = ng / 4;                              // 4-byte words per row
                const uint32_t* src = reinterpret_cast<const uint32_t*>(exbuf);
                for (int i = tid; i < nrows * wpr; i += kRcGroup) {
                    const int r = i / wpr, w = i % wpr;
                    reinterpret_cast<uint32_t*>(p.execute + (row0 + r) * p.NG + g0)[w] = src[i];
                }
                // the next tile writes exbuf after two more group barriers
            }
        }
    } else {
        // =============================== normalising warps ===============================
        const int gt = tid - kRcGroup, gw = warp - kRcGWarps;      // thread / warp index inside the group
        const int chunks = hc / 8;
        // a thread owns one 16-byte column chunk of `rows_per` consecutive rows
        int nsplit = kRcGroup / chunks;
        nsplit = nsplit < 1 ? 1 : (nsplit > kRcRows ? kRcRows : nsplit);
        while (kRcRows % nsplit) --nsplit;
        const int rows_per = kRcRows / nsplit;
        // chunks * nsplit <= kRcGroup: one chunk per thread, its gamma in registers for all tiles
        const bool norm_thread = p.xn && gt < chunks * nsplit;
        const int nc = gt % chunks, nr0 = (gt / chunks) * rows_per;
        uint32_t gv[4] = {0u, 0u, 0u, 0u};
        if (norm_thread) {
            const uint4 ga = __ldg(reinterpret_cast<const uint4*>(p.gamma + (col0 + nc * 8) * 2));
            gv[0] = ga.x;
            gv[1] = ga.y;
            gv[2] = ga.z;
            gv[3] = ga.w;
        }
        // lane r of the first warp moves row r of a stage, in and out; lane 0 announces the bytes
        // (the barrier cannot complete before that arrival, whichever comes first)
        auto load_tile = [&](int64_t t, int s) {
            const int n = rows_of(t);
            if (lane == 0) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(n) * hc * 2);
            if (lane < n)
                bulk_load_row(ring + (size_t(s) * kRcRows + lane) * pitch,
                              p.x + ((t * kRcRows + lane) * p.ldx + col0) * 2, hc * 2, &full[s]);
        };
        if (gw == 0)
            for (int s = 0; s < stages; ++s)
                if (first + s * step < ntiles) load_tile(first + s * step, s);

        int64_t it = 0;
        for (int64_t tile = first; tile < ntiles; tile += step, ++it) {
            const int s = static_cast<int>(it % stages);
            const uint32_t phase = static_cast<uint32_t>(it / stages) & 1u;
            const int64_t row0 = tile * kRcRows;
            const int nrows = rows_of(tile);
            uint8_t* rows = ring + size_t(s) * kRcRows * pitch;
            // ready[s] says that the scales are written and the contraction has read the rows;
            // full[s] completed long ago, but observing it is what makes the bulk copy's bytes
            // visible to this thread
            if (!group_all(2, mbar_wait(&ready[s], phase, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY) &&
                                  mbar_wait(&full[s], phase, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)))
                break;
            if (norm_thread) {
                uint8_t* src = rows + size_t(nr0) * pitch + nc * 16;
                const int rend = nrows - nr0 < rows_per ? nrows - nr0 : rows_per;
#pragma unroll 4
                for (int r = 0; r < rend; ++r) {
                    // the product dtype(x * scale) * weight is a packed multiply in the tensor
                    // dtype, which rounds exactly as the module's elementwise multiply does
                    const float scale = rs[s * kRcRows + nr0 + r];
                    const uint4 xa = *reinterpret_cast<const uint4*>(src + size_t(r) * pitch);
                    const uint32_t xv[4] = {xa.x, xa.y, xa.z, xa.w};
                    uint32_t ov[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float lo, hi;
                        unpack_half2<kBf16>(xv[j], lo, hi);
                        mul_s2(lo, hi, scale);
                        ov[j] = mul_half2<kBf16>(pack_half2<kBf16>(lo, hi), gv[j]);
                    }
                    *reinterpret_cast<uint4*>(src + size_t(r) * pitch) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
                }
                fence_proxy_async_smem();      // the bulk stores below read what this thread wrote
            }
            group_sync(2);
            if (gw == 0) {
                if (p.xn && lane < nrows)
                    bulk_store_row(p.xn + ((row0 + lane) * p.ldxn + col0) * 2, rows + size_t(lane) * pitch, hc * 2);
                bulk_commit();
                // the stage of the tile before this one: its rows left one tile ago; refill it
                if (it > 0) {
                    bulk_wait_read_but_one();
                    const int64_t next = tile - step + int64_t(stages) * step;
                    if (next < ntiles) load_tile(next, static_cast<int>((it - 1) % stages));
                }
            }
        }
        if (gw == 0) bulk_wait_all();         // the last rows have left shared memory
    }
    cluster_sync_all();           // nobody leaves while a peer may still push into its slots
}

}  // namespace dpk

using namespace dpk;

namespace {

int g_rn_cluster = 1;      // 1: column-split cluster kernel where the shape allows it; 0: never

// cluster size for H columns: the smallest of 1, 2, 4, 8 whose slice fits; 0 if none does
int rn_cluster_size(int H)
{
    for (int c = 1; c <= 8; c *= 2)
        if (H % (c * 32) == 0 && H / c <= kRcMaxSlice) return c;
    return 0;
}

size_t rn_cluster_smem(int hc, int stages, int csize)
{
    const size_t pitch = size_t(hc) * 2 + kRnSkew;
    return size_t(stages) * kRcRows * pitch +
           sizeof(float) * (kRcGWarps * kRcRows * kRnRank + kRcGWarps * kRcRows + 2 * csize * kRcPart +
                            kRcRows * kRnRank + kRcMaxStages * kRcRows) +
           kRcExBytes + sizeof(uint64_t) * (2 * kRcMaxStages + 2) + 16;
}

// a rank's share of the second-stage weights and biases staged in shared memory, as halves
size_t rn_route_smem(int NG, int csize) { return size_t(2 * ((NG + csize - 1) / csize)) * (kRnRank + 1) * 2 + 16; }

template <bool kBf16>
int launch_router_norm_cluster(const RouterNormParams& p, int csize, cudaStream_t s)
{
    const int hc = p.H / csize;
    int stages = kRcMaxStages;
    while (stages > 3 && rn_cluster_smem(hc, stages, csize) > 227 * 1024) --stages;
    // the second stage's operands go behind the ring if they fit (else they come from L2 per tile)
    const int wr_staged = rn_cluster_smem(hc, stages, csize) + rn_route_smem(p.NG, csize) <= 227 * 1024 ? 1 : 0;
    const size_t smem = rn_cluster_smem(hc, stages, csize) + (wr_staged ? rn_route_smem(p.NG, csize) : 0);
    DPK_CUDA(cudaFuncSetAttribute(router_norm_cluster_kernel<kBf16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(csize);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kRcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // as many clusters as the device holds at once (it depends on how the SMs are grouped),
    // asked once per (cluster size, shared memory) and kept
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, size_t>, int> resident;
    int dev = 0, clusters = 0;
    DPK_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lock(mu);
        const auto key = std::make_tuple(dev, int(kBf16), csize, smem);
        auto it = resident.find(key);
        if (it == resident.end()) {
            cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / csize * csize));
            DPK_CUDA(cudaOccupancyMaxActiveClusters(&clusters, router_norm_cluster_kernel<kBf16>, &cfg));
            resident[key] = clusters;
        } else {
            clusters = it->second;
        }
    }
    DPK_REQUIRE(clusters > 0, "no cluster of %d CTAs with %zu bytes of shared memory fits this device",
                csize, smem);
    const int64_t ntiles = (p.M + kRcRows - 1) / kRcRows;
    const int64_t nclusters = ntiles < clusters ? ntiles : clusters;
    cfg.gridDim = dim3(static_cast<unsigned>(nclusters * csize));
    DPK_CUDA(cudaLaunchKernelEx(&cfg, router_norm_cluster_kernel<kBf16>, p, hc, stages, wr_staged));
    return DPK_OK;
}

}  // namespace

extern "C" int dpk_set_router_norm_cluster(int on)
{
    DPK_REQUIRE(on == 0 || on == 1, "on must be 0 or 1");
    g_rn_cluster = on;
    return DPK_OK;
}

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
    DPK_REQUIRE((reinterpret_cast<uintptr_t>(w_route) & 3u) == 0, "w_route must be 4-byte aligned");
    if (M == 0) return DPK_OK;
    const size_t smem = size_t(kRnRows) * (size_t(H) * 2 + kRnSkew) +
                        sizeof(float) * (kRnWarps * kRnRows * kRnRank + kRnWarps * kRnRows +
                                         kRnRows * kRnRank + kRnRows) + 32;

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

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int csize = g_rn_cluster ? rn_cluster_size(H) : 0;
    if (csize > 0 && rn_cluster_smem(H / csize, 3, csize) <= 227 * 1024)
        return dtype == DPK_BF16 ? launch_router_norm_cluster<true>(p, csize, s)
                                 : launch_router_norm_cluster<false>(p, csize, s);

    DPK_REQUIRE(smem <= 227 * 1024, "H=%d is too wide for the %d-row tile in shared memory", H, kRnRows);
    const int64_t ntiles = (M + kRnRows - 1) / kRnRows;
    // rows up to ~6000 wide: two CTAs of 256 threads share an SM and overlap each other's
    // phases; wider rows leave room for one CTA, which then runs 512 threads
    const int per_sm = 2 * smem <= 227 * 1024 ? 2 : 1;
    const int threads = per_sm == 2 ? 256 : kRnThreads;
    int64_t grid = int64_t(sm_count()) * per_sm;
    if (grid > ntiles) grid = ntiles;
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
