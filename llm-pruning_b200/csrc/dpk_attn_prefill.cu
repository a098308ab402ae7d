// Head-group-routed prefill attention (flash style, online softmax in registers).
//
// A CTA owns 64 consecutive entries of one (batch, head group) list of active query
// tokens for one query head: it gathers those Q rows, streams the K/V rows of the
// head's KV head through a double-buffered cp.async pipeline, and scatters the
// output rows back to their tokens.  CTAs beyond a group's active count exit at
// once; rows of inactive (token, group) pairs are never touched.  Under causal
// masking the KV range ends at the tile's last (largest) token, and only KV tiles
// that reach past the tile's first token pay for per-element masking.
//
// Tensor path: warp-level mma.sync m16n8k16 (fp32 accumulate) with ldmatrix operand
// fetch; each of the 4 warps owns 16 query rows, the row maximum and sum live in
// registers and are combined across the 4 lanes of a quad with shuffles.
//
// Algorithmic work per launch: 4*D flops per (active query row, visible key) pair.
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kPfBM = 64;
constexpr int kPfBN = 64;
constexpr int kPfThreads = 128;

struct PrefillParams {
    const uint8_t* Q;
    const uint8_t* K;
    const uint8_t* V;
    uint8_t* O;
    const int64_t* sidx;     // [B, Tq, NG]
    const int32_t* counts;   // [B, NG]
    const uint32_t* leftpad; // [B] or null
    int B, Tq, Tk, Hq, Hk, NG;
    float scale_log2;        // scale * log2(e)
    int causal, causal_shift;
    int* status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <bool kBf16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1)
{
    if constexpr (kBf16) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// byte offset of 16-byte chunk `c` of row `r` in a [rows][D] half tile, XOR-swizzled
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c)
{
    return static_cast<uint32_t>(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kPfThreads)
attn_prefill_kernel(const PrefillParams p)
{
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int ROWB = D * 2;
    constexpr int KS = D / 16;           // k-steps of Q.K^T
    constexpr int NT_S = kPfBN / 8;      // score n-tiles per warp row block
    constexpr int NT_O = D / 8;          // output n-tiles
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kPfBM * ROWB;             // 2 buffers
    uint8_t* sV = sK + 2 * kPfBN * ROWB;         // 2 buffers

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, t4 = lane & 3;
    const int mt = gridDim.x - 1 - blockIdx.x;   // heavy (late) tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hpg = p.Hq / p.NG;
    const int g = h / hpg;
    const int kvh = h / (p.Hq / p.Hk);
    const int cnt = p.counts[b * p.NG + g];
    const int m0 = mt * kPfBM;
    if (m0 >= cnt) return;
    const int nrows = min(kPfBM, cnt - m0);
    const int64_t* sidx_b = p.sidx + static_cast<int64_t>(b) * p.Tq * p.NG;

    auto token_of = [&](int row) -> int {
        if (row >= nrows) return -1;
        int64_t t = sidx_b[static_cast<int64_t>(m0 + row) * p.NG + g];
        if (t < 0 || t >= p.Tq) {
            atomicCAS(p.status, 0, DPK_DEV_BAD_INDEX);
            return -1;
        }
        return static_cast<int>(t);
    };

    const int first_tok = token_of(0);
    const int last_tok = token_of(nrows - 1);
    const int lp = p.leftpad ? static_cast<int>(p.leftpad[b]) : 0;
    int kv_end = p.Tk;
    if (p.causal) kv_end = min(p.Tk, last_tok + p.causal_shift + 1);
    const int kv_begin = (lp / kPfBN) * kPfBN;
    const int ntiles = kv_end > kv_begin ? (kv_end - kv_begin + kPfBN - 1) / kPfBN : 0;

    // ---- gather Q rows ---------------------------------------------------------------
    for (int i = tid; i < kPfBM * CH; i += kPfThreads) {
        const int r = i / CH, c = i % CH;
        const int tok = token_of(r);
        const uint8_t* src = p.Q;
        if (tok >= 0)
            src = p.Q + ((static_cast<int64_t>(b) * p.Tq + tok) * p.Hq + h) * ROWB + c * 16;
        cp_async_16(smem_u32(sQ) + tile_off<D>(r, c), src, tok >= 0 ? 16u : 0u);
    }
    const uint8_t* Kb = p.K + (static_cast<int64_t>(b) * p.Tk * p.Hk + kvh) * ROWB;
    const uint8_t* Vb = p.V + (static_cast<int64_t>(b) * p.Tk * p.Hk + kvh) * ROWB;
    const int64_t kv_stride = static_cast<int64_t>(p.Hk) * ROWB;
    auto load_kv = [&](int tile, int buf) {
        const int kv0 = kv_begin + tile * kPfBN;
        for (int i = tid; i < kPfBN * CH; i += kPfThreads) {
            const int r = i / CH, c = i % CH;
            const int kv = kv0 + r;
            const bool on = kv < p.Tk;
            const int64_t off = static_cast<int64_t>(on ? kv : 0) * kv_stride + c * 16;
            cp_async_16(smem_u32(sK + buf * kPfBN * ROWB) + tile_off<D>(r, c), Kb + off, on ? 16u : 0u);
            cp_async_16(smem_u32(sV + buf * kPfBN * ROWB) + tile_off<D>(r, c), Vb + off, on ? 16u : 0u);
        }
    };
    if (ntiles > 0) load_kv(0, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // ---- Q fragments -----------------------------------------------------------------
    uint32_t qf[KS][4];
    {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 2 + (lane >> 4);
            ldsm_x4(smem_u32(sQ) + tile_off<D>(r, c), qf[ks]);
        }
    }
    const int tok_r0 = token_of(warp * 16 + gid);
    const int tok_r1 = token_of(warp * 16 + gid + 8);

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int i = 0; i < ntiles; ++i) {
        const int buf = i & 1;
        if (i + 1 < ntiles) {
            load_kv(i + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kbase = smem_u32(sK + buf * kPfBN * ROWB);
        const uint32_t vbase = smem_u32(sV + buf * kPfBN * ROWB);
        const int kv0 = kv_begin + i * kPfBN;

        // S = Q K^T
        float s[NT_S][4];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int jp = 0; jp < NT_S / 2; ++jp) {
                uint32_t kf[4];
                const int r = jp * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = ks * 2 + ((lane >> 3) & 1);
                ldsm_x4(kbase + tile_off<D>(r, c), kf);
                mma_16816<kBf16>(s[2 * jp], qf[ks], kf[0], kf[1]);
                mma_16816<kBf16>(s[2 * jp + 1], qf[ks], kf[2], kf[3]);
            }
        }

        // masking (only tiles that touch a boundary)
        const bool need_mask = (kv0 < lp) || (kv0 + kPfBN > p.Tk) ||
                               (p.causal && kv0 + kPfBN - 1 > first_tok + p.causal_shift);
        if (need_mask) {
            const int lim0 = p.causal ? min(p.Tk - 1, tok_r0 + p.causal_shift) : p.Tk - 1;
            const int lim1 = p.causal ? min(p.Tk - 1, tok_r1 + p.causal_shift) : p.Tk - 1;
#pragma unroll
            for (int j = 0; j < NT_S; ++j) {
                const int k0 = kv0 + j * 8 + 2 * t4;
                if (k0 < lp || k0 > lim0 || tok_r0 < 0) s[j][0] = -INFINITY;
                if (k0 + 1 < lp || k0 + 1 > lim0 || tok_r0 < 0) s[j][1] = -INFINITY;
                if (k0 < lp || k0 > lim1 || tok_r1 < 0) s[j][2] = -INFINITY;
                if (k0 + 1 < lp || k0 + 1 > lim1 || tok_r1 < 0) s[j][3] = -INFINITY;
            }
        }

        // online softmax
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            tmax0 = fmaxf(tmax0, fmaxf(s[j][0], s[j][1]));
            tmax1 = fmaxf(tmax1, fmaxf(s[j][2], s[j][3]));
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float nm0 = fmaxf(mx0, tmax0), nm1 = fmaxf(mx1, tmax1);
        // a row that has seen no key yet keeps a zero reference to avoid inf - inf
        const float ref0 = nm0 == -INFINITY ? 0.f : nm0 * p.scale_log2;
        const float ref1 = nm1 == -INFINITY ? 0.f : nm1 * p.scale_log2;
        const float corr0 = fast_exp2(mx0 * p.scale_log2 - ref0);
        const float corr1 = fast_exp2(mx1 * p.scale_log2 - ref1);
        mx0 = nm0;
        mx1 = nm1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pf[NT_S][2];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            const float p0 = fast_exp2(s[j][0] * p.scale_log2 - ref0);
            const float p1 = fast_exp2(s[j][1] * p.scale_log2 - ref0);
            const float p2 = fast_exp2(s[j][2] * p.scale_log2 - ref1);
            const float p3 = fast_exp2(s[j][3] * p.scale_log2 - ref1);
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            pf[j][0] = pack_half2<kBf16>(p0, p1);
            pf[j][1] = pack_half2<kBf16>(p2, p3);
        }
        l0 = l0 * corr0 + rs0;
        l1 = l1 * corr1 + rs1;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            o[j][0] *= corr0; o[j][1] *= corr0;
            o[j][2] *= corr1; o[j][3] *= corr1;
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < kPfBN / 16; ++kk) {
            const uint32_t af[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                uint32_t vf[4];
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = jp * 2 + (lane >> 4);
                ldsm_x4_trans(vbase + tile_off<D>(r, c), vf);
                mma_16816<kBf16>(o[2 * jp], af, vf[0], vf[1]);
                mma_16816<kBf16>(o[2 * jp + 1], af, vf[2], vf[3]);
            }
        }
        __syncthreads();
    }

    // ---- normalise, stage through shared memory, scatter rows -------------------------
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
    const float inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    {
        const int r0 = warp * 16 + gid, r1 = r0 + 8;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            // n-tile j = 16-byte chunk j of the row; this thread owns 4 bytes of it
            *reinterpret_cast<uint32_t*>(sQ + tile_off<D>(r0, j) + t4 * 4) =
                pack_half2<kBf16>(o[j][0] * inv0, o[j][1] * inv0);
            *reinterpret_cast<uint32_t*>(sQ + tile_off<D>(r1, j) + t4 * 4) =
                pack_half2<kBf16>(o[j][2] * inv1, o[j][3] * inv1);
        }
    }
    __syncthreads();
    for (int i = tid; i < kPfBM * CH; i += kPfThreads) {
        const int r = i / CH, c = i % CH;
        const int tok = token_of(r);
        if (tok >= 0) {
            uint4 v = *reinterpret_cast<const uint4*>(sQ + tile_off<D>(r, c));
            *reinterpret_cast<uint4*>(p.O + ((static_cast<int64_t>(b) * p.Tq + tok) * p.Hq + h) * ROWB +
                                      c * 16) = v;
        }
    }
}

template <int D, bool kBf16>
static int launch_prefill(const PrefillParams& p, cudaStream_t s)
{
    constexpr size_t smem = size_t(kPfBM + 4 * kPfBN) * D * 2;
    DPK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<D, kBf16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((p.Tq + kPfBM - 1) / kPfBM, p.Hq, p.B);
    attn_prefill_kernel<D, kBf16><<<grid, kPfThreads, smem, s>>>(p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_attn_prefill(const void* Q, const void* K, const void* V,
                                const int64_t* sorted_indices, const int32_t* counts,
                                const uint32_t* leftpad, void* O, int B, int Tq, int Tk, int Hq,
                                int Hk, int D, int NG, float scale, int causal, int causal_shift,
                                int dtype, void* stream)
{
    DPK_REQUIRE(Q && K && V && O && sorted_indices && counts, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(B >= 0 && Tq >= 0 && Tk >= 0 && Hq > 0 && Hk > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(D == 64 || D == 128, "head_dim %d not supported (64 or 128)", D);
    DPK_REQUIRE(Hq % Hk == 0, "Hq=%d must be a multiple of Hk=%d", Hq, Hk);
    DPK_REQUIRE(Hq % NG == 0, "Hq=%d must be a multiple of NG=%d", Hq, NG);
    DPK_REQUIRE(B <= 65535 && Hq <= 65535, "grid too large");
    DPK_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O),
                "tensors must be 16-byte aligned");
    if (B == 0 || Tq == 0) return DPK_OK;

    PrefillParams p;
    p.Q = static_cast<const uint8_t*>(Q);
    p.K = static_cast<const uint8_t*>(K);
    p.V = static_cast<const uint8_t*>(V);
    p.O = static_cast<uint8_t*>(O);
    p.sidx = sorted_indices;
    p.counts = counts;
    p.leftpad = leftpad;
    p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hk = Hk; p.NG = NG;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal ? 1 : 0;
    p.causal_shift = causal_shift;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (D == 64) return dtype == DPK_BF16 ? launch_prefill<64, true>(p, s) : launch_prefill<64, false>(p, s);
    return dtype == DPK_BF16 ? launch_prefill<128, true>(p, s) : launch_prefill<128, false>(p, s);
}
