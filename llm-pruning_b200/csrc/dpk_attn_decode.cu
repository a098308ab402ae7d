// Head-group-routed decode attention: one query token per sequence, split over the
// KV length and merged by log-sum-exp.
//
// Stage 1: a CTA owns one (KV split, KV head, sequence).  It exits at once when none
// of the query-head groups that read this KV head is active for the sequence, so the
// K/V rows of skipped heads are never fetched.  Otherwise its 4 warps walk disjoint
// 32-row K/V tiles of the split, each warp with its own 3-deep cp.async pipeline and
// its own online-softmax state; the Hq/Hk query heads that share the KV head form
// the (zero padded) 16-row operand of one mma.sync tile, so every K/V byte is read
// once for all of them.  The warps' partial results are combined in shared memory
// and written as one un-normalised fp32 row + (max, sum) per (sequence, head, split).
// Stage 2 merges the splits, normalises, converts, and writes zeros for inactive
// heads.
//
// This path is bounded by HBM: algorithmic bytes per launch = 2 * Tk * D * 2 bytes per
// active (sequence, KV head) pair.
#define DPK_KERNEL_ID 6   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kDecBN = 32;          // KV rows per warp tile
constexpr int kDecStages = 3;
constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kDecMaxSplits = 32;

struct DecodeParams {
    const uint8_t* Q;
    const uint8_t* K;
    const uint8_t* V;
    const uint8_t* mask;      // [B, NG]
    const uint32_t* leftpad;  // [B] or null
    float* pO;                // [B, Hq, splits, D]
    float* pML;               // [B, Hq, splits, 2]
    int B, Tk, Hq, Hk, NG;
    int64_t kv_ts, kv_bs;    // elements between consecutive cached tokens / sequences of K and V
    int splits, split_len;
    float scale_log2;
};

__device__ __forceinline__ void dec_ldsm_x4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void dec_ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <bool kBf16>
__device__ __forceinline__ void dec_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
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
__device__ __forceinline__ float dec_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int D>
__device__ __forceinline__ uint32_t dec_off(int r, int c)
{
    return static_cast<uint32_t>(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_kernel(const DecodeParams p)
{
    constexpr int CH = D / 8;
    constexpr int ROWB = D * 2;
    constexpr int KS = D / 16;
    constexpr int NT_S = kDecBN / 8;
    constexpr int NT_O = D / 8;
    constexpr int TILE_B = kDecBN * ROWB;                 // bytes of one K (or V) tile
    constexpr int WARP_B = kDecStages * 2 * TILE_B;       // per-warp pipeline bytes
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;                                   // [16][D]
    uint8_t* sPipe = smem + 16 * ROWB;                    // [warps][stages][K|V]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, t4 = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int rep = p.Hq / p.Hk;
    const int hpg = p.Hq / p.NG;
    const int h0 = kvh * rep;

    // is any query head of this KV head routed in?
    bool any = false;
    for (int i = 0; i < rep; ++i) any |= p.mask[b * p.NG + (h0 + i) / hpg] != 0;
    if (!any) return;

    const int lp = p.leftpad ? static_cast<int>(p.leftpad[b]) : 0;
    const int kv_lo = split * p.split_len;
    const int kv_hi = min(p.Tk, kv_lo + p.split_len);
    const int first_tile = max(kv_lo, (lp / kDecBN) * kDecBN);   // split_len is a multiple of 32
    const int ntiles_all = kv_hi > first_tile ? (kv_hi - first_tile + kDecBN - 1) / kDecBN : 0;
    // warp w takes tiles w, w+4, ...
    const int my_tiles = ntiles_all > warp ? (ntiles_all - warp + kDecWarps - 1) / kDecWarps : 0;

    // ---- Q rows of the rep heads, zero padded to 16 -----------------------------------
    for (int i = tid; i < 16 * CH; i += kDecThreads) {
        const int r = i / CH, c = i % CH;
        const bool on = r < rep;
        const uint8_t* src = p.Q + ((static_cast<int64_t>(b) * p.Hq + h0 + (on ? r : 0)) * ROWB) + c * 16;
        cp_async_16(smem_u32(sQ) + dec_off<D>(r, c), src, on ? 16u : 0u);
    }
    cp_async_commit();

    const uint8_t* Kb = p.K + static_cast<int64_t>(b) * p.kv_bs * 2 + static_cast<int64_t>(kvh) * ROWB;
    const uint8_t* Vb = p.V + static_cast<int64_t>(b) * p.kv_bs * 2 + static_cast<int64_t>(kvh) * ROWB;
    const int64_t kv_stride = p.kv_ts * 2;
    uint8_t* myPipe = sPipe + warp * WARP_B;
    auto load_tile = [&](int t, int stage) {
        const int kv0 = first_tile + (warp + t * kDecWarps) * kDecBN;
        const uint32_t kdst = smem_u32(myPipe + stage * 2 * TILE_B);
        const uint32_t vdst = kdst + TILE_B;
        for (int i = lane; i < kDecBN * CH; i += 32) {
            const int r = i / CH, c = i % CH;
            const int kv = kv0 + r;
            const bool on = kv < kv_hi;
            const int64_t off = static_cast<int64_t>(on ? kv : 0) * kv_stride + c * 16;
            cp_async_16(kdst + dec_off<D>(r, c), Kb + off, on ? 16u : 0u);
            cp_async_16(vdst + dec_off<D>(r, c), Vb + off, on ? 16u : 0u);
        }
    };
    // prologue: stages 0 .. kDecStages-2 (one commit group per stage, empty if past the end)
#pragma unroll
    for (int s = 0; s < kDecStages - 1; ++s) {
        if (s < my_tiles) load_tile(s, s);
        cp_async_commit();
    }
    // Q was the oldest group: everything but the kDecStages-1 tile groups is complete
    cp_async_wait<kDecStages - 1>();
    __syncthreads();

    uint32_t qf[KS][4];
    {
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
            dec_ldsm_x4(smem_u32(sQ) + dec_off<D>(r, ks * 2 + (lane >> 4)), qf[ks]);
    }

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int t = 0; t < my_tiles; ++t) {
        // keep kDecStages-1 tiles in flight
        const int nt = t + kDecStages - 1;
        if (nt < my_tiles) load_tile(nt, nt % kDecStages);
        cp_async_commit();
        cp_async_wait<kDecStages - 1>();
        __syncwarp();
        const int stage = t % kDecStages;
        const uint32_t kbase = smem_u32(myPipe + stage * 2 * TILE_B);
        const uint32_t vbase = kbase + TILE_B;
        const int kv0 = first_tile + (warp + t * kDecWarps) * kDecBN;

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
                dec_ldsm_x4(kbase + dec_off<D>(r, c), kf);
                dec_mma<kBf16>(s[2 * jp], qf[ks], kf[0], kf[1]);
                dec_mma<kBf16>(s[2 * jp + 1], qf[ks], kf[2], kf[3]);
            }
        }
        if (kv0 < lp || kv0 + kDecBN > kv_hi) {
#pragma unroll
            for (int j = 0; j < NT_S; ++j) {
                const int k0 = kv0 + j * 8 + 2 * t4;
                if (k0 < lp || k0 >= kv_hi) { s[j][0] = -INFINITY; s[j][2] = -INFINITY; }
                if (k0 + 1 < lp || k0 + 1 >= kv_hi) { s[j][1] = -INFINITY; s[j][3] = -INFINITY; }
            }
        }
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
        const float ref0 = nm0 == -INFINITY ? 0.f : nm0 * p.scale_log2;
        const float ref1 = nm1 == -INFINITY ? 0.f : nm1 * p.scale_log2;
        const float corr0 = dec_exp2(mx0 * p.scale_log2 - ref0);
        const float corr1 = dec_exp2(mx1 * p.scale_log2 - ref1);
        mx0 = nm0;
        mx1 = nm1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pf[NT_S][2];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            const float p0 = dec_exp2(s[j][0] * p.scale_log2 - ref0);
            const float p1 = dec_exp2(s[j][1] * p.scale_log2 - ref0);
            const float p2 = dec_exp2(s[j][2] * p.scale_log2 - ref1);
            const float p3 = dec_exp2(s[j][3] * p.scale_log2 - ref1);
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
#pragma unroll
        for (int kk = 0; kk < kDecBN / 16; ++kk) {
            const uint32_t af[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                uint32_t vf[4];
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = jp * 2 + (lane >> 4);
                dec_ldsm_x4_trans(vbase + dec_off<D>(r, c), vf);
                dec_mma<kBf16>(o[2 * jp], af, vf[0], vf[1]);
                dec_mma<kBf16>(o[2 * jp + 1], af, vf[2], vf[3]);
            }
        }
        __syncwarp();   // the stage is refilled by the next iteration's loads
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- combine the 4 warps through shared memory ---------------------------------------
    __syncthreads();   // every warp is done with its pipeline buffers
    float* cO = reinterpret_cast<float*>(sPipe);               // [warps][16][D]
    float* cML = cO + kDecWarps * 16 * D;                      // [warps][16][2]
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        float* r0p = cO + (warp * 16 + gid) * D + j * 8 + 2 * t4;
        float* r1p = cO + (warp * 16 + gid + 8) * D + j * 8 + 2 * t4;
        r0p[0] = o[j][0]; r0p[1] = o[j][1];
        r1p[0] = o[j][2]; r1p[1] = o[j][3];
    }
    if (t4 == 0) {
        cML[(warp * 16 + gid) * 2] = mx0;
        cML[(warp * 16 + gid) * 2 + 1] = l0;
        cML[(warp * 16 + gid + 8) * 2] = mx1;
        cML[(warp * 16 + gid + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int r = warp; r < rep; r += kDecWarps) {
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, cML[(w * 16 + r) * 2]);
        float wgt[kDecWarps];
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float mw = cML[(w * 16 + r) * 2];
            wgt[w] = (mw == -INFINITY) ? 0.f : dec_exp2((mw - m) * p.scale_log2);
            l += wgt[w] * cML[(w * 16 + r) * 2 + 1];
        }
        const int64_t slot = (static_cast<int64_t>(b) * p.Hq + h0 + r) * p.splits + split;
        for (int c = lane; c < D; c += 32) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) acc += wgt[w] * cO[(w * 16 + r) * D + c];
            p.pO[slot * D + c] = acc;
        }
        if (lane == 0) {
            p.pML[slot * 2] = m;
            p.pML[slot * 2 + 1] = l;
        }
    }
}

// stage 2: merge splits; grid (Hq, B), D threads
template <bool kBf16>
__global__ void attn_decode_merge_kernel(const float* __restrict__ pO, const float* __restrict__ pML,
                                         const uint8_t* __restrict__ mask, uint8_t* __restrict__ O,
                                         int Hq, int NG, int D, int splits, float scale_log2)
{
    const int h = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
    const int hpg = Hq / NG;
    const bool on = mask[b * NG + h / hpg] != 0;
    float out = 0.f;
    if (on) {
        const int64_t base = (static_cast<int64_t>(b) * Hq + h) * splits;
        float m = -INFINITY;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, pML[(base + s) * 2]);
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = pML[(base + s) * 2];
            const float w = (ms == -INFINITY) ? 0.f : exp2f((ms - m) * scale_log2);
            l += w * pML[(base + s) * 2 + 1];
            acc += w * pO[(base + s) * D + c];
        }
        out = l > 0.f ? acc / l : 0.f;
    }
    uint8_t* dst = O + ((static_cast<int64_t>(b) * Hq + h) * D + c) * 2;
    if constexpr (kBf16) *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(out);
    else *reinterpret_cast<__half*>(dst) = __float2half_rn(out);
}

static int decode_splits(int B, int Tk, int Hk)
{
    int splits = Tk / 1024;
    if (splits > kDecMaxSplits) splits = kDecMaxSplits;
    if (splits < 1) splits = 1;
    const long long max_ctas = 16ll * sm_count();
    while (splits > 1 && (long long)B * Hk * splits / 2 > max_ctas) splits /= 2;
    return splits;
}

template <int D, bool kBf16>
static int launch_decode(const DecodeParams& p, const uint8_t* mask, void* O, cudaStream_t s)
{
    constexpr size_t pipe = size_t(kDecWarps) * kDecStages * 2 * kDecBN * D * 2;
    constexpr size_t comb = size_t(kDecWarps) * 16 * (D + 2) * sizeof(float);
    constexpr size_t smem = 16 * D * 2 + (pipe > comb ? pipe : comb);
    DPK_CUDA(cudaFuncSetAttribute(attn_decode_kernel<D, kBf16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(p.splits, p.Hk, p.B);
    attn_decode_kernel<D, kBf16><<<grid, kDecThreads, smem, s>>>(p);
    dim3 mgrid(p.Hq, p.B);
    attn_decode_merge_kernel<kBf16><<<mgrid, D, 0, s>>>(p.pO, p.pML, mask, static_cast<uint8_t*>(O),
                                                         p.Hq, p.NG, D, p.splits, p.scale_log2);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk

using namespace dpk;

extern "C" {

size_t dpk_attn_decode_workspace_bytes(int B, int Tk, int Hq, int Hk, int D, int NG)
{
    (void)Tk; (void)Hk; (void)NG;
    if (B < 1 || Hq < 1 || D < 1) return 0;
    // sized for the largest split count so that the size does not depend on the device
    return size_t(B) * Hq * kDecMaxSplits * (size_t(D) + 2) * sizeof(float);
}

int dpk_attn_decode(const void* Q, const void* K, const void* V, const uint8_t* mask,
                    const uint32_t* leftpad, void* O, int B, int Tk, int Hq, int Hk, int D, int NG,
                    float scale, int dtype, int64_t kv_token_stride, int64_t kv_batch_stride,
                    void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(Q && K && V && O && mask, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(B >= 0 && Tk >= 0 && Hq > 0 && Hk > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(D == 64 || D == 128, "head_dim %d not supported (64 or 128)", D);
    DPK_REQUIRE(Hq % Hk == 0, "Hq=%d must be a multiple of Hk=%d", Hq, Hk);
    DPK_REQUIRE(Hq % NG == 0, "Hq=%d must be a multiple of NG=%d", Hq, NG);
    DPK_REQUIRE(Hq / Hk <= 16, "more than 16 query heads per KV head are not supported");
    DPK_REQUIRE(B <= 65535 && Hk <= 65535, "grid too large");
    DPK_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V), "tensors must be 16-byte aligned");
    const int64_t kv_ts = kv_token_stride ? kv_token_stride : static_cast<int64_t>(Hk) * D;
    const int64_t kv_bs = kv_batch_stride ? kv_batch_stride : static_cast<int64_t>(Tk) * kv_ts;
    DPK_REQUIRE(kv_ts >= static_cast<int64_t>(Hk) * D && kv_ts % 8 == 0 && kv_bs % 8 == 0,
                "K/V strides must cover a token's heads and be multiples of 8 elements (16 bytes)");
    if (B == 0) return DPK_OK;
    size_t need = dpk_attn_decode_workspace_bytes(B, Tk, Hq, Hk, D, NG);
    DPK_REQUIRE(workspace && workspace_bytes >= need, "workspace of %zu bytes needed, %zu given", need,
                workspace_bytes);
    DPK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15u) == 0, "workspace must be 16-byte aligned");

    DecodeParams p;
    p.Q = static_cast<const uint8_t*>(Q);
    p.K = static_cast<const uint8_t*>(K);
    p.V = static_cast<const uint8_t*>(V);
    p.mask = mask;
    p.leftpad = leftpad;
    p.B = B; p.Tk = Tk; p.Hq = Hq; p.Hk = Hk; p.NG = NG;
    p.kv_ts = kv_ts; p.kv_bs = kv_bs;
    p.splits = decode_splits(B, Tk, Hk);
    int len = (Tk + p.splits - 1) / p.splits;
    p.split_len = ((len + 127) / 128) * 128;
    if (p.split_len < 128) p.split_len = 128;
    p.pO = static_cast<float*>(workspace);
    p.pML = p.pO + size_t(B) * Hq * p.splits * D;
    p.scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (D == 64)
        return dtype == DPK_BF16 ? launch_decode<64, true>(p, mask, O, s)
                                 : launch_decode<64, false>(p, mask, O, s);
    return dtype == DPK_BF16 ? launch_decode<128, true>(p, mask, O, s)
                             : launch_decode<128, false>(p, mask, O, s);
}

}  // extern "C"
