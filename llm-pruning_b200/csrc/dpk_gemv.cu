// Routed projections on CUDA cores for very small token counts (and for group widths
// the tensor-core kernels do not take).  One warp owns one output channel n and up to
// four token rows: it streams W[n,:] once with 16-byte loads and keeps one fp32
// accumulator per row, skipping work on the fly from the byte mask.  Bounded by the
// HBM read of the weight rows that at least one of the rows uses.
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kGemvRows = 4;

template <bool kBf16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8])
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (kBf16) {
            __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            float2 t = __bfloat1622float2(h);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        } else {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 t = __half22float2(h);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
}

template <bool kBf16>
__device__ __forceinline__ void store_half(uint8_t* p, float v)
{
    if constexpr (kBf16) *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(v);
    else *reinterpret_cast<__half*>(p) = __float2half_rn(v);
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
gemv_routed_kernel(const uint8_t* __restrict__ A, int64_t lda, const uint8_t* __restrict__ W,
                   int64_t ldw, const uint8_t* __restrict__ mask, uint8_t* __restrict__ D,
                   int64_t ldd, int64_t M, int N, int K, int NG, int act, int reduce_k)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kGemvRows;
    if (n >= N) return;
    const int rows = (M - m0) < kGemvRows ? static_cast<int>(M - m0) : kGemvRows;
    float acc[kGemvRows] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* wrow = W + static_cast<int64_t>(n) * ldw * 2;

    if (!reduce_k) {
        const int G = N / NG;
        const int g = n / G;
        bool on[kGemvRows];
        bool any = false;
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
            on[r] = r < rows && mask[(m0 + r) * NG + g] != 0;
            any |= on[r];
        }
        if (!any) return;   // inactive blocks stay untouched
        for (int k = lane * 8; k < K; k += 256) {
            float wf[8];
            unpack8<kBf16>(*reinterpret_cast<const uint4*>(wrow + k * 2), wf);
#pragma unroll
            for (int r = 0; r < kGemvRows; ++r) {
                if (on[r]) {
                    float af[8];
                    unpack8<kBf16>(*reinterpret_cast<const uint4*>(A + ((m0 + r) * lda + k) * 2), af);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r] = fmaf(af[i], wf[i], acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
            float v = acc[r];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0 && on[r]) {
                if (act == DPK_ACT_RELU) v = fmaxf(v, 0.f);
                else if (act == DPK_ACT_SILU) v = silu_f(v);
                store_half<kBf16>(D + ((m0 + r) * ldd + n) * 2, v);
            }
        }
    } else {
        const int G = K / NG;
        for (int k = lane * 8; k < K; k += 256) {
            // an 8-element chunk lies inside one group when G % 8 == 0; otherwise it may
            // straddle two and the mask is looked up per element
            const bool one_group = (G % 8) == 0;
            float wf[8];
            bool w_loaded = false;
#pragma unroll
            for (int r = 0; r < kGemvRows; ++r) {
                if (r >= rows) continue;
                const uint8_t* mrow = mask + (m0 + r) * NG;
                if (one_group && mrow[k / G] == 0) continue;
                if (!w_loaded) {
                    unpack8<kBf16>(*reinterpret_cast<const uint4*>(wrow + k * 2), wf);
                    w_loaded = true;
                }
                float af[8];
                unpack8<kBf16>(*reinterpret_cast<const uint4*>(A + ((m0 + r) * lda + k) * 2), af);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool use = one_group || mrow[(k + i) / G] != 0;
                    if (use) acc[r] = fmaf(af[i], wf[i], acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
            float v = acc[r];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0 && r < rows) store_half<kBf16>(D + ((m0 + r) * ldd + n) * 2, v);
        }
    }
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_gemv_routed(const void* A, int64_t lda, const void* W, int64_t ldw,
                               const uint8_t* mask, void* D, int64_t ldd, int64_t M, int N, int K,
                               int NG, int dtype, int act, int reduce_k, void* stream)
{
    DPK_REQUIRE(A && W && D && mask, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(act >= DPK_ACT_IDENTITY && act <= DPK_ACT_SILU, "unknown activation %d", act);
    DPK_REQUIRE(M >= 0 && N > 0 && K > 0 && NG > 0, "bad shape");
    DPK_REQUIRE((reduce_k ? K : N) % NG == 0, "routed width is not divisible by NG=%d", NG);
    DPK_REQUIRE(K % 8 == 0, "K=%d must be a multiple of 8", K);
    DPK_REQUIRE(lda >= K && ldw >= K && ldd >= N, "row strides shorter than rows");
    DPK_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "input row strides must be multiples of 8");
    DPK_REQUIRE(aligned16(A) && aligned16(W), "inputs must be 16-byte aligned");
    if (M == 0) return DPK_OK;
    int64_t gy = (M + kGemvRows - 1) / kGemvRows;
    DPK_REQUIRE(gy <= 65535, "M=%lld too large for the CUDA-core path", (long long)M);
    dim3 grid((N + 7) / 8, (unsigned)gy);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t* a = static_cast<const uint8_t*>(A);
    const uint8_t* w = static_cast<const uint8_t*>(W);
    uint8_t* d = static_cast<uint8_t*>(D);
    if (dtype == DPK_BF16)
        gemv_routed_kernel<true><<<grid, 256, 0, s>>>(a, lda, w, ldw, mask, d, ldd, M, N, K, NG, act,
                                                       reduce_k);
    else
        gemv_routed_kernel<false><<<grid, 256, 0, s>>>(a, lda, w, ldw, mask, d, ldd, M, N, K, NG, act,
                                                        reduce_k);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
