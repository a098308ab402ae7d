// Rotary position embedding of q and k fused with the append of k and v to a
// preallocated sequence-first KV cache (sm_100a; elementwise, HBM-bound).
//
// Reference: apply_rotary_pos_emb (WIDE/wrapper/base_layer.py:18-44: q*cos + rotate_half(q)*sin
// with rotate_half(x) = cat(-x[D/2:], x[:D/2])) followed by past_key_values.update
// (WIDE/wrapper/attn_group_ffn_block.py:62-67), whose cache layer keeps [B,T,Hk,D] tensors
// and grows them with torch.cat (WIDE/wrapper/cache.py:24-46).  Here the cache is allocated
// once for `capacity` tokens and the new rows are written in place at `past_len`; the
// rotated keys never make a round trip through a separate tensor.
//
// A thread owns 8 channels i..i+7 of the lower half of a head and the matching 8 of the upper
// half, so each value is loaded once; arithmetic in fp32, one rounding.
#define DPK_KERNEL_ID 10
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

struct RopeParams {
    uint8_t* q;              // [B,T,Hq,D], rotated in place
    uint8_t* k;              // [B,T,Hk,D]; rotated in place when there is no cache
    const uint8_t* v;        // [B,T,Hk,D]
    const uint8_t* cos;      // [T,D] or [B,T,D]
    const uint8_t* sin;
    uint8_t* k_cache;        // [B,capacity,Hk,D] or NULL
    uint8_t* v_cache;
    int64_t cs_batch_stride; // elements between batches of cos/sin (0: shared)
    int64_t capacity, past_len;
    int64_t q_ts, kv_ts;     // elements between consecutive tokens of q / of k and v
    int B, T, Hq, Hk, D;
};

template <bool kBf16>
__device__ __forceinline__ void rotate8(const uint4& lo, const uint4& hi, const uint4& c_lo,
                                        const uint4& c_hi, const uint4& s_lo, const uint4& s_hi,
                                        uint4& out_lo, uint4& out_hi)
{
    const uint32_t l[4] = {lo.x, lo.y, lo.z, lo.w}, h[4] = {hi.x, hi.y, hi.z, hi.w};
    const uint32_t cl[4] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w}, ch[4] = {c_hi.x, c_hi.y, c_hi.z, c_hi.w};
    const uint32_t sl[4] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w}, sh[4] = {s_hi.x, s_hi.y, s_hi.z, s_hi.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float l0, l1, h0, h1, cl0, cl1, ch0, ch1, sl0, sl1, sh0, sh1;
        unpack_half2<kBf16>(l[j], l0, l1);
        unpack_half2<kBf16>(h[j], h0, h1);
        unpack_half2<kBf16>(cl[j], cl0, cl1);
        unpack_half2<kBf16>(ch[j], ch0, ch1);
        unpack_half2<kBf16>(sl[j], sl0, sl1);
        unpack_half2<kBf16>(sh[j], sh0, sh1);
        // lower half: x*cos - x_upper*sin ; upper half: x*cos + x_lower*sin
        ol[j] = pack_half2<kBf16>(fmaf(l0, cl0, -h0 * sl0), fmaf(l1, cl1, -h1 * sl1));
        oh[j] = pack_half2<kBf16>(fmaf(h0, ch0, l0 * sh0), fmaf(h1, ch1, l1 * sh1));
    }
    out_lo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    out_hi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
}

template <bool kBf16>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeParams p)
{
    const int half_chunks = p.D / 16;                  // 16-byte chunks in half a head
    const int heads = p.Hq + 2 * p.Hk;                 // q heads, k heads, v heads of one token
    const int64_t per_token = int64_t(heads) * half_chunks;
    const int64_t total = int64_t(p.B) * p.T * per_token;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t tok = i / per_token;
        const int rem = static_cast<int>(i - tok * per_token);
        const int head = rem / half_chunks, c = rem - head * half_chunks;
        const int b = static_cast<int>(tok / p.T), t = static_cast<int>(tok - int64_t(b) * p.T);
        const int64_t lo_off = c * 16, hi_off = (p.D / 2) * 2 + c * 16;       // bytes inside a head
        if (head >= p.Hq + p.Hk) {
            // value head: plain copy into the cache
            if (!p.v_cache) continue;
            const int hv = head - p.Hq - p.Hk;
            const uint8_t* src = p.v + (tok * p.kv_ts + int64_t(hv) * p.D) * 2;
            uint8_t* dst = p.v_cache + (((int64_t(b) * p.capacity + p.past_len + t) * p.Hk + hv) * p.D) * 2;
            *reinterpret_cast<uint4*>(dst + lo_off) = *reinterpret_cast<const uint4*>(src + lo_off);
            *reinterpret_cast<uint4*>(dst + hi_off) = *reinterpret_cast<const uint4*>(src + hi_off);
            continue;
        }
        const uint8_t* cs = p.cos + (int64_t(b) * p.cs_batch_stride + int64_t(t) * p.D) * 2;
        const uint8_t* sn = p.sin + (int64_t(b) * p.cs_batch_stride + int64_t(t) * p.D) * 2;
        const uint4 c_lo = __ldg(reinterpret_cast<const uint4*>(cs + lo_off));
        const uint4 c_hi = __ldg(reinterpret_cast<const uint4*>(cs + hi_off));
        const uint4 s_lo = __ldg(reinterpret_cast<const uint4*>(sn + lo_off));
        const uint4 s_hi = __ldg(reinterpret_cast<const uint4*>(sn + hi_off));
        uint8_t *src, *dst;
        if (head < p.Hq) {
            src = dst = p.q + (tok * p.q_ts + int64_t(head) * p.D) * 2;
        } else {
            const int hk = head - p.Hq;
            src = p.k + (tok * p.kv_ts + int64_t(hk) * p.D) * 2;
            dst = p.k_cache ? p.k_cache + (((int64_t(b) * p.capacity + p.past_len + t) * p.Hk + hk) * p.D) * 2
                            : src;
        }
        const uint4 lo = *reinterpret_cast<const uint4*>(src + lo_off);
        const uint4 hi = *reinterpret_cast<const uint4*>(src + hi_off);
        uint4 out_lo, out_hi;
        rotate8<kBf16>(lo, hi, c_lo, c_hi, s_lo, s_hi, out_lo, out_hi);
        *reinterpret_cast<uint4*>(dst + lo_off) = out_lo;
        *reinterpret_cast<uint4*>(dst + hi_off) = out_hi;
    }
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_rope_append(void* q, void* k, const void* v, const void* cos, const void* sin,
                               int64_t cs_batch_stride, void* k_cache, void* v_cache, int B, int T,
                               int Hq, int Hk, int D, int64_t capacity, int64_t past_len, int dtype,
                               int64_t q_token_stride, int64_t kv_token_stride, void* stream)
{
    DPK_REQUIRE(q && k && cos && sin, "NULL tensor");
    DPK_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "k_cache and v_cache go together");
    DPK_REQUIRE(!k_cache || v, "v is needed to fill the cache");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(B >= 0 && T >= 0 && Hq > 0 && Hk > 0, "bad shape");
    DPK_REQUIRE(D > 0 && D % 16 == 0, "head_dim=%d must be a multiple of 16", D);
    DPK_REQUIRE(cs_batch_stride == 0 || cs_batch_stride >= int64_t(T) * D, "bad cos/sin batch stride");
    DPK_REQUIRE(cs_batch_stride % 8 == 0, "cos/sin batch stride must be a multiple of 8");
    if (k_cache)
        DPK_REQUIRE(past_len >= 0 && past_len + T <= capacity,
                    "cache of %lld tokens cannot take %d more after %lld", (long long)capacity, T,
                    (long long)past_len);
    DPK_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(cos) && aligned16(sin) &&
                    aligned16(k_cache) && aligned16(v_cache), "tensors must be 16-byte aligned");
    const int64_t q_ts = q_token_stride ? q_token_stride : int64_t(Hq) * D;
    const int64_t kv_ts = kv_token_stride ? kv_token_stride : int64_t(Hk) * D;
    DPK_REQUIRE(q_ts >= int64_t(Hq) * D && kv_ts >= int64_t(Hk) * D && q_ts % 8 == 0 && kv_ts % 8 == 0,
                "token strides must cover a token's heads and be multiples of 8 elements");
    if (B == 0 || T == 0) return DPK_OK;
    RopeParams p;
    p.q = static_cast<uint8_t*>(q);
    p.k = static_cast<uint8_t*>(k);
    p.v = static_cast<const uint8_t*>(v);
    p.cos = static_cast<const uint8_t*>(cos);
    p.sin = static_cast<const uint8_t*>(sin);
    p.k_cache = static_cast<uint8_t*>(k_cache);
    p.v_cache = static_cast<uint8_t*>(v_cache);
    p.cs_batch_stride = cs_batch_stride;
    p.capacity = capacity;
    p.past_len = past_len;
    p.q_ts = q_ts;
    p.kv_ts = kv_ts;
    p.B = B;
    p.T = T;
    p.Hq = Hq;
    p.Hk = Hk;
    p.D = D;
    const int64_t total = int64_t(B) * T * (Hq + 2 * Hk) * (D / 16);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = int64_t(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DPK_BF16)
        rope_append_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, s>>>(p);
    else
        rope_append_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, s>>>(p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
