// C-ABI entry of head-group-routed prefill attention: argument checks, then one of the two
// tcgen05 kernels -- one query head per CTA, two CTAs per SM (dpk_attn_prefill_tc.cu, the
// default: 0.35 ms against 0.37 ms at 8192 tokens, 32 query / 8 KV heads), or, on request
// (dpk_set_attn_prefill_heads(2)) and where consecutive head pairs share their routing group and
// KV head, two query heads per CTA sharing one K/V stream (dpk_attn_prefill_tc2.cu).
#include "dpk_host.h"

namespace dpk {

int attn_prefill_tc(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                    const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq, int Tk,
                    int Hq, int Hk, int D, int NG, float scale, int causal, int causal_shift,
                    int dtype, int64_t q_ts, int64_t q_bs, int64_t kv_ts, int64_t kv_bs, cudaStream_t s);

bool attn_prefill_tc2_takes(int Hq, int Hk, int NG);
int attn_prefill_tc2(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                     const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq, int Tk,
                     int Hq, int Hk, int D, int NG, float scale, int causal, int causal_shift,
                     int dtype, int64_t q_ts, int64_t q_bs, int64_t kv_ts, int64_t kv_bs, cudaStream_t s);

static int g_prefill_heads = 0;      // 0 or 1: one head per CTA (the faster one as measured), 2: two where the shapes allow

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_set_attn_prefill_heads(int heads)
{
    DPK_REQUIRE(heads == 0 || heads == 1 || heads == 2, "heads per CTA must be 0 (automatic), 1 or 2");
    g_prefill_heads = heads;
    return DPK_OK;
}

extern "C" int dpk_attn_prefill(const void* Q, const void* K, const void* V,
                                const int64_t* sorted_indices, const int32_t* counts,
                                const uint32_t* leftpad, void* O, int B, int Tq, int Tk, int Hq,
                                int Hk, int D, int NG, float scale, int causal, int causal_shift,
                                int dtype, int64_t q_token_stride, int64_t q_batch_stride,
                                int64_t kv_token_stride, int64_t kv_batch_stride, void* stream)
{
    DPK_REQUIRE(Q && K && V && O && sorted_indices && counts, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(B >= 0 && Tq >= 0 && Tk >= 0 && Hq > 0 && Hk > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(D == 64 || D == 128, "head_dim %d not supported (64 or 128)", D);
    DPK_REQUIRE(Hq % Hk == 0, "Hq=%d must be a multiple of Hk=%d", Hq, Hk);
    DPK_REQUIRE(Hq % NG == 0, "Hq=%d must be a multiple of NG=%d", Hq, NG);
    DPK_REQUIRE(B <= 65535 && (Tq + 127) / 128 <= 65535, "grid too large");
    // 0 = packed: heads of a token back to back, tokens back to back, batch entries back to back
    const int64_t q_ts = q_token_stride ? q_token_stride : static_cast<int64_t>(Hq) * D;
    const int64_t q_bs = q_batch_stride ? q_batch_stride : static_cast<int64_t>(Tq) * q_ts;
    const int64_t kv_ts = kv_token_stride ? kv_token_stride : static_cast<int64_t>(Hk) * D;
    const int64_t kv_bs = kv_batch_stride ? kv_batch_stride : static_cast<int64_t>(Tk) * kv_ts;
    DPK_REQUIRE(q_ts >= static_cast<int64_t>(Hq) * D && kv_ts >= static_cast<int64_t>(Hk) * D,
                "token strides must cover the heads of a token");
    DPK_REQUIRE(q_ts % 8 == 0 && q_bs % 8 == 0 && kv_ts % 8 == 0 && kv_bs % 8 == 0,
                "strides must be multiples of 8 elements (16 bytes)");
    DPK_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O),
                "tensors must be 16-byte aligned");
    if (B == 0 || Tq == 0) return DPK_OK;
    if (Tk == 0) return DPK_OK;   // no key is visible: rows stay as the caller zero-filled them
    if (g_prefill_heads == 2 && attn_prefill_tc2_takes(Hq, Hk, NG))
        return attn_prefill_tc2(Q, K, V, sorted_indices, counts, leftpad, O, B, Tq, Tk, Hq, Hk, D, NG,
                                scale, causal, causal_shift, dtype, q_ts, q_bs, kv_ts, kv_bs,
                                static_cast<cudaStream_t>(stream));
    return attn_prefill_tc(Q, K, V, sorted_indices, counts, leftpad, O, B, Tq, Tk, Hq, Hk, D, NG, scale,
                           causal, causal_shift, dtype, q_ts, q_bs, kv_ts, kv_bs,
                           static_cast<cudaStream_t>(stream));
}
