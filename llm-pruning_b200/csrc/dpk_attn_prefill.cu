// C-ABI entry of head-group-routed prefill attention: argument checks, then the
// tcgen05 kernel of dpk_attn_prefill_tc.cu.
#include "dpk_host.h"

namespace dpk {

int attn_prefill_tc(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                    const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq, int Tk,
                    int Hq, int Hk, int D, int NG, float scale, int causal, int causal_shift,
                    int dtype, cudaStream_t s);

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
    DPK_REQUIRE(B <= 65535 && (Tq + 127) / 128 <= 65535, "grid too large");
    DPK_REQUIRE(static_cast<int64_t>(B) * Tk < (1ll << 31), "B*Tk too large for the K/V tensor map");
    DPK_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O),
                "tensors must be 16-byte aligned");
    if (B == 0 || Tq == 0) return DPK_OK;
    if (Tk == 0) return DPK_OK;   // no key is visible: rows stay as the caller zero-filled them
    return attn_prefill_tc(Q, K, V, sorted_indices, counts, leftpad, O, B, Tq, Tk, Hq, Hk, D, NG, scale,
                           causal, causal_shift, dtype, static_cast<cudaStream_t>(stream));
}
