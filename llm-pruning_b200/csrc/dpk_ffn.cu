// Dynamic-width SwiGLU FFN as one C-ABI call: routing layout, packed routing bits,
// fused gate/up projection (SwiGLU in the epilogue) and the reduction-width down
// projection, all enqueued on the caller's stream from one caller-owned workspace.
#include "dpk_host.h"

namespace {

struct FfnLayout {
    size_t sorted_mask, sorted_idx, counts, route_ws, row_bits, win_bits, h, acc, total;
};

size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

FfnLayout ffn_layout(int64_t M, int H, int I, int NG)
{
    FfnLayout L;
    const size_t words = (NG + 31) / 32;
    const size_t nwin = (M + 127) / 128;
    size_t off = 0;
    L.sorted_mask = off; off += up256(size_t(M) * NG);
    L.sorted_idx = off;  off += up256(size_t(M) * NG * sizeof(int64_t));
    L.counts = off;      off += up256(size_t(NG) * sizeof(int32_t));
    L.route_ws = off;    off += up256(dpk_route_workspace_bytes(1, M, NG));
    L.row_bits = off;    off += up256(size_t(M) * words * sizeof(uint32_t));
    L.win_bits = off;    off += up256(nwin * words * sizeof(uint32_t));
    L.h = off;           off += up256(size_t(M) * I * 2);
    L.acc = off;         off += up256(dpk_gemm_k_workspace_bytes(M, H));
    L.total = off;
    return L;
}

}  // namespace

extern "C" {

size_t dpk_ffn_workspace_bytes(int64_t M, int H, int I, int NG)
{
    if (M < 0 || I < 1 || NG < 1) return 0;
    return ffn_layout(M, H, I, NG).total;
}

int dpk_ffn_swiglu(const void* x, const void* Wg, const void* Wu, const void* Wd,
                   const uint8_t* mask, void* y, int64_t M, int H, int I, int NG, int dtype,
                   void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(x && Wg && Wu && Wd && mask && y, "NULL tensor");
    DPK_REQUIRE(M >= 0 && H > 0 && I > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(I % NG == 0, "I=%d is not divisible by NG=%d", I, NG);
    if (M == 0) return DPK_OK;
    const FfnLayout L = ffn_layout(M, H, I, NG);
    DPK_REQUIRE(workspace && workspace_bytes >= L.total, "workspace of %zu bytes needed, %zu given",
                L.total, workspace_bytes);
    DPK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
                "workspace must be 256-byte aligned");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint8_t* smask = ws + L.sorted_mask;
    int64_t* sidx = reinterpret_cast<int64_t*>(ws + L.sorted_idx);
    int32_t* counts = reinterpret_cast<int32_t*>(ws + L.counts);
    uint32_t* row_bits = reinterpret_cast<uint32_t*>(ws + L.row_bits);
    uint32_t* win_bits = reinterpret_cast<uint32_t*>(ws + L.win_bits);
    void* h = ws + L.h;

    int rc = dpk_route_plan(mask, M, NG, smask, sidx, counts, row_bits, win_bits, ws + L.route_ws,
                            up256(dpk_route_workspace_bytes(1, M, NG)), stream);
    if (rc) return rc;
    // h[t, g-block] = silu(x Wg^T) * (x Wu^T) for active (t, g); other blocks are left as
    // they are and never read: the down projection zeroes them on the fly.
    rc = dpk_gemm_mn(x, H, Wg, Wu, H, sidx, counts, h, I, M, I, H, NG, dtype, DPK_ACT_IDENTITY,
                     stream);
    if (rc) return rc;
    return dpk_gemm_k(h, I, Wd, I, row_bits, win_bits, y, H, M, H, I, NG, dtype, nullptr, 0, ws + L.acc,
                      up256(dpk_gemm_k_workspace_bytes(M, H)), stream);
}

}  // extern "C"
