// Head-group-routed prefill attention on tcgen05 tensor cores (sm_100a).
//
// A CTA owns 128 consecutive entries of one (batch, head group) list of active query
// tokens for one query head.  Per 64-key tile:
//     S = Q K^T          UMMA 128x64xD, both operands K-major in shared memory,
//                        accumulator in TMEM (double buffered)
//     P = softmax part   4 warps, one query row per thread: TMEM -> registers, running
//                        row maximum / sum in registers (no shuffles: a row lives in one
//                        thread), exp2, bf16, written back to TMEM over the S tile
//     O += P V           UMMA 128xDx64, A = P read from TMEM, B = V in its natural [key][d]
//                        layout (MN-major descriptor), accumulator in TMEM
// O is rescaled lazily: the reference maximum of a row only moves when the true maximum
// has grown by more than 2^8, so most tiles skip the TMEM read-modify-write.  K and V
// tiles arrive by TMA (128-byte swizzle) through two-stage rings; Q rows are gathered
// with cp.async.  Causal masking bounds the key range by the tile's last token and is
// applied element-wise only on tiles that cross a boundary.
//
// Warp roles (192 threads): warps 0-3 softmax + epilogue, warp 4 TMA producer, warp 5
// UMMA issuer and TMEM owner.  A CTA needs 96 KiB of shared memory and 256 TMEM columns,
// so two CTAs share an SM: while one waits for a tile or runs its softmax, the other
// keeps the tensor pipe and the exponential unit busy.  All waits are bounded.
//
// Algorithmic work per launch: 4*D flops per (active query row, visible key) pair.
#define DPK_KERNEL_ID 5   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"
#include "dpk_attn_tc.cuh"

namespace dpk {

constexpr int kTcBM = 128;        // query rows per CTA
#ifndef DPK_ATTN_BN
#define DPK_ATTN_BN 64
#endif
constexpr int kTcBN = DPK_ATTN_BN;          // keys per tile
constexpr int kTcSBuf = 128 / kTcBN;        // score buffers in TMEM and V stages in shared memory
#ifndef DPK_ATTN_KSTAGES
#define DPK_ATTN_KSTAGES kTcSBuf
#endif
constexpr int kTcKSt = DPK_ATTN_KSTAGES;    // K stages in shared memory (at most 4)
static_assert(kTcKSt >= 2 && kTcKSt <= 4, "K ring depth");
static_assert(kTcBN == 64 || kTcBN == 32, "tile width");
constexpr int kTcThreads = 192;
constexpr float kRescaleThreshold = 8.0f;   // log2 units
constexpr int kTcTmemCols = 256;            // 2 x 64 (S) + up to 128 (O)

struct PrefillTcParams {
    const uint8_t* Q;
    uint8_t* O;
    const int64_t* sidx;     // [B, Tq, NG]
    const int32_t* counts;   // [B, NG]
    const uint32_t* leftpad; // [B] or null
    int B, Tq, Tk, Hq, Hk, NG;
    int64_t q_ts, q_bs;      // elements between consecutive tokens / batch entries of Q
    float scale_log2;
    int causal, causal_shift;
    int* status;
};

template <int D>
struct TcSmem {
    static constexpr int kQBytes = kTcBM * D * 2;
    static constexpr int kKBytes = kTcBN * D * 2;      // one K stage
    static constexpr int kVBytes = kTcBN * D * 2;      // one V stage
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + kQBytes;
    static constexpr int kOffV = kOffK + kTcKSt * kKBytes;
    static constexpr int kOffBar = kOffV + kTcSBuf * kVBytes;
    static constexpr int kTotal = kOffBar + 30 * 8 + 16;   // base must be 1024-byte aligned
};

template <int D, bool kBf16>
__global__ void __launch_bounds__(kTcThreads, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const PrefillTcParams p)
{
    using L = TcSmem<D>;
    constexpr int KBQ = D / 64;            // 64-column K-major blocks of Q and K
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem + L::kOffQ;
    uint8_t* sK = smem + L::kOffK;
    uint8_t* sV = smem + L::kOffV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;      // [kTcSBuf]
    uint64_t* v_full = bars + 5;      // [kTcSBuf]
    uint64_t* k_empty = bars + 9;     // [kTcSBuf]
    uint64_t* v_empty = bars + 13;    // [kTcSBuf]
    uint64_t* s_full = bars + 17;     // [kTcSBuf]
    // one barrier per score buffer, not one per kernel: a warp role that runs ahead (the softmax
    // warps have up to kTcSBuf score tiles waiting for them) can then never complete two phases of
    // a barrier before the other side has looked at the first -- which a parity wait cannot tell
    // from "not completed yet"
    uint64_t* p_full = bars + 21;     // [kTcSBuf]
    uint64_t* pv_done = bars + 25;    // [kTcSBuf]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.x (fastest to be scheduled) walks the heads, blockIdx.y the row tiles from the
    // last (longest key range under causal masking) to the first: every head's heavy tiles
    // start first and the light ones fill the tail of the launch
    const int h = blockIdx.x, b = blockIdx.z;
    const int mt = gridDim.y - 1 - blockIdx.y;
    const int hpg = p.Hq / p.NG;
    const int g = h / hpg;
    const int kvh = h / (p.Hq / p.Hk);
    const int cnt = p.counts[b * p.NG + g];
    const int m0 = mt * kTcBM;
    if (m0 >= cnt) return;                          // whole CTA: nothing allocated yet
    if ((smem_u32(smem) & 1023u) != 0u) {           // swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_BAD_SMEM_BASE);
        return;
    }
    const int nrows = min(kTcBM, cnt - m0);
    const int64_t* sidx_b = p.sidx + static_cast<int64_t>(b) * p.Tq * p.NG;

    auto token_of = [&](int row) -> int {
        if (row >= nrows) return -1;
        int64_t t = sidx_b[static_cast<int64_t>(m0 + row) * p.NG + g];
        if (t < 0 || t >= p.Tq) {
            atomicCAS(p.status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_BAD_INDEX);
            return -1;
        }
        return static_cast<int>(t);
    };
    const int first_tok = token_of(0);
    const int last_tok = token_of(nrows - 1);
    const int lp = p.leftpad ? static_cast<int>(p.leftpad[b]) : 0;
    int kv_end = p.Tk;
    if (p.causal) kv_end = min(p.Tk, last_tok + p.causal_shift + 1);
    const int kv_begin = (lp / kTcBN) * kTcBN;
    const int ntiles = kv_end > kv_begin ? (kv_end - kv_begin + kTcBN - 1) / kTcBN : 0;

    if (warp == 4 && lane == 0) {
        mbar_init(q_full, 128);
        for (int s = 0; s < kTcKSt; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < kTcSBuf; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 128);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTcTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s0 = tmem_base;            // S buffers: kTcSBuf x kTcBN columns in [0,128)
    const uint32_t tmem_o = tmem_base + 128;       // O: columns [128, 128 + D)

    if (warp < 4) {
        // =================== softmax / epilogue: thread = query row =====================
        const int row = warp * 32 + lane;
        const int tok = token_of(row);
        // gather this CTA's Q rows into the swizzled K-major layout (8 lanes per 128 bytes)
        {
            const int chunk = threadIdx.x & 7, rsub = threadIdx.x >> 3;   // 16 rows per pass
            for (int r = rsub; r < kTcBM; r += 16) {
                const int t = token_of(r);
                const uint8_t* src_row =
                    t >= 0 ? p.Q + (static_cast<int64_t>(b) * p.q_bs + static_cast<int64_t>(t) * p.q_ts +
                                    static_cast<int64_t>(h) * D) * 2
                           : p.Q;
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb) {
                    const uint32_t dst = smem_u32(sQ) + kb * (kTcBM * 128) + r * 128 +
                                         ((chunk ^ (r & 7)) << 4);
                    cp_async_16(dst, src_row + kb * 128 + chunk * 16, t >= 0 ? 16u : 0u);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async_smem();
            mbar_arrive(q_full);
        }

        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        float m_ref = -INFINITY;    // reference maximum the stored P and O are scaled by
        float l_sum = 0.f;
        bool alive = true;
        for (int j = 0; j < ntiles; ++j) {
            const int sb = j % kTcSBuf;
            const bool got = mbar_wait(&s_full[sb], (j / kTcSBuf) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
            tc_fence_after_sync();
            const uint32_t ts = tmem_s0 + sb * kTcBN + lane_base;
            const int kv0 = kv_begin + j * kTcBN;
            const bool need_mask = (kv0 < lp) || (kv0 + kTcBN > p.Tk) ||
                                   (p.causal && kv0 + kTcBN - 1 > first_tok + p.causal_shift);
            int lim = p.Tk - 1;
            if (p.causal) lim = min(lim, tok + p.causal_shift);
            if (tok < 0) lim = -1;

            // the whole score row of this tile (64 values) stays in registers
            uint32_t sv[kTcBN];
            if constexpr (kTcBN == 64) {
                uint32_t a32[32], b32[32];
                tmem_ld_32x32b_x32(ts, a32);
                tmem_ld_32x32b_x32(ts + 32, b32);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) { sv[i] = a32[i]; sv[(32 + i) % kTcBN] = b32[i]; }
            } else {
                uint32_t a32[32];
                tmem_ld_32x32b_x32(ts, a32);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sv[i] = a32[i];
            }
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < kTcBN; ++i) {
                    const int kidx = kv0 + i;
                    if (kidx < lp || kidx > lim) sv[i] = __float_as_uint(-INFINITY);
                }
            }
            // row maximum with four independent chains of three-input maxima
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < kTcBN; i += 8) {
                t0 = tc_max3(t0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                t1 = tc_max3(t1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
                t2 = tc_max3(t2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
                t3 = tc_max3(t3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
            }
            const float tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
            // lazy reference update: move only when the maximum grew by more than 2^8
            float alpha = 1.f;
            bool moved = false;
            if (tmax > -INFINITY) {
                if (m_ref == -INFINITY) {
                    m_ref = tmax;                           // nothing accumulated yet for this row
                } else if ((tmax - m_ref) * p.scale_log2 > kRescaleThreshold) {
                    alpha = tc_exp2((m_ref - tmax) * p.scale_log2);
                    m_ref = tmax;
                    moved = true;
                }
            }
            const float ref = m_ref == -INFINITY ? 0.f : m_ref * p.scale_log2;

            // P = exp2(scale*S - ref) (masked entries are -inf -> 0), packed to half precision
            uint32_t pk[kTcBN / 2];
            // packed fp32 arithmetic (two values per instruction) for the scaling and the row sum
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float2 nref2 = make_float2(-ref, -ref);
            float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < kTcBN; i += 4) {
                const float2 a = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])),
                                            sc2, nref2);
                const float2 b = __ffma2_rn(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])),
                                            sc2, nref2);
                const float2 pa = make_float2(tc_exp2(a.x), tc_exp2(a.y));
                const float2 pb = make_float2(tc_exp2(b.x), tc_exp2(b.y));
                ra = __fadd2_rn(ra, pa);
                rb = __fadd2_rn(rb, pb);
                pk[i >> 1] = pack_half2<kBf16>(pa.x, pa.y);
                pk[(i >> 1) + 1] = pack_half2<kBf16>(pb.x, pb.y);
            }
            const float rs = (ra.x + ra.y) + (rb.x + rb.y);
            l_sum = l_sum * alpha + rs;

            // O may only be rescaled once the previous P V has finished (rare: the reference
            // maximum of some row of this warp moved)
            if (j > 0 && __any_sync(0xffffffffu, moved)) {
                const bool ok2 = mbar_wait(&pv_done[(j - 1) % kTcSBuf], ((j - 1) / kTcSBuf) & 1, abort_flag,
                                           p.status, DPK_DEV_TIMEOUT_TMEM_EMPTY);
                if (!__all_sync(0xffffffffu, ok2)) { alive = false; break; }
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_o + lane_base + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st_32x32b_x32(tmem_o + lane_base + c, v);
                }
                tmem_st_wait();
            }
            // P replaces the first 32 columns of this tile's S buffer in TMEM (two keys per
            // 32-bit column); the P V UMMA reads its A operand from there
            tmem_st_p(ts, pk);
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&p_full[sb]);
        }

        // ---- epilogue: O / l, scattered to the token's row ---------------------------------
        if (alive && ntiles > 0) {
            const bool ok3 = mbar_wait(&pv_done[(ntiles - 1) % kTcSBuf], ((ntiles - 1) / kTcSBuf) & 1,
                                       abort_flag, p.status, DPK_DEV_TIMEOUT_TMEM_EMPTY);
            alive = __all_sync(0xffffffffu, ok3);
            tc_fence_after_sync();
        }
        if (alive) {
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            uint8_t* out = p.O + ((static_cast<int64_t>(b) * p.Tq + (tok >= 0 ? tok : 0)) * p.Hq + h) *
                                     (D * 2);
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t v[32];
                if (ntiles > 0) {
                    tmem_ld_32x32b_x32(tmem_o + lane_base + c, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                if (tok >= 0) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w[i] = pack_half2<kBf16>(__uint_as_float(v[q4 * 8 + 2 * i]) * inv,
                                                     __uint_as_float(v[q4 * 8 + 2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(out + (c + q4 * 8) * 2) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    } else if (warp == 4) {
        // =================== TMA producer: K and V tiles ====================================
        if (lane == 0) {
            const int col_base = kvh * D;
            // K runs kTcKSt-1 tiles ahead of V: a K tile is needed one softmax earlier than the V
            // tile of the same keys, and its stage is released earlier too (by Q K^T, not by P V)
            bool live = true;
            auto load_k = [&](int j) {
                const int ks = j % kTcKSt;
                if (!mbar_wait(&k_empty[ks], ((j / kTcKSt) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_EMPTY)) {
                    live = false;
                    return;
                }
                mbar_arrive_expect_tx(&k_full[ks], L::kKBytes);
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb)
                    tma_load_3d(sK + ks * L::kKBytes + kb * (kTcBN * 128), &tmK, &k_full[ks],
                                col_base + kb * 64, kv_begin + j * kTcBN, b);
            };
            for (int j = 0; live && j < kTcKSt - 1 && j < ntiles; ++j) load_k(j);
            for (int j = 0; live && j < ntiles; ++j) {
                if (j + kTcKSt - 1 < ntiles) load_k(j + kTcKSt - 1);
                if (!live) break;
                const int s = j % kTcSBuf;
                if (!mbar_wait(&v_empty[s], ((j / kTcSBuf) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_EMPTY))
                    break;
                mbar_arrive_expect_tx(&v_full[s], L::kVBytes);
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb)
                    tma_load_3d(sV + s * L::kVBytes + kb * (kTcBN * 128), &tmV, &v_full[s],
                                col_base + kb * 64, kv_begin + j * kTcBN, b);
            }
        }
    } else {
        // =================== UMMA issuer ===================================================
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = umma_idesc_f16(kBf16 ? 1 : 0, kTcBM, kTcBN);
            // P V: A K-major, B (= V) MN-major -> bit 16
            const uint32_t idesc_o = umma_idesc_f16(kBf16 ? 1 : 0, kTcBM, D) | (1u << 16);
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL);
            auto issue_s = [&](int j) -> bool {
                const int s = j % kTcSBuf, ks = j % kTcKSt;
                if (!mbar_wait(&k_full[ks], (j / kTcKSt) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL))
                    return false;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_s0 + s * kTcBN;
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb) {
                    const uint64_t adesc = umma_desc_k_sw128(smem_u32(sQ) + kb * (kTcBM * 128));
                    const uint64_t bdesc =
                        umma_desc_k_sw128(smem_u32(sK) + ks * L::kKBytes + kb * (kTcBN * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_s, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&s_full[s]);
                umma_commit(&k_empty[ks]);
                return true;
            };
            for (int j = 0; ok && j < kTcSBuf && j < ntiles; ++j) ok = issue_s(j);
            for (int j = 0; ok && j < ntiles; ++j) {
                const int s = j % kTcSBuf;
                if (!mbar_wait(&p_full[s], (j / kTcSBuf) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL) ||
                    !mbar_wait(&v_full[s], (j / kTcSBuf) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // kTcBN keys in steps of 16: B advances 16 key rows = 2048 bytes; the d blocks of V
                // are kTcBN*128 bytes apart
#pragma unroll
                for (int k = 0; k < kTcBN / 16; ++k) {
                    const uint64_t bdesc =
                        umma_desc_mn_sw128(smem_u32(sV) + s * L::kVBytes + k * 2048, kTcBN * 128);
                    // 16 keys = 8 packed columns of the tile's S/P buffer
                    umma_f16_ts(tmem_o, tmem_s0 + s * kTcBN + k * 8, bdesc, idesc_o,
                                (j | k) != 0 ? 1u : 0u);
                }
                umma_commit(&pv_done[s]);
                umma_commit(&v_empty[s]);
                if (j + kTcSBuf < ntiles) ok = issue_s(j + kTcSBuf);
            }
        }
    }

    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

template <int D, bool kBf16>
static int launch_prefill_tc(const CUtensorMap& tmK, const CUtensorMap& tmV, const PrefillTcParams& p,
                             cudaStream_t s)
{
    constexpr size_t smem = TcSmem<D>::kTotal;
    dim3 grid(p.Hq, (p.Tq + kTcBM - 1) / kTcBM, p.B);
    DPK_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<D, kBf16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_prefill_tc_kernel<D, kBf16><<<grid, kTcThreads, smem, s>>>(tmK, tmV, p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

// Entry used by dpk_attn_prefill (dpk_attn_prefill.cu).
int attn_prefill_tc(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                    const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq, int Tk,
                    int Hq, int Hk, int D, int NG, float scale, int causal, int causal_shift,
                    int dtype, int64_t q_ts, int64_t q_bs, int64_t kv_ts, int64_t kv_bs, cudaStream_t s)
{
    // K and V as [batch][key][Hk*D] maps: a tile that runs past the last key of its batch entry
    // is zero-filled by the copy engine, whatever lies behind it in memory
    CUtensorMap tmK, tmV;
    const uint64_t cols = static_cast<uint64_t>(Hk) * D;
    int rc = make_tmap_3d_sw128(&tmK, K, cols, Tk, B, kv_ts, kv_bs, 64, kTcBN);
    if (rc) return rc;
    rc = make_tmap_3d_sw128(&tmV, V, cols, Tk, B, kv_ts, kv_bs, 64, kTcBN);
    if (rc) return rc;
    PrefillTcParams p;
    p.Q = static_cast<const uint8_t*>(Q);
    p.O = static_cast<uint8_t*>(O);
    p.sidx = sorted_indices;
    p.counts = counts;
    p.leftpad = leftpad;
    p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hk = Hk; p.NG = NG;
    p.q_ts = q_ts; p.q_bs = q_bs;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal ? 1 : 0;
    p.causal_shift = causal_shift;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");
    if (D == 64)
        return dtype == DPK_BF16 ? launch_prefill_tc<64, true>(tmK, tmV, p, s)
                                 : launch_prefill_tc<64, false>(tmK, tmV, p, s);
    return dtype == DPK_BF16 ? launch_prefill_tc<128, true>(tmK, tmV, p, s)
                             : launch_prefill_tc<128, false>(tmK, tmV, p, s);
}

}  // namespace dpk
