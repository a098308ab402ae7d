// Head-group-routed prefill attention, two query heads per CTA (sm_100a, tcgen05).
//
// Why two heads: with one head per CTA every (head, 128-row tile) streams the K/V tiles of its
// KV head through shared memory by itself.  At 4*D flops per (row, key) and 128 rows per tile
// that is 128 flops per byte brought in from L2; the tensor pipe would need 17 TB/s of L2
// bandwidth to stay busy, and a version of the one-head kernel with every MMA and all softmax
// arithmetic removed -- only the K/V tile traffic and the barrier hand-offs left -- still ran
// for 0.21 of the full kernel's 0.32-0.35 ms at 8192 tokens.  The query heads that share a KV
// head also share the routing group here (a group is whole KV heads' worth of query heads),
// hence the same active-token list and the same causal bounds: two of them take the same K/V
// tiles from ONE ring, which halves the L2 traffic per flop.
//
// CTA = 128 consecutive entries of one (batch, head group) list of active query tokens, for
// the query heads h and h+1 (h even).  Per head the pipeline is the one-head kernel's:
//     S = Q K^T          UMMA 128x64xD, operands in shared memory, accumulator in TMEM
//                        (two score buffers per head)
//     P = softmax part   4 warps per head, one query row per thread, exp2, running maximum and
//                        sum in registers, P written back to TMEM over the S tile
//     O += P V           UMMA 128xDx64, A = P from TMEM, B = V in its natural layout
// Warp roles (384 threads): warps 0-3 softmax + epilogue of head h, 4-7 of head h+1, warp 8
// TMA producer of the shared K/V ring (4 stages each), warps 9 and 10 the UMMA issuers of the
// two heads (two independent instruction streams into one tensor pipe: while one head's
// softmax runs, the other head's MMAs fill the pipe), warp 11 owns the 512 TMEM columns.
// A K or V stage is released when BOTH issuers have committed the MMAs that read it (its
// "empty" barrier counts two arrivals).  One CTA per SM: 192 KiB of shared memory.
// All waits are bounded.
//
// Algorithmic work per launch: 4*D flops per (active query row, visible key) pair and head.
#define DPK_KERNEL_ID 12   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"
#include "dpk_attn_tc.cuh"

namespace dpk {

constexpr int kT2BM = 128;          // query rows per CTA (per head)
constexpr int kT2BN = 64;           // keys per tile
constexpr int kT2SBuf = 2;          // score buffers per head in TMEM
constexpr int kT2St = 4;            // K stages and V stages in shared memory
constexpr int kT2Threads = 384;
constexpr float kT2Rescale = 8.0f;  // log2 units: O is rescaled only when a row maximum grew by more
constexpr int kT2TmemCols = 512;    // per head: 2 x 64 (S) + up to 128 (O)

struct PrefillTc2Params {
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
struct Tc2Smem {
    static constexpr int kQBytes = kT2BM * D * 2;      // one head's query tile
    static constexpr int kKBytes = kT2BN * D * 2;      // one K stage
    static constexpr int kVBytes = kT2BN * D * 2;      // one V stage
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + 2 * kQBytes;
    static constexpr int kOffV = kOffK + kT2St * kKBytes;
    static constexpr int kOffBar = kOffV + kT2St * kVBytes;
    static constexpr int kNumBars = 2 + 4 * kT2St + 2 * 3 * kT2SBuf;
    static constexpr int kTotal = kOffBar + kNumBars * 8 + 16;   // base must be 1024-byte aligned
};

template <int D, bool kBf16>
__global__ void __launch_bounds__(kT2Threads, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const PrefillTc2Params p)
{
    using L = Tc2Smem<D>;
    constexpr int KBQ = D / 64;            // 64-column K-major blocks of Q and K
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem + L::kOffK;
    uint8_t* sV = smem + L::kOffV;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* q_full = bars;                         // [2 heads]
    uint64_t* k_full = q_full + 2;                   // [kT2St]
    uint64_t* k_empty = k_full + kT2St;              // [kT2St], two arrivals
    uint64_t* v_full = k_empty + kT2St;              // [kT2St]
    uint64_t* v_empty = v_full + kT2St;              // [kT2St], two arrivals
    uint64_t* s_full = v_empty + kT2St;              // [2 heads][kT2SBuf]
    uint64_t* p_full = s_full + 2 * kT2SBuf;         // [2 heads][kT2SBuf], 128 arrivals
    uint64_t* pv_done = p_full + 2 * kT2SBuf;        // [2 heads][kT2SBuf]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.x walks the head pairs, blockIdx.y the row tiles from the last (longest key range
    // under causal masking) to the first, so the heavy tiles start first
    const int h0 = 2 * blockIdx.x, b = blockIdx.z;
    const int mt = gridDim.y - 1 - blockIdx.y;
    const int hpg = p.Hq / p.NG;
    const int g = h0 / hpg;                          // hpg is even: h0 and h0+1 share the group
    const int kvh = h0 / (p.Hq / p.Hk);              // and Hq/Hk is even: they share the KV head
    const int cnt = p.counts[b * p.NG + g];
    const int m0 = mt * kT2BM;
    if (m0 >= cnt) return;                          // whole CTA: nothing allocated yet
    if ((smem_u32(smem) & 1023u) != 0u) {           // swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_BAD_SMEM_BASE);
        return;
    }
    const int nrows = min(kT2BM, cnt - m0);
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
    const int kv_begin = (lp / kT2BN) * kT2BN;
    const int ntiles = kv_end > kv_begin ? (kv_end - kv_begin + kT2BN - 1) / kT2BN : 0;

    if (warp == 8 && lane == 0) {
        mbar_init(&q_full[0], 128);
        mbar_init(&q_full[1], 128);
        for (int s = 0; s < kT2St; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 2);
            mbar_init(&v_empty[s], 2);
        }
        for (int s = 0; s < 2 * kT2SBuf; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 128);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 11) tmem_alloc(tmem_slot, kT2TmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // =================== softmax / epilogue: thread = query row of one head =============
        const int hh = warp >> 2;                    // which of the CTA's two heads
        const int h = h0 + hh;
        const int wq = warp & 3;                     // TMEM lane quarter this warp may touch
        const int row = wq * 32 + lane;
        const int tg = threadIdx.x & 127;            // thread within the head's group
        const int tok = token_of(row);
        uint8_t* sQ = smem + L::kOffQ + hh * L::kQBytes;
        const uint32_t tmem_s0 = tmem_base + hh * 256;        // S buffers: columns [0,128) of the head
        const uint32_t tmem_o = tmem_base + hh * 256 + 128;   // O: columns [128, 128 + D)
        uint64_t* my_s_full = s_full + hh * kT2SBuf;
        uint64_t* my_p_full = p_full + hh * kT2SBuf;
        uint64_t* my_pv_done = pv_done + hh * kT2SBuf;
        // gather this head's Q rows into the swizzled K-major layout (8 lanes per 128 bytes)
        {
            const int chunk = tg & 7, rsub = tg >> 3;   // 16 rows per pass
            for (int r = rsub; r < kT2BM; r += 16) {
                const int t = token_of(r);
                const uint8_t* src_row =
                    t >= 0 ? p.Q + (static_cast<int64_t>(b) * p.q_bs + static_cast<int64_t>(t) * p.q_ts +
                                    static_cast<int64_t>(h) * D) * 2
                           : p.Q;
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb) {
                    const uint32_t dst = smem_u32(sQ) + kb * (kT2BM * 128) + r * 128 +
                                         ((chunk ^ (r & 7)) << 4);
                    cp_async_16(dst, src_row + kb * 128 + chunk * 16, t >= 0 ? 16u : 0u);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async_smem();
            mbar_arrive(&q_full[hh]);
        }

        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        float m_ref = -INFINITY;    // reference maximum the stored P and O are scaled by
        float l_sum = 0.f;
        bool alive = true;
        for (int j = 0; j < ntiles; ++j) {
            const int sb = j % kT2SBuf;
            const bool got = mbar_wait(&my_s_full[sb], (j / kT2SBuf) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
            tc_fence_after_sync();
            const uint32_t ts = tmem_s0 + sb * kT2BN + lane_base;
            const int kv0 = kv_begin + j * kT2BN;
            const bool need_mask = (kv0 < lp) || (kv0 + kT2BN > p.Tk) ||
                                   (p.causal && kv0 + kT2BN - 1 > first_tok + p.causal_shift);
            int lim = p.Tk - 1;
            if (p.causal) lim = min(lim, tok + p.causal_shift);
            if (tok < 0) lim = -1;

            // the whole score row of this tile (64 values) stays in registers
            uint32_t sv[kT2BN];
            {
                uint32_t a32[32], b32[32];
                tmem_ld_32x32b_x32(ts, a32);
                tmem_ld_32x32b_x32(ts + 32, b32);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) { sv[i] = a32[i]; sv[32 + i] = b32[i]; }
            }
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < kT2BN; ++i) {
                    const int kidx = kv0 + i;
                    if (kidx < lp || kidx > lim) sv[i] = __float_as_uint(-INFINITY);
                }
            }
            // row maximum with four independent chains of three-input maxima
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < kT2BN; i += 8) {
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
                } else if ((tmax - m_ref) * p.scale_log2 > kT2Rescale) {
                    alpha = tc_exp2((m_ref - tmax) * p.scale_log2);
                    m_ref = tmax;
                    moved = true;
                }
            }
            const float ref = m_ref == -INFINITY ? 0.f : m_ref * p.scale_log2;

            // P = exp2(scale*S - ref) (masked entries are -inf -> 0), packed to half precision
            uint32_t pk[kT2BN / 2];
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float2 nref2 = make_float2(-ref, -ref);
            float rs;
            {
                float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < kT2BN; i += 4) {
                    const float2 a = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])),
                                                sc2, nref2);
                    const float2 c = __ffma2_rn(make_float2(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])),
                                                sc2, nref2);
                    const float2 pa = make_float2(tc_exp2(a.x), tc_exp2(a.y));
                    const float2 pb = make_float2(tc_exp2(c.x), tc_exp2(c.y));
                    ra = __fadd2_rn(ra, pa);
                    rb = __fadd2_rn(rb, pb);
                    pk[i >> 1] = pack_half2<kBf16>(pa.x, pa.y);
                    pk[(i >> 1) + 1] = pack_half2<kBf16>(pb.x, pb.y);
                }
                rs = (ra.x + ra.y) + (rb.x + rb.y);
            }
            l_sum = l_sum * alpha + rs;

            // O may only be rescaled once the previous P V has finished (rare: the reference
            // maximum of some row of this warp moved)
            if (j > 0 && __any_sync(0xffffffffu, moved)) {
                const bool ok2 = mbar_wait(&my_pv_done[(j - 1) % kT2SBuf], ((j - 1) / kT2SBuf) & 1,
                                           abort_flag, p.status, DPK_DEV_TIMEOUT_TMEM_EMPTY);
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
            mbar_arrive(&my_p_full[sb]);
        }

        // ---- epilogue: O / l, scattered to the token's row ---------------------------------
        if (alive && ntiles > 0) {
            const bool ok3 = mbar_wait(&my_pv_done[(ntiles - 1) % kT2SBuf], ((ntiles - 1) / kT2SBuf) & 1,
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
    } else if (warp == 8) {
        // =================== TMA producer: the K/V ring both heads read =======================
        if (lane == 0) {
            const int col_base = kvh * D;
            for (int j = 0; j < ntiles; ++j) {
                const int s = j % kT2St;
                const uint32_t ph = ((j / kT2St) & 1) ^ 1;
                const int kv0 = kv_begin + j * kT2BN;
                if (!mbar_wait(&k_empty[s], ph, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) break;
                mbar_arrive_expect_tx(&k_full[s], L::kKBytes);
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb)
                    tma_load_3d(sK + s * L::kKBytes + kb * (kT2BN * 128), &tmK, &k_full[s],
                                col_base + kb * 64, kv0, b);
                if (!mbar_wait(&v_empty[s], ph, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) break;
                mbar_arrive_expect_tx(&v_full[s], L::kVBytes);
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb)
                    tma_load_3d(sV + s * L::kVBytes + kb * (kT2BN * 128), &tmV, &v_full[s],
                                col_base + kb * 64, kv0, b);
            }
        }
    } else if (warp == 9 || warp == 10) {
        // =================== UMMA issuer of one head =======================================
        if (lane == 0 && ntiles > 0) {
            const int hh = warp - 9;
            const uint8_t* sQ = smem + L::kOffQ + hh * L::kQBytes;
            const uint32_t tmem_s0 = tmem_base + hh * 256;
            const uint32_t tmem_o = tmem_base + hh * 256 + 128;
            uint64_t* my_s_full = s_full + hh * kT2SBuf;
            uint64_t* my_p_full = p_full + hh * kT2SBuf;
            uint64_t* my_pv_done = pv_done + hh * kT2SBuf;
            const uint32_t idesc_s = umma_idesc_f16(kBf16 ? 1 : 0, kT2BM, kT2BN);
            // P V: A K-major, B (= V) MN-major -> bit 16
            const uint32_t idesc_o = umma_idesc_f16(kBf16 ? 1 : 0, kT2BM, D) | (1u << 16);
            bool ok = mbar_wait(&q_full[hh], 0, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL);
            auto issue_s = [&](int j) -> bool {
                const int sb = j % kT2SBuf, ks = j % kT2St;
                if (!mbar_wait(&k_full[ks], (j / kT2St) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL))
                    return false;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_s0 + sb * kT2BN;
#pragma unroll
                for (int kb = 0; kb < KBQ; ++kb) {
                    const uint64_t adesc = umma_desc_k_sw128(smem_u32(sQ) + kb * (kT2BM * 128));
                    const uint64_t bdesc =
                        umma_desc_k_sw128(smem_u32(sK) + ks * L::kKBytes + kb * (kT2BN * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc_s, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&my_s_full[sb]);
                umma_commit(&k_empty[ks]);        // one of the two arrivals that free the stage
                return true;
            };
            for (int j = 0; ok && j < kT2SBuf && j < ntiles; ++j) ok = issue_s(j);
            for (int j = 0; ok && j < ntiles; ++j) {
                const int sb = j % kT2SBuf, vs = j % kT2St;
                if (!mbar_wait(&my_p_full[sb], (j / kT2SBuf) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                    ok = false;
                    break;
                }
                if (!mbar_wait(&v_full[vs], (j / kT2St) & 1, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // 64 keys in steps of 16: B advances 16 key rows = 2048 bytes; the d blocks of V
                // are kT2BN*128 bytes apart
#pragma unroll
                for (int k = 0; k < kT2BN / 16; ++k) {
                    const uint64_t bdesc =
                        umma_desc_mn_sw128(smem_u32(sV) + vs * L::kVBytes + k * 2048, kT2BN * 128);
                    // 16 keys = 8 packed columns of the tile's S/P buffer
                    umma_f16_ts(tmem_o, tmem_s0 + sb * kT2BN + k * 8, bdesc, idesc_o,
                                (j | k) != 0 ? 1u : 0u);
                }
                umma_commit(&my_pv_done[sb]);
                umma_commit(&v_empty[vs]);
                if (j + kT2SBuf < ntiles) ok = issue_s(j + kT2SBuf);
            }
        }
    }

    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 11) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kT2TmemCols);
    }
}

template <int D, bool kBf16>
static int launch_prefill_tc2(const CUtensorMap& tmK, const CUtensorMap& tmV, const PrefillTc2Params& p,
                              cudaStream_t s)
{
    constexpr size_t smem = Tc2Smem<D>::kTotal;
    dim3 grid(p.Hq / 2, (p.Tq + kT2BM - 1) / kT2BM, p.B);
    DPK_CUDA(cudaFuncSetAttribute(attn_prefill_tc2_kernel<D, kBf16>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_prefill_tc2_kernel<D, kBf16><<<grid, kT2Threads, smem, s>>>(tmK, tmV, p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

// True when query heads h and h+1 (h even) always share the routing group and the KV head.

bool attn_prefill_tc2_takes(int Hq, int Hk, int NG)
{
    return Hq % 2 == 0 && (Hq / NG) % 2 == 0 && (Hq / Hk) % 2 == 0;
}

// Entry used by dpk_attn_prefill (dpk_attn_prefill.cu) for shapes attn_prefill_tc2_takes().
int attn_prefill_tc2(const void* Q, const void* K, const void* V, const int64_t* sorted_indices,
                     const int32_t* counts, const uint32_t* leftpad, void* O, int B, int Tq, int Tk,
                     int Hq, int Hk, int D, int NG, float scale, int causal, int causal_shift,
                     int dtype, int64_t q_ts, int64_t q_bs, int64_t kv_ts, int64_t kv_bs, cudaStream_t s)
{
    CUtensorMap tmK, tmV;
    const uint64_t cols = static_cast<uint64_t>(Hk) * D;
    int rc = make_tmap_3d_sw128(&tmK, K, cols, Tk, B, kv_ts, kv_bs, 64, kT2BN);
    if (rc) return rc;
    rc = make_tmap_3d_sw128(&tmV, V, cols, Tk, B, kv_ts, kv_bs, 64, kT2BN);
    if (rc) return rc;
    PrefillTc2Params p;
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
        return dtype == DPK_BF16 ? launch_prefill_tc2<64, true>(tmK, tmV, p, s)
                                 : launch_prefill_tc2<64, false>(tmK, tmV, p, s);
    return dtype == DPK_BF16 ? launch_prefill_tc2<128, true>(tmK, tmV, p, s)
                             : launch_prefill_tc2<128, false>(tmK, tmV, p, s);
}

}  // namespace dpk
