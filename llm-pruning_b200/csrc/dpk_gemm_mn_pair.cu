// Output-width routed projection on CTA pairs (tcgen05 cta_group::2, sm_100a).
//
// Same mathematics and tile order as dpk_gemm_mn.cu, for the wide case (UMMA N = 256).
// Two CTAs of a cluster share one tile of 256 token rows: CTA r gathers rows
// [128r, 128r+128) of the tile into its own shared memory and loads HALF of the weight
// tile (with a second weight: CTA 0 the gate rows, CTA 1 the up rows; otherwise rows
// [128r, 128r+128) of the chunk).  One thread of the even CTA issues
// tcgen05.mma.cta_group::2 with M = 256: the tensor cores of both SMs read their own A
// rows and both halves of B, and each SM's TMEM receives its 128 rows x 256 columns.
// Per SM a 64-deep K block now costs 16 KiB of A + 16 KiB of B instead of 16 + 32 KiB,
// so the operand ring is 6 stages deep and the shared-memory read rate of the tensor
// core drops from 96 to 64 bytes per clock.
//
// Barriers.  The pair's "full" barriers live in the even CTA: its own TMA and the odd
// CTA's TMA (cta_group::2 form, barrier address with the peer bit cleared) complete their
// bytes there, and the 256 gather threads of both CTAs arrive there.  "empty" and the
// accumulator-ready barriers exist in both CTAs and are signalled by multicast commits.
// The accumulator-drained barrier is in the even CTA; the odd CTA's epilogue threads
// arrive on it remotely.  Every wait is bounded; a cluster barrier precedes the exit so
// that no CTA leaves while its partner can still touch its shared memory.
#define DPK_KERNEL_ID 2   // thousands digit of the device status word
#include "dpk_gemm_mn.cuh"

namespace dpk {

constexpr int kPairStageBytes = kAStageBytes + 128 * kBK * 2;     // 32 KiB
constexpr int kPairStages = kRingBytes / kPairStageBytes;         // 6

constexpr size_t kPairSmemBytes = 1024 + size_t(kRingBytes) + (2 * kMaxStages + 4) * sizeof(uint64_t) +
                                  16 + (kMaxGroups + 1) * sizeof(int);

template <bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMnThreads, 1)
gemm_mn_pair_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                    const __grid_constant__ CUtensorMap tmA, const MnParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + size_t(kRingBytes));
    uint64_t* empty = full + kMaxStages;
    uint64_t* tfull = empty + kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_tmin = reinterpret_cast<int*>(tmem_slot + 2);
    int* prefix = reinterpret_cast<int*>(tmem_slot + 4);   // [NG + 1]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());   // 0 = even CTA: issues the UMMAs
    const int pair = blockIdx.x >> 1;
    const int npairs = gridDim.x >> 1;
    const int KB = (p.K + kBK - 1) / kBK;
    constexpr int RT = 2 * kBM;                              // token rows per pair tile

    // ---- set-up (identical in both CTAs) ---------------------------------------------
    if (warp == 0) {
        int tmin = 0x7fffffff;
        for (int g = lane; g < p.NG; g += 32) {
            int c = p.counts[g];
            c = c < 0 ? 0 : c;
            tmin = min(tmin, (c + RT - 1) / RT);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) tmin = min(tmin, __shfl_xor_sync(0xffffffffu, tmin, d));
        int run = 0;
        for (int base = 0; base < p.NG; base += 32) {
            int g = base + lane;
            int v = 0;
            if (g < p.NG) {
                int c = p.counts[g];
                c = c < 0 ? 0 : c;
                v = ((c + RT - 1) / RT - tmin) * p.n_chunks;
            }
            int incl = v;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int o = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += o;
            }
            if (g < p.NG) prefix[g + 1] = run + incl;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            prefix[0] = 0;
            *s_tmin = tmin;
        }
    }
    if (warp == 4 && lane == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            // even CTA's expect_tx arrive (+ 2 x 128 gather threads when rows come by cp.async;
            // rows that come by TMA are counted in bytes)
            mbar_init(&full[s], p.gather4 ? 1 : 1 + 256);
            mbar_init(&empty[s], 1);        // one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);        // one multicast commit
            mbar_init(&tempty[b], 256);     // epilogue threads of both CTAs
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmW2);
        if (p.gather4) tma_prefetch_desc(&tmA);
    }
    if (warp == 5) tmem_alloc_pair(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                     // partner's barriers are initialised too
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    TileMap tmap;
    tmap.ragged_prefix = prefix;
    tmap.ng = p.NG;
    tmap.n_chunks = p.n_chunks;
    tmap.rows_per_block = p.rows_per_block;
    tmap.tmin = *s_tmin;
    tmap.regular_total = tmap.tmin * p.NG * p.n_chunks;
    tmap.total = tmap.regular_total + prefix[p.NG];
    const int total_tiles = tmap.total;
    const int BN = p.BN;                    // 128 with a second weight, 256 without

    if (warp < 4) {
        // ============================ epilogue (own 128 rows) ========================
        int acc_it = 0;
        for (int tile = pair; tile < total_tiles; tile += npairs, ++acc_it) {
            int g, mtile, nchunk;
            tmap.decode(tile, g, mtile, nchunk);
            const int cnt = p.counts[g];
            const int slot = mtile * RT + rank * kBM + warp * 32 + lane;
            bool valid = slot < cnt;
            int64_t tok = 0;
            if (valid) {
                tok = p.sidx[static_cast<int64_t>(slot) * p.NG + g];
                if (tok < 0 || tok >= p.M) {
                    atomicCAS(p.status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_BAD_INDEX);
                    valid = false;
                }
            }
            const int ab = acc_it & 1;
            const bool got = mbar_wait(&tfull[ab], (acc_it >> 1) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                   static_cast<uint32_t>(ab * 256);
            uint8_t* out = p.D + (tok * p.ldd + static_cast<int64_t>(g) * p.G +
                                  static_cast<int64_t>(nchunk) * BN) * 2;
            if (p.fused) {
                for (int c = 0; c < 128; c += 32) {
                    uint32_t gate[32], up[32];
                    tmem_ld_32x32b_x32(taddr + c, gate);
                    tmem_ld_32x32b_x32(taddr + 128 + c, up);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float g0 = __uint_as_float(gate[q * 8 + 2 * j]);
                                float g1 = __uint_as_float(gate[q * 8 + 2 * j + 1]);
                                float u0 = __uint_as_float(up[q * 8 + 2 * j]);
                                float u1 = __uint_as_float(up[q * 8 + 2 * j + 1]);
                                w[j] = pack_half2<kBf16>(silu_f(g0) * u0, silu_f(g1) * u1);
                            }
                            *reinterpret_cast<uint4*>(out + (c + q * 8) * 2) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            } else {
                for (int c = 0; c < 256; c += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c, v);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float a0 = apply_act(__uint_as_float(v[q * 8 + 2 * j]), p.act);
                                float a1 = apply_act(__uint_as_float(v[q * 8 + 2 * j + 1]), p.act);
                                w[j] = pack_half2<kBf16>(a0, a1);
                            }
                            *reinterpret_cast<uint4*>(out + (c + q * 8) * 2) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive_leader(&tempty[ab]);
        }
    } else if (warp == 4) {
        // ============================ weight TMA producer (own half of B) ===========
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const CUtensorMap* map = (p.fused && rank == 1) ? &tmW2 : &tmW;
            for (int tile = pair; ok && tile < total_tiles; tile += npairs) {
                int g, mtile, nchunk;
                tmap.decode(tile, g, mtile, nchunk);
                const int row0 = g * p.G + nchunk * BN + (p.fused ? 0 : rank * 128);
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sb = smem + size_t(s) * kPairStageBytes + kAStageBytes;
                    // the even CTA announces the bytes of both halves (and of both CTAs' token
                    // rows when they come by TMA)
                    if (rank == 0)
                        mbar_arrive_expect_tx(&full[s], 2u * 128 * kBK * 2 + (p.gather4 ? 2u * kAStageBytes : 0u));
                    tma_load_2d_pair(sb, map, &full[s], kb * kBK, row0);
                    if (++s == kPairStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ============================ UMMA issuer (even CTA only) ====================
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_f16(kBf16 ? 1 : 0, 256, 256);
            int s = 0, acc_it = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < total_tiles; tile += npairs, ++acc_it) {
                const int ab = acc_it & 1;
                if (!mbar_wait(&tempty[ab], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * 256);
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(&full[s], ph, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + size_t(s) * kPairStageBytes);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kAStageBytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma_f16_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc,
                                         (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                    if (++s == kPairStages) { s = 0; ph ^= 1; }
                }
                if (ok) umma_commit_pair(&tfull[ab]);
            }
        }
    } else if (p.gather4) {
        // ============================ A-row gather by TMA (own 128 rows) =============
        // one warp: lane l owns rows 4l .. 4l+3 of the tile and issues one four-row copy per
        // 64-wide k-block; rows past the group's count get an index outside the tensor and
        // arrive as zeros
        if (warp == 6) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const int oob = static_cast<int>(p.M);
            for (int tile = pair; ok && tile < total_tiles; tile += npairs) {
                int g, mtile, nchunk;
                tmap.decode(tile, g, mtile, nchunk);
                const int cnt = p.counts[g];
                int r[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int slot = mtile * RT + rank * kBM + 4 * lane + i;
                    r[i] = oob;
                    if (slot < cnt) {
                        const int64_t tok = p.sidx[static_cast<int64_t>(slot) * p.NG + g];
                        if (tok >= 0 && tok < p.M) r[i] = static_cast<int>(tok);
                    }
                }
                for (int kb = 0; kb < KB; ++kb) {
                    const bool got = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY);
                    if (!__all_sync(0xffffffffu, got)) {
                        ok = false;
                        break;
                    }
                    uint8_t* dst = smem + size_t(s) * kPairStageBytes + lane * (4 * 128);
                    tma_gather4_pair(dst, &tmA, &full[s], kb * kBK, r[0], r[1], r[2], r[3]);
                    if (++s == kPairStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else {
        // ============================ A-row gather (own 128 rows) ====================
        const int gt = threadIdx.x - 6 * 32;
        const int chunk = gt & 7;
        const int rsub = gt >> 3;
        const uint32_t dst_off = static_cast<uint32_t>(rsub * 128 + ((chunk ^ (rsub & 7)) << 4));
        int it = 0, s = 0, s_lag = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < total_tiles; tile += npairs) {
            int g, mtile, nchunk;
            tmap.decode(tile, g, mtile, nchunk);
            const int cnt = p.counts[g];
            const uint8_t* src_row[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int slot = mtile * RT + rank * kBM + i * 16 + rsub;
                src_row[i] = nullptr;
                if (slot < cnt) {
                    int64_t tok = p.sidx[static_cast<int64_t>(slot) * p.NG + g];
                    if (tok >= 0 && tok < p.M) src_row[i] = p.A + tok * p.lda * 2;
                }
            }
            for (int kb = 0; kb < KB; ++kb, ++it) {
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) {
                    ok = false;
                    break;
                }
                const int kcol = kb * kBK + chunk * 8;
                const bool kvalid = kcol < p.K;
                const uint32_t dst = smem_u32(smem + size_t(s) * kPairStageBytes) + dst_off;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool on = kvalid && src_row[i] != nullptr;
                    const void* src = on ? static_cast<const void*>(src_row[i] + kcol * 2)
                                         : static_cast<const void*>(p.A);
                    cp_async_16(dst + i * 16 * 128, src, on ? 16u : 0u);
                }
                cp_async_commit();
                if (++s == kPairStages) { s = 0; ph ^= 1; }
                if (it >= kGatherLag) {
                    cp_async_wait<kGatherLag>();
                    fence_proxy_async_smem();
                    mbar_arrive_leader(&full[s_lag]);
                    if (++s_lag == kPairStages) s_lag = 0;
                }
            }
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (ok) {
            for (int j = (it > kGatherLag ? it - kGatherLag : 0); j < it; ++j) {
                mbar_arrive_leader(&full[s_lag]);
                if (++s_lag == kPairStages) s_lag = 0;
            }
        }
    }

    // ---- tear-down -------------------------------------------------------------------
    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // the partner no longer reads this CTA's memory or barriers
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

int gemm_mn_pair_launch(const CUtensorMap& tmW, const CUtensorMap& tmW2, const CUtensorMap& tmA,
                        MnParams p, int dtype, cudaStream_t s)
{
    int grid = sm_count() & ~1;
    if (grid < 2) return fail(DPK_ERR_UNSUPPORTED, "no CTA pair available");
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(gemm_mn_pair_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmemBytes));
        gemm_mn_pair_kernel<true><<<grid, kMnThreads, kPairSmemBytes, s>>>(tmW, tmW2, tmA, p);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(gemm_mn_pair_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmemBytes));
        gemm_mn_pair_kernel<false><<<grid, kMnThreads, kPairSmemBytes, s>>>(tmW, tmW2, tmA, p);
    }
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk
