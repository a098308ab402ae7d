// Output-width routed projection on tcgen05 tensor cores (sm_100a).
//
// Work decomposition.  A tile is (group g, 128 consecutive entries of g's list of
// active tokens, one chunk of BN output channels of g).  The tile list is derived
// on the device from counts[] (no host synchronisation): a persistent grid of one
// CTA per SM walks it in group-major order, so that the CTAs running at the same
// time share one group's weight slab in L2.  No CTA exists for inactive work.
//
// Per tile, D[128 x N] = A_gathered[128 x K] * W_slab[N x K]^T with N = BN, or
// N = 2*BN when a second weight is given: the gate rows and the up rows of the same
// channels sit back to back in one shared-memory B tile, one UMMA of N = 2*BN
// produces both, and the epilogue writes silu(gate)*up.
//
// Warp roles (320 threads):
//   warps 0-3  epilogue: TMEM -> registers -> activation -> row scatter to D
//   warp  4    TMA producer of the weight tiles (one lane)
//   warp  5    UMMA issuer (one lane); also owns the TMEM allocation
//   warps 6-9  A-row gather: 16-byte cp.async of token rows into the 128B-swizzled
//              K-major layout UMMA reads, followed by a generic->async proxy fence
// The accumulator is double buffered in TMEM (2 x 256 columns), so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// Algorithmic work per launch: 2*K*G flops per active (token, group) pair per weight.
#define DPK_KERNEL_ID 1   // thousands digit of the device status word
#include "dpk_gemm_mn.cuh"

namespace dpk {

template <bool kBf16>
__global__ void __launch_bounds__(kMnThreads, 1)
gemm_mn_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
               const MnParams p)
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
    const int KB = (p.K + kBK - 1) / kBK;
    const int nst = p.stages;
    const int stage_bytes = p.stage_bytes;
    const int halves = p.halves;
    const int RT = kBM * halves;              // token rows per tile
    const int a_bytes = kAStageBytes * halves;

    // ---- set-up --------------------------------------------------------------------
    if (warp == 0) {
        // smallest row-tile count over the groups
        int tmin = 0x7fffffff;
        for (int g = lane; g < p.NG; g += 32) {
            int c = p.counts[g];
            c = c < 0 ? 0 : c;
            tmin = min(tmin, (c + RT - 1) / RT);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) tmin = min(tmin, __shfl_xor_sync(0xffffffffu, tmin, d));
        // prefix of the tiles beyond the regular part: (tiles(g) - tmin) * n_chunks
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
        for (int s = 0; s < nst; ++s) {
            mbar_init(&full[s], 1 + 128);   // TMA arrive.expect_tx + 128 gather threads
            mbar_init(&empty[s], 1);        // one tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);        // one tcgen05.commit
            mbar_init(&tempty[b], 128);     // 128 epilogue threads
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmW);
        if (p.fused) tma_prefetch_desc(&tmW2);
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
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
    const int BN = p.BN;
    const int umma_n = p.fused ? 2 * BN : BN;

    if (warp < 4) {
        // ============================ epilogue ======================================
        int acc_it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++acc_it) {
            int g, mtile, nchunk;
            tmap.decode(tile, g, mtile, nchunk);
            const int cnt = p.counts[g];
            const int ab = acc_it & 1;
            // the TMEM loads below are warp-collective: leave only as a whole warp
            const bool got = mbar_wait(&tfull[ab], (acc_it >> 1) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after_sync();
            for (int half = 0; half < halves; ++half) {
            const int slot = mtile * RT + half * kBM + warp * 32 + lane;
            bool valid = slot < cnt;
            int64_t tok = 0;
            if (valid) {
                tok = p.sidx[static_cast<int64_t>(slot) * p.NG + g];
                if (tok < 0 || tok >= p.M) {
                    atomicCAS(p.status, 0, 1000 * DPK_KERNEL_ID + DPK_DEV_BAD_INDEX);
                    valid = false;
                }
            }
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                   static_cast<uint32_t>(ab * 256 + half * 128);
            uint8_t* out = p.D + (tok * p.ldd + static_cast<int64_t>(g) * p.G +
                                  static_cast<int64_t>(nchunk) * BN) * 2;
            if (p.fused) {
                for (int c = 0; c < BN; c += 32) {
                    uint32_t gate[32], up[32];
                    if (BN - c >= 32) {
                        tmem_ld_32x32b_x32(taddr + c, gate);
                        tmem_ld_32x32b_x32(taddr + BN + c, up);
                    } else {   // BN == 16
                        uint32_t g16[16], u16[16];
                        tmem_ld_32x32b_x16(taddr + c, g16);
                        tmem_ld_32x32b_x16(taddr + BN + c, u16);
#pragma unroll
                        for (int i = 0; i < 16; ++i) { gate[i] = g16[i]; up[i] = u16[i]; }
                    }
                    tmem_ld_wait();
                    const int n = (BN - c >= 32) ? 32 : 16;
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (q * 8 < n) {
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
                }
            } else {
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    if (BN - c >= 32) {
                        tmem_ld_32x32b_x32(taddr + c, v);
                    } else {
                        uint32_t v16[16];
                        tmem_ld_32x32b_x16(taddr + c, v16);
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = v16[i];
                    }
                    tmem_ld_wait();
                    const int n = (BN - c >= 32) ? 32 : 16;
                    if (valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (q * 8 < n) {
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
            }
            }   // halves
            tc_fence_before_sync();
            mbar_arrive(&tempty[ab]);
        }
    } else if (warp == 4) {
        // ============================ weight TMA producer ===========================
        if (lane == 0) {
            const uint32_t tx_bytes = static_cast<uint32_t>(umma_n) * kBK * 2;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                int g, mtile, nchunk;
                tmap.decode(tile, g, mtile, nchunk);
                const int row0 = g * p.G + nchunk * BN;
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sb = smem + size_t(s) * stage_bytes + a_bytes;
                    mbar_arrive_expect_tx(&full[s], tx_bytes);
                    tma_load_2d(sb, &tmW, &full[s], kb * kBK, row0);
                    if (p.fused) tma_load_2d(sb + BN * kBK * 2, &tmW2, &full[s], kb * kBK, row0);
                    if (++s == nst) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 5) {
        // ============================ UMMA issuer ===================================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kBf16 ? 1 : 0, kBM, umma_n);
            int s = 0, acc_it = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++acc_it) {
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
                    const uint32_t sa = smem_u32(smem + size_t(s) * stage_bytes);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + a_bytes);
                    for (int half = 0; half < halves; ++half) {
                        const uint64_t adesc = umma_desc_k_sw128(sa + half * kAStageBytes);
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k) {
                            // 16 elements = 32 bytes further along K inside the swizzle atom
                            umma_f16_ss(d_tmem + half * 128, adesc + 2 * k, bdesc + 2 * k, idesc,
                                        (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty[s]);
                    if (++s == nst) { s = 0; ph ^= 1; }
                }
                if (ok) umma_commit(&tfull[ab]);
            }
        }
    } else {
        // ============================ A-row gather ==================================
        const int gt = threadIdx.x - 6 * 32;     // 0..127
        const int chunk = gt & 7;                // 16-byte chunk of the 128-byte row
        const int rsub = gt >> 3;                // 0..15
        const uint32_t dst_off = static_cast<uint32_t>(rsub * 128 + ((chunk ^ (rsub & 7)) << 4));
        int it = 0;              // k-blocks issued so far
        int s = 0;               // stage being filled
        int s_lag = 0;           // stage whose copies are signalled next (kGatherLag behind)
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
            int g, mtile, nchunk;
            tmap.decode(tile, g, mtile, nchunk);
            const int cnt = p.counts[g];
            const uint8_t* src_row[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int slot = mtile * RT + i * 16 + rsub;
                src_row[i] = nullptr;
                if (i < 8 * halves && slot < cnt) {
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
                const uint32_t dst = smem_u32(smem + size_t(s) * stage_bytes) + dst_off;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i < 8 * halves) {
                        const bool on = kvalid && src_row[i] != nullptr;
                        const void* src = on ? static_cast<const void*>(src_row[i] + kcol * 2)
                                             : static_cast<const void*>(p.A);
                        cp_async_16(dst + i * 16 * 128, src, on ? 16u : 0u);
                    }
                }
                cp_async_commit();
                if (++s == nst) { s = 0; ph ^= 1; }
                if (it >= kGatherLag) {
                    cp_async_wait<kGatherLag>();
                    fence_proxy_async_smem();
                    mbar_arrive(&full[s_lag]);
                    if (++s_lag == nst) s_lag = 0;
                }
            }
        }
        // drain the groups still in flight
        cp_async_wait<0>();
        fence_proxy_async_smem();
        if (ok) {
            for (int j = (it > kGatherLag ? it - kGatherLag : 0); j < it; ++j) {
                mbar_arrive(&full[s_lag]);
                if (++s_lag == nst) s_lag = 0;
            }
        }
    }

    // ---- tear-down -----------------------------------------------------------------
    if (*abort_flag) __nanosleep(2000000);   // let copies already in flight land
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();   // lanes 1-31 skipped the role loop: reconverge before the aligned op
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

static int pick_bn(int G, int cap)
{
    for (int bn = cap; bn >= 16; bn >>= 1)
        if (G % bn == 0) return bn;
    return 0;
}

}  // namespace dpk

using namespace dpk;

static int g_mn_gather4 = 0;     // CTA-pair kernel: 0 = token rows by cp.async, 1 = by TMA tile::gather4

extern "C" int dpk_set_gemm_mn_gather(int mode)
{
    DPK_REQUIRE(mode == 0 || mode == 1, "mode must be 0 (cp.async row gather) or 1 (TMA tile::gather4)");
    g_mn_gather4 = mode;
    return DPK_OK;
}

extern "C" int dpk_gemm_mn(const void* A, int64_t lda, const void* W, const void* W2, int64_t ldw,
                           const int64_t* sorted_indices, const int32_t* counts, void* D,
                           int64_t ldd, int64_t M, int N, int K, int NG, int dtype, int act,
                           void* stream)
{
    DPK_REQUIRE(A && W && D && sorted_indices && counts, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(act >= DPK_ACT_IDENTITY && act <= DPK_ACT_SILU, "unknown activation %d", act);
    DPK_REQUIRE(M >= 0 && M < (1ll << 31) && N > 0 && K > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(NG <= kMaxGroups, "NG=%d exceeds %d", NG, kMaxGroups);
    DPK_REQUIRE(N % NG == 0, "N=%d is not divisible by NG=%d", N, NG);
    const int G = N / NG;
    DPK_REQUIRE(G % 16 == 0, "group width G=%d must be a multiple of 16", G);
    DPK_REQUIRE(K % 8 == 0, "K=%d must be a multiple of 8", K);
    DPK_REQUIRE(lda >= K && ldw >= K && ldd >= N, "row strides shorter than rows");
    DPK_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ldd % 8 == 0, "row strides must be multiples of 8");
    DPK_REQUIRE(aligned16(A) && aligned16(W) && aligned16(D) && (!W2 || aligned16(W2)),
                "tensors must be 16-byte aligned");
    if (M == 0) return DPK_OK;

    const int fused = W2 != nullptr;
    const int BN = pick_bn(G, fused ? 128 : 256);
    DPK_REQUIRE(BN >= 16, "no tile width divides G=%d", G);
    CUtensorMap tmW, tmW2;
    int rc = make_tmap_2d_sw128(&tmW, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK, BN);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmW2, fused ? W2 : W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK, BN);
    if (rc) return rc;

    MnParams p;
    p.A = static_cast<const uint8_t*>(A);
    p.D = static_cast<uint8_t*>(D);
    p.sidx = sorted_indices;
    p.counts = counts;
    p.lda = lda;
    p.ldd = ldd;
    p.M = M;
    p.K = K;
    p.NG = NG;
    p.G = G;
    p.BN = BN;
    p.n_chunks = G / BN;
    p.fused = fused;
    p.act = act;
    const int umma_n = fused ? 2 * BN : BN;
    // Two accumulators of <= 128 columns fit next to their double buffers in TMEM: let one
    // weight tile feed 256 token rows, which halves the weight bytes per flop.
    p.halves = (umma_n <= 128 && M >= 1024) ? 2 : 1;
    {
        // a block of R row tiles spans about 2*rows*R token rows at a 50 % keep ratio; keep the
        // rows it gathers (K*2 bytes each) within ~48 MiB so that they stay in L2
        const int64_t span_rows = (48ll << 20) / (static_cast<int64_t>(K) * 2);
        int r = static_cast<int>(span_rows / (2 * kBM * p.halves));
        p.rows_per_block = r < 4 ? 4 : (r > 4096 ? 4096 : r);
    }
    p.stage_bytes = kAStageBytes * p.halves + umma_n * kBK * 2;
    p.stages = kRingBytes / p.stage_bytes;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    p.gather4 = 0;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");

    // upper bound of the tile count, known without reading counts[] back
    int64_t bound = ((M + kBM * p.halves - 1) / (kBM * p.halves) + 1) * (int64_t)NG * p.n_chunks;
    int grid = sm_count();
    if (bound < grid) grid = (int)bound;
    if (grid < 1) grid = 1;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    {
        // wide tiles with many tokens: CTA pairs (tcgen05 cta_group::2) share each weight tile
        if (umma_n == 256 && M >= 2048 && sm_count() >= 2) {
            CUtensorMap pw, pw2;
            rc = make_tmap_2d_sw128(&pw, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK, 128);
            if (rc) return rc;
            rc = make_tmap_2d_sw128(&pw2, fused ? W2 : W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK,
                                    128);
            if (rc) return rc;
            MnParams q = p;
            q.halves = 2;
            // token rows by TMA tile::gather4 (row indices must fit 32 bits, which M does here)
            CUtensorMap pa;
            q.gather4 = g_mn_gather4;
            rc = make_tmap_2d_sw128(&pa, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, 1);
            if (rc) return rc;
            const int64_t span_rows = (48ll << 20) / (static_cast<int64_t>(K) * 2);
            int r = static_cast<int>(span_rows / (4 * kBM));
            q.rows_per_block = r < 4 ? 4 : (r > 4096 ? 4096 : r);
            return gemm_mn_pair_launch(pw, pw2, pa, q, dtype, s);
        }
    }
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(gemm_mn_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMnSmemBytes));
        gemm_mn_kernel<true><<<grid, kMnThreads, kMnSmemBytes, s>>>(tmW, tmW2, p);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(gemm_mn_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMnSmemBytes));
        gemm_mn_kernel<false><<<grid, kMnThreads, kMnSmemBytes, s>>>(tmW, tmW2, p);
    }
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
