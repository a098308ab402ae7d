// Reduction-width routed projection on tcgen05 tensor cores (sm_100a).
//
//   D[t, n] = sum over groups g active for token t of A[t, g-cols] . W[n, g-cols]
//
// The K range differs per token, so partial products of different groups must be
// summed per token.  This kernel keeps the sum output-stationary: a CTA owns a
// [128-token window x BN] fp32 accumulator in TMEM and walks the groups; for each
// group it loads the window's A columns with one TMA tile load, overwrites the rows
// of tokens that do not use the group with zeros in shared memory, and issues the
// UMMAs.  Groups that no token of the window uses are skipped entirely (loads and
// MMAs).  There are no global atomics and the result is deterministic; the price is
// that an inactive row of a visited (window, group) block still occupies MMA rows.
//
// Warp roles (320 threads):
//   warps 0-3  epilogue: TMEM -> registers -> half -> global rows
//   warp  4    TMA producer (A window tile + weight tile), one lane
//   warp  5    UMMA issuer, one lane; owns the TMEM allocation
//   warps 6-9  row fix-up: thread r zeroes row r of the landed A tile when token
//              m0+r does not use the group, then fences generic->async proxy
//
// Algorithmic work per launch: 2*N*G flops per active (token, group) pair; executed
// work: 2*N*G*128 per visited (window, group) block.
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kAStageBytes = kBM * kBK * 2;
constexpr int kRingBytes = 4 * (kAStageBytes + 256 * kBK * 2);   // 192 KiB of operand ring
constexpr int kMaxStages = 12;
constexpr int kKThreads = 320;
constexpr int kTmemCols = 512;

struct KParams {
    uint8_t* D;              // [M, ldd] half
    const uint32_t* row_bits;   // [M, words]
    const uint32_t* win_bits;   // [nwin, words]
    int64_t ldd;
    int64_t M;
    int N, K, NG, G;
    int BN;                  // accumulator width (UMMA N)
    int n_chunks;            // ceil(N / BN)
    int words;               // ceil(NG / 32)
    int kb_per_group;        // G / 64
    int total_tiles;
    int stages;              // ring depth: kRingBytes / stage_bytes, at most kMaxStages
    int stage_bytes;         // kAStageBytes + BN * 128
    int* status;
};

constexpr size_t kKSmemBytes = 1024 + size_t(kRingBytes) +
                               (3 * kMaxStages + 4) * sizeof(uint64_t) + 16;

template <bool kBf16>
__global__ void __launch_bounds__(kKThreads, 1)
gemm_k_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
              const KParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    uint64_t* tma_full = reinterpret_cast<uint64_t*>(smem + size_t(kRingBytes));
    uint64_t* full = tma_full + kMaxStages;
    uint64_t* empty = full + kMaxStages;
    uint64_t* tfull = empty + kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nst = p.stages;
    const int stage_bytes = p.stage_bytes;

    if (warp == 4 && lane == 0) {
        for (int s = 0; s < nst; ++s) {
            mbar_init(&tma_full[s], 1);   // arrive.expect_tx by the producer
            mbar_init(&full[s], 128);     // fix-up threads
            mbar_init(&empty[s], 1);      // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 128);
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int BN = p.BN;

    // Does window `mwin` use any group at all?
    auto window_any = [&](int mwin) -> bool {
        uint32_t any = 0;
        for (int w = 0; w < p.words; ++w) any |= p.win_bits[static_cast<int64_t>(mwin) * p.words + w];
        return any != 0;
    };

    if (warp < 4) {
        // ============================ epilogue ======================================
        int acc_it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
            const int mwin = tile / p.n_chunks, nchunk = tile - mwin * p.n_chunks;
            const int64_t r = static_cast<int64_t>(mwin) * kBM + warp * 32 + lane;
            const bool valid = r < p.M;
            const int n0 = nchunk * BN;
            uint8_t* out = p.D + (r * p.ldd + n0) * 2;
            if (!window_any(mwin)) {
                // no group is active for any token of the window: the rows are zero
                if (valid)
                    for (int c = 0; c < BN && n0 + c < p.N; c += 8)
                        *reinterpret_cast<uint4*>(out + c * 2) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const int ab = acc_it & 1;
            const bool got = mbar_wait(&tfull[ab], (acc_it >> 1) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                   static_cast<uint32_t>(ab * 256);
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
                        if (q * 8 < n && n0 + c + q * 8 < p.N) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                w[j] = pack_half2<kBf16>(__uint_as_float(v[q * 8 + 2 * j]),
                                                         __uint_as_float(v[q * 8 + 2 * j + 1]));
                            *reinterpret_cast<uint4*>(out + (c + q * 8) * 2) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty[ab]);
            ++acc_it;
        }
    } else if (warp == 4) {
        // ============================ TMA producer ==================================
        if (lane == 0) {
            const uint32_t tx_bytes = static_cast<uint32_t>(kBM + BN) * kBK * 2;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                const int mwin = tile / p.n_chunks, nchunk = tile - mwin * p.n_chunks;
                const uint32_t* wb = p.win_bits + static_cast<int64_t>(mwin) * p.words;
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = wb[w];
                    while (ok && bits) {
                        const int g = w * 32 + __ffs(bits) - 1;
                        bits &= bits - 1;
                        for (int j = 0; j < p.kb_per_group; ++j) {
                            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status,
                                           DPK_DEV_TIMEOUT_EMPTY)) {
                                ok = false;
                                break;
                            }
                            uint8_t* sa = smem + size_t(s) * stage_bytes;
                            const int kcol = g * p.G + j * kBK;
                            mbar_arrive_expect_tx(&tma_full[s], tx_bytes);
                            tma_load_2d(sa, &tmA, &tma_full[s], kcol, mwin * kBM);
                            tma_load_2d(sa + kAStageBytes, &tmW, &tma_full[s], kcol, nchunk * BN);
                            if (++s == nst) { s = 0; ph ^= 1; }
                        }
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ============================ UMMA issuer ===================================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kBf16 ? 1 : 0, kBM, BN);
            int s = 0, acc_it = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                const int mwin = tile / p.n_chunks;
                if (!window_any(mwin)) continue;
                const int ab = acc_it & 1;
                if (!mbar_wait(&tempty[ab], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * 256);
                const uint32_t* wb = p.win_bits + static_cast<int64_t>(mwin) * p.words;
                uint32_t first = 0;
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = wb[w];
                    while (ok && bits) {
                        bits &= bits - 1;
                        for (int j = 0; j < p.kb_per_group; ++j) {
                            if (!mbar_wait(&tma_full[s], ph, abort_flag, p.status,
                                           DPK_DEV_TIMEOUT_FULL) ||
                                !mbar_wait(&full[s], ph, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t sa = smem_u32(smem + size_t(s) * stage_bytes);
                            const uint64_t adesc = umma_desc_k_sw128(sa);
                            const uint64_t bdesc = umma_desc_k_sw128(sa + kAStageBytes);
#pragma unroll
                            for (int k = 0; k < kBK / 16; ++k) {
                                umma_f16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, first);
                                first = 1;
                            }
                            umma_commit(&empty[s]);
                            if (++s == nst) { s = 0; ph ^= 1; }
                        }
                    }
                }
                if (ok) umma_commit(&tfull[ab]);
                ++acc_it;
            }
        }
    } else {
        // ============================ row fix-up ====================================
        // Warp w owns rows [32w, 32w+32) of the tile.  The rows to clear are found with a
        // ballot and cleared four per store instruction, eight lanes per 128-byte row
        // (a lane-per-row loop would put all 32 lanes on the same banks and starve the
        // tensor core's own operand reads).  The work per stage must stay far below the
        // 512 cycles the UMMAs of a stage take, since these warps handle stages in order.
        const int wrow0 = (warp - 6) * 32;
        const int row = wrow0 + lane;            // 0..127
        const int sub = lane >> 3;               // which of the 4 rows of a store this lane serves
        const int chunk = lane & 7;              // 16-byte chunk inside the row
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
            const int mwin = tile / p.n_chunks;
            const int64_t r = static_cast<int64_t>(mwin) * kBM + row;
            const bool in_range = r < p.M;
            const uint32_t* wb = p.win_bits + static_cast<int64_t>(mwin) * p.words;
            const uint32_t* rb = p.row_bits + (in_range ? r : 0) * p.words;
            uint32_t next_row = in_range ? rb[0] : 0u;
            for (int w = 0; ok && w < p.words; ++w) {
                uint32_t bits = wb[w];
                const uint32_t mine = next_row;
                if (w + 1 < p.words) next_row = in_range ? rb[w + 1] : 0u;
                while (ok && bits) {
                    const int b = __ffs(bits) - 1;
                    bits &= bits - 1;
                    const bool active = (mine >> b) & 1u;
                    const unsigned clear = __ballot_sync(0xffffffffu, !active);
                    for (int j = 0; j < p.kb_per_group; ++j) {
                        const bool got = mbar_wait(&tma_full[s], ph, abort_flag,
                                                   p.status, DPK_DEV_TIMEOUT_FULL);
                        if (!__all_sync(0xffffffffu, got)) {
                            ok = false;
                            break;
                        }
                        if (clear) {
                            // 8 stores, each covering rows 4i..4i+3 of the warp's 32 (8 lanes
                            // per 128-byte row), predicated on the row's bit in `clear`
                            uint8_t* base = smem + size_t(s) * stage_bytes + (wrow0 + sub) * 128 +
                                            chunk * 16;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if ((clear >> (i * 4 + sub)) & 1u)
                                    *reinterpret_cast<uint4*>(base + i * 4 * 128) =
                                        make_uint4(0, 0, 0, 0);
                            fence_proxy_async_smem();
                        }
                        mbar_arrive(&full[s]);
                        if (++s == nst) { s = 0; ph ^= 1; }
                    }
                }
            }
        }
    }

    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();   // lanes 1-31 skipped the role loop: reconverge before the aligned op
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace dpk

using namespace dpk;

extern "C" int dpk_gemm_k(const void* A, int64_t lda, const void* W, int64_t ldw,
                          const uint32_t* row_bits, const uint32_t* win_bits, void* D, int64_t ldd,
                          int64_t M, int N, int K, int NG, int dtype, void* stream)
{
    DPK_REQUIRE(A && W && D && row_bits && win_bits, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(M >= 0 && M < (1ll << 31) && N > 0 && K > 0 && NG > 0, "bad shape");
    DPK_REQUIRE(K % NG == 0, "K=%d is not divisible by NG=%d", K, NG);
    const int G = K / NG;
    DPK_REQUIRE(G % kBK == 0, "group width G=%d must be a multiple of %d", G, kBK);
    DPK_REQUIRE(N % 8 == 0, "N=%d must be a multiple of 8", N);
    DPK_REQUIRE(lda >= K && ldw >= K && ldd >= N, "row strides shorter than rows");
    DPK_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ldd % 8 == 0, "row strides must be multiples of 8");
    DPK_REQUIRE(aligned16(A) && aligned16(W) && aligned16(D), "tensors must be 16-byte aligned");
    if (M == 0) return DPK_OK;

    int BN = 256;
    if (N < 256) BN = ((N + 15) / 16) * 16;
    const int64_t nwin = (M + kBM - 1) / kBM;
    // Few token windows (decode): narrower output chunks until there is about one tile per
    // SM, so that the weight matrix is streamed by many CTAs in parallel.
    while (BN > 32 && BN % 32 == 0 && nwin * ((N + BN - 1) / BN) < sm_count()) BN /= 2;
    const int n_chunks = (N + BN - 1) / BN;
    DPK_REQUIRE(nwin * n_chunks < (1ll << 31), "too many tiles");

    CUtensorMap tmA, tmW;
    int rc = make_tmap_2d_sw128(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, kBM);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmW, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK, BN);
    if (rc) return rc;

    KParams p;
    p.D = static_cast<uint8_t*>(D);
    p.row_bits = row_bits;
    p.win_bits = win_bits;
    p.ldd = ldd;
    p.M = M;
    p.N = N;
    p.K = K;
    p.NG = NG;
    p.G = G;
    p.BN = BN;
    p.n_chunks = n_chunks;
    p.words = (NG + 31) / 32;
    p.kb_per_group = G / kBK;
    p.total_tiles = (int)(nwin * n_chunks);
    p.stage_bytes = kAStageBytes + BN * kBK * 2;
    p.stage_bytes = (p.stage_bytes + 1023) / 1024 * 1024;     // swizzled tiles need 1024-byte bases
    p.stages = kRingBytes / p.stage_bytes;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");

    int grid = sm_count();
    if (p.total_tiles < grid) grid = p.total_tiles;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(gemm_k_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKSmemBytes));
        gemm_k_kernel<true><<<grid, kKThreads, kKSmemBytes, s>>>(tmA, tmW, p);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(gemm_k_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKSmemBytes));
        gemm_k_kernel<false><<<grid, kKThreads, kKSmemBytes, s>>>(tmA, tmW, p);
    }
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}
