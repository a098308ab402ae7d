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
#define DPK_KERNEL_ID 3   // thousands digit of the device status word
#include "dpk_gemm_k.cuh"

namespace dpk {

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

    // Routing bits of window `mwin`, word `w`, restricted to the groups of K-split `split`.
    auto win_word = [&](int mwin, int w, int split) -> uint32_t {
        uint32_t bits = p.win_bits[static_cast<int64_t>(mwin) * p.words + w];
        if (p.ksplit > 1) {
            const int g0 = static_cast<int>(static_cast<int64_t>(split) * p.NG / p.ksplit);
            const int g1 = static_cast<int>(static_cast<int64_t>(split + 1) * p.NG / p.ksplit);
            const int lo = max(g0 - w * 32, 0), hi = min(g1 - w * 32, 32);
            if (hi <= lo) return 0u;
            const uint32_t m_hi = hi >= 32 ? 0xffffffffu : ((1u << hi) - 1u);
            const uint32_t m_lo = (1u << lo) - 1u;
            bits &= m_hi & ~m_lo;
        }
        return bits;
    };
    // Does window `mwin` use any group of this split at all?
    auto window_any = [&](int mwin, int split) -> bool {
        uint32_t any = 0;
        for (int w = 0; w < p.words; ++w) any |= win_word(mwin, w, split);
        return any != 0;
    };
    // tile -> (window, output chunk, K-split); the split is the fastest index
    auto decode = [&](int tile, int& mwin, int& nchunk, int& split) {
        split = tile % p.ksplit;
        const int rest = tile / p.ksplit;
        mwin = rest / p.n_chunks;
        nchunk = rest - mwin * p.n_chunks;
    };

    if (warp < 4) {
        // ============================ epilogue ======================================
        int acc_it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
            int mwin, nchunk, split;
            decode(tile, mwin, nchunk, split);
            const int64_t r = static_cast<int64_t>(mwin) * kBM + warp * 32 + lane;
            const bool valid = r < p.M;
            const int n0 = nchunk * BN;
            uint8_t* out = p.D + (r * p.ldd + n0) * 2;
            // residual row of this thread (with split accumulation the conversion pass adds it)
            const uint8_t* res = (p.R && p.acc32 == nullptr) ? p.R + (r * p.ldr + n0) * 2 : nullptr;
            if (!window_any(mwin, split)) {
                // no group (of this split) is active for any token of the window: the rows
                // are zero (plus the residual); with split accumulation there is nothing to add
                if (valid && p.acc32 == nullptr)
                    for (int c = 0; c < BN && n0 + c < p.N; c += 8)
                        *reinterpret_cast<uint4*>(out + c * 2) =
                            res ? *reinterpret_cast<const uint4*>(res + c * 2) : make_uint4(0, 0, 0, 0);
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
                if (valid && p.acc32 != nullptr) {
                    float* acc = p.acc32 + r * p.N + n0 + c;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i < n && n0 + c + i < p.N) atomicAdd(acc + i, __uint_as_float(v[i]));
                } else if (valid) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (q * 8 < n && n0 + c + q * 8 < p.N)
                            *reinterpret_cast<uint4*>(out + (c + q * 8) * 2) =
                                pack8_plus_residual<kBf16>(v + q * 8, res ? res + (c + q * 8) * 2 : nullptr);
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
                int mwin, nchunk, split;
                decode(tile, mwin, nchunk, split);
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = win_word(mwin, w, split);
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
                int mwin, nchunk, split;
                decode(tile, mwin, nchunk, split);
                if (!window_any(mwin, split)) continue;
                const int ab = acc_it & 1;
                if (!mbar_wait(&tempty[ab], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * 256);
                uint32_t first = 0;
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = win_word(mwin, w, split);
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
            int mwin, nchunk, split;
            decode(tile, mwin, nchunk, split);
            const int64_t r = static_cast<int64_t>(mwin) * kBM + row;
            const bool in_range = r < p.M;
            const uint32_t* rb = p.row_bits + (in_range ? r : 0) * p.words;
            uint32_t next_row = in_range ? rb[0] : 0u;
            for (int w = 0; ok && w < p.words; ++w) {
                uint32_t bits = win_word(mwin, w, split);
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

// fp32 partial sums -> half output (after a split-K launch)
template <bool kBf16>
__global__ void gemm_k_convert_kernel(const float* __restrict__ acc, uint8_t* D, int64_t ldd,
                                      const uint8_t* R, int64_t ldr, int64_t M, int N)
{
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    if (i >= M * N) return;
    const int64_t r = i / N;
    const int n = static_cast<int>(i - r * N);      // N is even: the pair stays in one row
    float lo = acc[i], hi = acc[i + 1];
    if (R) {
        float rl, rh;
        unpack_half2<kBf16>(*reinterpret_cast<const uint32_t*>(R + (r * ldr + n) * 2), rl, rh);
        lo += rl;
        hi += rh;
    }
    *reinterpret_cast<uint32_t*>(D + (r * ldd + n) * 2) = pack_half2<kBf16>(lo, hi);
}

}  // namespace dpk

using namespace dpk;

extern "C" size_t dpk_gemm_k_workspace_bytes(int64_t M, int N)
{
    // split accumulation is only used for a handful of token windows (decode)
    if (M <= 0 || N <= 0 || M > 4 * kBM) return 0;
    return static_cast<size_t>(M) * N * sizeof(float);
}

namespace dpk {

// Where the output goes when it is not the caller's D (tensor-parallel scatter).
struct PeerOut {
    void* const* stage;      // [world] staging buffers, one per owner
    int world, rank;
    int64_t rows_per_owner;
};

// rows of a local [M, ldd] matrix -> slab `rank` of the owners' staging buffers
__global__ void peer_push_rows_kernel(const uint8_t* __restrict__ src, KParams p)
{
    const int64_t chunks_per_row = p.N / 8;
    const int64_t total = p.M * chunks_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / chunks_per_row;
        const int64_t c = i - r * chunks_per_row;
        const int64_t owner = r / p.rows_per_owner;
        const int64_t slab_row = int64_t(p.my_rank) * p.rows_per_owner + (r - owner * p.rows_per_owner);
        *reinterpret_cast<uint4*>(p.peer[owner] + (slab_row * p.ldd + c * 8) * 2) =
            *reinterpret_cast<const uint4*>(src + (r * p.ldd + c * 8) * 2);
    }
}

static int gemm_k_run(const void* A, int64_t lda, const void* W, int64_t ldw,
                      const uint32_t* row_bits, const uint32_t* win_bits, void* D, int64_t ldd,
                      int64_t M, int N, int K, int NG, int dtype, void* workspace,
                      size_t workspace_bytes, void* stream, const PeerOut* peer,
                      const void* residual = nullptr, int64_t ldr = 0)
{
    DPK_REQUIRE(!residual || (!peer && ldr >= N && ldr % 8 == 0 && aligned16(residual)),
                "residual: [M, ldr] with ldr >= N, a multiple of 8, 16-byte aligned, plain output only");
    DPK_REQUIRE(A && W && (D || peer) && row_bits && win_bits, "NULL tensor");
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
    const int64_t nwin_all = (M + kBM - 1) / kBM;
    const bool pair_shape = N >= 256 && nwin_all >= 16 && sm_count() >= 2;
    if (peer) {
        DPK_REQUIRE(peer->world >= 1 && peer->world <= kMaxPeers, "world must be 1..%d", kMaxPeers);
        DPK_REQUIRE(peer->rank >= 0 && peer->rank < peer->world, "rank outside the world");
        DPK_REQUIRE(peer->rows_per_owner > 0 && peer->rows_per_owner % kBM == 0,
                    "rows_per_owner must be a positive multiple of %d", kBM);
        DPK_REQUIRE(M <= peer->rows_per_owner * peer->world, "M exceeds world * rows_per_owner");
        for (int i = 0; i < peer->world; ++i)
            DPK_REQUIRE(peer->stage[i] && aligned16(peer->stage[i]), "staging buffer %d", i);
        if (!pair_shape) {
            // shapes the pair kernel does not take: compute into the workspace, then push rows
            const size_t split = dpk_gemm_k_workspace_bytes(M, N);
            const size_t need = split + static_cast<size_t>(M) * ldd * 2;
            DPK_REQUIRE(workspace && workspace_bytes >= need, "workspace of %zu bytes needed", need);
            uint8_t* tmp = static_cast<uint8_t*>(workspace) + split;
            int rc = gemm_k_run(A, lda, W, ldw, row_bits, win_bits, tmp, ldd, M, N, K, NG, dtype,
                                split ? workspace : nullptr, split, stream, nullptr);
            if (rc) return rc;
            KParams q{};
            q.M = M;
            q.N = N;
            q.ldd = ldd;
            q.world = peer->world;
            q.my_rank = peer->rank;
            q.rows_per_owner = peer->rows_per_owner;
            for (int i = 0; i < peer->world; ++i) q.peer[i] = static_cast<uint8_t*>(peer->stage[i]);
            const int64_t total = M * (N / 8);
            int blocks = static_cast<int>((total + 255) / 256);
            if (blocks > 8 * sm_count()) blocks = 8 * sm_count();
            peer_push_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(tmp, q);
            DPK_CUDA(cudaGetLastError());
            return DPK_OK;
        }
    }

    int BN = 256;
    if (N < 256) BN = ((N + 15) / 16) * 16;
    const int64_t nwin = (M + kBM - 1) / kBM;
    const int n_chunks = (N + BN - 1) / BN;
    DPK_REQUIRE(nwin * n_chunks < (1ll << 27), "too many tiles");
    // Few token windows (decode): there are not enough [window x 256] tiles to keep the SMs
    // streaming weights, so the group range is split over several CTAs per tile which add
    // their fp32 partial sums into the caller's zero-filled workspace.
    int ksplit = 1;
    const size_t ws_need = dpk_gemm_k_workspace_bytes(M, N);
    if (workspace != nullptr && ws_need != 0 && workspace_bytes >= ws_need && N % 2 == 0 &&
        nwin * n_chunks * 2 <= sm_count()) {
        ksplit = static_cast<int>(sm_count() / (nwin * n_chunks));
        if (ksplit > 16) ksplit = 16;
        if (ksplit > NG) ksplit = NG;
        if (ksplit < 1) ksplit = 1;
    }
    CUtensorMap tmA, tmW;
    int rc = make_tmap_2d_sw128(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, kBM);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmW, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, kBK, BN);
    if (rc) return rc;

    KParams p;
    p.D = static_cast<uint8_t*>(D);
    p.R = static_cast<const uint8_t*>(residual);
    p.ldr = ldr;
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
    p.total_tiles = (int)(nwin * n_chunks) * ksplit;
    p.ksplit = ksplit;
    p.acc32 = ksplit > 1 ? static_cast<float*>(workspace) : nullptr;
    p.stage_bytes = kAStageBytes + BN * kBK * 2;
    p.stage_bytes = (p.stage_bytes + 1023) / 1024 * 1024;     // swizzled tiles need 1024-byte bases
    p.stages = kRingBytes / p.stage_bytes;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");
    p.world = 0;
    p.my_rank = 0;
    p.rows_per_owner = 0;
    for (int i = 0; i < kMaxPeers; ++i) p.peer[i] = nullptr;
    if (peer) {
        p.world = peer->world;
        p.my_rank = peer->rank;
        p.rows_per_owner = peer->rows_per_owner;
        for (int i = 0; i < peer->world; ++i) p.peer[i] = static_cast<uint8_t*>(peer->stage[i]);
    }

    int grid = sm_count();
    if (p.total_tiles < grid) grid = p.total_tiles;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // many token windows and full-width chunks: CTA pairs share each weight tile
    if (peer) ksplit = 1, p.ksplit = 1, p.acc32 = nullptr, p.total_tiles = (int)(nwin * n_chunks);
    if (ksplit == 1 && pair_shape) return gemm_k_pair_launch(A, lda, W, ldw, p, dtype, s);
    if (ksplit > 1) DPK_CUDA(cudaMemsetAsync(workspace, 0, ws_need, s));
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(gemm_k_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKSmemBytes));
        gemm_k_kernel<true><<<grid, kKThreads, kKSmemBytes, s>>>(tmA, tmW, p);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(gemm_k_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kKSmemBytes));
        gemm_k_kernel<false><<<grid, kKThreads, kKSmemBytes, s>>>(tmA, tmW, p);
    }
    if (ksplit > 1) {
        const int64_t pairs = (M * N + 1) / 2;
        const unsigned blocks = static_cast<unsigned>((pairs + 255) / 256);
        uint8_t* d = static_cast<uint8_t*>(D);
        if (dtype == DPK_BF16)
            gemm_k_convert_kernel<true><<<blocks, 256, 0, s>>>(p.acc32, d, ldd, p.R, p.ldr, M, N);
        else
            gemm_k_convert_kernel<false><<<blocks, 256, 0, s>>>(p.acc32, d, ldd, p.R, p.ldr, M, N);
    }
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk

extern "C" int dpk_gemm_k(const void* A, int64_t lda, const void* W, int64_t ldw,
                          const uint32_t* row_bits, const uint32_t* win_bits, void* D, int64_t ldd,
                          int64_t M, int N, int K, int NG, int dtype, const void* residual,
                          int64_t ldr, void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(D != nullptr, "NULL tensor");
    return dpk::gemm_k_run(A, lda, W, ldw, row_bits, win_bits, D, ldd, M, N, K, NG, dtype, workspace,
                           workspace_bytes, stream, nullptr, residual, ldr);
}

extern "C" size_t dpk_gemm_k_scatter_workspace_bytes(int64_t M, int N, int64_t ldd)
{
    if (M <= 0 || N <= 0) return 0;
    const bool pair_shape = N >= 256 && (M + dpk::kBM - 1) / dpk::kBM >= 16;
    return dpk_gemm_k_workspace_bytes(M, N) + (pair_shape ? 0 : static_cast<size_t>(M) * ldd * 2);
}

extern "C" int dpk_gemm_k_scatter(const void* A, int64_t lda, const void* W, int64_t ldw,
                                  const uint32_t* row_bits, const uint32_t* win_bits,
                                  void* const* stage, int world, int rank, int64_t rows_per_owner,
                                  int64_t ldd, int64_t M, int N, int K, int NG, int dtype,
                                  void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(stage != nullptr, "NULL staging table");
    dpk::PeerOut peer{stage, world, rank, rows_per_owner};
    return dpk::gemm_k_run(A, lda, W, ldw, row_bits, win_bits, nullptr, ldd, M, N, K, NG, dtype,
                           workspace, workspace_bytes, stream, &peer);
}
