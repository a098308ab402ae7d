// Reduction-width routed projection on CTA pairs (tcgen05 cta_group::2, sm_100a).
//
// Same mathematics as dpk_gemm_k.cu for many token windows and N >= 256.  Two CTAs of
// a cluster own two consecutive 128-token windows and one 256-column output chunk:
// CTA r loads window (2*pw + r)'s A columns by TMA into its own shared memory, clears
// the rows of tokens that do not use the group, and loads rows [n0 + 128r, n0 + 128r +
// 128) of the weight chunk.  One thread of the even CTA issues tcgen05.mma.cta_group::2
// with M = 256, so every weight byte feeds 256 token rows and each SM reads 16 + 16 KiB
// per 64-deep K block instead of 16 + 32 KiB.  The pair walks the union of the groups its
// two windows use; a window's rows are cleared for groups only the other window uses.
//
// Barriers.  a_full (each CTA): its own A tile has landed (TMA bytes).  full (even CTA):
// both weight halves have landed (TMA bytes, the odd CTA's load counts there through the
// cta_group::2 form) and the 256 fix-up threads of both CTAs have cleared their rows.
// empty / tfull (both CTAs): multicast commits.  tempty (even CTA): 256 epilogue threads.
// Every wait is bounded; a cluster barrier precedes the exit.
//
// Peer output (kPeer).  Under tensor parallelism the partial sums of a token window go to the
// rank that owns the window: rows [o*R, (o+1)*R) belong to rank o, and rank r's partial lands in
// slab r of owner o's staging buffer, a plain pointer into that GPU's memory.  The epilogue
// transposes each 32 x 64 piece through shared memory so that every store instruction writes
// four 128-byte row segments -- link packets are filled, which per-thread 16-byte stores to 32
// different rows would not do.  Nothing here waits on another GPU.
#define DPK_KERNEL_ID 4   // thousands digit of the device status word
#include "dpk_gemm_k.cuh"

namespace dpk {

constexpr int kKPairStageBytes = kAStageBytes + 128 * kBK * 2;    // 32 KiB
constexpr int kKPairStages = kRingBytes / kKPairStageBytes;       // 6
constexpr size_t kKPairSmemBytes = 1024 + size_t(kRingBytes) + (3 * kMaxStages + 4) * sizeof(uint64_t) + 16;
constexpr int kPeerXposeOffset = kRingBytes + 512;        // past the barriers, 128-byte aligned
constexpr int kPeerXposeBytes = 4 * 32 * 128;             // 4 epilogue warps x 32 rows x 64 halves
constexpr size_t kKPairPeerSmemBytes = 1024 + size_t(kPeerXposeOffset) + kPeerXposeBytes;
static_assert((3 * kMaxStages + 4) * sizeof(uint64_t) + 16 <= 512, "barriers overlap the transpose area");

struct KPairParams {
    KParams k;
    int64_t nwin;       // 128-token windows
    int pair_tiles;     // ceil(nwin / 2) * n_chunks
    int pair_windows;   // ceil(nwin / 2)
    int window_shift;   // peer output: the walk over the pair windows starts here (and wraps)
    int chunk_group;    // 0: tiles walk all weight chunks of one pair window, then the next window;
                        // g > 0: groups of g chunks outermost, pair windows inside, the g chunks innermost
    unsigned int* wave_counter;   // NULL, or one zeroed counter per wave of tiles: the producers of all
                                  // CTAs start a wave together (a bounded wait, given up silently)
    int wave_slots;
};

template <bool kBf16, bool kPeer>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kKThreads, 1)
gemm_k_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                   const KPairParams pp)
{
    const KParams& p = pp.k;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    uint64_t* a_full = reinterpret_cast<uint64_t*>(smem + size_t(kRingBytes));
    uint64_t* full = a_full + kMaxStages;
    uint64_t* empty = full + kMaxStages;
    uint64_t* tfull = empty + kMaxStages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());
    const int pair = blockIdx.x >> 1;
    const int npairs = gridDim.x >> 1;

    if (warp == 4 && lane == 0) {
        for (int s = 0; s < kKPairStages; ++s) {
            mbar_init(&a_full[s], 1);       // own A tile: arrive.expect_tx
            mbar_init(&full[s], 1 + 256);   // even CTA's expect_tx for both weight halves + fix-up threads
            mbar_init(&empty[s], 1);        // multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 256);
        }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
    }
    if (warp == 5) tmem_alloc_pair(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // routing bits of window `win`, word `w` (0 beyond the last window)
    auto win_word = [&](int64_t win, int w) -> uint32_t {
        return win < pp.nwin ? p.win_bits[win * p.words + w] : 0u;
    };
    // groups used by either window of pair-window `pw`
    auto pair_word = [&](int pw, int w) -> uint32_t {
        return win_word(2ll * pw, w) | win_word(2ll * pw + 1, w);
    };
    auto pair_any = [&](int pw) -> bool {
        uint32_t any = 0;
        for (int w = 0; w < p.words; ++w) any |= pair_word(pw, w);
        return any != 0;
    };
    // Peer output: rank r starts its walk at the windows owned by rank r + 1, so that at any
    // moment the ranks store into different owners instead of all into the same one.
    auto decode = [&](int tile, int& pw, int& nchunk) {
        if (pp.chunk_group > 0) {
            const int g = pp.chunk_group, per = pp.pair_windows * g, full = p.n_chunks / g;
            if (tile < full * per) {
                const int cg = tile / per, rem = tile - cg * per;
                pw = rem / g;
                nchunk = cg * g + rem - pw * g;
            } else {                                   // the last, narrower group of chunks
                const int rem = tile - full * per, wl = p.n_chunks - full * g;
                pw = rem / wl;
                nchunk = full * g + rem - pw * wl;
            }
        } else {
            pw = tile / p.n_chunks;
            nchunk = tile - pw * p.n_chunks;
        }
        if constexpr (kPeer) {
            pw += pp.window_shift;
            if (pw >= pp.pair_windows) pw -= pp.pair_windows;
        }
    };

    if (warp < 4) {
        // ============================ epilogue (own window) ==========================
        int acc_it = 0;
        for (int tile = pair; tile < pp.pair_tiles; tile += npairs) {
            int pw, nchunk;
            decode(tile, pw, nchunk);
            const int64_t r = (2ll * pw + rank) * kBM + warp * 32 + lane;
            const bool valid = r < p.M;
            const int n0 = nchunk * 256;
            uint8_t* out;                 // local: this thread's row; peer: the warp's first row
            int64_t rows_left = 0;        // peer: rows of this warp's 32 inside the token range
            if constexpr (kPeer) {
                const int64_t row0 = (2ll * pw + rank) * kBM + warp * 32;
                // (a pair's second window may lie past the last token: it stores nothing)
                const int64_t owner = min(row0 / p.rows_per_owner, int64_t(p.world - 1));
                const int64_t slab_row = int64_t(p.my_rank) * p.rows_per_owner +
                                         (row0 - owner * p.rows_per_owner);
                out = p.peer[owner] + (slab_row * p.ldd + n0) * 2;
                rows_left = p.M - row0;
            } else {
                out = p.D + (r * p.ldd + n0) * 2;
            }
            const uint8_t* res = nullptr;     // this thread's residual row (plain output only)
            if constexpr (!kPeer) {
                if (p.R) res = p.R + (r * p.ldr + n0) * 2;
            }
            if (!pair_any(pw)) {
                if constexpr (kPeer) {
                    // the owner sums every slab: an unused window still contributes zeros
                    if (n0 + lane * 8 < p.N)
                        for (int i = 0; i < 32 && i < rows_left; ++i)
                            *reinterpret_cast<uint4*>(out + (int64_t(i) * p.ldd + lane * 8) * 2) =
                                make_uint4(0, 0, 0, 0);
                } else if (valid) {
                    for (int c = 0; c < 256 && n0 + c < p.N; c += 8)
                        *reinterpret_cast<uint4*>(out + c * 2) =
                            res ? *reinterpret_cast<const uint4*>(res + c * 2) : make_uint4(0, 0, 0, 0);
                }
                continue;
            }
            const int ab = acc_it & 1;
            const bool got = mbar_wait(&tfull[ab], (acc_it >> 1) & 1, abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                   static_cast<uint32_t>(ab * 256);
            if constexpr (kPeer) {
                uint8_t* xp = smem + kPeerXposeOffset + warp * (32 * 128);
                for (int c = 0; c < 256; c += 64) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(taddr + c + 32 * h, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                w[j] = pack_half2<kBf16>(__uint_as_float(v[q * 8 + 2 * j]),
                                                         __uint_as_float(v[q * 8 + 2 * j + 1]));
                            // row = lane, 16-byte chunk h*4+q, swizzled by the row: conflict free
                            *reinterpret_cast<uint4*>(xp + lane * 128 + (((h * 4 + q) ^ (lane & 7)) << 4)) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                    __syncwarp();
                    const int chunk = lane & 7;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int row = i * 4 + (lane >> 3);
                        const uint4 val = *reinterpret_cast<const uint4*>(
                            xp + row * 128 + ((chunk ^ (row & 7)) << 4));
                        if (row < rows_left && n0 + c + chunk * 8 < p.N)
                            *reinterpret_cast<uint4*>(out + (int64_t(row) * p.ldd + c + chunk * 8) * 2) = val;
                    }
                    __syncwarp();
                }
            } else {
            for (int c = 0; c < 256; c += 32) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + c, v);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (n0 + c + q * 8 < p.N)
                            *reinterpret_cast<uint4*>(out + (c + q * 8) * 2) =
                                pack8_plus_residual<kBf16>(v + q * 8, res ? res + (c + q * 8) * 2 : nullptr);
                    }
                }
            }
            }
            tc_fence_before_sync();
            mbar_arrive_leader(&tempty[ab]);
            ++acc_it;
        }
    } else if (warp == 4) {
        // ============================ TMA producer ===================================
        // own window's A tile -> a_full (local); own half of the weight tile -> the pair's full
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            unsigned int* wave_counter = pp.wave_counter;
            for (int tile = pair; ok && tile < pp.pair_tiles; tile += npairs) {
                int pw, nchunk;
                decode(tile, pw, nchunk);
                if (wave_counter) {
                    // Tiles that share an operand find it in L2 only while their CTAs walk K at the
                    // same time, and over tens of waves the CTAs drift apart (measured at 16384
                    // tokens, K = 28672: 24.2 GB of DRAM reads per launch; with the producers lined
                    // up at the start of every wave 7.9 GB).  Purely a hint: a producer that has
                    // waited ~50 us (CTAs of this grid not resident, another launch using the same
                    // counters) goes on alone and does not wait again.
                    const int wv = (tile - pair) / npairs;
                    if (wv > 0 && wv < pp.wave_slots) {
                        // both CTAs of every pair that has a tile in this wave (the last wave is short)
                        const int left = pp.pair_tiles - wv * npairs;
                        const unsigned int expected = 2u * static_cast<unsigned int>(left < npairs ? left : npairs);
                        atomicAdd(&wave_counter[wv], 1u);
                        const long long t0 = clock64();
                        while (*reinterpret_cast<volatile unsigned int*>(&wave_counter[wv]) < expected) {
                            if (clock64() - t0 > 100000ll) {
                                wave_counter = nullptr;
                                break;
                            }
                            __nanosleep(200);
                        }
                    }
                }
                const int a_row = static_cast<int>((2ll * pw + rank) * kBM);
                const int w_row = nchunk * 256 + rank * 128;
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = pair_word(pw, w);
                    while (ok && bits) {
                        const int g = w * 32 + __ffs(bits) - 1;
                        bits &= bits - 1;
                        for (int j = 0; j < p.kb_per_group; ++j) {
                            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status,
                                           DPK_DEV_TIMEOUT_EMPTY)) {
                                ok = false;
                                break;
                            }
                            uint8_t* sa = smem + size_t(s) * kKPairStageBytes;
                            const int kcol = g * p.G + j * kBK;
                            mbar_arrive_expect_tx(&a_full[s], kAStageBytes);
                            tma_load_2d(sa, &tmA, &a_full[s], kcol, a_row);
                            if (rank == 0) mbar_arrive_expect_tx(&full[s], 2u * 128 * kBK * 2);
                            tma_load_2d_pair(sa + kAStageBytes, &tmW, &full[s], kcol, w_row);
                            if (++s == kKPairStages) { s = 0; ph ^= 1; }
                        }
                    }
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
            for (int tile = pair; ok && tile < pp.pair_tiles; tile += npairs) {
                int pw, nchunk;
                decode(tile, pw, nchunk);
                if (!pair_any(pw)) continue;
                const int ab = acc_it & 1;
                if (!mbar_wait(&tempty[ab], ((acc_it >> 1) & 1) ^ 1, abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * 256);
                uint32_t first = 0;
                for (int w = 0; ok && w < p.words; ++w) {
                    uint32_t bits = pair_word(pw, w);
                    while (ok && bits) {
                        bits &= bits - 1;
                        for (int j = 0; j < p.kb_per_group; ++j) {
                            if (!mbar_wait(&full[s], ph, abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                            const uint32_t sa = smem_u32(smem + size_t(s) * kKPairStageBytes);
                            const uint64_t adesc = umma_desc_k_sw128(sa);
                            const uint64_t bdesc = umma_desc_k_sw128(sa + kAStageBytes);
#pragma unroll
                            for (int k = 0; k < kBK / 16; ++k) {
                                umma_f16_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, first);
                                first = 1;
                            }
                            umma_commit_pair(&empty[s]);
                            if (++s == kKPairStages) { s = 0; ph ^= 1; }
                        }
                    }
                }
                if (ok) umma_commit_pair(&tfull[ab]);
                ++acc_it;
            }
        }
    } else {
        // ============================ row fix-up (own window) ========================
        const int wrow0 = (warp - 6) * 32;
        const int row = wrow0 + lane;
        const int sub = lane >> 3;
        const int chunk = lane & 7;
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < pp.pair_tiles; tile += npairs) {
            int pw, nchunk;
            decode(tile, pw, nchunk);
            const int64_t r = (2ll * pw + rank) * kBM + row;
            const bool in_range = r < p.M;
            const uint32_t* rb = p.row_bits + (in_range ? r : 0) * p.words;
            uint32_t next_row = in_range ? rb[0] : 0u;
            for (int w = 0; ok && w < p.words; ++w) {
                uint32_t bits = pair_word(pw, w);
                const uint32_t mine = next_row;
                if (w + 1 < p.words) next_row = in_range ? rb[w + 1] : 0u;
                while (ok && bits) {
                    const int b = __ffs(bits) - 1;
                    bits &= bits - 1;
                    const bool active = (mine >> b) & 1u;
                    const unsigned clear = __ballot_sync(0xffffffffu, !active);
                    for (int j = 0; j < p.kb_per_group; ++j) {
                        const bool got = mbar_wait(&a_full[s], ph, abort_flag, p.status,
                                                   DPK_DEV_TIMEOUT_FULL);
                        if (!__all_sync(0xffffffffu, got)) {
                            ok = false;
                            break;
                        }
                        if (clear) {
                            uint8_t* base = smem + size_t(s) * kKPairStageBytes + (wrow0 + sub) * 128 +
                                            chunk * 16;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if ((clear >> (i * 4 + sub)) & 1u)
                                    *reinterpret_cast<uint4*>(base + i * 4 * 128) =
                                        make_uint4(0, 0, 0, 0);
                        }
                        // also orders the landed A tile before the partner CTA's UMMA issue
                        fence_proxy_async_smem();
                        mbar_arrive_leader(&full[s]);
                        if (++s == kKPairStages) { s = 0; ph ^= 1; }
                    }
                }
            }
        }
    }

    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// 1: groups of 8 weight chunks outermost and the producers of all CTAs lined up at every wave of
// tiles (the default); 0: all chunks of one pair window, then the next window, no alignment
int g_k_pair_wave_order = 1;
constexpr int kWaveSlots = 1024;
constexpr int kChunkGroup = 8;
__device__ unsigned int g_k_pair_wave_counter[kWaveSlots];

int gemm_k_pair_launch(const void* A, int64_t lda, const void* W, int64_t ldw, KParams p, int dtype,
                       cudaStream_t s)
{
    int grid = sm_count() & ~1;
    if (grid < 2) return fail(DPK_ERR_UNSUPPORTED, "no CTA pair available");
    CUtensorMap tmA, tmW;
    int rc = make_tmap_2d_sw128(&tmA, A, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda, kBK, kBM);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmW, W, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldw, kBK, 128);
    if (rc) return rc;
    KPairParams pp;
    pp.k = p;
    pp.k.BN = 256;
    pp.k.n_chunks = (p.N + 255) / 256;
    pp.k.ksplit = 1;
    pp.k.acc32 = nullptr;
    pp.nwin = (p.M + kBM - 1) / kBM;
    pp.pair_windows = static_cast<int>((pp.nwin + 1) / 2);
    pp.pair_tiles = pp.pair_windows * pp.k.n_chunks;
    pp.window_shift = 0;
    // A weight matrix that fits L2 is best left in the plain order (it stays resident while the
    // activations stream through once; grouping the chunks would read the activations once per
    // group instead).  Measured: N = 4096, K = 14336 (117 MB of weights, 8192 tokens) 0.80 ms plain
    // against 0.86 ms grouped; N = 8192, K = 28672 (470 MB, 16384 tokens) 6.7 against 6.4 ms.
    int l2_bytes = 0, dev = 0;
    DPK_CUDA(cudaGetDevice(&dev));
    DPK_CUDA(cudaDeviceGetAttribute(&l2_bytes, cudaDevAttrL2CacheSize, dev));
    const bool grouped = g_k_pair_wave_order && 2.0 * p.N * p.K > 1.0 * l2_bytes;
    pp.chunk_group = grouped ? kChunkGroup : 0;
    pp.wave_counter = nullptr;
    pp.wave_slots = 0;
    if (p.world > 1)
        pp.window_shift = static_cast<int>((int64_t((p.my_rank + 1) % p.world) * p.rows_per_owner / (2 * kBM)) %
                                           pp.pair_windows);
    if (2 * pp.pair_tiles < grid) grid = 2 * pp.pair_tiles;
    if (grouped) {
        // one counter per wave, zeroed on the stream ahead of the launch (the counters are one
        // array per device: launches that overlap on two streams disturb each other's alignment,
        // never their results)
        const int waves = (pp.pair_tiles + grid / 2 - 1) / (grid / 2);
        if (waves > 1 && waves <= kWaveSlots) {
            void* ptr = nullptr;
            DPK_CUDA(cudaGetSymbolAddress(&ptr, g_k_pair_wave_counter));
            DPK_CUDA(cudaMemsetAsync(ptr, 0, sizeof(unsigned int) * waves, s));
            pp.wave_counter = static_cast<unsigned int*>(ptr);
            pp.wave_slots = waves;
        }
    }
    auto launch = [&](auto kernel, size_t smem_bytes) -> int {
        DPK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem_bytes));
        kernel<<<grid, kKThreads, smem_bytes, s>>>(tmA, tmW, pp);
        return DPK_OK;
    };
    const bool peer = p.world > 0;
    if (peer) {
        if (p.rows_per_owner % kBM) return fail(DPK_ERR_INVALID, "rows_per_owner must be a multiple of 128");
        rc = dtype == DPK_BF16 ? launch(gemm_k_pair_kernel<true, true>, kKPairPeerSmemBytes)
                               : launch(gemm_k_pair_kernel<false, true>, kKPairPeerSmemBytes);
    } else {
        rc = dtype == DPK_BF16 ? launch(gemm_k_pair_kernel<true, false>, kKPairSmemBytes)
                               : launch(gemm_k_pair_kernel<false, false>, kKPairSmemBytes);
    }
    if (rc) return rc;
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk

extern "C" int dpk_set_gemm_k_wave_order(int on)
{
    DPK_REQUIRE(on == 0 || on == 1, "on must be 0 or 1");
    dpk::g_k_pair_wave_order = on;
    return DPK_OK;
}
