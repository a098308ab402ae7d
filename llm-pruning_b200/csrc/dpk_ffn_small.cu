// Dynamic-width SwiGLU FFN for a handful of tokens (decode steps, M <= 128), sm_100a.
//
// With a few dozen tokens every channel group is used by some token, so every weight byte
// has to cross HBM once whatever the routing says, and the tensor cores idle either way.  The
// prefill kernels (gathered token rows as the M operand, routing layout, row fix-up) pay for
// machinery that buys nothing here.  This kernel turns the product round instead: the weights
// are the M operand -- a tile is 128 weight rows -- and all tokens are the N operand (UMMA N =
// tokens rounded up to 16), re-read from L2 for every 64-wide k-block.
//
// One SM pulls ~45 GB/s from HBM, so the weights have to be spread evenly over ALL SMs.  The
// work is the flat list of (weight tile, k-block) units, cut into one contiguous range per CTA
// (a tile is shared by two or three CTAs where a cut falls inside it).  Every CTA adds its
// partial sums into an fp32 buffer with coalesced red.add; a per-block counter of finished
// k-blocks tells the CTA that completes a block to run the epilogue for it:
//
//   up   (tiles: gate rows and up rows of W_gate / W_up; a block = 128 intermediate channels,
//         complete when its gate tile and its up tile are): h = mask * silu(gate) * up -- a
//         routed-out (token, group) block becomes exact zeros, which is all the routing means
//         for the result;
//   down (tiles: rows of W_down, token operand h): y = dtype(sum).
//
// The epilogue also clears the buffer entries and the counter it used, so the workspace is
// zero again when the kernel ends: no memset, no conversion launch, no routing layout -- two
// launches per FFN instead of seven.  Same mathematics as the reference's
// gemm_mn(silu)*gemm_mn -> gemm_k composition (PruningInferSim/ops/mlp/m_pruning.py:76-105;
// WIDE/wrapper/attn_group_ffn_block.py:33-38).
#define DPK_KERNEL_ID 11   // thousands digit of the device status word
#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kSmBK = 64;
constexpr int kSmWTile = 128 * kSmBK * 2;         // 16 KiB: 128 weight rows x 64 k
constexpr int kSmThreads = 192;                   // 4 epilogue warps, TMA, UMMA
constexpr int kSmRing = 200 * 1024;
constexpr int kSmMaxStages = 12;
constexpr int kSmTmemCols = 256;
constexpr size_t kSmSmemBytes = 1024 + size_t(kSmRing) + (2 * kSmMaxStages + 4) * sizeof(uint64_t) + 32;

struct SmallParams {
    const uint8_t* mask;     // [M, NG] bytes (up)
    uint8_t* out;            // up: h [M, ldo]; down: y [M, ldo]
    float* acc;              // [M, acc_ld] fp32, zero between calls
    int* counters;           // [blocks], zero between calls
    int64_t ldo, acc_ld;
    int M, NG, G;
    int NT;                  // tokens rounded up to a multiple of 16 (UMMA N)
    int KB;                  // 64-wide k-blocks per tile
    int tiles;               // up: 2 * blocks (gate tile, up tile of block 0, of block 1, ...); down: blocks
    int blocks;              // 128-row blocks of the output
    int stages, stage_bytes;
    int* status;
};

struct SmallSmem {
    uint8_t* ring;
    uint64_t *full, *empty, *tfull, *tempty;
    uint32_t* tmem_slot;
    volatile int* abort_flag;
    int* flag;
    volatile int* gave_up;     // an epilogue warp's wait ran out: all four leave together
};

__device__ __forceinline__ SmallSmem small_smem(uint8_t* raw)
{
    SmallSmem s;
    s.ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    s.full = reinterpret_cast<uint64_t*>(s.ring + size_t(kSmRing));
    s.empty = s.full + kSmMaxStages;
    s.tfull = s.empty + kSmMaxStages;
    s.tempty = s.tfull + 2;
    s.tmem_slot = reinterpret_cast<uint32_t*>(s.tempty + 2);
    s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
    s.flag = reinterpret_cast<int*>(s.tmem_slot + 2);
    s.gave_up = reinterpret_cast<volatile int*>(s.tmem_slot + 3);
    return s;
}

__device__ __forceinline__ void named_barrier_128(int id)
{
    asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}

// The CTA's next part: (tile, k-blocks [k0, k1)) of its unit range [u, u1).
__device__ __forceinline__ void small_part(int64_t u, int64_t u1, int KB, int& tile, int& k0, int& k1)
{
    tile = static_cast<int>(u / KB);
    k0 = static_cast<int>(u - static_cast<int64_t>(tile) * KB);
    const int64_t left = u1 - u;
    k1 = left < KB - k0 ? k0 + static_cast<int>(left) : KB;
}

template <bool kBf16>
__device__ __forceinline__ void store_half(uint8_t* dst, float v)
{
    *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(pack_half2<kBf16>(v, 0.f) & 0xffffu);
}

// kUp: tile 2b is rows [128b, 128b+128) of W0 (gate), tile 2b+1 the same rows of W1 (up) -- the two
// tiles of a block are neighbours in the unit list, so blocks complete (and are converted by the
// epilogue warps) all through the kernel while the other warps keep streaming; the token operand is x.  !kUp: tiles are rows of W0 (down), the token operand is h.
template <bool kBf16, bool kUp>
__global__ void __launch_bounds__(kSmThreads, 1)
ffn_small_kernel(const __grid_constant__ CUtensorMap tmTok, const __grid_constant__ CUtensorMap tmW0,
                 const __grid_constant__ CUtensorMap tmW1, const SmallParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const SmallSmem sm = small_smem(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 4 && lane == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(&sm.full[i], 1);      // arrive.expect_tx of the TMA thread
            mbar_init(&sm.empty[i], 1);     // one tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.tfull[b], 1);
            mbar_init(&sm.tempty[b], 128);
        }
        *sm.abort_flag = 0;
        *sm.gave_up = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(sm.tmem_slot, kSmTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *sm.tmem_slot;
    const int NT = p.NT, KB = p.KB;
    const int64_t total = static_cast<int64_t>(p.tiles) * KB;
    const int64_t u_begin = total * blockIdx.x / gridDim.x;
    const int64_t u_end = total * (blockIdx.x + 1) / gridDim.x;

    if (warp < 4) {
        // ============================ epilogue ======================================
        const int row = warp * 32 + lane;
        int acc_it = 0;
        for (int64_t u = u_begin; u < u_end; ++acc_it) {
            int tile, k0, k1;
            small_part(u, u_end, KB, tile, k0, k1);
            u += k1 - k0;
            const int ab = acc_it & 1;
            const bool got = mbar_wait(&sm.tfull[ab], (acc_it >> 1) & 1, sm.abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            // A wait that ran out must not let this warp leave on its own: the other three would
            // sit at the named barriers below for good.  The warp only records the failure and
            // skips its share of the work; all four warps pass the three barriers of this
            // iteration, read the same flag between the second and the third, and leave together.
            // (gave_up is written before the first barrier and read after the second, so a
            // write of the next iteration cannot reach a reader of this one.)
            const bool warp_ok = __all_sync(0xffffffffu, got);
            const int block = kUp ? tile >> 1 : tile;
            if (warp_ok) {
                tc_fence_after_sync();
                // partial sums of this part -> fp32 buffer (a warp adds 32 consecutive floats)
                const bool second = kUp && (tile & 1);          // an up tile: its sums live past the gate sums
                float* dst = p.acc + (second ? static_cast<int64_t>(p.blocks) * 128 : 0) +
                             static_cast<int64_t>(block) * 128 + row;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                       static_cast<uint32_t>(ab * NT);
                for (int c = 0; c < NT; c += 16) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 16; ++t)
                        if (c + t < p.M) atomicAdd(dst + static_cast<int64_t>(c + t) * p.acc_ld, __uint_as_float(v[t]));
                }
                tc_fence_before_sync();
                mbar_arrive(&sm.tempty[ab]);
            } else if (lane == 0) {
                *sm.gave_up = 1;
            }
            // count the finished k-blocks of the block; whoever completes it runs its epilogue
            const int full_count = kUp ? 2 * KB : KB;
            __threadfence();
            named_barrier_128(1);
            if (threadIdx.x == 0)
                *sm.flag = *sm.gave_up ? -1 : atomicAdd(p.counters + block, k1 - k0) + (k1 - k0);
            named_barrier_128(1);
            const int seen = *sm.flag;
            named_barrier_128(1);              // everyone has read the flag before it is reused
            if (seen < 0) break;               // the same value in all 128 threads
            const bool last = seen == full_count;
            if (!last) continue;
            __threadfence();
            // The block's epilogue: a thread takes (token, 4 channels) pieces -- a warp covers the 128
            // channels of one token with 16-byte loads -- and requests eight pieces before it uses
            // the first, so the conversion costs a few L2 round trips, not one per token.
            const int pieces = p.M * 32;
            float* base = p.acc + static_cast<int64_t>(block) * 128;
            const int64_t up_off = static_cast<int64_t>(p.blocks) * 128;
            for (int i0 = threadIdx.x; i0 < pieces; i0 += 128 * 8) {
                float4 a[8], b[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + j * 128;
                    if (i < pieces) {
                        float* src = base + static_cast<int64_t>(i >> 5) * p.acc_ld + (i & 31) * 4;
                        a[j] = __ldcg(reinterpret_cast<const float4*>(src));
                        if constexpr (kUp) b[j] = __ldcg(reinterpret_cast<const float4*>(src + up_off));
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + j * 128;
                    if (i < pieces) {
                        const int tok = i >> 5, c = (i & 31) * 4;
                        float* src = base + static_cast<int64_t>(tok) * p.acc_ld + c;
                        *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
                        float v[4] = {a[j].x, a[j].y, a[j].z, a[j].w};
                        if constexpr (kUp) {
                            *reinterpret_cast<float4*>(src + up_off) = make_float4(0.f, 0.f, 0.f, 0.f);
                            const float u[4] = {b[j].x, b[j].y, b[j].z, b[j].w};
                            const int ch = block * 128 + c;
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                // groups narrower than four channels are possible: look each up
                                const bool on = p.mask[static_cast<int64_t>(tok) * p.NG + (ch + q) / p.G] != 0;
                                v[q] = on ? silu_f(v[q]) * u[q] : 0.f;
                            }
                        }
                        uint2 packed;
                        packed.x = pack_half2<kBf16>(v[0], v[1]);
                        packed.y = pack_half2<kBf16>(v[2], v[3]);
                        *reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(tok) * p.ldo + block * 128 + c) * 2) = packed;
                    }
                }
            }
            if (threadIdx.x == 0) p.counters[block] = 0;
        }
    } else if (warp == 4) {
        // ============================ TMA producer ==================================
        if (lane == 0) {
            tma_prefetch_desc(&tmTok);
            tma_prefetch_desc(&tmW0);
            if (kUp) tma_prefetch_desc(&tmW1);
            const uint32_t tx = static_cast<uint32_t>(kSmWTile) + static_cast<uint32_t>(NT) * kSmBK * 2;
            // every weight byte is used once; the token tile, the fp32 buffer and h are what should
            // stay in L2
            const uint64_t stream_once = l2_policy_evict_first();
            const uint64_t keep = l2_policy_evict_last();
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int64_t u = u_begin; ok && u < u_end;) {
                int tile, k0, k1;
                small_part(u, u_end, KB, tile, k0, k1);
                u += k1 - k0;
                const bool second = kUp && (tile & 1);
                const CUtensorMap* tmW = second ? &tmW1 : &tmW0;
                const int wrow = (kUp ? tile >> 1 : tile) * 128;
                for (int kb = k0; kb < k1; ++kb) {
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, sm.abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = sm.ring + size_t(s) * p.stage_bytes;
                    mbar_arrive_expect_tx(&sm.full[s], tx);
                    tma_load_2d_hint(st, tmW, &sm.full[s], kb * kSmBK, wrow, stream_once);
                    tma_load_2d_hint(st + kSmWTile, &tmTok, &sm.full[s], kb * kSmBK, 0, keep);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else {
        // ============================ UMMA issuer ===================================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kBf16 ? 1 : 0, 128, NT);
            int s = 0, acc_it = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int64_t u = u_begin; ok && u < u_end; ++acc_it) {
                int tile, k0, k1;
                small_part(u, u_end, KB, tile, k0, k1);
                u += k1 - k0;
                const int ab = acc_it & 1;
                if (!mbar_wait(&sm.tempty[ab], ((acc_it >> 1) & 1) ^ 1, sm.abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d = tmem_base + static_cast<uint32_t>(ab * NT);
                for (int kb = k0; kb < k1; ++kb) {
                    if (!mbar_wait(&sm.full[s], ph, sm.abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(sm.ring + size_t(s) * p.stage_bytes);
                    const uint64_t wdesc = umma_desc_k_sw128(sa);
                    const uint64_t tdesc = umma_desc_k_sw128(sa + kSmWTile);
#pragma unroll
                    for (int k = 0; k < kSmBK / 16; ++k)
                        umma_f16_ss(d, wdesc + 2 * k, tdesc + 2 * k, idesc, (kb != k0 || k != 0) ? 1u : 0u);
                    umma_commit(&sm.empty[s]);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                if (ok) umma_commit(&sm.tfull[ab]);
            }
        }
    }
    if (*sm.abort_flag) __nanosleep(2000000);   // let copies already in flight land
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kSmTmemCols);
    }
}

// up, one CTA per 128-channel block: gate and up tiles stream side by side into two accumulators
// and the epilogue writes h directly -- no partial sums in memory.  Measured faster for the
// gate/up matrices than the unit-range split above (60 vs 74 us at H=4096, I=14336, 64 tokens):
// with [I,H] weights a k-block touches 128 rows 2*H bytes apart, and more concurrent streams of
// that pattern lowered the aggregate HBM rate instead of raising it.
template <bool kBf16>
__global__ void __launch_bounds__(kSmThreads, 1)
ffn_small_up_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmWg,
                    const __grid_constant__ CUtensorMap tmWu, const SmallParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const SmallSmem sm = small_smem(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 4 && lane == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.tfull[b], 1);
            mbar_init(&sm.tempty[b], 128);
        }
        *sm.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(sm.tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *sm.tmem_slot;
    const int NT = p.NT, KB = p.KB;

    if (warp < 4) {
        int acc_it = 0;
        for (int item = blockIdx.x; item < p.blocks; item += gridDim.x, ++acc_it) {
            const int ab = acc_it & 1;
            const bool got = mbar_wait(&sm.tfull[ab], (acc_it >> 1) & 1, sm.abort_flag, p.status,
                                       DPK_DEV_TIMEOUT_TMEM_FULL);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after_sync();
            const int ch = item * 128 + warp * 32 + lane;       // intermediate channel of this thread
            const int g = ch / p.G;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) +
                                   static_cast<uint32_t>(ab * 2 * NT);
            for (int c = 0; c < NT; c += 16) {
                uint32_t gate[16], up[16];
                uint8_t on[16];
                tmem_ld_32x32b_x16(taddr + c, gate);
                tmem_ld_32x32b_x16(taddr + NT + c, up);
#pragma unroll
                for (int t = 0; t < 16; ++t)
                    on[t] = c + t < p.M ? p.mask[static_cast<int64_t>(c + t) * p.NG + g] : 0;
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 16; ++t)
                    if (c + t < p.M)
                        store_half<kBf16>(p.out + (static_cast<int64_t>(c + t) * p.ldo + ch) * 2,
                                          on[t] ? silu_f(__uint_as_float(gate[t])) * __uint_as_float(up[t]) : 0.f);
            }
            tc_fence_before_sync();
            mbar_arrive(&sm.tempty[ab]);
        }
    } else if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&tmX);
            tma_prefetch_desc(&tmWg);
            tma_prefetch_desc(&tmWu);
            const uint32_t tx = 2u * kSmWTile + static_cast<uint32_t>(NT) * kSmBK * 2;
            const uint64_t stream_once = l2_policy_evict_first();
            const uint64_t keep = l2_policy_evict_last();
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.blocks; item += gridDim.x) {
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, sm.abort_flag, p.status, DPK_DEV_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = sm.ring + size_t(s) * p.stage_bytes;
                    mbar_arrive_expect_tx(&sm.full[s], tx);
                    tma_load_2d_hint(st, &tmWg, &sm.full[s], kb * kSmBK, item * 128, stream_once);
                    tma_load_2d_hint(st + kSmWTile, &tmWu, &sm.full[s], kb * kSmBK, item * 128, stream_once);
                    tma_load_2d_hint(st + 2 * kSmWTile, &tmX, &sm.full[s], kb * kSmBK, 0, keep);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(kBf16 ? 1 : 0, 128, NT);
            int s = 0, acc_it = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < p.blocks; item += gridDim.x, ++acc_it) {
                const int ab = acc_it & 1;
                if (!mbar_wait(&sm.tempty[ab], ((acc_it >> 1) & 1) ^ 1, sm.abort_flag, p.status,
                               DPK_DEV_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after_sync();
                const uint32_t d_gate = tmem_base + static_cast<uint32_t>(ab * 2 * NT);
                const uint32_t d_up = d_gate + static_cast<uint32_t>(NT);
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(&sm.full[s], ph, sm.abort_flag, p.status, DPK_DEV_TIMEOUT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(sm.ring + size_t(s) * p.stage_bytes);
                    const uint64_t gdesc = umma_desc_k_sw128(sa);
                    const uint64_t udesc = umma_desc_k_sw128(sa + kSmWTile);
                    const uint64_t xdesc = umma_desc_k_sw128(sa + 2 * kSmWTile);
#pragma unroll
                    for (int k = 0; k < kSmBK / 16; ++k) {
                        const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
                        umma_f16_ss(d_gate, gdesc + 2 * k, xdesc + 2 * k, idesc, accum);
                        umma_f16_ss(d_up, udesc + 2 * k, xdesc + 2 * k, idesc, accum);
                    }
                    umma_commit(&sm.empty[s]);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                if (ok) umma_commit(&sm.tfull[ab]);
            }
        }
    }
    if (*sm.abort_flag) __nanosleep(2000000);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
static size_t small_counter_bytes(int H, int I) { return align256(sizeof(int) * static_cast<size_t>((H > I ? H : I) / 128)); }
static size_t small_acc_ld(int H, int I) { return static_cast<size_t>(2 * I > H ? 2 * I : H); }

template <bool kBf16, bool kUp>
static int small_launch(const CUtensorMap& tmTok, const CUtensorMap& tmW0, const CUtensorMap& tmW1,
                        const SmallParams& p, int grid, cudaStream_t s)
{
    DPK_CUDA(cudaFuncSetAttribute(ffn_small_kernel<kBf16, kUp>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kSmSmemBytes));
    ffn_small_kernel<kBf16, kUp><<<grid, kSmThreads, kSmSmemBytes, s>>>(tmTok, tmW0, tmW1, p);
    DPK_CUDA(cudaGetLastError());
    return DPK_OK;
}

}  // namespace dpk

using namespace dpk;

extern "C" size_t dpk_ffn_small_workspace_bytes(int64_t M, int H, int I)
{
    if (M <= 0 || M > 128 || H <= 0 || I <= 0) return 0;
    // counters and accumulator first, at offsets that do not depend on M: they are the part
    // that has to stay zero between calls of different sizes
    return small_counter_bytes(H, I) + align256(128 * small_acc_ld(H, I) * sizeof(float)) +
           align256(static_cast<size_t>(M) * I * 2);
}

extern "C" int dpk_ffn_swiglu_small(const void* x, const void* Wg, const void* Wu, const void* Wd,
                                    const uint8_t* mask, void* y, int64_t M, int H, int I, int NG,
                                    int dtype, void* workspace, size_t workspace_bytes, void* stream)
{
    DPK_REQUIRE(x && Wg && Wu && Wd && mask && y, "NULL tensor");
    DPK_REQUIRE(dtype == DPK_F16 || dtype == DPK_BF16, "dtype must be DPK_F16 or DPK_BF16");
    DPK_REQUIRE(M >= 0 && M <= 128, "this entry point takes at most 128 tokens, got %lld", (long long)M);
    DPK_REQUIRE(H > 0 && I > 0 && NG > 0 && I % NG == 0, "bad shape H=%d I=%d NG=%d", H, I, NG);
    if (H % 128 != 0 || I % 128 != 0)
        return fail(DPK_ERR_UNSUPPORTED, "H=%d and I=%d must be multiples of 128 for the small-M kernels", H, I);
    DPK_REQUIRE(aligned16(x) && aligned16(Wg) && aligned16(Wu) && aligned16(Wd) && aligned16(y),
                "tensors must be 16-byte aligned");
    if (M == 0) return DPK_OK;
    const size_t need = dpk_ffn_small_workspace_bytes(M, H, I);
    DPK_REQUIRE(workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
                "a 256-byte aligned workspace of %zu bytes is needed", need);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int* counters = reinterpret_cast<int*>(ws);
    float* acc = reinterpret_cast<float*>(ws + small_counter_bytes(H, I));
    uint8_t* h = reinterpret_cast<uint8_t*>(acc) + align256(128 * small_acc_ld(H, I) * sizeof(float));

    SmallParams p{};
    p.mask = mask;
    p.acc = acc;
    p.counters = counters;
    p.acc_ld = static_cast<int64_t>(small_acc_ld(H, I));
    p.M = static_cast<int>(M);
    p.NG = NG;
    p.G = I / NG;
    p.NT = static_cast<int>((M + 15) / 16 * 16);
    p.stage_bytes = (kSmWTile + p.NT * kSmBK * 2 + 1023) / 1024 * 1024;
    p.stages = kSmRing / p.stage_bytes;
    if (p.stages > kSmMaxStages) p.stages = kSmMaxStages;
    p.status = device_status_ptr();
    if (!p.status) return fail(DPK_ERR_CUDA, "no status word on this device");
    const int sms = sm_count();
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    CUtensorMap tmX, tmWg, tmWu, tmH, tmWd;
    int rc = make_tmap_2d_sw128(&tmX, x, (uint64_t)H, (uint64_t)M, (uint64_t)H, kSmBK, p.NT);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmWg, Wg, (uint64_t)H, (uint64_t)I, (uint64_t)H, kSmBK, 128);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmWu, Wu, (uint64_t)H, (uint64_t)I, (uint64_t)H, kSmBK, 128);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmH, h, (uint64_t)I, (uint64_t)M, (uint64_t)I, kSmBK, p.NT);
    if (rc) return rc;
    rc = make_tmap_2d_sw128(&tmWd, Wd, (uint64_t)I, (uint64_t)H, (uint64_t)I, kSmBK, 128);
    if (rc) return rc;

    SmallParams up = p;
    up.out = h;
    up.ldo = I;
    up.KB = H / kSmBK;
    up.blocks = I / 128;
    up.tiles = 2 * up.blocks;
    up.stage_bytes = (2 * kSmWTile + p.NT * kSmBK * 2 + 1023) / 1024 * 1024;
    up.stages = kSmRing / up.stage_bytes;
    if (up.stages > kSmMaxStages) up.stages = kSmMaxStages;
    int grid = up.blocks < sms ? up.blocks : sms;
    if (dtype == DPK_BF16) {
        DPK_CUDA(cudaFuncSetAttribute(ffn_small_up_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmSmemBytes));
        ffn_small_up_kernel<true><<<grid, kSmThreads, kSmSmemBytes, s>>>(tmX, tmWg, tmWu, up);
    } else {
        DPK_CUDA(cudaFuncSetAttribute(ffn_small_up_kernel<false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmSmemBytes));
        ffn_small_up_kernel<false><<<grid, kSmThreads, kSmSmemBytes, s>>>(tmX, tmWg, tmWu, up);
    }
    DPK_CUDA(cudaGetLastError());

    SmallParams dn = p;
    dn.out = static_cast<uint8_t*>(y);
    dn.ldo = H;
    dn.KB = I / kSmBK;
    dn.blocks = H / 128;
    dn.tiles = dn.blocks;
    const int64_t units = static_cast<int64_t>(dn.tiles) * dn.KB;
    grid = units < sms ? static_cast<int>(units) : sms;
    return dtype == DPK_BF16 ? small_launch<true, false>(tmH, tmWd, tmWd, dn, grid, s)
                             : small_launch<false, false>(tmH, tmWd, tmWd, dn, grid, s);
}
