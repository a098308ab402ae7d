// Definitions shared by the single-CTA and the CTA-pair output-width routed GEMM kernels:
// tile geometry, launch parameters, activation, and the tile order.
#pragma once

#include "dpk_host.h"
#include "dpk_sm100.cuh"

namespace dpk {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kAStageBytes = kBM * kBK * 2;         // 16 KiB of gathered token rows
constexpr int kRingBytes = 4 * (kAStageBytes + 256 * kBK * 2);   // 192 KiB of operand ring
constexpr int kMaxStages = 12;
constexpr int kMnThreads = 320;
constexpr int kMaxGroups = 2048;
constexpr int kGatherLag = 2;                       // cp.async groups kept in flight
constexpr int kTmemCols = 512;

struct MnParams {
    const uint8_t* A;       // [M, lda] half
    uint8_t* D;             // [M, ldd] half
    const int64_t* sidx;    // [M, NG]
    const int32_t* counts;  // [NG]
    int64_t lda, ldd;       // elements
    int64_t M;
    int K, NG, G;
    int BN;                 // output channels per tile and weight
    int n_chunks;           // G / BN
    int fused;              // second weight present: silu(gate)*up
    int act;
    int rows_per_block;     // row tiles of one group scheduled back to back (L2 blocking of A)
    int halves;             // 128-row halves per tile: 2 when two accumulators of <= 128 columns
                            // fit, so that one weight tile feeds 256 token rows
    int stages;             // ring depth: kRingBytes / stage_bytes, at most kMaxStages
    int stage_bytes;        // kAStageBytes + (UMMA N) * 128
    int gather4;            // CTA-pair kernel: token rows by TMA tile::gather4 (one warp issues 32
                            // four-row copies per stage) instead of 16-byte cp.async by four warps
    int* status;
};

constexpr size_t kMnSmemBytes = 1024 /*alignment slack*/ + size_t(kRingBytes) +
                                (2 * kMaxStages + 4) * sizeof(uint64_t) + 16 +
                                (kMaxGroups + 1) * sizeof(int);

__device__ __forceinline__ float apply_act(float x, int act)
{
    if (act == DPK_ACT_RELU) return fmaxf(x, 0.f);
    if (act == DPK_ACT_SILU) return silu_f(x);
    return x;
}

// Tile order.  Row tile i of every group covers roughly the same token range (the routing
// keeps a similar fraction of every stretch of tokens), so the schedule walks blocks of R row
// tiles and, inside a block, the groups: the token rows a block gathers stay L2-resident
// while all groups use them, and one group's weight slab is shared by the R*n_chunks tiles
// that run back to back.  Row tiles up to the smallest group's count form this regular part
// (decoded arithmetically); the few tiles beyond it are appended group by group.
struct TileMap {
    const int* ragged_prefix;   // [NG + 1] tiles of group g beyond the regular part
    int ng, n_chunks, rows_per_block, tmin, regular_total, total;

    __device__ __forceinline__ void decode(int tile, int& g, int& mtile, int& nchunk) const
    {
        if (tile < regular_total) {
            const int per_block = rows_per_block * ng * n_chunks;
            const int mb = tile / per_block;
            const int off = tile - mb * per_block;
            const int rows = min(rows_per_block, tmin - mb * rows_per_block);
            const int per_group = rows * n_chunks;
            g = off / per_group;
            const int rem = off - g * per_group;
            mtile = mb * rows_per_block + rem / n_chunks;
            nchunk = rem % n_chunks;
        } else {
            const int u0 = tile - regular_total;
            int lo = 0, hi = ng;   // invariant: ragged_prefix[lo] <= u0 < ragged_prefix[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (ragged_prefix[mid] <= u0) lo = mid; else hi = mid;
            }
            g = lo;
            const int u = u0 - ragged_prefix[g];
            mtile = tmin + u / n_chunks;
            nchunk = u % n_chunks;
        }
    }
};

// CTA-pair (cta_group::2) variant, dpk_gemm_mn_pair.cu.  Returns DPK_ERR_UNSUPPORTED when the
// shape is not eligible.
int gemm_mn_pair_launch(const CUtensorMap& tmW, const CUtensorMap& tmW2, const CUtensorMap& tmA,
                        MnParams p, int dtype, cudaStream_t stream);

}  // namespace dpk
