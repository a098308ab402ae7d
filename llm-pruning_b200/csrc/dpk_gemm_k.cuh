// Definitions shared by the single-CTA and the CTA-pair reduction-width routed GEMM kernels.
#pragma once

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
constexpr int kMaxPeers = 8;

struct KParams {
    uint8_t* D;              // [M, ldd] half
    const uint8_t* R;        // optional [M, ldr] half added to the result before the one rounding
    int64_t ldr;             // (the residual of a transformer sub-block); may alias D
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
    int ksplit;              // splits of the group range (1 = none); > 1 needs acc32
    float* acc32;            // [M, N] fp32, zero-filled: partial sums of the splits land here
    int stages;              // ring depth: kRingBytes / stage_bytes, at most kMaxStages
    int stage_bytes;         // kAStageBytes + BN * 128
    int* status;
    // Output scattered to the owners of the token windows (tensor parallel; 0 = plain D):
    // rows [o*rows_per_owner, (o+1)*rows_per_owner) go to slab `my_rank` of peer[o], each slab
    // [rows_per_owner, ldd].
    int world, my_rank;
    int64_t rows_per_owner;
    uint8_t* peer[kMaxPeers];
};

// Eight consecutive outputs of a row: accumulator values (+ residual), rounded once.
template <bool kBf16>
__device__ __forceinline__ uint4 pack8_plus_residual(const uint32_t* v, const uint8_t* res)
{
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]);
    if (res) {
        const uint4 r4 = *reinterpret_cast<const uint4*>(res);
        const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float lo, hi;
            unpack_half2<kBf16>(rw[j], lo, hi);
            f[2 * j] += lo;
            f[2 * j + 1] += hi;
        }
    }
    return make_uint4(pack_half2<kBf16>(f[0], f[1]), pack_half2<kBf16>(f[2], f[3]),
                      pack_half2<kBf16>(f[4], f[5]), pack_half2<kBf16>(f[6], f[7]));
}

constexpr size_t kKSmemBytes = 1024 + size_t(kRingBytes) +
                               (3 * kMaxStages + 4) * sizeof(uint64_t) + 16;

// CTA-pair (cta_group::2) variant, dpk_gemm_k_pair.cu: many token windows, N >= 256.
int gemm_k_pair_launch(const void* A, int64_t lda, const void* W, int64_t ldw, KParams p, int dtype,
                       cudaStream_t stream);

}  // namespace dpk
