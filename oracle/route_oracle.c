/*
 * CPU oracle for the routing layout.  TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped library links or loads this file.
 *
 * Plain-C restatement of the integer part of the hot path:
 *
 *   - oracle_topk_mask     : per-token top-k over fp32 router logits -> 0/1 mask.
 *                            The reference has no top-k router (its kernels take a
 *                            ready Boolean mask, DynamicPruningKernels/README.md:35);
 *                            the benchmark defines the mask this way.  Ties go to the
 *                            lower group index.
 *   - oracle_route_compact : the routing layout the reference derives with
 *                            torch.sort(mask, dim=0, descending=True)
 *                            (DynamicPruningKernels/python/gemm_mn/jit.py:410-415),
 *                            with the stable order fixed: per group column the
 *                            active rows ascending, then the inactive rows ascending.
 *   - oracle_row_bits      : per-row packed group bits and the per-window OR that
 *                            the reduction-width GEMM uses to skip whole windows.
 *
 * Parity status: pinned through tests/test_oracle_golden.py, which compares this
 * file's output with torch.sort(stable=True) results stored in tests/golden/.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oracle_topk_mask(const float *logits, int64_t rows, int ng, int keep, uint8_t *mask)
{
    if (keep < 0 || keep > ng) return 1;
    for (int64_t r = 0; r < rows; ++r) {
        const float *l = logits + r * ng;
        uint8_t *m = mask + r * ng;
        for (int g = 0; g < ng; ++g) {
            /* rank of g = number of groups that beat it (strictly larger, or equal
             * with a lower index) */
            int rank = 0;
            for (int h = 0; h < ng; ++h)
                rank += (l[h] > l[g]) || (l[h] == l[g] && h < g);
            m[g] = (uint8_t)(rank < keep);
        }
    }
    return 0;
}

int oracle_route_compact(const uint8_t *mask, int64_t m, int ng, uint8_t *sorted_mask,
                         int64_t *sorted_indices, int32_t *counts)
{
    for (int g = 0; g < ng; ++g) {
        int64_t c = 0;
        for (int64_t r = 0; r < m; ++r) c += mask[r * ng + g] != 0;
        counts[g] = (int32_t)c;
        int64_t a = 0, i = c;
        for (int64_t r = 0; r < m; ++r) {
            if (mask[r * ng + g]) sorted_indices[(a++) * ng + g] = r;
            else                  sorted_indices[(i++) * ng + g] = r;
        }
        for (int64_t r = 0; r < m; ++r) sorted_mask[r * ng + g] = (uint8_t)(r < c);
    }
    return 0;
}

int oracle_row_bits(const uint8_t *mask, int64_t m, int ng, int window, uint32_t *row_bits,
                    uint32_t *win_bits)
{
    int words = (ng + 31) / 32;
    int64_t nwin = (m + window - 1) / window;
    memset(win_bits, 0, (size_t)(nwin * words) * sizeof(uint32_t));
    for (int64_t r = 0; r < m; ++r) {
        for (int w = 0; w < words; ++w) {
            uint32_t bits = 0;
            for (int b = 0; b < 32 && w * 32 + b < ng; ++b)
                if (mask[r * ng + w * 32 + b]) bits |= 1u << b;
            row_bits[r * words + w] = bits;
            win_bits[(r / window) * words + w] |= bits;
        }
    }
    return 0;
}
