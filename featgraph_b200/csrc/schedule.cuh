// Row schedule object shared by schedule.cu (which builds it) and spmm.cu (which reads it).
#pragma once
#include <cstdint>

#include <cuda_runtime.h>

namespace fg {
constexpr int kSplitLevels = 16;  // candidate long-row thresholds 64, 128, ..., 2^21
inline int64_t split_threshold(int level) { return (int64_t)64 << level; }
constexpr int64_t kFixedHeavyFactor = 16;
}  // namespace fg

struct fg_row_schedule {
    int32_t* d_order = nullptr;  // row ids, nonzero count descending, ties in row order
    // (first nonzero, nonzero count) of row d_order[p], at position p: a kernel that walks the order reads
    // a row's extent with one coalesced load instead of two dependent ones through the row id
    int2* d_extent = nullptr;
    int64_t n_rows = 0;
    int64_t nnz = 0;
    int64_t max_row_nnz = 0;
    // Rows with at least threshold nonzeros ("long" rows) sit at the front of d_order.  For every
    // candidate threshold: how many rows that is and how many nonzeros they hold.
    int64_t rows_at_least[fg::kSplitLevels] = {0};
    int64_t nnz_at_least[fg::kSplitLevels] = {0};
    // A caller-fixed threshold (0 = let each launch choose among the candidates): rows with at least
    // fixed_threshold nonzeros are long, those with at least kFixedHeavyFactor times as many are heavy.
    int64_t fixed_threshold = 0;
    int64_t fixed_rows = 0;
    int64_t fixed_nnz = 0;
    int64_t fixed_heavy_rows = 0;
    int64_t fixed_heavy_nnz = 0;
    bool fixed_wide = false;  // heavy rows with 8 warps per block instead of 4
};
