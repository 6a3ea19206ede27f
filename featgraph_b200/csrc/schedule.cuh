// Row schedule object shared by schedule.cu (which builds it) and spmm.cu (which reads it).
#pragma once
#include <cstdint>

namespace fg {
// Rows with at least this many nonzeros are "long": they come first in the order and SpMM
// runs them with the deep gather pipeline.
constexpr uint32_t kLongRowThreshold = 1024;
}  // namespace fg

struct fg_row_schedule {
    int32_t* d_order = nullptr;  // row ids, nonzero count descending, ties in row order
    int64_t n_rows = 0;
    int64_t n_long = 0;  // the first n_long entries of d_order are long rows
    int64_t max_row_nnz = 0;
};
