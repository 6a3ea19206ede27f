// Row schedule: row ids ordered by descending nonzero count (stable), built on the device.
//
// SpMM has to add a row's nonzeros one after another (the result must equal a sequential
// sum), so a long row cannot be split between workers.  Balance therefore comes from
// ORDER: rows are handed to thread blocks heaviest first, and the hardware block
// scheduler, which starts blocks in index order as SMs free up, turns that into
// longest-job-first scheduling.  Neighbouring rows in the order also have similar
// lengths, which keeps the row groups sharing a warp in step.
#include <cub/device/device_radix_sort.cuh>

#include <vector>

#include "common.cuh"
#include "schedule.cuh"

namespace {

__global__ void degree_keys_kernel(const int32_t* __restrict__ indptr, int64_t n_rows,
                                   uint32_t* __restrict__ keys, int32_t* __restrict__ rows) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_rows) {
        keys[r] = (uint32_t)(indptr[r + 1] - indptr[r]);
        rows[r] = (int32_t)r;
    }
}

__global__ void row_extents_kernel(const int32_t* __restrict__ indptr, const int32_t* __restrict__ order,
                                   int64_t n_rows, int2* __restrict__ extent) {
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p < n_rows) {
        const int32_t r = order[p];
        const int32_t start = indptr[r];
        extent[p] = make_int2(start, indptr[r + 1] - start);
    }
}

}  // namespace

extern "C" {

int fg_row_schedule_create(const int32_t* d_indptr, int64_t n_rows, int32_t long_row_threshold,
                           void* stream, fg_row_schedule** out_schedule) {
    if (!out_schedule) return fg::fail(FG_ERR_INVALID_ARGUMENT, "out_schedule is NULL");
    *out_schedule = nullptr;
    if (n_rows < 0 || n_rows > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "n_rows=%lld out of range", (long long)n_rows);
    if (n_rows > 0 && !d_indptr) return fg::fail(FG_ERR_INVALID_ARGUMENT, "d_indptr is NULL");
    if (long_row_threshold == INT32_MIN)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "long_row_threshold out of range");
    // a negative threshold fixes |threshold| and asks for the 8-warp form of the heavy-row kernel
    const bool fixed_wide = long_row_threshold < 0;
    if (fixed_wide) long_row_threshold = -long_row_threshold;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    fg_row_schedule* sch = new fg_row_schedule();
    sch->n_rows = n_rows;
    if (n_rows == 0) {
        *out_schedule = sch;
        return FG_OK;
    }
    uint32_t *keys_in = nullptr, *keys_out = nullptr;
    int32_t* rows_in = nullptr;
    std::vector<uint32_t> h_keys;
    void* temp = nullptr;
    size_t temp_bytes = 0;
    int rc = FG_OK;
    auto cleanup = [&]() {
        cudaFree(keys_in);
        cudaFree(keys_out);
        cudaFree(rows_in);
        cudaFree(temp);
    };
#define FG_TRY_OR_CLEAN(expr)                                                              \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess) {                                                          \
            rc = fg::fail(e__ == cudaErrorMemoryAllocation ? FG_ERR_OUT_OF_MEMORY          \
                                                           : FG_ERR_CUDA,                  \
                          "%s failed: %s", #expr, cudaGetErrorString(e__));                \
            cleanup();                                                                     \
            cudaFree(sch->d_order);                                                        \
            cudaFree(sch->d_extent);                                                       \
            delete sch;                                                                    \
            return rc;                                                                     \
        }                                                                                  \
    } while (0)
    FG_TRY_OR_CLEAN(cudaMalloc(&sch->d_order, sizeof(int32_t) * n_rows));
    FG_TRY_OR_CLEAN(cudaMalloc(&sch->d_extent, sizeof(int2) * n_rows));
    FG_TRY_OR_CLEAN(cudaMalloc(&keys_in, sizeof(uint32_t) * n_rows));
    FG_TRY_OR_CLEAN(cudaMalloc(&keys_out, sizeof(uint32_t) * n_rows));
    FG_TRY_OR_CLEAN(cudaMalloc(&rows_in, sizeof(int32_t) * n_rows));
    const int threads = 256;
    const unsigned blocks = (unsigned)((n_rows + threads - 1) / threads);
    degree_keys_kernel<<<blocks, threads, 0, s>>>(d_indptr, n_rows, keys_in, rows_in);
    FG_TRY_OR_CLEAN(cudaGetLastError());
    // LSD radix sort is stable: equal degrees keep ascending row order.
    FG_TRY_OR_CLEAN(cub::DeviceRadixSort::SortPairsDescending(
        nullptr, temp_bytes, keys_in, keys_out, rows_in, sch->d_order, (int)n_rows, 0, 32, s));
    FG_TRY_OR_CLEAN(cudaMalloc(&temp, temp_bytes ? temp_bytes : 1));
    FG_TRY_OR_CLEAN(cub::DeviceRadixSort::SortPairsDescending(
        temp, temp_bytes, keys_in, keys_out, rows_in, sch->d_order, (int)n_rows, 0, 32, s));
    row_extents_kernel<<<blocks, threads, 0, s>>>(d_indptr, sch->d_order, n_rows, sch->d_extent);
    FG_TRY_OR_CLEAN(cudaGetLastError());
    // the sorted nonzero counts come back once; the split statistics are computed on the host
    h_keys.resize((size_t)n_rows);
    FG_TRY_OR_CLEAN(cudaMemcpyAsync(h_keys.data(), keys_out, sizeof(uint32_t) * n_rows,
                                    cudaMemcpyDeviceToHost, s));
    FG_TRY_OR_CLEAN(cudaStreamSynchronize(s));
#undef FG_TRY_OR_CLEAN
    cleanup();
    sch->max_row_nnz = h_keys[0];
    sch->fixed_threshold = long_row_threshold;
    sch->fixed_wide = fixed_wide;
    int level = fg::kSplitLevels - 1;
    int64_t running = 0;
    for (int64_t i = 0; i < n_rows; ++i) {  // descending counts: thresholds are crossed downwards
        const int64_t k = h_keys[(size_t)i];
        while (level >= 0 && k < fg::split_threshold(level)) {
            sch->rows_at_least[level] = i;
            sch->nnz_at_least[level] = running;
            --level;
        }
        if (long_row_threshold > 0 && k >= long_row_threshold) {
            sch->fixed_rows = i + 1;
            sch->fixed_nnz = running + k;
            if (k >= fg::kFixedHeavyFactor * long_row_threshold) {
                sch->fixed_heavy_rows = i + 1;
                sch->fixed_heavy_nnz = running + k;
            }
        }
        running += k;
    }
    for (; level >= 0; --level) {
        sch->rows_at_least[level] = n_rows;
        sch->nnz_at_least[level] = running;
    }
    sch->nnz = running;
    *out_schedule = sch;
    return FG_OK;
}

const int32_t* fg_row_schedule_order(const fg_row_schedule* schedule) {
    return schedule ? schedule->d_order : nullptr;
}

int64_t fg_row_schedule_num_rows(const fg_row_schedule* schedule) {
    return schedule ? schedule->n_rows : 0;
}

int64_t fg_row_schedule_rows_at_least(const fg_row_schedule* schedule, int64_t min_nnz) {
    if (!schedule) return 0;
    if (schedule->fixed_threshold > 0 && min_nnz == schedule->fixed_threshold) return schedule->fixed_rows;
    for (int level = 0; level < fg::kSplitLevels; ++level)
        if (fg::split_threshold(level) == min_nnz) return schedule->rows_at_least[level];
    return -1;
}

void fg_row_schedule_destroy(fg_row_schedule* schedule) {
    if (!schedule) return;
    cudaFree(schedule->d_order);
    cudaFree(schedule->d_extent);
    delete schedule;
}

}  // extern "C"
