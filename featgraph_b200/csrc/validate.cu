// Range and ordering checks for adjacency arrays, run once when an adjacency is uploaded.
// Each kernel ORs violation bits into one device word; nothing is dereferenced through an
// unchecked index, so a bad adjacency is reported instead of faulting later.
#include "common.cuh"

namespace {

enum : uint32_t {
    kBadStart = 1u,      // indptr[0] != 0
    kBadEnd = 2u,        // indptr[n_rows] != nnz
    kNotMonotone = 4u,   // indptr decreases
    kBadColumn = 8u,     // column id outside [0, n_cols)
    kBadRow = 16u,       // row id outside [0, n_rows)
    kRowsUnsorted = 32u  // COO row ids decrease somewhere (informational)
};

__global__ void check_indptr_kernel(const int32_t* __restrict__ indptr, int64_t n_rows, int64_t nnz,
                                    uint32_t* flags) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t f = 0;
    if (i == 0) {
        if (indptr[0] != 0) f |= kBadStart;
        if ((int64_t)indptr[n_rows] != nnz) f |= kBadEnd;
    }
    if (i < n_rows && indptr[i + 1] < indptr[i]) f |= kNotMonotone;
    if (f) atomicOr(flags, f);
}

__global__ void check_range_kernel(const int32_t* __restrict__ ids, int64_t count, int64_t bound,
                                   uint32_t bit, bool want_sorted, uint32_t* flags) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    uint32_t f = 0;
    const int32_t v = ids[i];
    if (v < 0 || (int64_t)v >= bound) f |= bit;
    if (want_sorted && i + 1 < count && ids[i + 1] < v) f |= kRowsUnsorted;
    if (f) atomicOr(flags, f);
}

int run_checks(const int32_t* indptr, const int32_t* rows, const int32_t* cols, int64_t n_rows,
               int64_t n_cols, int64_t nnz, uint32_t* host_flags, cudaStream_t s) {
    uint32_t* d_flags = nullptr;
    FG_CUDA_TRY(cudaMalloc(&d_flags, sizeof(uint32_t)));
    int rc = FG_OK;
    cudaError_t e = cudaMemsetAsync(d_flags, 0, sizeof(uint32_t), s);
    const int threads = 256;
    if (e == cudaSuccess && indptr) {
        const unsigned blocks = (unsigned)((n_rows + threads) / threads);
        check_indptr_kernel<<<blocks, threads, 0, s>>>(indptr, n_rows, nnz, d_flags);
    }
    if (e == cudaSuccess && nnz > 0) {
        const unsigned blocks = (unsigned)((nnz + threads - 1) / threads);
        if (rows) check_range_kernel<<<blocks, threads, 0, s>>>(rows, nnz, n_rows, kBadRow, true, d_flags);
        if (cols) check_range_kernel<<<blocks, threads, 0, s>>>(cols, nnz, n_cols, kBadColumn, false, d_flags);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(host_flags, d_flags, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) rc = fg::fail(FG_ERR_CUDA, "adjacency check failed: %s", cudaGetErrorString(e));
    cudaFree(d_flags);
    return rc;
}

}  // namespace

extern "C" {

int fg_csr_validate(const int32_t* d_indptr, const int32_t* d_indices, int64_t n_rows,
                    int64_t n_cols, int64_t nnz, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || n_rows > INT32_MAX || nnz > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes");
    if (!d_indptr || (nnz > 0 && !d_indices)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array");
    uint32_t flags = 0;
    int rc = run_checks(d_indptr, nullptr, d_indices, n_rows, n_cols, nnz, &flags,
                        static_cast<cudaStream_t>(stream));
    if (rc != FG_OK) return rc;
    if (flags & kBadStart) return fg::fail(FG_ERR_BAD_INDEX, "indptr[0] is not 0");
    if (flags & kBadEnd) return fg::fail(FG_ERR_BAD_INDEX, "indptr[n_rows] does not equal nnz");
    if (flags & kNotMonotone) return fg::fail(FG_ERR_BAD_INDEX, "indptr is not non-decreasing");
    if (flags & kBadColumn) return fg::fail(FG_ERR_BAD_INDEX, "a column index is outside [0, n_cols)");
    return FG_OK;
}

int fg_coo_validate(const int32_t* d_row, const int32_t* d_col, int64_t n_rows, int64_t n_cols,
                    int64_t nnz, int32_t* rows_sorted, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0) return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes");
    if (nnz > 0 && (!d_row || !d_col)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array");
    uint32_t flags = 0;
    int rc = run_checks(nullptr, d_row, d_col, n_rows, n_cols, nnz, &flags,
                        static_cast<cudaStream_t>(stream));
    if (rc != FG_OK) return rc;
    if (rows_sorted) *rows_sorted = (flags & kRowsUnsorted) ? 0 : 1;
    if (flags & kBadRow) return fg::fail(FG_ERR_BAD_INDEX, "a row index is outside [0, n_rows)");
    if (flags & kBadColumn) return fg::fail(FG_ERR_BAD_INDEX, "a column index is outside [0, n_cols)");
    return FG_OK;
}

}  // extern "C"
