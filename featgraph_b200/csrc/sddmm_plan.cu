// SDDMM over column blocks: one pass over the edge list for feature matrices larger than L2.
//
//   out[e] = sum_k src[col[e], k] * dst[row[e], k]      python/featgraph/op/vanilla_sddmm.py:47
//
// fg_sddmm_coo_f32 keeps the gathered part of src in L2 by cutting the FEATURE dimension into tiles and
// walking the whole edge list once per tile: the id arrays are streamed once per tile and out[e] is read
// and written once per tile.  Here the COLUMN range is cut instead, into num_col_partitions blocks of
// ceil(n_cols / P) columns - the column blocks of the reference's 2-D edge partitioning
// (python/featgraph/util/adj_partitioning.py:100-101), used as a traversal order - and the edges are visited
// block by block: while block k is being worked on, only rows [k*w, (k+1)*w) of src are gathered from, whole
// rows of d floats, and those stay in L2.  Every edge is visited exactly once, so its dot product is
// finished in one go: ids are read once, out[e] is written once and never read.
//
// In a row-sorted edge list whose column ids ascend within each row (CSR order) the edges of (block k,
// row r) are a contiguous run of the ORIGINAL list, so nothing is permuted: the plan is a list of batch
// descriptors (row, first edge, count <= 32) in block-major order, built once per adjacency on the
// device.  A warp takes 16 consecutive descriptors.  For one batch the 32 lanes share every edge: lane l
// holds float4 number l, l + 32, ... of the row-side row in registers (loaded together with the first
// gathers when the row changes) and gathers the same float4s of src[col[e]] - whole 128-byte lines,
// 512 contiguous bytes per load instruction - for U edges at a time; a transposed butterfly (31 shuffles
// for 32 edges) leaves lane i with edge i's dot product, which is the layout of the coalesced store.
//
// Arithmetic: FMAs within a lane, a fixed tree across the 32 lanes; within fp32 rounding of d terms of the
// sequential sum, like fg_sddmm_coo_f32 (whose tree differs, so the two agree to rounding, not bit for bit).
#include <cub/device/device_scan.cuh>

#include "common.cuh"

struct fg_sddmm_plan {
    int4* d_desc = nullptr;  // (row, first edge, count, column block) per batch, block-major
    int64_t n_batches = 0;
    int64_t n_rows = 0, n_cols = 0, nnz = 0;
    int32_t parts = 1;
};

namespace {

constexpr int kThreads = 256;
constexpr int kBatchesPerWarp = 16;

// edges whose gathers are in flight together, per float4 count NV = 1..4 (16 loads per lane where registers allow)
#ifndef FG_CB_U1
#define FG_CB_U1 16
#endif
#ifndef FG_CB_U2
#define FG_CB_U2 8
#endif
#ifndef FG_CB_U3
#define FG_CB_U3 4
#endif
#ifndef FG_CB_U4
#define FG_CB_U4 4
#endif

__device__ __forceinline__ float dot4(float acc, const float4& a, const float4& b) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

struct PlanArgs {
    const int4* desc;
    int64_t n_batches;
    const int32_t* col;
    const float* src;
    const float* dst;
    float* out;
    int32_t ld_src, ld_dst;  // row strides in floats
    int32_t width;           // feature columns (<= 128 * NV)
    int32_t accumulate;
};

// NV float4 per lane and edge (d <= 128 * NV), U edges' gathers in flight (U * NV 128-bit loads per lane).
// MASKED: d < 128 * NV (float4s beyond the row's end are read from the lane's first one and zeroed).
template <int NV, int U, bool MASKED>
__global__ void __launch_bounds__(kThreads, 2) sddmm_colblock_kernel(const PlanArgs a) {
    static_assert(32 % U == 0, "U must divide 32");
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t first = warp * kBatchesPerWarp;
    if (first >= a.n_batches) return;  // whole warp

    const int lane_col = (!MASKED || lane * 4 < a.width) ? lane * 4 : 0;
    int moff[NV];
    bool ok[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ok[i] = !MASKED || (lane + i * 32) * 4 < a.width;
        moff[i] = ok[i] ? (lane + i * 32) * 4 - lane_col : 0;
    }
    auto off = [&](int i) { return MASKED ? moff[i] : i * 128; };
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint64_t keep_policy = fg::l2_keep_policy();
    const float* sbase = a.src + lane_col;

    // this warp's descriptors: lane b holds batch first + b (count 0 past the end of the list)
    int4 my = make_int4(0, 0, 0, 0);
    if (lane < kBatchesPerWarp && first + lane < a.n_batches) my = fg::ld_stream(a.desc + first + lane);

    float4 dcache[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) dcache[i] = zero4;
    int cur_row = -1;

    // column ids one batch ahead of their use (a DRAM stream)
    int c_next = 0;
    {
        const int start0 = __shfl_sync(0xffffffffu, my.y, 0), len0 = __shfl_sync(0xffffffffu, my.z, 0);
        if (lane < len0) c_next = fg::ld_stream(a.col + start0 + lane);
    }
#pragma unroll 1
    for (int b = 0; b < kBatchesPerWarp; ++b) {
        const int row = __shfl_sync(0xffffffffu, my.x, b);
        const int start = __shfl_sync(0xffffffffu, my.y, b);
        const int len = __shfl_sync(0xffffffffu, my.z, b);
        if (len == 0) break;  // warp-uniform: the end of the list
        const int c_l = c_next;  // lanes >= len hold column 0: a valid row, its product is never stored
        c_next = 0;
        if (b + 1 < kBatchesPerWarp) {
            const int start1 = __shfl_sync(0xffffffffu, my.y, b + 1), len1 = __shfl_sync(0xffffffffu, my.z, b + 1);
            if (lane < len1) c_next = fg::ld_stream(a.col + start1 + lane);
        }
        float prev = 0.f;
        if (a.accumulate && lane < len) prev = fg::ld_stream(a.out + start + lane);
        const bool new_row = row != cur_row;  // warp-uniform
        cur_row = row;

        float r[32 / U];  // one partly reduced value per chunk of U edges
#pragma unroll
        for (int s = 0; s < 32; s += U) {
            if (s >= len) {  // warp-uniform: nothing left in this batch
                r[s / U] = 0.f;
                continue;
            }
            int c[U];
            float pc[U];
            float4 xs[U][NV];
#pragma unroll
            for (int u = 0; u < U; ++u) c[u] = __shfl_sync(0xffffffffu, c_l, s + u);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* ps = sbase + (int64_t)c[u] * a.ld_src;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    xs[u][i] = fg::ldg4_keep(ps + off(i), keep_policy);
                    if (MASKED && !ok[i]) xs[u][i] = zero4;
                }
            }
            if (s == 0 && new_row) {
                // the row-side row rides along with the first gathers of its first batch: read once per
                // (row, column block), streamed (it is not gathered from again soon)
                const float* pd = a.dst + (int64_t)row * a.ld_dst + lane_col;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    dcache[i] = fg::ld_stream(reinterpret_cast<const float4*>(pd + off(i)));
                    if (MASKED && !ok[i]) dcache[i] = zero4;  // 0 * 0, never 0 * (a stray Inf or NaN)
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < NV; ++i) acc = dot4(acc, xs[u][i], dcache[i]);
                pc[u] = acc;
            }
            // first log2(U) steps of the transposed butterfly, inside the chunk
#pragma unroll
            for (int o = 1; o < U; o <<= 1) {
                const bool upper = (lane & o) != 0;
#pragma unroll
                for (int i = 0; i < U / (2 * o); ++i) {
                    const float send = upper ? pc[2 * i] : pc[2 * i + 1];
                    const float keep = upper ? pc[2 * i + 1] : pc[2 * i];
                    pc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            r[s / U] = pc[0];
        }
        // remaining steps across the chunks: afterwards r[0] on lane i is edge i's total
#pragma unroll
        for (int o = U; o < 32; o <<= 1) {
            const bool upper = (lane & o) != 0;
            const int h = o / U;
#pragma unroll
            for (int i = 0; i < 32 / U / (2 * h); ++i) {
                const float send = upper ? r[2 * i] : r[2 * i + 1];
                const float keep = upper ? r[2 * i + 1] : r[2 * i];
                r[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        if (lane < len) fg::st_stream(a.out + start + lane, prev + r[0]);
    }
}

// ---------------------------------------------------------------------------------------------
// Plan construction (device, once per adjacency and partition count)
// ---------------------------------------------------------------------------------------------

// indptr from a row-sorted row array, and the order checks the plan relies on:
// flags bit 0: rows not non-decreasing; bit 1: column ids descend somewhere inside a row; bit 2: a row id
// outside [0, n_rows).
__global__ void rows_to_indptr_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                                      int64_t nnz, int64_t n_rows, int32_t* __restrict__ indptr,
                                      int32_t* __restrict__ flags) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row[e];
    const int prev = e > 0 ? row[e - 1] : -1;
    if (r < 0 || r >= n_rows) {
        atomicOr(flags, 4);
        return;
    }
    if (r < prev) atomicOr(flags, 1);
    if (r == prev && col[e] < col[e - 1]) atomicOr(flags, 2);
    for (int q = prev + 1; q <= r; ++q) indptr[q] = (int32_t)e;  // rows prev+1 .. r start here (empty ones included)
    if (e == nnz - 1)
        for (int64_t q = (int64_t)r + 1; q <= n_rows; ++q) indptr[q] = (int32_t)nnz;
}

// For row r: where each column block starts inside the row's (ascending) column ids, and how many batches
// of 32 edges each (block, row) run needs.  Layout of starts / counts: block-major, [k * n_rows + r].
__global__ void block_runs_kernel(const int32_t* __restrict__ indptr, const int32_t* __restrict__ col,
                                  int64_t n_rows, int32_t parts, int32_t block_cols,
                                  int32_t* __restrict__ starts, int32_t* __restrict__ counts) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int end = indptr[r + 1];
    int lo = indptr[r];
    for (int k = 0; k < parts; ++k) {
        // first position in [lo, end) whose column id is >= (k + 1) * block_cols
        const int64_t limit = (int64_t)(k + 1) * block_cols;
        int a = lo, b = end;
        while (a < b) {
            const int mid = a + (b - a) / 2;
            if ((int64_t)col[mid] < limit)
                a = mid + 1;
            else
                b = mid;
        }
        starts[(int64_t)k * n_rows + r] = lo;
        counts[(int64_t)k * n_rows + r] = (a - lo + 31) / 32;
        lo = a;
    }
}

__global__ void fill_descriptors_kernel(const int32_t* __restrict__ indptr, const int32_t* __restrict__ starts,
                                        const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                                        int64_t n_rows, int32_t parts, int4* __restrict__ desc) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // index into the block-major tables
    if (i >= n_rows * parts) return;
    const int k = (int)(i / n_rows);
    const int64_t r = i - (int64_t)k * n_rows;
    const int n = counts[i];
    if (n == 0) return;
    const int start = starts[i];
    // the run ends where the next block's run of the same row starts (or at the row's end)
    const int end = k + 1 < parts ? starts[i + n_rows] : indptr[r + 1];
    const int o = offsets[i];
    for (int j = 0; j < n; ++j) {
        const int s = start + 32 * j;
        desc[o + j] = make_int4((int)r, s, min(32, end - s), k);
    }
}

template <int NV, int U>
int launch_colblock(const PlanArgs& a, bool masked, cudaStream_t s) {
    const int64_t warps = (a.n_batches + kBatchesPerWarp - 1) / kBatchesPerWarp;
    const int64_t blocks = (warps + kThreads / 32 - 1) / (kThreads / 32);
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    if (masked)
        sddmm_colblock_kernel<NV, (U > 1 ? U / 2 : 1), true><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    else
        sddmm_colblock_kernel<NV, U, false><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

}  // namespace

#define FG_STR_(x) #x
#define FG_STR(x) FG_STR_(x)
const char* fg::sddmm_plan_signature() {
    // edges in flight per float4 count 1..4, blocks per SM
    return "sddmm_colblock<u" FG_STR(FG_CB_U1) "," FG_STR(FG_CB_U2) "," FG_STR(FG_CB_U3) "," FG_STR(FG_CB_U4) "|2/SM>";
}

extern "C" {

int32_t fg_sddmm_auto_partitions(int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d) {
    if (n_rows <= 0 || n_cols <= 0 || nnz <= 0 || d < 1 || d > 512 || d % 4 != 0) return 1;
    const int64_t l2 = fg::device_props().l2_bytes;
    const int64_t bytes = n_cols * (int64_t)d * 4;
    // a single pass of fg_sddmm_coo_f32 wins while the whole matrix fits three quarters of L2
    if (bytes <= l2 - l2 / 4) return 1;
    // Each half of the chip caches its own copy, and the block shares L2 with the streams (ids, outputs,
    // row-side rows): blocks of about 0.42 x L2 measured best (233K-node graph, d = 512: 9 or 10 blocks
    // 12.05 ms, 8 blocks 12.5, 16 blocks 12.4; the tiled call 14.6).
    const int64_t budget = l2 / 2 - l2 / 12;
    const int64_t parts = (bytes + budget - 1) / budget;
    // up to three feature tiles the tiled call is as fast (d = 128 on that graph: 3.47 ms either way)
    if (parts < 4 || parts > 64) return 1;
    // Worth it only while a (block, row) run still fills a good part of a 32-edge batch: on a graph of
    // short rows the runs shrink to single edges and whole-warp batches idle most of their lanes.
    if (nnz / (parts * n_rows) < 16) return 1;
    return (int32_t)parts;
}

int fg_sddmm_plan_create(const int32_t* d_row, const int32_t* d_col, int64_t n_rows, int64_t n_cols,
                         int64_t nnz, int32_t num_col_partitions, void* stream, fg_sddmm_plan** out_plan) {
    if (!out_plan) return fg::fail(FG_ERR_INVALID_ARGUMENT, "out_plan is NULL");
    *out_plan = nullptr;
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || n_rows > INT32_MAX || n_cols > INT32_MAX || nnz > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld", (long long)n_rows,
                        (long long)n_cols, (long long)nnz);
    if (num_col_partitions < 1 || num_col_partitions > 1024)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "num_col_partitions=%d: want 1..1024", num_col_partitions);
    if (nnz > 0 && (!d_row || !d_col)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL index array");
    const int64_t table = n_rows * num_col_partitions;
    if (table > INT32_MAX) return fg::fail(FG_ERR_INVALID_ARGUMENT, "n_rows * num_col_partitions beyond int32");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    fg_sddmm_plan* plan = new fg_sddmm_plan();
    plan->n_rows = n_rows;
    plan->n_cols = n_cols;
    plan->nnz = nnz;
    plan->parts = num_col_partitions;
    if (nnz == 0 || n_rows == 0) {
        *out_plan = plan;
        return FG_OK;
    }
    int32_t *indptr = nullptr, *starts = nullptr, *counts = nullptr, *offsets = nullptr, *flags = nullptr;
    void* temp = nullptr;
    size_t temp_bytes = 0;
    int rc = FG_OK;
    auto cleanup = [&]() {
        cudaFree(indptr);
        cudaFree(starts);
        cudaFree(counts);
        cudaFree(offsets);
        cudaFree(flags);
        cudaFree(temp);
    };
#define FG_TRY_OR_CLEAN(expr)                                                                      \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            rc = fg::fail(e__ == cudaErrorMemoryAllocation ? FG_ERR_OUT_OF_MEMORY : FG_ERR_CUDA,   \
                          "%s failed: %s", #expr, cudaGetErrorString(e__));                        \
            cleanup();                                                                             \
            cudaFree(plan->d_desc);                                                                \
            delete plan;                                                                           \
            return rc;                                                                             \
        }                                                                                          \
    } while (0)
    FG_TRY_OR_CLEAN(cudaMalloc(&indptr, sizeof(int32_t) * (n_rows + 1)));
    FG_TRY_OR_CLEAN(cudaMalloc(&starts, sizeof(int32_t) * table));
    FG_TRY_OR_CLEAN(cudaMalloc(&counts, sizeof(int32_t) * (table + 1)));
    FG_TRY_OR_CLEAN(cudaMalloc(&offsets, sizeof(int32_t) * (table + 1)));
    FG_TRY_OR_CLEAN(cudaMalloc(&flags, sizeof(int32_t)));
    FG_TRY_OR_CLEAN(cudaMemsetAsync(flags, 0, sizeof(int32_t), s));
    FG_TRY_OR_CLEAN(cudaMemsetAsync(counts + table, 0, sizeof(int32_t), s));
    const int threads = 256;
    rows_to_indptr_kernel<<<(unsigned)((nnz + threads - 1) / threads), threads, 0, s>>>(d_row, d_col, nnz, n_rows,
                                                                                         indptr, flags);
    FG_TRY_OR_CLEAN(cudaGetLastError());
    int32_t h_flags = 0;
    FG_TRY_OR_CLEAN(cudaMemcpyAsync(&h_flags, flags, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    FG_TRY_OR_CLEAN(cudaStreamSynchronize(s));
    if (h_flags != 0) {
        cleanup();
        delete plan;
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "the edge list is not in CSR order (%s): a column-block plan needs rows non-decreasing and "
                        "column ids ascending within each row",
                        (h_flags & 4) ? "a row id is out of range"
                                      : (h_flags & 1) ? "row ids decrease" : "column ids decrease inside a row");
    }
    const int32_t block_cols = (int32_t)((n_cols + num_col_partitions - 1) / num_col_partitions);
    block_runs_kernel<<<(unsigned)((n_rows + threads - 1) / threads), threads, 0, s>>>(
        indptr, d_col, n_rows, num_col_partitions, block_cols, starts, counts);
    FG_TRY_OR_CLEAN(cudaGetLastError());
    // exclusive scan over table + 1 entries: the last one is the number of batches
    FG_TRY_OR_CLEAN(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, counts, offsets, (int)(table + 1), s));
    FG_TRY_OR_CLEAN(cudaMalloc(&temp, temp_bytes ? temp_bytes : 1));
    FG_TRY_OR_CLEAN(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, counts, offsets, (int)(table + 1), s));
    int32_t n_batches = 0;
    FG_TRY_OR_CLEAN(cudaMemcpyAsync(&n_batches, offsets + table, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    FG_TRY_OR_CLEAN(cudaStreamSynchronize(s));
    // nnz / 32 + table bounds the count well below 2^31 for every size accepted above
    plan->n_batches = n_batches;
    FG_TRY_OR_CLEAN(cudaMalloc(&plan->d_desc, sizeof(int4) * (size_t)(n_batches > 0 ? n_batches : 1)));
    fill_descriptors_kernel<<<(unsigned)((table + threads - 1) / threads), threads, 0, s>>>(
        indptr, starts, counts, offsets, n_rows, num_col_partitions, plan->d_desc);
    FG_TRY_OR_CLEAN(cudaGetLastError());
    FG_TRY_OR_CLEAN(cudaStreamSynchronize(s));
#undef FG_TRY_OR_CLEAN
    cleanup();
    *out_plan = plan;
    return FG_OK;
}

int32_t fg_sddmm_plan_partitions(const fg_sddmm_plan* plan) { return plan ? plan->parts : 0; }

int64_t fg_sddmm_plan_batches(const fg_sddmm_plan* plan) { return plan ? plan->n_batches : 0; }

void fg_sddmm_plan_destroy(fg_sddmm_plan* plan) {
    if (!plan) return;
    cudaFree(plan->d_desc);
    delete plan;
}

int fg_sddmm_coo_f32_planned(const fg_sddmm_plan* plan, const int32_t* d_col, const float* d_src, int64_t ld_src,
                             const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                             int64_t nnz, int32_t d, int32_t accumulate, void* stream) {
    if (!plan) return fg::fail(FG_ERR_INVALID_ARGUMENT, "plan is NULL");
    if (n_rows != plan->n_rows || n_cols != plan->n_cols || nnz != plan->nnz)
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "the plan was built for %lld x %lld with %lld edges, this call has %lld x %lld with %lld: "
                        "rebuild the plan when the adjacency changes",
                        (long long)plan->n_rows, (long long)plan->n_cols, (long long)plan->nnz, (long long)n_rows,
                        (long long)n_cols, (long long)nnz);
    if (d < 1 || d > 512) return fg::fail(FG_ERR_INVALID_ARGUMENT, "d=%d: the planned call takes 1 <= d <= 512", d);
    if (ld_src == 0) ld_src = d;
    if (ld_dst == 0) ld_dst = d;
    if (ld_src < d || ld_dst < d || ld_src > INT32_MAX || ld_dst > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides ld_src=%lld ld_dst=%lld must be 0 or in [d=%d, 2^31)",
                        (long long)ld_src, (long long)ld_dst, d);
    if ((d % 4) || (ld_src % 4) || (ld_dst % 4) || !fg::aligned16(d_src) || !fg::aligned16(d_dst))
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "the planned call needs d and the row strides to be multiples of 4 floats and 16-byte aligned "
                        "feature matrices (use fg_sddmm_coo_f32 otherwise)");
    if (nnz == 0 || plan->n_batches == 0) return FG_OK;
    if (!d_col || !d_src || !d_dst || !d_out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    PlanArgs a;
    a.desc = plan->d_desc;
    a.n_batches = plan->n_batches;
    a.col = d_col;
    a.src = d_src;
    a.dst = d_dst;
    a.out = d_out;
    a.ld_src = (int32_t)ld_src;
    a.ld_dst = (int32_t)ld_dst;
    a.width = d;
    a.accumulate = accumulate;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nv = (d + 127) / 128;
    const bool masked = d != nv * 128;
    switch (nv) {
        case 1: return launch_colblock<1, FG_CB_U1>(a, masked, s);
        case 2: return launch_colblock<2, FG_CB_U2>(a, masked, s);
        case 3: return launch_colblock<3, FG_CB_U3>(a, masked, s);
        default: return launch_colblock<4, FG_CB_U4>(a, masked, s);
    }
}

}  // extern "C"
