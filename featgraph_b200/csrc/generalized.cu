// Generalized SpMM / SDDMM: other reductions than the sum, and per-edge outputs that are vectors.
//
// The reference checkout holds the sum-aggregating SpMM and the dot-product SDDMM only; its README
// (lines 9-11) mentions "generalized SpMM and generalized SDDMM w/ broadcasting" on a branch that is not
// part of it, so there is no source to follow here.  These are the plain forms of what GNN layers ask for
// beside the two hot ops, with the semantics stated in include/featgraph_b200.h:
//   reduce SpMM :  out[r, f] = reduce_{e in row r} ( vals[e] * x[col[e], f] ),  reduce in {max, min, mean}
//   edge-wise   :  out[e, f] = src[col[e], f]  (op)  dst[row[e], f],            op in {add, sub, mul}
// Neither is on the benchmarked path.  One warp per row (or per edge), 128-bit gathers, eight in flight; no
// row schedule, no rings: a max or a min has no summation order to preserve, so long rows need none of that
// machinery to be right, only to be fast.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;

enum { kMax = 1, kMin = 2, kMean = 3 };

template <int REDUCE>
__device__ __forceinline__ float combine(float acc, float v) {
    if (REDUCE == kMax) return fmaxf(acc, v);
    if (REDUCE == kMin) return fminf(acc, v);
    return __fadd_rn(acc, v);
}

// A warp owns a row; lane l owns columns 4 (l + 32 t) .. + 3 of every 128-float tile t (VEC) or column l + 32 t.
template <int REDUCE, bool VEC, bool UNIT>
__global__ void __launch_bounds__(kThreads) reduce_spmm_kernel(const int32_t* __restrict__ indptr,
                                                               const int32_t* __restrict__ indices,
                                                               const float* __restrict__ vals,
                                                               const float* __restrict__ x, int64_t ldx,
                                                               float* __restrict__ out, int64_t ldo, int64_t n_rows,
                                                               int32_t d) {
    constexpr int W = VEC ? 4 : 1;
    constexpr int CH = 8;  // gathers in flight
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int start = indptr[row], len = indptr[row + 1] - start;
    const float init = REDUCE == kMax ? -FLT_MAX : (REDUCE == kMin ? FLT_MAX : 0.f);
    for (int c0 = lane * W; c0 < d; c0 += 32 * W) {
        float acc[W];
#pragma unroll
        for (int w = 0; w < W; ++w) acc[w] = init;
        for (int base = 0; base < len; base += CH) {
            float xs[CH][W];
            float vs[CH];
            const int n = min(CH, len - base);
#pragma unroll
            for (int j = 0; j < CH; ++j) {
                if (j < n) {
                    const int c = indices[start + base + j];
                    vs[j] = UNIT ? 1.f : vals[start + base + j];
                    const float* p = x + (int64_t)c * ldx + c0;
                    if (VEC) {
                        const float4 q = fg::ldg4(p);
                        xs[j][0] = q.x;
                        xs[j][W > 1 ? 1 : 0] = q.y;
                        xs[j][W > 2 ? 2 : 0] = q.z;
                        xs[j][W > 3 ? 3 : 0] = q.w;
                    } else {
                        xs[j][0] = __ldg(p);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < CH; ++j)
                if (j < n)
#pragma unroll
                    for (int w = 0; w < W; ++w) acc[w] = combine<REDUCE>(acc[w], UNIT ? xs[j][w] : __fmul_rn(vs[j], xs[j][w]));
        }
#pragma unroll
        for (int w = 0; w < W; ++w) {
            float r = acc[w];
            if (len == 0) r = 0.f;  // a row without nonzeros reduces to 0, whatever the reduction
            if (REDUCE == kMean && len > 0) r = r / (float)len;
            if (c0 + w < d) out[row * ldo + c0 + w] = r;
        }
    }
}

enum { kAdd = 0, kSub = 1, kMul = 2 };

// A warp owns an edge; lanes stride over the feature columns.
template <bool VEC>
__global__ void __launch_bounds__(kThreads) edge_binary_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                                                               const float* __restrict__ src, int64_t ld_src,
                                                               const float* __restrict__ dst, int64_t ld_dst,
                                                               float* __restrict__ out, int64_t ldo, int64_t nnz, int32_t d,
                                                               int32_t op) {
    const int lane = threadIdx.x & 31;
    const int64_t e = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (e >= nnz) return;
    const float* s = src + (int64_t)col[e] * ld_src;
    const float* t = dst + (int64_t)row[e] * ld_dst;
    float* o = out + e * ldo;
    auto apply = [op](float a, float b) { return op == kAdd ? __fadd_rn(a, b) : (op == kSub ? __fsub_rn(a, b) : __fmul_rn(a, b)); };
    if (VEC) {
        for (int c = lane * 4; c < d; c += 128) {
            const float4 a = fg::ldg4(s + c), b = fg::ldg4(t + c);
            *reinterpret_cast<float4*>(o + c) = make_float4(apply(a.x, b.x), apply(a.y, b.y), apply(a.z, b.z), apply(a.w, b.w));
        }
    } else {
        for (int c = lane; c < d; c += 32) o[c] = apply(__ldg(s + c), __ldg(t + c));
    }
}

template <int REDUCE>
int launch_reduce(const int32_t* indptr, const int32_t* indices, const float* vals, const float* x, int64_t ldx, float* out,
                  int64_t ldo, int64_t n_rows, int32_t d, bool vec, cudaStream_t s) {
    const int64_t blocks = (n_rows + kThreads / 32 - 1) / (kThreads / 32);
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const unsigned b = (unsigned)blocks;
    if (vec && vals)
        reduce_spmm_kernel<REDUCE, true, false><<<b, kThreads, 0, s>>>(indptr, indices, vals, x, ldx, out, ldo, n_rows, d);
    else if (vec)
        reduce_spmm_kernel<REDUCE, true, true><<<b, kThreads, 0, s>>>(indptr, indices, vals, x, ldx, out, ldo, n_rows, d);
    else if (vals)
        reduce_spmm_kernel<REDUCE, false, false><<<b, kThreads, 0, s>>>(indptr, indices, vals, x, ldx, out, ldo, n_rows, d);
    else
        reduce_spmm_kernel<REDUCE, false, true><<<b, kThreads, 0, s>>>(indptr, indices, vals, x, ldx, out, ldo, n_rows, d);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

}  // namespace

extern "C" {

int fg_spmm_csr_reduce_f32(const int32_t* d_indptr, const int32_t* d_indices, const float* d_vals, const float* d_x,
                           int64_t ldx, float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                           int32_t reduce, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d", (long long)n_rows,
                        (long long)n_cols, (long long)nnz, d);
    if (n_rows > INT32_MAX || n_cols > INT32_MAX || nnz > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "sizes beyond int32 indexing are not supported");
    if (reduce != FG_REDUCE_MAX && reduce != FG_REDUCE_MIN && reduce != FG_REDUCE_MEAN)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "reduce=%d: want FG_REDUCE_MAX, FG_REDUCE_MIN or FG_REDUCE_MEAN "
                        "(the sum is fg_spmm_csr_f32)", reduce);
    if (ldx == 0) ldx = d;
    if (ldo == 0) ldo = d;
    if (ldx < d || ldo < d) return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides must be 0 or >= d=%d", d);
    if (n_rows == 0) return FG_OK;
    if (!d_indptr || !d_out || (nnz > 0 && (!d_indices || !d_x))) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    const bool vec = (d % 4 == 0) && (ldx % 4 == 0) && fg::aligned16(d_x);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (reduce) {
        case FG_REDUCE_MAX: return launch_reduce<kMax>(d_indptr, d_indices, d_vals, d_x, ldx, d_out, ldo, n_rows, d, vec, s);
        case FG_REDUCE_MIN: return launch_reduce<kMin>(d_indptr, d_indices, d_vals, d_x, ldx, d_out, ldo, n_rows, d, vec, s);
        default: return launch_reduce<kMean>(d_indptr, d_indices, d_vals, d_x, ldx, d_out, ldo, n_rows, d, vec, s);
    }
}

int fg_edge_binary_f32(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src, const float* d_dst,
                       int64_t ld_dst, float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                       int32_t op, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d", (long long)n_rows,
                        (long long)n_cols, (long long)nnz, d);
    if (op != FG_EDGE_ADD && op != FG_EDGE_SUB && op != FG_EDGE_MUL)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "op=%d: want FG_EDGE_ADD, FG_EDGE_SUB or FG_EDGE_MUL", op);
    if (ld_src == 0) ld_src = d;
    if (ld_dst == 0) ld_dst = d;
    if (ldo == 0) ldo = d;
    if (ld_src < d || ld_dst < d || ldo < d) return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides must be 0 or >= d=%d", d);
    if (nnz == 0) return FG_OK;
    if (!d_row || !d_col || !d_src || !d_dst || !d_out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    const int64_t blocks = (nnz + kThreads / 32 - 1) / (kThreads / 32);
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const bool vec = (d % 4 == 0) && (ld_src % 4 == 0) && (ld_dst % 4 == 0) && (ldo % 4 == 0) && fg::aligned16(d_src) &&
                     fg::aligned16(d_dst) && fg::aligned16(d_out);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (vec)
        edge_binary_kernel<true><<<(unsigned)blocks, kThreads, 0, s>>>(d_row, d_col, d_src, ld_src, d_dst, ld_dst, d_out, ldo,
                                                                        nnz, d, op);
    else
        edge_binary_kernel<false><<<(unsigned)blocks, kThreads, 0, s>>>(d_row, d_col, d_src, ld_src, d_dst, ld_dst, d_out, ldo,
                                                                         nnz, d, op);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

}  // extern "C"
