// SDDMM (per-edge dot product of a column-side and a row-side feature row) for sm_100a.
//
//   out[e] = sum_k src[col[e], k] * dst[row[e], k]      python/featgraph/op/vanilla_sddmm.py:47
//
// Work decomposition.  A warp takes 32 consecutive edges at a time: it reads their row and
// column ids with one coalesced load each, and writes their 32 results with one coalesced
// store.  In between, groups of G lanes (G*4*NV >= d) each take G consecutive edges of the
// 32; for one edge the group's lanes gather the d floats of src[col[e]] with 128-bit loads
// (consecutive lanes, consecutive 16 bytes), multiply by the matching slice of dst[row[e]],
// add up their own products and finish with a log2(G)-step butterfly of warp shuffles.
// Several edges' gathers are issued before the first reduction.
//
// When the edge list is row-sorted (CSR order) the row-side slice stays in registers for
// as long as consecutive edges share the row, so it is read once per row, not once per
// edge.  Otherwise both rows are gathered for every edge.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kBatchesPerWarp = 8;  // 8 x 32 consecutive edges per warp

__device__ __forceinline__ float dot4(float acc, const float4& a, const float4& b) {
    acc = fg::mul_then_add(acc, a.x, b.x);
    acc = fg::mul_then_add(acc, a.y, b.y);
    acc = fg::mul_then_add(acc, a.z, b.z);
    acc = fg::mul_then_add(acc, a.w, b.w);
    return acc;
}

// G lanes per edge, NV float4 per lane, U edges in flight per group.
template <int G, int NV, int U, bool CACHE_DST>
__global__ void __launch_bounds__(kThreads, 4)
sddmm_vec4_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                  const float* __restrict__ src, const float* __restrict__ dst,
                  float* __restrict__ out, int64_t nnz, int32_t d) {
    static_assert(G % U == 0, "U must divide G");
    const int lane = threadIdx.x & 31;
    const int lig = lane & (G - 1);
    const int gbase = lane & ~(G - 1);  // first lane of this lane's group
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);

    int colv[NV];
    bool ok[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        colv[i] = (lig + i * G) * 4;
        ok[i] = colv[i] < d;
    }

    int cur_row = -1;
    float4 dcache[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) dcache[i] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int b = 0; b < kBatchesPerWarp; ++b) {
        const int64_t e0 = (warp * kBatchesPerWarp + b) * 32;
        if (e0 >= nnz) break;  // warp-uniform
        const int64_t e = e0 + lane;
        int r_l = -1, c_l = -1;
        if (e < nnz) {
            r_l = row[e];
            c_l = col[e];
        }
        float res = 0.f;
#pragma unroll 1
        for (int s = 0; s < G; s += U) {
            int r[U], c[U];
            float4 xs[U][NV];
            float4 xd[U][NV];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                r[u] = __shfl_sync(0xffffffffu, r_l, gbase + s + u);
                c[u] = __shfl_sync(0xffffffffu, c_l, gbase + s + u);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    xs[u][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (c[u] >= 0 && ok[i]) xs[u][i] = fg::ldg4(src + (int64_t)c[u] * d + colv[i]);
                    if (!CACHE_DST) {
                        xd[u][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (r[u] >= 0 && ok[i])
                            xd[u][i] = fg::ldg4(dst + (int64_t)r[u] * d + colv[i]);
                    }
                }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float p = 0.f;
                if (CACHE_DST) {
                    if (r[u] >= 0 && r[u] != cur_row) {
                        cur_row = r[u];
#pragma unroll
                        for (int i = 0; i < NV; ++i)
                            if (ok[i]) dcache[i] = fg::ldg4(dst + (int64_t)cur_row * d + colv[i]);
                    }
#pragma unroll
                    for (int i = 0; i < NV; ++i) p = dot4(p, xs[u][i], dcache[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < NV; ++i) p = dot4(p, xs[u][i], xd[u][i]);
                }
#pragma unroll
                for (int off = G / 2; off > 0; off >>= 1)
                    p = __fadd_rn(p, __shfl_xor_sync(0xffffffffu, p, off));
                if (lig == s + u) res = p;
            }
        }
        if (e < nnz) out[e] = res;
    }
}

// Any d, any alignment: a warp per 32 edges, lanes stride over the feature columns.
__global__ void __launch_bounds__(kThreads, 4)
sddmm_generic_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                     const float* __restrict__ src, const float* __restrict__ dst,
                     float* __restrict__ out, int64_t nnz, int32_t d) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    for (int b = 0; b < kBatchesPerWarp; ++b) {
        const int64_t e0 = (warp * kBatchesPerWarp + b) * 32;
        if (e0 >= nnz) break;
        const int64_t e = e0 + lane;
        int r_l = -1, c_l = -1;
        if (e < nnz) {
            r_l = row[e];
            c_l = col[e];
        }
        float res = 0.f;
        for (int s = 0; s < 32; ++s) {
            const int r = __shfl_sync(0xffffffffu, r_l, s);
            const int c = __shfl_sync(0xffffffffu, c_l, s);
            if (r < 0) break;  // warp-uniform: the tail of the last batch
            const float* ps = src + (int64_t)c * d;
            const float* pd = dst + (int64_t)r * d;
            float p = 0.f;
            for (int k = lane; k < d; k += 32) p = fg::mul_then_add(p, __ldg(ps + k), __ldg(pd + k));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                p = __fadd_rn(p, __shfl_xor_sync(0xffffffffu, p, off));
            if (lane == s) res = p;
        }
        if (e < nnz) out[e] = res;
    }
}

template <int G, int NV, int U>
int launch_vec4(const int32_t* row, const int32_t* col, const float* src, const float* dst,
                float* out, int64_t nnz, int32_t d, bool cache_dst, unsigned blocks,
                cudaStream_t s) {
    if (cache_dst)
        sddmm_vec4_kernel<G, NV, U, true><<<blocks, kThreads, 0, s>>>(row, col, src, dst, out, nnz, d);
    else
        sddmm_vec4_kernel<G, NV, U, false><<<blocks, kThreads, 0, s>>>(row, col, src, dst, out, nnz, d);
    FG_CUDA_TRY(cudaGetLastError());
    return FG_OK;
}

}  // namespace

extern "C" {

int fg_sddmm_coo_f32(const int32_t* d_row, const int32_t* d_col, const float* d_src,
                     const float* d_dst, float* d_out, int64_t n_rows, int64_t n_cols, int64_t nnz,
                     int32_t d, int32_t rows_sorted, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (n_rows > INT32_MAX || n_cols > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "sizes beyond int32 indexing are not supported");
    if (nnz == 0) return FG_OK;
    if (!d_row || !d_col || !d_src || !d_dst || !d_out)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t edges_per_block = (int64_t)(kThreads / 32) * kBatchesPerWarp * 32;
    const int64_t nblocks = (nnz + edges_per_block - 1) / edges_per_block;
    if (nblocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const unsigned blocks = (unsigned)nblocks;
    const bool cache = rows_sorted != 0;
    const bool vec = (d % 4 == 0) && d <= 512 && fg::aligned16(d_src) && fg::aligned16(d_dst);
    if (!vec) {
        sddmm_generic_kernel<<<blocks, kThreads, 0, s>>>(d_row, d_col, d_src, d_dst, d_out, nnz, d);
        FG_CUDA_TRY(cudaGetLastError());
        return FG_OK;
    }
#define FG_SDDMM(G, NV, U) \
    return launch_vec4<G, NV, U>(d_row, d_col, d_src, d_dst, d_out, nnz, d, cache, blocks, s)
    const int q = d / 4;  // float4 per feature row
    if (q <= 1) FG_SDDMM(1, 1, 1);
    if (q <= 2) FG_SDDMM(2, 1, 2);
    if (q <= 4) FG_SDDMM(4, 1, 4);
    if (q <= 8) FG_SDDMM(8, 1, 8);
    if (q <= 16) FG_SDDMM(16, 1, 8);
    if (q <= 32) FG_SDDMM(32, 1, 8);
    if (q <= 64) FG_SDDMM(32, 2, 4);
    if (q <= 96) FG_SDDMM(32, 3, 2);
    FG_SDDMM(32, 4, 2);
#undef FG_SDDMM
}

}  // extern "C"
