// SDDMM (per-edge dot product of a column-side and a row-side feature row) for sm_100a.
//
//   out[e] = sum_k src[col[e], k] * dst[row[e], k]      python/featgraph/op/vanilla_sddmm.py:47
//
// Work decomposition.  A warp takes 32 consecutive edges at a time: it reads their row and
// column ids with one coalesced load each and writes their 32 results with one coalesced
// store.  In between, groups of G lanes each take G consecutive edges of the 32.  For one
// edge the group's lanes gather a slice of src[col[e]] with 128-bit loads (consecutive lanes,
// consecutive 16 bytes) and multiply-accumulate it against the matching slice of dst[row[e]];
// each lane ends up with one partial sum per edge, and a transposed butterfly - G-1 shuffles
// for G edges instead of log2(G) per edge, its first steps done chunk by chunk so that only a
// few partial sums are ever live - leaves lane i of the group holding the finished dot product
// of edge i, which is exactly the layout of the coalesced store.
//
// Row side.  When the edge list is row-sorted (CSR order) the row-side slice stays in
// registers while consecutive edges share the row (a ballot marks where rows change), so it is
// read once per row, not once per edge.  Otherwise both rows are gathered for every edge.
//
// Feature tiling.  When the column-side matrix is too large for L2, the feature dimension is
// cut into tiles whose n_cols x tile slice does fit; one launch per tile, tile t > 0 adding
// its partial dot product to out[e] (stream order makes the read-modify-write safe).  This is
// the reference's num_feat_partitions loop order (fo -> edge -> fi, op/vanilla_sddmm.py:70-72)
// used to keep the gathered slice resident in L2.
//
// Arithmetic: fp32 FMA inside a lane, fixed-shape tree across lanes, ascending order across
// tiles.  Not the sequential k order of the x86 loop; the difference is bounded by fp32
// rounding of d terms.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kBatchesPerWarp = 16;  // 16 x 32 consecutive edges per warp
#ifndef FG_SDDMM_UNROLL
#define FG_SDDMM_UNROLL 1
#endif
constexpr int kBatchUnroll = FG_SDDMM_UNROLL;

__device__ __forceinline__ float dot4(float acc, const float4& a, const float4& b) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

struct SddmmArgs {
    const int32_t* row;
    const int32_t* col;
    const float* src;  // already offset to the tile's first column
    const float* dst;  // already offset to the tile's first column
    float* out;
    int64_t nnz;
    int64_t ld_src;  // row strides in floats
    int64_t ld_dst;
    int32_t width;  // columns in this tile (<= 4*G*NV)
    int32_t accumulate;
};

// G lanes per edge, NV float4 per lane, U edges' gathers in flight per group (U * NV 128-bit loads per
// lane), MINB resident blocks per SM asked of the compiler (the register budget: 64 for 4, 128 for 2).
// PF: how many batches ahead the row / column ids are requested.
// CACHE_DST: edge list is row-sorted, keep the row-side slice in registers.
// MASKED: the tile is narrower than 4*G*NV floats (ragged last tile).
template <int G, int NV, int U, int MINB, int PF, bool CACHE_DST, bool MASKED>
__global__ void __launch_bounds__(kThreads, MINB) sddmm_tile_kernel(const SddmmArgs a) {
    static_assert(G % U == 0, "U must divide G");
    const int lane = threadIdx.x & 31;
    const int lig = lane & (G - 1);
    const int gbase = lane & ~(G - 1);  // first lane of this lane's group
    const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << gbase);
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);

    // This lane's float4 number i of an edge's slice sits off(i) floats behind the lane's first one:
    // a compile-time constant (an immediate in the load) unless the tile is ragged, where a float4
    // beyond the tile's width is read from column 0 instead and zeroed.
    const int lane_col = (!MASKED || lig * 4 < a.width) ? lig * 4 : 0;
    int moff[NV];
    bool ok[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ok[i] = !MASKED || (lig + i * G) * 4 < a.width;
        moff[i] = ok[i] ? (lig + i * G) * 4 - lane_col : -lane_col;
    }
    auto off = [&](int i) { return MASKED ? moff[i] : i * G * 4; };
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint64_t keep_policy = fg::l2_keep_policy();
    const int ld_src = (int)a.ld_src, ld_dst = (int)a.ld_dst;  // 32 x 32 -> 64 bit multiply-add per gather
    const float* sbase = a.src + lane_col;
    // the row side is loaded once per row when the list is row-sorted: its base is not worth a register pair
    const float* dbase_reg = CACHE_DST ? nullptr : a.dst + lane_col;
#define dbase (CACHE_DST ? a.dst + lane_col : dbase_reg)
    float4 dcache[NV];  // row-side slice of cur_row (meaningful with CACHE_DST only)
#pragma unroll
    for (int i = 0; i < NV; ++i) dcache[i] = zero4;
    int cur_row = -1;

    // Row / column ids are a DRAM stream (one fresh 128-byte line of each per batch), slower to arrive
    // than a gather from L2: they are requested PF batches before their batch starts, in a small
    // register ring, so that the wait for them overlaps whole batches of gathers.
    const int64_t first = warp * kBatchesPerWarp * 32;
    int r_ring[PF], c_ring[PF];  // padding edges read row 0 / column 0 and are never stored
#pragma unroll
    for (int q = 0; q < PF; ++q) {
        r_ring[q] = 0;
        c_ring[q] = 0;
        const int64_t e = first + (int64_t)q * 32 + lane;
        if (e < a.nnz) {
            r_ring[q] = fg::ld_stream(a.row + e);
            c_ring[q] = fg::ld_stream(a.col + e);
        }
    }
    static_assert(kBatchesPerWarp % PF == 0 && FG_SDDMM_UNROLL % PF == 0, "PF must divide the unroll factor");
#pragma unroll kBatchUnroll
    for (int b = 0; b < kBatchesPerWarp; ++b) {
      {
        const int q = b % PF;  // a compile-time constant after unrolling
        const int64_t e0 = first + (int64_t)b * 32;
        if (e0 >= a.nnz) break;  // warp-uniform
        const int64_t e = e0 + lane;
        const bool valid = e < a.nnz;
        const int r_l = r_ring[q], c_l = c_ring[q];
        r_ring[q] = 0;
        c_ring[q] = 0;
        if (b + PF < kBatchesPerWarp && e + 32 * PF < a.nnz) {
            r_ring[q] = fg::ld_stream(a.row + e + 32 * PF);
            c_ring[q] = fg::ld_stream(a.col + e + 32 * PF);
        }
        float prev = 0.f;  // earlier tiles' partial dot product
        if (a.accumulate && valid) prev = fg::ld_stream(a.out + e);
        // Row side.  ONE_ROW: all 32 edges of the batch share a row (the common case in a row-sorted
        // list with long rows): its slice is loaded once, and only if it differs from the previous
        // batch's.  Otherwise a ballot marks where rows change (bit l: edge l starts a new row; always
        // set at a group's first edge) and each group reloads at its marks.
        float r[G / U];  // one partly reduced value per chunk of U edges
        auto run_batch = [&](auto one_row_tag) {
            constexpr bool ONE_ROW = decltype(one_row_tag)::value;
            unsigned change = 0;
            if (CACHE_DST && !ONE_ROW) {
                const int r_prev = __shfl_up_sync(0xffffffffu, r_l, 1);
                change = __ballot_sync(0xffffffffu, lig == 0 || r_prev != r_l);
            }
#pragma unroll
            for (int s = 0; s < G; s += U) {
                int c[U], rr[U];
                float pc[U];
                float4 xs[U][NV];
                float4 xd[U][NV];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    c[u] = __shfl_sync(0xffffffffu, c_l, gbase + s + u);
                    if (!CACHE_DST) rr[u] = __shfl_sync(0xffffffffu, r_l, gbase + s + u);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float* ps = sbase + (int64_t)c[u] * ld_src;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        xs[u][i] = fg::ldg4_keep(ps + off(i), keep_policy);
                        if (MASKED && !ok[i]) xs[u][i] = zero4;
                    }
                    if (!CACHE_DST) {
                        const float* pd = dbase + (int64_t)rr[u] * ld_dst;
#pragma unroll
                        for (int i = 0; i < NV; ++i) {
                            xd[u][i] = fg::ldg4(pd + off(i));
                            if (MASKED && !ok[i]) xd[u][i] = zero4;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float acc = 0.f;
                    if (CACHE_DST) {
                        if (!ONE_ROW && ((change >> (gbase + s + u)) & 1u)) {  // uniform within the group
                            const int rnew = __shfl_sync(gmask, r_l, gbase + s + u);
                            const float* pd = dbase + (int64_t)rnew * ld_dst;
#pragma unroll
                            for (int i = 0; i < NV; ++i) {
                                dcache[i] = fg::ldg4(pd + off(i));
                                if (MASKED && !ok[i]) dcache[i] = zero4;  // 0 * 0, never 0 * (a stray Inf or NaN)
                            }
                        }
#pragma unroll
                        for (int i = 0; i < NV; ++i) acc = dot4(acc, xs[u][i], dcache[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < NV; ++i) acc = dot4(acc, xs[u][i], xd[u][i]);
                    }
                    pc[u] = acc;
                }
                // first log2(U) steps of the transposed butterfly, inside the chunk: afterwards pc[0]
                // on a lane holds, for the chunk's edge picked by the lane's low bits, the sum over
                // the 2^k lanes that differ from it in those bits
#pragma unroll
                for (int off2 = 1; off2 < U; off2 <<= 1) {
                    const bool upper = (lig & off2) != 0;
#pragma unroll
                    for (int i = 0; i < U / (2 * off2); ++i) {
                        const float send = upper ? pc[2 * i] : pc[2 * i + 1];
                        const float keep = upper ? pc[2 * i + 1] : pc[2 * i];
                        pc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off2);
                    }
                }
                r[s / U] = pc[0];
            }
        };
        const int r_first = __shfl_sync(0xffffffffu, r_l, 0);
        if (CACHE_DST && __all_sync(0xffffffffu, r_l == r_first)) {
            if (r_first != cur_row) {
                cur_row = r_first;
                const float* pd = dbase + (int64_t)r_first * ld_dst;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                                dcache[i] = fg::ldg4(pd + off(i));
                                if (MASKED && !ok[i]) dcache[i] = zero4;  // 0 * 0, never 0 * (a stray Inf or NaN)
                            }
            }
            run_batch(std::true_type{});
        } else {
            run_batch(std::false_type{});
            cur_row = -1;  // the groups ended on different rows
        }

        // remaining steps across the chunks: afterwards r[0] on lane i of the group is edge i's total
#pragma unroll
        for (int off2 = U; off2 < G; off2 <<= 1) {
            const bool upper = (lig & off2) != 0;
            const int h = off2 / U;
#pragma unroll
            for (int i = 0; i < G / U / (2 * h); ++i) {
                const float send = upper ? r[2 * i] : r[2 * i + 1];
                const float keep = upper ? r[2 * i + 1] : r[2 * i];
                r[i] = keep + __shfl_xor_sync(0xffffffffu, send, off2);
            }
        }
        if (valid) fg::st_stream(a.out + e, prev + r[0]);
      }
    }
#undef dbase
}

// Any d, any alignment: a warp per 32 edges, lanes stride over the feature columns.
__global__ void __launch_bounds__(kThreads, 4)
sddmm_generic_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                     const float* __restrict__ src, int64_t ld_src, const float* __restrict__ dst,
                     int64_t ld_dst, float* __restrict__ out, int64_t nnz, int32_t d, int32_t accumulate) {
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
            const float* ps = src + (int64_t)c * ld_src;
            const float* pd = dst + (int64_t)r * ld_dst;
            float p = 0.f;
            for (int k = lane; k < d; k += 32) p = fmaf(__ldg(ps + k), __ldg(pd + k), p);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) p += __shfl_xor_sync(0xffffffffu, p, off);
            if (lane == s) res = p;
        }
        if (e < nnz) out[e] = accumulate ? out[e] + res : res;
    }
}


// ---------------------------------------------------------------------------------------------
// Exact-order SDDMM: out[e] = ((s0*t0 + s1*t1) + s2*t2) + ... with every product and every sum
// rounded separately and k strictly ascending - the value the x86 loop of the reference
// produces (python/featgraph/op/vanilla_sddmm.py:43-62), bit for bit.
//
// One lane owns one edge and walks k alone, so nothing is re-associated.  To keep the global
// loads coalesced the warp first stages, for its 32 edges and 32 consecutive k, both feature
// rows in shared memory: eight 128-bit loads per matrix (4 edges per load, 8 lanes x 16 bytes per
// edge) are stored k-major with a rotation, tile[k][(edge + k) % 32], which makes both the
// scattered stores and the per-lane reads tile[k][(lane + k) % 32] bank-conflict free.
// Three to four times slower than sddmm_tile_kernel (both rows of every edge cross shared memory
// twice and the per-edge sum is a serial chain); an opt-in for callers that want bit-for-bit
// agreement.
// ---------------------------------------------------------------------------------------------
constexpr int kExactWarps = 4;  // 32 KB of static shared memory per block

__global__ void __launch_bounds__(kExactWarps * 32, 6)
sddmm_exact_kernel(const int32_t* __restrict__ row, const int32_t* __restrict__ col,
                   const float* __restrict__ src, int ld_src, const float* __restrict__ dst, int ld_dst,
                   float* __restrict__ out, int64_t nnz, int32_t d, int32_t accumulate, bool vec) {
    __shared__ float tiles[kExactWarps][2][32 * 32];
    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    float* ts = tiles[w][0];
    float* td = tiles[w][1];
    const int64_t warp = (int64_t)blockIdx.x * kExactWarps + w;
    const int piece = lane & 7;  // 16-byte piece of a 32-float chunk
    const int sub = lane >> 3;   // which of the 4 edges of a load instruction
    for (int b = 0; b < kBatchesPerWarp; ++b) {
        const int64_t e0 = (warp * kBatchesPerWarp + b) * 32;
        if (e0 >= nnz) break;  // warp-uniform
        const int64_t e = e0 + lane;
        const bool valid = e < nnz;
        int r_l = 0, c_l = 0;  // padding edges read row 0 / column 0 and are never stored
        if (valid) {
            r_l = row[e];
            c_l = col[e];
        }
        float acc = (accumulate && valid) ? out[e] : 0.f;
        for (int k0 = 0; k0 < d; k0 += 32) {
            const int kw = d - k0 < 32 ? d - k0 : 32;  // columns in this chunk
            __syncwarp();  // the previous chunk has been read
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int edge = i * 4 + sub;
                const int c = __shfl_sync(0xffffffffu, c_l, edge);
                const int r = __shfl_sync(0xffffffffu, r_l, edge);
                const float* ps = src + (int64_t)c * ld_src + k0 + piece * 4;
                const float* pd = dst + (int64_t)r * ld_dst + k0 + piece * 4;
                float sv[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
                if (vec && piece * 4 + 4 <= kw) {
                    const float4 a4 = fg::ldg4(ps), b4 = fg::ldg4(pd);
                    sv[0] = a4.x; sv[1] = a4.y; sv[2] = a4.z; sv[3] = a4.w;
                    dv[0] = b4.x; dv[1] = b4.y; dv[2] = b4.z; dv[3] = b4.w;
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (piece * 4 + q < kw) {
                            sv[q] = __ldg(ps + q);
                            dv[q] = __ldg(pd + q);
                        }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int k = piece * 4 + q;
                    ts[k * 32 + ((edge + k) & 31)] = sv[q];
                    td[k * 32 + ((edge + k) & 31)] = dv[q];
                }
            }
            __syncwarp();
            if (kw == 32) {
#pragma unroll
                for (int k = 0; k < 32; ++k)
                    acc = fg::mul_then_add(acc, ts[k * 32 + ((lane + k) & 31)], td[k * 32 + ((lane + k) & 31)]);
            } else {
                for (int k = 0; k < kw; ++k)
                    acc = fg::mul_then_add(acc, ts[k * 32 + ((lane + k) & 31)], td[k * 32 + ((lane + k) & 31)]);
            }
        }
        if (valid) out[e] = acc;
    }
}

#ifndef FG_SDDMM_PF
#define FG_SDDMM_PF 1
#endif

template <int G, int NV, int U, int MINB>
int launch_tile(const SddmmArgs& a, bool cache_dst, bool masked, unsigned blocks, cudaStream_t s) {
    // Variants that hold more live registers (both rows gathered per edge; masked loads) keep
    // half as many edges in flight so that they stay within the register budget.
    constexpr int UH = U > 1 ? U / 2 : 1;
    if (cache_dst) {
        if (masked)
            sddmm_tile_kernel<G, NV, UH, MINB, FG_SDDMM_PF, true, true><<<blocks, kThreads, 0, s>>>(a);
        else
            sddmm_tile_kernel<G, NV, U, MINB, FG_SDDMM_PF, true, false><<<blocks, kThreads, 0, s>>>(a);
    } else {
        if (masked)
            sddmm_tile_kernel<G, NV, UH, MINB, FG_SDDMM_PF, false, true><<<blocks, kThreads, 0, s>>>(a);
        else
            sddmm_tile_kernel<G, NV, UH, MINB, FG_SDDMM_PF, false, false><<<blocks, kThreads, 0, s>>>(a);
    }
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

// Lane layout per tile width: G, NV, U, MINB.  Overridable at build time (kernel sweeps).
#ifndef FG_Q8_G
#define FG_Q8_G 8
#define FG_Q8_NV 1
#define FG_Q8_U 8
#define FG_Q8_MINB 4
#endif
#ifndef FG_Q16_G  // 64-float tiles: 4 edges per warp step measured fastest
#define FG_Q16_G 8
#define FG_Q16_NV 2
#define FG_Q16_U 4
#define FG_Q16_MINB 4
#endif
#ifndef FG_Q32_G
#define FG_Q32_G 32
#define FG_Q32_NV 1
#define FG_Q32_U 8
#define FG_Q32_MINB 4
#endif

// One tile of `width` floats (a multiple of 4, at most 512).
int launch_width(const SddmmArgs& a, bool cache, unsigned blocks, cudaStream_t s) {
    const int q = (a.width + 3) / 4;  // float4 per edge in this tile
#define FG_SDDMM(G, NV, U, MINB) return launch_tile<G, NV, U, MINB>(a, cache, q != (G) * (NV), blocks, s)
    if (q <= 1) FG_SDDMM(1, 1, 1, 4);
    if (q <= 2) FG_SDDMM(2, 1, 2, 4);
    if (q <= 4) FG_SDDMM(4, 1, 4, 4);
    if (q <= 8) FG_SDDMM(FG_Q8_G, FG_Q8_NV, FG_Q8_U, FG_Q8_MINB);
    if (q <= 16) FG_SDDMM(FG_Q16_G, FG_Q16_NV, FG_Q16_U, FG_Q16_MINB);
    if (q <= 32) FG_SDDMM(FG_Q32_G, FG_Q32_NV, FG_Q32_U, FG_Q32_MINB);
    if (q <= 64) FG_SDDMM(32, 2, 4, 2);
    if (q <= 96) FG_SDDMM(32, 3, 2, 2);
    FG_SDDMM(32, 4, 2, 2);
#undef FG_SDDMM
}

int64_t l2_size_bytes() { return fg::device_props().l2_bytes; }

}  // namespace

#define FG_STR_(x) #x
#define FG_STR(x) FG_STR_(x)
const char* fg::sddmm_signature() {
    // lane layout per tile width as G,NV,U,MINB for 32-, 64- and 128-float tiles; id prefetch depth
    return "sddmm_tile<q8:" FG_STR(FG_Q8_G) "," FG_STR(FG_Q8_NV) "," FG_STR(FG_Q8_U) "," FG_STR(FG_Q8_MINB) "|q16:" FG_STR(
        FG_Q16_G) "," FG_STR(FG_Q16_NV) "," FG_STR(FG_Q16_U) "," FG_STR(FG_Q16_MINB) "|q32:" FG_STR(FG_Q32_G) "," FG_STR(
        FG_Q32_NV) "," FG_STR(FG_Q32_U) "," FG_STR(FG_Q32_MINB) "|pf" FG_STR(FG_SDDMM_PF) ">";
}

extern "C" {

int fg_sddmm_coo_f32(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src,
                     const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                     int64_t nnz, int32_t d, int32_t rows_sorted, int32_t accumulate, int32_t feat_tile,
                     void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (n_rows > INT32_MAX || n_cols > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "sizes beyond int32 indexing are not supported");
    if (feat_tile != 0 && (feat_tile < 4 || feat_tile > 512 || (feat_tile & (feat_tile - 1))))
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "feat_tile=%d: want 0 or a power of two in 4..512",
                        feat_tile);
    if (ld_src == 0) ld_src = d;
    if (ld_dst == 0) ld_dst = d;
    if (ld_src < d || ld_dst < d || ld_src > INT32_MAX || ld_dst > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides ld_src=%lld ld_dst=%lld must be 0 or in [d=%d, 2^31)",
                        (long long)ld_src, (long long)ld_dst, d);
    if (nnz == 0) return FG_OK;
    if (!d_row || !d_col || !d_src || !d_dst || !d_out)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t edges_per_block = (int64_t)(kThreads / 32) * kBatchesPerWarp * 32;
    const int64_t nblocks = (nnz + edges_per_block - 1) / edges_per_block;
    if (nblocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const unsigned blocks = (unsigned)nblocks;
    const bool cache = rows_sorted != 0;
    const bool vec = (d % 4 == 0) && (ld_src % 4 == 0) && (ld_dst % 4 == 0) && fg::aligned16(d_src) &&
                     fg::aligned16(d_dst);
    if (!vec) {
        sddmm_generic_kernel<<<blocks, kThreads, 0, s>>>(d_row, d_col, d_src, ld_src, d_dst, ld_dst, d_out, nnz,
                                                          d, accumulate);
        FG_CUDA_TRY(cudaGetLastError());
        fg::count_launches(1);
        return FG_OK;
    }
    // Tile width: the whole row if the column-side matrix fits the resident share of L2 (or if
    // not even a 32-float slice does); otherwise the widest power of two whose slice fits.
    int tile = feat_tile;
    if (tile == 0) {
        // A single pass wins while the whole matrix fits three quarters of L2 (no second read of
        // the edge list, no read-modify-write of out); a slice should fit in half of L2.
        const int64_t l2 = l2_size_bytes();
        const int64_t budget = l2 / 2;
        if (n_cols * (int64_t)d * 4 <= l2 - l2 / 4 || n_cols * 32 * 4 > budget) {
            tile = d <= 512 ? d : 512;
        } else {
            tile = 32;
            while (tile * 2 <= 512 && n_cols * (int64_t)(tile * 2) * 4 <= budget) tile *= 2;
        }
    }
    if (tile > d) tile = d;
    SddmmArgs a;
    a.row = d_row;
    a.col = d_col;
    a.out = d_out;
    a.nnz = nnz;
    a.ld_src = ld_src;
    a.ld_dst = ld_dst;
    for (int f0 = 0; f0 < d; f0 += tile) {
        a.src = d_src + f0;
        a.dst = d_dst + f0;
        a.width = (d - f0 < tile) ? d - f0 : tile;
        a.accumulate = (f0 > 0) || accumulate;
        const int rc = launch_width(a, cache, blocks, s);
        if (rc != FG_OK) return rc;
    }
    return FG_OK;
}

int fg_sddmm_coo_f32_exact(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src,
                           const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                           int64_t nnz, int32_t d, int32_t accumulate, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (ld_src == 0) ld_src = d;
    if (ld_dst == 0) ld_dst = d;
    if (ld_src < d || ld_dst < d || ld_src > INT32_MAX || ld_dst > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides ld_src=%lld ld_dst=%lld must be 0 or in [d=%d, 2^31)",
                        (long long)ld_src, (long long)ld_dst, d);
    if (nnz == 0) return FG_OK;
    if (!d_row || !d_col || !d_src || !d_dst || !d_out)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    const int64_t edges_per_block = (int64_t)kExactWarps * kBatchesPerWarp * 32;
    const int64_t nblocks = (nnz + edges_per_block - 1) / edges_per_block;
    if (nblocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const bool vec = (ld_src % 4 == 0) && (ld_dst % 4 == 0) && fg::aligned16(d_src) && fg::aligned16(d_dst);
    // Column windows keep the gathered slice of src in L2, as in fg_sddmm_coo_f32; a window continues
    // the sequential sum from out[e], so the k order - and every bit - is that of a single pass.
    int tile = d;
    const int64_t l2 = l2_size_bytes();
    if (n_cols * (int64_t)d * 4 > l2 - l2 / 4 && n_cols * 32 * 4 <= l2 / 2) {
        tile = 32;
        while (tile * 2 < d && n_cols * (int64_t)(tile * 2) * 4 <= l2 / 2) tile *= 2;
    }
    for (int f0 = 0; f0 < d; f0 += tile) {
        const int wd = d - f0 < tile ? d - f0 : tile;
        sddmm_exact_kernel<<<(unsigned)nblocks, kExactWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
            d_row, d_col, d_src + f0, (int)ld_src, d_dst + f0, (int)ld_dst, d_out, nnz, wd,
            (f0 > 0 || accumulate) ? 1 : 0, vec);
        fg::count_launches(1);
    }
    FG_CUDA_TRY(cudaGetLastError());
    return FG_OK;
}

}  // extern "C"
