/*
 * CPU oracle for vanilla SpMM / SDDMM: a plain-C restatement of the loop nests
 * that the reference's x86 schedules describe to its code generator.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the parity tests,
 * the smoke test and the benchmark's CPU-baseline leg compare against or time.
 * Nothing the library ships calls it, links it or falls back to it.
 *
 * PARITY STATUS.  The reference executes these loops through a third-party code generator
 * (Apache TVM, not vendored, version not pinned by the reference), and its own tests hold no
 * numeric golden vectors for SpMM/SDDMM (they compare random inputs with scipy/numpy at
 * rtol = atol = 1e-4: tests/test_module_spmm.py:29-30, tests/test_module_sddmm.py:34-37).
 *  - SDDMM: PINNED.  The reference's own compute definition (op/vanilla_sddmm.py:6-63), lowered
 *    and compiled by a TVM build (the 0.23.dev0 fork shipped inside the tilelang package, C
 *    backend), gives bit-identical output to fgo_sddmm_x86 with use_fma = 0 on every committed
 *    case (tests/golden/sddmm_reference_tvm.npz, made by make_sddmm_reference_golden.py).
 *  - SpMM (CSR x86, CSR CUDA and DDS definitions, op/vanilla_spmm.py:6-62, 83-125, 149-224):
 *    PINNED the same way, on random non-unit values: fgo_spmm_csr_x86 / fgo_spmm_dds_x86 with
 *    use_fma = 0 are bit-identical to the TVM-compiled outputs in
 *    tests/golden/spmm_reference_tvm.npz (make_spmm_reference_golden.py; that script repairs one
 *    lowering artefact of the fork - a tensor-expression load left in a loop extent - and touches
 *    neither arithmetic nor loop order).  Also bit-equal to scipy's CSR product on the
 *    reference's test shape (scipy is what the reference's tests compare against).
 *    What the pin does not cover: the exact TVM release and LLVM backend the reference was run
 *    with (unpinned by the reference itself); the fixtures come from that fork's C backend.
 *
 * Arithmetic model: fp32 throughout, one rounding for the product and one for the
 * sum (no fused multiply-add): the reference's x86 target string is the bare
 * 'llvm' (python/featgraph/module/spmm.py:202, module/sddmm.py:173), i.e. baseline
 * x86-64 without an FMA unit.  Build with -ffp-contract=off.  Every function takes
 * use_fma: 0 = that model, 1 = fused, so a test can state which one a GPU result
 * matches.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int fgo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* -ffp-contract=off keeps `acc + a * b` as two roundings; use_fma is a literal at
 * every call site after inlining, so the branch folds away. */
static inline __attribute__((always_inline)) float mul_add(float acc, float a, float b,
                                                           const int use_fma) {
    return use_fma ? fmaf(a, b, acc) : acc + a * b;
}

/* ---------------------------------------------------------------------------------
 * SpMM, CSR.  python/featgraph/op/vanilla_spmm.py:41-62 (math) with the schedule at
 * :65-80: three stages, each parallel over the vertex axis,
 *   (1) ReshapedSrcFeat[fo][nn][fi] = X[nn][fo*F + fi]                    (:43-44, :76)
 *   (2) ReshapedOut[fo][row][fi] = sum_e vals[e] * ReshapedSrcFeat[fo][indices[e]][fi]
 *       loop nest fo -> row (parallel) -> e -> fi                        (:46-56, :73, :77)
 *   (3) Out[nn][ff] = ReshapedOut[ff / F][nn][ff % F]                     (:58-60, :78)
 * with F = d / num_feat_partitions.  The accumulator starts at 0 and takes the
 * row's nonzeros in storage order.  with_copies = 0 skips (1) and (3) (same values,
 * used where only the numbers matter); 1 runs them, as the reference's timed function
 * does.  Rows are split over threads in contiguous static chunks, as a 'parallel'
 * loop of the reference's thread pool is.
 * Returns 0, or 1 when scratch memory for the copies cannot be had.
 * --------------------------------------------------------------------------------- */
static inline __attribute__((always_inline)) int fgo_spmm_csr_x86_impl(int64_t n_rows, int64_t n_cols, int32_t d, int32_t num_feat_partitions,
                     const int32_t* indptr, const int32_t* indices, const float* vals,
                     const float* X, float* out, int use_fma, int with_copies) {
    const int64_t P = num_feat_partitions;
    const int64_t F = d / P;
    const float* src = X;
    float* dst = out;
    float* rs = NULL;
    float* ro = NULL;
    if (with_copies) {
        rs = (float*)malloc(sizeof(float) * (size_t)(P * n_cols * F + 1));
        ro = (float*)malloc(sizeof(float) * (size_t)(P * n_rows * F + 1));
        if (!rs || !ro) { free(rs); free(ro); return 1; }
        for (int64_t fo = 0; fo < P; ++fo) {
#pragma omp parallel for schedule(static)
            for (int64_t nn = 0; nn < n_cols; ++nn)
                for (int64_t fi = 0; fi < F; ++fi)
                    rs[(fo * n_cols + nn) * F + fi] = X[nn * d + fo * F + fi];
        }
        src = rs;
        dst = ro;
    }
    for (int64_t fo = 0; fo < P; ++fo) {
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < n_rows; ++row) {
            /* with copies: [fo][row][fi]; without: straight into Out[row][fo*F + fi] */
            float* o = with_copies ? dst + (fo * n_rows + row) * F : dst + row * d + fo * F;
            for (int64_t fi = 0; fi < F; ++fi) o[fi] = 0.0f;
            for (int64_t e = indptr[row]; e < indptr[row + 1]; ++e) {
                const float v = vals[e];
                const int64_t c = indices[e];
                const float* x = with_copies ? src + (fo * n_cols + c) * F : src + c * d + fo * F;
                for (int64_t fi = 0; fi < F; ++fi) o[fi] = mul_add(o[fi], v, x[fi], use_fma);
            }
        }
    }
    if (with_copies) {
#pragma omp parallel for schedule(static)
        for (int64_t nn = 0; nn < n_rows; ++nn)
            for (int64_t ff = 0; ff < d; ++ff)
                out[nn * d + ff] = ro[((ff / F) * n_rows + nn) * F + ff % F];
        free(rs);
        free(ro);
    }
    return 0;
}

/* Same sums with rows handed out dynamically and no copies: not the reference's
 * schedule, reported only as a "best-effort CPU" figure next to the faithful one. */
static inline __attribute__((always_inline)) int fgo_spmm_csr_dynamic_impl(int64_t n_rows, int32_t d, const int32_t* indptr, const int32_t* indices,
                         const float* vals, const float* X, float* out, int use_fma) {
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t row = 0; row < n_rows; ++row) {
        float* o = out + row * d;
        for (int32_t f = 0; f < d; ++f) o[f] = 0.0f;
        for (int64_t e = indptr[row]; e < indptr[row + 1]; ++e) {
            const float v = vals[e];
            const float* x = X + (int64_t)indices[e] * d;
            for (int32_t f = 0; f < d; ++f) o[f] = mul_add(o[f], v, x[f], use_fma);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------
 * SpMM, DDS (1-D column partitioning).  python/featgraph/op/vanilla_spmm.py:195-224
 * with the schedule at :227-246.  s1_pos has P blocks of (n_rows + 1) positions,
 * s1_idx holds column ids local to the partition (global = local + k * ceil(n_cols / P),
 * :196, :208).  Per feature partition fo and per column partition k:
 *   Intermediate[fo][k][row][fi] = sum over that (k,row) segment, from 0, in order (:201-213)
 * and then ReshapedOut[fo][row][fi] = sum_k Intermediate[fo][k][row][fi], from 0, k ascending
 * (:215-218; Intermediate is computed at the k loop of ReshapedOut, :238).
 * Layout copies (:198-199, :220-222) do not change values and are left out here.
 * --------------------------------------------------------------------------------- */
static inline __attribute__((always_inline)) int fgo_spmm_dds_x86_impl(int64_t n_rows, int64_t n_cols, int32_t d, int32_t num_feat_partitions,
                     int32_t num_col_partitions, const int32_t* s1_pos, const int32_t* s1_idx,
                     const float* vals, const float* X, float* out, int use_fma) {
    const int64_t P = num_feat_partitions;
    const int64_t F = d / P;
    const int64_t K = num_col_partitions;
    const int64_t d2 = n_rows + 1;
    const int64_t cols_per_part = (n_cols + K - 1) / K;
    for (int64_t fo = 0; fo < P; ++fo) {
#pragma omp parallel
        {
            float* inter = (float*)malloc(sizeof(float) * (size_t)(F + 1));
#pragma omp for schedule(static)
            for (int64_t row = 0; row < n_rows; ++row) {
                float* o = out + row * d + fo * F;
                for (int64_t fi = 0; fi < F; ++fi) o[fi] = 0.0f;
                for (int64_t k = 0; k < K; ++k) {
                    for (int64_t fi = 0; fi < F; ++fi) inter[fi] = 0.0f;
                    for (int64_t e = s1_pos[k * d2 + row]; e < s1_pos[k * d2 + row + 1]; ++e) {
                        const float v = vals[e];
                        const float* x = X + ((int64_t)s1_idx[e] + k * cols_per_part) * d + fo * F;
                        for (int64_t fi = 0; fi < F; ++fi)
                            inter[fi] = mul_add(inter[fi], v, x[fi], use_fma);
                    }
                    for (int64_t fi = 0; fi < F; ++fi) o[fi] = o[fi] + inter[fi];
                }
            }
            free(inter);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------
 * SDDMM.  python/featgraph/op/vanilla_sddmm.py:43-62 with the x86 schedule at :66-74:
 *   out[e] = sum_k Src[col[e]][k] * Dst[row[e]][k]
 * Src is indexed by the COLUMN id and Dst by the ROW id (:47).  One thread (the
 * reference's x86 schedule has no parallel axis, :11, :73).  With feature
 * partitions the reduce axis is split and the outer part hoisted: fo -> e -> fi
 * (:70-72); k still ascends for each edge, so the values do not depend on it.
 * threads <= 1 runs the loop serially as the reference does; threads > 1 spreads
 * edges over OpenMP threads (a labelled extra, same values).
 * --------------------------------------------------------------------------------- */
static inline __attribute__((always_inline)) int fgo_sddmm_x86_impl(int64_t nnz, int32_t d, int32_t num_feat_partitions, const int32_t* row,
                  const int32_t* col, const float* src, const float* dst, float* out,
                  int use_fma, int threads) {
    const int64_t P = num_feat_partitions;
    const int64_t F = d / P;
    if (threads <= 1) {
        for (int64_t fo = 0; fo < P; ++fo) {
            for (int64_t e = 0; e < nnz; ++e) {
                const float* s = src + (int64_t)col[e] * d + fo * F;
                const float* t = dst + (int64_t)row[e] * d + fo * F;
                float acc = fo == 0 ? 0.0f : out[e];
                for (int64_t fi = 0; fi < F; ++fi) acc = mul_add(acc, s[fi], t[fi], use_fma);
                out[e] = acc;
            }
        }
        return 0;
    }
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t e = 0; e < nnz; ++e) {
        const float* s = src + (int64_t)col[e] * d;
        const float* t = dst + (int64_t)row[e] * d;
        float acc = 0.0f;
        for (int32_t k = 0; k < d; ++k) acc = mul_add(acc, s[k], t[k], use_fma);
        out[e] = acc;
    }
    return 0;
}

/* Exported entry points: each hands its implementation a literal use_fma. */
int fgo_spmm_csr_x86(int64_t n_rows, int64_t n_cols, int32_t d, int32_t num_feat_partitions,
    const int32_t* indptr, const int32_t* indices, const float* vals,
    const float* X, float* out, int use_fma, int with_copies) {
    return use_fma ? fgo_spmm_csr_x86_impl(n_rows, n_cols, d, num_feat_partitions, indptr, indices, vals, X, out, 1, with_copies)
                   : fgo_spmm_csr_x86_impl(n_rows, n_cols, d, num_feat_partitions, indptr, indices, vals, X, out, 0, with_copies);
}

int fgo_spmm_csr_dynamic(int64_t n_rows, int32_t d, const int32_t* indptr, const int32_t* indices,
    const float* vals, const float* X, float* out, int use_fma) {
    return use_fma ? fgo_spmm_csr_dynamic_impl(n_rows, d, indptr, indices, vals, X, out, 1)
                   : fgo_spmm_csr_dynamic_impl(n_rows, d, indptr, indices, vals, X, out, 0);
}

int fgo_spmm_dds_x86(int64_t n_rows, int64_t n_cols, int32_t d, int32_t num_feat_partitions,
    int32_t num_col_partitions, const int32_t* s1_pos, const int32_t* s1_idx,
    const float* vals, const float* X, float* out, int use_fma) {
    return use_fma ? fgo_spmm_dds_x86_impl(n_rows, n_cols, d, num_feat_partitions, num_col_partitions, s1_pos, s1_idx, vals, X, out, 1)
                   : fgo_spmm_dds_x86_impl(n_rows, n_cols, d, num_feat_partitions, num_col_partitions, s1_pos, s1_idx, vals, X, out, 0);
}

int fgo_sddmm_x86(int64_t nnz, int32_t d, int32_t num_feat_partitions, const int32_t* row,
    const int32_t* col, const float* src, const float* dst, float* out,
    int use_fma, int threads) {
    return use_fma ? fgo_sddmm_x86_impl(nnz, d, num_feat_partitions, row, col, src, dst, out, 1, threads)
                   : fgo_sddmm_x86_impl(nnz, d, num_feat_partitions, row, col, src, dst, out, 0, threads);
}
