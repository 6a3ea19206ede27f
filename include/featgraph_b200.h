/*
 * featgraph_b200 - C ABI of the sm_100a SpMM / SDDMM library (libfeatgraph_b200.so).
 *
 * What this boundary replaces.  The reference builds each kernel with its code
 * generator and then calls the resulting packed function with positional array
 * arguments, destination last:
 *     SpMM  : func(SrcFeat, indptr, indices, vals, Out)        python/featgraph/module/spmm.py:108-109,159-160
 *     SpMM  : func(SrcFeat, s1_pos, s1_idx, vals, Out)  (DDS)  python/featgraph/module/spmm.py:100-101,156-157
 *     SDDMM : func(SrcFeat, DstFeat, row, col, Out)            python/featgraph/module/sddmm.py:89-90,128
 * The entry points below take the same arrays as plain pointers plus explicit sizes.
 *
 * Conventions
 *  - Every pointer named d_* is a DEVICE pointer on the current CUDA device; h_* is a host
 *    pointer.  int32 index arrays and fp32 values, as the reference keeps scipy's dtypes
 *    (module/spmm.py:59-64).  Feature matrices are dense row-major; the row stride is d unless a
 *    stride argument says otherwise.
 *  - The caller owns every array.  The library owns only the fg_row_schedule / fg_sddmm_plan objects it
 *    hands out (freed by their destroy calls), a pair of copy streams and a pool of events per host
 *    thread that uses the host-buffer calls, and one static scratch array (fg_spmm_csr_f32_static).
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Device
 *    entry points only enqueue work on it; they do not synchronise.
 *  - Return value: FG_OK or an FG_ERR_* code; fg_last_error() gives the text for the
 *    calling thread.  Nothing aborts or traps.  Arguments are checked on the host only:
 *    index arrays are trusted to be in range (fg_csr_validate / fg_coo_validate check them).
 *  - Arithmetic: fp32.  SpMM (all entry points) and fg_sddmm_coo_f32_exact round product and
 *    sum separately (no fused multiply-add) and add in storage / ascending-k order: the values of
 *    the reference's x86 loops, bit for bit, whatever the launch parameters.  fg_sddmm_coo_f32
 *    sums each dot product as a fixed tree of FMAs (within fp32 rounding of d terms of that).
 *  - Re-entrant; the mutable global state is the thread-local error text, the per-thread copy
 *    streams, a launch counter and the static scratch array of fg_spmm_csr_f32_static.
 */
#ifndef FEATGRAPH_B200_H_
#define FEATGRAPH_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FG_OK 0
#define FG_ERR_INVALID_ARGUMENT 1
#define FG_ERR_CUDA 2
#define FG_ERR_OUT_OF_MEMORY 3
#define FG_ERR_BAD_INDEX 4

/* Library version (major*10000 + minor*100 + patch). */
int fg_version(void);

/* Compile-time shapes of the hot kernels in this build (lane layouts, gathers in flight, ring depths) as
 * one short string.  Measurements that were taken from one build of the kernels (profiler counters kept
 * beside a benchmark) carry this string, so that a reader can tell whether they still describe the
 * kernels that ran.  No counterpart in the reference (its kernels are generated per call). */
const char* fg_kernel_signature(void);

/* Text of the last error raised on the calling thread ("" if none). Never NULL. */
const char* fg_last_error(void);

/* How many SpMM / SDDMM kernels this library has launched in this process so far (the
 * reference's timer counts calls of the built function, module/spmm.py:179; this counts the
 * launches behind them). */
int64_t fg_kernel_launch_count(void);

/* Number of SMs, compute capability and L2 size of the current device.
 * Replaces the reference's device handle query (tvm.gpu(0), module/spmm.py:218). */
int fg_device_info(int32_t* sm_count, int32_t* cc_major, int32_t* cc_minor, int64_t* l2_bytes);

/* --------------------------------------------------------------------------------------
 * Row schedule: the order in which SpMM visits rows (heaviest rows first, ties in
 * row order).  It takes the place of the reference's launch-shape knobs
 * num_cuda_blocks / num_threads_per_cuda_block (python/featgraph/op/vanilla_spmm.py:128-146),
 * which only choose how rows map to blocks.  Built once per adjacency on the device; holds
 * 12 bytes of device memory per row: the row ids in visiting order and, beside each, a copy of
 * that row's (first nonzero, count) taken from d_indptr.  The kernels read those copies instead of
 * the position array of the call, so a schedule belongs to the exact d_indptr it was built from:
 * rebuild it when the adjacency changes.  A call whose nnz differs from the schedule's is refused
 * (FG_ERR_INVALID_ARGUMENT).  With the matching adjacency the schedule never changes a result bit.
 * -------------------------------------------------------------------------------------- */
typedef struct fg_row_schedule fg_row_schedule;

/* d_indptr: n_rows+1 ascending positions.  long_row_threshold: 0 = each SpMM launch decides
 * which rows count as long and which as heavy (see fg_spmm_csr_f32); > 0 fixes it: rows with at
 * least that many nonzeros always take the long-row kernel, rows with at least 16 times as many
 * the heavy-row kernel (INT32_MAX = none ever do); < 0 fixes |long_row_threshold| in the same way
 * and selects the 8-warp form of the heavy-row kernel instead of the 4-warp one.  Every setting
 * gives the same result bits.  Synchronises `stream` before returning. */
int fg_row_schedule_create(const int32_t* d_indptr, int64_t n_rows, int32_t long_row_threshold,
                           void* stream, fg_row_schedule** out_schedule);
/* Device pointer to the n_rows row ids in visiting order (valid until destroy). */
const int32_t* fg_row_schedule_order(const fg_row_schedule* schedule);
int64_t fg_row_schedule_num_rows(const fg_row_schedule* schedule);
/* Number of rows with at least min_nnz nonzeros, for min_nnz a power of two in 64..2^21 or the
 * fixed threshold given at creation; -1 for any other value. */
int64_t fg_row_schedule_rows_at_least(const fg_row_schedule* schedule, int64_t min_nnz);
void fg_row_schedule_destroy(fg_row_schedule* schedule);

/* --------------------------------------------------------------------------------------
 * SpMM, CSR:  out[r, f] = sum_{e in [indptr[r], indptr[r+1])} vals[e] * x[indices[e], f]
 * Replaces the function built from vanilla_spmm_csr_x86 / vanilla_spmm_csr_cuda
 * (python/featgraph/op/vanilla_spmm.py:6-62, 83-125) and called at module/spmm.py:159-160.
 *   d_vals     NULL means every adjacency value is 1.0 (an unweighted graph, as the reference's
 *              dataset script stores it, benchmark/download_reddit_dataset.py:11): the value array is
 *              then neither read nor multiplied in (1.0 * x == x exactly, so the result bits are
 *              those of an all-ones value array).  Also accepted by the DDS and static entry points.
 *   schedule   NULL = visit rows in index order, one kernel.  With a schedule, rows are visited
 *              heaviest first and each launch may hand its longest rows to two further kernels
 *              (long rows: one warp per row and 32-float tile, slices staged through a
 *              shared-memory ring; heavy rows: one block per row and tile, its warps taking
 *              turns).  When no 32-float slice of x can stay in L2 those kernels run on an
 *              internal second stream beside the main one, forked from and joined to `stream`
 *              by events (legal under stream capture; the streams and events are created on a
 *              host thread's first such call per device, so make that call outside a capture).
 *              No effect on the values, provided the schedule was built from this d_indptr.
 *   feat_tile  width in floats of the feature slice handled per pass over the rows
 *              (power of two, 4..128), 0 = choose from n_cols and the L2 size.  It is the
 *              reference's num_feat_partitions idea (op/vanilla_spmm.py:41-44) used to keep
 *              the gathered slice of x resident in L2.  No effect on the values.
 *   ldx, ldo   row strides of x and out in floats (0 = d).  A stride larger than d computes a
 *              window of d columns of wider matrices: pass x + c0 and out + c0 to work on columns
 *              [c0, c0 + d).  Column windows are how the host-buffer calls below pipeline copies
 *              against compute.
 * x: [n_cols, d], out: [n_rows, d].  Any d >= 1; 128-bit gathers need d, ldx, ldo % 4 == 0 and
 * 16-byte aligned x / out, otherwise a scalar kernel runs.
 * -------------------------------------------------------------------------------------- */
int fg_spmm_csr_f32(const fg_row_schedule* schedule, const int32_t* d_indptr,
                    const int32_t* d_indices, const float* d_vals, const float* d_x, int64_t ldx,
                    float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                    int32_t feat_tile, void* stream);

/* SpMM, DDS (column-partitioned CSR made by util_convert_csr_to_dds,
 * python/featgraph/util/adj_partitioning.py:7-57):
 *   out[r, f] = sum_{k < num_col_partitions} ( sum_{e in segment(k, r)} vals[e] * x[s1_idx[e] + k*w, f] )
 * with w = ceil(n_cols / num_col_partitions) and segment(k, r) =
 * [s1_pos[k*(n_rows+1) + r], s1_pos[k*(n_rows+1) + r + 1]).  Inner sums start at 0 and run in
 * storage order, the outer sum starts at 0 and adds partitions in ascending k: the
 * association of vanilla_spmm_dds_x86 (op/vanilla_spmm.py:195-218), called at
 * module/spmm.py:156-157. */
int fg_spmm_dds_f32(const fg_row_schedule* schedule, const int32_t* d_s1_pos,
                    const int32_t* d_s1_idx, const float* d_vals, const float* d_x, int64_t ldx,
                    float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                    int32_t num_col_partitions, int32_t feat_tile, void* stream);

/* --------------------------------------------------------------------------------------
 * Aggregate, then score, in one pass over the rows (one GCN-style layer step):
 *     h = A . x                              the values (bits) of fg_spmm_csr_f32
 *     edge_out[e] = dot(h[row e], y[col e])  for the nonzeros in CSR order, as fg_sddmm_coo_f32 sums it
 * It replaces the two built functions a caller of the reference runs back to back for this step
 * (python/featgraph/module/spmm.py:159-160, then python/featgraph/module/sddmm.py:128 with the SpMM output
 * as the row-side input).  The lanes that have just finished a row of h still hold it in registers and
 * score the row's edges at once: h is not read back, the row ids are not walked a second time.
 * x, y: [n_cols, d]; h: [n_rows, d] (always written); edge_out: [nnz].  d <= 128 and a multiple of 4, all
 * matrices 16-byte aligned with strides that are multiples of 4 (0 = d).  d_vals may be NULL (all ones).
 * With a schedule (built from this d_indptr) long rows take the ring kernels for h and a kernel of their
 * own for their edges, on internal streams forked from and joined to `stream` as in fg_spmm_csr_f32.
 * -------------------------------------------------------------------------------------- */
int fg_spmm_sddmm_fused_f32(const fg_row_schedule* schedule, const int32_t* d_indptr, const int32_t* d_indices,
                            const float* d_vals, const float* d_x, int64_t ldx, const float* d_y, int64_t ldy,
                            float* d_h, int64_t ldh, float* d_edge_out, int64_t n_rows, int64_t n_cols, int64_t nnz,
                            int32_t d, void* stream);

/* --------------------------------------------------------------------------------------
 * SpMM, CSR, without any device allocation (no counterpart in the reference; it exists for
 * callers that cannot tolerate a cudaMalloc - a process whose own pool already owns all device
 * memory, or a latency-critical loop that must not hit the device-wide synchronisation an
 * allocation implies).  Same arguments, same result bits as fg_spmm_csr_f32, but no
 * fg_row_schedule: the row order is rebuilt on every call inside a fixed device array that the
 * library image carries (about 4 MB, resident on every GPU that loads the library until exit).
 *  - At most FG_SPMM_STATIC_MAX_ROWS rows; more is refused with FG_ERR_INVALID_ARGUMENT.
 *  - Calls no cudaMalloc, no cudaFree and no other allocating routine.  The first call on each device looks up
 *    the array's device address (cudaGetSymbolAddress); make that first call outside any stream
 *    capture.
 *  - All calls on a device share the one array (its counters are cleared at the start of each
 *    call): two calls that overlap on the GPU - different streams, no ordering between them -
 *    race on it.  Calls on one stream are safe.
 * -------------------------------------------------------------------------------------- */
#define FG_SPMM_STATIC_MAX_ROWS 1048576
int fg_spmm_csr_f32_static(const int32_t* d_indptr, const int32_t* d_indices, const float* d_vals,
                           const float* d_x, float* d_out, int64_t n_rows, int64_t n_cols,
                           int64_t nnz, int32_t d, int32_t feat_tile, void* stream);

/* --------------------------------------------------------------------------------------
 * SDDMM, COO:  out[e] = sum_k src[col[e], k] * dst[row[e], k]
 * (src is indexed by the COLUMN id, dst by the ROW id: python/featgraph/op/vanilla_sddmm.py:47).
 * Replaces the function built from vanilla_sddmm (op/vanilla_sddmm.py:6-63) and called at
 * module/sddmm.py:128.  Edges may come in any order; out keeps that order.
 *   rows_sorted  non-zero promises that d_row is non-decreasing (a CSR-ordered edge list):
 *                the row-side feature row is then kept in registers across a row's edges.
 *                Zero is always safe.
 *   ld_src, ld_dst  row strides in floats (0 = d); larger strides select a window of d columns
 *                of wider matrices (pass src + c0, dst + c0).
 *   accumulate   non-zero adds the dot products to what out already holds (a caller walking
 *                column windows passes 0 for the first window and 1 afterwards).
 *   feat_tile    width in floats of the feature slice handled per pass over the edges (power
 *                of two, 4..512), 0 = the whole row if the column-side matrix fits in L2, else
 *                the widest slice that does.  With more than one pass, pass t > 0 adds its
 *                partial dot product to out[e]: the reference's num_feat_partitions loop
 *                order (op/vanilla_sddmm.py:70-72).
 * src: [n_cols, d], dst: [n_rows, d], out: [nnz].  The dot product is summed with FMAs as a
 * fixed tree (per-lane partial sums, then a butterfly; tiles in ascending order), not in
 * ascending k; the difference from the sequential sum is bounded by fp32 rounding of d terms.
 * -------------------------------------------------------------------------------------- */
int fg_sddmm_coo_f32(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src,
                     const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                     int64_t nnz, int32_t d, int32_t rows_sorted, int32_t accumulate, int32_t feat_tile,
                     void* stream);

/* --------------------------------------------------------------------------------------
 * SDDMM in one pass over column blocks, for feature matrices too large for L2.
 * fg_sddmm_coo_f32 keeps its gathers in L2 by walking the whole edge list once per feature tile.  This
 * call cuts the COLUMN range instead - num_col_partitions blocks of ceil(n_cols / P) columns, the column
 * blocks of the reference's 2-D edge partitioning (python/featgraph/util/adj_partitioning.py:100-101,
 * the num_col_partitions knob of VanillaSDDMMx86, module/sddmm.py:169) used as a traversal order - and
 * visits the edges block by block, so that only ceil(n_cols / P) whole rows of src are gathered from at
 * a time.  Every edge is visited once: ids are read once, out[e] is written once.  Unlike the reference's
 * partitioning nothing is permuted: out keeps the caller's edge order, no edge_mapping is needed.
 *   plan   built once per adjacency by fg_sddmm_plan_create from the SAME d_row / d_col the calls use
 *          (16 bytes of device memory per 32 edges plus 16 per non-empty (block, row) run).  It needs
 *          a CSR-ordered edge list: rows non-decreasing, column ids ascending within a row; anything
 *          else is refused with FG_ERR_INVALID_ARGUMENT (use fg_sddmm_coo_f32).  Synchronises `stream`.
 *   fg_sddmm_auto_partitions   the block count that makes one block of src (ceil(n_cols / P) rows of d
 *          floats) fit the share of L2 that stays resident, or 1 where fg_sddmm_coo_f32 is the better
 *          call: the matrix fits L2 anyway, d > 512, d % 4 != 0, or rows so short that a (block, row)
 *          run would hold only a few edges.
 * The planned call needs d <= 512, d and the strides multiples of 4, 16-byte aligned matrices.
 * Values: FMAs within a lane, a fixed tree across the 32 lanes of a warp; within fp32 rounding of d terms
 * of the sequential sum (and of fg_sddmm_coo_f32, whose tree differs).
 * -------------------------------------------------------------------------------------- */
typedef struct fg_sddmm_plan fg_sddmm_plan;
int32_t fg_sddmm_auto_partitions(int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d);
int fg_sddmm_plan_create(const int32_t* d_row, const int32_t* d_col, int64_t n_rows, int64_t n_cols,
                         int64_t nnz, int32_t num_col_partitions, void* stream, fg_sddmm_plan** out_plan);
int32_t fg_sddmm_plan_partitions(const fg_sddmm_plan* plan);
/* Number of 32-edge batches the plan holds. */
int64_t fg_sddmm_plan_batches(const fg_sddmm_plan* plan);
void fg_sddmm_plan_destroy(fg_sddmm_plan* plan);
int fg_sddmm_coo_f32_planned(const fg_sddmm_plan* plan, const int32_t* d_col, const float* d_src, int64_t ld_src,
                             const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                             int64_t nnz, int32_t d, int32_t accumulate, void* stream);

/* SDDMM with the reference's x86 summation order, bit for bit: every product and every sum
 * rounded separately, k strictly ascending (python/featgraph/op/vanilla_sddmm.py:43-62 with the
 * loop order of :66-74).  Same arrays and strides as fg_sddmm_coo_f32; accumulate != 0 continues
 * the sequential sum from what out holds (column windows in ascending order then still give the
 * sequential sum over all columns).  Three to four times slower than fg_sddmm_coo_f32. */
int fg_sddmm_coo_f32_exact(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src,
                           const float* d_dst, int64_t ld_dst, float* d_out, int64_t n_rows, int64_t n_cols,
                           int64_t nnz, int32_t d, int32_t accumulate, void* stream);

/* --------------------------------------------------------------------------------------
 * Host-buffer calls: features in HOST memory (h_*), results back to HOST memory, adjacency
 * already on the device.  They replace the three steps a caller of the reference performs
 * around the built function - tvm.nd.array(x_np, ctx), func(...), out.asnumpy()
 * (tests/test_module_spmm.py:50-52, tests/test_module_sddmm.py:57-62) - and overlap them: the
 * feature dimension is cut into column windows of `chunk` floats (0 = 64 for d >= 128, else one
 * window), window c+1 is copied in while window c is computed and window c-1 is copied out.
 * The caller supplies device staging buffers of the full shapes (d_*_staging); no device memory
 * is allocated.  Pinned host memory gives full copy speed, pageable memory works.  The call
 * returns when the host result is complete (it synchronises `stream`).  Values: SpMM as
 * fg_spmm_csr_f32; SDDMM as fg_sddmm_coo_f32 with feat_tile = chunk.
 *   flags  0, or FG_HOST_DEFERRED: enqueue everything and return at once; the host result is
 *          complete after fg_host_sync(stream) on the same host thread.  Deferred calls let the
 *          copy-out of one call overlap the copy-in and kernels of the next.  The caller promises
 *          that the staging buffers of a deferred call are not touched by anything else (another
 *          call with the same buffers included) until that fg_host_sync.
 *   h_src  of the SDDMM call may be NULL: the column-side matrix is then taken as already present in
 *          d_src_staging, complete by the time `stream` reaches this call - e.g. the d_x_staging of an SpMM host
 *          call on the same features enqueued just before, so that a layer running both ops uploads them once.
 * -------------------------------------------------------------------------------------- */
#define FG_HOST_DEFERRED 1
int fg_spmm_csr_f32_host(const fg_row_schedule* schedule, const int32_t* d_indptr,
                         const int32_t* d_indices, const float* d_vals, const float* h_x, float* h_out,
                         float* d_x_staging, float* d_out_staging, int64_t n_rows, int64_t n_cols,
                         int64_t nnz, int32_t d, int32_t chunk, int32_t flags, void* stream);
int fg_sddmm_coo_f32_host(const int32_t* d_row, const int32_t* d_col, const float* h_src,
                          const float* h_dst, float* h_out, float* d_src_staging, float* d_dst_staging,
                          float* d_out_staging, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                          int32_t rows_sorted, int32_t chunk, int32_t flags, void* stream);
/* The host-buffer form of fg_sddmm_coo_f32_planned for a column-side matrix that is already on the device
 * (d_src, dense rows of d floats): the row-side matrix is copied in whole beside the caller's earlier work, the
 * one-pass kernel runs, the result leaves on the copy-out stream.  flags as above. */
int fg_sddmm_coo_f32_planned_host(const fg_sddmm_plan* plan, const int32_t* d_col, const float* d_src, const float* h_dst,
                                  float* h_out, float* d_dst_staging, float* d_out_staging, int64_t n_rows, int64_t n_cols,
                                  int64_t nnz, int32_t d, int32_t flags, void* stream);
/* Wait until every host-buffer call issued by this host thread (on `stream` and on the library's
 * copy streams) has finished. */
int fg_host_sync(void* stream);

/* --------------------------------------------------------------------------------------
 * Generalized forms (off the benchmarked path).  The reference checkout has none: its README (lines 9-11)
 * only points to a branch with "generalized SpMM and generalized SDDMM w/ broadcasting", so the semantics are
 * stated here rather than matched:
 *   fg_spmm_csr_reduce_f32   out[r, f] = reduce over the row's nonzeros of vals[e] * x[indices[e], f], with
 *                            reduce = FG_REDUCE_MAX, FG_REDUCE_MIN or FG_REDUCE_MEAN (the sum in storage order,
 *                            divided by the row's nonzero count).  A row without nonzeros gives 0.  d_vals may
 *                            be NULL (all ones).  The sum itself is fg_spmm_csr_f32.
 *   fg_edge_binary_f32       out[e, f] = src[col[e], f] (op) dst[row[e], f] with op = FG_EDGE_ADD, FG_EDGE_SUB or
 *                            FG_EDGE_MUL: a vector per edge, [nnz, d] (the dot product of FG_EDGE_MUL's rows is
 *                            fg_sddmm_coo_f32).  Edges in any order.
 * Strides in floats (0 = d); any d; 128-bit accesses where d, the strides and the bases allow.
 * -------------------------------------------------------------------------------------- */
#define FG_REDUCE_MAX 1
#define FG_REDUCE_MIN 2
#define FG_REDUCE_MEAN 3
#define FG_EDGE_ADD 0
#define FG_EDGE_SUB 1
#define FG_EDGE_MUL 2
int fg_spmm_csr_reduce_f32(const int32_t* d_indptr, const int32_t* d_indices, const float* d_vals, const float* d_x,
                           int64_t ldx, float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                           int32_t reduce, void* stream);
int fg_edge_binary_f32(const int32_t* d_row, const int32_t* d_col, const float* d_src, int64_t ld_src, const float* d_dst,
                       int64_t ld_dst, float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                       int32_t op, void* stream);

/* --------------------------------------------------------------------------------------
 * Row gather: dst[i, :] = src[rows[i], :] for i < n_rows_out (int64 row ids on the device, trusted to be in
 * range).  Plumbing of the multi-GPU layer, which has no counterpart in the reference (its modules are
 * single-device, module/spmm.py:218): a rank packs the feature rows each peer's shard references into one
 * send buffer for an all-to-all, instead of every rank receiving every row; or, the other way round, a rank
 * fetches the rows it needs itself: d_src may be another GPU's memory mapped into this process (peer access
 * over NVLink; the kernel reads it with plain loads), d_rows and d_dst this GPU's.  Strides in floats (0 = d).
 * -------------------------------------------------------------------------------------- */
int fg_gather_rows_f32(const float* d_src, int64_t ld_src, const int64_t* d_rows, int64_t n_rows_out, int32_t d,
                       float* d_dst, int64_t ld_dst, void* stream);

/* --------------------------------------------------------------------------------------
 * Index checks (the code generator of the reference emits shape asserts only; these add
 * the range checks that keep a bad adjacency from reading out of bounds).  Both
 * synchronise `stream` and return FG_ERR_BAD_INDEX with a message naming the first kind
 * of violation found.  *rows_sorted (may be NULL) reports whether d_row is non-decreasing.
 * -------------------------------------------------------------------------------------- */
int fg_csr_validate(const int32_t* d_indptr, const int32_t* d_indices, int64_t n_rows,
                    int64_t n_cols, int64_t nnz, void* stream);
int fg_coo_validate(const int32_t* d_row, const int32_t* d_col, int64_t n_rows, int64_t n_cols,
                    int64_t nnz, int32_t* rows_sorted, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FEATGRAPH_B200_H_ */
