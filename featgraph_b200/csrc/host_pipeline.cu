// Host-buffer entry points: features come from host memory and results go back to it, with the
// copies pipelined against the kernels.
//
// The reference's callers upload features with tvm.nd.array(x_np, ctx), run, and read the result
// with .asnumpy() (tests/test_module_spmm.py:50-52), three steps one after another.  Here the
// feature dimension is cut into column windows; window c+1 is copied in (copy-in stream) while
// window c is computed (the caller's stream) and window c-1 is copied out (copy-out stream), so
// a call costs about max(copy in, compute, copy out) instead of their sum.  The windows use the
// row-stride arguments of the device entry points; the sums are the same as in one call over
// all columns (SpMM) or the ascending-tile sum (SDDMM).
//
// The caller provides the device staging buffers (the library allocates no device memory here).
// Streams and events are created once per host thread and device and reused.
#include <vector>

#include "common.cuh"

namespace {

struct Pipeline {
    cudaStream_t in = nullptr, out = nullptr;
    std::vector<cudaEvent_t> events;
    size_t next = 0;

    int prepare() {
        if (!in) FG_CUDA_TRY(cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking));
        if (!out) FG_CUDA_TRY(cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking));
        // events are handed out round robin; 512 in rotation is far more than the calls that can be
        // in flight between two host synchronisations need (two per column window)
        if (next >= 512) next = 0;
        return FG_OK;
    }
    int event(cudaEvent_t* e) {
        if (next == events.size()) {
            cudaEvent_t ev;
            FG_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            events.push_back(ev);
        }
        *e = events[next++];
        return FG_OK;
    }
};

// One pipeline per host thread and device: a thread that alternates between devices finds its streams
// and events again when it returns to a device.
Pipeline* pipeline() {
    static thread_local Pipeline table[fg::kMaxDevices];
    const int dev = fg::current_device_slot();
    return dev < 0 ? nullptr : &table[dev];
}

// columns [c0, c0 + w) of a row-major [rows, d] matrix, host <-> device
cudaError_t copy_window(float* dst, const float* src, int64_t rows, int64_t d, int64_t c0, int64_t w,
                        cudaMemcpyKind kind, cudaStream_t s) {
    if (rows == 0 || w == 0) return cudaSuccess;
    if (w == d) return cudaMemcpyAsync(dst, src, sizeof(float) * rows * d, kind, s);
    return cudaMemcpy2DAsync(dst + c0, sizeof(float) * d, src + c0, sizeof(float) * d, sizeof(float) * w,
                             (size_t)rows, kind, s);
}

int window_width(int32_t d, int32_t chunk) {
    if (chunk > 0) return chunk < d ? chunk : d;
    // 64-float windows keep the gathered slice L2-sized on graphs of a few hundred thousand
    // nodes and give the pipeline several stages from d = 128 up
    return d >= 128 ? 64 : d;
}

#define FG_TRY_RC(expr)            \
    do {                           \
        const int rc__ = (expr);   \
        if (rc__ != FG_OK) return rc__; \
    } while (0)

}  // namespace

extern "C" {

int fg_spmm_csr_f32_host(const fg_row_schedule* schedule, const int32_t* d_indptr,
                         const int32_t* d_indices, const float* d_vals, const float* h_x, float* h_out,
                         float* d_x_staging, float* d_out_staging, int64_t n_rows, int64_t n_cols,
                         int64_t nnz, int32_t d, int32_t chunk, int32_t flags, void* stream) {
    if (d < 1 || n_rows < 0 || n_cols < 0)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld d=%d", (long long)n_rows,
                        (long long)n_cols, d);
    if (chunk < 0 || (chunk % 4 != 0)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "chunk must be 0 or a multiple of 4");
    if (n_rows == 0) return FG_OK;
    if (!h_out || !d_out_staging || (n_cols > 0 && (!h_x || !d_x_staging)))
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL host or staging buffer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Pipeline* pp = pipeline();
    if (!pp) return fg::fail(FG_ERR_CUDA, "no current CUDA device (or its ordinal is beyond %d)", fg::kMaxDevices);
    Pipeline& p = *pp;
    FG_TRY_RC(p.prepare());
    const int w = window_width(d, chunk);
    const bool deferred = (flags & FG_HOST_DEFERRED) != 0;
    if (!deferred) {
        // the staging buffers may still be in use by earlier work on the caller's stream.  A deferred
        // call does not wait (its copy-in is meant to run beside the previous call's kernels); there the
        // caller keeps the staging buffers of calls in flight apart, as the header says.
        cudaEvent_t start;
        FG_TRY_RC(p.event(&start));
        FG_CUDA_TRY(cudaEventRecord(start, s));
        FG_CUDA_TRY(cudaStreamWaitEvent(p.in, start, 0));
        FG_CUDA_TRY(cudaStreamWaitEvent(p.out, start, 0));
    }
    for (int c0 = 0; c0 < d; c0 += w) {
        const int wc = d - c0 < w ? d - c0 : w;
        cudaEvent_t in_done, k_done;
        FG_TRY_RC(p.event(&in_done));
        FG_TRY_RC(p.event(&k_done));
        FG_CUDA_TRY(copy_window(d_x_staging, h_x, n_cols, d, c0, wc, cudaMemcpyHostToDevice, p.in));
        FG_CUDA_TRY(cudaEventRecord(in_done, p.in));
        FG_CUDA_TRY(cudaStreamWaitEvent(s, in_done, 0));
        FG_TRY_RC(fg_spmm_csr_f32(schedule, d_indptr, d_indices, d_vals, d_x_staging + c0, d,
                                  d_out_staging + c0, d, n_rows, n_cols, nnz, wc, 0, stream));
        FG_CUDA_TRY(cudaEventRecord(k_done, s));
        FG_CUDA_TRY(cudaStreamWaitEvent(p.out, k_done, 0));
        FG_CUDA_TRY(copy_window(h_out, d_out_staging, n_rows, d, c0, wc, cudaMemcpyDeviceToHost, p.out));
    }
    if (deferred) return FG_OK;
    FG_CUDA_TRY(cudaStreamSynchronize(p.out));
    FG_CUDA_TRY(cudaStreamSynchronize(s));
    return FG_OK;
}

int fg_sddmm_coo_f32_host(const int32_t* d_row, const int32_t* d_col, const float* h_src,
                          const float* h_dst, float* h_out, float* d_src_staging, float* d_dst_staging,
                          float* d_out_staging, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                          int32_t rows_sorted, int32_t chunk, int32_t flags, void* stream) {
    if (d < 1 || n_rows < 0 || n_cols < 0 || nnz < 0)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (chunk < 0 || (chunk % 4 != 0)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "chunk must be 0 or a multiple of 4");
    if (nnz == 0) return FG_OK;
    // h_src == NULL: the column-side matrix is already on the device, in d_src_staging (e.g. uploaded by an SpMM
    // host call on the same features just before: a layer that runs both ops uploads them once)
    if (!h_dst || !h_out || !d_src_staging || !d_dst_staging || !d_out_staging)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL host or staging buffer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Pipeline* pp = pipeline();
    if (!pp) return fg::fail(FG_ERR_CUDA, "no current CUDA device (or its ordinal is beyond %d)", fg::kMaxDevices);
    Pipeline& p = *pp;
    FG_TRY_RC(p.prepare());
    const int w = window_width(d, chunk);
    const bool deferred = (flags & FG_HOST_DEFERRED) != 0;
    if (!deferred) {  // as above
        cudaEvent_t start;
        FG_TRY_RC(p.event(&start));
        FG_CUDA_TRY(cudaEventRecord(start, s));
        FG_CUDA_TRY(cudaStreamWaitEvent(p.in, start, 0));
    }
    for (int c0 = 0; c0 < d; c0 += w) {
        const int wc = d - c0 < w ? d - c0 : w;
        cudaEvent_t in_done;
        FG_TRY_RC(p.event(&in_done));
        if (h_src) FG_CUDA_TRY(copy_window(d_src_staging, h_src, n_cols, d, c0, wc, cudaMemcpyHostToDevice, p.in));
        FG_CUDA_TRY(copy_window(d_dst_staging, h_dst, n_rows, d, c0, wc, cudaMemcpyHostToDevice, p.in));
        FG_CUDA_TRY(cudaEventRecord(in_done, p.in));
        FG_CUDA_TRY(cudaStreamWaitEvent(s, in_done, 0));
        FG_TRY_RC(fg_sddmm_coo_f32(d_row, d_col, d_src_staging + c0, d, d_dst_staging + c0, d, d_out_staging,
                                   n_rows, n_cols, nnz, wc, rows_sorted, c0 > 0 ? 1 : 0, 0, stream));
    }
    // the result leaves on the copy-out stream, so that a following call's kernels need not wait for it
    cudaEvent_t k_done;
    FG_TRY_RC(p.event(&k_done));
    FG_CUDA_TRY(cudaEventRecord(k_done, s));
    FG_CUDA_TRY(cudaStreamWaitEvent(p.out, k_done, 0));
    FG_CUDA_TRY(cudaMemcpyAsync(h_out, d_out_staging, sizeof(float) * nnz, cudaMemcpyDeviceToHost, p.out));
    if (deferred) return FG_OK;
    FG_CUDA_TRY(cudaStreamSynchronize(p.out));
    FG_CUDA_TRY(cudaStreamSynchronize(s));
    return FG_OK;
}

int fg_sddmm_coo_f32_planned_host(const fg_sddmm_plan* plan, const int32_t* d_col, const float* d_src, const float* h_dst,
                                  float* h_out, float* d_dst_staging, float* d_out_staging, int64_t n_rows, int64_t n_cols,
                                  int64_t nnz, int32_t d, int32_t flags, void* stream) {
    if (d < 1 || n_rows < 0 || n_cols < 0 || nnz < 0)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (nnz == 0) return FG_OK;
    if (!plan || !d_src || !h_dst || !h_out || !d_dst_staging || !d_out_staging)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL plan, host or staging buffer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Pipeline* pp = pipeline();
    if (!pp) return fg::fail(FG_ERR_CUDA, "no current CUDA device (or its ordinal is beyond %d)", fg::kMaxDevices);
    Pipeline& p = *pp;
    FG_TRY_RC(p.prepare());
    const bool deferred = (flags & FG_HOST_DEFERRED) != 0;
    if (!deferred) {  // the staging buffers may still be in use by earlier work on the caller's stream
        cudaEvent_t start;
        FG_TRY_RC(p.event(&start));
        FG_CUDA_TRY(cudaEventRecord(start, s));
        FG_CUDA_TRY(cudaStreamWaitEvent(p.in, start, 0));
    }
    // the one-pass kernel needs whole rows: the row-side matrix goes in as one copy, beside whatever the
    // caller's stream is still computing; the column side is on the device already
    cudaEvent_t in_done, k_done;
    FG_TRY_RC(p.event(&in_done));
    FG_TRY_RC(p.event(&k_done));
    FG_CUDA_TRY(copy_window(d_dst_staging, h_dst, n_rows, d, 0, d, cudaMemcpyHostToDevice, p.in));
    FG_CUDA_TRY(cudaEventRecord(in_done, p.in));
    FG_CUDA_TRY(cudaStreamWaitEvent(s, in_done, 0));
    FG_TRY_RC(fg_sddmm_coo_f32_planned(plan, d_col, d_src, d, d_dst_staging, d, d_out_staging, n_rows, n_cols, nnz, d, 0,
                                       stream));
    FG_CUDA_TRY(cudaEventRecord(k_done, s));
    FG_CUDA_TRY(cudaStreamWaitEvent(p.out, k_done, 0));
    FG_CUDA_TRY(cudaMemcpyAsync(h_out, d_out_staging, sizeof(float) * nnz, cudaMemcpyDeviceToHost, p.out));
    if (deferred) return FG_OK;
    FG_CUDA_TRY(cudaStreamSynchronize(p.out));
    FG_CUDA_TRY(cudaStreamSynchronize(s));
    return FG_OK;
}

int fg_host_sync(void* stream) {
    Pipeline* p = pipeline();
    if (p && p->in) FG_CUDA_TRY(cudaStreamSynchronize(p->in));
    FG_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (p && p->out) FG_CUDA_TRY(cudaStreamSynchronize(p->out));
    return FG_OK;
}

}  // extern "C"
