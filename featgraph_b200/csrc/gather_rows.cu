// Row gather for the needed-rows exchange of the sharded layer: dst[i, :] = src[rows[i], :].
//
// When a graph's rows are spread over several GPUs, a shard's column ids reference only part of the
// feature matrix (on an R-MAT graph a fraction of it).  Each rank then sends every peer just the rows
// that peer asked for: this kernel packs them, in the peer's order, into one contiguous send buffer for
// the all-to-all.  The same kernel serves the exchange without a sender: src is then a peer GPU's feature
// block (symmetric memory mapped into this process) and the rank that needs the rows reads them itself over
// NVLink - plain loads, 64 warps per SM each with 512 bytes in flight.  One warp per row, 128-bit copies;
// d % 4 == 0 and 16-byte aligned buffers take the vector path, anything else a scalar one.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ src, int64_t ld_src,
                                                          const int64_t* __restrict__ rows, int64_t n,
                                                          int32_t d, float* __restrict__ dst, int64_t ld_dst,
                                                          bool vec) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) return;
    const float* s = src + rows[i] * ld_src;
    float* o = dst + i * ld_dst;
    if (vec) {
        for (int c = lane * 4; c < d; c += 128)
            *reinterpret_cast<float4*>(o + c) = fg::ld_stream(reinterpret_cast<const float4*>(s + c));
    } else {
        for (int c = lane; c < d; c += 32) o[c] = s[c];
    }
}

}  // namespace

extern "C" {

int fg_gather_rows_f32(const float* d_src, int64_t ld_src, const int64_t* d_rows, int64_t n_rows_out, int32_t d,
                       float* d_dst, int64_t ld_dst, void* stream) {
    if (n_rows_out < 0 || d < 1) return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n=%lld d=%d", (long long)n_rows_out, d);
    if (ld_src == 0) ld_src = d;
    if (ld_dst == 0) ld_dst = d;
    if (ld_src < d || ld_dst < d) return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides must be 0 or >= d=%d", d);
    if (n_rows_out == 0) return FG_OK;
    if (!d_src || !d_rows || !d_dst) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    const int64_t blocks = (n_rows_out + 7) / 8;
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    const bool vec = (d % 4 == 0) && (ld_src % 4 == 0) && (ld_dst % 4 == 0) && fg::aligned16(d_src) && fg::aligned16(d_dst);
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_src, ld_src, d_rows, n_rows_out,
                                                                                        d, d_dst, ld_dst, vec);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

}  // extern "C"
