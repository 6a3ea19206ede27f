// Seeded synthetic-graph and feature generators (host code, OpenMP).
//
// These stand in for the adjacency file the reference's benchmarks load
// (benchmark/download_reddit_dataset.py:9-17 writes a CSR / COO .npz of the Reddit
// graph: 232,965 nodes, 114,615,892 edges), which needs a network download.  Every
// value is a pure function of (seed, row or edge number, draw number), so the output
// does not depend on the number of threads and the same arrays can be handed to the
// GPU path and to a CPU checker.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#include <parallel/algorithm>
#endif

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

inline uint64_t mix64(uint64_t x) {
    x += kGolden;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// draw number j of stream `a` under `seed`
inline uint64_t draw64(uint64_t seed, uint64_t a, uint64_t j) {
    const uint64_t base = mix64(mix64(seed) ^ (a * 0xD1342543DE82EF95ull + 1));
    return mix64(base + j * kGolden);
}

// uniform integer in [0, n) by multiply-shift on the top 32 bits (n < 2^31)
inline uint32_t bounded(uint64_t h, uint32_t n) {
    return (uint32_t)(((h >> 32) * (uint64_t)n) >> 32);
}

}  // namespace

extern "C" {

int fg_gen_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// out[i] = 2*u - 1 with u a 24-bit uniform in [0,1): fp32 values in [-1, 1).
void fg_gen_uniform_f32(uint64_t seed, int64_t count, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const uint32_t u = (uint32_t)(draw64(seed, (uint64_t)i >> 20, (uint64_t)i & 0xFFFFF) >> 40);
        out[i] = (float)u * (2.0f / 16777216.0f) - 1.0f;
    }
}

// 53-bit uniforms in [0,1) (used for degree draws on the Python side).
void fg_gen_uniform_f64(uint64_t seed, int64_t count, double* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i)
        out[i] = (double)(draw64(seed, (uint64_t)i >> 20, (uint64_t)i & 0xFFFFF) >> 11) *
                 (1.0 / 9007199254740992.0);
}

// Row r receives the first (indptr[r+1]-indptr[r]) DISTINCT values of its draw
// sequence bounded(draw64(seed, r, 0)), bounded(draw64(seed, r, 1)), ... over
// [0, n_cols), written in ascending order: uniform neighbours without replacement,
// sorted CSR.  Returns 0, or 1 if a row asks for more than n_cols neighbours.
//
// row_offset: id of the first row, so that a slice of rows [row_offset, row_offset + n_rows)
// of a larger graph can be generated alone and comes out identical to that slice.
int fg_gen_neighbors(uint64_t seed, int64_t row_offset, int64_t n_rows, int64_t n_cols,
                     const int64_t* indptr, int32_t* indices) {
    for (int64_t r = 0; r < n_rows; ++r)
        if (indptr[r + 1] - indptr[r] > n_cols || indptr[r + 1] < indptr[r]) return 1;
    const int64_t words = (n_cols + 63) / 64;
#pragma omp parallel
    {
        std::vector<uint64_t> bits((size_t)words, 0);
        std::vector<int32_t> small;
#pragma omp for schedule(dynamic, 64)
        for (int64_t r = 0; r < n_rows; ++r) {
            const int64_t deg = indptr[r + 1] - indptr[r];
            int32_t* dst = indices + indptr[r];
            if (deg == 0) continue;
            uint64_t j = 0;
            if (deg * 64 < n_cols) {
                // few neighbours: keep them in a small sorted vector
                small.clear();
                while ((int64_t)small.size() < deg) {
                    const int32_t c = (int32_t)bounded(draw64(seed, (uint64_t)(row_offset + r), j++), (uint32_t)n_cols);
                    auto it = std::lower_bound(small.begin(), small.end(), c);
                    if (it == small.end() || *it != c) small.insert(it, c);
                }
                std::memcpy(dst, small.data(), sizeof(int32_t) * (size_t)deg);
            } else {
                int64_t have = 0;
                while (have < deg) {
                    const uint32_t c = bounded(draw64(seed, (uint64_t)(row_offset + r), j++), (uint32_t)n_cols);
                    uint64_t& w = bits[c >> 6];
                    const uint64_t m = 1ull << (c & 63);
                    if (!(w & m)) { w |= m; ++have; }
                }
                int64_t k = 0;
                for (int64_t wi = 0; wi < words; ++wi) {
                    uint64_t w = bits[(size_t)wi];
                    bits[(size_t)wi] = 0;
                    while (w) {
                        dst[k++] = (int32_t)(wi * 64 + __builtin_ctzll(w));
                        w &= w - 1;
                    }
                }
            }
        }
    }
    return 0;
}

// R-MAT: edge i takes `scale` quadrant draws with probabilities (a, b, c, 1-a-b-c);
// quadrant b sets the column bit, c the row bit, d both.  Self-loops and duplicate
// edges are dropped and the rest is written as sorted CSR over 2^scale vertices.
// indices must have room for n_edges entries.  Returns the number of edges kept.
int64_t fg_gen_rmat_csr(uint64_t seed, int32_t scale, int64_t n_edges, double a, double b, double c,
                        int32_t* indptr, int32_t* indices) {
    const int64_t n = (int64_t)1 << scale;
    std::vector<uint64_t> keys((size_t)n_edges);
    const uint64_t ta = (uint64_t)(a * 4294967296.0);
    const uint64_t tb = (uint64_t)((a + b) * 4294967296.0);
    const uint64_t tc = (uint64_t)((a + b + c) * 4294967296.0);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_edges; ++i) {
        uint64_t r = 0, col = 0;
        uint64_t h = 0;
        for (int32_t l = 0; l < scale; ++l) {
            // one 64-bit draw feeds two levels (32 bits each)
            if ((l & 1) == 0) h = draw64(seed, (uint64_t)i, (uint64_t)(l >> 1));
            const uint64_t u = (l & 1) ? (h & 0xFFFFFFFFull) : (h >> 32);
            const uint64_t q = (u >= ta) + (u >= tb) + (u >= tc);  // 0:a 1:b 2:c 3:d
            r = (r << 1) | (q >> 1);
            col = (col << 1) | (q & 1);
        }
        keys[(size_t)i] = (r == col) ? ~0ull : ((r << 32) | col);
    }
#ifdef _OPENMP
    __gnu_parallel::sort(keys.begin(), keys.end());
#else
    std::sort(keys.begin(), keys.end());
#endif
    std::memset(indptr, 0, sizeof(int32_t) * (size_t)(n + 1));
    int64_t kept = 0;
    uint64_t prev = ~0ull;
    for (int64_t i = 0; i < n_edges; ++i) {
        const uint64_t k = keys[(size_t)i];
        if (k == ~0ull) break;
        if (k == prev) continue;
        prev = k;
        indices[kept++] = (int32_t)(k & 0xFFFFFFFFull);
        indptr[(k >> 32) + 1] += 1;
    }
    for (int64_t r = 0; r < n; ++r) indptr[r + 1] += indptr[r];
    return kept;
}

}  // extern "C"
