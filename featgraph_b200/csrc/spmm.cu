// SpMM (CSR and DDS adjacency times dense features, sum aggregation) for sm_100a.
//
// Work decomposition.  The unit of work is (feature tile, row): a group of G lanes owns
// one row's slice of G*VEC output columns (VEC = 4 floats per lane with 128-bit gathers).
// Each lane keeps its VEC accumulators in registers and walks the row's nonzeros in
// storage order, so every output element is a strictly sequential fp32 sum - the value
// the x86 loop nest of the reference produces (python/featgraph/op/vanilla_spmm.py:46-56
// with the loop order of :73) - and no launch parameter can change a result bit.
//
// Memory behaviour.  Units are numbered tile-major: all rows of feature tile 0, then tile
// 1, ...  While a tile is being processed only the n_cols x (G*VEC*4 B) slice of x is
// gathered from, and the tile width is chosen so that this slice stays resident in L2;
// the CSR arrays are then the only DRAM stream.  The G lanes of a group read G*16
// contiguous bytes per nonzero (one or more full 128-byte lines for G >= 8).  Column
// indices (and values, unless the adjacency is unweighted) are fetched G at a time,
// coalesced, one batch ahead of use, and passed to the group's lanes with shuffles; the
// gathers of up to 16 nonzeros are issued before the first of them is consumed.
//
// Balance.  Rows are visited in the order of an fg_row_schedule (heaviest first), blocks
// are launched in that order, and the groups sharing a warp hold neighbouring (hence
// similar-length) rows, so the warp-uniform loop below wastes few iterations.
//
// Long rows.  A row cannot be split between workers (its sum is sequential), so the time of
// the longest row is a floor under the whole launch: with 16 gathers in flight a 20,000-nonzero
// row costs 1,250 dependent round trips to L2.  Rows the launch counts as long therefore go to
// spmm_long_rows_kernel, which stages feature slices through a shared-memory ring filled by
// cp.async (64 nonzeros in flight per row; the same sums, a deeper pipeline, 15 ns per nonzero of
// a row instead of 40), and the very longest to spmm_heavy_rows_kernel, where the warps of a block
// share one row's ring and take turns at its sum (7 ns per nonzero).  They are launched first; the
// remaining rows follow in spmm_rows_kernel.
#include <cmath>
#include <mutex>

#include "common.cuh"
#include "schedule.cuh"

namespace {

constexpr int kThreads = 256;

// rows kernel shapes: gathers issued back to back per row and resident blocks per SM, regular / SHORT form
#define FG_ROWS_CH 16
#define FG_ROWS_MINB 2
#define FG_SHORT_CH 4
#define FG_SHORT_MINB 6
#define FG_RING_SLOTS 3
#define FG_RING_WARPS 4

struct SpmmArgs {
    const int32_t* pos;    // indptr (CSR) or s1_pos (DDS: parts blocks of n_rows+1)
    const int32_t* idx;    // column ids (DDS: relative to the partition's first column)
    const float* vals;
    const float* x;
    float* out;
    const int32_t* order;  // row visiting order or nullptr
    const int2* extent;    // (first nonzero, count) of row order[p] at position p, or nullptr (CSR only)
    int32_t order_begin;   // this launch covers order[order_begin, order_begin + n_sched)
    int32_t n_sched;
    int32_t n_rows;
    int32_t d;        // feature columns computed by this launch
    int64_t ldx;      // row stride of x in floats (>= d)
    int64_t ldo;      // row stride of out in floats (>= d)
    int32_t n_tiles;
    int32_t parts;          // 1 for CSR
    int32_t cols_per_part;  // DDS only
};

template <int VEC>
struct Slice;
template <>
struct Slice<4> {
    float4 v;
    __device__ __forceinline__ void load(const float* p, uint64_t policy) { v = fg::ldg4_keep(p, policy); }
    __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void axpy(float a, const Slice& x) {
        v.x = fg::mul_then_add(v.x, a, x.v.x);
        v.y = fg::mul_then_add(v.y, a, x.v.y);
        v.z = fg::mul_then_add(v.z, a, x.v.z);
        v.w = fg::mul_then_add(v.w, a, x.v.w);
    }
    __device__ __forceinline__ void add(const Slice& x) {
        v.x = __fadd_rn(v.x, x.v.x);
        v.y = __fadd_rn(v.y, x.v.y);
        v.z = __fadd_rn(v.z, x.v.z);
        v.w = __fadd_rn(v.w, x.v.w);
    }
    __device__ __forceinline__ void select(bool take, const Slice& x) {
        v.x = take ? x.v.x : v.x;
        v.y = take ? x.v.y : v.y;
        v.z = take ? x.v.z : v.z;
        v.w = take ? x.v.w : v.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Slice<1> {
    float v;
    __device__ __forceinline__ void load(const float* p, uint64_t) { v = __ldg(p); }
    __device__ __forceinline__ void zero() { v = 0.f; }
    __device__ __forceinline__ void axpy(float a, const Slice& x) { v = fg::mul_then_add(v, a, x.v); }
    __device__ __forceinline__ void add(const Slice& x) { v = __fadd_rn(v, x.v); }
    __device__ __forceinline__ void select(bool take, const Slice& x) { v = take ? x.v : v; }
    __device__ __forceinline__ void store(float* p) const { *p = v; }
};

// G lanes per (row, tile) unit; VEC floats per lane; DDS selects the two-level sum; UNIT: every
// adjacency value is 1.0 (no value array is read, and 1.0 * x == x exactly, so nothing is multiplied).
// The regular form keeps 16 gathers (16 x 128 bits per lane) in flight per row with 2 blocks per SM:
// the same bytes in flight per SM as 8 gathers with 4 blocks, but a row advances twice as fast
// (about 40 instead of 75 ns per nonzero), which is what bounds a launch on a shard, and the
// throughput measured slightly higher as well (233K-node graph, d = 64: 1.60 -> 1.42 ms).
// SHORT: the form for rows of a few nonzeros, where what counts is how many rows an SM has in
// flight, not how many gathers a row has: 4 gathers back to back and 6 blocks per SM.
template <int G, int VEC, bool DDS, bool UNIT, bool SHORT>
__global__ void __launch_bounds__(kThreads, SHORT ? FG_SHORT_MINB : FG_ROWS_MINB) spmm_rows_kernel(const SpmmArgs a) {
    constexpr int CHMAX = SHORT ? FG_SHORT_CH : FG_ROWS_CH;
    constexpr int CH = G < CHMAX ? G : CHMAX;  // gathers issued back to back
    const int lane = threadIdx.x & 31;
    const int lig = lane & (G - 1);
    const int64_t unit = (int64_t)blockIdx.x * (kThreads / G) + (threadIdx.x / G);
    const int64_t n_units = (int64_t)a.n_sched * a.n_tiles;
    const bool live = unit < n_units;

    int row = 0, tile = 0;
    int2 extent = make_int2(0, 0);
    if (live) {
        tile = (int)(unit / a.n_sched);
        const int p = a.order_begin + (int)(unit - (int64_t)tile * a.n_sched);
        row = a.order ? a.order[p] : p;
        if (!DDS && a.extent) extent = a.extent[p];
    }
    const int col = tile * (G * VEC) + lig * VEC;
    const bool col_ok = live && col < a.d;
    const float* xcol = a.x + (col_ok ? col : 0);  // idle lanes read (and discard) column 0

    Slice<VEC> total;
    total.zero();
    const uint64_t keep_policy = fg::l2_keep_policy();

    for (int k = 0; k < (DDS ? a.parts : 1); ++k) {
        int start = extent.x, len = extent.y;
        if (live && (DDS || !a.extent)) {
            const int32_t* p = a.pos + (int64_t)k * ((int64_t)a.n_rows + 1) + row;
            start = p[0];
            len = p[1] - start;
        }
        // partition k's first column folded into the base pointer; a 32 x 32 -> 64 bit multiply per gather
        const float* xbase = DDS ? xcol + (int64_t)k * a.cols_per_part * a.ldx : xcol;
        const int ldx32 = (int)a.ldx;
        Slice<VEC> acc;
        acc.zero();

        // every lane of the warp runs the same number of batches
        const int max_len = __reduce_max_sync(0xffffffffu, len);
        int my_c = -1;
        float my_v = 0.f;
        if (lig < len) {
            my_c = fg::ld_stream(a.idx + start + lig);
            if (!UNIT) my_v = fg::ld_stream(a.vals + start + lig);
        }
        for (int base = 0; base < max_len; base += G) {
            // next batch of indices / values, one iteration ahead of its use
            int nx_c = -1;
            float nx_v = 0.f;
            if (base + G + lig < len) {
                nx_c = fg::ld_stream(a.idx + start + base + G + lig);
                if (!UNIT) nx_v = fg::ld_stream(a.vals + start + base + G + lig);
            }
#pragma unroll
            for (int j0 = 0; j0 < G; j0 += CH) {
                if (base + j0 >= max_len) break;  // warp-uniform
                int c[CH];
                float v[CH];
                Slice<VEC> xr[CH];
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    c[j] = __shfl_sync(0xffffffffu, my_c, j0 + j, G);
                    v[j] = UNIT ? 1.f : __shfl_sync(0xffffffffu, my_v, j0 + j, G);
                }
                // Unconditional loads (padding slots re-read row 0 of the slice) so that all
                // CH gathers are in flight before the first dependent add.
#pragma unroll
                for (int j = 0; j < CH; ++j)
                    xr[j].load(xbase + (int64_t)(c[j] < 0 ? 0 : c[j]) * ldx32, keep_policy);
                // Branch-free commit: a branch here would let the compiler sink each load
                // next to its use and serialise the gathers.
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    Slice<VEC> next = acc;
                    if (UNIT)
                        next.add(xr[j]);
                    else
                        next.axpy(v[j], xr[j]);
                    acc.select(c[j] >= 0, next);
                }
            }
            my_c = nx_c;
            my_v = nx_v;
        }
        if (DDS)
            total.add(acc);
        else
            total = acc;
    }
    if (col_ok) total.store(a.out + (int64_t)row * a.ldo + col);
}


// ---------------------------------------------------------------------------------------------
// Long rows: one warp per (row, 32-float tile) unit, feature slices staged through a shared
// memory ring filled by cp.async.
//
// The warp owns kRingStages slots of 32 nonzeros x 128 bytes.  Filling a slot: the lanes read 32
// column ids / values (coalesced, requested one stage ahead), and eight cp.async instructions
// copy the 32 slices - each instruction moves 4 slices, 8 lanes x 16 bytes per slice - straight
// from L2 into the slot; the values go into the slot's value array.  Draining a slot: lane f
// owns output column f of the tile and adds value[j] * slice[j][f] for j = 0..31 in storage
// order (conflict-free 4-byte shared loads), i.e. the same strictly sequential sum as
// spmm_rows_kernel.  A row streams through the ring with kRingStages - 1 slots (2 x 4 KB) in
// flight and pays the memory latency once instead of once per 8 nonzeros.  Three slots (12.7 KB
// per warp, 16 resident warps per SM) measured faster than deeper rings with fewer warps: the
// per-lane add chain needs the other warps to fill its 4-cycle gaps.
// ---------------------------------------------------------------------------------------------
constexpr int kRingStages = FG_RING_SLOTS;
constexpr int kRingNnz = 32;                 // nonzeros per slot
constexpr int kLongWarps = FG_RING_WARPS;    // warps (= units) per block
constexpr int kLongThreads = kLongWarps * 32;
constexpr int kSlotFloats = kRingNnz * 32 + kRingNnz;  // 32 slices of 32 floats + 32 values
constexpr int kLongSmemBytes = kLongWarps * kRingStages * kSlotFloats * 4;
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src, uint64_t policy) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
#if FG_HINT_KEEP
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "l"(policy)
                 : "memory");
#else
    (void)policy;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
#endif
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// A shared-memory load the compiler may not move: the consumers below issue a batch of these before
// the first add of their (strictly sequential) chain, which keeps the load latency off that chain.
__device__ __forceinline__ float lds_pinned(unsigned addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds4_pinned(unsigned addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
// adds (UNIT) or multiply-adds the kRingNnz slices of a full slot to acc, in order
template <bool UNIT>
__device__ __forceinline__ float drain_full_slot(float acc, const float* slot, int lane) {
    constexpr int kBatch = 16;
    const unsigned base = (unsigned)__cvta_generic_to_shared(slot);
#pragma unroll
    for (int h = 0; h < kRingNnz; h += kBatch) {
        float t[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) t[j] = lds_pinned(base + ((h + j) * 32 + lane) * 4);
        if (!UNIT) {
#pragma unroll
            for (int j4 = 0; j4 < kBatch; j4 += 4) {
                const float4 v = lds4_pinned(base + (kRingNnz * 32 + h + j4) * 4);
                t[j4 + 0] = __fmul_rn(v.x, t[j4 + 0]);
                t[j4 + 1] = __fmul_rn(v.y, t[j4 + 1]);
                t[j4 + 2] = __fmul_rn(v.z, t[j4 + 2]);
                t[j4 + 3] = __fmul_rn(v.w, t[j4 + 3]);
            }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) acc = __fadd_rn(acc, t[j]);
    }
    return acc;
}

template <bool UNIT>
__global__ void __launch_bounds__(kLongThreads) spmm_long_rows_kernel(const SpmmArgs a) {
    extern __shared__ __align__(16) float ring_smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float* ring = ring_smem + warp * (kRingStages * kSlotFloats);

    const int64_t unit = (int64_t)blockIdx.x * kLongWarps + warp;
    const int64_t n_units = (int64_t)a.n_sched * a.n_tiles;
    if (unit >= n_units) return;  // whole warp
    const int tile = (int)(unit / a.n_sched);
    const int row = a.order[a.order_begin + (int)(unit - (int64_t)tile * a.n_sched)];
    const int col0 = tile * 32;
    const int start = a.pos[row];
    const int len = a.pos[row + 1] - start;
    const int n_stages = (len + kRingNnz - 1) / kRingNnz;

    // this lane's part in filling a slot: 16-byte piece `piece` of the slices of nonzeros
    // sub, sub + 4, sub + 8, ... of the stage
    const int piece = lane & 7;
    const int sub = lane >> 3;
    const bool piece_ok = col0 + piece * 4 < a.d;  // ragged last tile (d % 4 == 0)
    const float* xpiece = a.x + col0 + piece * 4;
    const int ldx32 = (int)a.ldx;
    const uint64_t keep_policy = fg::l2_keep_policy();

    auto fetch_ids = [&](int stage, int& c, float& v) {  // nonzero `lane` of `stage`
        const int k = stage * kRingNnz + lane;
        c = -1;
        v = 0.f;
        if (k < len) {
            c = fg::ld_stream(a.idx + start + k);
            if (!UNIT) v = fg::ld_stream(a.vals + start + k);
        }
    };
    auto fill = [&](int stage, int c_mine, float v_mine) {
        float* slot = ring + (stage % kRingStages) * kSlotFloats;
        if (stage < n_stages) {
            if (!UNIT) slot[kRingNnz * 32 + lane] = v_mine;
#pragma unroll
            for (int i = 0; i < kRingNnz / 4; ++i) {
                const int nz = i * 4 + sub;
                const int c = __shfl_sync(0xffffffffu, c_mine, nz);
                if (c >= 0 && piece_ok) cp_async16(slot + nz * 32 + piece * 4, xpiece + (int64_t)c * ldx32, keep_policy);
            }
        }
        cp_async_commit();  // one group per stage, empty past the end, so the wait count is fixed
    };

    // Column ids / values are requested kIdsAhead stages before the stage is filled (they stream
    // from DRAM), in a small register ring.
    constexpr int kInFlight = kRingStages - 1;
    constexpr int kIdsAhead = 4;
    int c_ring[kIdsAhead];
    float v_ring[kIdsAhead];
    {
        int c0[kInFlight];
        float v0[kInFlight];
#pragma unroll
        for (int s = 0; s < kInFlight; ++s) fetch_ids(s, c0[s], v0[s]);
#pragma unroll
        for (int q = 0; q < kIdsAhead; ++q) fetch_ids(kInFlight + q, c_ring[q], v_ring[q]);
#pragma unroll
        for (int s = 0; s < kInFlight; ++s) fill(s, c0[s], v0[s]);
    }

    float acc = 0.f;
#pragma unroll 1
    for (int s0 = 0; s0 < n_stages; s0 += kIdsAhead) {
#pragma unroll
        for (int q = 0; q < kIdsAhead; ++q) {
            const int s = s0 + q;
            if (s >= n_stages) break;  // whole warp
            fill(s + kInFlight, c_ring[q], v_ring[q]);
            fetch_ids(s + kInFlight + kIdsAhead, c_ring[q], v_ring[q]);
            cp_async_wait<kInFlight>();  // this lane's copies of stage s have landed ...
            __syncwarp();                // ... and so have the other lanes'
            const float* slot = ring + (s % kRingStages) * kSlotFloats;
            const int cnt = min(kRingNnz, len - s * kRingNnz);
            if (cnt == kRingNnz) {
                acc = drain_full_slot<UNIT>(acc, slot, lane);
            } else if (UNIT) {
                for (int j = 0; j < cnt; ++j) acc = __fadd_rn(acc, slot[j * 32 + lane]);
            } else {
                for (int j = 0; j < cnt; ++j)
                    acc = fg::mul_then_add(acc, slot[kRingNnz * 32 + j], slot[j * 32 + lane]);
            }
            __syncwarp();  // the slot is refilled by the next iteration's fill()
        }
    }
    if (col0 + lane < a.d) a.out[(int64_t)row * a.ldo + col0 + lane] = acc;
}

// ---------------------------------------------------------------------------------------------
// Heaviest rows: one BLOCK per (row, 32-float tile) unit.
//
// In spmm_long_rows_kernel one warp does everything for its row - column ids, address arithmetic,
// copies, waits and the adds - about 130 mostly dependent instructions per 32 nonzeros, and that
// chain, not the ring's depth, sets the row's pace (15 ns per nonzero; a ring of 12 slots gave 11).
// Here the W warps of a block share one row, and only the adds stay on the row's chain.  The row is
// cut into turns of TURN stages (32 nonzeros each); turn t belongs to warp t % W, which copies its
// stages into its own ring (3 turns deep) exactly as above.  The sum stays one sequential chain:
// the warps take their turns in order and hand the 32 running sums (lane f = output column f) on
// through shared memory and a named barrier shared by just the two warps involved (barrier 1 + w:
// warp w arrives, warp w + 1 waits).  A warp whose turn is over refills its slots, fetches ids and
// waits for its next copies while the other warps have their turns; before its turn it has
// already loaded the first stage's 32 values into registers, so a turn costs the barrier, one
// shared load of the sums and the chain of adds: about 3 to 4 ns per nonzero.
// Each turn after the first has one arrival (by the previous turn's owner) and one wait (by its
// owner) on the same barrier, so the counts always match; there is no spinning anywhere.
// Instantiated with TURN = 1 and 4 or 8 warps.  Measured on one 200,000-nonzero row: 5.4 ns per
// nonzero with 4 warps, 4.0 with 8; TURN = 2 with 4 warps gave 4.3 but needs twice the shared memory.
// ---------------------------------------------------------------------------------------------
constexpr int kHeavyTurnsDeep = 3;  // turns of its own that a warp keeps in its ring

template <int W, int TURN>
constexpr int heavy_smem_bytes() {
    return (W * kHeavyTurnsDeep * TURN * kSlotFloats + 32) * 4;
}

template <bool UNIT, int W, int TURN>
__global__ void __launch_bounds__(W * 32) spmm_heavy_rows_kernel(const SpmmArgs a) {
    static_assert(W >= 2 && (W & (W - 1)) == 0, "W: a power of two, at least 2");
    constexpr int kSlots = kHeavyTurnsDeep * TURN;  // per warp
    extern __shared__ __align__(16) float ring_smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float* ring = ring_smem + warp * (kSlots * kSlotFloats);
    float* sums = ring_smem + W * kSlots * kSlotFloats;  // the 32 running sums between turns

    const int tile = (int)(blockIdx.x / (unsigned)a.n_sched);
    const int row = a.order[a.order_begin + (int)(blockIdx.x - (unsigned)tile * (unsigned)a.n_sched)];
    const int col0 = tile * 32;
    const int start = a.pos[row];
    const int len = a.pos[row + 1] - start;
    const int n_stages = (len + kRingNnz - 1) / kRingNnz;  // the same for every warp of the block
    if (n_stages == 0) {
        if (warp == 0 && col0 + lane < a.d) a.out[(int64_t)row * a.ldo + col0 + lane] = 0.f;
        return;
    }
    const int n_turns = (n_stages + TURN - 1) / TURN;
    const int my_turns = n_turns > warp ? (n_turns - warp + W - 1) / W : 0;
    // this warp's local stage i = (its turn i / TURN, stage i % TURN of that turn) is stage
    // ((i / TURN) * W + warp) * TURN + i % TURN of the row
    auto row_stage = [&](int i) { return ((i / TURN) * W + warp) * TURN + i % TURN; };

    const int piece = lane & 7;
    const int sub = lane >> 3;
    const bool piece_ok = col0 + piece * 4 < a.d;
    const float* xpiece = a.x + col0 + piece * 4;
    const int ldx32 = (int)a.ldx;
    const uint64_t keep_policy = fg::l2_keep_policy();

    auto fetch_ids = [&](int i, int& c, float& v) {  // nonzero `lane` of local stage i
        const int k = row_stage(i) * kRingNnz + lane;
        c = -1;
        v = 0.f;
        if (k < len) {  // also false for every stage past the row's end
            c = fg::ld_stream(a.idx + start + k);
            if (!UNIT) v = fg::ld_stream(a.vals + start + k);
        }
    };
    auto fill = [&](int i, int c_mine, float v_mine) {
        float* slot = ring + (i % kSlots) * kSlotFloats;
        if (row_stage(i) < n_stages) {
            if (!UNIT) slot[kRingNnz * 32 + lane] = v_mine;
#pragma unroll
            for (int j = 0; j < kRingNnz / 4; ++j) {
                const int nz = j * 4 + sub;
                const int c = __shfl_sync(0xffffffffu, c_mine, nz);
                if (c >= 0 && piece_ok) cp_async16(slot + nz * 32 + piece * 4, xpiece + (int64_t)c * ldx32, keep_policy);
            }
        }
        cp_async_commit();  // one group per local stage, empty past the end
    };

    // every slot is filled up front; the ids of the two turns after those wait in registers (they
    // stream from DRAM and must be there when the refill needs them)
    int c_next[TURN], c_after[TURN];
    float v_next[TURN], v_after[TURN];
    {
        int c0[kSlots];
        float v0[kSlots];
#pragma unroll
        for (int i = 0; i < kSlots; ++i) fetch_ids(i, c0[i], v0[i]);
#pragma unroll
        for (int u = 0; u < TURN; ++u) {
            fetch_ids(kSlots + u, c_next[u], v_next[u]);
            fetch_ids(kSlots + TURN + u, c_after[u], v_after[u]);
        }
#pragma unroll
        for (int i = 0; i < kSlots; ++i) fill(i, c0[i], v0[i]);
    }

    const int bar_mine = 1 + warp;
    const int bar_prev = 1 + ((warp + W - 1) & (W - 1));
#pragma unroll 1
    for (int t = 0; t < my_turns; ++t) {
        const int i0 = t * TURN;        // first local stage of the turn
        const int s0 = row_stage(i0);   // and its stage of the row
        // my copies of this turn: all but the (kHeavyTurnsDeep - 1) * TURN newest groups
        cp_async_wait<(kHeavyTurnsDeep - 1) * TURN>();
        __syncwarp();
        // the first stage's values (products) go to registers before the turn starts
        const float* slot0 = ring + (i0 % kSlots) * kSlotFloats;
        const int cnt0 = min(kRingNnz, len - s0 * kRingNnz);
        float first[kRingNnz];
        if (cnt0 == kRingNnz) {
            const unsigned base = (unsigned)__cvta_generic_to_shared(slot0);
#pragma unroll
            for (int j = 0; j < kRingNnz; ++j) first[j] = lds_pinned(base + (j * 32 + lane) * 4);
            if (!UNIT) {
#pragma unroll
                for (int j4 = 0; j4 < kRingNnz; j4 += 4) {
                    const float4 v = lds4_pinned(base + (kRingNnz * 32 + j4) * 4);
                    first[j4 + 0] = __fmul_rn(v.x, first[j4 + 0]);
                    first[j4 + 1] = __fmul_rn(v.y, first[j4 + 1]);
                    first[j4 + 2] = __fmul_rn(v.z, first[j4 + 2]);
                    first[j4 + 3] = __fmul_rn(v.w, first[j4 + 3]);
                }
            }
        }
        float acc = 0.f;
        if (s0 > 0) {
            asm volatile("bar.sync %0, 64;\n" ::"r"(bar_prev) : "memory");
            acc = sums[lane];
        }
        if (cnt0 == kRingNnz) {
#pragma unroll
            for (int j = 0; j < kRingNnz; ++j) acc = __fadd_rn(acc, first[j]);
        } else if (UNIT) {
            for (int j = 0; j < cnt0; ++j) acc = __fadd_rn(acc, slot0[j * 32 + lane]);
        } else {
            for (int j = 0; j < cnt0; ++j)
                acc = fg::mul_then_add(acc, slot0[kRingNnz * 32 + j], slot0[j * 32 + lane]);
        }
#pragma unroll
        for (int u = 1; u < TURN; ++u) {
            const int cnt = min(kRingNnz, len - (s0 + u) * kRingNnz);  // <= 0 past the row's end
            const float* slot = ring + ((i0 + u) % kSlots) * kSlotFloats;
            if (cnt == kRingNnz) {
                acc = drain_full_slot<UNIT>(acc, slot, lane);
            } else if (UNIT) {
                for (int j = 0; j < cnt; ++j) acc = __fadd_rn(acc, slot[j * 32 + lane]);
            } else {
                for (int j = 0; j < cnt; ++j)
                    acc = fg::mul_then_add(acc, slot[kRingNnz * 32 + j], slot[j * 32 + lane]);
            }
        }
        if (s0 + TURN < n_stages) {  // another turn follows
            sums[lane] = acc;
            __threadfence_block();
            asm volatile("bar.arrive %0, 64;\n" ::"r"(bar_mine) : "memory");
        } else if (col0 + lane < a.d) {
            a.out[(int64_t)row * a.ldo + col0 + lane] = acc;  // the row's last turn
        }
        __syncwarp();  // every lane has read the slots
        // refill the slots just drained, off the chain of turns
#pragma unroll
        for (int u = 0; u < TURN; ++u) {
            fill(i0 + kSlots + u, c_next[u], v_next[u]);
            c_next[u] = c_after[u];
            v_next[u] = v_after[u];
            fetch_ids(i0 + kSlots + 2 * TURN + u, c_after[u], v_after[u]);
        }
    }
}

// Which rows (from the front of the schedule) go to the heavy-row and long-row kernels for this launch.
//
// The three kernels trade throughput against the time of one row.  Measured on B200 (C2 graph):
//   spmm_rows_kernel       streams gathers at about 19 TB/s, about 40 ns per nonzero of one row
//                          (16 gathers per L2 round trip; 75 ns with tiles of 32 floats, where a row
//                          has 8 lanes and 8 gathers): a 20,000-nonzero row alone takes 0.8 ms;
//   spmm_long_rows_kernel  about 13 TB/s (every slice crosses shared memory twice), 15 ns per nonzero;
//   spmm_heavy_rows_kernel with 4 warps per block about 9 TB/s and 7 ns per nonzero, with 8 warps
//                          about 6 TB/s and 5 ns (more time for a warp to refill between turns).
// Units run tile-major, so a kernel's longest rows are met again in its last feature tile: alone, a
// kernel takes
//     (1 - 1/tiles) * bytes / rate  +  max(bytes / rate / tiles, longest row's time).
// Run one after the other, the launch takes the sum of the parts.  Run side by side (each kernel on
// a stream of its own, see spmm_dispatch) they share the path from L2, and the launch is modelled
// as the largest of: all bytes one after the other, and each kernel's own time with its streaming
// part stretched to that sum.  Every pair of candidate thresholds is tried and the
// cheapest wins.  A threshold fixed at schedule creation overrides the choice.  The choice never
// affects a result bit.
constexpr double kRowsRate = 19e12;
// per nonzero of one row: about 40 ns measured with 16 gathers in flight, 75 with 8 (tiles of 32 floats: 8
// lanes per row); the model uses a cautious 55 for the former - too low a figure leaves long rows in this
// kernel, and their time is then added to the whole launch
constexpr double kRowsSecPerNnz16 = 55e-9, kRowsSecPerNnz8 = 75e-9;
constexpr double kRingRate = 13e12, kRingSecPerNnz = 15e-9;
constexpr double kHeavyRate[2] = {9e12, 6e12}, kHeavySecPerNnz[2] = {7.5e-9, 5e-9};  // 4 / 8 warps

int sm_count() { return fg::device_props().sm_count; }

struct RowSplit {
    int64_t heavy = 0;  // order[0, heavy): spmm_heavy_rows_kernel
    int64_t ring = 0;   // order[heavy, ring): spmm_long_rows_kernel; the rest: spmm_rows_kernel
    bool wide = false;  // heavy rows with 8 warps per block instead of 4
};

RowSplit choose_row_split(const fg_row_schedule& sch, int d, int short_tile, bool side_by_side) {
    RowSplit best_split;
    if (sch.fixed_threshold > 0) {
        best_split.heavy = sch.fixed_heavy_rows;
        best_split.ring = sch.fixed_rows;
        best_split.wide = sch.fixed_wide;
        return best_split;
    }
    const double short_tiles = (d + short_tile - 1) / short_tile;
    const double long_tiles = (d + 31) / 32;
    const double longest = (double)sch.max_row_nnz;
    const double long_bytes = 4.0 * d + 8.0 * long_tiles, short_bytes = 4.0 * d + 8.0 * short_tiles;
    auto part = [](double stream, double tiles, double row_time) {
        return stream <= 0.0 ? 0.0 : stream * (1.0 - 1.0 / tiles) + fmax(stream / tiles, row_time);
    };
    // thresholds t_heavy >= t_ring; "none" is a threshold above the longest row
    auto estimate = [&](double nnz_heavy, double t_heavy, double nnz_ring_up, double t_ring, int wide) {
        const double nnz_ring = nnz_ring_up - nnz_heavy, nnz_rows = (double)sch.nnz - nnz_ring_up;
        const double s_heavy = nnz_heavy * long_bytes / kHeavyRate[wide];
        const double s_ring = nnz_ring * long_bytes / kRingRate;
        const double s_rows = nnz_rows * short_bytes / kRowsRate;
        const double heavy_row = longest * kHeavySecPerNnz[wide];
        const double ring_row = fmin(t_heavy, longest) * kRingSecPerNnz;
        const double rows_row = fmin(t_ring, longest) * (short_tile >= 64 ? kRowsSecPerNnz16 : kRowsSecPerNnz8);
        if (!side_by_side)
            return part(s_heavy, long_tiles, heavy_row) + part(s_ring, long_tiles, ring_row) +
                   part(s_rows, short_tiles, rows_row);
        // three streams side by side: each kernel's streaming part stretched to the time of all bytes
        const double all = s_heavy + s_ring + s_rows;
        double t = all;
        if (s_heavy > 0.0) t = fmax(t, part(all, long_tiles, heavy_row));
        if (s_ring > 0.0) t = fmax(t, part(all, long_tiles, ring_row));
        if (s_rows > 0.0) t = fmax(t, part(all, short_tiles, rows_row));
        return t;
    };
    const double none = longest + 1.0;
    double best = estimate(0.0, none, 0.0, none, 0);
    for (int lr = 0; lr < fg::kSplitLevels; ++lr) {  // ring threshold
        if (sch.rows_at_least[lr] == 0) break;
        const double t_ring = (double)fg::split_threshold(lr);
        for (int lh = lr; lh <= fg::kSplitLevels; ++lh) {  // heavy threshold, kSplitLevels = none
            const bool no_heavy = lh == fg::kSplitLevels || sch.rows_at_least[lh] == 0;
            // the 8-warp form only where all its blocks are resident at once (two per SM): it is
            // there for a handful of hub rows, not for throughput
            const bool wide_ok = !no_heavy && (double)sch.rows_at_least[lh] * long_tiles <= 2.0 * sm_count();
            for (int wide = 0; wide < (wide_ok ? 2 : 1); ++wide) {
                const double t =
                    no_heavy ? estimate(0.0, none, (double)sch.nnz_at_least[lr], t_ring, 0)
                             : estimate((double)sch.nnz_at_least[lh], (double)fg::split_threshold(lh),
                                        (double)sch.nnz_at_least[lr], t_ring, wide);
                if (t < best) {
                    best = t;
                    best_split.heavy = no_heavy ? 0 : sch.rows_at_least[lh];
                    best_split.ring = sch.rows_at_least[lr];
                    best_split.wide = wide != 0;
                }
            }
            if (no_heavy) break;
        }
    }
    return best_split;
}

// Three more streams (per host thread and device) on which the heavy-row, the long-row and the
// short-row kernel can run beside spmm_rows_kernel.  Fork and join are event waits on the device:
// the caller's stream sees one call that is complete when all kernels are, also under stream capture.
struct SideStream {
    enum { kHeavy = 0, kRing = 1, kShort = 2, kStreams = 3 };
    cudaStream_t stream[kStreams] = {nullptr, nullptr, nullptr};
    cudaEvent_t fork = nullptr, join[kStreams] = {nullptr, nullptr, nullptr};
    bool prepare() {
        if (fork) return true;
        int least = 0, greatest = 0;
        cudaDeviceGetStreamPriorityRange(&least, &greatest);
        bool ok = cudaEventCreateWithFlags(&fork, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < kStreams; ++i)
            // the heaviest rows bound the launch: their blocks go first
            ok = cudaStreamCreateWithPriority(&stream[i], cudaStreamNonBlocking,
                                              i == kShort ? least : greatest) == cudaSuccess &&
                 cudaEventCreateWithFlags(&join[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            (void)cudaGetLastError();
            fork = nullptr;
            return false;
        }
        return true;
    }
    // every side stream starts after what the caller's stream holds so far
    bool fork_from(cudaStream_t s) {
        if (!prepare() || cudaEventRecord(fork, s) != cudaSuccess) return false;
        for (int i = 0; i < kStreams; ++i)
            if (cudaStreamWaitEvent(stream[i], fork, 0) != cudaSuccess) return false;
        return true;
    }
    // and the caller's stream continues after all of them
    int join_to(cudaStream_t s) {
        for (int i = 0; i < kStreams; ++i) {
            FG_CUDA_TRY(cudaEventRecord(join[i], stream[i]));
            FG_CUDA_TRY(cudaStreamWaitEvent(s, join[i], 0));
        }
        return FG_OK;
    }
};

// One set per host thread and device: a thread that alternates between devices (one process driving
// several GPUs) finds its objects again when it returns to a device.  nullptr: no usable device slot.
SideStream* side_stream() {
    static thread_local SideStream table[fg::kMaxDevices];
    const int dev = fg::current_device_slot();
    return dev < 0 ? nullptr : &table[dev];
}

int launch_long(const SpmmArgs& a, cudaStream_t s) {
    const int64_t n_units = (int64_t)a.n_sched * a.n_tiles;
    const int64_t blocks = (n_units + kLongWarps - 1) / kLongWarps;
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    if (blocks == 0) return FG_OK;
    static_assert(kLongSmemBytes <= 227 * 1024, "ring does not fit in shared memory");
    if (a.vals == nullptr) {
        FG_CUDA_TRY(cudaFuncSetAttribute(spmm_long_rows_kernel<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kLongSmemBytes));
        spmm_long_rows_kernel<true><<<(unsigned)blocks, kLongThreads, kLongSmemBytes, s>>>(a);
    } else {
        FG_CUDA_TRY(cudaFuncSetAttribute(spmm_long_rows_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kLongSmemBytes));
        spmm_long_rows_kernel<false><<<(unsigned)blocks, kLongThreads, kLongSmemBytes, s>>>(a);
    }
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

template <bool UNIT, int W, int TURN>
int launch_heavy_w(const SpmmArgs& a, cudaStream_t s) {
    const int64_t blocks = (int64_t)a.n_sched * a.n_tiles;
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    if (blocks == 0) return FG_OK;
    static_assert(heavy_smem_bytes<W, TURN>() <= 227 * 1024, "rings do not fit in shared memory");
    FG_CUDA_TRY(cudaFuncSetAttribute(spmm_heavy_rows_kernel<UNIT, W, TURN>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, heavy_smem_bytes<W, TURN>()));
    spmm_heavy_rows_kernel<UNIT, W, TURN><<<(unsigned)blocks, W * 32, heavy_smem_bytes<W, TURN>(), s>>>(a);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

int launch_heavy(const SpmmArgs& a, bool wide, cudaStream_t s) {
    if (wide) return a.vals == nullptr ? launch_heavy_w<true, 8, 1>(a, s) : launch_heavy_w<false, 8, 1>(a, s);
    return a.vals == nullptr ? launch_heavy_w<true, 4, 1>(a, s) : launch_heavy_w<false, 4, 1>(a, s);
}

template <int G, int VEC, bool SHORT = false>
int launch(const SpmmArgs& a, bool dds, cudaStream_t s) {
    const int64_t n_units = (int64_t)a.n_sched * a.n_tiles;
    const int64_t units_per_block = kThreads / G;
    const int64_t blocks = (n_units + units_per_block - 1) / units_per_block;
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    if (blocks == 0) return FG_OK;
    const bool unit = a.vals == nullptr;
    if (SHORT) {  // CSR only
        if (unit)
            spmm_rows_kernel<G, VEC, false, true, SHORT><<<(unsigned)blocks, kThreads, 0, s>>>(a);
        else
            spmm_rows_kernel<G, VEC, false, false, SHORT><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    } else if (dds && unit)
        spmm_rows_kernel<G, VEC, true, true, false><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    else if (dds)
        spmm_rows_kernel<G, VEC, true, false, false><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    else if (unit)
        spmm_rows_kernel<G, VEC, false, true, false><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    else
        spmm_rows_kernel<G, VEC, false, false, false><<<(unsigned)blocks, kThreads, 0, s>>>(a);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

template <bool SHORT>
int launch_tile(const SpmmArgs& a, int tile, bool dds, cudaStream_t s) {
    switch (tile / 4) {
        case 1: return launch<1, 4, SHORT>(a, dds, s);
        case 2: return launch<2, 4, SHORT>(a, dds, s);
        case 4: return launch<4, 4, SHORT>(a, dds, s);
        case 8: return launch<8, 4, SHORT>(a, dds, s);
        case 16: return launch<16, 4, SHORT>(a, dds, s);
        default: return launch<32, 4, SHORT>(a, dds, s);
    }
}

// The share of L2 in which a gathered slice of x stays resident under all-SM random access.
int64_t l2_budget() {
    return fg::device_props().l2_bytes / 2;  // each half of the chip caches its own copy
}

// Can a 32-float slice of x (the narrowest tile that gathers whole 128-byte lines) stay in L2?
bool slice_can_stay_in_l2(int64_t n_cols) { return n_cols * 32 * 4 <= l2_budget(); }

// Feature-tile width (floats) when the caller leaves the choice to the library: the widest
// power of two, at most 128, whose gathered slice of x (n_cols rows of tile*4 bytes) fits the
// share of L2 that stays resident under all-SM random access; never below 32 floats, one full
// 128-byte line per gather.  If not even a 32-float slice fits, residency is out of reach and
// the widest tile wins (fewest passes over the index arrays, longest contiguous gathers).
int auto_tile(int64_t n_cols, int d) {
    const int64_t budget = l2_budget();
    const int cap = fg::pow2_ceil(d < 128 ? d : 128);
    if (!slice_can_stay_in_l2(n_cols)) return cap;
    int tile = 32;
    while (tile * 2 <= cap && n_cols * (int64_t)(tile * 2) * 4 <= budget) tile *= 2;
    return tile < cap ? tile : cap;
}

int spmm_dispatch(const fg_row_schedule* schedule, const int32_t* pos, const int32_t* idx,
                  const float* vals, const float* x, int64_t ldx, float* out, int64_t ldo,
                  int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d, int32_t parts,
                  int32_t feat_tile, void* stream, bool dds) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d",
                        (long long)n_rows, (long long)n_cols, (long long)nnz, d);
    if (n_rows > INT32_MAX || n_cols > INT32_MAX || nnz > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "sizes beyond int32 indexing are not supported");
    if (parts < 1) return fg::fail(FG_ERR_INVALID_ARGUMENT, "num_col_partitions must be >= 1");
    if (ldx == 0) ldx = d;
    if (ldo == 0) ldo = d;
    if (ldx < d || ldo < d || ldx > INT32_MAX || ldo > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides ldx=%lld ldo=%lld must be 0 or in [d=%d, 2^31)",
                        (long long)ldx, (long long)ldo, d);
    if (feat_tile != 0 && (feat_tile < 4 || feat_tile > 128 || (feat_tile & (feat_tile - 1))))
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "feat_tile=%d: want 0 or a power of two in 4..128",
                        feat_tile);
    if (n_rows == 0) return FG_OK;
    if (!pos || !out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL position or output array");
    if (nnz > 0 && (!idx || !x))  // vals may be NULL: every value is 1.0
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL adjacency or feature array");
    if (schedule && fg_row_schedule_num_rows(schedule) != n_rows)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row schedule was built for %lld rows, not %lld",
                        (long long)fg_row_schedule_num_rows(schedule), (long long)n_rows);
    // The rows kernels read each row's extent from the schedule's cache, not from the position array
    // of this call: a schedule built from another adjacency would send gathers out of bounds.
    if (schedule && !dds && schedule->d_extent && schedule->nnz != nnz)
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "row schedule was built from an adjacency of %lld nonzeros, this call has %lld: "
                        "rebuild the schedule when the adjacency changes",
                        (long long)schedule->nnz, (long long)nnz);

    SpmmArgs a;
    a.pos = pos;
    a.idx = idx;
    a.vals = vals;
    a.x = x;
    a.out = out;
    a.order = schedule ? fg_row_schedule_order(schedule) : nullptr;
    a.extent = (schedule && !dds) ? schedule->d_extent : nullptr;
    a.order_begin = 0;
    a.n_sched = (int32_t)n_rows;
    a.n_rows = (int32_t)n_rows;
    a.d = d;
    a.ldx = ldx;
    a.ldo = ldo;
    a.parts = parts;
    a.cols_per_part = dds ? (int32_t)((n_cols + parts - 1) / parts) : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const bool vec = (d % 4 == 0) && (ldx % 4 == 0) && (ldo % 4 == 0) && fg::aligned16(x) && fg::aligned16(out);
    if (!vec) {
        // scalar path: 32 lanes x 1 float per unit
        a.n_tiles = (d + 31) / 32;
        return launch<32, 1>(a, dds, s);
    }
    int tile = feat_tile ? feat_tile : auto_tile(n_cols, d);
    const int cap = fg::pow2_ceil(d);
    if (tile > cap) tile = cap;
    if (tile < 4) tile = 4;
    // Heavy and long rows go through the shared-memory rings (CSR with a schedule only).  Where it pays,
    // the kernels of a call run SIDE BY SIDE - heavy, long and short rows on three internal streams
    // forked from and joined to the caller's - so that the last long rows, a few warps each bound by its
    // row's length (a 20,000-nonzero row takes 0.15 ms even in the heavy-row kernel, a 160,000-nonzero hub
    // row 2.4 ms in the long-row kernel), finish under the bulk of the work instead of idling the GPU:
    //  * no slice of x can stay in L2 (millions of columns): always (R-MAT scale 22, d = 128: 7.5 -> 5.7 ms);
    //  * a slice stays resident and the call is a single feature tile: all kernels gather from that one
    //    slice (1/8 shard of the 233K-node graph: d = 32 0.225 -> 0.197 ms, d = 64 0.365 -> 0.320);
    //  * a slice stays resident and the call walks several tiles: one after the other.  Side by side each
    //    kernel walks its own tile sequence and evicts the slice the other one lives on; measured on that
    //    shard at d = 512: in sequence 1.98 ms, whole call side by side 2.38 (2.95 with the split the
    //    side-by-side model prefers; evict-first gathers in the ring kernels changed nothing), one fork /
    //    join per tile 2.78 (each tile then pays the longest row's 0.15 ms and a drained GPU).
    const bool resident = slice_can_stay_in_l2(n_cols);
    SideStream* side = side_stream();
    // the kernels of one launch on feature columns [c0, c0 + w)
    auto columns = [&](int c0, int w, const RowSplit& split, bool beside) -> int {
        // Rows of fewer than 64 nonzeros (the schedule's first threshold) take the SHORT form of the
        // rows kernel, launched last (beside the others on a stream of its own).
        int64_t first_short = n_rows;
        if (schedule && !dds) {
            first_short = schedule->rows_at_least[0];
            if (first_short < split.ring) first_short = split.ring;
        }
        const bool forked = beside && side && (split.ring > 0 || first_short < n_rows) && side->fork_from(s);
        auto stream_for = [&](int which) { return forked ? side->stream[which] : s; };
        SpmmArgs h = a;
        h.x = a.x + c0;
        h.out = a.out + c0;
        h.d = w;
        int rc = FG_OK;
        {
            SpmmArgs r = h;
            r.n_tiles = (w + 31) / 32;
            r.order_begin = 0;
            r.n_sched = (int32_t)split.heavy;
            rc = launch_heavy(r, split.wide, stream_for(SideStream::kHeavy));
            if (rc == FG_OK) {
                r.order_begin = (int32_t)split.heavy;
                r.n_sched = (int32_t)(split.ring - split.heavy);
                rc = launch_long(r, stream_for(SideStream::kRing));
            }
        }
        h.n_tiles = (w + tile - 1) / tile;
        if (rc == FG_OK) {
            h.order_begin = (int32_t)split.ring;
            h.n_sched = (int32_t)(first_short - split.ring);
            rc = launch_tile<false>(h, tile, dds, s);
        }
        if (rc == FG_OK && first_short < n_rows) {
            h.order_begin = (int32_t)first_short;
            h.n_sched = (int32_t)(n_rows - first_short);
            rc = launch_tile<true>(h, tile, dds, stream_for(SideStream::kShort));
        }
        // join even after a failed launch: the side streams must come back to the caller's stream (a
        // capture could not end otherwise); work enqueued on it afterwards waits for all kernels
        if (forked) {
            const int rcj = side->join_to(s);
            if (rc == FG_OK) rc = rcj;
        }
        return rc;
    };
    const RowSplit none;
    if (!schedule || dds) return columns(0, d, none, false);
    if (!resident) return columns(0, d, choose_row_split(*schedule, d, tile, true), true);
    if (d <= tile) return columns(0, d, choose_row_split(*schedule, d, tile, true), true);
    return columns(0, d, choose_row_split(*schedule, d, tile, false), false);
}

// ---------------------------------------------------------------------------------------------
// Aggregate, then score, in one pass over the rows (one GCN-style layer step):
//     H = A . X                         as fg_spmm_csr_f32 (sequential sums, the same bits)
//     out[e] = dot(H[row e], Y[col e])  as fg_sddmm_coo_f32 on the CSR-ordered edge list
// which a caller of the reference runs as two built functions back to back
// (python/featgraph/module/spmm.py:142-161, then python/featgraph/module/sddmm.py:115-129).
//
// A group of G lanes owns a row, as in spmm_rows_kernel, and all d columns of it (d <= 4 G): when the
// row's sum is finished its slice of H is in the lanes' registers, so the same group walks the row's
// nonzeros a second time, gathers the slices of y and reduces each edge's dot product with the
// transposed butterfly of the SDDMM kernels.  Against two calls this saves reading H back (once per
// row), the second kernel's pass over the row ids, and a kernel's tail; H is still written (a layer
// needs it).  Rows too long for one group (the launch's long / heavy rows) take the ring kernels for
// H and score_long_rows_kernel for their edges.
// ---------------------------------------------------------------------------------------------
struct FusedArgs {
    SpmmArgs a;        // a.out = H
    const float* y;    // [n_cols, d], row stride ldy
    int64_t ldy;
    float* edge_out;   // [nnz], CSR order
};

__device__ __forceinline__ float dot4f(float acc, const float4& p, const float4& q) {
    acc = fmaf(p.x, q.x, acc);
    acc = fmaf(p.y, q.y, acc);
    acc = fmaf(p.z, q.z, acc);
    acc = fmaf(p.w, q.w, acc);
    return acc;
}

// Transposed butterfly over the G lanes of a group.  In: pc[j] = this lane's partial dot product of
// chunk edge j (U edges).  Out (after the in-chunk steps): pc[0] = for the edge picked by the lane's low
// log2(U) bits, the sum over the lanes that differ from it in those bits.
template <int U>
__device__ __forceinline__ float butterfly_in_chunk(float (&pc)[U], int lig) {
#pragma unroll
    for (int o = 1; o < U; o <<= 1) {
        const bool upper = (lig & o) != 0;
#pragma unroll
        for (int i = 0; i < U / (2 * o); ++i) {
            const float send = upper ? pc[2 * i] : pc[2 * i + 1];
            const float keep = upper ? pc[2 * i + 1] : pc[2 * i];
            pc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    return pc[0];
}
// The remaining steps across the G / U chunks: afterwards r[0] on lane i of the group is edge i's total.
template <int G, int U>
__device__ __forceinline__ float butterfly_across_chunks(float (&r)[G / U], int lig) {
#pragma unroll
    for (int o = U; o < G; o <<= 1) {
        const bool upper = (lig & o) != 0;
        const int h = o / U;
#pragma unroll
        for (int i = 0; i < G / U / (2 * h); ++i) {
            const float send = upper ? r[2 * i] : r[2 * i + 1];
            const float keep = upper ? r[2 * i + 1] : r[2 * i];
            r[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    return r[0];
}

// G lanes x 4 floats cover all d columns (one feature tile).  SHORT as in spmm_rows_kernel.
template <int G, bool UNIT, bool SHORT>
__global__ void __launch_bounds__(kThreads, SHORT ? FG_SHORT_MINB : FG_ROWS_MINB) fused_rows_kernel(const FusedArgs f) {
    const SpmmArgs& a = f.a;
    constexpr int CHMAX = SHORT ? FG_SHORT_CH : FG_ROWS_CH;
    constexpr int CH = G < CHMAX ? G : CHMAX;
    const int lane = threadIdx.x & 31;
    const int lig = lane & (G - 1);
    const int64_t unit = (int64_t)blockIdx.x * (kThreads / G) + (threadIdx.x / G);
    const bool live = unit < a.n_sched;
    int row = 0;
    int2 extent = make_int2(0, 0);
    if (live) {
        const int p = a.order_begin + (int)unit;
        row = a.order ? a.order[p] : p;
        if (a.extent) {
            extent = a.extent[p];
        } else {
            extent.x = a.pos[row];
            extent.y = a.pos[row + 1] - extent.x;
        }
    }
    const int col = lig * 4;
    const bool col_ok = live && col < a.d;
    const float* xcol = a.x + (col_ok ? col : 0);  // idle lanes read (and discard) column 0
    const float* ycol = f.y + (col_ok ? col : 0);
    const int ldx32 = (int)a.ldx, ldy32 = (int)f.ldy;
    const uint64_t keep_policy = fg::l2_keep_policy();
    const int start = extent.x, len = extent.y;
    const int max_len = __reduce_max_sync(0xffffffffu, len);  // every lane of the warp runs the same batches

    // ---- aggregate: the loop of spmm_rows_kernel ----
    Slice<4> acc;
    acc.zero();
    {
        int my_c = -1;
        float my_v = 0.f;
        if (lig < len) {
            my_c = fg::ld_stream(a.idx + start + lig);
            if (!UNIT) my_v = fg::ld_stream(a.vals + start + lig);
        }
        for (int base = 0; base < max_len; base += G) {
            int nx_c = -1;
            float nx_v = 0.f;
            if (base + G + lig < len) {
                nx_c = fg::ld_stream(a.idx + start + base + G + lig);
                if (!UNIT) nx_v = fg::ld_stream(a.vals + start + base + G + lig);
            }
#pragma unroll
            for (int j0 = 0; j0 < G; j0 += CH) {
                if (base + j0 >= max_len) break;  // warp-uniform
                int c[CH];
                float v[CH];
                Slice<4> xr[CH];
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    c[j] = __shfl_sync(0xffffffffu, my_c, j0 + j, G);
                    v[j] = UNIT ? 1.f : __shfl_sync(0xffffffffu, my_v, j0 + j, G);
                }
#pragma unroll
                for (int j = 0; j < CH; ++j) xr[j].load(xcol + (int64_t)(c[j] < 0 ? 0 : c[j]) * ldx32, keep_policy);
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    Slice<4> next = acc;
                    if (UNIT)
                        next.add(xr[j]);
                    else
                        next.axpy(v[j], xr[j]);
                    acc.select(c[j] >= 0, next);
                }
            }
            my_c = nx_c;
            my_v = nx_v;
        }
    }
    if (col_ok) acc.store(a.out + (int64_t)row * a.ldo + col);
    if (!col_ok) acc.zero();  // lanes beyond the row's width add nothing to a dot product

    // ---- score: the same nonzeros again (their ids are still in L1 / L2), against y ----
    {
        int my_c = -1;
        if (lig < len) my_c = a.idx[start + lig];
        for (int base = 0; base < max_len; base += G) {
            int nx_c = -1;
            if (base + G + lig < len) nx_c = a.idx[start + base + G + lig];
            float r[G / CH];
#pragma unroll
            for (int j0 = 0; j0 < G; j0 += CH) {
                if (base + j0 >= max_len) {  // warp-uniform
                    r[j0 / CH] = 0.f;
                    continue;
                }
                int c[CH];
                float pc[CH];
                Slice<4> yr[CH];
#pragma unroll
                for (int j = 0; j < CH; ++j) c[j] = __shfl_sync(0xffffffffu, my_c, j0 + j, G);
#pragma unroll
                for (int j = 0; j < CH; ++j) yr[j].load(ycol + (int64_t)(c[j] < 0 ? 0 : c[j]) * ldy32, keep_policy);
#pragma unroll
                for (int j = 0; j < CH; ++j) pc[j] = dot4f(0.f, acc.v, yr[j].v);
                r[j0 / CH] = butterfly_in_chunk<CH>(pc, lig);
            }
            const float total = butterfly_across_chunks<G, CH>(r, lig);
            if (base + lig < len) fg::st_stream(f.edge_out + start + base + lig, total);
            my_c = nx_c;
        }
    }
}

// Edges of the long rows (order[0, n_sched)): H is in memory (written by the ring kernels).  A block takes
// (row, share); its warps stride over the row's 32-edge batches, each lane holding one float4 of H[row]
// and of the gathered y rows (d <= 128), with the whole-warp butterfly of the column-block SDDMM kernel.
constexpr int kScoreShares = 8;
__global__ void __launch_bounds__(kThreads, 2) score_long_rows_kernel(const FusedArgs f) {
    const SpmmArgs& a = f.a;
    constexpr int U = 16;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int row = a.order[a.order_begin + blockIdx.x];
    const int start = a.pos[row];
    const int len = a.pos[row + 1] - start;
    const int n_batches = (len + 31) / 32;
    const int col = lane * 4;
    const bool col_ok = col < a.d;
    float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col_ok) h = *reinterpret_cast<const float4*>(a.out + (int64_t)row * a.ldo + col);
    const float* ycol = f.y + (col_ok ? col : 0);
    const int ldy32 = (int)f.ldy;
    const uint64_t keep_policy = fg::l2_keep_policy();
    for (int b = blockIdx.y * (kThreads / 32) + warp; b < n_batches; b += gridDim.y * (kThreads / 32)) {
        const int e0 = start + 32 * b;
        const int cnt = min(32, len - 32 * b);
        int c_l = 0;  // lanes past the end gather row 0 of y; their products are never stored
        if (lane < cnt) c_l = fg::ld_stream(a.idx + e0 + lane);
        float r[32 / U];
#pragma unroll
        for (int s = 0; s < 32; s += U) {
            if (s >= cnt) {  // warp-uniform
                r[s / U] = 0.f;
                continue;
            }
            int c[U];
            float pc[U];
            float4 yr[U];
#pragma unroll
            for (int u = 0; u < U; ++u) c[u] = __shfl_sync(0xffffffffu, c_l, s + u);
#pragma unroll
            for (int u = 0; u < U; ++u) yr[u] = fg::ldg4_keep(ycol + (int64_t)c[u] * ldy32, keep_policy);
#pragma unroll
            for (int u = 0; u < U; ++u) pc[u] = col_ok ? dot4f(0.f, h, yr[u]) : 0.f;
            r[s / U] = butterfly_in_chunk<U>(pc, lane);
        }
        const float total = butterfly_across_chunks<32, U>(r, lane);
        if (lane < cnt) fg::st_stream(f.edge_out + e0 + lane, total);
    }
}

template <int G, bool SHORT>
int launch_fused(const FusedArgs& f, cudaStream_t s) {
    const int64_t units_per_block = kThreads / G;
    const int64_t blocks = (f.a.n_sched + units_per_block - 1) / units_per_block;
    if (blocks > 0x7fffffffLL) return fg::fail(FG_ERR_INVALID_ARGUMENT, "grid too large");
    if (blocks == 0) return FG_OK;
    if (f.a.vals == nullptr)
        fused_rows_kernel<G, true, SHORT><<<(unsigned)blocks, kThreads, 0, s>>>(f);
    else
        fused_rows_kernel<G, false, SHORT><<<(unsigned)blocks, kThreads, 0, s>>>(f);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(1);
    return FG_OK;
}

template <bool SHORT>
int launch_fused_width(const FusedArgs& f, int lanes, cudaStream_t s) {
    switch (lanes) {
        case 1: return launch_fused<1, SHORT>(f, s);
        case 2: return launch_fused<2, SHORT>(f, s);
        case 4: return launch_fused<4, SHORT>(f, s);
        case 8: return launch_fused<8, SHORT>(f, s);
        case 16: return launch_fused<16, SHORT>(f, s);
        default: return launch_fused<32, SHORT>(f, s);
    }
}

int fused_dispatch(const fg_row_schedule* schedule, const int32_t* pos, const int32_t* idx, const float* vals,
                   const float* x, int64_t ldx, const float* y, int64_t ldy, float* h, int64_t ldh, float* edge_out,
                   int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d, void* stream) {
    if (n_rows < 0 || n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld n_cols=%lld nnz=%lld d=%d", (long long)n_rows,
                        (long long)n_cols, (long long)nnz, d);
    if (n_rows > INT32_MAX || n_cols > INT32_MAX || nnz > INT32_MAX)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "sizes beyond int32 indexing are not supported");
    if (d > 128 || d % 4 != 0)
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "d=%d: the fused call keeps a whole row of H in one group's registers and takes d <= 128, "
                        "a multiple of 4 (use fg_spmm_csr_f32 + fg_sddmm_coo_f32 otherwise)", d);
    if (ldx == 0) ldx = d;
    if (ldy == 0) ldy = d;
    if (ldh == 0) ldh = d;
    if (ldx < d || ldy < d || ldh < d || ldx > INT32_MAX || ldy > INT32_MAX || ldh > INT32_MAX || (ldx % 4) || (ldy % 4) ||
        (ldh % 4))
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row strides must be 0 or multiples of 4 in [d=%d, 2^31)", d);
    if (n_rows == 0) return FG_OK;
    if (!pos || !h) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL position or output array");
    if (nnz > 0 && (!idx || !x || !y || !edge_out)) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL array argument");
    if (!fg::aligned16(x) || !fg::aligned16(y) || !fg::aligned16(h))
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "the fused call needs 16-byte aligned feature matrices");
    if (schedule && fg_row_schedule_num_rows(schedule) != n_rows)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "row schedule was built for %lld rows, not %lld",
                        (long long)fg_row_schedule_num_rows(schedule), (long long)n_rows);
    if (schedule && schedule->d_extent && schedule->nnz != nnz)
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "row schedule was built from an adjacency of %lld nonzeros, this call has %lld: rebuild the "
                        "schedule when the adjacency changes", (long long)schedule->nnz, (long long)nnz);
    FusedArgs f;
    SpmmArgs& a = f.a;
    a.pos = pos;
    a.idx = idx;
    a.vals = vals;
    a.x = x;
    a.out = h;
    a.order = schedule ? fg_row_schedule_order(schedule) : nullptr;
    a.extent = schedule ? schedule->d_extent : nullptr;
    a.order_begin = 0;
    a.n_sched = (int32_t)n_rows;
    a.n_rows = (int32_t)n_rows;
    a.d = d;
    a.ldx = ldx;
    a.ldo = ldh;
    a.n_tiles = 1;
    a.parts = 1;
    a.cols_per_part = 0;
    f.y = y;
    f.ldy = ldy;
    f.edge_out = edge_out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int lanes = fg::pow2_ceil(d) / 4;  // G: lanes per row
    // Long rows: the split a side-by-side SpMM launch would choose (their sums need the rings whatever
    // follows); their edges are scored afterwards from H in memory.
    RowSplit split;
    int64_t first_short = n_rows;
    if (schedule) {
        split = choose_row_split(*schedule, d, fg::pow2_ceil(d), true);
        first_short = schedule->rows_at_least[0];
        if (first_short < split.ring) first_short = split.ring;
    }
    SideStream* side = side_stream();
    const bool forked = side && (split.ring > 0 || first_short < n_rows) && side->fork_from(s);
    auto stream_for = [&](int which) { return forked ? side->stream[which] : s; };
    int rc = FG_OK;
    if (split.ring > 0) {
        // heavy rows, long rows and then their edges, one after the other on one stream
        cudaStream_t ls = stream_for(SideStream::kHeavy);
        SpmmArgs r = a;
        r.n_tiles = (d + 31) / 32;
        r.order_begin = 0;
        r.n_sched = (int32_t)split.heavy;
        rc = launch_heavy(r, split.wide, ls);
        if (rc == FG_OK) {
            r.order_begin = (int32_t)split.heavy;
            r.n_sched = (int32_t)(split.ring - split.heavy);
            rc = launch_long(r, ls);
        }
        if (rc == FG_OK) {
            FusedArgs g = f;
            g.a.order_begin = 0;
            g.a.n_sched = (int32_t)split.ring;
            score_long_rows_kernel<<<dim3((unsigned)split.ring, kScoreShares), kThreads, 0, ls>>>(g);
            const cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) rc = fg::fail(FG_ERR_CUDA, "score_long_rows_kernel: %s", cudaGetErrorString(e));
            fg::count_launches(1);
        }
    }
    if (rc == FG_OK) {
        FusedArgs g = f;
        g.a.order_begin = (int32_t)split.ring;
        g.a.n_sched = (int32_t)(first_short - split.ring);
        rc = launch_fused_width<false>(g, lanes, s);
    }
    if (rc == FG_OK && first_short < n_rows) {
        FusedArgs g = f;
        g.a.order_begin = (int32_t)first_short;
        g.a.n_sched = (int32_t)(n_rows - first_short);
        rc = launch_fused_width<true>(g, lanes, stream_for(SideStream::kShort));
    }
    if (forked) {
        const int rcj = side->join_to(s);
        if (rc == FG_OK) rc = rcj;
    }
    return rc;
}

}  // namespace

#define FG_STR_(x) #x
#define FG_STR(x) FG_STR_(x)
const char* fg::spmm_signature() {
    // rows kernel: gathers in flight, blocks per SM (regular / short form); ring: slots x nonzeros, warps;
    // heavy: warps (narrow|wide), turns deep
    return "spmm_rows<ch" FG_STR(FG_ROWS_CH) "," FG_STR(FG_ROWS_MINB) "/SM|short:ch" FG_STR(FG_SHORT_CH) "," FG_STR(
        FG_SHORT_MINB) "/SM>,ring<" FG_STR(FG_RING_SLOTS) "x32," FG_STR(FG_RING_WARPS) "w>,heavy<4|8w,3deep>,hints<" FG_STR(
        FG_HINT_KEEP) FG_STR(FG_HINT_STREAM) ">";
}

extern "C" {

int fg_spmm_csr_f32(const fg_row_schedule* schedule, const int32_t* d_indptr,
                    const int32_t* d_indices, const float* d_vals, const float* d_x, int64_t ldx,
                    float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                    int32_t feat_tile, void* stream) {
    return spmm_dispatch(schedule, d_indptr, d_indices, d_vals, d_x, ldx, d_out, ldo, n_rows, n_cols,
                         nnz, d, 1, feat_tile, stream, false);
}

int fg_spmm_sddmm_fused_f32(const fg_row_schedule* schedule, const int32_t* d_indptr, const int32_t* d_indices,
                            const float* d_vals, const float* d_x, int64_t ldx, const float* d_y, int64_t ldy,
                            float* d_h, int64_t ldh, float* d_edge_out, int64_t n_rows, int64_t n_cols, int64_t nnz,
                            int32_t d, void* stream) {
    return fused_dispatch(schedule, d_indptr, d_indices, d_vals, d_x, ldx, d_y, ldy, d_h, ldh, d_edge_out, n_rows,
                          n_cols, nnz, d, stream);
}

int fg_spmm_dds_f32(const fg_row_schedule* schedule, const int32_t* d_s1_pos,
                    const int32_t* d_s1_idx, const float* d_vals, const float* d_x, int64_t ldx,
                    float* d_out, int64_t ldo, int64_t n_rows, int64_t n_cols, int64_t nnz, int32_t d,
                    int32_t num_col_partitions, int32_t feat_tile, void* stream) {
    return spmm_dispatch(schedule, d_s1_pos, d_s1_idx, d_vals, d_x, ldx, d_out, ldo, n_rows, n_cols,
                         nnz, d, num_col_partitions, feat_tile, stream, true);
}

}  // extern "C"

// =============================================================================================
// SpMM without any allocation: fg_spmm_csr_f32_static
//
// For callers that must not see a cudaMalloc: a serving process that has handed all of the
// device's memory to its own pool (an allocation by this library would fail or eat into that
// pool's reserve), or a latency-critical loop where the device-wide synchronisation hidden in
// cudaMalloc / cudaFree is not acceptable.  The regular path needs an fg_row_schedule, which
// is built with cudaMalloc'ed buffers; here the row order is rebuilt on every call inside one
// statically allocated device array, so the entry point only launches kernels.
//
// The order is a bucket order (rows grouped by floor(log2(nonzeros)), heaviest bucket first)
// rather than a full sort: any order gives the same output bits, the grouping is what the
// kernel needs for balance.  No long-row kernel is used on this path.
// =============================================================================================
namespace {

constexpr int kStaticBuckets = 64;  // bucket = number of significant bits of the row's nonzero count
// Scratch layout (int32 words): [0, FG_SPMM_STATIC_MAX_ROWS) row order,
// then kStaticBuckets bucket sizes, then kStaticBuckets fill cursors.
constexpr int64_t kStaticWords = (int64_t)FG_SPMM_STATIC_MAX_ROWS + 2 * kStaticBuckets;
static __device__ __align__(256) int32_t g_spmm_static_scratch[kStaticWords];

__device__ __forceinline__ int static_bucket(int nnz_in_row) { return nnz_in_row <= 0 ? 0 : 32 - __clz(nnz_in_row); }

// Every call starts from zeroed counters: the array keeps whatever the previous call left.
__global__ void static_clear_kernel(int32_t* counters) {
    if (threadIdx.x < 2 * kStaticBuckets) counters[threadIdx.x] = 0;
}

__global__ void static_count_kernel(const int32_t* __restrict__ indptr, int32_t n_rows, int32_t* sizes) {
    __shared__ int local[kStaticBuckets];
    if (threadIdx.x < kStaticBuckets) local[threadIdx.x] = 0;
    __syncthreads();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_rows) atomicAdd(&local[static_bucket(indptr[r + 1] - indptr[r])], 1);
    __syncthreads();
    if (threadIdx.x < kStaticBuckets && local[threadIdx.x]) atomicAdd(&sizes[threadIdx.x], local[threadIdx.x]);
}

// cursor[b] = first slot of bucket b when buckets are laid out from the heaviest down
__global__ void static_offsets_kernel(const int32_t* sizes, int32_t* cursors) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int at = 0;
        for (int b = kStaticBuckets - 1; b >= 0; --b) {
            cursors[b] = at;
            at += sizes[b];
        }
    }
}

__global__ void static_scatter_kernel(const int32_t* __restrict__ indptr, int32_t n_rows, int32_t* cursors,
                                      int32_t* __restrict__ order) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_rows) order[atomicAdd(&cursors[static_bucket(indptr[r + 1] - indptr[r])], 1)] = r;
}

// Device address of the scratch array, looked up once per device.  In host code the array's
// name is only a handle for the runtime; cudaGetSymbolAddress gives the pointer kernels can use.
int static_scratch_address(int32_t** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex lock;
    static int32_t* address[kMaxDevices] = {nullptr};
    int dev = 0;
    FG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fg::fail(FG_ERR_INVALID_ARGUMENT, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> hold(lock);
    if (!address[dev]) {
        void* p = nullptr;
        FG_CUDA_TRY(cudaGetSymbolAddress(&p, g_spmm_static_scratch));
        if (!p) return fg::fail(FG_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        address[dev] = static_cast<int32_t*>(p);
    }
    *out = address[dev];
    return FG_OK;
}

}  // namespace

extern "C" {

int fg_spmm_csr_f32_static(const int32_t* d_indptr, const int32_t* d_indices, const float* d_vals,
                           const float* d_x, float* d_out, int64_t n_rows, int64_t n_cols, int64_t nnz,
                           int32_t d, int32_t feat_tile, void* stream) {
    if (n_rows < 0) return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_rows=%lld", (long long)n_rows);
    if (n_rows > FG_SPMM_STATIC_MAX_ROWS)
        return fg::fail(FG_ERR_INVALID_ARGUMENT,
                        "n_rows=%lld is beyond the %d rows the static scratch array holds; use "
                        "fg_row_schedule_create + fg_spmm_csr_f32 for larger matrices",
                        (long long)n_rows, (int)FG_SPMM_STATIC_MAX_ROWS);
    if (n_cols < 0 || nnz < 0 || d < 1)
        return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad sizes n_cols=%lld nnz=%lld d=%d", (long long)n_cols,
                        (long long)nnz, d);
    if (n_rows == 0) return FG_OK;
    if (!d_indptr || !d_out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "NULL position or output array");
    int32_t* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != FG_OK) return rc;
    int32_t* order = scratch;
    int32_t* sizes = scratch + FG_SPMM_STATIC_MAX_ROWS;
    int32_t* cursors = sizes + kStaticBuckets;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = 256;
    const unsigned blocks = (unsigned)((n_rows + threads - 1) / threads);
    static_clear_kernel<<<1, 2 * kStaticBuckets, 0, s>>>(sizes);
    static_count_kernel<<<blocks, threads, 0, s>>>(d_indptr, (int32_t)n_rows, sizes);
    static_offsets_kernel<<<1, 32, 0, s>>>(sizes, cursors);
    static_scatter_kernel<<<blocks, threads, 0, s>>>(d_indptr, (int32_t)n_rows, cursors, order);
    FG_CUDA_TRY(cudaGetLastError());
    fg::count_launches(4);
    // a schedule view over the scratch array; "fixed threshold, no rows" keeps the long-row kernel off
    fg_row_schedule view;
    view.d_order = order;
    view.n_rows = n_rows;
    view.nnz = nnz;
    view.fixed_threshold = INT32_MAX;
    view.fixed_rows = 0;
    view.rows_at_least[0] = n_rows;  // no degree statistics here: one kernel form for all rows, no side streams
    return spmm_dispatch(&view, d_indptr, d_indices, d_vals, d_x, d, d_out, d, n_rows, n_cols, nnz, d,
                         1, feat_tile, stream, false);
}

}  // extern "C"

