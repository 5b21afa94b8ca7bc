// Sum / mean / sym-norm aggregation over a block CSR, forward (gather) and backward (scatter), sm_100a.
//
// The work is HBM-bound (one FMA per 4 bytes read), so no tensor cores: a warp owns one destination row,
// its lanes sweep the feature dimension with 128-bit loads (64- or 32-bit when the row stride is not a
// multiple of 16 bytes, e.g. 602 floats), the neighbour ids of the row are read once, coalesced, and handed
// round by shuffle, the loads of several neighbours are issued before the first FMA, the ids of the warp's
// next row are fetched while the current row is summed, and the row's sum stays in registers until one
// coalesced store.  The number of accumulators is a template parameter chosen from
// the row width, so narrow rows (100 / 128 floats) run with few registers and full occupancy.
//
// The forward kernel also runs over a whole window of mini-batches (per-batch strides, rows in batch-major
// order), so the first layer of the window -- which reads only the feature table and does not depend on the
// weights -- is one launch that is long enough to reach a steady state.
//
// Replaces K8 / K10 (aggregate_acc_kernel.cu:271-331, :376-427: 8 rows x 4 floats per warp, shared-memory
// read-modify-write per neighbour) and K9 / K11 (:468-517, :555-596: scalar atomics, the GCN one built from
// two atomicExch in a retry loop).
#include <algorithm>

#include <cooperative_groups.h>

#include "common.cuh"

namespace fgl {

#ifndef FGL_AGG_THREADS
#define FGL_AGG_THREADS 256
#endif
constexpr int kAggThreads = FGL_AGG_THREADS;
constexpr int kAggWarps = kAggThreads / 32;
#ifndef FGL_AGG_UNR1
#define FGL_AGG_UNR1 8  // neighbour rows in flight per lane for rows of up to 32 vectors
#endif
#ifndef FGL_AGG_MIN_CTAS
#define FGL_AGG_MIN_CTAS 2
#endif

template <int VEC>
struct Vec;
template <>
struct Vec<4> {
    using T = float4;
    static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    static __device__ __forceinline__ void fma(T& a, float w, const T& x) {
        a.x = fmaf(w, x.x, a.x);
        a.y = fmaf(w, x.y, a.y);
        a.z = fmaf(w, x.z, a.z);
        a.w = fmaf(w, x.w, a.w);
    }
    static __device__ __forceinline__ T scale(const T& a, float w) { return make_float4(a.x * w, a.y * w, a.z * w, a.w * w); }
};
template <>
struct Vec<2> {
    using T = float2;
    static __device__ __forceinline__ T zero() { return make_float2(0.f, 0.f); }
    static __device__ __forceinline__ void fma(T& a, float w, const T& x) {
        a.x = fmaf(w, x.x, a.x);
        a.y = fmaf(w, x.y, a.y);
    }
    static __device__ __forceinline__ T scale(const T& a, float w) { return make_float2(a.x * w, a.y * w); }
};
template <>
struct Vec<1> {
    using T = float;
    static __device__ __forceinline__ T zero() { return 0.f; }
    static __device__ __forceinline__ void fma(T& a, float w, const T& x) { a = fmaf(w, x, a); }
    static __device__ __forceinline__ T scale(const T& a, float w) { return a * w; }
};

struct AggParams {
    const int32_t* indptr;
    const int32_t* src;
    const int32_t* src_deg;
    const int32_t* dst_deg;
    const int32_t* row_map;
    const float* x;  // forward: input rows; backward: dy
    float* out;      // forward: out; backward: dx
    float* self_out; // forward, optional: copy of the row's own input row x[row(d)]
    int64_t ldx, ldo, ld_self;
    int32_t dim, n_dst, n_src;
    int32_t passthrough;
    // window forward: all zero / NULL for a single block
    int64_t indptr_stride, src_stride, row_map_stride;
    int32_t n_batches;
    const int64_t* out_row_off;  // [n_batches + 1]: first output row of batch b, then the total
    // optional: the real number of destination rows, read on the device (n_dst is then the padded row count
    // the launch is sized for; forward rows beyond the real count are zero-filled)
    const int32_t* n_dst_dev;
    // optional: x is row-sharded over several tables (one per GPU, peer-mapped); global row r lives in
    // shards[r / rows_per_shard] at local row r % rows_per_shard
    const float* const* shards;
    int64_t rows_per_shard;
    // FGL_AGG_EDGE: one weight per (edge, head), edge_w[e * n_heads + h]; head h covers dim / n_heads columns
    const float* edge_w;
    int32_t n_heads;
    // bounds of the ids the kernels dereference: x (or the sharded table) has n_rows rows; with a row map the local
    // ids index a map of n_map entries.  An id outside its range is never dereferenced: the edge (or the gathered
    // row) contributes zeros and FGL_ERR_BOUNDS goes to *status (may be NULL).
    int64_t n_rows;
    int64_t n_map;
    int32_t* status;
};

__device__ __forceinline__ void agg_bad_id(const AggParams& p) {
    if (p.status) set_status(p.status, FGL_ERR_BOUNDS);
}

// Row of x that local id s stands for, or -1 (recorded) when s or the mapped row is out of range.
template <bool HAS_MAP>
__device__ __forceinline__ int64_t checked_row(const AggParams& p, const int32_t* row_map, int s) {
    int64_t r = (int64_t)s;
    if (HAS_MAP) {
        if (s < 0 || (int64_t)s >= p.n_map) {
            agg_bad_id(p);
            return -1;
        }
        r = (int64_t)__ldg(row_map + s);
    }
    if (r < 0 || r >= p.n_rows) {
        agg_bad_id(p);
        return -1;
    }
    return r;
}

// Start of input row r: in the single table, or in the shard (possibly another GPU's HBM, read with plain
// peer loads over NVLink) that owns it.
__device__ __forceinline__ const float* x_row(const AggParams& p, int64_t r) {
    if (p.shards == nullptr) return p.x + r * p.ldx;
    const int64_t s = r / p.rows_per_shard;
    return p.shards[s] + (r - s * p.rows_per_shard) * p.ldx;
}

// Forward: out[d,:] = scale_d * sum_e w_e * x[row(src[e]),:]
// NACC vector accumulators per lane cover 32 * NACC * VEC floats per pass; UNR neighbours' loads are in
// flight before their FMAs.  In window mode (out_row_off != NULL) the rows of all mini-batches form one
// sequence in batch-major order and the grid sweeps it front to back, so that at any moment the CTAs work
// on one or two mini-batches and the rows those batches re-read stay in L2.
//
// A warp issues its instructions in order, so a value that was just requested from memory stalls the warp at its
// first use.  The ids of a row form a dependent chain -- indptr[d] -> src[a + lane] -> row_map[s] -> the feature
// rows -- and walked one row at a time that chain is four round trips per destination row, more than the row data
// itself costs.  The chain is therefore software-pipelined over the warp's rows: while row i is summed, the map
// entries of row i+1, the source ids of row i+2 and the offsets of row i+3 are in flight, and every loaded value is
// first touched one iteration after it was requested.  The row's own input row (the "self" copy) is requested
// together with the first batch of neighbour rows, not before it.
constexpr int kAggMaxWindow = 512;  // mini-batches per window launch (their row offsets are staged in shared memory)

template <int VEC, int MODE, bool HAS_MAP, int NACC, int UNR>
__global__ void __launch_bounds__(kAggThreads, FGL_AGG_MIN_CTAS) agg_fwd_kernel(const AggParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    __shared__ long long s_off[kAggMaxWindow + 1];
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;  // dim % VEC == 0 by dispatch
    const bool window = p.out_row_off != nullptr;
    if (window) {
        for (int i = threadIdx.x; i <= p.n_batches; i += blockDim.x) s_off[i] = __ldg(p.out_row_off + i);
        __syncthreads();
    }
    const int64_t padded = window ? s_off[p.n_batches] : (int64_t)p.n_dst;
    const int64_t total = p.n_dst_dev ? min((int64_t)max(__ldg(p.n_dst_dev), 0), padded) : padded;
    // padding rows of a launch sized for more rows than the block has: zero them
    for (int64_t g = total + warp_global; g < padded; g += n_warps) {
        T* orow = reinterpret_cast<T*>(p.out + g * p.ldo);
        for (int c = lane; c < chunks; c += 32) orow[c] = V::zero();
    }
    const bool want_self = p.self_out != nullptr || p.passthrough != 0;

    // ---- pipeline state: stage A (offsets), B (source ids), C (map entries / degrees) ------------------------------
    int bA = 0, dA = 0, aA = 0, eA = 0;              // row i+3 after its stage A: batch, local row, edge range
    int bB = 0, dB = 0, aB = 0, eB = 0, sB = -1;      // row i+2 after stage B: + this lane's source id
    int selfB = -1;                                   //                         + the row's own input row (raw)
    int ddegB = 1;
    int bC = 0, dC = 0, aC = 0, eC = 0, sC = -1;      // row i+1 after stage C: + raw map entry / degree of the lane's source
    int rowC = 0, selfC = -1;
    int sdegC = 1, ddegC = 1;
    int batch_ptr = 0;                                // window mode: batch of the row stage A looks at (monotonic)

    auto stage_a = [&](int64_t g) {  // offsets of row g
        aA = 0;
        eA = 0;
        if (g >= total) return;
        if (window) {
            while (g >= s_off[batch_ptr + 1]) ++batch_ptr;
            bA = batch_ptr;
            dA = (int)(g - s_off[batch_ptr]);
        } else {
            bA = 0;
            dA = (int)g;
        }
        const int32_t* indptr = p.indptr + (int64_t)bA * p.indptr_stride;
        aA = __ldg(indptr + dA);
        eA = __ldg(indptr + dA + 1);
    };
    auto stage_b = [&]() {  // source ids of the row stage A saw one iteration ago (its offsets have arrived)
        bB = bA;
        dB = dA;
        aB = aA;
        eB = eA;
        sB = -1;
        selfB = -1;
        if (lane < eB - aB) sB = __ldg(p.src + (int64_t)bB * p.src_stride + aB + lane);
        if (want_self) {
            if (HAS_MAP)
                selfB = (int64_t)dB < p.n_map ? __ldg(p.row_map + (int64_t)bB * p.row_map_stride + dB) : -1;
            else
                selfB = dB;
        }
        if (MODE == FGL_AGG_SYMNORM && eB > aB) ddegB = __ldg(p.dst_deg + dB);
    };
    auto stage_c = [&]() {  // map entry and degree of this lane's source (the id has arrived)
        bC = bB;
        dC = dB;
        aC = aB;
        eC = eB;
        sC = sB;
        selfC = selfB;
        ddegC = ddegB;
        rowC = sB;
        sdegC = 1;
        const bool id_ok = sB >= 0 && (HAS_MAP ? (int64_t)sB < p.n_map : (int64_t)sB < p.n_rows);
        if (id_ok) {
            if (HAS_MAP) rowC = __ldg(p.row_map + (int64_t)bC * p.row_map_stride + sB);
            if (MODE == FGL_AGG_SYMNORM) sdegC = __ldg(p.src_deg + sB);
        } else {
            rowC = -1;  // no such edge in this lane, or an id out of range (told apart when the row is summed)
        }
    };

    // prologue: fill the pipeline (each stage waits for the one before it, once)
    stage_a(warp_global);
    stage_b();
    stage_c();
    stage_a(warp_global + (int64_t)n_warps);
    stage_b();
    stage_a(warp_global + 2 * (int64_t)n_warps);

    for (int64_t g = warp_global; g < total; g += n_warps) {
        // ---- the current row: everything below was requested at least one iteration ago ----------------------------
        const int b = bC, a = aC, e_end = eC;
        const int cnt_first = min(32, e_end - a);
        const bool has_edge = lane < cnt_first;
        bool bad = has_edge && (rowC < 0 || (int64_t)rowC >= p.n_rows);
        if (bad) agg_bad_id(p);
        const int first_row = (has_edge && !bad) ? rowC : 0;
        const unsigned first_bad = __ballot_sync(0xffffffffu, bad);
        float first_w = 1.0f;
        if (MODE == FGL_AGG_SYMNORM && has_edge && !bad) first_w = 1.0f / sqrtf((float)sdegC);
        int self_row = selfC;
        const int ddeg = ddegC;
        const bool need_self = p.self_out != nullptr || (a >= e_end && p.passthrough);
        if (need_self && (self_row < 0 || (int64_t)self_row >= p.n_rows)) {
            agg_bad_id(p);
            self_row = -1;
        }
        const int32_t* src = p.src + (int64_t)b * p.src_stride;
        const int32_t* row_map = HAS_MAP ? p.row_map + (int64_t)b * p.row_map_stride : nullptr;
        T* orow = reinterpret_cast<T*>(p.out + g * p.ldo);

        // ---- requests of this iteration, all issued before anything is consumed ------------------------------------
        // (1) the row's own input row (narrow rows: one vector per lane, kept in a register until it is stored)
        T self_v = V::zero();
        const bool self_in_reg = NACC == 1 && need_self && self_row >= 0;
        if (self_in_reg && lane < chunks) self_v = __ldg(reinterpret_cast<const T*>(x_row(p, self_row)) + lane);
        // (2) the first batch of neighbour rows, first pass over the columns
        T v0[UNR][NACC];
        if (a < e_end) {
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int j = min(u, cnt_first - 1);  // past the end: reload the last row, skip its FMA
                const int r = __shfl_sync(0xffffffffu, first_row, j);
                const T* xr = reinterpret_cast<const T*>(x_row(p, r));
#pragma unroll
                for (int k = 0; k < NACC; ++k) {
                    const int c = k * 32 + lane;
                    v0[u][k] = (c < chunks) ? __ldg(xr + c) : V::zero();
                }
            }
        }
        // (3) the pipeline stages of the warp's next rows
        stage_c();
        stage_b();
        stage_a(g + 3 * (int64_t)n_warps);

        // ---- consume ------------------------------------------------------------------------------------------------
        if (p.self_out) {
            T* srow = reinterpret_cast<T*>(p.self_out + g * p.ld_self);
            if (NACC == 1) {
                if (lane < chunks) srow[lane] = self_v;
            } else {
                const T* xr = reinterpret_cast<const T*>(x_row(p, self_row < 0 ? 0 : self_row));
                for (int c = lane; c < chunks; c += 32) srow[c] = self_row < 0 ? V::zero() : __ldg(xr + c);
            }
        }
        if (a >= e_end) {  // aggregate_acc_kernel.cu:307-308, :405-406
            if (NACC == 1) {
                if (lane < chunks) orow[lane] = p.passthrough ? self_v : V::zero();
            } else {
                const T* xr = reinterpret_cast<const T*>(x_row(p, self_row < 0 ? 0 : self_row));
                for (int c = lane; c < chunks; c += 32) orow[c] = (p.passthrough && self_row >= 0) ? __ldg(xr + c) : V::zero();
            }
            continue;
        }
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(e_end - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)ddeg);

        for (int c0 = 0; c0 < chunks; c0 += 32 * NACC) {
            T acc[NACC];
            int head[NACC];
#pragma unroll
            for (int k = 0; k < NACC; ++k) {
                acc[k] = V::zero();
                head[k] = (MODE == FGL_AGG_EDGE) ? min(((c0 + k * 32 + lane) * VEC) / (p.dim / p.n_heads), p.n_heads - 1) : 0;
            }
            for (int e0 = a; e0 < e_end; e0 += 32) {
                const int cnt = min(32, e_end - e0);
                int my_row = first_row;
                float my_w = first_w;
                unsigned bad_mask = first_bad;
                if (e0 != a) {  // rows with more than 32 in-edges: their further ids are fetched in line
                    my_row = 0;
                    my_w = 1.0f;
                    bool bad2 = false;
                    if (lane < cnt) {
                        const int s = __ldg(src + e0 + lane);
                        my_row = (int)checked_row<HAS_MAP>(p, row_map, s);
                        bad2 = my_row < 0;
                        if (bad2) my_row = 0;
                        if (MODE == FGL_AGG_SYMNORM && !bad2) my_w = 1.0f / sqrtf((float)__ldg(p.src_deg + s));
                    }
                    bad_mask = __ballot_sync(0xffffffffu, bad2);
                }
                int j0 = 0;
                if (c0 == 0 && e0 == a) {  // warp-uniform: the batch requested before the pipeline stages
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const float wu = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, min(u, cnt - 1)) : 1.0f;
                        if (u < cnt && !((bad_mask >> u) & 1u)) {
#pragma unroll
                            for (int k = 0; k < NACC; ++k) {
                                const float wk = (MODE == FGL_AGG_EDGE) ? __ldg(p.edge_w + (int64_t)(e0 + u) * p.n_heads + head[k]) : wu;
                                V::fma(acc[k], wk, v0[u][k]);
                            }
                        }
                    }
                    j0 = UNR;
                }
                for (; j0 < cnt; j0 += UNR) {
                    T v[UNR][NACC];
                    float w[UNR];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int j = min(j0 + u, cnt - 1);  // past the end: reload the last row, skip its FMA
                        const int r = __shfl_sync(0xffffffffu, my_row, j);
                        w[u] = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, j) : 1.0f;
                        const T* xr = reinterpret_cast<const T*>(x_row(p, r));
#pragma unroll
                        for (int k = 0; k < NACC; ++k) {
                            const int c = c0 + k * 32 + lane;
                            v[u][k] = (c < chunks) ? __ldg(xr + c) : V::zero();
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        if (j0 + u < cnt && !((bad_mask >> (j0 + u)) & 1u)) {  // warp-uniform
#pragma unroll
                            for (int k = 0; k < NACC; ++k) {
                                const float wk = (MODE == FGL_AGG_EDGE)
                                                     ? __ldg(p.edge_w + (int64_t)(e0 + j0 + u) * p.n_heads + head[k])
                                                     : w[u];
                                V::fma(acc[k], wk, v[u][k]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < NACC; ++k) {
                const int c = c0 + k * 32 + lane;
                if (c < chunks) orow[c] = (MODE == FGL_AGG_SUM || MODE == FGL_AGG_EDGE) ? acc[k] : V::scale(acc[k], scale);
            }
        }
    }
}

// The same forward aggregation for the shapes a sampled mini-batch has on its widest hop -- rows of at most 32
// 128-bit vectors (D <= 128 floats), a single dense table, sum / mean / sym-norm -- with the rows staged through
// shared memory by asynchronous copies (cp.async, 16 bytes per lane, L2 only) instead of through registers.
//
// Why: a warp of agg_fwd_kernel holds every byte it has in flight in registers; at 120 registers a thread an SM keeps
// 16 warps x 8 rows = 50 KB in flight, and on 400-byte rows fetched at random from HBM that -- not bandwidth -- bounds
// the kernel (measured: 2.6 TB/s of DRAM traffic, 40 % of the copy peak).  Here every warp owns kAggSlots row slots of
// shared memory and needs few registers, so an SM runs 24 warps with 16 rows each in flight (150 KB; measured best).  Per
// destination row a warp requests its own input row (slot 0, the self copy) and up to 15 neighbour rows (a row sampled
// with fanout 15 is exactly one pass), moves the id pipeline (indptr -> src -> row_map, three rows ahead, as in
// agg_fwd_kernel) while the copies fly, waits for its copies, and adds the rows out of shared memory.  Per neighbour
// row that is one shuffle, one multiply-add and one cp.async, later one 128-bit shared-memory load and four adds.  Rows
// with more than 15 in-edges take further passes whose ids are fetched in line.
constexpr int kAggSlots = 16;
#ifndef FGL_AGG_STAGED_WARPS
#define FGL_AGG_STAGED_WARPS 24
#endif
constexpr int kAggStagedMaxWarps = FGL_AGG_STAGED_WARPS;  // per CTA (one CTA per SM); fewer when the rows are wider

__device__ __forceinline__ void cp_async16(unsigned smem_dst, const void* gmem_src) {  // smem_dst: shared-space address
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ float4 lds128(unsigned smem_src) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_src));
    return v;
}

template <int MODE, bool HAS_MAP>
__global__ void __launch_bounds__(kAggStagedMaxWarps * 32, 1) agg_fwd_staged_kernel(const AggParams p) {
    using V = Vec<4>;
    using T = float4;
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ long long s_off[kAggMaxWindow + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cta_warps = blockDim.x >> 5;
    const int warp_global = blockIdx.x * cta_warps + warp;
    const int n_warps = gridDim.x * cta_warps;
    const int chunks = p.dim / 4;  // <= 32
    const unsigned slot_bytes = (unsigned)chunks * 16u;
    const bool window = p.out_row_off != nullptr;
    if (window) {
        for (int i = threadIdx.x; i <= p.n_batches; i += blockDim.x) s_off[i] = __ldg(p.out_row_off + i);
        __syncthreads();
    }
    const int64_t padded = window ? s_off[p.n_batches] : (int64_t)p.n_dst;
    const int64_t total = p.n_dst_dev ? min((int64_t)max(__ldg(p.n_dst_dev), 0), padded) : padded;
    const bool lane_on = lane < chunks;
    for (int64_t g = total + warp_global; g < padded; g += n_warps)
        if (lane_on) reinterpret_cast<T*>(p.out + g * p.ldo)[lane] = V::zero();
    const bool want_self = p.self_out != nullptr || p.passthrough != 0;
    // Lanes beyond the row's last vector repeat that vector (same source, same destination: a duplicate request inside
    // one instruction), so that no copy, load or add in the loops below needs a per-lane predicate.
    const int lane_c = min(lane, chunks - 1);
    const char* lane_base = reinterpret_cast<const char*>(p.x) + lane_c * 16;
    const unsigned ld_bytes = (unsigned)(p.ldx * 4);
    auto row_ptr = [&](int r) { return lane_base + (uint64_t)(unsigned)r * ld_bytes; };  // one 32 x 32 + 64 multiply-add
    const unsigned slots = (unsigned)__cvta_generic_to_shared(dyn_smem) + (unsigned)warp * kAggSlots * slot_bytes + lane_c * 16;

    // ---- id pipeline, three destination rows ahead (see agg_fwd_kernel) ------------------------------------------------
    int bA = 0, dA = 0, aA = 0, eA = 0;
    int bB = 0, dB = 0, aB = 0, eB = 0, sB = -1, selfB = -1, ddegB = 1;
    int bC = 0, aC = 0, eC = 0, rowC = 0, selfC = -1, sdegC = 1, ddegC = 1;
    int batch_ptr = 0;
    auto stage_a = [&](int64_t g) {
        aA = 0;
        eA = 0;
        if (g >= total) return;
        if (window) {
            while (g >= s_off[batch_ptr + 1]) ++batch_ptr;
            bA = batch_ptr;
            dA = (int)(g - s_off[batch_ptr]);
        } else {
            bA = 0;
            dA = (int)g;
        }
        const int32_t* indptr = p.indptr + (int64_t)bA * p.indptr_stride;
        aA = __ldg(indptr + dA);
        eA = __ldg(indptr + dA + 1);
    };
    auto stage_b = [&]() {
        bB = bA;
        dB = dA;
        aB = aA;
        eB = eA;
        sB = -1;
        selfB = -1;
        if (lane < min(eB - aB, kAggSlots - 1)) sB = __ldg(p.src + (int64_t)bB * p.src_stride + aB + lane);
        if (want_self) {
            if (HAS_MAP)
                selfB = (int64_t)dB < p.n_map ? __ldg(p.row_map + (int64_t)bB * p.row_map_stride + dB) : -1;
            else
                selfB = dB;
        }
        if (MODE == FGL_AGG_SYMNORM && eB > aB) ddegB = __ldg(p.dst_deg + dB);
    };
    auto stage_c = [&]() {
        bC = bB;
        aC = aB;
        eC = eB;
        selfC = selfB;
        ddegC = ddegB;
        rowC = sB;
        sdegC = 1;
        const bool id_ok = sB >= 0 && (HAS_MAP ? (int64_t)sB < p.n_map : (int64_t)sB < p.n_rows);
        if (id_ok) {
            if (HAS_MAP) rowC = __ldg(p.row_map + (int64_t)bC * p.row_map_stride + sB);
            if (MODE == FGL_AGG_SYMNORM) sdegC = __ldg(p.src_deg + sB);
        } else {
            rowC = -1;
        }
    };
    stage_a(warp_global);
    stage_b();
    stage_c();
    stage_a(warp_global + (int64_t)n_warps);
    stage_b();
    stage_a(warp_global + 2 * (int64_t)n_warps);

    // Copy `cnt` rows (lane u holds row u) into slots 1 .. cnt; add them out of shared memory.
    auto request = [&](int my_row, int cnt) {
        unsigned dst = slots;
        if (cnt == kAggSlots - 1) {  // the common case: a row sampled with the full fanout
#pragma unroll
            for (int u = 0; u < kAggSlots - 1; ++u) {
                dst += slot_bytes;
                cp_async16(dst, row_ptr(__shfl_sync(0xffffffffu, my_row, u)));
            }
        } else {
            for (int u = 0; u < cnt; ++u) {
                dst += slot_bytes;
                cp_async16(dst, row_ptr(__shfl_sync(0xffffffffu, my_row, u)));
            }
        }
    };
    auto add_up = [&](T& acc, int cnt, unsigned bad_mask, float my_w) {
        unsigned from = slots;
        if (cnt == kAggSlots - 1 && bad_mask == 0u) {
#pragma unroll
            for (int u = 0; u < kAggSlots - 1; ++u) {
                from += slot_bytes;
                V::fma(acc, (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, u) : 1.0f, lds128(from));
            }
        } else {
            for (int u = 0; u < cnt; ++u) {
                from += slot_bytes;
                const float wu = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, u) : 1.0f;
                if (!((bad_mask >> u) & 1u)) V::fma(acc, wu, lds128(from));
            }
        }
    };

    for (int64_t g = warp_global; g < total; g += n_warps) {
        // the current row: its ids were requested at least one iteration ago
        const int b = bC, a = aC, e_end = eC, ddeg = ddegC;
        const int cnt = min(kAggSlots - 1, e_end - a);
        const bool has_edge = lane < cnt;
        const bool bad = has_edge && (rowC < 0 || (int64_t)rowC >= p.n_rows);
        if (bad) agg_bad_id(p);
        const int my_row = (has_edge && !bad) ? rowC : 0;
        const unsigned bad_mask = __ballot_sync(0xffffffffu, bad);
        float my_w = 1.0f;
        if (MODE == FGL_AGG_SYMNORM && has_edge && !bad) my_w = 1.0f / sqrtf((float)sdegC);
        int self_row = selfC;
        const bool need_self = p.self_out != nullptr || (a >= e_end && p.passthrough);
        if (need_self && (self_row < 0 || (int64_t)self_row >= p.n_rows)) {
            agg_bad_id(p);
            self_row = -1;
        }
        // requests: the row's own input row, its first 15 neighbours, the next rows' ids
        if (need_self && self_row >= 0) cp_async16(slots, row_ptr(self_row));
        request(my_row, cnt);
        stage_c();
        stage_b();
        stage_a(g + 3 * (int64_t)n_warps);
        cp_async_wait_all();
        __syncwarp();
        // consume
        T self_v = V::zero();
        if (need_self && self_row >= 0) self_v = lds128(slots);
        if (p.self_out && lane_on) reinterpret_cast<T*>(p.self_out + g * p.ld_self)[lane] = self_v;
        T* orow = reinterpret_cast<T*>(p.out + g * p.ldo);
        if (a >= e_end) {  // aggregate_acc_kernel.cu:307-308, :405-406
            if (lane_on) orow[lane] = p.passthrough ? self_v : V::zero();
            __syncwarp();
            continue;
        }
        T acc = V::zero();
        add_up(acc, cnt, bad_mask, my_w);
        __syncwarp();  // every lane is done with the slots before the next copies overwrite them
        if (e_end - a > kAggSlots - 1) {  // further passes of a long row: ids in line, same slots
            const int32_t* src = p.src + (int64_t)b * p.src_stride;
            const int32_t* row_map = HAS_MAP ? p.row_map + (int64_t)b * p.row_map_stride : nullptr;
            for (int e0 = a + kAggSlots - 1; e0 < e_end; e0 += kAggSlots - 1) {
                const int n = min(kAggSlots - 1, e_end - e0);
                int row2 = 0;
                float w2 = 1.0f;
                bool bad2 = false;
                if (lane < n) {
                    const int s = __ldg(src + e0 + lane);
                    row2 = (int)checked_row<HAS_MAP>(p, row_map, s);
                    bad2 = row2 < 0;
                    if (bad2) row2 = 0;
                    if (MODE == FGL_AGG_SYMNORM && !bad2) w2 = 1.0f / sqrtf((float)__ldg(p.src_deg + s));
                }
                const unsigned bad2_mask = __ballot_sync(0xffffffffu, bad2);
                request(row2, n);
                cp_async_wait_all();
                __syncwarp();
                add_up(acc, n, bad2_mask, w2);
                __syncwarp();
            }
        }
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(e_end - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)ddeg);
        if (lane_on) orow[lane] = (MODE == FGL_AGG_SUM) ? acc : V::scale(acc, scale);
    }
}

// Row gather: out[i,:] = x[ids[i],:] (single or sharded table).  A warp per row, UNR rows in flight per warp.
// Replaces the CPU index_select + host-to-device copy of load_subtensors (train_fastgl.py:161-184).
template <int VEC>
__global__ void __launch_bounds__(kAggThreads) gather_rows_kernel(const AggParams p, const int32_t* __restrict__ ids, int64_t n_ids) {
    using T = typename Vec<VEC>::T;
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (int64_t)blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;
    constexpr int UNR = 4;
    for (int64_t i0 = warp_global * UNR; i0 < n_ids; i0 += n_warps * UNR) {
        const T* src[UNR];
        bool ok[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t i = i0 + u < n_ids ? i0 + u : n_ids - 1;
            const int64_t r = (int64_t)__ldg(ids + i);
            ok[u] = r >= 0 && r < p.n_rows;
            if (!ok[u]) agg_bad_id(p);
            src[u] = reinterpret_cast<const T*>(x_row(p, ok[u] ? r : 0));
        }
        for (int c = lane; c < chunks; c += 32) {
            T v[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) v[u] = __ldg(src[u] + c);
#pragma unroll
            for (int u = 0; u < UNR; ++u)
                if (i0 + u < n_ids) reinterpret_cast<T*>(p.out + (i0 + u) * p.ldo)[c] = ok[u] ? v[u] : Vec<VEC>::zero();
        }
    }
}

__device__ __forceinline__ void red_add(float4* addr, const float4& v) { atomicAdd(addr, v); }
__device__ __forceinline__ void red_add(float2* addr, const float2& v) { atomicAdd(addr, v); }
__device__ __forceinline__ void red_add(float* addr, const float& v) { atomicAdd(addr, v); }

// Backward: dx[src[e],:] += w_e * scale_d * dy[d,:]; vector reductions (red.global.add.v4.f32 on sm_100a)
template <int VEC, int MODE, int NACC>
__global__ void __launch_bounds__(kAggThreads) agg_bwd_kernel(const AggParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;

    const int n_dst = p.n_dst_dev ? min(max(__ldg(p.n_dst_dev), 0), p.n_dst) : p.n_dst;
    for (int d = warp_global; d < n_dst; d += n_warps) {
        const int a = __ldg(p.indptr + d), b = __ldg(p.indptr + d + 1);
        if (a >= b) continue;  // aggregate_acc_kernel.cu:498-500, :580-582
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(b - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)__ldg(p.dst_deg + d));
        const T* grow = reinterpret_cast<const T*>(p.x + (int64_t)d * p.ldx);

        for (int c0 = 0; c0 < chunks; c0 += 32 * NACC) {
            T g[NACC];
            int head[NACC];
#pragma unroll
            for (int k = 0; k < NACC; ++k) {
                const int c = c0 + k * 32 + lane;
                g[k] = (c < chunks) ? V::scale(__ldg(grow + c), scale) : V::zero();
                head[k] = (MODE == FGL_AGG_EDGE) ? min((c * VEC) / (p.dim / p.n_heads), p.n_heads - 1) : 0;
            }
            for (int e0 = a; e0 < b; e0 += 32) {
                const int cnt = min(32, b - e0);
                int my_s = 0;
                float my_w = 1.0f;
                if (lane < cnt) {
                    my_s = __ldg(p.src + e0 + lane);
                    if (MODE == FGL_AGG_SYMNORM && my_s >= 0 && my_s < p.n_src) my_w = 1.0f / sqrtf((float)__ldg(p.src_deg + my_s));
                }
                for (int j = 0; j < cnt; ++j) {
                    const int s = __shfl_sync(0xffffffffu, my_s, j);
                    const float w = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, j) : 1.0f;
                    if (s < 0 || s >= p.n_src) {  // warp-uniform
                        agg_bad_id(p);
                        continue;
                    }
                    T* xr = reinterpret_cast<T*>(p.out + (int64_t)s * p.ldo);
#pragma unroll
                    for (int k = 0; k < NACC; ++k) {
                        const int c = c0 + k * 32 + lane;
                        if (c < chunks) {
                            if (MODE == FGL_AGG_EDGE)
                                red_add(xr + c, V::scale(g[k], __ldg(p.edge_w + (int64_t)(e0 + j) * p.n_heads + head[k])));
                            else
                                red_add(xr + c, (MODE == FGL_AGG_SYMNORM) ? V::scale(g[k], w) : g[k]);
                        }
                    }
                }
            }
        }
    }
}

// Gradient of the edge weights: dw[e, h] = sum over head h's columns f of dy[d, f] * x[src[e], f] for every edge e of
// row d (the term the reference drops, GraphConv.py:227).  A warp per destination row; per neighbour the lanes
// multiply their vectors, reduce within runs of lanes that share a head, and the first lane of each run adds.
template <int VEC>
__global__ void __launch_bounds__(kAggThreads) agg_edge_wgrad_kernel(const AggParams p, float* __restrict__ dw) {
    using T = typename Vec<VEC>::T;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;
    const int unit = p.dim / p.n_heads;
    for (int d = warp_global; d < p.n_dst; d += n_warps) {
        const int a = __ldg(p.indptr + d), b = __ldg(p.indptr + d + 1);
        const T* grow = reinterpret_cast<const T*>(p.out + (int64_t)d * p.ldo);  // dy
        for (int c0 = 0; c0 < chunks; c0 += 32) {
            const int c = c0 + lane;
            const bool live = c < chunks;
            const int head = live ? (c * VEC) / unit : -1;
            T g = Vec<VEC>::zero();
            if (live) g = __ldg(grow + c);
            const int prev_head = __shfl_up_sync(0xffffffffu, head, 1);
            const bool leader = live && (lane == 0 || prev_head != head);
            for (int e = a; e < b; ++e) {
                const int s = __ldg(p.src + e);
                if (s < 0 || s >= p.n_src) {  // warp-uniform: dw[e, :] stays zero
                    agg_bad_id(p);
                    continue;
                }
                float v = 0.0f;
                if (live) {
                    const T xv = __ldg(reinterpret_cast<const T*>(p.x + (int64_t)s * p.ldx) + c);
                    const float* gp = reinterpret_cast<const float*>(&g);
                    const float* xp = reinterpret_cast<const float*>(&xv);
#pragma unroll
                    for (int q = 0; q < VEC; ++q) v = fmaf(gp[q], xp[q], v);
                }
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {  // segmented suffix sum over lanes of the same head
                    const float ov = __shfl_down_sync(0xffffffffu, v, off);
                    const int oh = __shfl_down_sync(0xffffffffu, head, off);
                    if (lane + off < 32 && oh == head) v += ov;
                }
                if (leader) atomicAdd(dw + (int64_t)e * p.n_heads + head, v);
            }
        }
    }
}

static bool aligned_for(int v, const void* a, int64_t lda) { return lda % v == 0 && ((uintptr_t)a % (4 * v)) == 0; }

static int pick_vec(int dim, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c = nullptr, int64_t ldc = 4) {
    auto ok = [&](int v) {
        return dim % v == 0 && aligned_for(v, a, lda) && aligned_for(v, b, ldb) && (!c || aligned_for(v, c, ldc));
    };
    if (ok(4)) return 4;
    if (ok(2)) return 2;
    return 1;
}

static int agg_grid_x(int n_rows, int n_batches) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = ((int64_t)n_rows + kAggWarps - 1) / kAggWarps;
    const int64_t cap = std::max<int64_t>(1, ((int64_t)sms * 8 + n_batches - 1) / n_batches);
    return (int)std::max<int64_t>(1, std::min<int64_t>(want, cap));
}

template <int VEC, int MODE, int NACC, int UNR>
static void launch_fwd(const AggParams& p, dim3 grid, cudaStream_t st) {
    if (p.row_map)
        agg_fwd_kernel<VEC, MODE, true, NACC, UNR><<<grid, kAggThreads, 0, st>>>(p);
    else
        agg_fwd_kernel<VEC, MODE, false, NACC, UNR><<<grid, kAggThreads, 0, st>>>(p);
}

// Whether agg_fwd_staged_kernel applies: 128-bit rows of at most 32 vectors in a single dense table.
static bool staged_applies(const AggParams& p, int vec) {
    return vec == 4 && p.shards == nullptr && p.dim / 4 <= 32 && p.ldx * 4 <= 0xffffffffLL;
}

template <int MODE>
static void launch_fwd_staged(const AggParams& p, cudaStream_t st) {
    static int sms = 0, smem_optin = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // as many warps per SM as their row slots fit beside the kernel's static shared memory
    const int64_t per_warp = (int64_t)kAggSlots * (p.dim / 4) * 16;
    const int warps = (int)std::max<int64_t>(1, std::min<int64_t>(kAggStagedMaxWarps, ((int64_t)smem_optin - 8 * 1024) / per_warp));
    const size_t dyn = (size_t)warps * per_warp;
    const int64_t rows = p.out_row_off ? 0x7fffffff : p.n_dst;  // window launches fill the GPU
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(sms, (rows + warps - 1) / warps));
    if (p.row_map) {
        cudaFuncSetAttribute(agg_fwd_staged_kernel<MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
        agg_fwd_staged_kernel<MODE, true><<<grid, warps * 32, dyn, st>>>(p);
    } else {
        cudaFuncSetAttribute(agg_fwd_staged_kernel<MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn);
        agg_fwd_staged_kernel<MODE, false><<<grid, warps * 32, dyn, st>>>(p);
    }
}

template <int VEC, int MODE>
static void launch_fwd_nacc(const AggParams& p, dim3 grid, cudaStream_t st) {
    const int chunks = p.dim / VEC;
    if (MODE != FGL_AGG_EDGE && staged_applies(p, VEC)) {
        launch_fwd_staged<MODE == FGL_AGG_EDGE ? FGL_AGG_SUM : MODE>(p, st);
    } else if (chunks <= 32)
        launch_fwd<VEC, MODE, 1, FGL_AGG_UNR1>(p, grid, st);
    else if (chunks <= 64)
        launch_fwd<VEC, MODE, 2, 4>(p, grid, st);
    else
        launch_fwd<VEC, MODE, 4, 2>(p, grid, st);
}

template <int VEC>
static void launch_fwd_mode(int mode, const AggParams& p, dim3 grid, cudaStream_t st) {
    if (mode == FGL_AGG_SUM) launch_fwd_nacc<VEC, FGL_AGG_SUM>(p, grid, st);
    if (mode == FGL_AGG_MEAN) launch_fwd_nacc<VEC, FGL_AGG_MEAN>(p, grid, st);
    if (mode == FGL_AGG_SYMNORM) launch_fwd_nacc<VEC, FGL_AGG_SYMNORM>(p, grid, st);
    if (mode == FGL_AGG_EDGE) launch_fwd_nacc<VEC, FGL_AGG_EDGE>(p, grid, st);
}

static int launch_fwd_any(int mode, const AggParams& p, dim3 grid, int vec, cudaStream_t st) {
    switch (vec) {
        case 4: launch_fwd_mode<4>(mode, p, grid, st); break;
        case 2: launch_fwd_mode<2>(mode, p, grid, st); break;
        default: launch_fwd_mode<1>(mode, p, grid, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}


template <int VEC, int MODE>
static void launch_bwd_nacc(const AggParams& p, int grid, cudaStream_t st) {
    const int chunks = p.dim / VEC;
    if (chunks <= 32)
        agg_bwd_kernel<VEC, MODE, 1><<<grid, kAggThreads, 0, st>>>(p);
    else if (chunks <= 64)
        agg_bwd_kernel<VEC, MODE, 2><<<grid, kAggThreads, 0, st>>>(p);
    else
        agg_bwd_kernel<VEC, MODE, 4><<<grid, kAggThreads, 0, st>>>(p);
}

template <int VEC>
static void launch_bwd_mode(int mode, const AggParams& p, int grid, cudaStream_t st) {
    if (mode == FGL_AGG_SUM) launch_bwd_nacc<VEC, FGL_AGG_SUM>(p, grid, st);
    if (mode == FGL_AGG_MEAN) launch_bwd_nacc<VEC, FGL_AGG_MEAN>(p, grid, st);
    if (mode == FGL_AGG_SYMNORM) launch_bwd_nacc<VEC, FGL_AGG_SYMNORM>(p, grid, st);
    if (mode == FGL_AGG_EDGE) launch_bwd_nacc<VEC, FGL_AGG_EDGE>(p, grid, st);
}

// dx[r, :] = dy_self[r, :] for r < n_dst (the real count when n_dst_dev is given), 0 for n_dst <= r < n_src: the
// start value of the scatter of a layer with a self term.  Scalar columns: the two matrices may have different
// alignment.
__global__ void __launch_bounds__(256)
init_self_rows_kernel(float* __restrict__ dx, int64_t ldx, const float* __restrict__ dy_self, int64_t ld_self, int dim,
                      int n_dst, int n_src, const int32_t* __restrict__ n_dst_dev) {
    if (n_dst_dev) n_dst = min(max(__ldg(n_dst_dev), 0), n_dst);  // padded launch: rows at or beyond the real count are zero
    const int groups = (dim + 3) / 4;
    const int64_t total = (int64_t)n_src * groups;
    const bool vec = dim % 4 == 0 && ldx % 4 == 0 && ld_self % 4 == 0 && (((uintptr_t)dx | (uintptr_t)dy_self) & 15) == 0;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = g / groups;
        const int c = (int)(g - r * groups) * 4;
        if (vec) {
            const float4 v = r < n_dst ? *reinterpret_cast<const float4*>(dy_self + r * ld_self + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(dx + r * ldx + c) = v;
        } else {
            for (int j = c; j < c + 4 && j < dim; ++j) dx[r * ldx + j] = r < n_dst ? dy_self[r * ld_self + j] : 0.f;
        }
    }
}

}  // namespace fgl

using namespace fgl;

static int32_t* status_of(fgl_ws* ws) { return ws ? ws->status : nullptr; }

extern "C" {

int fgl_agg_fwd(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                const int32_t* dst_deg, const int32_t* row_map, int64_t n_map, const float* x, int64_t n_rows, int64_t ldx,
                int32_t dim, int32_t n_dst, int32_t flags, float* out, int64_t ldo, const int32_t* n_dst_dev, void* stream) {
    return fgl_agg_fwd_sharded(ws, mode, indptr, src, src_deg, dst_deg, row_map, n_map, x, nullptr, 0, n_rows, ldx, dim, n_dst,
                               flags, out, ldo, n_dst_dev, stream);
}

int fgl_agg_fwd_sharded(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                        const int32_t* dst_deg, const int32_t* row_map, int64_t n_map, const float* x,
                        const float* const* shards, int64_t rows_per_shard, int64_t n_rows, int64_t ldx, int32_t dim,
                        int32_t n_dst, int32_t flags, float* out, int64_t ldo, const int32_t* n_dst_dev, void* stream) {
    if (mode < FGL_AGG_SUM || mode > FGL_AGG_SYMNORM || n_dst < 0 || dim < 1 || ldx < dim || ldo < dim || n_rows < 0 ||
        (row_map && n_map < 0))
        return FGL_ERR_INVALID;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || (!x && !shards) || (shards && rows_per_shard < 1) || !out || n_rows < 1) return FGL_ERR_INVALID;
    if (mode == FGL_AGG_SYMNORM && (!src_deg || !dst_deg)) return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.src_deg = src_deg;
    p.dst_deg = dst_deg;
    p.row_map = row_map;
    p.x = x;
    p.out = out;
    p.ldx = ldx;
    p.ldo = ldo;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_dst_dev = n_dst_dev;
    p.shards = shards;
    p.rows_per_shard = rows_per_shard;
    p.n_rows = n_rows;
    p.n_map = n_map;
    p.status = status_of(ws);
    p.passthrough = (flags & FGL_AGG_ZERO_DEG_PASSTHROUGH) ? 1 : 0;
    return launch_fwd_any(mode, p, dim3(agg_grid_x(n_dst, 1), 1), pick_vec(dim, shards ? nullptr : x, ldx, out, ldo),
                          (cudaStream_t)stream);
}

int fgl_agg_fwd_window(fgl_ws* ws, int32_t mode, int32_t n_batches, const int32_t* indptr, int64_t indptr_stride,
                       const int32_t* src, int64_t src_stride, const int32_t* row_map, int64_t row_map_stride,
                       const int64_t* out_row_off, int64_t total_rows, const float* x, const float* const* shards,
                       int64_t rows_per_shard, int64_t n_rows, int64_t ldx, int32_t dim, int32_t flags, float* out,
                       int64_t ldo, float* self_out, int64_t ld_self, void* stream) {
    if ((mode != FGL_AGG_SUM && mode != FGL_AGG_MEAN) || n_batches < 0 || n_batches > kAggMaxWindow || total_rows < 0 ||
        total_rows > 0x7fffffffLL ||
        dim < 1 || ldx < dim || ldo < dim || (self_out && ld_self < dim) || n_rows < 0)
        return FGL_ERR_INVALID;
    if (n_batches == 0 || total_rows == 0) return FGL_OK;
    if (!indptr || !src || !out_row_off || (!x && !shards) || (shards && rows_per_shard < 1) || !out || n_rows < 1)
        return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.row_map = row_map;
    p.x = x;
    p.shards = shards;
    p.rows_per_shard = rows_per_shard;
    p.n_rows = n_rows;
    p.n_map = row_map_stride;  // a batch's local ids index its own row of the map
    p.status = status_of(ws);
    p.out = out;
    p.self_out = self_out;
    p.ldx = ldx;
    p.ldo = ldo;
    p.ld_self = ld_self;
    p.dim = dim;
    p.passthrough = (flags & FGL_AGG_ZERO_DEG_PASSTHROUGH) ? 1 : 0;
    p.indptr_stride = indptr_stride;
    p.src_stride = src_stride;
    p.row_map_stride = row_map_stride;
    p.n_batches = n_batches;
    p.out_row_off = out_row_off;
    const int vec = pick_vec(dim, shards ? nullptr : x, ldx, out, ldo, self_out, self_out ? ld_self : 4);
    timing_begin(ws, (cudaStream_t)stream);
    const int rc = launch_fwd_any(mode, p, dim3(agg_grid_x((int)total_rows, 1), 1), vec, (cudaStream_t)stream);
    timing_end(ws, (cudaStream_t)stream);
    return rc;
}

int fgl_agg_edge_fwd(fgl_ws* ws, const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads,
                     const float* x, int32_t n_src, int64_t ldx, int32_t dim, int32_t n_dst, int32_t flags, float* out,
                     int64_t ldo, void* stream) {
    if (n_dst < 0 || n_src < 0 || dim < 1 || n_heads < 1 || dim % n_heads != 0 || ldx < dim || ldo < dim) return FGL_ERR_INVALID;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !x || !out || !edge_w || n_src < 1) return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.x = x;
    p.out = out;
    p.ldx = ldx;
    p.ldo = ldo;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_rows = n_src;
    p.status = status_of(ws);
    p.edge_w = edge_w;
    p.n_heads = n_heads;
    p.passthrough = (flags & FGL_AGG_ZERO_DEG_PASSTHROUGH) ? 1 : 0;
    int vec = pick_vec(dim, x, ldx, out, ldo);
    while (vec > 1 && (dim / n_heads) % vec != 0) vec /= 2;  // a vector never straddles two heads
    return launch_fwd_any(FGL_AGG_EDGE, p, dim3(agg_grid_x(n_dst, 1), 1), vec, (cudaStream_t)stream);
}

int fgl_agg_edge_bwd(fgl_ws* ws, const int32_t* indptr, const int32_t* src, const float* edge_w, int32_t n_heads,
                     const float* dy, int64_t ldy, int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx,
                     void* stream) {
    if (n_dst < 0 || n_src < 0 || dim < 1 || n_heads < 1 || dim % n_heads != 0 || ldy < dim || ldx < dim) return FGL_ERR_INVALID;
    if (n_src == 0) return FGL_OK;
    if (!dx) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemset2DAsync(dx, sizeof(float) * (size_t)ldx, 0, sizeof(float) * (size_t)dim, (size_t)n_src, st) != cudaSuccess)
        return FGL_ERR_CUDA;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !dy || !edge_w) return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.x = dy;
    p.out = dx;
    p.ldx = ldy;
    p.ldo = ldx;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_src = n_src;
    p.status = status_of(ws);
    p.edge_w = edge_w;
    p.n_heads = n_heads;
    int vec = pick_vec(dim, dy, ldy, dx, ldx);
    while (vec > 1 && (dim / n_heads) % vec != 0) vec /= 2;
    const int grid = agg_grid_x(n_dst, 1);
    switch (vec) {
        case 4: launch_bwd_mode<4>(FGL_AGG_EDGE, p, grid, st); break;
        case 2: launch_bwd_mode<2>(FGL_AGG_EDGE, p, grid, st); break;
        default: launch_bwd_mode<1>(FGL_AGG_EDGE, p, grid, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_agg_edge_wgrad(fgl_ws* ws, const int32_t* indptr, const int32_t* src, int32_t n_heads, const float* x, int32_t n_src,
                       int64_t ldx, const float* dy, int64_t ldy, int32_t dim, int32_t n_dst, int64_t n_edges, float* dw,
                       void* stream) {
    if (n_dst < 0 || n_src < 0 || n_edges < 0 || dim < 1 || n_heads < 1 || dim % n_heads != 0 || ldx < dim || ldy < dim)
        return FGL_ERR_INVALID;
    if (n_edges == 0) return FGL_OK;
    if (!dw) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(dw, 0, sizeof(float) * (size_t)n_edges * (size_t)n_heads, st) != cudaSuccess) return FGL_ERR_CUDA;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !src || !x || !dy) return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.x = x;
    p.out = const_cast<float*>(dy);
    p.ldx = ldx;
    p.ldo = ldy;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_src = n_src;
    p.status = status_of(ws);
    p.n_heads = n_heads;
    int vec = pick_vec(dim, x, ldx, dy, ldy);
    while (vec > 1 && (dim / n_heads) % vec != 0) vec /= 2;
    const int grid = agg_grid_x(n_dst, 1);
    switch (vec) {
        case 4: agg_edge_wgrad_kernel<4><<<grid, kAggThreads, 0, st>>>(p, dw); break;
        case 2: agg_edge_wgrad_kernel<2><<<grid, kAggThreads, 0, st>>>(p, dw); break;
        default: agg_edge_wgrad_kernel<1><<<grid, kAggThreads, 0, st>>>(p, dw); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_gather_rows(fgl_ws* ws, const float* table, const float* const* shards, int64_t rows_per_shard, int64_t n_rows,
                    int64_t ld, int32_t dim, const int32_t* ids, int64_t n_ids, float* out, int64_t ldo, void* stream) {
    if ((!table && !shards) || (shards && rows_per_shard < 1) || dim < 1 || ld < dim || ldo < dim || n_ids < 0 || n_rows < 0)
        return FGL_ERR_INVALID;
    if (n_ids == 0) return FGL_OK;
    if (!ids || !out || n_rows < 1) return FGL_ERR_INVALID;
    AggParams p{};
    p.x = table;
    p.shards = shards;
    p.rows_per_shard = rows_per_shard;
    p.n_rows = n_rows;
    p.status = status_of(ws);
    p.out = out;
    p.ldx = ld;
    p.ldo = ldo;
    p.dim = dim;
    // the shard bases cannot be inspected on the host: rely on the leading dimension and cudaMalloc alignment
    const int vec = pick_vec(dim, shards ? (const void*)nullptr : (const void*)table, ld, out, ldo);
    const int grid = agg_grid_x((int)std::min<int64_t>((n_ids + 3) / 4, 0x7fffffff), 1);
    cudaStream_t st = (cudaStream_t)stream;
    switch (vec) {
        case 4: gather_rows_kernel<4><<<grid, kAggThreads, 0, st>>>(p, ids, n_ids); break;
        case 2: gather_rows_kernel<2><<<grid, kAggThreads, 0, st>>>(p, ids, n_ids); break;
        default: gather_rows_kernel<1><<<grid, kAggThreads, 0, st>>>(p, ids, n_ids); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

static int agg_bwd_impl(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                        const int32_t* dst_deg, const float* dy, int64_t ldy, const float* dy_self, int64_t ld_self,
                        int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx, const int32_t* n_dst_dev,
                        void* stream) {
    if (mode < FGL_AGG_SUM || mode > FGL_AGG_SYMNORM || n_dst < 0 || n_src < 0 || dim < 1 || ldy < dim || ldx < dim)
        return FGL_ERR_INVALID;
    if (dy_self && (ld_self < dim || n_dst > n_src)) return FGL_ERR_INVALID;
    if (n_src == 0) return FGL_OK;
    if (!dx) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (dy_self && n_dst > 0) {
        const int64_t items = (int64_t)n_src * ((dim + 3) / 4);
        const int grid = (int)std::min<int64_t>((items + 255) / 256, 148 * 16);
        init_self_rows_kernel<<<grid, 256, 0, st>>>(dx, ldx, dy_self, ld_self, dim, n_dst, n_src, n_dst_dev);
    } else if (cudaMemset2DAsync(dx, sizeof(float) * (size_t)ldx, 0, sizeof(float) * (size_t)dim, (size_t)n_src, st) !=
               cudaSuccess) {
        return FGL_ERR_CUDA;
    }
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !dy) return FGL_ERR_INVALID;
    if (mode == FGL_AGG_SYMNORM && (!src_deg || !dst_deg)) return FGL_ERR_INVALID;
    AggParams p{};
    p.indptr = indptr;
    p.src = src;
    p.src_deg = src_deg;
    p.dst_deg = dst_deg;
    p.x = dy;
    p.out = dx;
    p.ldx = ldy;
    p.ldo = ldx;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_src = n_src;
    p.n_dst_dev = n_dst_dev;
    p.status = status_of(ws);
    const int grid = agg_grid_x(n_dst, 1);
    switch (pick_vec(dim, dy, ldy, dx, ldx)) {
        case 4: launch_bwd_mode<4>(mode, p, grid, st); break;
        case 2: launch_bwd_mode<2>(mode, p, grid, st); break;
        default: launch_bwd_mode<1>(mode, p, grid, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_agg_bwd(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                const int32_t* dst_deg, const float* dy, int64_t ldy, int32_t dim, int32_t n_dst, int32_t n_src, float* dx,
                int64_t ldx, const int32_t* n_dst_dev, void* stream) {
    return agg_bwd_impl(ws, mode, indptr, src, src_deg, dst_deg, dy, ldy, nullptr, 0, dim, n_dst, n_src, dx, ldx, n_dst_dev,
                        stream);
}

int fgl_agg_bwd_self(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg,
                     const int32_t* dst_deg, const float* dy, int64_t ldy, const float* dy_self, int64_t ld_self,
                     int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx, const int32_t* n_dst_dev,
                     void* stream) {
    if (!dy_self && n_dst > 0) return FGL_ERR_INVALID;
    return agg_bwd_impl(ws, mode, indptr, src, src_deg, dst_deg, dy, ldy, dy_self, ld_self, dim, n_dst, n_src, dx, ldx,
                        n_dst_dev, stream);
}

}  // extern "C"

// ================================================================================================================
// Backward as a gather over the transposed block CSR (deterministic, no atomics on the gradient, no zero-fill pass)
// ================================================================================================================
// The scatter above adds every edge's contribution with a vector reduction: its speed is the L2's reduction rate
// and the order of the additions -- hence the last bits of the result -- changes from run to run.  Here the block is
// transposed once (per-source lists of destination rows: histogram, scan, fill) and every gradient row dx[s] is
// then produced by exactly one warp (sources with at most 32 in-block out-edges) or one CTA (hubs), which adds the
// rows dy[d] of its list in ascending order of d.  The order is a property of the block, not of the schedule, so two
// runs give the same bits; dx[s] is written once, with the self term folded in, so it needs no initialisation.
// Replaces K9 / K11 (aggregate_acc_kernel.cu:468-517, :555-596) like agg_bwd_kernel does.
namespace fgl {

struct GatherParams {
    const int32_t* indptr;    // block CSR over destinations (mean weights)
    const int32_t* t_indptr;  // transposed: per source, [n_src + 1]
    const int32_t* t_dst;     // destination rows, grouped by source (order within a group: arbitrary)
    const int32_t* hubs;      // [0] number of sources with more than 32 entries, then their ids
    const int32_t* src_deg;
    const int32_t* dst_deg;
    const float* dy;
    const float* dy_self;
    float* dx;
    int64_t ldy, ld_self, ldx;
    int32_t dim, n_dst, n_src;
    const int32_t* n_dst_dev;
    int32_t hub_ctas;  // agg_bwd_gather_kernel: the first hub_ctas CTAs take the hubs of 33 .. kHubSplitMin entries
};

constexpr int kHubThreshold = 32;

template <int MODE>
__device__ __forceinline__ float gather_weight(const GatherParams& p, int d) {
    if (MODE == FGL_AGG_MEAN) return 1.0f / (float)(__ldg(p.indptr + d + 1) - __ldg(p.indptr + d));
    if (MODE == FGL_AGG_SYMNORM) return 1.0f / sqrtf((float)__ldg(p.dst_deg + d));
    return 1.0f;
}

// Histogram of the sources (pass 0) and placement of every edge's destination row behind its source's cursor (pass 1).
__global__ void __launch_bounds__(256) transpose_edges_kernel(const int32_t* __restrict__ indptr, const int32_t* __restrict__ src,
                                                              int n_dst, int n_src, const int32_t* __restrict__ n_dst_dev,
                                                              int32_t* __restrict__ cnt, const int32_t* __restrict__ t_indptr,
                                                              int32_t* __restrict__ cursor, int32_t* __restrict__ t_dst,
                                                              int64_t t_cap, int32_t* __restrict__ status, int pass) {
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = gridDim.x * 8;
    if (n_dst_dev) n_dst = min(max(__ldg(n_dst_dev), 0), n_dst);
    for (int d = warp_global; d < n_dst; d += n_warps) {
        const int a = __ldg(indptr + d), b = __ldg(indptr + d + 1);
        for (int e = a + lane; e < b; e += 32) {
            const int s = __ldg(src + e);
            if (s < 0 || s >= n_src) {
                if (status) set_status(status, FGL_ERR_BOUNDS);
                continue;
            }
            if (pass == 0) {
                atomicAdd(cnt + s, 1);
            } else {
                const int64_t at = (int64_t)__ldg(t_indptr + s) + atomicAdd(cursor + s, 1);
                if (at < t_cap) t_dst[at] = d;
                else if (status) set_status(status, FGL_ERR_CAPACITY);
            }
        }
    }
}

// The list of hubs: sources with more than kHubThreshold entries.  hubs[0] was zeroed by the host.
__global__ void __launch_bounds__(256) list_hubs_kernel(const int32_t* __restrict__ t_indptr, int n_src, int32_t* __restrict__ hubs) {
    for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < n_src; s += gridDim.x * blockDim.x)
        if (__ldg(t_indptr + s + 1) - __ldg(t_indptr + s) > kHubThreshold) hubs[1 + atomicAdd(hubs, 1)] = s;
}

// acc += sum over j < deg of w_j * dy[d_j, columns c0 ..], lane j holding (d_j, w_j); U rows' loads in flight.
template <int VEC, int NACC, int U>
__device__ __forceinline__ void gather_add_rows(const GatherParams& p, int d, float w, int deg, int c0, int chunks, int lane,
                                                typename Vec<VEC>::T (&acc)[NACC]) {
    using V = Vec<VEC>;
    using T = typename V::T;
    for (int j0 = 0; j0 < deg; j0 += U) {
        T v[U][NACC];
        float wj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = min(j0 + u, deg - 1);
            const int dj = __shfl_sync(0xffffffffu, d, j);
            wj[u] = __shfl_sync(0xffffffffu, w, j);
            const T* row = reinterpret_cast<const T*>(p.dy + (int64_t)dj * p.ldy);
#pragma unroll
            for (int k = 0; k < NACC; ++k) {
                const int c = c0 + k * 32 + lane;
                v[u][k] = c < chunks ? __ldg(row + c) : V::zero();
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (j0 + u < deg) {
#pragma unroll
                for (int k = 0; k < NACC; ++k) V::fma(acc[k], wj[u], v[u][k]);
            }
    }
}

__device__ __forceinline__ int warp_sort_ascending(int v, int lane) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const int other = __shfl_xor_sync(0xffffffffu, v, j);
            const bool up = (lane & k) == 0, lower = (lane & j) == 0;
            v = (lower == up) ? min(v, other) : max(v, other);
        }
    }
    return v;
}

// A warp per source row with at most 32 entries: sort the destination rows, add them in that order.  Most sources of a
// sampled block have one or two entries: those skip the sorting network (one entry) and request only as many rows as
// they have (the unrolled batch of eight would otherwise load a single row eight times).  Software-pipelining the id
// chain over the warp's sources, as the forward kernel does, was measured and bought nothing here: with 64 warps per
// SM the chain is hidden already, and the launch is bound by the rows it reads and the full output row it writes per
// source.
template <int VEC, int MODE, int NACC>
__device__ __forceinline__ void gather_small_sources(const GatherParams& p, int block, int n_blocks) {
    using V = Vec<VEC>;
    using T = typename V::T;
    constexpr int UNR = NACC == 1 ? 8 : (NACC == 2 ? 4 : 2);
    const int lane = threadIdx.x & 31;
    const int warp_global = block * 8 + (threadIdx.x >> 5), n_warps = n_blocks * 8;
    const int chunks = p.dim / VEC;
    const int n_dst = p.n_dst_dev ? min(max(__ldg(p.n_dst_dev), 0), p.n_dst) : p.n_dst;
    for (int s = warp_global; s < p.n_src; s += n_warps) {
        const int a = __ldg(p.t_indptr + s), deg = __ldg(p.t_indptr + s + 1) - a;
        if (deg > kHubThreshold) continue;  // a hub CTA owns this row
        int d = lane < deg ? __ldg(p.t_dst + a + lane) : 0x7fffffff;
        if (deg > 1) d = warp_sort_ascending(d, lane);
        const float w = lane < deg ? gather_weight<MODE>(p, d) : 0.0f;
        const float ws = (MODE == FGL_AGG_SYMNORM && deg > 0) ? 1.0f / sqrtf((float)__ldg(p.src_deg + s)) : 1.0f;
        const bool self = p.dy_self != nullptr && s < n_dst;
        const T* self_row = reinterpret_cast<const T*>(p.dy_self + (self ? (int64_t)s * p.ld_self : 0));
        T* out = reinterpret_cast<T*>(p.dx + (int64_t)s * p.ldx);
        for (int c0 = 0; c0 < chunks; c0 += 32 * NACC) {
            T acc[NACC];
#pragma unroll
            for (int k = 0; k < NACC; ++k) acc[k] = V::zero();
            if (deg <= 1)
                gather_add_rows<VEC, NACC, 1>(p, d, w, deg, c0, chunks, lane, acc);
            else if (deg <= 2 || UNR <= 2)
                gather_add_rows<VEC, NACC, 2>(p, d, w, deg, c0, chunks, lane, acc);
            else if (deg <= 4 || UNR <= 4)
                gather_add_rows<VEC, NACC, 4>(p, d, w, deg, c0, chunks, lane, acc);
            else
                gather_add_rows<VEC, NACC, 8>(p, d, w, deg, c0, chunks, lane, acc);
#pragma unroll
            for (int k = 0; k < NACC; ++k) {
                const int c = c0 + k * 32 + lane;
                if (c < chunks) {
                    T r = (MODE == FGL_AGG_SYMNORM) ? V::scale(acc[k], ws) : acc[k];
                    if (self) V::fma(r, 1.0f, __ldg(self_row + c));
                    out[c] = r;
                }
            }
        }
    }
}

// Hubs of at most kHubSortMax entries.  The hub's destination rows are sorted in shared memory (bitonic network over the
// list padded to a power of two), warp k then adds the rows of the k-th eighth of the sorted list in order and the eight
// partial sums are folded in a fixed order: the result does not depend on the order in which the transposition's
// atomics filled the list.  16 KB of list per CTA, so several hubs are in flight per SM.
//   CLUSTER = false: a CTA per hub of up to kHubSplitMin entries.
//   CLUSTER = true:  a thread-block cluster of eight CTAs per hub of kHubSplitMin + 1 .. kHubSortMax entries.  CTA r
//                    keeps the entries whose destination lies in the r-th eighth of the destination range (a fixed
//                    partition, whatever the order of the list), sorts and adds them as above, and rank 0 folds the
//                    eight CTA sums in rank order, reading them through distributed shared memory.  A hub of 4000
//                    entries is then 8 x 8 warps deep instead of 8.
constexpr int kHubSortMax = 4096;
constexpr int kHubSplitMin = 512;
constexpr int kHubCluster = 8;

template <int VEC, int MODE, int NACC, bool CLUSTER>
__device__ __forceinline__ void gather_hubs_sorted(const GatherParams& p, int block, int n_blocks) {
    namespace cg = cooperative_groups;
    using V = Vec<VEC>;
    using T = typename V::T;
    extern __shared__ __align__(16) unsigned char hub_smem[];
    __shared__ int s_count;
    int* list = reinterpret_cast<int*>(hub_smem);                          // kHubSortMax entries
    T* part = reinterpret_cast<T*>(hub_smem + kHubSortMax * sizeof(int));  // [8][NACC][32]
    T* cta_sum = part + 8 * NACC * 32;                                     // [NACC][32], CLUSTER only
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = p.dim / VEC;
    const int n_dst = p.n_dst_dev ? min(max(__ldg(p.n_dst_dev), 0), p.n_dst) : p.n_dst;
    const int n_hubs = min(__ldg(p.hubs), p.n_src);
    const int rank = CLUSTER ? (int)cg::this_cluster().block_rank() : 0;
    const int unit = CLUSTER ? block / kHubCluster : block;
    const int n_units = CLUSTER ? n_blocks / kHubCluster : n_blocks;
    const int seg = (n_dst + kHubCluster - 1) / kHubCluster;  // destination rows per cluster rank
    constexpr int UNR = NACC == 1 ? 8 : (NACC == 2 ? 4 : 2);
    // This unit (CTA or cluster) looks after the hubs h = unit (mod n_units).  Which of them are of its size class is
    // found 256 at a time, a thread per hub, and compacted in index order -- every CTA of a cluster arrives at the same
    // list -- instead of one dependent pair of loads per hub in turn; longer lists are counted by agg_bwd_hub_kernel.
    __shared__ int s_sel[256];
    __shared__ int s_wcnt[8];
    for (int base = 0; base < n_hubs; base += 256 * n_units) {
        const int h_t = base + (int)threadIdx.x * n_units + unit;
        bool ok = false;
        if (h_t < n_hubs) {
            const int s_t = __ldg(p.hubs + 1 + h_t);
            const int deg_t = __ldg(p.t_indptr + s_t + 1) - __ldg(p.t_indptr + s_t);
            ok = CLUSTER ? (deg_t > kHubSplitMin && deg_t <= kHubSortMax) : (deg_t <= kHubSplitMin);
        }
        const unsigned bal = __ballot_sync(0xffffffffu, ok);
        if (lane == 0) s_wcnt[warp] = __popc(bal);
        __syncthreads();
        int sel_before = 0, n_sel = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (q < warp) sel_before += s_wcnt[q];
            n_sel += s_wcnt[q];
        }
        if (ok) s_sel[sel_before + __popc(bal & ((1u << lane) - 1u))] = h_t;
        __syncthreads();
        for (int q_sel = 0; q_sel < n_sel; ++q_sel) {
            const int s = __ldg(p.hubs + 1 + s_sel[q_sel]);
            const int a = __ldg(p.t_indptr + s), deg = __ldg(p.t_indptr + s + 1) - a;
            int m = deg;
            if (CLUSTER) {
                if (threadIdx.x == 0) s_count = 0;
                __syncthreads();
                for (int i = threadIdx.x; i < deg; i += 256) {
                    const int d = __ldg(p.t_dst + a + i);
                    if (d >= rank * seg && d < (rank + 1) * seg) list[atomicAdd(&s_count, 1)] = d;
                }
                __syncthreads();
                m = s_count;
            } else {
                for (int i = threadIdx.x; i < deg; i += 256) list[i] = __ldg(p.t_dst + a + i);
            }
            int n2 = 64;
            while (n2 < m) n2 <<= 1;
            for (int i = m + (int)threadIdx.x; i < n2; i += 256) list[i] = 0x7fffffff;
            __syncthreads();
            for (int k = 2; k <= n2; k <<= 1) {
                for (int j = k >> 1; j > 0; j >>= 1) {
                    for (int i = threadIdx.x; i < n2; i += 256) {
                        const int l = i ^ j;
                        if (l > i) {
                            const int x = list[i], y = list[l];
                            if ((x > y) == ((i & k) == 0)) {
                                list[i] = y;
                                list[l] = x;
                            }
                        }
                    }
                    __syncthreads();
                }
            }
            const float ws = (MODE == FGL_AGG_SYMNORM) ? 1.0f / sqrtf((float)__ldg(p.src_deg + s)) : 1.0f;
            const bool self = p.dy_self != nullptr && s < n_dst;
            const int per = (m + 7) / 8;
            const int lo = warp * per, hi = min(lo + per, m);
            for (int c0 = 0; c0 < chunks; c0 += 32 * NACC) {
                T acc[NACC];
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc[k] = V::zero();
                for (int j0 = lo; j0 < hi; j0 += UNR) {
                    T v[UNR][NACC];
                    float wj[UNR];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int dj = list[min(j0 + u, hi - 1)];
                        wj[u] = gather_weight<MODE>(p, dj);
                        const T* row = reinterpret_cast<const T*>(p.dy + (int64_t)dj * p.ldy);
#pragma unroll
                        for (int k = 0; k < NACC; ++k) {
                            const int c = c0 + k * 32 + lane;
                            v[u][k] = c < chunks ? __ldg(row + c) : V::zero();
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UNR; ++u)
                        if (j0 + u < hi) {
#pragma unroll
                            for (int k = 0; k < NACC; ++k) V::fma(acc[k], wj[u], v[u][k]);
                        }
                }
#pragma unroll
                for (int k = 0; k < NACC; ++k) part[(warp * NACC + k) * 32 + lane] = acc[k];
                __syncthreads();
                T total[NACC];
                if (warp == 0) {  // the CTA's sum: the eight warps' partial sums in warp order
#pragma unroll
                    for (int k = 0; k < NACC; ++k) {
                        total[k] = V::zero();
                        for (int q = 0; q < 8; ++q) V::fma(total[k], 1.0f, part[(q * NACC + k) * 32 + lane]);
                        if (CLUSTER) cta_sum[k * 32 + lane] = total[k];
                    }
                }
                if (CLUSTER) {
                    cg::this_cluster().sync();  // every CTA's sum is in its shared memory
                    if (rank == 0 && warp == 0) {
#pragma unroll
                        for (int k = 0; k < NACC; ++k) {
                            for (int q = 1; q < kHubCluster; ++q)
                                V::fma(total[k], 1.0f, cg::this_cluster().map_shared_rank(cta_sum, q)[k * 32 + lane]);
                        }
                    }
                }
                if (rank == 0 && warp == 0) {
                    T* out = reinterpret_cast<T*>(p.dx + (int64_t)s * p.ldx);
#pragma unroll
                    for (int k = 0; k < NACC; ++k) {
                        const int c = c0 + k * 32 + lane;
                        if (c < chunks) {
                            T r = (MODE == FGL_AGG_SYMNORM) ? V::scale(total[k], ws) : total[k];
                            if (self) V::fma(r, 1.0f, __ldg(reinterpret_cast<const T*>(p.dy_self + (int64_t)s * p.ld_self) + c));
                            out[c] = r;
                        }
                    }
                }
                if (CLUSTER) cg::this_cluster().sync();  // rank 0 has read the sums: they may be overwritten
                __syncthreads();
            }
        }
        __syncthreads();  // the selection is consumed: the next 256 candidates may overwrite it
    }
}

// One launch for the sources of up to kHubSplitMin entries: the first hub_ctas CTAs (they run longest, so they start
// first) each take hubs of 33 .. kHubSplitMin entries, the others take the small sources a warp at a time.
template <int VEC, int MODE, int NACC>
__global__ void __launch_bounds__(256) agg_bwd_gather_kernel(const GatherParams p) {
    if ((int)blockIdx.x < p.hub_ctas)
        gather_hubs_sorted<VEC, MODE, NACC, false>(p, (int)blockIdx.x, p.hub_ctas);
    else
        gather_small_sources<VEC, MODE, NACC>(p, (int)blockIdx.x - p.hub_ctas, (int)gridDim.x - p.hub_ctas);
}

// Clusters of kHubCluster CTAs for the hubs of kHubSplitMin + 1 .. kHubSortMax entries.
template <int VEC, int MODE, int NACC>
__global__ void __launch_bounds__(256) agg_bwd_hub_cluster_kernel(const GatherParams p) {
    gather_hubs_sorted<VEC, MODE, NACC, true>(p, (int)blockIdx.x, (int)gridDim.x);
}

// A CTA per hub with more than kHubSortMax entries.  The hub's destination rows are counted into a shared-memory array
// over a window of the destination range (16-bit counts, two per word), which orders them without sorting; warp k then
// adds the rows of the k-th eighth of the window in ascending order, and the eight partial sums are folded in a fixed
// order.  The 64 KB counting pass costs microseconds per hub whatever its size, hence only for the very long lists.
constexpr int kHubWindow = 32768;

template <int VEC, int MODE, int NACC>
__global__ void __launch_bounds__(256) agg_bwd_hub_kernel(const GatherParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    extern __shared__ __align__(16) unsigned char hub_smem[];
    uint32_t* cnt32 = reinterpret_cast<uint32_t*>(hub_smem);                            // kHubWindow / 2 words
    T* part = reinterpret_cast<T*>(hub_smem + kHubWindow * 2);                           // [8][NACC][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = p.dim / VEC;
    const int n_dst = p.n_dst_dev ? min(max(__ldg(p.n_dst_dev), 0), p.n_dst) : p.n_dst;
    const int n_hubs = min(__ldg(p.hubs), p.n_src);
    constexpr int UNR = 4;
    for (int h = blockIdx.x; h < n_hubs; h += gridDim.x) {
        const int s = __ldg(p.hubs + 1 + h);
        const int a = __ldg(p.t_indptr + s), b = __ldg(p.t_indptr + s + 1);
        if (b - a <= kHubSortMax) continue;  // sorted by a CTA or a cluster instead
        const float ws = (MODE == FGL_AGG_SYMNORM) ? 1.0f / sqrtf((float)__ldg(p.src_deg + s)) : 1.0f;
        const bool self = p.dy_self != nullptr && s < n_dst;
        for (int c0 = 0; c0 < chunks; c0 += 32 * NACC) {
            T total[NACC];  // warp 0 keeps the row's running sum over the windows
#pragma unroll
            for (int k = 0; k < NACC; ++k) total[k] = V::zero();
            for (int w0 = 0; w0 < n_dst; w0 += kHubWindow) {
                for (int i = threadIdx.x; i < kHubWindow / 2; i += 256) cnt32[i] = 0u;
                __syncthreads();
                for (int e = a + (int)threadIdx.x; e < b; e += 256) {
                    const int off = __ldg(p.t_dst + e) - w0;
                    if (off >= 0 && off < kHubWindow) atomicAdd(cnt32 + (off >> 1), 1u << (16 * (off & 1)));
                }
                __syncthreads();
                T acc[NACC];
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc[k] = V::zero();
                const int lo = warp * (kHubWindow / 8), hi = min(lo + kHubWindow / 8, n_dst - w0);
                for (int base = lo; base < hi; base += 32) {
                    const uint32_t word = cnt32[(base + lane) >> 1];
                    const int c = (int)((word >> (16 * ((base + lane) & 1))) & 0xffffu);
                    unsigned m = __ballot_sync(0xffffffffu, c > 0);
                    while (m) {  // warp-uniform
                        int dd[UNR];
                        float wd[UNR];
                        T v[UNR][NACC];
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                            dd[u] = -1;
                            wd[u] = 0.0f;
                            if (m) {
                                const int j = __ffs(m) - 1;
                                m &= m - 1;
                                dd[u] = w0 + base + j;
                                wd[u] = (float)__shfl_sync(0xffffffffu, c, j);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                            const int dj = dd[u] < 0 ? 0 : dd[u];
                            if (dd[u] >= 0) wd[u] *= gather_weight<MODE>(p, dj);
                            const T* row = reinterpret_cast<const T*>(p.dy + (int64_t)dj * p.ldy);
#pragma unroll
                            for (int k = 0; k < NACC; ++k) {
                                const int cc = c0 + k * 32 + lane;
                                v[u][k] = cc < chunks ? __ldg(row + cc) : V::zero();
                            }
                        }
#pragma unroll
                        for (int u = 0; u < UNR; ++u)
                            if (dd[u] >= 0) {
#pragma unroll
                                for (int k = 0; k < NACC; ++k) V::fma(acc[k], wd[u], v[u][k]);
                            }
                    }
                }
#pragma unroll
                for (int k = 0; k < NACC; ++k) part[(warp * NACC + k) * 32 + lane] = acc[k];
                __syncthreads();
                if (warp == 0) {
                    for (int q = 0; q < 8; ++q)
#pragma unroll
                        for (int k = 0; k < NACC; ++k) V::fma(total[k], 1.0f, part[(q * NACC + k) * 32 + lane]);
                }
                __syncthreads();
            }
            if (warp == 0) {
                T* out = reinterpret_cast<T*>(p.dx + (int64_t)s * p.ldx);
#pragma unroll
                for (int k = 0; k < NACC; ++k) {
                    const int c = c0 + k * 32 + lane;
                    if (c < chunks) {
                        T r = (MODE == FGL_AGG_SYMNORM) ? V::scale(total[k], ws) : total[k];
                        if (self) V::fma(r, 1.0f, __ldg(reinterpret_cast<const T*>(p.dy_self + (int64_t)s * p.ld_self) + c));
                        out[c] = r;
                    }
                }
            }
        }
    }
}

// Clusters of kHubCluster CTAs, one cluster per hub at a time; about two clusters' worth of CTAs per SM-octet.
static void launch_hub_clusters(void (*kernel)(const GatherParams), const GatherParams& p, int sms, size_t dyn, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    const int n_clusters = std::max(1, 2 * sms / kHubCluster);
    cfg.gridDim = dim3((unsigned)(n_clusters * kHubCluster));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = dyn;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kHubCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int VEC, int MODE>
static void launch_gather_nacc(const GatherParams& p, int sms, cudaStream_t st) {
    const int chunks = p.dim / VEC;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(((int64_t)p.n_src + 7) / 8, (int64_t)sms * 8));
    const int hub_grid = 2 * sms;
#define FGL_GATHER(NACC)                                                                                           \
    {                                                                                                              \
        const size_t dyn = (size_t)kHubWindow * 2 + sizeof(typename Vec<VEC>::T) * 8 * NACC * 32;                  \
        const size_t dyn_sorted = (size_t)kHubSortMax * sizeof(int) + sizeof(typename Vec<VEC>::T) * 9 * NACC * 32; \
        GatherParams q = p;                                                                                        \
        q.hub_ctas = 6 * sms;                                                                                      \
        agg_bwd_gather_kernel<VEC, MODE, NACC><<<grid + q.hub_ctas, 256, dyn_sorted, st>>>(q);                     \
        launch_hub_clusters(agg_bwd_hub_cluster_kernel<VEC, MODE, NACC>, p, sms, dyn_sorted, st);                  \
        cudaFuncSetAttribute(agg_bwd_hub_kernel<VEC, MODE, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn); \
        agg_bwd_hub_kernel<VEC, MODE, NACC><<<hub_grid, 256, dyn, st>>>(p);                                        \
    }
    if (chunks <= 32) FGL_GATHER(1)
    else if (chunks <= 64) FGL_GATHER(2)
    else FGL_GATHER(4)
#undef FGL_GATHER
}

template <int VEC>
static void launch_gather_mode(int mode, const GatherParams& p, int sms, cudaStream_t st) {
    if (mode == FGL_AGG_SUM) launch_gather_nacc<VEC, FGL_AGG_SUM>(p, sms, st);
    if (mode == FGL_AGG_MEAN) launch_gather_nacc<VEC, FGL_AGG_MEAN>(p, sms, st);
    if (mode == FGL_AGG_SYMNORM) launch_gather_nacc<VEC, FGL_AGG_SYMNORM>(p, sms, st);
}

}  // namespace fgl

extern "C" {

int fgl_block_transpose(fgl_ws* ws, const int32_t* indptr, const int32_t* src, int32_t n_dst, int32_t n_src, int32_t* t_indptr,
                        int32_t* t_dst, int64_t t_cap, int32_t* hubs, int32_t* work, const int32_t* n_dst_dev, void* stream) {
    if (!ws || n_dst < 0 || n_src < 0 || t_cap < 0) return FGL_ERR_INVALID;
    if (!t_indptr || !hubs || (n_src > 0 && !work) || (t_cap > 0 && !t_dst) || (n_dst > 0 && (!indptr || !src))) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    int sms = ws->sm_count > 0 ? ws->sm_count : 148;
    if (cudaMemsetAsync(hubs, 0, sizeof(int32_t), st) != cudaSuccess) return FGL_ERR_CUDA;
    if (n_src == 0) return cudaMemsetAsync(t_indptr, 0, sizeof(int32_t), st) == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
    if (cudaMemsetAsync(work, 0, sizeof(int32_t) * 2 * (size_t)n_src, st) != cudaSuccess) return FGL_ERR_CUDA;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(((int64_t)n_dst + 7) / 8, (int64_t)sms * 8));
    {
        DeviceGuard guard(ws->device);
        if (n_dst > 0)
            transpose_edges_kernel<<<grid, 256, 0, st>>>(indptr, src, n_dst, n_src, n_dst_dev, work, nullptr, nullptr, nullptr, 0,
                                                         ws->status, 0);
    }
    int rc = fgl_exclusive_sum(ws, work, n_src, t_indptr, stream);
    if (rc != FGL_OK) return rc;
    DeviceGuard guard(ws->device);
    if (n_dst > 0)
        transpose_edges_kernel<<<grid, 256, 0, st>>>(indptr, src, n_dst, n_src, n_dst_dev, nullptr, t_indptr, work + n_src, t_dst,
                                                     t_cap, ws->status, 1);
    list_hubs_kernel<<<std::max(1, std::min((n_src + 255) / 256, sms * 4)), 256, 0, st>>>(t_indptr, n_src, hubs);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_agg_bwd_gather(fgl_ws* ws, int32_t mode, const int32_t* indptr, const int32_t* t_indptr, const int32_t* t_dst,
                       const int32_t* hubs, const int32_t* src_deg, const int32_t* dst_deg, const float* dy, int64_t ldy,
                       const float* dy_self, int64_t ld_self, int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx,
                       const int32_t* n_dst_dev, void* stream) {
    if (!ws || mode < FGL_AGG_SUM || mode > FGL_AGG_SYMNORM || n_dst < 0 || n_src < 0 || dim < 1 || ldy < dim || ldx < dim)
        return FGL_ERR_INVALID;
    if (dy_self && (ld_self < dim || n_dst > n_src)) return FGL_ERR_INVALID;
    if (n_src == 0) return FGL_OK;
    if (!dx || !t_indptr || !hubs || (n_dst > 0 && (!dy || !t_dst || !indptr))) return FGL_ERR_INVALID;
    if (mode == FGL_AGG_SYMNORM && (!src_deg || !dst_deg)) return FGL_ERR_INVALID;
    GatherParams p{};
    p.indptr = indptr;
    p.t_indptr = t_indptr;
    p.t_dst = t_dst;
    p.hubs = hubs;
    p.src_deg = src_deg;
    p.dst_deg = dst_deg;
    p.dy = dy;
    p.dy_self = dy_self;
    p.dx = dx;
    p.ldy = ldy;
    p.ld_self = ld_self;
    p.ldx = ldx;
    p.dim = dim;
    p.n_dst = n_dst;
    p.n_src = n_src;
    p.n_dst_dev = n_dst_dev;
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int sms = ws->sm_count > 0 ? ws->sm_count : 148;
    switch (pick_vec(dim, dy, ldy, dx, ldx, dy_self, dy_self ? ld_self : 4)) {
        case 4: launch_gather_mode<4>(mode, p, sms, st); break;
        case 2: launch_gather_mode<2>(mode, p, sms, st); break;
        default: launch_gather_mode<1>(mode, p, sms, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

}  // extern "C"
