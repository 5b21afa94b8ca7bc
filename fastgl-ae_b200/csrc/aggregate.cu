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

#include "common.cuh"

namespace fgl {

constexpr int kAggThreads = 256;
constexpr int kAggWarps = kAggThreads / 32;
#ifndef FGL_AGG_UNR1
#define FGL_AGG_UNR1 8  // neighbour rows in flight per lane for rows of up to 32 vectors
#endif
#ifndef FGL_AGG_MIN_CTAS
#define FGL_AGG_MIN_CTAS 3
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
template <int VEC, int MODE, bool HAS_MAP, int NACC, int UNR>
__global__ void __launch_bounds__(kAggThreads, FGL_AGG_MIN_CTAS) agg_fwd_kernel(const AggParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;  // dim % VEC == 0 by dispatch
    const bool window = p.out_row_off != nullptr;
    const int64_t padded = window ? __ldg(p.out_row_off + p.n_batches) : (int64_t)p.n_dst;
    const int64_t total = p.n_dst_dev ? min((int64_t)max(__ldg(p.n_dst_dev), 0), padded) : padded;
    // padding rows of a launch sized for more rows than the block has: zero them
    for (int64_t g = total + warp_global; g < padded; g += n_warps) {
        T* orow = reinterpret_cast<T*>(p.out + g * p.ldo);
        for (int c = lane; c < chunks; c += 32) orow[c] = V::zero();
    }

    // State of the row after the current one.  Its ids are fetched one row ahead so that the dependent chain
    // indptr -> src -> row_map is off the critical path.
    int b_n = 0, d_n = 0, a_n = 0, e_n = 0;
    int64_t lo_n = 0, hi_n = window ? __ldg(p.out_row_off + 1) : total;
    int64_t row_n = 0, self_n = 0;
    float w_n = 1.0f;
    unsigned bad_n = 0;  // neighbours (of the first 32) whose id is out of range: loaded from row 0, never added
    auto prefetch = [&](int64_t g) {
        a_n = 0;
        e_n = 0;
        row_n = 0;
        w_n = 1.0f;
        bad_n = 0;
        if (g >= total) return;
        while (g >= hi_n) {  // window mode only: step to the mini-batch that holds row g
            ++b_n;
            lo_n = hi_n;
            hi_n = __ldg(p.out_row_off + b_n + 1);
        }
        d_n = (int)(g - lo_n);
        const int32_t* indptr = p.indptr + (int64_t)b_n * p.indptr_stride;
        const int32_t* src = p.src + (int64_t)b_n * p.src_stride;
        const int32_t* row_map = HAS_MAP ? p.row_map + (int64_t)b_n * p.row_map_stride : nullptr;
        a_n = __ldg(indptr + d_n);
        e_n = __ldg(indptr + d_n + 1);
        bool bad = false;
        if (lane < e_n - a_n) {
            const int s = __ldg(src + a_n + lane);
            row_n = checked_row<HAS_MAP>(p, row_map, s);
            bad = row_n < 0;
            if (bad) row_n = 0;
            if (MODE == FGL_AGG_SYMNORM && !bad) w_n = 1.0f / sqrtf((float)__ldg(p.src_deg + s));
        }
        bad_n = __ballot_sync(0xffffffffu, bad);
        // the row's own input row, only validated where it is used (self copy, zero-degree pass-through)
        self_n = HAS_MAP ? ((int64_t)d_n < p.n_map ? (int64_t)__ldg(row_map + d_n) : -1) : (int64_t)d_n;
    };
    prefetch(warp_global);

    for (int64_t g = warp_global; g < total; g += n_warps) {
        const int b = b_n, d = d_n, a = a_n, e_end = e_n;
        const int64_t first_row = row_n;  // neighbours a .. a+31
        int64_t self_row = self_n;        // the row's own source row
        const float first_w = w_n;
        const unsigned first_bad = bad_n;
        if ((p.self_out || (a >= e_end && p.passthrough)) && (self_row < 0 || self_row >= p.n_rows)) {
            agg_bad_id(p);
            self_row = -1;
        }
        prefetch(g + n_warps);
        const int32_t* src = p.src + (int64_t)b * p.src_stride;
        const int32_t* row_map = HAS_MAP ? p.row_map + (int64_t)b * p.row_map_stride : nullptr;
        T* orow = reinterpret_cast<T*>(p.out + g * p.ldo);
        if (p.self_out) {
            const T* xr = reinterpret_cast<const T*>(x_row(p, self_row < 0 ? 0 : self_row));
            T* srow = reinterpret_cast<T*>(p.self_out + g * p.ld_self);
            for (int c = lane; c < chunks; c += 32) srow[c] = self_row < 0 ? V::zero() : __ldg(xr + c);
        }
        if (a >= e_end) {  // aggregate_acc_kernel.cu:307-308, :405-406
            const T* xr = reinterpret_cast<const T*>(x_row(p, self_row < 0 ? 0 : self_row));
            for (int c = lane; c < chunks; c += 32) orow[c] = (p.passthrough && self_row >= 0) ? __ldg(xr + c) : V::zero();
            continue;
        }
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(e_end - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)__ldg(p.dst_deg + d));

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
                int64_t my_row = first_row;
                float my_w = first_w;
                unsigned bad_mask = first_bad;
                if (e0 != a) {
                    my_row = 0;
                    my_w = 1.0f;
                    bool bad = false;
                    if (lane < cnt) {
                        const int s = __ldg(src + e0 + lane);
                        my_row = checked_row<HAS_MAP>(p, row_map, s);
                        bad = my_row < 0;
                        if (bad) my_row = 0;
                        if (MODE == FGL_AGG_SYMNORM && !bad) my_w = 1.0f / sqrtf((float)__ldg(p.src_deg + s));
                    }
                    bad_mask = __ballot_sync(0xffffffffu, bad);
                }
                for (int j0 = 0; j0 < cnt; j0 += UNR) {
                    T v[UNR][NACC];
                    float w[UNR];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int j = min(j0 + u, cnt - 1);  // past the end: reload the last row, skip its FMA
                        const int64_t r = __shfl_sync(0xffffffffu, my_row, j);
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

template <int VEC, int MODE>
static void launch_fwd_nacc(const AggParams& p, dim3 grid, cudaStream_t st) {
    const int chunks = p.dim / VEC;
    if (chunks <= 32)
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
    if ((mode != FGL_AGG_SUM && mode != FGL_AGG_MEAN) || n_batches < 0 || total_rows < 0 || total_rows > 0x7fffffffLL ||
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
    return launch_fwd_any(mode, p, dim3(agg_grid_x((int)total_rows, 1), 1), vec, (cudaStream_t)stream);
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
