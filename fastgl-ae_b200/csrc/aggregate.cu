// Sum / mean / sym-norm aggregation over a block CSR, forward (gather) and backward (scatter), sm_100a.
//
// The work is HBM-bound (one FMA per 4 bytes read), so no tensor cores: a warp owns one destination row,
// its lanes sweep the feature dimension with 128-bit loads (64- or 32-bit when the row stride is not a
// multiple of 16 bytes, e.g. 602 floats), the neighbour ids of the row are read once, coalesced, and handed
// round by shuffle, and the row's sum stays in registers until one coalesced store.
//
// Replaces K8 / K10 (aggregate_acc_kernel.cu:271-331, :376-427: 8 rows x 4 floats per warp, shared-memory
// read-modify-write per neighbour) and K9 / K11 (:468-517, :555-596: scalar atomics, the GCN one built from
// two atomicExch in a retry loop).
#include <algorithm>

#include "common.cuh"

namespace fgl {

constexpr int kAggThreads = 256;
constexpr int kAggWarps = kAggThreads / 32;
constexpr int kAcc = 4;  // vector accumulators per lane per pass: 32 lanes x 4 x VEC floats per pass

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
    int64_t ldx, ldo;
    int32_t dim, n_dst, n_src;
    int32_t passthrough;
};

// Forward: out[d,:] = scale_d * sum_e w_e * x[row(src[e]),:]
template <int VEC, int MODE, bool HAS_MAP>
__global__ void __launch_bounds__(kAggThreads) agg_fwd_kernel(const AggParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;  // dim % VEC == 0 by dispatch

    for (int d = warp_global; d < p.n_dst; d += n_warps) {
        const int a = __ldg(p.indptr + d), b = __ldg(p.indptr + d + 1);
        T* orow = reinterpret_cast<T*>(p.out + (int64_t)d * p.ldo);
        if (a >= b) {  // aggregate_acc_kernel.cu:307-308, :405-406
            const int64_t r = HAS_MAP ? (int64_t)__ldg(p.row_map + d) : (int64_t)d;
            const T* xr = reinterpret_cast<const T*>(p.x + r * p.ldx);
            for (int c = lane; c < chunks; c += 32) orow[c] = p.passthrough ? __ldg(xr + c) : V::zero();
            continue;
        }
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(b - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)__ldg(p.dst_deg + d));

        for (int c0 = 0; c0 < chunks; c0 += 32 * kAcc) {
            T acc[kAcc];
#pragma unroll
            for (int k = 0; k < kAcc; ++k) acc[k] = V::zero();
            for (int e0 = a; e0 < b; e0 += 32) {
                const int cnt = min(32, b - e0);
                int64_t my_row = 0;
                float my_w = 1.0f;
                if (lane < cnt) {
                    const int s = __ldg(p.src + e0 + lane);
                    my_row = HAS_MAP ? (int64_t)__ldg(p.row_map + s) : (int64_t)s;
                    if (MODE == FGL_AGG_SYMNORM) my_w = 1.0f / sqrtf((float)__ldg(p.src_deg + s));
                }
#pragma unroll 4
                for (int j = 0; j < cnt; ++j) {
                    const int64_t r = __shfl_sync(0xffffffffu, my_row, j);
                    const float w = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, j) : 1.0f;
                    const T* xr = reinterpret_cast<const T*>(p.x + r * p.ldx);
#pragma unroll
                    for (int k = 0; k < kAcc; ++k) {
                        const int c = c0 + k * 32 + lane;
                        if (c < chunks) V::fma(acc[k], w, __ldg(xr + c));
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < kAcc; ++k) {
                const int c = c0 + k * 32 + lane;
                if (c < chunks) orow[c] = (MODE == FGL_AGG_SUM) ? acc[k] : V::scale(acc[k], scale);
            }
        }
    }
}

__device__ __forceinline__ void red_add(float4* addr, const float4& v) { atomicAdd(addr, v); }
__device__ __forceinline__ void red_add(float2* addr, const float2& v) { atomicAdd(addr, v); }
__device__ __forceinline__ void red_add(float* addr, const float& v) { atomicAdd(addr, v); }

// Backward: dx[src[e],:] += w_e * scale_d * dy[d,:]; vector reductions (red.global.add.v4.f32 on sm_100a)
template <int VEC, int MODE>
__global__ void __launch_bounds__(kAggThreads) agg_bwd_kernel(const AggParams p) {
    using V = Vec<VEC>;
    using T = typename V::T;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kAggWarps + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * kAggWarps;
    const int chunks = p.dim / VEC;

    for (int d = warp_global; d < p.n_dst; d += n_warps) {
        const int a = __ldg(p.indptr + d), b = __ldg(p.indptr + d + 1);
        if (a >= b) continue;  // aggregate_acc_kernel.cu:498-500, :580-582
        float scale = 1.0f;
        if (MODE == FGL_AGG_MEAN) scale = 1.0f / (float)(b - a);
        if (MODE == FGL_AGG_SYMNORM) scale = 1.0f / sqrtf((float)__ldg(p.dst_deg + d));
        const T* grow = reinterpret_cast<const T*>(p.x + (int64_t)d * p.ldx);

        for (int c0 = 0; c0 < chunks; c0 += 32 * kAcc) {
            T g[kAcc];
#pragma unroll
            for (int k = 0; k < kAcc; ++k) {
                const int c = c0 + k * 32 + lane;
                g[k] = (c < chunks) ? V::scale(__ldg(grow + c), scale) : V::zero();
            }
            for (int e0 = a; e0 < b; e0 += 32) {
                const int cnt = min(32, b - e0);
                int my_s = 0;
                float my_w = 1.0f;
                if (lane < cnt) {
                    my_s = __ldg(p.src + e0 + lane);
                    if (MODE == FGL_AGG_SYMNORM) my_w = 1.0f / sqrtf((float)__ldg(p.src_deg + my_s));
                }
                for (int j = 0; j < cnt; ++j) {
                    const int s = __shfl_sync(0xffffffffu, my_s, j);
                    const float w = (MODE == FGL_AGG_SYMNORM) ? __shfl_sync(0xffffffffu, my_w, j) : 1.0f;
                    if (s < 0 || s >= p.n_src) continue;  // warp-uniform
                    T* xr = reinterpret_cast<T*>(p.out + (int64_t)s * p.ldo);
#pragma unroll
                    for (int k = 0; k < kAcc; ++k) {
                        const int c = c0 + k * 32 + lane;
                        if (c < chunks) red_add(xr + c, (MODE == FGL_AGG_SYMNORM) ? V::scale(g[k], w) : g[k]);
                    }
                }
            }
        }
    }
}

static int pick_vec(const void* a, int64_t lda, const void* b, int64_t ldb, int dim) {
    auto ok = [&](int v) {
        return dim % v == 0 && lda % v == 0 && ldb % v == 0 && ((uintptr_t)a % (4 * v)) == 0 && ((uintptr_t)b % (4 * v)) == 0;
    };
    if (ok(4)) return 4;
    if (ok(2)) return 2;
    return 1;
}

static int agg_grid(int n_rows) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = ((int64_t)n_rows + kAggWarps - 1) / kAggWarps;
    return (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)sms * 8));
}

template <int VEC, int MODE>
static void launch_fwd(const AggParams& p, int grid, cudaStream_t st) {
    if (p.row_map)
        agg_fwd_kernel<VEC, MODE, true><<<grid, kAggThreads, 0, st>>>(p);
    else
        agg_fwd_kernel<VEC, MODE, false><<<grid, kAggThreads, 0, st>>>(p);
}

template <int VEC>
static void launch_fwd_mode(int mode, const AggParams& p, int grid, cudaStream_t st) {
    if (mode == FGL_AGG_SUM) launch_fwd<VEC, FGL_AGG_SUM>(p, grid, st);
    if (mode == FGL_AGG_MEAN) launch_fwd<VEC, FGL_AGG_MEAN>(p, grid, st);
    if (mode == FGL_AGG_SYMNORM) launch_fwd<VEC, FGL_AGG_SYMNORM>(p, grid, st);
}

template <int VEC>
static void launch_bwd_mode(int mode, const AggParams& p, int grid, cudaStream_t st) {
    if (mode == FGL_AGG_SUM) agg_bwd_kernel<VEC, FGL_AGG_SUM><<<grid, kAggThreads, 0, st>>>(p);
    if (mode == FGL_AGG_MEAN) agg_bwd_kernel<VEC, FGL_AGG_MEAN><<<grid, kAggThreads, 0, st>>>(p);
    if (mode == FGL_AGG_SYMNORM) agg_bwd_kernel<VEC, FGL_AGG_SYMNORM><<<grid, kAggThreads, 0, st>>>(p);
}

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_agg_fwd(int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg, const int32_t* dst_deg,
                const int32_t* row_map, const float* x, int64_t ldx, int32_t dim, int32_t n_dst, int32_t flags,
                float* out, int64_t ldo, void* stream) {
    if (mode < FGL_AGG_SUM || mode > FGL_AGG_SYMNORM || n_dst < 0 || dim < 1 || ldx < dim || ldo < dim) return FGL_ERR_INVALID;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !x || !out) return FGL_ERR_INVALID;
    if (mode == FGL_AGG_SYMNORM && (!src_deg || !dst_deg)) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    AggParams p{indptr, src, src_deg, dst_deg, row_map, x, out, ldx, ldo, dim, n_dst, 0,
                (flags & FGL_AGG_ZERO_DEG_PASSTHROUGH) ? 1 : 0};
    const int grid = agg_grid(n_dst);
    switch (pick_vec(x, ldx, out, ldo, dim)) {
        case 4: launch_fwd_mode<4>(mode, p, grid, st); break;
        case 2: launch_fwd_mode<2>(mode, p, grid, st); break;
        default: launch_fwd_mode<1>(mode, p, grid, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_agg_bwd(int32_t mode, const int32_t* indptr, const int32_t* src, const int32_t* src_deg, const int32_t* dst_deg,
                const float* dy, int64_t ldy, int32_t dim, int32_t n_dst, int32_t n_src, float* dx, int64_t ldx,
                void* stream) {
    if (mode < FGL_AGG_SUM || mode > FGL_AGG_SYMNORM || n_dst < 0 || n_src < 0 || dim < 1 || ldy < dim || ldx < dim)
        return FGL_ERR_INVALID;
    if (n_src == 0) return FGL_OK;
    if (!dx) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemset2DAsync(dx, sizeof(float) * (size_t)ldx, 0, sizeof(float) * (size_t)dim, (size_t)n_src, st) != cudaSuccess)
        return FGL_ERR_CUDA;
    if (n_dst == 0) return FGL_OK;
    if (!indptr || !dy) return FGL_ERR_INVALID;
    if (mode == FGL_AGG_SYMNORM && (!src_deg || !dst_deg)) return FGL_ERR_INVALID;
    AggParams p{indptr, src, src_deg, dst_deg, nullptr, dy, dx, ldy, ldx, dim, n_dst, n_src, 0};
    const int grid = agg_grid(n_dst);
    switch (pick_vec(dy, ldy, dx, ldx, dim)) {
        case 4: launch_bwd_mode<4>(mode, p, grid, st); break;
        case 2: launch_bwd_mode<2>(mode, p, grid, st); break;
        default: launch_bwd_mode<1>(mode, p, grid, st); break;
    }
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

}  // extern "C"
