// Element-wise kernels of the training step around the aggregation path: the bias / ReLU / dropout epilogue
// of a dense layer and its backward (with the bias gradient), softmax cross-entropy with its gradient, and
// Adam over one flat parameter buffer.  The reference leaves all of these to PyTorch op by op
// (GraphConv.py:86-99, train_fastgl.py:366-372); here each is one launch, so that a captured training step
// is a few dozen kernels instead of a few hundred.  All are HBM/L2-bound streaming kernels: 128-bit accesses,
// grid sized from the element count, no shared-memory staging needed.
#include <cstdint>
#include <cuda_runtime.h>

#include "common.cuh"
#include "fastgl_b200.h"

namespace fgl {

constexpr int kEwThreads = 256;

// Dropout decision of element e = row * dim + column: word (e & 3) of the Philox4x32-10 block whose counter is
// (lo32(e >> 2), hi32(e >> 2), lo32(ctr), hi32(ctr)) under the key (lo32(seed), hi32(seed)).
__device__ __forceinline__ uint4 dropout_block(uint64_t seed, uint64_t ctr, uint64_t group) {
    return philox_block(seed, ctr, (uint32_t)(group >> 32), (uint32_t)group);
}

// y = dropout(relu(y + bias)), in place; the first n_copy_rows rows also go to copy_out (the self operand of the
// next layer).  VEC = 4: dim % 4 == 0, leading dimensions % 4 == 0, 16-byte aligned bases.
template <int VEC>
__global__ void __launch_bounds__(kEwThreads)
bias_relu_dropout_kernel(float* __restrict__ y, int64_t ld, int64_t n_rows, int dim, const float* __restrict__ bias,
                         uint32_t drop_below, float keep_scale, uint64_t rng_seed, uint64_t rng_ctr,
                         const int32_t* __restrict__ rng_ctr_dev, int flags, float* __restrict__ copy_out,
                         int64_t ld_copy, int64_t n_copy_rows) {
    const int64_t groups_per_row = dim / VEC;
    const int64_t total = n_rows * groups_per_row;
    const uint64_t ctr = rng_ctr + (rng_ctr_dev ? (uint64_t)(uint32_t)rng_ctr_dev[0] : 0ull);
    const bool relu = flags & FGL_EW_RELU, drop = drop_below != 0;
    for (int64_t g = (int64_t)blockIdx.x * kEwThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kEwThreads) {
        const int64_t r = g / groups_per_row;
        const int c = (int)(g - r * groups_per_row) * VEC;
        float* p = y + r * ld + c;
        if (VEC == 4) {
            float4 v = *reinterpret_cast<float4*>(p);
            const float4 b = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            if (relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            if (drop) {
                // element index e = r * dim + c is a multiple of 4: one Philox block serves the four columns
                const uint4 w = dropout_block(rng_seed, ctr, (uint64_t)(r * dim + c) >> 2);
                v.x = w.x < drop_below ? 0.f : v.x * keep_scale;
                v.y = w.y < drop_below ? 0.f : v.y * keep_scale;
                v.z = w.z < drop_below ? 0.f : v.z * keep_scale;
                v.w = w.w < drop_below ? 0.f : v.w * keep_scale;
            }
            *reinterpret_cast<float4*>(p) = v;
            if (r < n_copy_rows) *reinterpret_cast<float4*>(copy_out + r * ld_copy + c) = v;
        } else {
            float v = *p + (bias ? bias[c] : 0.f);
            if (relu) v = fmaxf(v, 0.f);
            if (drop) {
                const uint64_t e = (uint64_t)(r * dim + c);
                const uint32_t w = philox_word(dropout_block(rng_seed, ctr, e >> 2), (int)(e & 3));
                v = w < drop_below ? 0.f : v * keep_scale;
            }
            *p = v;
            if (r < n_copy_rows) copy_out[r * ld_copy + c] = v;
        }
    }
}

// dz = dy * (mask ? (out > 0 ? keep_scale : 0) : 1), in place over dy; dbias[c] += sum over rows of dz[:, c].
// A CTA owns a band of consecutive rows; thread t owns columns t, t + blockDim, ... so the column sums stay in
// registers and leave with one atomic per column per CTA.  Rows are taken eight at a time with all sixteen loads
// issued before the first store, so that the band is bandwidth- rather than latency-bound.
constexpr int kBwdMaxColsPerThread = 8;   // dim <= 8 * 256
constexpr int kBwdRowBatch = 8;

// SPLIT: dz is not written back over dy but as [hi | lo | hi] TF32 parts (see split_tf32_kernel) into split3, the three
// blocks block_stride columns apart: the form in which the error-compensated products read it.
// x rounded to TF32 (10-bit mantissa, round to nearest), as an fp32 value
__device__ __forceinline__ float to_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

template <bool SPLIT>
__global__ void __launch_bounds__(kEwThreads)
relu_dropout_bwd_kernel(float* __restrict__ dy, int64_t ldy, const float* __restrict__ out, int64_t ldo, int64_t n_rows,
                        int rows_per_cta, int dim, float keep_scale, float* __restrict__ dbias, int flags,
                        float* __restrict__ split3, int64_t ld3, int block_stride) {
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t r1 = r0 + rows_per_cta < n_rows ? r0 + rows_per_cta : n_rows;
    const bool mask = flags & FGL_EW_RELU;
    for (int c = threadIdx.x; c < dim; c += kEwThreads) {
        float acc = 0.f;
        for (int64_t r = r0; r < r1; r += kBwdRowBatch) {
            float g[kBwdRowBatch], o[kBwdRowBatch];
#pragma unroll
            for (int k = 0; k < kBwdRowBatch; ++k) {
                const bool in = r + k < r1;
                g[k] = in ? dy[(r + k) * ldy + c] : 0.f;
                o[k] = (in && mask) ? out[(r + k) * ldo + c] : 1.f;
            }
#pragma unroll
            for (int k = 0; k < kBwdRowBatch; ++k) {
                if (mask) g[k] = o[k] > 0.f ? g[k] * keep_scale : 0.f;
                if (SPLIT) {
                    if (r + k < r1) {
                        const float h = to_tf32(g[k]), l = to_tf32(g[k] - h);
                        float* d3 = split3 + (r + k) * ld3 + c;
                        d3[0] = h;
                        d3[block_stride] = l;
                        d3[2 * block_stride] = h;
                    }
                } else if (mask) {
                    if (r + k < r1) dy[(r + k) * ldy + c] = g[k];
                }
                acc += g[k];
            }
        }
        if (dbias && acc != 0.f) atomicAdd(dbias + c, acc);
    }
}

// The same backward for matrices whose rows are whole 16-byte vectors (dim % 4 == 0, dim <= 1024): a thread owns four
// consecutive columns, the CTA's 256 threads cover 256 / (dim / 4) rows per pass and four passes are in flight, so
// every access is 16 bytes wide.  The column sums of the threads that share a column group meet in shared memory.
// A CTA walks several bands of rows (grid-stride) and keeps its column sums in registers across them, so the bias
// gradient costs one 16-byte reduction per column group per CTA, from four CTAs per SM: with a CTA per band of 16
// rows the 450 k same-address atomics of a 28 k x 256 matrix took twice as long as moving the matrix (86 vs 29 us),
// and only when the columns were not all zero -- the step time followed the number of live ReLU units.
template <bool SPLIT>
__global__ void __launch_bounds__(kEwThreads)
relu_dropout_bwd_vec_kernel(float* __restrict__ dy, int64_t ldy, const float* __restrict__ out, int64_t ldo, int64_t n_rows,
                            int rows_per_cta, int dim, float keep_scale, float* __restrict__ dbias, int flags,
                            float* __restrict__ split3, int64_t ld3, int block_stride) {
    __shared__ float4 sums[kEwThreads];
    const int groups = dim >> 2;                       // column groups of four floats; <= 256
    const int lanes = kEwThreads / groups;             // rows covered per pass
    const int cg = threadIdx.x % groups, rl = threadIdx.x / groups;
    const bool active = rl < lanes;
    const bool mask = flags & FGL_EW_RELU;
    constexpr int kPasses = 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t r0 = (int64_t)blockIdx.x * rows_per_cta; active && r0 < n_rows; r0 += (int64_t)gridDim.x * rows_per_cta) {
        const int64_t r1 = r0 + rows_per_cta < n_rows ? r0 + rows_per_cta : n_rows;
        for (int64_t r = r0 + rl; r < r1; r += (int64_t)lanes * kPasses) {
            float4 g[kPasses], o[kPasses];
#pragma unroll
            for (int k = 0; k < kPasses; ++k) {
                const int64_t rr = r + (int64_t)k * lanes;
                const bool in = rr < r1;
                g[k] = in ? *reinterpret_cast<const float4*>(dy + rr * ldy + 4 * cg) : make_float4(0.f, 0.f, 0.f, 0.f);
                o[k] = (in && mask) ? *reinterpret_cast<const float4*>(out + rr * ldo + 4 * cg) : make_float4(1.f, 1.f, 1.f, 1.f);
            }
#pragma unroll
            for (int k = 0; k < kPasses; ++k) {
                const int64_t rr = r + (int64_t)k * lanes;
                if (mask) {
                    g[k].x = o[k].x > 0.f ? g[k].x * keep_scale : 0.f;
                    g[k].y = o[k].y > 0.f ? g[k].y * keep_scale : 0.f;
                    g[k].z = o[k].z > 0.f ? g[k].z * keep_scale : 0.f;
                    g[k].w = o[k].w > 0.f ? g[k].w * keep_scale : 0.f;
                }
                if (rr < r1) {
                    if (SPLIT) {
                        float4 h, l;
                        h.x = to_tf32(g[k].x); l.x = to_tf32(g[k].x - h.x);
                        h.y = to_tf32(g[k].y); l.y = to_tf32(g[k].y - h.y);
                        h.z = to_tf32(g[k].z); l.z = to_tf32(g[k].z - h.z);
                        h.w = to_tf32(g[k].w); l.w = to_tf32(g[k].w - h.w);
                        float* d3 = split3 + rr * ld3 + 4 * cg;
                        *reinterpret_cast<float4*>(d3) = h;
                        *reinterpret_cast<float4*>(d3 + block_stride) = l;
                        *reinterpret_cast<float4*>(d3 + 2 * block_stride) = h;
                    } else if (mask) {
                        *reinterpret_cast<float4*>(dy + rr * ldy + 4 * cg) = g[k];
                    }
                }
                acc.x += g[k].x;
                acc.y += g[k].y;
                acc.z += g[k].z;
                acc.w += g[k].w;
            }
        }
    }
    if (!dbias) return;
    sums[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x < groups) {
        float4 t = sums[threadIdx.x];
        for (int q = 1; q < lanes; ++q) {
            const float4 v = sums[q * groups + threadIdx.x];
            t.x += v.x;
            t.y += v.y;
            t.z += v.z;
            t.w += v.w;
        }
        float* b = dbias + 4 * threadIdx.x;   // 16-byte aligned: one vector reduction for the four columns
        if (t.x != 0.f || t.y != 0.f || t.z != 0.f || t.w != 0.f)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(b), "f"(t.x), "f"(t.y), "f"(t.z), "f"(t.w) : "memory");
    }
}

// Mean softmax cross-entropy over the first n_valid rows, and its gradient; a warp per row.
// row_loss[r] = logsumexp(z_r) - z_r[label_r] (0 for rows that do not count);
// dlogits[r, c] = (softmax(z_r)[c] - [c == label_r]) / n_valid for r < n_valid and 0 below.
constexpr int kXentWarps = 8;

__global__ void __launch_bounds__(kXentWarps * 32)
softmax_xent_rows_kernel(const float* __restrict__ logits, int64_t ld, const int64_t* __restrict__ labels,
                         const int32_t* __restrict__ label_ids, int64_t n_labels, int n_rows, int n_classes,
                         const int32_t* __restrict__ n_valid_dev, int n_valid_host, float* __restrict__ row_loss,
                         float* __restrict__ dlogits, int64_t ldd, int32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x * kXentWarps + warp;
    if (r >= n_rows) return;
    int n_valid = n_valid_dev ? n_valid_dev[0] : n_valid_host;
    n_valid = n_valid < 0 ? 0 : (n_valid > n_rows ? n_rows : n_valid);
    const float inv = n_valid > 0 ? 1.f / (float)n_valid : 0.f;
    const float* z = logits + (int64_t)r * ld;
    float* d = dlogits + (int64_t)r * ldd;
    float mine = 0.f;
    bool counted = false;
    if (r < n_valid) {
        const int64_t at = label_ids ? (int64_t)label_ids[r] : (int64_t)r;
        const int64_t label = at >= 0 && at < n_labels ? labels[at] : -1;
        if (label < 0 || label >= n_classes) {
            if (lane == 0) atomicCAS(status, FGL_OK, FGL_ERR_BOUNDS);
        } else {
            counted = true;
            float m = -INFINITY;
            for (int c = lane; c < n_classes; c += 32) m = fmaxf(m, z[c]);
#pragma unroll
            for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            float s = 0.f;
            for (int c = lane; c < n_classes; c += 32) s += expf(z[c] - m);
#pragma unroll
            for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            mine = m + logf(s) - z[label];
            const float rs = inv / s;
            for (int c = lane; c < n_classes; c += 32) d[c] = expf(z[c] - m) * rs - (c == (int)label ? inv : 0.f);
        }
    }
    if (!counted)
        for (int c = lane; c < n_classes; c += 32) d[c] = 0.f;
    if (lane == 0) row_loss[r] = mine;
}

// The output layer and its loss in one pass: logits = x W + b for a narrow W (n_classes <= 32 * CPL), then the
// softmax cross-entropy row loss, the gradient of the logits and the bias gradient.  Replaces a small GEMM that
// runs at a few TFLOP/s, a bias add, the loss and a column sum.
// A CTA of eight warps owns kLinXentRows rows.  Warp w multiplies the w-th eighth of the k range for all of the
// CTA's rows at once: lane l keeps x[row][k0 + l] of a 32-column chunk and hands it around by shuffle, every lane
// owns the classes lane, lane + 32, ... and reads W row by row (coalesced over the classes; W is k x n_classes
// floats and stays in L1/L2), so one W load feeds kLinXentRows FMAs.  The eight partial products meet in shared
// memory; warp r then finishes row r.
constexpr int kLinXentWarps = 8;
constexpr int kLinXentRows = 4;

template <int CPL>
__global__ void __launch_bounds__(kLinXentWarps * 32)
linear_xent_kernel(const float* __restrict__ x, int64_t ldx, int k, const float* __restrict__ w, int64_t ldw,
                   const float* __restrict__ bias, const int64_t* __restrict__ labels, const int32_t* __restrict__ label_ids,
                   int64_t n_labels, int n_rows, int n_classes, const int32_t* __restrict__ n_valid_dev, int n_valid_host,
                   float* __restrict__ row_loss, float* __restrict__ dlogits, int64_t ldd, float* __restrict__ dbias,
                   float* __restrict__ logits_out, int64_t ldl, int32_t* __restrict__ status) {
    __shared__ float part[kLinXentWarps][kLinXentRows][32 * CPL];
    __shared__ float db[32 * CPL];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = blockIdx.x * kLinXentRows;
    for (int c = threadIdx.x; c < 32 * CPL; c += blockDim.x) db[c] = 0.f;
    int n_valid = n_valid_dev ? n_valid_dev[0] : n_valid_host;
    n_valid = n_valid < 0 ? 0 : (n_valid > n_rows ? n_rows : n_valid);
    const float inv = n_valid > 0 ? 1.f / (float)n_valid : 0.f;
    // rows that need their logits: the valid ones, or all of them when the caller wants the logits
    const int rows_here = min(kLinXentRows, (logits_out ? n_rows : n_valid) - row0);

    float acc[kLinXentRows][CPL];
#pragma unroll
    for (int r = 0; r < kLinXentRows; ++r)
#pragma unroll
        for (int q = 0; q < CPL; ++q) acc[r][q] = 0.f;
    if (rows_here > 0) {
        const int slice = ((k + kLinXentWarps - 1) / kLinXentWarps + 31) / 32 * 32;   // columns per warp, whole chunks
        const int k_lo = warp * slice, k_hi = min(k, k_lo + slice);
        for (int kb = k_lo; kb < k_hi; kb += 32) {
            float xr[kLinXentRows];
#pragma unroll
            for (int r = 0; r < kLinXentRows; ++r)
                xr[r] = (r < rows_here && kb + lane < k_hi) ? x[(int64_t)(row0 + r) * ldx + kb + lane] : 0.f;
            const int cols = min(32, k_hi - kb);
#pragma unroll 8
            for (int t = 0; t < cols; ++t) {
                const float* wr = w + (int64_t)(kb + t) * ldw;
                float wv[CPL];
#pragma unroll
                for (int q = 0; q < CPL; ++q) wv[q] = (lane + 32 * q < n_classes) ? __ldg(wr + lane + 32 * q) : 0.f;
#pragma unroll
                for (int r = 0; r < kLinXentRows; ++r) {
                    const float xv = __shfl_sync(0xffffffffu, xr[r], t);
#pragma unroll
                    for (int q = 0; q < CPL; ++q) acc[r][q] = fmaf(xv, wv[q], acc[r][q]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kLinXentRows; ++r)
#pragma unroll
        for (int q = 0; q < CPL; ++q) part[warp][r][lane + 32 * q] = acc[r][q];
    __syncthreads();

    // warp r finishes row row0 + r
    const int r = row0 + warp;
    if (warp < kLinXentRows && r < n_rows) {
        float* d = dlogits + (int64_t)r * ldd;
        float z[CPL];
#pragma unroll
        for (int q = 0; q < CPL; ++q) {
            const int c = lane + 32 * q;
            float t = (bias && c < n_classes) ? bias[c] : 0.f;
#pragma unroll
            for (int ww = 0; ww < kLinXentWarps; ++ww) t += part[ww][warp][c];
            z[q] = t;
        }
        if (logits_out) {
#pragma unroll
            for (int q = 0; q < CPL; ++q)
                if (lane + 32 * q < n_classes) logits_out[(int64_t)r * ldl + lane + 32 * q] = z[q];
        }
        float mine = 0.f;
        bool counted = false;
        if (r < n_valid) {
            const int64_t at = label_ids ? (int64_t)label_ids[r] : (int64_t)r;
            const int64_t label = at >= 0 && at < n_labels ? labels[at] : -1;
            if (label < 0 || label >= n_classes) {
                if (lane == 0) atomicCAS(status, FGL_OK, FGL_ERR_BOUNDS);
            } else {
                counted = true;
                float m = -INFINITY;
#pragma unroll
                for (int q = 0; q < CPL; ++q)
                    if (lane + 32 * q < n_classes) m = fmaxf(m, z[q]);
#pragma unroll
                for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                float e[CPL], sum = 0.f, at_label = 0.f;
#pragma unroll
                for (int q = 0; q < CPL; ++q) {
                    const int c = lane + 32 * q;
                    e[q] = c < n_classes ? expf(z[q] - m) : 0.f;
                    sum += e[q];
                    if (c == (int)label) at_label = z[q];
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    sum += __shfl_xor_sync(0xffffffffu, sum, o);
                    at_label += __shfl_xor_sync(0xffffffffu, at_label, o);
                }
                mine = m + logf(sum) - at_label;
                const float rs = inv / sum;
#pragma unroll
                for (int q = 0; q < CPL; ++q) {
                    const int c = lane + 32 * q;
                    if (c < n_classes) {
                        const float g = e[q] * rs - (c == (int)label ? inv : 0.f);
                        d[c] = g;
                        if (dbias) atomicAdd(&db[c], g);
                    }
                }
            }
        }
        if (!counted)
            for (int c = lane; c < n_classes; c += 32) d[c] = 0.f;
        if (lane == 0) row_loss[r] = mine;
    }
    __syncthreads();
    if (dbias)
        for (int c = threadIdx.x; c < n_classes; c += blockDim.x)
            if (db[c] != 0.f) atomicAdd(dbias + c, db[c]);
}

// loss[0] = (sum of row_loss in a fixed order) / n_valid: thread t adds rows t, t + 256, ... in order, then the
// 256 partial sums are folded by a fixed tree, so the loss is reproducible from run to run.
__global__ void __launch_bounds__(kEwThreads)
softmax_xent_mean_kernel(const float* __restrict__ row_loss, int n_rows, const int32_t* __restrict__ n_valid_dev,
                         int n_valid_host, float* __restrict__ loss) {
    __shared__ float part[kEwThreads];
    float t = 0.f;
    for (int r = threadIdx.x; r < n_rows; r += kEwThreads) t += row_loss[r];
    part[threadIdx.x] = t;
    __syncthreads();
    for (int w = kEwThreads / 2; w; w >>= 1) {
        if ((int)threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int n_valid = n_valid_dev ? n_valid_dev[0] : n_valid_host;
        n_valid = n_valid < 0 ? 0 : (n_valid > n_rows ? n_rows : n_valid);
        loss[0] = n_valid > 0 ? part[0] / (float)n_valid : 0.f;
    }
}

// Adam with L2 weight decay over flat buffers, torch.optim.Adam's arithmetic:
//   g += wd * p;  m = b1 m + (1 - b1) g;  v = b2 v + (1 - b2) g^2;
//   p -= lr / (1 - b1^t) * m / (sqrt(v) / sqrt(1 - b2^t) + eps),   t = step[0] + 1.
// The last CTA to finish stores t back, so that a captured launch advances the step on every replay.
__global__ void __launch_bounds__(kEwThreads)
adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, int64_t n,
            float lr, float b1, float b2, float eps, float wd, int32_t* __restrict__ step, unsigned int* __restrict__ ticket) {
    const int t = *(volatile int32_t*)step + 1;
    const AdamCoef c = adam_coef(lr, b1, b2, eps, wd, t);
    for (int64_t i = ((int64_t)blockIdx.x * kEwThreads + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * kEwThreads * 4) {
        if (i + 4 <= n) {
            float4 pp = *reinterpret_cast<float4*>(p + i), gg = *reinterpret_cast<const float4*>(g + i);
            float4 mm = *reinterpret_cast<float4*>(m + i), vv = *reinterpret_cast<float4*>(v + i);
            adam_update(c, pp.x, gg.x, mm.x, vv.x);
            adam_update(c, pp.y, gg.y, mm.y, vv.y);
            adam_update(c, pp.z, gg.z, mm.z, vv.z);
            adam_update(c, pp.w, gg.w, mm.w, vv.w);
            *reinterpret_cast<float4*>(p + i) = pp;
            *reinterpret_cast<float4*>(m + i) = mm;
            *reinterpret_cast<float4*>(v + i) = vv;
        } else {
            for (int64_t j = i; j < n; ++j) {
                float pj = p[j], mj = m[j], vj = v[j];
                adam_update(c, pj, g[j], mj, vj);
                p[j] = pj; m[j] = mj; v[j] = vj;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            ticket[0] = 0;
            step[0] = t;
        }
    }
}

// Splits fp32 values into two TF32-representable parts, x = hi + lo + O(2^-22 |x|): hi = x rounded to TF32's 10-bit
// mantissa, lo = the (exactly representable) remainder rounded likewise.  A product A.B evaluated as
// Ahi.Bhi + Alo.Bhi + Ahi.Blo by TF32 tensor-core GEMMs that accumulate in fp32 then carries fp32-level error (the
// dropped lo.lo term is 2^-22 relative): the parts are stored with their low 13 mantissa bits zero, so the GEMM's own
// conversion to TF32 loses nothing.  Each part can be written to several places (column or row blocks of wider
// matrices), so that the three products become ONE GEMM over a three times longer inner dimension,
// [Ahi | Alo | Ahi] . [Bhi ; Bhi ; Blo], instead of three launches.
constexpr int kSplitMaxDst = 8;
struct SplitDst {
    float* ptr[kSplitMaxDst];
    long long ld[kSplitMaxDst];
    int lo_part[kSplitMaxDst];
    int n;
};

template <bool VEC4>
__global__ void __launch_bounds__(kEwThreads)
split_tf32_kernel(const float* __restrict__ x, int64_t rows, int cols, int64_t ldx, const SplitDst d) {
    const int per_row = VEC4 ? cols / 4 : cols;
    const int64_t total = rows * per_row;
    for (int64_t g = (int64_t)blockIdx.x * kEwThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kEwThreads) {
        const int64_t r = g / per_row;
        const int c = (int)(g - r * per_row) * (VEC4 ? 4 : 1);
        if (VEC4) {
            const float4 v = *reinterpret_cast<const float4*>(x + r * ldx + c);
            float4 h, l;
            h.x = to_tf32(v.x); l.x = to_tf32(v.x - h.x);
            h.y = to_tf32(v.y); l.y = to_tf32(v.y - h.y);
            h.z = to_tf32(v.z); l.z = to_tf32(v.z - h.z);
            h.w = to_tf32(v.w); l.w = to_tf32(v.w - h.w);
            for (int q = 0; q < d.n; ++q) *reinterpret_cast<float4*>(d.ptr[q] + r * d.ld[q] + c) = d.lo_part[q] ? l : h;
        } else {
            const float v = x[r * ldx + c];
            const float h = to_tf32(v), l = to_tf32(v - h);
            for (int q = 0; q < d.n; ++q) d.ptr[q][r * d.ld[q] + c] = d.lo_part[q] ? l : h;
        }
    }
}

// out[r, c] = sum over slabs s and blocks (a, b) of part[s][a * rows + r][b * block_stride + c]: folds the 2 x 2 block
// product [X_hi | X_lo]^T [dZ_hi | dZ_lo] (and its split-K slabs) into the weight gradient.  A warp per group of 32
// consecutive outputs of one row; the slabs are spread over the warps of a CTA (every lane keeps the n_a * n_b loads of
// its slab in flight together) and meet in shared memory, where they are added in slab order.
constexpr int kFoldWarps = 8;

__global__ void __launch_bounds__(kFoldWarps * 32)
fold_blocks_kernel(const float* __restrict__ part, int n_slabs, int n_a, int n_b, int rows, int cols, int block_stride,
                   int64_t ld_part, int64_t slab_stride, float* __restrict__ out, int64_t ldo) {
    __shared__ float partial[kFoldWarps][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int groups_per_row = (cols + 31) / 32;
    const int64_t n_groups = (int64_t)rows * groups_per_row;
    for (int64_t g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const int r = (int)(g / groups_per_row), c = (int)(g - (int64_t)r * groups_per_row) * 32 + lane;
        float acc = 0.f;
        if (c < cols) {
            for (int s = warp; s < n_slabs; s += kFoldWarps) {
                const float* base = part + s * slab_stride + (int64_t)r * ld_part + c;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (n_a == 2 && n_b == 2) {   // the 2 x 2 block product: four independent loads
                    v[0] = base[0];
                    v[1] = base[block_stride];
                    v[2] = base[(int64_t)rows * ld_part];
                    v[3] = base[(int64_t)rows * ld_part + block_stride];
                } else {
                    for (int a = 0; a < n_a; ++a)
                        for (int b = 0; b < n_b; ++b) v[0] += base[(int64_t)a * rows * ld_part + (int64_t)b * block_stride];
                }
                acc += (v[0] + v[1]) + (v[2] + v[3]);
            }
        }
        partial[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && c < cols) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < kFoldWarps; ++w) t += partial[w][lane];
            out[(int64_t)r * ldo + c] = t;
        }
        __syncthreads();
    }
}

static int ew_grid(int64_t work_items) {
    const int64_t blocks = (work_items + kEwThreads - 1) / kEwThreads;
    return (int)(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_bias_relu_dropout(float* y, int64_t ld, int64_t n_rows, int32_t dim, const float* bias, float p_drop,
                          uint64_t rng_seed, uint64_t rng_ctr, const int32_t* rng_ctr_dev, int32_t flags, float* copy_out,
                          int64_t ld_copy, int64_t n_copy_rows, void* stream) {
    if (n_rows < 0 || dim <= 0 || ld < dim || (n_rows > 0 && !y) || !(p_drop >= 0.f && p_drop < 1.f)) return FGL_ERR_INVALID;
    if (!copy_out) n_copy_rows = 0;
    if (n_copy_rows < 0 || n_copy_rows > n_rows || (n_copy_rows > 0 && ld_copy < dim)) return FGL_ERR_INVALID;
    if (n_rows == 0) return FGL_OK;
    // an element is dropped when its 32-bit word is below p * 2^32
    const double thresh = (double)p_drop * 4294967296.0;
    const uint32_t drop_below = p_drop > 0.f ? (uint32_t)(thresh >= 4294967295.0 ? 4294967295.0 : thresh) : 0u;
    const float keep_scale = p_drop > 0.f ? 1.f / (1.f - p_drop) : 1.f;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = dim % 4 == 0 && ld % 4 == 0 && aligned16(y) && (!bias || aligned16(bias)) &&
                     (n_copy_rows == 0 || (ld_copy % 4 == 0 && aligned16(copy_out)));
    if (vec)
        bias_relu_dropout_kernel<4><<<ew_grid(n_rows * (dim / 4)), kEwThreads, 0, st>>>(
            y, ld, n_rows, dim, bias, drop_below, keep_scale, rng_seed, rng_ctr, rng_ctr_dev, flags, copy_out, ld_copy,
            n_copy_rows);
    else
        bias_relu_dropout_kernel<1><<<ew_grid(n_rows * dim), kEwThreads, 0, st>>>(
            y, ld, n_rows, dim, bias, drop_below, keep_scale, rng_seed, rng_ctr, rng_ctr_dev, flags, copy_out, ld_copy,
            n_copy_rows);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

static int relu_dropout_bwd_launch(float* dy, int64_t ldy, const float* out, int64_t ldo, int64_t n_rows, int32_t dim, float p_drop,
                                   float* dbias, int32_t flags, float* split3, int64_t ld3, int64_t block_stride, void* stream) {
    if (n_rows < 0 || dim <= 0 || dim > kBwdMaxColsPerThread * kEwThreads || ldy < dim || (n_rows > 0 && !dy) ||
        !(p_drop >= 0.f && p_drop < 1.f))
        return FGL_ERR_INVALID;
    if ((flags & FGL_EW_RELU) && (!out || ldo < dim)) return FGL_ERR_INVALID;
    if (split3 && (block_stride < dim || block_stride > 0x3fffffffLL || ld3 < 2 * block_stride + dim)) return FGL_ERR_INVALID;
    if (n_rows == 0) return FGL_OK;
    // bands of 8..64 rows, sized so that the grid has at least two CTAs per SM where the matrix allows it
    int64_t rows_per_cta = (n_rows / (2 * 148)) / kBwdRowBatch * kBwdRowBatch;
    const int64_t band_max = split3 ? 16 : 64;   // three stores per element: shorter bands, more CTAs in flight
    rows_per_cta = rows_per_cta < kBwdRowBatch ? kBwdRowBatch : (rows_per_cta > band_max ? band_max : rows_per_cta);
    const int64_t blocks = (n_rows + rows_per_cta - 1) / rows_per_cta;
    if (blocks > 0x7fffffffLL) return FGL_ERR_INVALID;
    const float keep = p_drop > 0.f ? 1.f / (1.f - p_drop) : 1.f;
    const bool mask = (flags & FGL_EW_RELU) != 0;
    const bool vec = dim % 4 == 0 && dim <= 4 * kEwThreads && ldy % 4 == 0 && aligned16(dy) && (!mask || (ldo % 4 == 0 && aligned16(out))) &&
                     (!dbias || aligned16(dbias)) && (!split3 || (ld3 % 4 == 0 && block_stride % 4 == 0 && aligned16(split3)));
    if (vec) {
        // whole 16-byte vectors: 16 rows x (256 threads / column groups) per CTA pass
        const int lanes = kEwThreads / (dim / 4);
        int64_t band = (int64_t)lanes * 4 * (split3 ? 1 : 2);
        while (band < 16) band *= 2;
        int64_t nb = (n_rows + band - 1) / band;
        nb = nb < 4 * 148 ? nb : 4 * 148;   // four CTAs per SM, each walking its share of the bands
        if (split3)
            relu_dropout_bwd_vec_kernel<true><<<(unsigned)nb, kEwThreads, 0, (cudaStream_t)stream>>>(
                dy, ldy, out, ldo, n_rows, (int)band, dim, keep, dbias, flags, split3, ld3, (int)block_stride);
        else
            relu_dropout_bwd_vec_kernel<false><<<(unsigned)nb, kEwThreads, 0, (cudaStream_t)stream>>>(
                dy, ldy, out, ldo, n_rows, (int)band, dim, keep, dbias, flags, nullptr, 0, 0);
        return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
    }
    if (split3)
        relu_dropout_bwd_kernel<true><<<(unsigned)blocks, kEwThreads, 0, (cudaStream_t)stream>>>(
            dy, ldy, out, ldo, n_rows, (int)rows_per_cta, dim, keep, dbias, flags, split3, ld3, (int)block_stride);
    else
        relu_dropout_bwd_kernel<false><<<(unsigned)blocks, kEwThreads, 0, (cudaStream_t)stream>>>(
            dy, ldy, out, ldo, n_rows, (int)rows_per_cta, dim, keep, dbias, flags, nullptr, 0, 0);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_relu_dropout_bwd(float* dy, int64_t ldy, const float* out, int64_t ldo, int64_t n_rows, int32_t dim, float p_drop,
                         float* dbias, int32_t flags, void* stream) {
    return relu_dropout_bwd_launch(dy, ldy, out, ldo, n_rows, dim, p_drop, dbias, flags, nullptr, 0, 0, stream);
}

int fgl_relu_dropout_bwd_split(const float* dy, int64_t ldy, const float* out, int64_t ldo, int64_t n_rows, int32_t dim,
                               float p_drop, float* dbias, int32_t flags, float* split3, int64_t ld3, int64_t block_stride,
                               void* stream) {
    if (!split3) return FGL_ERR_INVALID;
    return relu_dropout_bwd_launch(const_cast<float*>(dy), ldy, out, ldo, n_rows, dim, p_drop, dbias, flags, split3, ld3,
                                   block_stride, stream);
}

int fgl_softmax_xent(fgl_ws* ws, const float* logits, int64_t ld, const int64_t* labels, const int32_t* label_ids,
                     int64_t n_labels, int32_t n_rows, int32_t n_classes, const int32_t* n_valid_dev, int32_t n_valid,
                     float* loss, float* dlogits, int64_t ldd, float* row_loss, void* stream) {
    if (!ws || n_rows < 0 || n_classes <= 0 || ld < n_classes || ldd < n_classes || !loss ||
        (n_rows > 0 && (!logits || !labels || !dlogits || !row_loss)))
        return FGL_ERR_INVALID;
    if (n_rows == 0) {
        return cudaMemsetAsync(loss, 0, sizeof(float), (cudaStream_t)stream) == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
    }
    cudaStream_t st = (cudaStream_t)stream;
    softmax_xent_rows_kernel<<<(n_rows + kXentWarps - 1) / kXentWarps, kXentWarps * 32, 0, st>>>(
        logits, ld, labels, label_ids, n_labels, n_rows, n_classes, n_valid_dev, n_valid, row_loss, dlogits, ldd, ws->status);
    softmax_xent_mean_kernel<<<1, kEwThreads, 0, st>>>(row_loss, n_rows, n_valid_dev, n_valid, loss);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_linear_softmax_xent(fgl_ws* ws, const float* x, int64_t ldx, int32_t k, const float* w, int64_t ldw, const float* bias,
                            const int64_t* labels, const int32_t* label_ids, int64_t n_labels, int32_t n_rows,
                            int32_t n_classes, const int32_t* n_valid_dev, int32_t n_valid, float* loss, float* dlogits,
                            int64_t ldd, float* dbias, float* logits_out, int64_t ldl, float* row_loss, void* stream) {
    if (!ws || n_rows < 0 || k <= 0 || n_classes <= 0 || n_classes > 128 || ldx < k || ldw < n_classes || ldd < n_classes ||
        !loss || (logits_out && ldl < n_classes) || (n_rows > 0 && (!x || !w || !labels || !dlogits || !row_loss)))
        return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_rows == 0) return cudaMemsetAsync(loss, 0, sizeof(float), st) == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
    const int grid = (n_rows + kLinXentRows - 1) / kLinXentRows;
#define FGL_LINXENT(CPL)                                                                                              \
    linear_xent_kernel<CPL><<<grid, kLinXentWarps * 32, 0, st>>>(x, ldx, k, w, ldw, bias, labels, label_ids, n_labels, \
                                                                 n_rows, n_classes, n_valid_dev, n_valid, row_loss,   \
                                                                 dlogits, ldd, dbias, logits_out, ldl, ws->status)
    if (n_classes <= 32) FGL_LINXENT(1);
    else if (n_classes <= 64) FGL_LINXENT(2);
    else FGL_LINXENT(4);
#undef FGL_LINXENT
    softmax_xent_mean_kernel<<<1, kEwThreads, 0, st>>>(row_loss, n_rows, n_valid_dev, n_valid, loss);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_adam_step(float* param, const float* grad, float* exp_avg, float* exp_avg_sq, int64_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int32_t* step_dev, void* stream) {
    if (n < 0 || (n > 0 && (!param || !grad || !exp_avg || !exp_avg_sq)) || !step_dev) return FGL_ERR_INVALID;
    if (n == 0) return FGL_OK;
    if (!aligned16(param) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq)) return FGL_ERR_INVALID;
    // step_dev[0] = completed steps, step_dev[1] = the kernel's arrival ticket (zero between launches)
    adam_kernel<<<ew_grid((n + 3) / 4), kEwThreads, 0, (cudaStream_t)stream>>>(
        param, grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, step_dev, (unsigned int*)(step_dev + 1));
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_split_tf32(const float* x, int64_t rows, int64_t cols, int64_t ldx, int n_dst, float* const* dst, const int64_t* ld_dst,
                   const int32_t* lo_part, void* stream) {
    if (rows < 0 || cols < 0 || cols > 0x7fffffffLL || ldx < cols || n_dst < 1 || n_dst > kSplitMaxDst || !dst || !ld_dst || !lo_part)
        return FGL_ERR_INVALID;
    if (rows == 0 || cols == 0) return FGL_OK;
    if (!x) return FGL_ERR_INVALID;
    SplitDst d{};
    d.n = n_dst;
    bool vec = cols % 4 == 0 && ldx % 4 == 0 && aligned16(x);
    for (int q = 0; q < n_dst; ++q) {
        if (!dst[q] || ld_dst[q] < cols) return FGL_ERR_INVALID;
        d.ptr[q] = dst[q];
        d.ld[q] = ld_dst[q];
        d.lo_part[q] = lo_part[q] ? 1 : 0;
        vec = vec && ld_dst[q] % 4 == 0 && aligned16(dst[q]);
    }
    const int64_t items = rows * (vec ? cols / 4 : cols);
    if (vec)
        split_tf32_kernel<true><<<ew_grid(items), kEwThreads, 0, (cudaStream_t)stream>>>(x, rows, (int)cols, ldx, d);
    else
        split_tf32_kernel<false><<<ew_grid(items), kEwThreads, 0, (cudaStream_t)stream>>>(x, rows, (int)cols, ldx, d);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_fold_blocks(const float* part, int32_t n_slabs, int32_t n_a, int32_t n_b, int32_t rows, int32_t cols, int32_t block_stride,
                    int64_t ld_part, int64_t slab_stride, float* out, int64_t ldo, void* stream) {
    if (n_slabs < 1 || n_a < 1 || n_b < 1 || rows < 0 || cols < 0 || block_stride < cols || ldo < cols ||
        ld_part < (int64_t)(n_b - 1) * block_stride + cols || slab_stride < (int64_t)n_a * rows * ld_part)
        return FGL_ERR_INVALID;
    if (rows == 0 || cols == 0) return FGL_OK;
    if (!part || !out) return FGL_ERR_INVALID;
    const int64_t groups = (int64_t)rows * ((cols + 31) / 32);
    fold_blocks_kernel<<<(unsigned)std::min<int64_t>(groups, 148 * 16), kFoldWarps * 32, 0, (cudaStream_t)stream>>>(
        part, n_slabs, n_a, n_b, rows, cols, block_stride, ld_part, slab_stride, out, ldo);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

}  // extern "C"
