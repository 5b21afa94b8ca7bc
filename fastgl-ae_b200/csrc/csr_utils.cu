// Block-CSR helpers: id histogram and exclusive scan (replace cal_deg_cuda and exclusive_sum_cuda,
// utilis.cu:17-79).  The fused sampler emits the block CSR itself; these stay for callers that build
// it from a COO edge list the way GraphConv.py:93-96 does.
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace fgl {

constexpr int kScanThreads = 512;
constexpr int kScanItems = 8;  // ints per thread per tile

__global__ void __launch_bounds__(256) cal_deg_kernel(const int32_t* __restrict__ ids, int64_t n_ids,
                                                      int32_t* __restrict__ deg, int32_t n_nodes) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_ids; i += stride) {
        const int32_t v = ids[i];
        if (v >= 0 && v < n_nodes) atomicAdd(deg + v, 1);  // utilis.cu:55-57
    }
}

// Two-level scan in one cooperative launch: per-CTA totals, team barrier, per-CTA rescan with its base.
__global__ void __launch_bounds__(kScanThreads) exclusive_sum_kernel(const int32_t* __restrict__ in, int64_t n,
                                                                     int32_t* __restrict__ out,
                                                                     unsigned long long* bar, int32_t* partial,
                                                                     int32_t* status) {
    __shared__ int s_scan[40];
    __shared__ int s_flag;
    constexpr int kTile = kScanThreads * kScanItems;
    const int64_t n_tiles = (n + kTile - 1) / kTile;
    const int64_t tiles_per = (n_tiles + gridDim.x - 1) / gridDim.x;
    const int64_t t0 = min((long long)n_tiles, (long long)blockIdx.x * (long long)tiles_per);
    const int64_t t1 = min((long long)n_tiles, (long long)(t0 + tiles_per));
    const int64_t lo = t0 * kTile, hi = min((long long)n, (long long)(t1 * kTile));

    int acc = 0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kScanThreads) acc += in[i];
    const int total = block_sum(acc, s_scan);
    if (threadIdx.x == 0) __stcg(partial + blockIdx.x, total);

    Team t;
    t.rank = blockIdx.x;
    t.size = gridDim.x;
    t.epoch = 0;
    t.bar = bar;
    t.status = status;
    if (!team_barrier(t, &s_flag)) return;

    int a = 0, b = 0;
    for (int q = threadIdx.x; q < (int)gridDim.x; q += kScanThreads) {
        const int x = __ldcg(partial + q);
        b += x;
        if (q < (int)blockIdx.x) a += x;
    }
    int running = block_sum(a, s_scan);
    const int grand = block_sum(b, s_scan);
    if (blockIdx.x == 0 && threadIdx.x == 0) out[n] = grand;

    for (int64_t tile = lo; tile < hi; tile += kTile) {
        // each thread owns kScanItems consecutive entries
        const int64_t base = tile + (int64_t)threadIdx.x * kScanItems;
        int v[kScanItems];
        int sum = 0;
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) {
            v[k] = (base + k < hi) ? in[base + k] : 0;
            sum += v[k];
        }
        int tile_total;
        int excl = running + block_excl_scan(sum, s_scan, tile_total);
#pragma unroll
        for (int k = 0; k < kScanItems; ++k) {
            if (base + k < hi) out[base + k] = excl;
            excl += v[k];
        }
        running += tile_total;
    }
}

// Up to FGL_MAX_SEGMENTS device-to-device copies and a few int32 words in one launch: stages one mini-batch's
// blocks into the fixed buffers a captured CUDA graph reads, without one cudaMemcpyAsync per piece.
struct StageParams {
    fgl_segment seg[FGL_MAX_SEGMENTS];
    int64_t first_block[FGL_MAX_SEGMENTS + 1];  // CTA range of every segment
    int32_t n_segs;
    int32_t* words_dst;
    int32_t words[FGL_MAX_SEGMENTS];
    int32_t n_words;
};

constexpr int kStageThreads = 256;
constexpr int64_t kStageBytesPerBlock = kStageThreads * 16 * 8;  // 32 KB per CTA

__global__ void __launch_bounds__(kStageThreads) stage_segments_kernel(const __grid_constant__ StageParams p) {
    if (blockIdx.x == 0 && threadIdx.x < p.n_words) p.words_dst[threadIdx.x] = p.words[threadIdx.x];
    int s = 0;
    while (s + 1 < p.n_segs && (int64_t)blockIdx.x >= p.first_block[s + 1]) ++s;
    if (s >= p.n_segs) return;
    const int64_t lo = ((int64_t)blockIdx.x - p.first_block[s]) * kStageBytesPerBlock;
    const int64_t hi = lo + kStageBytesPerBlock < p.seg[s].bytes ? lo + kStageBytesPerBlock : p.seg[s].bytes;
    char* dst = static_cast<char*>(p.seg[s].dst);
    const char* src = static_cast<const char*>(p.seg[s].src);
    if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
        const int64_t v_hi = lo + ((hi - lo) / 16) * 16;
        for (int64_t o = lo + (int64_t)threadIdx.x * 16; o < v_hi; o += kStageThreads * 16)
            *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
        for (int64_t o = v_hi + (int64_t)threadIdx.x * 4; o < hi; o += kStageThreads * 4)
            *reinterpret_cast<uint32_t*>(dst + o) = *reinterpret_cast<const uint32_t*>(src + o);
    } else {
        for (int64_t o = lo + (int64_t)threadIdx.x * 4; o < hi; o += kStageThreads * 4)
            *reinterpret_cast<uint32_t*>(dst + o) = *reinterpret_cast<const uint32_t*>(src + o);
    }
}

// Measurement probe: the rate at which this GPU serves the sampler's access pattern when nothing else is done --
// isolated 4-byte reads at hashed positions of an array (a pick in a hub's neighbour list), each followed, if a
// table is given, by a dependent 8-byte load of a hashed slot and a compare-and-swap when the slot looks empty (the
// first probe of the id map's insert).  Four independent chains per thread are in flight.  The sampler's roofline
// by bytes assumes 32 useful bytes per pick at streaming bandwidth; this is what the memory system really sustains.
__device__ __forceinline__ uint32_t probe_mix(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

__global__ void __launch_bounds__(512, 2) access_probe_kernel(const int32_t* __restrict__ a, uint32_t n_words,
                                                              unsigned long long* __restrict__ table, uint32_t table_mask,
                                                              int iters, int32_t* __restrict__ sink) {
    constexpr int K = 4;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long acc = 0;
    for (int it = 0; it < iters; ++it) {
        int v[K];
#pragma unroll
        for (int q = 0; q < K; ++q) {
            const uint32_t r = probe_mix(tid * 977u + (uint32_t)(it * K + q) * 0x9E3779B1u);
            v[q] = __ldg(a + (uint32_t)(((uint64_t)r * n_words) >> 32));
        }
        if (table) {
            unsigned long long s[K];
#pragma unroll
            for (int q = 0; q < K; ++q) s[q] = *(volatile unsigned long long*)(table + (probe_mix((uint32_t)v[q]) & table_mask));
#pragma unroll
            for (int q = 0; q < K; ++q) {
                if (s[q] == 0ULL)
                    s[q] = atomicCAS(table + (probe_mix((uint32_t)v[q]) & table_mask), 0ULL, ((unsigned long long)(uint32_t)v[q] << 32) | 1u);
                acc += s[q];
            }
        } else {
#pragma unroll
            for (int q = 0; q < K; ++q) acc += (unsigned)v[q];
        }
    }
    if (acc == 0x7fffffffffffULL) sink[0] = (int32_t)acc;   // keeps the loads alive
}

// Pairwise overlap of the node lists of a window: overlap[i][j] = |nodes_i & nodes_j| (Match-Reorder's match degree,
// utilis.py:41-48, without one N-sized boolean mask per mini-batch).  One word per node holds a bit per mini-batch:
// pass 0 sets the bits, pass 1 reads every node's word back and counts, per mini-batch, the other mini-batches that
// hold the node too, pass 2 clears the words the lists touched, so the mask is zero again when the call returns.
__global__ void __launch_bounds__(256) window_overlap_kernel(const int32_t* __restrict__ nodes, int64_t nodes_stride,
                                                             const int32_t* __restrict__ counts, int64_t counts_stride,
                                                             int64_t n_nodes, uint32_t* __restrict__ mask,
                                                             int32_t* __restrict__ overlap, int n_batches, int pass) {
    __shared__ int hist[32];
    const int b = blockIdx.y;
    const int n = min(max(__ldg(counts + (int64_t)b * counts_stride), 0), (int)min((int64_t)0x7fffffff, nodes_stride));
    if (pass == 1) {
        if (threadIdx.x < 32) hist[threadIdx.x] = 0;
        __syncthreads();
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int id = __ldg(nodes + (int64_t)b * nodes_stride + i);
        if (id < 0 || (int64_t)id >= n_nodes) continue;
        if (pass == 0) {
            atomicOr(mask + id, 1u << b);
        } else if (pass == 1) {
            unsigned m = __ldcg(mask + id);
            while (m) {
                atomicAdd(&hist[__ffs(m) - 1], 1);
                m &= m - 1;
            }
        } else {
            mask[id] = 0u;
        }
    }
    if (pass == 1) {
        __syncthreads();
        if ((int)threadIdx.x < n_batches && hist[threadIdx.x] != 0) atomicAdd(overlap + b * n_batches + threadIdx.x, hist[threadIdx.x]);
    }
}

// Self-test of the bounded wait: every CTA arrives at a team barrier that expects one arrival more than the grid
// has, so the wait runs out after spin_limit polls, records FGL_ERR_TIMEOUT, raises the abort flag and returns.
__global__ void __launch_bounds__(32) barrier_timeout_kernel(unsigned long long* bar, int32_t* status, long long spin_limit,
                                                             int32_t* passed) {
    __shared__ int s_flag;
    Team t;
    t.rank = blockIdx.x;
    t.size = gridDim.x + 1;
    t.epoch = 0;
    t.bar = bar;
    t.status = status;
    t.spin_limit = spin_limit;
    if (team_barrier(t, &s_flag) && threadIdx.x == 0) atomicAdd(passed, 1);  // cannot happen: nobody sends the last arrival
}

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_cal_deg(const int32_t* ids, int64_t n_ids, int32_t* deg, int32_t n_nodes, void* stream) {
    if (n_ids < 0 || n_nodes < 0 || (n_ids > 0 && !ids) || (n_nodes > 0 && !deg)) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_nodes > 0 && cudaMemsetAsync(deg, 0, sizeof(int32_t) * (size_t)n_nodes, st) != cudaSuccess) return FGL_ERR_CUDA;
    if (n_ids == 0 || n_nodes == 0) return FGL_OK;
    const int grid = (int)std::min<int64_t>((n_ids + 255) / 256, 148 * 16);
    cal_deg_kernel<<<grid, 256, 0, st>>>(ids, n_ids, deg, n_nodes);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_stage_segments(const fgl_segment* segs, int32_t n_segs, int32_t* words_dst, const int32_t* words, int32_t n_words,
                       void* stream) {
    if (n_segs < 0 || n_segs > FGL_MAX_SEGMENTS || n_words < 0 || n_words > FGL_MAX_SEGMENTS || (n_segs > 0 && !segs) ||
        (n_words > 0 && (!words || !words_dst)))
        return FGL_ERR_INVALID;
    StageParams p;
    std::memset(&p, 0, sizeof(p));
    int64_t blocks = 0;
    for (int i = 0; i < n_segs; ++i) {
        if (segs[i].bytes < 0 || segs[i].bytes % 4 != 0 || (segs[i].bytes > 0 && (!segs[i].dst || !segs[i].src)) ||
            ((uintptr_t)segs[i].dst & 3) || ((uintptr_t)segs[i].src & 3))
            return FGL_ERR_INVALID;
        p.seg[i] = segs[i];
        p.first_block[i] = blocks;
        blocks += (segs[i].bytes + kStageBytesPerBlock - 1) / kStageBytesPerBlock;
    }
    for (int i = n_segs; i <= FGL_MAX_SEGMENTS; ++i) p.first_block[i] = blocks;
    p.n_segs = n_segs;
    p.words_dst = words_dst;
    for (int i = 0; i < n_words; ++i) p.words[i] = words[i];
    p.n_words = n_words;
    if (blocks == 0) blocks = 1;
    if (blocks > 0x7fffffffLL) return FGL_ERR_INVALID;
    stage_segments_kernel<<<(unsigned)blocks, kStageThreads, 0, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_window_overlap(const int32_t* nodes, int64_t nodes_stride, const int32_t* counts, int64_t counts_stride,
                       int32_t n_batches, int64_t n_nodes, uint32_t* mask, int32_t* overlap, void* stream) {
    if (n_batches < 0 || n_batches > 32 || nodes_stride < 0 || counts_stride < 1 || n_nodes < 0) return FGL_ERR_INVALID;
    if (n_batches == 0) return FGL_OK;
    if (!nodes || !counts || !mask || !overlap) return FGL_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(overlap, 0, sizeof(int32_t) * (size_t)n_batches * n_batches, st) != cudaSuccess) return FGL_ERR_CUDA;
    const dim3 grid((unsigned)std::max<int64_t>(1, std::min<int64_t>(148 * 4 / n_batches + 1, (nodes_stride + 255) / 256)), n_batches);
    for (int pass = 0; pass < 3; ++pass)
        window_overlap_kernel<<<grid, 256, 0, st>>>(nodes, nodes_stride, counts, counts_stride, n_nodes, mask, overlap, n_batches, pass);
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_probe_access_pattern(const int32_t* array, int64_t n_words, uint64_t* table, int64_t table_slots, int32_t iters,
                             int32_t* sink, int64_t* n_accesses, void* stream) {
    if (!array || n_words < 1 || n_words > 0xffffffffLL || iters < 1 || !sink || !n_accesses) return FGL_ERR_INVALID;
    if (table && (table_slots < 1 || table_slots > 0x80000000LL || (table_slots & (table_slots - 1)))) return FGL_ERR_INVALID;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = sms * 2;
    access_probe_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(array, (uint32_t)n_words, (unsigned long long*)table,
                                                               table ? (uint32_t)(table_slots - 1) : 0u, iters, sink);
    *n_accesses = (int64_t)grid * 512 * 4 * iters;
    return cudaGetLastError() == cudaSuccess ? FGL_OK : FGL_ERR_CUDA;
}

int fgl_selftest_barrier_timeout(fgl_ws* ws, int32_t n_ctas, int64_t spin_limit, void* stream) {
    if (!ws || n_ctas < 1 || n_ctas > 64 || spin_limit < 1 || spin_limit > kSpinLimit) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    int rc = ws_ensure(ws, 0, 256);
    if (rc != FGL_OK) return rc;
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->scratch, 0, 256, st));
    barrier_timeout_kernel<<<n_ctas, 32, 0, st>>>((unsigned long long*)ws->scratch, ws->status, (long long)spin_limit,
                                                  (int32_t*)(ws->scratch + 128));
    FGL_CUDA_OK(ws, cudaGetLastError());
    return FGL_OK;
}

int fgl_exclusive_sum(fgl_ws* ws, const int32_t* in, int64_t n, int32_t* out, void* stream) {
    if (!ws || n < 0 || (n > 0 && !in) || !out) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    int per_sm = 0;
    FGL_CUDA_OK(ws, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, exclusive_sum_kernel, kScanThreads, 0));
    const int64_t tiles = (n + kScanThreads * kScanItems - 1) / (kScanThreads * kScanItems);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((int64_t)per_sm * ws->sm_count, tiles));
    const int64_t need = 128 + (int64_t)grid * 4;
    int rc = ws_ensure(ws, 0, need);
    if (rc != FGL_OK) return rc;
    unsigned long long* bar = (unsigned long long*)ws->scratch;
    int32_t* partial = (int32_t*)(ws->scratch + 128);
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->scratch, 0, 128, st));
    int32_t* status = ws->status;
    void* args[] = {(void*)&in, (void*)&n, (void*)&out, (void*)&bar, (void*)&partial, (void*)&status};
    FGL_CUDA_OK(ws, cudaLaunchCooperativeKernel((const void*)exclusive_sum_kernel, dim3(grid), dim3(kScanThreads), args, 0, st));
    return FGL_OK;
}

}  // extern "C"
