// Exclusive scan entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a block-CSR offset array: a
// plugin whose framework allocator owns all device memory and hands out a fixed budget, a process whose
// HBM is already carved up between other pools (a 180 GB feature table plus graph leaves little slack), or
// a latency-critical loop that cannot take the implicit device synchronisation of an allocation.
// fgl_exclusive_sum needs a few KB of scratch (one arrival counter for the two-level scan's barrier and one
// partial sum per CTA) and takes it from the workspace, which grows with cudaMalloc.  The variant below
// keeps that scratch in a file-scope __device__ array instead: every GPU that loads the library holds
// these ~4.5 KB until the process exits, and the call itself allocates nothing.
//
// The array's name is only a host-side handle.  The device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) the first time the entry point runs there; that first
// call should come before any stream capture.  All calls share the array, which keeps the previous call's
// contents: each call clears the words that must start at zero, and two calls whose kernels overlap on the
// GPU (different streams) would race.  If the scan's bounded barrier ever gives up, FGL_ERR_TIMEOUT is left
// in the array's status word and the output is incomplete.  That word is not cleared by later scans: it keeps
// the first failure until fgl_exclusive_sum_noalloc_status copies it to the caller's host memory and clears it
// (again without allocating anything).
#include <algorithm>

#include "common.cuh"

namespace fgl {

constexpr int kNaThreads = 512;
constexpr int kNaItems = 8;
constexpr int kNaMaxCtas = 1024;
constexpr int64_t kNaMaxN = FGL_NOALLOC_MAX_N;
// layout: [0] arrival counter (u64) | [2] status, [3] abort flag (i32) | [32 ..) one partial sum per CTA
constexpr int kNaWords = 32 + kNaMaxCtas;

static __device__ __align__(256) unsigned long long g_noalloc_scratch[(kNaWords * 4 + 7) / 8 + 32];

__global__ void __launch_bounds__(kNaThreads) exclusive_sum_noalloc_kernel(const int32_t* __restrict__ in, int64_t n,
                                                                           int32_t* __restrict__ out, int32_t* scratch) {
    __shared__ int s_scan[40];
    __shared__ int s_flag;
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(scratch);
    int32_t* status = scratch + 2;
    int32_t* partial = scratch + 32;
    constexpr int kTile = kNaThreads * kNaItems;
    const int64_t n_tiles = (n + kTile - 1) / kTile;
    const int64_t tiles_per = (n_tiles + gridDim.x - 1) / gridDim.x;
    const int64_t t0 = min((long long)n_tiles, (long long)blockIdx.x * (long long)tiles_per);
    const int64_t t1 = min((long long)n_tiles, (long long)(t0 + tiles_per));
    const int64_t lo = t0 * kTile, hi = min((long long)n, (long long)(t1 * kTile));

    int acc = 0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kNaThreads) acc += in[i];
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
    for (int q = threadIdx.x; q < (int)gridDim.x; q += kNaThreads) {
        const int x = __ldcg(partial + q);
        b += x;
        if (q < (int)blockIdx.x) a += x;
    }
    int running = block_sum(a, s_scan);
    const int grand = block_sum(b, s_scan);
    if (blockIdx.x == 0 && threadIdx.x == 0) out[n] = grand;

    for (int64_t tile = lo; tile < hi; tile += kTile) {
        const int64_t base = tile + (int64_t)threadIdx.x * kNaItems;
        int v[kNaItems];
        int sum = 0;
#pragma unroll
        for (int k = 0; k < kNaItems; ++k) {
            v[k] = (base + k < hi) ? in[base + k] : 0;
            sum += v[k];
        }
        int tile_total;
        int excl = running + block_excl_scan(sum, s_scan, tile_total);
#pragma unroll
        for (int k = 0; k < kNaItems; ++k) {
            if (base + k < hi) out[base + k] = excl;
            excl += v[k];
        }
        running += tile_total;
    }
}

constexpr int kMaxDevices = 64;
static std::mutex g_na_mu;
static int32_t* g_na_ptr[kMaxDevices] = {nullptr};  // device address of g_noalloc_scratch, per device
static int g_na_max_grid[kMaxDevices] = {0};

// One-time set-up for the current device: resolve the symbol to a device address and size the grid.
static int noalloc_setup(int dev) {
    std::lock_guard<std::mutex> lock(g_na_mu);
    if (g_na_ptr[dev]) return FGL_OK;
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
        cudaGetLastError();
        return FGL_ERR_CUDA;
    }
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, exclusive_sum_noalloc_kernel, kNaThreads, 0) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1 || sms < 1) {
        cudaGetLastError();
        return FGL_ERR_CUDA;
    }
    g_na_max_grid[dev] = std::min(kNaMaxCtas, per_sm * sms);
    g_na_ptr[dev] = static_cast<int32_t*>(ptr);
    return FGL_OK;
}

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_exclusive_sum_noalloc(const int32_t* in, int64_t n, int32_t* out, void* stream) {
    if (n < 0 || (n > 0 && !in) || !out) return FGL_ERR_INVALID;
    if (n > kNaMaxN) return FGL_ERR_CAPACITY;  // beyond FGL_NOALLOC_MAX_N entries: use fgl_exclusive_sum
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FGL_ERR_CUDA;
    int rc = noalloc_setup(dev);
    if (rc != FGL_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* scratch = g_na_ptr[dev];
    const int64_t tiles = (n + kNaThreads * kNaItems - 1) / (kNaThreads * kNaItems);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(g_na_max_grid[dev], tiles));
    // the arrival counter (words 0-1) and the abort flag (word 3) must start at zero; the status word (2) keeps the
    // first failure until fgl_exclusive_sum_noalloc_status reads it; the partials are rewritten by every CTA
    if (cudaMemsetAsync(scratch, 0, 2 * sizeof(int32_t), st) != cudaSuccess ||
        cudaMemsetAsync(scratch + 3, 0, sizeof(int32_t), st) != cudaSuccess)
        return FGL_ERR_CUDA;
    void* args[] = {(void*)&in, (void*)&n, (void*)&out, (void*)&scratch};
    if (cudaLaunchCooperativeKernel((const void*)exclusive_sum_noalloc_kernel, dim3(grid), dim3(kNaThreads), args, 0, st) !=
        cudaSuccess) {
        cudaGetLastError();
        return FGL_ERR_CUDA;
    }
    return FGL_OK;
}

int fgl_exclusive_sum_noalloc_status(int32_t* host_dst, void* stream) {
    if (!host_dst) return FGL_ERR_INVALID;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FGL_ERR_CUDA;
    int rc = noalloc_setup(dev);
    if (rc != FGL_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* status = g_na_ptr[dev] + 2;
    if (cudaMemcpyAsync(host_dst, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemsetAsync(status, 0, sizeof(int32_t), st) != cudaSuccess) {
        cudaGetLastError();
        return FGL_ERR_CUDA;
    }
    return FGL_OK;
}

}  // extern "C"
