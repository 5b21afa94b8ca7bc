// Shared device / host helpers of the fastgl_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

#include "fastgl_b200.h"

namespace fgl {

// ---------------------------------------------------------------------------------------------
// Workspace: one per device; owns the hashtable, scratch for scans / team barriers and the device
// status word.  Replaces the per-call cudaMalloc/cudaFree of the reference (sample.cu:118-197,
// id_map.cu:45-58, utilis.cu:33,38).
// ---------------------------------------------------------------------------------------------
struct Workspace {
    int device = 0;
    int sm_count = 0;
    unsigned long long* table = nullptr;  // hashtable slots (64 bit each)
    int64_t table_slots = 0;
    bool table_dirty = true;              // slots may hold keys: clear the whole table before the next fused launch
    char* scratch = nullptr;              // scan partials, barrier words, per-call counters
    int64_t scratch_bytes = 0;
    int32_t* status = nullptr;            // device: [0] first error, [1] abort flag
    int32_t* host_pinned = nullptr;       // pinned: small read-backs (status, counts)
    cudaEvent_t time_start = nullptr;     // fgl_ws_time_next_launch: recorded directly around the next window-level launch
    cudaEvent_t time_end = nullptr;
    std::mutex mu;
    std::string last_error;
};

int ws_ensure(Workspace* ws, int64_t table_slots, int64_t scratch_bytes);

// The pair of events a caller asked to have recorded around the next window-level launch (fgl_ws_time_next_launch):
// timing_begin records the first, timing_end the second and forgets both.
inline void timing_begin(Workspace* ws, cudaStream_t st) {
    if (ws->time_start) cudaEventRecord(ws->time_start, st);
}
inline void timing_end(Workspace* ws, cudaStream_t st) {
    if (ws->time_end) cudaEventRecord(ws->time_end, st);
    ws->time_start = nullptr;
    ws->time_end = nullptr;
}
int ws_fail_cuda(Workspace* ws, cudaError_t e, const char* what);

#define FGL_CUDA_OK(ws, call)                                      \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return fgl::ws_fail_cuda((ws), e__, #call); \
    } while (0)

// RAII: make the workspace's device current for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            changed = (cudaSetDevice(dev) == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

// ---------------------------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ void set_status(int32_t* status, int code) {
    // first error wins
    atomicCAS(status, FGL_OK, code);
}

// Philox4x32-10 (Salmon et al., SC'11); the reference draws from cuRAND's generator of the same family
// (sample.cu:68-70,91).  One block = counter (block_idx, seed_slot, lo32(ctr), hi32(ctr)) under key
// (lo32(seed), hi32(seed)) gives four words; pick slot i of a seed uses word i % 4 of block i / 4.
__device__ __forceinline__ uint4 philox_block(uint64_t rng_seed, uint64_t rng_ctr, uint32_t seed_slot, uint32_t block_idx) {
    uint32_t c0 = block_idx, c1 = seed_slot, c2 = (uint32_t)rng_ctr, c3 = (uint32_t)(rng_ctr >> 32);
    uint32_t k0 = (uint32_t)rng_seed, k1 = (uint32_t)(rng_seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
}

__device__ __forceinline__ uint32_t philox_word(const uint4& b, int i) {
    return i == 0 ? b.x : (i == 1 ? b.y : (i == 2 ? b.z : b.w));
}

__device__ __forceinline__ uint32_t philox_draw(uint64_t rng_seed, uint64_t rng_ctr, uint32_t seed_slot,
                                                uint32_t pick_slot) {
    return philox_word(philox_block(rng_seed, rng_ctr, seed_slot, pick_slot >> 2), (int)(pick_slot & 3));
}

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// Block-wide exclusive scan of one int per thread; returns the exclusive prefix and the block total.
// smem must hold 33 ints.  blockDim.x must be a multiple of 32 and <= 1024.  Contains __syncthreads.
__device__ __forceinline__ int block_excl_scan(int v, int* smem, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int incl = warp_incl_scan(v, lane);
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarp ? smem[lane] : 0;
        int wi = warp_incl_scan(w, lane);
        smem[lane] = wi - w;
        if (lane == 31) smem[32] = wi;
    }
    __syncthreads();
    const int res = smem[warp] + incl - v;
    total = smem[32];
    __syncthreads();
    return res;
}

// Block-wide sum (all threads get the result).  smem must hold 33 ints.
__device__ __forceinline__ int block_sum(int v, int* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarp ? smem[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
        if (lane == 0) smem[32] = w;
    }
    __syncthreads();
    const int res = smem[32];
    __syncthreads();
    return res;
}

// One Adam update with L2 weight decay (torch.optim.Adam's arithmetic), spelled with explicit roundings so that
// every kernel that applies it -- the plain optimizer launch and the one fused with the gradient exchange -- rounds
// the same way, whatever the compiler would contract around it.
struct AdamCoef {
    float b1, b2, eps, wd, step_size, c2;
};

__device__ __forceinline__ AdamCoef adam_coef(float lr, float b1, float b2, float eps, float wd, int t) {
    AdamCoef c;
    c.b1 = b1;
    c.b2 = b2;
    c.eps = eps;
    c.wd = wd;
    c.step_size = __fdiv_rn(lr, __fsub_rn(1.f, powf(b1, (float)t)));
    c.c2 = __fsqrt_rn(__fsub_rn(1.f, powf(b2, (float)t)));
    return c;
}

__device__ __forceinline__ void adam_update(const AdamCoef& c, float& p, float g, float& m, float& v) {
    const float grad = __fmaf_rn(c.wd, p, g);
    m = __fmaf_rn(c.b1, m, __fmul_rn(__fsub_rn(1.f, c.b1), grad));
    v = __fmaf_rn(c.b2, v, __fmul_rn(__fmul_rn(__fsub_rn(1.f, c.b2), grad), grad));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(c.step_size, m), __fadd_rn(__fdiv_rn(__fsqrt_rn(v), c.c2), c.eps)));
}

constexpr long long kSpinLimit = 20LL * 1000 * 1000;  // x ~50 ns: a second or so, then give up

// ----------------------------------------------------------------------------------------------
// team barrier: monotonic arrival counter, bounded spin
// ----------------------------------------------------------------------------------------------
struct Team {
    int rank, size;
    unsigned epoch;
    unsigned long long* bar;
    int32_t* status;
    long long spin_limit = kSpinLimit;
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Returns false when the launch was aborted (another CTA timed out); the caller then returns.
__device__ __forceinline__ bool team_barrier(Team& t, int* s_flag) {
    t.epoch += 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int aborted = 0;
        __threadfence();
        atomicAdd(t.bar, 1ULL);
        const unsigned long long target = (unsigned long long)t.epoch * (unsigned long long)t.size;
        long long spins = 0;
        while (ld_acquire_u64(t.bar) < target) {
            if (*(volatile int32_t*)(t.status + 1) != 0) {
                aborted = 1;
                break;
            }
            if (++spins > t.spin_limit) {
                set_status(t.status, FGL_ERR_TIMEOUT);
                atomicExch(t.status + 1, 1);
                aborted = 1;
                break;
            }
            __nanosleep(32);
        }
        __threadfence();
        *s_flag = aborted;
    }
    __syncthreads();
    const bool ok = (*s_flag == 0);
    __syncthreads();
    return ok;
}


#endif  // __CUDACC__

}  // namespace fgl

struct fgl_ws : public fgl::Workspace {};
