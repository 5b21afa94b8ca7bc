// Data-parallel gradient averaging fused with the Adam step: one launch per training step, no library collective.
//
// Every rank holds, mapped into its address space, the receive buffers and flag arrays of all ranks of the box
// (CUDA IPC; NVLink through NVSwitch).  A CTA owns a fixed set of 8 KB chunks of the flat gradient.  For each of
// its chunks it (1) pushes the local gradient into every peer's receive buffer with plain 128-bit peer stores and
// then raises that chunk's flag on every peer (st.release.sys), (2) waits until every peer's flag for the chunk
// has arrived in its own flag array (ld.acquire.sys, bounded), (3) adds the world's contributions in rank order --
// the same order on every rank, so the replicas stay bit-identical -- scales by 1 / world and applies Adam to the
// chunk.  Chunks are independent, so there is no grid-wide barrier, and the transfer of one chunk overlaps the
// arithmetic of another.  0.8 MB of gradients (3-layer GraphSAGE, 256 hidden) are 98 chunks.
//
// Receive buffers and flags are double-buffered by the parity of a device-side epoch counter that the launch
// itself advances, so the launch can sit inside a captured CUDA graph and be replayed.  A peer can be at most one
// step ahead (it needs this rank's flags of step e to finish step e), so two buffers suffice.
//
// The reference has no counterpart: it trains data-parallel replicas without ever synchronising their gradients
// (train_fastgl.py:204-212,404-405).
#include <algorithm>

#include "common.cuh"

namespace fgl {

constexpr int kSyncThreads = 256;
constexpr int kSyncChunk = 2048;  // floats per chunk: two float4 per thread

struct SyncParams {
    int rank, world;
    float* recv[FGL_MAX_PEERS];
    uint32_t* flags[FGL_MAX_PEERS];
    int64_t n, n_pad;
    int n_chunks;
    float* param;
    float* grad;
    float* m;
    float* v;
    float lr, b1, b2, eps, wd;
    int32_t* step;  // [0] completed Adam steps, [1] arrival ticket, [2] completed exchanges (epoch)
    int32_t* status;
    long long spin_limit;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kSyncThreads) allreduce_adam_kernel(const __grid_constant__ SyncParams p) {
    __shared__ int s_fail;
    const uint32_t e = (uint32_t)(*(volatile int32_t*)(p.step + 2)) + 1u;
    const int t = *(volatile int32_t*)p.step + 1;
    const int parity = (int)(e & 1u);
    const int64_t slot_mine = ((int64_t)parity * p.world + p.rank) * p.n_pad;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    // (1) push this rank's chunks to every peer, then raise the chunks' flags there
    for (int c = blockIdx.x; c < p.n_chunks; c += gridDim.x) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int64_t i = (int64_t)c * kSyncChunk + ((int64_t)k * kSyncThreads + threadIdx.x) * 4;
            const float4 g = i < p.n ? *reinterpret_cast<const float4*>(p.grad + i) : zero4;
            for (int q = 0; q < p.world; ++q)
                if (q != p.rank) *reinterpret_cast<float4*>(p.recv[q] + slot_mine + i) = g;
        }
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
        uint32_t* f = p.flags[threadIdx.x] + ((int64_t)parity * p.world + p.rank) * p.n_chunks;
        for (int c = blockIdx.x; c < p.n_chunks; c += gridDim.x) st_release_sys(f + c, e);
    }

    // (2) + (3) per chunk: wait for the peers' contributions, reduce in rank order, Adam
    const AdamCoef coef = adam_coef(p.lr, p.b1, p.b2, p.eps, p.wd, t);
    const float inv_world = 1.f / (float)p.world;
    const float* mine = p.recv[p.rank];
    for (int c = blockIdx.x; c < p.n_chunks; c += gridDim.x) {
        if (threadIdx.x == 0) s_fail = 0;
        __syncthreads();
        if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
            const uint32_t* f = p.flags[p.rank] + ((int64_t)parity * p.world + threadIdx.x) * p.n_chunks + c;
            long long spins = 0;
            while ((int32_t)(ld_acquire_sys(f) - e) < 0) {  // flags only grow: e, e + 2, ...
                if (++spins > p.spin_limit) {
                    set_status(p.status, FGL_ERR_TIMEOUT);
                    s_fail = 1;
                    break;
                }
                __nanosleep(64);
            }
        }
        __syncthreads();
        if (s_fail) {  // a peer never delivered: leave the chunk's parameters untouched, the status word says why
            __syncthreads();
            continue;
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int64_t i = (int64_t)c * kSyncChunk + ((int64_t)k * kSyncThreads + threadIdx.x) * 4;
            if (i >= p.n) continue;
            float4 g = zero4;
            for (int q = 0; q < p.world; ++q) {
                const float4 x = q == p.rank ? *reinterpret_cast<const float4*>(p.grad + i)
                                             : __ldcg(reinterpret_cast<const float4*>(mine + ((int64_t)parity * p.world + q) * p.n_pad + i));
                g.x += x.x;
                g.y += x.y;
                g.z += x.z;
                g.w += x.w;
            }
            g.x *= inv_world;
            g.y *= inv_world;
            g.z *= inv_world;
            g.w *= inv_world;
            *reinterpret_cast<float4*>(p.grad + i) = g;
            float4 pp = *reinterpret_cast<float4*>(p.param + i);
            float4 mm = *reinterpret_cast<float4*>(p.m + i), vv = *reinterpret_cast<float4*>(p.v + i);
            adam_update(coef, pp.x, g.x, mm.x, vv.x);
            adam_update(coef, pp.y, g.y, mm.y, vv.y);
            adam_update(coef, pp.z, g.z, mm.z, vv.z);
            adam_update(coef, pp.w, g.w, mm.w, vv.w);
            *reinterpret_cast<float4*>(p.param + i) = pp;
            *reinterpret_cast<float4*>(p.m + i) = mm;
            *reinterpret_cast<float4*>(p.v + i) = vv;
        }
        __syncthreads();
    }
    // the last CTA to finish advances the step and the epoch, so that a captured launch moves on with every replay
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd((unsigned int*)(p.step + 1), 1u) == gridDim.x - 1) {
            p.step[1] = 0;
            p.step[0] = t;
            p.step[2] = (int32_t)e;
        }
    }
}

}  // namespace fgl

using namespace fgl;

extern "C" {

int fgl_sizeof_peer_sync(void) { return (int)sizeof(fgl_peer_sync); }

int64_t fgl_peer_sync_chunks(int64_t n) { return n <= 0 ? 0 : (n + kSyncChunk - 1) / kSyncChunk; }

int fgl_allreduce_adam(fgl_ws* ws, const fgl_peer_sync* peers, float* param, float* grad, float* exp_avg, float* exp_avg_sq,
                       int64_t n, float lr, float beta1, float beta2, float eps, float weight_decay, int32_t* step_dev,
                       int64_t spin_limit, void* stream) {
    if (!ws || !peers || n < 0 || n % 4 != 0 || !step_dev || peers->world < 1 || peers->world > FGL_MAX_PEERS ||
        peers->rank < 0 || peers->rank >= peers->world || spin_limit < 1)
        return FGL_ERR_INVALID;
    if (n == 0) return FGL_OK;
    if (!param || !grad || !exp_avg || !exp_avg_sq) return FGL_ERR_INVALID;
    const int64_t chunks = fgl_peer_sync_chunks(n);
    if (peers->n_chunks != chunks || peers->n_pad < chunks * kSyncChunk || chunks > 0x7fffffffLL) return FGL_ERR_INVALID;
    auto misaligned = [](const void* q) { return ((uintptr_t)q & 15) != 0; };
    if (misaligned(param) || misaligned(grad) || misaligned(exp_avg) || misaligned(exp_avg_sq)) return FGL_ERR_INVALID;
    SyncParams p{};
    p.rank = peers->rank;
    p.world = peers->world;
    for (int q = 0; q < peers->world; ++q) {
        if (peers->world > 1 && (!peers->recv[q] || !peers->flags[q] || misaligned(peers->recv[q]))) return FGL_ERR_INVALID;
        p.recv[q] = peers->recv[q];
        p.flags[q] = peers->flags[q];
    }
    p.n = n;
    p.n_pad = peers->n_pad;
    p.n_chunks = (int)chunks;
    p.param = param;
    p.grad = grad;
    p.m = exp_avg;
    p.v = exp_avg_sq;
    p.lr = lr;
    p.b1 = beta1;
    p.b2 = beta2;
    p.eps = eps;
    p.wd = weight_decay;
    p.step = step_dev;
    p.status = ws->status;
    p.spin_limit = spin_limit;
    DeviceGuard guard(ws->device);
    // every CTA of the grid is resident at once: a CTA that waits for a peer never keeps one that the peer waits for
    // off the GPU
    int per_sm = 0;
    FGL_CUDA_OK(ws, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_adam_kernel, kSyncThreads, 0));
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(chunks, (int64_t)std::max(1, per_sm) * ws->sm_count));
    allreduce_adam_kernel<<<grid, kSyncThreads, 0, (cudaStream_t)stream>>>(p);
    FGL_CUDA_OK(ws, cudaGetLastError());
    return FGL_OK;
}

}  // extern "C"
