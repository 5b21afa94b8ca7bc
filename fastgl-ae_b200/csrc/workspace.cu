// Workspace management and status plumbing of the fastgl_b200 C ABI.
#include <cstdio>
#include <new>

#include "common.cuh"

namespace fgl {

int ws_fail_cuda(Workspace* ws, cudaError_t e, const char* what) {
    if (ws) {
        ws->last_error = std::string(what) + ": " + cudaGetErrorString(e);
    }
    return FGL_ERR_CUDA;
}

// Grows (never shrinks) the table / scratch.  Allocation synchronises the device, so callers that
// capture streams reserve up front.
int ws_ensure(Workspace* ws, int64_t table_slots, int64_t scratch_bytes) {
    if (table_slots > ws->table_slots) {
        if (ws->table) FGL_CUDA_OK(ws, cudaFree(ws->table));
        ws->table = nullptr;
        ws->table_slots = 0;
        cudaError_t e = cudaMalloc(&ws->table, sizeof(unsigned long long) * (size_t)table_slots);
        if (e != cudaSuccess) {
            ws->last_error = "hashtable allocation failed: " + std::string(cudaGetErrorString(e));
            cudaGetLastError();
            return FGL_ERR_NOMEM;
        }
        ws->table_slots = table_slots;
        ws->table_dirty = true;
    }
    if (scratch_bytes > ws->scratch_bytes) {
        if (ws->scratch) FGL_CUDA_OK(ws, cudaFree(ws->scratch));
        ws->scratch = nullptr;
        ws->scratch_bytes = 0;
        cudaError_t e = cudaMalloc(&ws->scratch, (size_t)scratch_bytes);
        if (e != cudaSuccess) {
            ws->last_error = "scratch allocation failed: " + std::string(cudaGetErrorString(e));
            cudaGetLastError();
            return FGL_ERR_NOMEM;
        }
        ws->scratch_bytes = scratch_bytes;
    }
    return FGL_OK;
}

}  // namespace fgl

extern "C" {

int fgl_abi_version(void) { return FGL_ABI_VERSION; }

int fgl_sizeof_fused_args(void) { return (int)sizeof(fgl_fused_args); }

const char* fgl_status_str(int status) {
    switch (status) {
        case FGL_OK: return "ok";
        case FGL_ERR_INVALID: return "invalid argument";
        case FGL_ERR_CUDA: return "CUDA runtime error";
        case FGL_ERR_NOMEM: return "workspace allocation failed";
        case FGL_ERR_CAPACITY: return "output buffer or hashtable capacity exceeded";
        case FGL_ERR_PROBE: return "hashtable probe limit reached";
        case FGL_ERR_BOUNDS: return "node id out of range";
        case FGL_ERR_TIMEOUT: return "bounded device-side wait gave up";
        default: return "unknown status";
    }
}

int fgl_ws_create(int device, fgl_ws** out) {
    if (!out || device < 0) return FGL_ERR_INVALID;
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device >= n_dev) {
        cudaGetLastError();
        return FGL_ERR_CUDA;
    }
    fgl_ws* ws = new (std::nothrow) fgl_ws();
    if (!ws) return FGL_ERR_NOMEM;
    ws->device = device;
    fgl::DeviceGuard guard(device);
    cudaError_t e = cudaDeviceGetAttribute(&ws->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaMalloc(&ws->status, 16 * sizeof(int32_t) + 512 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(ws->status, 0, 16 * sizeof(int32_t) + 512 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMallocHost(&ws->host_pinned, 64 * sizeof(int32_t));
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (ws->status) cudaFree(ws->status);
        delete ws;
        return FGL_ERR_CUDA;
    }
    *out = ws;
    return FGL_OK;
}

int fgl_ws_destroy(fgl_ws* ws) {
    if (!ws) return FGL_OK;
    {
        fgl::DeviceGuard guard(ws->device);
        if (ws->table) cudaFree(ws->table);
        if (ws->scratch) cudaFree(ws->scratch);
        if (ws->status) cudaFree(ws->status);
        if (ws->host_pinned) cudaFreeHost(ws->host_pinned);
    }
    delete ws;
    return FGL_OK;
}

int fgl_ws_reserve(fgl_ws* ws, int64_t table_slots, int64_t scratch_bytes) {
    if (!ws || table_slots < 0 || scratch_bytes < 0) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    fgl::DeviceGuard guard(ws->device);
    return fgl::ws_ensure(ws, table_slots, scratch_bytes);
}

const char* fgl_last_error(fgl_ws* ws) { return ws ? ws->last_error.c_str() : ""; }

int fgl_ws_check(fgl_ws* ws, void* stream) {
    if (!ws) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    fgl::DeviceGuard guard(ws->device);
    cudaStream_t st = (cudaStream_t)stream;
    FGL_CUDA_OK(ws, cudaMemcpyAsync(ws->host_pinned, ws->status, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    FGL_CUDA_OK(ws, cudaMemsetAsync(ws->status, 0, 2 * sizeof(int32_t), st));
    FGL_CUDA_OK(ws, cudaStreamSynchronize(st));
    const int code = ws->host_pinned[0];
    if (code != FGL_OK) {
        ws->last_error = std::string("device status: ") + fgl_status_str(code);
        ws->table_dirty = true;  // a failed launch may have left keys behind
    }
    return code;
}

int fgl_ws_status_peek(fgl_ws* ws, int32_t* host_dst, void* stream) {
    if (!ws || !host_dst) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    fgl::DeviceGuard guard(ws->device);
    FGL_CUDA_OK(ws, cudaMemcpyAsync(host_dst, ws->status, sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return FGL_OK;
}

int fgl_ws_time_next_launch(fgl_ws* ws, void* start_event, void* end_event) {
    if (!ws || !start_event != !end_event) return FGL_ERR_INVALID;
    std::lock_guard<std::mutex> lock(ws->mu);
    ws->time_start = (cudaEvent_t)start_event;
    ws->time_end = (cudaEvent_t)end_event;
    return FGL_OK;
}

}  // extern "C"
