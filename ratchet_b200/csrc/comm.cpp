// N-sharded prefill support: a small NCCL shim, CUDA IPC peer mapping and weight-shard packing.
// The reference is single-device ("Ordinal should always be 0", crates/ratchet-core/src/gpu/device.rs:15-16),
// so nothing here has a counterpart in it.  One process per GPU: the processes exchange the
// 128-byte NCCL id and the 64-byte IPC handles through whatever control plane they already have
// (torch.distributed in this repository's benchmark and tests).
//
// NCCL is looked up with dlopen at first use, so the library loads (and the single-GPU path runs)
// on a machine without NCCL, and a process that already holds a copy of NCCL (PyTorch's) shares it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "ratchet_b200.h"
#include "spec.hpp"

namespace rt {
Status dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int *n);
}
using namespace rt;

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};

NcclApi *nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.error = std::string("NCCL not found: ") + (dlerror() ? dlerror() : "dlopen failed");
            return;
        }
#define LOAD(field, sym)                                                              \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym));         \
    if (!api.field) api.error = std::string("NCCL symbol missing: ") + sym;
        LOAD(GetUniqueId, "ncclGetUniqueId")
        LOAD(CommInitRankConfig, "ncclCommInitRankConfig")
        LOAD(CommGetAsyncError, "ncclCommGetAsyncError")
        LOAD(CommAbort, "ncclCommAbort")
        LOAD(CommDestroy, "ncclCommDestroy")
        LOAD(AllGather, "ncclAllGather")
        LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    });
    return &api;
}

} // namespace

struct rt_comm {
    ncclComm_t comm = nullptr;
    int n_ranks = 0, rank = 0, ordinal = 0;
    cudaStream_t stream = nullptr;
};

extern "C" {

rt_status rt_comm_unique_id(void *id) {
    if (!id) return fail(RT_ERR_ARG, "rt_comm_unique_id: null argument");
    NcclApi *n = nccl();
    if (!n->error.empty()) return fail(RT_ERR_COMM, n->error);
    static_assert(sizeof(ncclUniqueId) == RT_COMM_ID_BYTES, "NCCL id size");
    ncclUniqueId uid;
    ncclResult_t r = n->GetUniqueId(&uid);
    if (r != ncclSuccess) return fail(RT_ERR_COMM, std::string("ncclGetUniqueId: ") + n->GetErrorString(r));
    std::memcpy(id, &uid, sizeof(uid));
    return RT_OK;
}

// Joins the communicator without blocking and polls until every rank has joined or `timeout_ms`
// has passed; a rank that never shows up therefore costs a bounded wait and RT_ERR_COMM_TIMEOUT,
// not a hang.
rt_status rt_comm_init_rank(rt_device *dev, int32_t n_ranks, int32_t rank, const void *id, int32_t timeout_ms, rt_comm **comm) {
    if (!dev || !id || !comm || n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(RT_ERR_ARG, "rt_comm_init_rank: bad argument");
    NcclApi *n = nccl();
    if (!n->error.empty()) return fail(RT_ERR_COMM, n->error);
    cudaError_t ce = cudaSetDevice(rt_device_ordinal(dev));
    if (ce != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(ce));
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    ncclComm_t c = nullptr;
    ncclResult_t r = n->CommInitRankConfig(&c, n_ranks, uid, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) return fail(RT_ERR_COMM, std::string("ncclCommInitRankConfig: ") + n->GetErrorString(r));
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : 60000);
    ncclResult_t state = ncclInProgress;
    while (true) {
        r = n->CommGetAsyncError(c, &state);
        if (r != ncclSuccess) state = r;
        if (state != ncclInProgress) break;
        if (std::chrono::steady_clock::now() > deadline) {
            n->CommAbort(c);
            return fail(RT_ERR_COMM_TIMEOUT, "rt_comm_init_rank: not every rank joined within " + std::to_string(timeout_ms) + " ms");
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    if (state != ncclSuccess) {
        n->CommAbort(c);
        return fail(RT_ERR_COMM, std::string("NCCL communicator: ") + n->GetErrorString(state));
    }
    rt_comm *out = new rt_comm();
    out->comm = c;
    out->n_ranks = n_ranks;
    out->rank = rank;
    out->ordinal = rt_device_ordinal(dev);
    out->stream = (cudaStream_t)rt_device_stream(dev);
    *comm = out;
    return RT_OK;
}

// recv holds n_ranks chunks of bytes_per_rank; chunk r is rank r's send buffer.  Asynchronous on `stream`.
rt_status rt_comm_all_gather(rt_comm *comm, const void *send, void *recv, uint64_t bytes_per_rank, void *stream) {
    if (!comm || !send || !recv) return fail(RT_ERR_ARG, "rt_comm_all_gather: null argument");
    NcclApi *n = nccl();
    cudaError_t ce = cudaSetDevice(comm->ordinal);
    if (ce != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(ce));
    cudaStream_t st = stream ? (cudaStream_t)stream : comm->stream;
    ncclResult_t r = n->AllGather(send, recv, bytes_per_rank, ncclUint8, comm->comm, st);
    if (r == ncclInProgress) {
        // the communicator is non-blocking: wait (bounded) for the enqueue itself to finish
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30);
        ncclResult_t state = ncclInProgress;
        while (state == ncclInProgress && std::chrono::steady_clock::now() < deadline) {
            if (n->CommGetAsyncError(comm->comm, &state) != ncclSuccess) break;
            if (state == ncclInProgress) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
        r = state;
        if (r == ncclInProgress) return fail(RT_ERR_COMM_TIMEOUT, "ncclAllGather did not enqueue within 30 s");
    }
    if (r != ncclSuccess) return fail(RT_ERR_COMM, std::string("ncclAllGather: ") + n->GetErrorString(r));
    return RT_OK;
}

rt_status rt_comm_destroy(rt_comm *comm) {
    if (!comm) return RT_OK;
    NcclApi *n = nccl();
    cudaSetDevice(comm->ordinal);
    if (comm->comm) n->CommDestroy(comm->comm);
    delete comm;
    return RT_OK;
}

/* ---- peer mapping */

rt_status rt_ipc_export(rt_buffer *buf, void *handle) {
    if (!buf || !handle) return fail(RT_ERR_ARG, "rt_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == RT_IPC_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, rt_buffer_ptr(buf));
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    std::memcpy(handle, &h, sizeof(h));
    return RT_OK;
}

rt_status rt_ipc_open(rt_device *dev, const void *handle, void **ptr) {
    if (!dev || !handle || !ptr) return fail(RT_ERR_ARG, "rt_ipc_open: null argument");
    cudaError_t e = cudaSetDevice(rt_device_ordinal(dev));
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
    return RT_OK;
}

rt_status rt_ipc_close(rt_device *dev, void *ptr) {
    if (!dev || !ptr) return RT_OK;
    cudaSetDevice(rt_device_ordinal(dev));
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("cudaIpcCloseMemHandle: ") + cudaGetErrorString(e));
    return RT_OK;
}

/* ---- weight shards */

// Rows [r0, r1) of a [rows][k] tensor, repacked in the dtype's own layout (for Q8_0: the rows' codes,
// padding, the rows' scales, padding), so that a shard is an ordinary tensor of shape [r1-r0][k].
rt_status rt_shard_rows(rt_dtype dt, const void *src, uint64_t rows, uint64_t k, uint64_t r0, uint64_t r1, void *dst) {
    if (!src || !dst || r0 > r1 || r1 > rows || !dtype_valid(dt)) return fail(RT_ERR_ARG, "rt_shard_rows: bad argument");
    rt_segment full[2], part[2];
    int nf = 0, np = 0;
    Status st = dtype_segments(dt, rows * k, full, &nf);
    if (st.ok()) st = dtype_segments(dt, (r1 - r0) * k, part, &np);
    if (!st.ok()) return fail(st);
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    std::memset(d, 0, part[np - 1].offset + part[np - 1].size);
    const uint64_t n = (r1 - r0) * k;
    switch (dt) {
    case RT_Q8_0H:
    case RT_Q8_0F: {
        if (k % 32) return fail(RT_ERR_SHAPE, "Q8_0 rows hold a multiple of 32 values");
        const uint64_t sb = dt == RT_Q8_0H ? 2 : 4;
        std::memcpy(d, s + r0 * k, n);
        std::memcpy(d + part[1].offset, s + full[1].offset + r0 * (k / 32) * sb, n / 32 * sb);
        break;
    }
    case RT_Q4_K:
        if (k % 256) return fail(RT_ERR_SHAPE, "Q4_K rows hold a multiple of 256 values");
        std::memcpy(d, s + r0 * (k / 256) * 144, n / 256 * 144);
        break;
    default:
        std::memcpy(d, s + r0 * k * dtype_size(dt), n * dtype_size(dt));
    }
    return RT_OK;
}

} // extern "C"
