// comm.cu — tensor-parallel collectives: NCCL over NVLink/NVSwitch, one rank per process.
// The reference is single-GPU (no counterpart).  NCCL is bound at run time with dlopen so that
// the library shares whichever libnccl the host process already uses and single-GPU callers
// need no NCCL at all.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <vector>

#include "common.cuh"
#include "comm.h"
#include "gemv.cuh"

namespace {

typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm_t;
enum { kNcclFloat32 = 7, kNcclSum = 0, kNcclSuccess = 0 };

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(nccl_uid*) = nullptr;
    int (*CommInitRank)(nccl_comm_t*, int, nccl_uid, int) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*CommGetAsyncError)(nccl_comm_t, int*) = nullptr;
};
NcclApi g_nccl;

int load_nccl() {
    if (g_nccl.lib) return ATLASX_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);          // already in the process?
    if (!h) { const char* p = getenv("ATLAS_NCCL_LIB"); if (p && *p) h = dlopen(p, RTLD_NOW | RTLD_GLOBAL); }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return atlasx_fail(ATLASX_ERR_COMM, "cannot load libnccl.so.2: %s", dlerror());
    g_nccl.GetUniqueId = (int (*)(nccl_uid*))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(nccl_comm_t*, int, nccl_uid, int))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (int (*)(nccl_comm_t))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce = (int (*)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t))dlsym(h, "ncclAllReduce");
    g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t))dlsym(h, "ncclAllGather");
    g_nccl.GetErrorString = (const char* (*)(int))dlsym(h, "ncclGetErrorString");
    g_nccl.CommGetAsyncError = (int (*)(nccl_comm_t, int*))dlsym(h, "ncclCommGetAsyncError");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.AllGather || !g_nccl.CommDestroy)
        return atlasx_fail(ATLASX_ERR_COMM, "libnccl is missing a required symbol");
    g_nccl.lib = h;
    return ATLASX_OK;
}
const char* nccl_err(int e) { return g_nccl.GetErrorString ? g_nccl.GetErrorString(e) : "nccl error"; }

}  // namespace

struct atlasx_comm {
    nccl_comm_t comm = nullptr;
    int rank = 0, world = 1;
    AxPeerMail mail; bool mail_ready = false, mail_failed = false;
    void* mail_local = nullptr;
};

void atlasx_comm_destroy(atlasx_ctx* ctx) {
    if (ctx && ctx->comm) {
        atlasx_comm* cm = ctx->comm;
        if (cm->mail_ready) {
            for (int p = 0; p < cm->world; p++)
                if (p != cm->rank && cm->mail.base[p]) cudaIpcCloseMemHandle(cm->mail.base[p]);
        }
        if (cm->mail_local) cudaFree(cm->mail_local);
        if (ctx->comm->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->comm->comm);
        delete ctx->comm;
        ctx->comm = nullptr;
    }
}

int ax_comm_world(const atlasx_ctx* ctx) { return ctx && ctx->comm ? ctx->comm->world : 1; }
int ax_comm_rank(const atlasx_ctx* ctx) { return ctx && ctx->comm ? ctx->comm->rank : 0; }

int ax_comm_allreduce_sum(atlasx_ctx* ctx, float* buf, size_t n) {
    if (!ctx->comm || ctx->comm->world == 1) return ATLASX_OK;
    const int e = g_nccl.AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->comm->comm, ctx->stream);
    if (e != kNcclSuccess) return atlasx_fail(ATLASX_ERR_COMM, "ncclAllReduce: %s", nccl_err(e));
    return ATLASX_OK;
}
int ax_comm_allgather(atlasx_ctx* ctx, const float* send, float* recv, size_t n_each) {
    if (!ctx->comm || ctx->comm->world == 1) {
        if (send != recv) AX_CUDA(cudaMemcpyAsync(recv, send, n_each * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        return ATLASX_OK;
    }
    const int e = g_nccl.AllGather(send, recv, n_each, kNcclFloat32, ctx->comm->comm, ctx->stream);
    if (e != kNcclSuccess) return atlasx_fail(ATLASX_ERR_COMM, "ncclAllGather: %s", nccl_err(e));
    return ATLASX_OK;
}

int ax_comm_stream_sync(atlasx_ctx* ctx) {
    atlasx_comm* cm = ctx->comm;
    if (!cm || cm->world == 1) { AX_CUDA(cudaStreamSynchronize(ctx->stream)); return ATLASX_OK; }
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spin = 0;; spin++) {
        const cudaError_t q = cudaStreamQuery(ctx->stream);
        if (q == cudaSuccess) return ATLASX_OK;
        if (q != cudaErrorNotReady) return atlasx_fail(ATLASX_ERR_CUDA, "stream failed: %s", cudaGetErrorString(q));
        if ((spin & 63) != 63) continue;                     // the checks below every 64th poll
        if (g_nccl.CommGetAsyncError) {
            int async_err = 0;
            const int e = g_nccl.CommGetAsyncError(cm->comm, &async_err);
            if (e != kNcclSuccess || async_err != kNcclSuccess)
                return atlasx_fail(ATLASX_ERR_COMM, "NCCL reported an asynchronous error: %s", nccl_err(e != kNcclSuccess ? e : async_err));
        }
        const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > ctx->tune.comm_timeout_ms)
            return atlasx_fail(ATLASX_ERR_TIMEOUT, "the tensor-parallel step did not complete within %d ms (a rank that never joined?); "
                                                   "the work is still queued: destroy the context", ctx->tune.comm_timeout_ms);
    }
}

// The mailboxes are exchanged as CUDA IPC handles through an NCCL all-gather of raw bytes; every
// rank must call this at the same point of its program.  A failure to map a peer (no peer access,
// different IPC namespace) is not an error: all ranks learn of it through a second all-gather and
// all of them keep the NCCL path.
int ax_comm_peer_setup(atlasx_ctx* ctx, int d, const AxPeerMail** out) {
    *out = nullptr;
    atlasx_comm* cm = ctx->comm;
    if (!cm || cm->world == 1 || cm->world > kMaxPeers) return ATLASX_OK;
    if (cm->mail_ready) {
        if (cm->mail.d < d) return atlasx_fail(ATLASX_ERR_STATE, "peer mailboxes were sized for %d floats, %d asked", cm->mail.d, d);
        *out = &cm->mail;
        return ATLASX_OK;
    }
    if (cm->mail_failed) return ATLASX_OK;
    if (!ctx->tune.peer_allreduce) { cm->mail_failed = true; return ATLASX_OK; }
    const int W = cm->world;
    const size_t mail_bytes = (((size_t)2 * W * d * sizeof(uint2)) + 255) / 256 * 256;
    const size_t total = mail_bytes + 512;                  // + the use counter, + the selection slots
    AX_CUDA(cudaMalloc(&cm->mail_local, total));
    AX_CUDA(cudaMemset(cm->mail_local, 0, total));
    AX_CUDA(cudaDeviceSynchronize());

    struct Wire { cudaIpcMemHandle_t h; int ok; int pad[15]; };          // 128 bytes
    static_assert(sizeof(Wire) == 128, "wire record size");
    Wire mine = {}; mine.ok = 1;
    if (cudaIpcGetMemHandle(&mine.h, cm->mail_local) != cudaSuccess) { cudaGetLastError(); mine.ok = 0; }
    Wire* dev = nullptr;
    AX_CUDA(cudaMalloc((void**)&dev, sizeof(Wire) * (W + 1)));
    std::vector<Wire> all((size_t)W);
    auto gather = [&](const Wire& w) -> int {
        AX_CUDA(cudaMemcpyAsync(dev + W, &w, sizeof(Wire), cudaMemcpyHostToDevice, ctx->stream));
        const int e = g_nccl.AllGather(dev + W, dev, sizeof(Wire), /*ncclInt8*/ 0, cm->comm, ctx->stream);
        if (e != kNcclSuccess) return atlasx_fail(ATLASX_ERR_COMM, "ncclAllGather: %s", nccl_err(e));
        AX_CUDA(cudaMemcpyAsync(all.data(), dev, sizeof(Wire) * W, cudaMemcpyDeviceToHost, ctx->stream));
        AX_CUDA(cudaStreamSynchronize(ctx->stream));
        return ATLASX_OK;
    };
    int rc = gather(mine);
    if (rc) { cudaFree(dev); return rc; }
    bool ok = true;
    for (int p = 0; p < W; p++) ok = ok && all[p].ok;
    AxPeerMail mail;
    mail.world = W; mail.rank = cm->rank; mail.d = d;
    mail.useq = reinterpret_cast<unsigned*>((uint8_t*)cm->mail_local + mail_bytes);
    if (ok) {
        for (int p = 0; p < W && ok; p++) {
            if (p == cm->rank) { mail.base[p] = (uint2*)cm->mail_local; continue; }
            void* ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, all[p].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = false; }
            mail.base[p] = (uint2*)ptr;
        }
        for (int p = 0; p < W && ok; p++) mail.sel_base[p] = reinterpret_cast<uint4*>((uint8_t*)mail.base[p] + mail_bytes + 256);
    }
    Wire mapped = {}; mapped.ok = ok ? 1 : 0;
    rc = gather(mapped);                                    // second exchange: did every rank map every peer?
    cudaFree(dev);
    if (rc) return rc;
    for (int p = 0; p < W; p++) ok = ok && all[p].ok;
    if (!ok) {
        for (int p = 0; p < W; p++) if (p != cm->rank && mail.base[p]) cudaIpcCloseMemHandle(mail.base[p]);
        cudaFree(cm->mail_local); cm->mail_local = nullptr;
        cm->mail_failed = true;
        return ATLASX_OK;
    }
    cm->mail = mail; cm->mail_ready = true;
    *out = &cm->mail;
    return ATLASX_OK;
}

extern "C" int atlasx_comm_unique_id(void* id128_out) {
    AX_ARG(id128_out, "id buffer is null");
    int rc = load_nccl(); if (rc) return rc;
    nccl_uid id;
    const int e = g_nccl.GetUniqueId(&id);
    if (e != kNcclSuccess) return atlasx_fail(ATLASX_ERR_COMM, "ncclGetUniqueId: %s", nccl_err(e));
    memcpy(id128_out, &id, sizeof(id));
    return ATLASX_OK;
}
extern "C" int atlasx_comm_init(atlasx_ctx* ctx, const void* id128, int rank, int world) {
    AX_ARG(ctx && id128, "null argument");
    AX_ARG(world >= 1 && rank >= 0 && rank < world, "rank/world out of range");
    AX_ARG(!ctx->comm, "communicator already initialised");
    int rc = load_nccl(); if (rc) return rc;
    AX_CUDA(cudaSetDevice(ctx->device));
    nccl_uid id; memcpy(&id, id128, sizeof(id));
    atlasx_comm* cm = new atlasx_comm();
    cm->rank = rank; cm->world = world;
    const int e = g_nccl.CommInitRank(&cm->comm, world, id, rank);
    if (e != kNcclSuccess) { delete cm; return atlasx_fail(ATLASX_ERR_COMM, "ncclCommInitRank: %s", nccl_err(e)); }
    ctx->comm = cm;
    return ATLASX_OK;
}
extern "C" int atlasx_comm_world(const atlasx_ctx* ctx) { return ax_comm_world(ctx); }

// Self-test of the bounded device-side waits: the mailbox reduction is launched on a zeroed part
// whose sequence words nothing will ever set.  The kernel must give up after its limit (2 s), set
// the context's error word and return — the context stays usable.  *code receives the word (3).
// keep != 0 leaves the word set (the state a real expiry leaves behind) for the caller to clear
// with atlasx_ctx_poll_device_error.
extern "C" int atlasx_comm_selftest_wait_expiry(atlasx_ctx* ctx, int* code, int keep) {
    AX_ARG(ctx && code, "null argument");
    const int d = 512;
    uint2* part = nullptr; float* out = nullptr; unsigned* epoch = nullptr;
    AX_CUDA(cudaMalloc((void**)&part, d * sizeof(uint2)));
    AX_CUDA(cudaMalloc((void**)&out, d * sizeof(float)));
    AX_CUDA(cudaMalloc((void**)&epoch, sizeof(unsigned)));
    AX_CUDA(cudaMemsetAsync(part, 0, d * sizeof(uint2), ctx->stream));
    AX_CUDA(cudaMemsetAsync(epoch, 0, sizeof(unsigned), ctx->stream));
    int rc = ax_mail_reduce_launch(ctx, part, 1, (size_t)d, d, epoch, 1u, 7u, out, false);   // waits for sequence 7
    if (!rc) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = atlasx_fail(ATLASX_ERR_CUDA, "self-test kernel failed: %s", cudaGetErrorString(e));
    }
    *code = 0;
    if (!rc && keep) {                                    // report the word and leave it set
        cudaError_t e = cudaMemcpyAsync(ctx->host_pin, ctx->dev_error, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = atlasx_fail(ATLASX_ERR_CUDA, "reading the error word failed: %s", cudaGetErrorString(e));
        else *code = ctx->host_pin[0];
    } else if (!rc) {
        atlasx_ctx_poll_device_error(ctx, code);          // returns ATLASX_ERR_TIMEOUT when the word is set: expected here
        rc = ATLASX_OK;
    }
    cudaFree(part); cudaFree(out); cudaFree(epoch);
    return rc;
}
extern "C" int atlasx_comm_allreduce(atlasx_ctx* ctx, float* buf, int n) {
    AX_ARG(ctx && buf && n >= 0, "bad argument");
    return ax_comm_allreduce_sum(ctx, buf, (size_t)n);
}
