// C ABI of include/xs_moe_comm.h: NCCL resolved at run time (no link-time dependency), plus stream / event helpers.
// Included at the end of xs_moe_api.cu (one translation unit: shares fail() and the error string).
#include <dlfcn.h>
#include <nccl.h>

#include "xs_moe_comm.h"

namespace {

struct NcclApi {
    bool ok = false;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclSend) Send = nullptr;
    decltype(&ncclRecv) Recv = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
};

const NcclApi &nccl_api()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h)
            h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h)
            return;
        bool all = true;
        auto get = [&](auto &fn, const char *name) {
            fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
            all = all && fn != nullptr;
        };
        get(api.GetUniqueId, "ncclGetUniqueId");
        get(api.CommInitRank, "ncclCommInitRank");
        get(api.CommDestroy, "ncclCommDestroy");
        get(api.CommAbort, "ncclCommAbort");
        get(api.CommGetAsyncError, "ncclCommGetAsyncError");
        get(api.GetErrorString, "ncclGetErrorString");
        get(api.AllGather, "ncclAllGather");
        get(api.AllReduce, "ncclAllReduce");
        get(api.Send, "ncclSend");
        get(api.Recv, "ncclRecv");
        get(api.GroupStart, "ncclGroupStart");
        get(api.GroupEnd, "ncclGroupEnd");
        api.ok = all;
    });
    return api;
}

#define XS_NCCL(call)                                                                                             \
    do {                                                                                                          \
        ncclResult_t r__ = (call);                                                                                \
        if (r__ != ncclSuccess)                                                                                   \
            return fail(XS_MOE_ERR_CUDA, "NCCL error: %s (%s) at %s:%d", nccl_api().GetErrorString(r__), #call, \
                        __FILE__, __LINE__);                                                                      \
    } while (0)

int need_nccl()
{
    if (!nccl_api().ok)
        return fail(XS_MOE_ERR_UNSUPPORTED, "NCCL error: libnccl.so.2 could not be loaded");
    return 0;
}

static_assert(sizeof(ncclUniqueId) == XS_MOE_COMM_ID_BYTES, "NCCL unique id size");

} // namespace

extern "C" {

int xs_moe_comm_available(void)
{
    return need_nccl();
}

int xs_moe_comm_unique_id(uint8_t *id)
{
    if (int rc = need_nccl())
        return rc;
    if (!id)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    ncclUniqueId u;
    XS_NCCL(nccl_api().GetUniqueId(&u));
    memcpy(id, &u, sizeof(u));
    return 0;
}

int xs_moe_comm_create(void **comm, const uint8_t *id, int32_t rank, int32_t ranks)
{
    if (int rc = need_nccl())
        return rc;
    if (!comm || !id || ranks < 1 || rank < 0 || rank >= ranks)
        return fail(XS_MOE_ERR_INVALID_ARG, "bad communicator arguments (rank %d of %d)", rank, ranks);
    ncclUniqueId u;
    memcpy(&u, id, sizeof(u));
    ncclComm_t c = nullptr;
    XS_NCCL(nccl_api().CommInitRank(&c, ranks, u, rank));
    *comm = c;
    return 0;
}

int xs_moe_comm_destroy(void *comm)
{
    if (!comm)
        return 0;
    if (int rc = need_nccl())
        return rc;
    XS_NCCL(nccl_api().CommDestroy(static_cast<ncclComm_t>(comm)));
    return 0;
}

int xs_moe_comm_abort(void *comm)
{
    if (!comm)
        return 0;
    if (int rc = need_nccl())
        return rc;
    XS_NCCL(nccl_api().CommAbort(static_cast<ncclComm_t>(comm)));
    return 0;
}

int xs_moe_comm_async_error(void *comm, int32_t *code)
{
    if (int rc = need_nccl())
        return rc;
    if (!comm || !code)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    ncclResult_t r = ncclSuccess;
    XS_NCCL(nccl_api().CommGetAsyncError(static_cast<ncclComm_t>(comm), &r));
    *code = static_cast<int32_t>(r);
    if (r != ncclSuccess && r != ncclInProgress)
        fail(XS_MOE_ERR_CUDA, "NCCL error: %s (asynchronous)", nccl_api().GetErrorString(r));
    return 0;
}

int xs_moe_comm_all_gather(void *comm, const void *send, void *recv, size_t bytes, void *stream)
{
    if (int rc = need_nccl())
        return rc;
    if (!comm || !send || !recv)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    XS_NCCL(nccl_api().AllGather(send, recv, bytes, ncclInt8, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_comm_barrier(void *comm, int32_t *token, void *stream)
{
    if (int rc = need_nccl())
        return rc;
    if (!comm || !token)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    XS_NCCL(nccl_api().AllReduce(token, token, 1, ncclInt32, ncclSum, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_comm_all_to_all_v(void *comm, int32_t ranks, const void *send, const size_t *send_bytes, const size_t *send_offset, void *recv,
                             const size_t *recv_bytes, const size_t *recv_offset, void *stream)
{
    if (int rc = need_nccl())
        return rc;
    if (!comm || !send_bytes || !send_offset || !recv_bytes || !recv_offset || ranks < 1)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    const NcclApi &n = nccl_api();
    ncclComm_t c = static_cast<ncclComm_t>(comm);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    XS_NCCL(n.GroupStart());
    ncclResult_t first = ncclSuccess;
    for (int r = 0; r < ranks; r++) {
        ncclResult_t a = ncclSuccess, b = ncclSuccess;
        if (send_bytes[r])
            a = n.Send(static_cast<const uint8_t *>(send) + send_offset[r], send_bytes[r], ncclInt8, r, c, st);
        if (recv_bytes[r])
            b = n.Recv(static_cast<uint8_t *>(recv) + recv_offset[r], recv_bytes[r], ncclInt8, r, c, st);
        if (first == ncclSuccess)
            first = a != ncclSuccess ? a : b;
    }
    ncclResult_t end = n.GroupEnd(); // always close the group, also after a failed post
    XS_NCCL(first);
    XS_NCCL(end);
    return 0;
}

int xs_moe_stream_create(void **stream)
{
    if (!stream)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    cudaStream_t s = nullptr;
    XS_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return 0;
}

int xs_moe_stream_destroy(void *stream)
{
    if (stream)
        XS_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_event_create(void **event)
{
    if (!event)
        return fail(XS_MOE_ERR_INVALID_ARG, "null pointer");
    cudaEvent_t e = nullptr;
    XS_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    *event = e;
    return 0;
}

int xs_moe_event_destroy(void *event)
{
    if (event)
        XS_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    return 0;
}

int xs_moe_event_record(void *event, void *stream)
{
    XS_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_stream_wait_event(void *stream, void *event)
{
    XS_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
    return 0;
}

int xs_moe_memset_async(void *ptr, int32_t value, size_t bytes, void *stream)
{
    if (bytes)
        XS_CUDA(cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream)));
    return 0;
}

int xs_moe_enable_peer_access(int32_t peer)
{
    int dev = 0;
    XS_CUDA(cudaGetDevice(&dev));
    if (peer == dev)
        return 0;
    int can = 0;
    XS_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer));
    if (!can)
        return fail(XS_MOE_ERR_DEVICE, "device %d cannot map the memory of device %d", dev, peer);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return 0;
    }
    XS_CUDA(e);
    return 0;
}

} // extern "C"
