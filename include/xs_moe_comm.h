/* Collectives and stream plumbing for the expert-parallel host of the MoE layer: a thin C ABI over NCCL and the CUDA
 * runtime so that host code compiled without any CUDA or NCCL header (the reference keeps its host C++ CUDA-free the
 * same way, xstar_cpp/include/cuda/cuda_allocator.h:1-30) can drive one GPU per thread or per process.
 *
 * The reference has no collective layer: its multi-GPU rows (README.md:27-31) are roadmap entries.  What the expert-
 * parallel step needs is small -- an all-gather of per-expert row counts, a barrier between peer stores and their first
 * reader, and an all-to-all of rows for boxes without peer access -- and maps one to one onto ncclAllGather, a one-element
 * ncclAllReduce and grouped ncclSend / ncclRecv.
 *
 * NCCL is loaded at run time (libnccl.so.2, by name): the kernel library has no link-time dependency on it, and a process
 * that already holds an NCCL (PyTorch's) shares that copy.  Every call returns an XS_MOE_* status; xs_moe_last_error()
 * carries NCCL's message. */
#ifndef XS_MOE_COMM_H
#define XS_MOE_COMM_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define XS_MOE_COMM_ID_BYTES 128

/* 0 when NCCL could be loaded and has every entry point used here. */
int xs_moe_comm_available(void);
/* ncclGetUniqueId: call on one rank, hand the bytes to the others (a host-side broadcast of the caller's choosing). */
int xs_moe_comm_unique_id(uint8_t id[XS_MOE_COMM_ID_BYTES]);
/* ncclCommInitRank on the calling thread's current device.  Collective over the `ranks` callers. */
int xs_moe_comm_create(void **comm, const uint8_t id[XS_MOE_COMM_ID_BYTES], int32_t rank, int32_t ranks);
/* ncclCommDestroy (collective-safe shutdown) / ncclCommAbort (after a peer was lost; never blocks on the peer). */
int xs_moe_comm_destroy(void *comm);
int xs_moe_comm_abort(void *comm);
/* ncclCommGetAsyncError: *code = 0 while the communicator is healthy. */
int xs_moe_comm_async_error(void *comm, int32_t *code);

/* recv(ranks * bytes_per_rank) = concatenation over ranks of send(bytes_per_rank).  ncclAllGather of bytes. */
int xs_moe_comm_all_gather(void *comm, const void *send_dev, void *recv_dev, size_t bytes_per_rank, void *stream);
/* One-element int32 sum all-reduce on `token_dev`: orders everything the ranks enqueued before it on their streams
 * (peer stores among them) before everything they enqueue after it. */
int xs_moe_comm_barrier(void *comm, int32_t *token_dev, void *stream);
/* Rows to and from every rank in one group call: send_bytes[r] bytes from send_dev + send_offset[r] go to rank r,
 * recv_bytes[r] bytes from rank r land at recv_dev + recv_offset[r].  Host arrays of `ranks` entries (the transport for
 * boxes where peer mappings cannot be made). */
int xs_moe_comm_all_to_all_v(void *comm, int32_t ranks, const void *send_dev, const size_t *send_bytes, const size_t *send_offset,
                             void *recv_dev, const size_t *recv_bytes, const size_t *recv_offset, void *stream);

/* Streams and events for host code that overlaps the always-on expert with the exchange. */
int xs_moe_stream_create(void **stream);
int xs_moe_stream_destroy(void *stream);
int xs_moe_event_create(void **event);
int xs_moe_event_destroy(void *event);
int xs_moe_event_record(void *event, void *stream);
int xs_moe_stream_wait_event(void *stream, void *event);
int xs_moe_memset_async(void *ptr_dev, int32_t byte_value, size_t bytes, void *stream);
/* cudaDeviceEnablePeerAccess from the current device to `peer_device` (already enabled counts as success);
 * XS_MOE_ERR_DEVICE when the pair cannot be mapped. */
int xs_moe_enable_peer_access(int32_t peer_device);

#ifdef __cplusplus
}
#endif
#endif
