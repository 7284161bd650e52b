// Ring transport on a private NCCL communicator: one grouped ncclSend + ncclRecv per hop on a stream owned
// by the transport, fenced to the caller's compute stream with events.  Replaces the reference's
// `DoubleBufRingComm.send_recv_packed` / `wait` (optimized_ring_flash_attn.py:163-188) without the per-call
// cost of a Python process-group round trip (tens of microseconds per hop, which is what bounds short shards).
//
// NCCL is not a link-time dependency: the symbols are taken from the libnccl.so.2 that the host process has
// already loaded (PyTorch's), or loaded on demand.
#include <dlfcn.h>
#include <string.h>

#include "common.h"

namespace {

struct NcclUniqueId { char internal[128]; };
typedef void* NcclComm;
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(NcclComm*, int, NcclUniqueId, int);
typedef int (*CommDestroyFn)(NcclComm);
typedef int (*SendFn)(const void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*RecvFn)(void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*GroupFn)();

struct NcclApi {
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  SendFn send = nullptr;
  RecvFn recv = nullptr;
  GroupFn group_start = nullptr;
  GroupFn group_end = nullptr;
  bool ok = false;
};

const NcclApi& nccl_api() {
  static NcclApi api = [] {
    NcclApi a;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return a;
    a.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
    a.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
    a.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
    a.send = reinterpret_cast<SendFn>(dlsym(h, "ncclSend"));
    a.recv = reinterpret_cast<RecvFn>(dlsym(h, "ncclRecv"));
    a.group_start = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupStart"));
    a.group_end = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupEnd"));
    a.ok = a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.send && a.recv && a.group_start && a.group_end;
    return a;
  }();
  return api;
}

constexpr int kDoneSlots = 8;
constexpr int kNcclChar = 0;  // ncclInt8 / ncclChar

struct RingComm {
  NcclComm comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_ready = nullptr;
  cudaEvent_t ev_done[kDoneSlots] = {};
  unsigned next_slot = 0;
};

}  // namespace

extern "C" int rfa_comm_unique_id(void* out128) {
  const NcclApi& api = nccl_api();
  if (!api.ok) return RFA_ERR_NCCL;
  if (!out128) return RFA_ERR_INVALID_ARG;
  NcclUniqueId id;
  if (api.get_unique_id(&id) != 0) return RFA_ERR_NCCL;
  memcpy(out128, &id, sizeof(id));
  return RFA_OK;
}

extern "C" int rfa_comm_init(const void* id128, int rank, int world, void** handle) {
  const NcclApi& api = nccl_api();
  if (!api.ok) return RFA_ERR_NCCL;
  if (!id128 || !handle || world < 2 || rank < 0 || rank >= world) return RFA_ERR_INVALID_ARG;
  RingComm* c = new RingComm();
  c->rank = rank;
  c->world = world;
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  bool ok = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < kDoneSlots; ++i)
    ok = cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    delete c;
    return RFA_ERR_CUDA;
  }
  if (api.comm_init_rank(&c->comm, world, id, rank) != 0) {
    delete c;
    return RFA_ERR_NCCL;
  }
  *handle = c;
  return RFA_OK;
}

extern "C" int rfa_comm_destroy(void* handle) {
  if (!handle) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  const NcclApi& api = nccl_api();
  if (c->comm && api.ok) api.comm_destroy(c->comm);
  if (c->stream) cudaStreamDestroy(c->stream);
  if (c->ev_ready) cudaEventDestroy(c->ev_ready);
  for (int i = 0; i < kDoneSlots; ++i)
    if (c->ev_done[i]) cudaEventDestroy(c->ev_done[i]);
  delete c;
  return RFA_OK;
}

extern "C" int rfa_ring_post(void* handle, const void* send, void* recv, size_t bytes, void* compute_stream) {
  const NcclApi& api = nccl_api();
  if (!handle || !send || !recv || bytes == 0 || send == recv) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  // everything enqueued so far on the compute stream (producer of `send`, last reader of `recv`) comes first
  if (cudaEventRecord(c->ev_ready, cs) != cudaSuccess || cudaStreamWaitEvent(c->stream, c->ev_ready, 0) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  const int next = (c->rank + 1) % c->world;
  const int prev = (c->rank + c->world - 1) % c->world;
  int rc = api.group_start();
  if (rc == 0) rc = api.send(send, bytes, kNcclChar, next, c->comm, c->stream);
  if (rc == 0) rc = api.recv(recv, bytes, kNcclChar, prev, c->comm, c->stream);
  const int rc_end = api.group_end();
  if (rc != 0 || rc_end != 0) return RFA_ERR_NCCL;
  const int slot = static_cast<int>(c->next_slot++ % kDoneSlots);
  if (cudaEventRecord(c->ev_done[slot], c->stream) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return slot;
}

extern "C" int rfa_ring_wait(void* handle, int slot, void* compute_stream) {
  if (!handle || slot < 0 || slot >= kDoneSlots) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  if (cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), c->ev_done[slot], 0) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return RFA_OK;
}
