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
  cudaEvent_t ev_begin[kDoneSlots] = {};  // timing mode only
  bool timing = false;
  unsigned next_slot = 0;
  unsigned posted = 0, waited = 0;  // a slot's event is reused after kDoneSlots posts: bound what is outstanding
};

// Releases everything the handle owns (also the partly built handle of a failed rfa_comm_init).
void destroy_ring(RingComm* c) {
  const NcclApi& api = nccl_api();
  if (c->comm && api.ok) api.comm_destroy(c->comm);
  if (c->stream) cudaStreamDestroy(c->stream);
  if (c->ev_ready) cudaEventDestroy(c->ev_ready);
  for (int i = 0; i < kDoneSlots; ++i) {
    if (c->ev_done[i]) cudaEventDestroy(c->ev_done[i]);
    if (c->ev_begin[i]) cudaEventDestroy(c->ev_begin[i]);
  }
  cudaGetLastError();
  delete c;
}

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
  // Highest stream priority: while a hop kernel keeps every SM busy with CTAs that fill its shared memory, the
  // blocks of NCCL's send/recv kernel can only start on an SM between two hop CTAs, and the block scheduler serves
  // the higher-priority stream first.  At default priority the transfer queues behind all pending hop CTAs.
  int prio_lo = 0, prio_hi = 0;
  bool ok = cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi) == cudaSuccess;
  ok = ok && cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, prio_hi) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < kDoneSlots; ++i)
    ok = cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    destroy_ring(c);
    return RFA_ERR_CUDA;
  }
  if (api.comm_init_rank(&c->comm, world, id, rank) != 0) {
    c->comm = nullptr;
    destroy_ring(c);
    return RFA_ERR_NCCL;
  }
  *handle = c;
  return RFA_OK;
}

extern "C" int rfa_comm_destroy(void* handle) {
  if (!handle) return RFA_ERR_INVALID_ARG;
  destroy_ring(static_cast<RingComm*>(handle));
  return RFA_OK;
}

extern "C" int rfa_ring_post(void* handle, const void* send, void* recv, size_t bytes, void* compute_stream) {
  const NcclApi& api = nccl_api();
  if (!handle || !send || !recv || bytes == 0 || send == recv) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  if (c->posted - c->waited >= static_cast<unsigned>(kDoneSlots)) return RFA_ERR_INVALID_ARG;  // slot still in use
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  // everything enqueued so far on the compute stream (producer of `send`, last reader of `recv`) comes first
  if (cudaEventRecord(c->ev_ready, cs) != cudaSuccess || cudaStreamWaitEvent(c->stream, c->ev_ready, 0) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  const int next = (c->rank + 1) % c->world;
  const int prev = (c->rank + c->world - 1) % c->world;
  const int slot = static_cast<int>(c->next_slot % kDoneSlots);
  if (c->timing && cudaEventRecord(c->ev_begin[slot], c->stream) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  int rc = api.group_start();
  if (rc == 0) rc = api.send(send, bytes, kNcclChar, next, c->comm, c->stream);
  if (rc == 0) rc = api.recv(recv, bytes, kNcclChar, prev, c->comm, c->stream);
  const int rc_end = api.group_end();
  if (rc != 0 || rc_end != 0) return RFA_ERR_NCCL;
  if (cudaEventRecord(c->ev_done[slot], c->stream) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  ++c->next_slot;
  ++c->posted;
  return slot;
}

extern "C" int rfa_ring_wait(void* handle, int slot, void* compute_stream) {
  if (!handle || slot < 0 || slot >= kDoneSlots) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  if (c->waited == c->posted) return RFA_ERR_INVALID_ARG;  // nothing outstanding
  if (cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), c->ev_done[slot], 0) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  ++c->waited;
  return RFA_OK;
}

// Diagnostics (declared in rfa_b200_debug.h): with timing on, every post is bracketed by two timing events on the
// transport stream and rfa_debug_ring_elapsed returns the device time of the transfer in that slot.
extern "C" int rfa_debug_ring_timing(void* handle, int on) {
  if (!handle) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  if (c->posted != c->waited) return RFA_ERR_INVALID_ARG;  // switch only while nothing is in flight
  for (int i = 0; i < kDoneSlots; ++i) {
    if (c->ev_done[i]) cudaEventDestroy(c->ev_done[i]);
    if (c->ev_begin[i]) cudaEventDestroy(c->ev_begin[i]);
    c->ev_done[i] = c->ev_begin[i] = nullptr;
    const unsigned flags = on ? cudaEventDefault : cudaEventDisableTiming;
    bool ok = cudaEventCreateWithFlags(&c->ev_done[i], flags) == cudaSuccess;
    if (ok && on) ok = cudaEventCreateWithFlags(&c->ev_begin[i], cudaEventDefault) == cudaSuccess;
    if (!ok) { cudaGetLastError(); return RFA_ERR_CUDA; }
  }
  c->timing = on != 0;
  return RFA_OK;
}

extern "C" int rfa_debug_ring_elapsed(void* handle, int slot, float* ms) {
  if (!handle || !ms || slot < 0 || slot >= kDoneSlots) return RFA_ERR_INVALID_ARG;
  RingComm* c = static_cast<RingComm*>(handle);
  if (!c->timing || !c->ev_begin[slot]) return RFA_ERR_INVALID_ARG;
  if (cudaEventElapsedTime(ms, c->ev_begin[slot], c->ev_done[slot]) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return RFA_OK;
}
