// Ring transport over peer memory: the copy engines move the packed buffers across NVLink, no SM is involved.
//
// Same role as the reference's `DoubleBufRingComm.send_recv_packed` / `wait`
// (optimized_ring_flash_attn.py:163-188) and as the NCCL transport in comm.cu, for ranks that are processes on one
// node whose GPUs can map each other's memory.  A grouped ncclSend/ncclRecv needs thread blocks on both GPUs at the
// same time, and a hop kernel keeps every SM occupied with CTAs that fill its shared memory; on an 8-GPU ring that
// left the transfers at 50-85 GB/s.  Here a transfer is one cudaMemcpyAsync from the previous rank's buffer (mapped
// through CUDA IPC) into the local one, ordered by 32-bit sequence flags that the neighbours write into each other's
// memory and that the streams wait on with stream memory operations -- no kernel spins, nothing runs on an SM.
//
// The ring buffers are allocated by the handle (cudaMalloc, so that they can be exported) in the same order on
// every rank: buffer i of one rank corresponds to buffer i of its neighbours.  Per post with sequence number n:
//   transport stream:  wait "compute stream is done with send/recv buffers" (event)
//                      next.flags[kPosted] = n           (4-byte copy into the next rank's memory)
//                      wait  flags[kPosted] >= n          (the previous rank's buffer is ready)
//                      recv <- prev.buffer[index of send]  (the transfer: peer read by the copy engine)
//                      prev.flags[kPulled] = n           (the previous rank may reuse its buffer)
//                      wait  flags[kPulled] >= n          (the next rank has my data: my send buffer is free)
//                      record done event
// Every rank writes before it waits, so the waits cannot form a cycle.  A peer that never posts leaves the stream
// waiting: like an NCCL ring with a missing rank, that ends only with the process.
#include <string.h>
#include <time.h>

#include "common.h"

namespace {

constexpr int kDoneSlots = 8;
constexpr int kMaxBuffers = 8;
constexpr int kPosted = 0, kPulled = 1;
constexpr int kFlagWords = 64;     // flags + staging words for the 4-byte copies
constexpr int kStage0 = 16;        // staging words start here (one per outstanding post and direction)

typedef CUresult (*StreamWaitValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
typedef CUresult (*StreamWriteValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

struct DriverOps {
  StreamWaitValueFn wait_value = nullptr;
  StreamWriteValueFn write_value = nullptr;
  bool ok = false;
};

const DriverOps& driver_ops() {
  static DriverOps ops = [] {
    DriverOps o;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      o.wait_value = reinterpret_cast<StreamWaitValueFn>(p);
    p = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      o.write_value = reinterpret_cast<StreamWriteValueFn>(p);
    cudaGetLastError();
    o.ok = o.wait_value && o.write_value;
    return o;
  }();
  return ops;
}

// What one rank publishes to its neighbours.
struct ExportBlob {
  int n_buffers;
  int reserved;
  unsigned long long bytes[kMaxBuffers];
  cudaIpcMemHandle_t flags;
  cudaIpcMemHandle_t buffers[kMaxBuffers];
};

struct PeerRing {
  int rank = 0, world = 1;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_ready = nullptr;
  cudaEvent_t ev_done[kDoneSlots] = {};
  cudaEvent_t ev_begin[kDoneSlots] = {};
  bool timing = false;
  unsigned next_slot = 0, posted = 0, waited = 0;
  unsigned seq = 0;
  int n_buffers = 0;
  void* buf[kMaxBuffers] = {};
  size_t bytes[kMaxBuffers] = {};
  uint32_t* flags = nullptr;        // local: [kPosted], [kPulled], staging words
  bool connected = false;
  void* prev_buf[kMaxBuffers] = {};  // previous rank's buffers, mapped here
  uint32_t* prev_flags = nullptr;
  uint32_t* next_flags = nullptr;
  bool same_peer = false;            // world size 2: previous and next rank are one process
};

// True once everything enqueued on the transport stream has run; gives up after about two seconds (a neighbour that
// never posts leaves a wait in the stream for good).
bool stream_drained(cudaStream_t s) {
  for (int i = 0; i < 2000; ++i) {
    const cudaError_t e = cudaStreamQuery(s);
    if (e == cudaSuccess) return true;
    if (e != cudaErrorNotReady) { cudaGetLastError(); return false; }
    struct timespec ts = {0, 1000000};
    nanosleep(&ts, nullptr);
  }
  return false;
}

void destroy_peer(PeerRing* c) {
  if (c->stream && !stream_drained(c->stream)) {
    // The stream still waits on a neighbour: unmapping or freeing what it refers to is not safe and waiting for it
    // could block the caller for ever (typically at process exit after another rank failed).  Leave everything to
    // the teardown of the CUDA context.
    delete c;
    return;
  }
  if (c->connected) {
    for (int i = 0; i < c->n_buffers; ++i)
      if (c->prev_buf[i]) cudaIpcCloseMemHandle(c->prev_buf[i]);
    if (c->prev_flags) cudaIpcCloseMemHandle(c->prev_flags);
    if (c->next_flags && !c->same_peer) cudaIpcCloseMemHandle(c->next_flags);
  }
  for (int i = 0; i < c->n_buffers; ++i)
    if (c->buf[i]) cudaFree(c->buf[i]);
  if (c->flags) cudaFree(c->flags);
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

extern "C" size_t rfa_peer_export_bytes(void) { return sizeof(ExportBlob); }

extern "C" int rfa_peer_create(int rank, int world, void** handle) {
  if (!handle || world < 2 || rank < 0 || rank >= world) return RFA_ERR_INVALID_ARG;
  if (!driver_ops().ok) return RFA_ERR_DRIVER;
  PeerRing* c = new PeerRing();
  c->rank = rank;
  c->world = world;
  int lo = 0, hi = 0;
  bool ok = cudaDeviceGetStreamPriorityRange(&lo, &hi) == cudaSuccess;
  ok = ok && cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, hi) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; ok && i < kDoneSlots; ++i)
    ok = cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaMalloc(reinterpret_cast<void**>(&c->flags), kFlagWords * sizeof(uint32_t)) == cudaSuccess;
  ok = ok && cudaMemset(c->flags, 0, kFlagWords * sizeof(uint32_t)) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    destroy_peer(c);
    return RFA_ERR_CUDA;
  }
  *handle = c;
  return RFA_OK;
}

extern "C" int rfa_peer_alloc(void* handle, size_t bytes, void** dev_ptr) {
  if (!handle || !dev_ptr || bytes == 0) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (c->connected || c->n_buffers >= kMaxBuffers) return RFA_ERR_INVALID_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  c->buf[c->n_buffers] = p;
  c->bytes[c->n_buffers] = bytes;
  ++c->n_buffers;
  *dev_ptr = p;
  return RFA_OK;
}

extern "C" int rfa_peer_export(void* handle, void* out, size_t cap) {
  if (!handle || !out || cap < sizeof(ExportBlob)) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  ExportBlob b;
  memset(&b, 0, sizeof(b));
  b.n_buffers = c->n_buffers;
  bool ok = cudaIpcGetMemHandle(&b.flags, c->flags) == cudaSuccess;
  for (int i = 0; ok && i < c->n_buffers; ++i) {
    b.bytes[i] = c->bytes[i];
    ok = cudaIpcGetMemHandle(&b.buffers[i], c->buf[i]) == cudaSuccess;
  }
  if (!ok) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  memcpy(out, &b, sizeof(b));
  return RFA_OK;
}

extern "C" int rfa_peer_connect(void* handle, const void* prev_blob, const void* next_blob) {
  if (!handle || !prev_blob || !next_blob) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (c->connected) return RFA_ERR_INVALID_ARG;
  ExportBlob pb, nb;
  memcpy(&pb, prev_blob, sizeof(pb));
  memcpy(&nb, next_blob, sizeof(nb));
  if (pb.n_buffers != c->n_buffers || nb.n_buffers != c->n_buffers) return RFA_ERR_INVALID_ARG;
  for (int i = 0; i < c->n_buffers; ++i)
    if (pb.bytes[i] != c->bytes[i]) return RFA_ERR_INVALID_ARG;  // ranks must allocate the same buffers in the same order
  c->same_peer = (c->world == 2);
  c->connected = true;  // from here on destroy_peer closes what was opened
  bool ok = cudaIpcOpenMemHandle(reinterpret_cast<void**>(&c->prev_flags), pb.flags, cudaIpcMemLazyEnablePeerAccess) ==
            cudaSuccess;
  for (int i = 0; ok && i < c->n_buffers; ++i)
    ok = cudaIpcOpenMemHandle(&c->prev_buf[i], pb.buffers[i], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
  if (ok) {
    if (c->same_peer) c->next_flags = c->prev_flags;  // a handle can be opened once per process
    else ok = cudaIpcOpenMemHandle(reinterpret_cast<void**>(&c->next_flags), nb.flags, cudaIpcMemLazyEnablePeerAccess) ==
              cudaSuccess;
  }
  if (!ok) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return RFA_OK;
}

extern "C" int rfa_peer_destroy(void* handle) {
  if (!handle) return RFA_ERR_INVALID_ARG;
  destroy_peer(static_cast<PeerRing*>(handle));
  return RFA_OK;
}

extern "C" int rfa_peer_post(void* handle, const void* send, void* recv, size_t bytes, void* compute_stream) {
  if (!handle || !send || !recv || bytes == 0 || send == recv) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (!c->connected) return RFA_ERR_INVALID_ARG;
  if (c->posted - c->waited >= static_cast<unsigned>(kDoneSlots)) return RFA_ERR_INVALID_ARG;
  int si = -1, ri = -1;
  for (int i = 0; i < c->n_buffers; ++i) {
    if (c->buf[i] == send) si = i;
    if (c->buf[i] == recv) ri = i;
  }
  // both must be whole ring buffers of this handle: the source of the transfer is the previous rank's buffer `si`
  if (si < 0 || ri < 0 || bytes > c->bytes[si] || bytes > c->bytes[ri]) return RFA_ERR_INVALID_ARG;
  const DriverOps& drv = driver_ops();
  cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
  cudaStream_t ts = c->stream;
  const unsigned n = ++c->seq;
  const int slot = static_cast<int>(c->next_slot % kDoneSlots);
  uint32_t* stage_posted = c->flags + kStage0 + 2 * slot;
  uint32_t* stage_pulled = stage_posted + 1;
  bool ok = cudaEventRecord(c->ev_ready, cs) == cudaSuccess && cudaStreamWaitEvent(ts, c->ev_ready, 0) == cudaSuccess;
  if (ok && c->timing) ok = cudaEventRecord(c->ev_begin[slot], ts) == cudaSuccess;
  // tell the next rank that buffer `si` holds message n
  ok = ok && drv.write_value(ts, reinterpret_cast<CUdeviceptr>(stage_posted), n, 0) == CUDA_SUCCESS;
  ok = ok && cudaMemcpyAsync(c->next_flags + kPosted, stage_posted, sizeof(uint32_t), cudaMemcpyDefault, ts) == cudaSuccess;
  // wait for the previous rank's message n, then pull it
  ok = ok && drv.wait_value(ts, reinterpret_cast<CUdeviceptr>(c->flags + kPosted), n, CU_STREAM_WAIT_VALUE_GEQ) == CUDA_SUCCESS;
  ok = ok && cudaMemcpyAsync(recv, c->prev_buf[si], bytes, cudaMemcpyDefault, ts) == cudaSuccess;
  // the previous rank may reuse its buffer; my own is free once the next rank has pulled it
  ok = ok && drv.write_value(ts, reinterpret_cast<CUdeviceptr>(stage_pulled), n, 0) == CUDA_SUCCESS;
  ok = ok && cudaMemcpyAsync(c->prev_flags + kPulled, stage_pulled, sizeof(uint32_t), cudaMemcpyDefault, ts) == cudaSuccess;
  ok = ok && drv.wait_value(ts, reinterpret_cast<CUdeviceptr>(c->flags + kPulled), n, CU_STREAM_WAIT_VALUE_GEQ) == CUDA_SUCCESS;
  ok = ok && cudaEventRecord(c->ev_done[slot], ts) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  ++c->next_slot;
  ++c->posted;
  return slot;
}

extern "C" int rfa_peer_wait(void* handle, int slot, void* compute_stream) {
  if (!handle || slot < 0 || slot >= kDoneSlots) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (c->waited == c->posted) return RFA_ERR_INVALID_ARG;
  if (cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), c->ev_done[slot], 0) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  ++c->waited;
  return RFA_OK;
}

// Diagnostics (rfa_b200_debug.h): transfer timing, as for the NCCL transport.
extern "C" int rfa_debug_peer_timing(void* handle, int on) {
  if (!handle) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (c->posted != c->waited) return RFA_ERR_INVALID_ARG;
  if (cudaStreamSynchronize(c->stream) != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
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

extern "C" int rfa_debug_peer_elapsed(void* handle, int slot, float* ms) {
  if (!handle || !ms || slot < 0 || slot >= kDoneSlots) return RFA_ERR_INVALID_ARG;
  PeerRing* c = static_cast<PeerRing*>(handle);
  if (!c->timing || !c->ev_begin[slot]) return RFA_ERR_INVALID_ARG;
  if (cudaEventElapsedTime(ms, c->ev_begin[slot], c->ev_done[slot]) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return RFA_OK;
}
