/*
 * C ABI of the B200 (sm_100a) ring-flash-attention hop kernels.
 *
 * This is the drop-in boundary for the sequence-parallel attention operator
 * `ring_flash_attn(q, k, v, softmax_scale, causal, zigzag, group)` of
 * AntonotnaWang/opt_ring_flash_attn (optimized_ring_flash_attn.py:1297-1367).
 * The reference is pure Python + Triton and has no FFI of its own; every entry
 * point below replaces one Triton kernel launch or torch elementwise op that
 * the reference's ring schedulers issue once per ring hop, and cites it.
 *
 * Rules of the ABI
 *  - plain pointers and sizes only; all pointers are device pointers unless
 *    stated otherwise; the compute entry points allocate nothing and keep no
 *    pointer after a call returns (the transport handle of rfa_comm_init owns a
 *    communicator, a stream and a few events until rfa_comm_destroy);
 *  - the device the stream belongs to must be the current device of the calling
 *    thread;
 *  - every call is asynchronous on `stream` (a cudaStream_t passed as void*);
 *    no call synchronises the device;
 *  - return value: RFA_OK or a negative RFA_ERR_* code (never an exception,
 *    abort or trap);
 *  - `status` points to one int32 in device memory, zero-initialised by the
 *    caller.  A kernel whose internal pipeline wait runs out of time writes a
 *    non-zero code there and returns early; later launches that see a non-zero
 *    status return immediately.  The host reads it whenever it wants to.
 *
 * Tensor contract (same as the reference, optimized_ring_flash_attn.py:1346-1360):
 *  q [B, Sq, Hq, D], k/v [B, Skv, Hkv, D], contiguous, bf16 or fp16,
 *  Hq % Hkv == 0, D % 8 == 0, D <= 256, q head h uses kv head h / (Hq / Hkv).
 */
#ifndef RFA_B200_H_
#define RFA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RFA_OK 0
#define RFA_ERR_INVALID_ARG (-1) /* null pointer, non-positive size, Hq % Hkv != 0, ... */
#define RFA_ERR_UNSUPPORTED (-2) /* head dim not a multiple of 8 or above 256, unknown dtype */
#define RFA_ERR_CUDA (-3)        /* a CUDA runtime call or the launch failed */
#define RFA_ERR_DRIVER (-4)      /* the driver rejected a tensor-map descriptor */
#define RFA_ERR_NCCL (-6)        /* NCCL is not loadable or an NCCL call failed */
#define RFA_ERR_TOO_LARGE (-5)   /* the shape needs more scratch than rfa_bwd_hop_noalloc's fixed array holds */

#define RFA_DTYPE_BF16 0
#define RFA_DTYPE_FP16 1

/* Version of this ABI (major * 100 + minor). */
int rfa_version(void);

/* Rows per sequence tile; per-row statistics (lse, delta) are stored with the
 * sequence length rounded up to a multiple of this. */
int rfa_seq_tile(void);

/*
 * Copies the device status word to `host_copy` (one int32 of pinned host memory) in stream order, without
 * synchronising: host_copy is set to -1 at once and holds the status word once the stream has reached the copy.
 * The host side of this library calls it at the end of every pass and looks at the copy at the start of the next
 * one, which is how a kernel's "bounded wait ran out" reaches the caller as an error.
 */
int rfa_status_publish(const int* status, int* host_copy, void* stream);

/* Number of fp32 elements of the forward accumulator state for the given shape
 * (private tiled layout; allocate once per shape, opaque to the caller). */
size_t rfa_fwd_acc_elems(int B, int Sq, int Hq, int D);

/*
 * One ring hop of the forward pass: attention of the local queries against one
 * K/V block, folded into the running fp32 (m, l, acc) state.
 * Replaces `_native_fwd_step_kernel` (optimized_ring_flash_attn.py:519-615) and
 * the online-softmax merge `_merge_kernel` (optimized_ring_flash_attn.py:328-417).
 *
 *  acc   fp32 [rfa_fwd_acc_elems]        unnormalised output accumulator (state)
 *  m, l  fp32 [B, Hq, Spad]              running maximum (log2 domain) and sum
 *  out   dtype [B, Sq, Hq, D]            written only when last != 0
 *  lse   fp32 [B, Hq, Spad]              natural-log LSE, written only when last != 0
 *  first != 0: the state is initialised by this hop (not read)
 *  last  != 0: out and lse are produced (the state is not written)
 *  causal_diag != 0: the K/V block is the queries' own block; key j is visible
 *                    to query i iff j <= i.  Otherwise the block is fully visible.
 *  Spad = Sq rounded up to rfa_seq_tile().
 */
int rfa_fwd_hop(const void* q, const void* k, const void* v, float* acc, float* m, float* l, void* out, float* lse,
                int B, int Sq, int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale, int first, int last,
                int causal_diag, int* status, void* stream);

/*
 * rfa_fwd_hop restricted to a window, for the zigzag layout (`_zigzag_forward`,
 * optimized_ring_flash_attn.py:1140-1196): only query rows >= q_begin are processed (q_begin % 128 == 0), only
 * keys < kv_len are visible, and query rows < q_split take `last_lo` where the others take `last` (in the
 * zigzag schedule the front half of a rank's rows sees its final K/V block earlier than the back half).
 * rfa_fwd_hop(...) == rfa_fwd_hop_window(..., q_begin=0, kv_len=Skv, q_split=0, last_lo=0).
 */
int rfa_fwd_hop_window(const void* q, const void* k, const void* v, float* acc, float* m, float* l, void* out,
                       float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale,
                       int first, int last, int causal_diag, int q_begin, int kv_len, int q_split, int last_lo,
                       int* status, void* stream);

/* Number of fp32 elements of the dQ accumulator (private tiled layout that makes the
 * per-tile reductions of the backward hop 16-byte vector operations; opaque to the caller). */
size_t rfa_dq_acc_elems(int B, int Sq, int Hq, int D);

/*
 * Backward preprocessing, once per backward pass:
 *   delta[b,h,s] = sum_d out[b,s,h,d] * dout[b,s,h,d]
 *   lse2[b,h,s]  = lse[b,h,s] * log2(e)      (rows s >= Sq: lse2 = +inf, delta = 0)
 * and, when dq_acc != NULL, the dQ accumulator (rfa_dq_acc_elems floats) is cleared.
 * Replaces `_bwd_preprocess_kernel` (optimized_ring_flash_attn.py:645-669) and the
 * `is_first` overwrite of `_dq_accum_kernel` (optimized_ring_flash_attn.py:441-460).
 */
int rfa_bwd_prepare(const void* out, const void* dout, const float* lse, float* delta, float* lse2, float* dq_acc,
                    int B, int Sq, int Hq, int D, int dtype, int* status, void* stream);

/*
 * One ring hop of the backward pass against one K/V block:
 *   dq_acc (fp32, rfa_dq_acc_elems)  +=  scale * dS  K
 *   dkdv_out[0] = (accumulate_prev ? dkdv_prev[0] : 0) + scale * dS^T Q
 *   dkdv_out[1] = (accumulate_prev ? dkdv_prev[1] : 0) + P^T dO
 * with P = exp2(scale*log2e * Q K^T - lse2), dS = P o (dO V^T - delta).
 * dkdv_* are fp32 [2, B, Skv, Hkv, D] (the packed buffer that travels round the
 * ring); dkdv_out may alias dkdv_prev.  dq_acc is updated with fp32 reductions.
 * Replaces `_bwd_dq_kernel` (optimized_ring_flash_attn.py:672-735),
 * `_bwd_dkdv_kernel` (optimized_ring_flash_attn.py:738-805) and the accumulate
 * kernels `_dq_accum_kernel` / `_dkdv_accum_kernel` (optimized_ring_flash_attn.py:441-503).
 */
int rfa_bwd_hop(const void* q, const void* k, const void* v, const void* dout, const float* lse2, const float* delta,
                float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B, int Sq, int Skv, int Hq, int Hkv,
                int D, int dtype, float softmax_scale, int accumulate_prev, int causal_diag, int* status,
                void* stream);

/*
 * rfa_bwd_hop restricted to a window, for the zigzag layout (`_zigzag_backward`,
 * optimized_ring_flash_attn.py:1198-1275): only query rows >= q_begin contribute and only keys < kv_len are
 * processed (kv_len need not be a multiple of the 128-row tile: keys at or beyond it inside the last tile are masked
 * out of P, so they add nothing to dQ); rows of dkdv_out at or beyond kv_len receive the previous partial sums
 * (accumulate_prev) or zero.
 * rfa_bwd_hop(...) == rfa_bwd_hop_window(..., q_begin=0, kv_len=Skv).
 */
int rfa_bwd_hop_window(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                       const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B, int Sq,
                       int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev,
                       int causal_diag, int q_begin, int kv_len, int* status, void* stream);

/*
 * rfa_bwd_hop_window with bit-reproducible dQ: the contributions of the K/V tiles to a dQ accumulator tile are
 * added in K/V-tile order (a counter per accumulator tile; each CTA waits, bounded, for the tiles before it), and
 * a GQA group is never split over CTAs.  This restores what the reference's dQ kernel has by construction (it owns
 * its tile and updates it with a plain read-modify-write, optimized_ring_flash_attn.py:730-735) and is what
 * `deterministic=True` of the baseline-style wrappers (ring_flash_attn.py:179, 245) selects.  Slower than the
 * unordered hop (CTAs of neighbouring K/V tiles run one query tile apart).
 *  dq_order  int32 [rfa_dq_order_elems(B,Sq,Hq,D)] scratch, cleared by the call itself.
 */
size_t rfa_dq_order_elems(int B, int Sq, int Hq, int D);
int rfa_bwd_hop_ordered(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                        const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B, int Sq,
                        int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev,
                        int causal_diag, int q_begin, int kv_len, int* dq_order, int* status, void* stream);

/*
 * out[i] = prev[i] + block[i] for n fp32 elements (n % 4 == 0; out may alias prev or block).
 * The ring accumulate of the travelling dK/dV buffer as a kernel of its own, for schedules that launch the
 * backward hop before the previous rank's partial sums have arrived (the hop then runs with
 * accumulate_prev = 0 into a block buffer, and this kernel folds the block in once the receive completed).
 * Replaces `_dkdv_accum_kernel` / `_launch_dkdv_accum` (optimized_ring_flash_attn.py:476-503, 1007-1012).
 */
int rfa_dkdv_accumulate(const float* prev, const float* block, float* out, size_t n, void* stream);

/*
 * 16-bit transport of the travelling dK/dV buffer: out[i] = round16(float(prev[i]) + block[i]) for n elements
 * (n % 8 == 0), prev and out in `dtype` (RFA_DTYPE_BF16 / RFA_DTYPE_FP16), block fp32; prev == NULL writes
 * round16(block[i]) (first active hop); out may alias prev.  Halves the backward wire bytes at the price of one
 * rounding per hop.  Replaces `_dkdv_accum_kernel` with a 16-bit comm dtype, selected in the reference by
 * OPTIMIZED_RING_BWD_COMM_BF16=1 (optimized_ring_flash_attn.py:205-208, 455-475).
 */
int rfa_dkdv_accumulate_to16(const void* prev, const float* block, void* out, size_t n, int dtype, void* stream);

/*
 * rfa_bwd_hop for callers that cannot allocate device memory (no counterpart in the reference).
 *
 * Same computation as rfa_bwd_hop followed by rfa_bwd_dq_finalize, but the caller passes no dQ
 * accumulator: dq (dtype [B,Sq,Hq,D]) receives scale * dS K of THIS hop only, and the fp32
 * accumulator the kernel needs lives in a fixed array of RFA_NOALLOC_SCRATCH_BYTES inside the library
 * (held by every GPU that loads it, until the process exits).  Meant for hosts where cudaMalloc is
 * off limits: a memory pool that was handed out completely at start-up, a plugin boundary that only
 * passes tensors in and out, or a section of the program that must not enter the driver's allocator.
 * The call itself performs no cudaMalloc/cudaFree and calls no allocating library routine.
 *
 *  - Shapes whose accumulator (rfa_dq_acc_elems(B,Sq,Hq,D) * 4 bytes) exceeds the array are rejected
 *    with RFA_ERR_TOO_LARGE; nothing is launched.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current); make that first call before any stream capture begins.
 *  - All calls on a device share the one array: it is cleared at the start of every call, and two
 *    calls that overlap on the GPU (different streams) race on it -- issue them on one stream.
 *  - The array is chosen by the calling thread's current device, which must be the stream's device.
 *  - Every argument is checked before anything is enqueued: a refused call leaves the stream untouched.
 */
#define RFA_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)
size_t rfa_noalloc_scratch_bytes(void);
int rfa_bwd_hop_noalloc(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                        const float* delta, void* dq, const float* dkdv_prev, float* dkdv_out, int B, int Sq, int Skv,
                        int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev, int causal_diag,
                        int* status, void* stream);

/*
 * dq[B,Sq,Hq,D] = (dtype) dq_acc: converts the accumulated dQ out of its private layout.
 * Replaces `dq_acc.to(q.dtype)` (optimized_ring_flash_attn.py:1027).
 */
int rfa_bwd_dq_finalize(const float* dq_acc, void* dq, int B, int Sq, int Hq, int D, int dtype, void* stream);

/*
 * dst[i] = (dtype) src[i] for n elements.  Replaces the final `.to(q.dtype)`
 * casts of the fp32 dK/dV buffers (optimized_ring_flash_attn.py:1028-1029).
 */
int rfa_cast_from_f32(const float* src, void* dst, size_t n, int dtype, void* stream);

/*
 * Packs K and V ([B, Skv, Hkv, D] each, `bytes_each` bytes) into one contiguous
 * [2, B, Skv, Hkv, D] transport buffer.  Replaces `kv_send[0].copy_(k);
 * kv_send[1].copy_(v)` (optimized_ring_flash_attn.py:836-838, 974-976).
 */
int rfa_pack_kv(const void* k, const void* v, void* dst, size_t bytes_each, void* stream);

/*
 * Ring transport on a private NCCL communicator (the transfers of `DoubleBufRingComm`,
 * optimized_ring_flash_attn.py:163-188, without a Python process-group round trip per hop).
 *
 *  rfa_comm_unique_id(out128)   rank 0 of the ring: fills 128 bytes of host memory to be sent to every rank
 *  rfa_comm_init(id, rank, W, &handle)   collective over the W ranks of the ring (W >= 2), current device;
 *                               the handle owns the communicator, one stream and a few events
 *  rfa_ring_post(handle, send, recv, bytes, compute_stream)
 *        after everything already enqueued on compute_stream: send `bytes` from `send` to rank+1 and receive
 *        `bytes` into `recv` from rank-1, as one NCCL group on the handle's own stream.  Returns a slot >= 0
 *        (or a negative error).  Asynchronous.  send and recv must differ.
 *  rfa_ring_wait(handle, slot, compute_stream)   compute_stream waits for that transfer; the host does not.
 *  rfa_comm_destroy(handle)
 * At most 8 posts may be outstanding (not yet waited for) per handle; a ninth is refused with
 * RFA_ERR_INVALID_ARG, as is a wait with nothing outstanding.  The handle's stream has the highest stream priority
 * of the device, so that the transfer's blocks are scheduled ahead of pending blocks of a running hop kernel.
 * Host pointers: out128, id, handle.
 */
int rfa_comm_unique_id(void* out128);
int rfa_comm_init(const void* id128, int rank, int world, void** handle);
int rfa_comm_destroy(void* handle);
int rfa_ring_post(void* handle, const void* send, void* recv, size_t bytes, void* compute_stream);
int rfa_ring_wait(void* handle, int slot, void* compute_stream);

/*
 * Ring transport over peer memory (same role as DoubleBufRingComm, optimized_ring_flash_attn.py:163-188, and as the
 * rfa_comm_* transport above): for ranks that are processes on one node whose GPUs can map each other's memory.
 * A transfer is one copy-engine copy out of the previous rank's buffer, ordered by sequence flags the neighbours
 * write into each other's memory and the transport's stream waits on with stream memory operations: no thread
 * block is involved, so a transfer neither waits for an SM nor takes one from the hop kernel.
 *
 *  rfa_peer_create(rank, W, &handle)    local; the handle owns a stream, events and a small flag buffer
 *  rfa_peer_alloc(handle, bytes, &ptr)  allocates ring buffer number i (cudaMalloc: the ring buffers must be
 *                                       exportable, so the handle owns them); every rank allocates the same buffers
 *                                       in the same order; at most 8
 *  rfa_peer_export(handle, out, cap)    fills rfa_peer_export_bytes() bytes of host memory to hand to both neighbours
 *  rfa_peer_connect(handle, prev, next) maps the previous rank's buffers and both neighbours' flags (after every
 *                                       rank has exported; no more rfa_peer_alloc afterwards)
 *  rfa_peer_post(handle, send, recv, bytes, compute_stream) / rfa_peer_wait(handle, slot, compute_stream)
 *        as rfa_ring_post / rfa_ring_wait; send and recv must be buffers of this handle, and every rank must pass
 *        the buffer with the same number as `send` (the receiver reads it from its predecessor's memory)
 *  rfa_peer_destroy(handle)             unmaps, frees the buffers; call it on every rank before a neighbour exits.  It
 *                                       waits (about two seconds at most) for the transport's stream; if that still
 *                                       waits on a neighbour, nothing is unmapped or freed before the context goes
 * A rank that never posts leaves its neighbours' transport streams waiting (as a missing rank does to an NCCL ring).
 * Host pointers: handle, out, prev, next, ptr.
 */
size_t rfa_peer_export_bytes(void);
int rfa_peer_create(int rank, int world, void** handle);
int rfa_peer_alloc(void* handle, size_t bytes, void** dev_ptr);
int rfa_peer_export(void* handle, void* out, size_t cap);
int rfa_peer_connect(void* handle, const void* prev_blob, const void* next_blob);
int rfa_peer_destroy(void* handle);
int rfa_peer_post(void* handle, const void* send, void* recv, size_t bytes, void* compute_stream);
int rfa_peer_wait(void* handle, int slot, void* compute_stream);

#ifdef __cplusplus
}
#endif

#endif /* RFA_B200_H_ */
