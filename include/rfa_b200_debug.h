/*
 * Diagnostic entry points of librfa_b200.so.  They are not part of the drop-in boundary (rfa_b200.h) and have no
 * counterpart in the reference: a tensor-core operand-path probe, an in-kernel event trace and transfer timing.
 */
#ifndef RFA_B200_DEBUG_H_
#define RFA_B200_DEBUG_H_

#ifdef __cplusplus
extern "C" {
#endif

/*
 * One 128x128x128 tensor-core product through each operand path the hop kernels use (mode 0..4), C fp32
 * [128,128] row-major, A and B bf16 [128,128] row-major.  Modes: 0 C=A*B^T (both K-major, shared memory);
 * 1 C=A*B (B MN-major); 2 C=A*B with A staged in tensor memory; 3 C=A^T*B (both MN-major); 4 as 0 with A
 * written to shared memory by threads.
 */
int rfa_debug_mma_probe(int mode, const void* a, const void* b, float* c, int* status, void* stream);

/*
 * Launches one small kernel whose only pipeline wait can never be satisfied (an mbarrier nobody arrives on).  The
 * bounded wait every hop kernel uses runs out after about two seconds, the kernel writes the time-out code into
 * `status` and returns: the way to see, without any fault, what a stuck pipeline does to the status word and that the
 * context stays usable afterwards.
 */
int rfa_debug_wait_timeout(int* status, void* stream);

/*
 * When `buf` is non-NULL, the hop kernels launched afterwards record per-role pipeline events of their first
 * `n_ctas` CTAs into buf, laid out [n_ctas][5 roles][cap] 64-bit words (tag << 48 | SM clock; roles: 0 loader,
 * 1 MMA issuer, 2/3 elementwise groups, 4 dQ reduction).  NULL switches tracing off.  Host-side state; not
 * thread safe.
 */
int rfa_debug_set_trace(unsigned long long* buf, int n_ctas, int cap);

/*
 * Transfer timing of a ring transport handle (rfa_comm_init): with `on`, every rfa_ring_post is bracketed by two
 * timing events on the transport's stream; rfa_debug_ring_elapsed gives the device time in milliseconds of the
 * transfer posted into `slot` (call it after that transfer has completed and before the slot is reused, 8 posts
 * later).  Switch only while no transfer is outstanding.
 */
int rfa_debug_ring_timing(void* handle, int on);
int rfa_debug_ring_elapsed(void* handle, int slot, float* ms);
/* The same for a peer-memory transport handle (rfa_peer_create). */
int rfa_debug_peer_timing(void* handle, int on);
int rfa_debug_peer_elapsed(void* handle, int slot, float* ms);

#ifdef __cplusplus
}
#endif

#endif /* RFA_B200_DEBUG_H_ */
