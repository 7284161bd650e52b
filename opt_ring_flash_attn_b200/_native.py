"""ctypes binding of ``librfa_b200.so`` (the C ABI declared in ``include/rfa_b200.h``; diagnostics in
``include/rfa_b200_debug.h``).

There is no fallback: if the library is missing or a call fails, a
``RuntimeError`` is raised.  Tensors are passed as raw device pointers
(``tensor.data_ptr()``); the stream is the current torch CUDA stream of the
tensors' device unless given, and that device is made current for the call.
"""
from __future__ import annotations

import contextlib
import ctypes
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent / "librfa_b200.so"
_lib: Optional[ctypes.CDLL] = None

RFA_OK = 0
ERROR_NAMES = {
    -1: "RFA_ERR_INVALID_ARG",
    -2: "RFA_ERR_UNSUPPORTED",
    -3: "RFA_ERR_CUDA",
    -4: "RFA_ERR_DRIVER",
    -5: "RFA_ERR_TOO_LARGE",
    -6: "RFA_ERR_NCCL",
}
STATUS_NAMES = {0: "ok", 1: "a bounded pipeline wait inside a kernel ran out of time"}

DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1}

# name -> (restype, argtypes); must list every symbol of include/rfa_b200.h and include/rfa_b200_debug.h
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
SIGNATURES = {
    "rfa_version": (_i, []),
    "rfa_seq_tile": (_i, []),
    "rfa_status_publish": (_i, [_vp, _vp, _vp]),
    "rfa_fwd_acc_elems": (_sz, [_i, _i, _i, _i]),
    "rfa_dq_acc_elems": (_sz, [_i, _i, _i, _i]),
    "rfa_bwd_dq_finalize": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "rfa_fwd_hop": (_i, [_vp] * 8 + [_i] * 7 + [_f] + [_i] * 3 + [_vp, _vp]),
    "rfa_fwd_hop_window": (_i, [_vp] * 8 + [_i] * 7 + [_f] + [_i] * 7 + [_vp, _vp]),
    "rfa_bwd_hop_window": (_i, [_vp] * 9 + [_i] * 7 + [_f] + [_i] * 4 + [_vp, _vp]),
    "rfa_bwd_prepare": (_i, [_vp] * 6 + [_i] * 5 + [_vp, _vp]),
    "rfa_bwd_hop": (_i, [_vp] * 9 + [_i] * 7 + [_f] + [_i] * 2 + [_vp, _vp]),
    "rfa_dq_order_elems": (_sz, [_i, _i, _i, _i]),
    "rfa_bwd_hop_ordered": (_i, [_vp] * 9 + [_i] * 7 + [_f] + [_i] * 4 + [_vp, _vp, _vp]),
    "rfa_noalloc_scratch_bytes": (_sz, []),
    "rfa_bwd_hop_noalloc": (_i, [_vp] * 9 + [_i] * 7 + [_f] + [_i] * 2 + [_vp, _vp]),
    "rfa_dkdv_accumulate": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "rfa_dkdv_accumulate_to16": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "rfa_cast_from_f32": (_i, [_vp, _vp, _sz, _i, _vp]),
    "rfa_pack_kv": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "rfa_comm_unique_id": (_i, [_vp]),
    "rfa_comm_init": (_i, [_vp, _i, _i, ctypes.POINTER(ctypes.c_void_p)]),
    "rfa_comm_destroy": (_i, [_vp]),
    "rfa_ring_post": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "rfa_ring_wait": (_i, [_vp, _i, _vp]),
    "rfa_peer_export_bytes": (_sz, []),
    "rfa_peer_create": (_i, [_i, _i, ctypes.POINTER(ctypes.c_void_p)]),
    "rfa_peer_alloc": (_i, [_vp, _sz, ctypes.POINTER(ctypes.c_void_p)]),
    "rfa_peer_export": (_i, [_vp, _vp, _sz]),
    "rfa_peer_connect": (_i, [_vp, _vp, _vp]),
    "rfa_peer_destroy": (_i, [_vp]),
    "rfa_peer_post": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "rfa_peer_wait": (_i, [_vp, _i, _vp]),
    "rfa_debug_peer_timing": (_i, [_vp, _i]),
    "rfa_debug_peer_elapsed": (_i, [_vp, _i, ctypes.POINTER(ctypes.c_float)]),
    "rfa_debug_mma_probe": (_i, [_i, _vp, _vp, _vp, _vp, _vp]),
    "rfa_debug_set_trace": (_i, [_vp, _i, _i]),
    "rfa_debug_wait_timeout": (_i, [_vp, _vp]),
    "rfa_debug_ring_timing": (_i, [_vp, _i]),
    "rfa_debug_ring_elapsed": (_i, [_vp, _i, ctypes.POINTER(ctypes.c_float)]),
}


def library_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (building nothing: see ``build.py``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m opt_ring_flash_attn_b200.build` "
            "(there is no non-CUDA fallback for ring_flash_attn)"
        )
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


_launches = 0


def launch_count() -> int:
    """Number of kernels of this library launched so far by this process (memcpy-only calls excluded)."""
    return _launches


def _check(rc: int, what: str, kernels: int = 1) -> None:
    global _launches
    if rc != RFA_OK:
        raise RuntimeError(f"{what} failed: {ERROR_NAMES.get(rc, rc)}")
    _launches += kernels


def _stream(stream: Optional[torch.cuda.Stream], ref: Optional[torch.Tensor] = None) -> int:
    """Raw stream handle: the given stream, else the current stream of ``ref``'s device."""
    if stream is not None:
        return stream.cuda_stream
    return torch.cuda.current_stream(ref.device if ref is not None else None).cuda_stream


_NO_GUARD = contextlib.nullcontext()


def _on_device(t: torch.Tensor):
    """Context that makes ``t``'s device current (tensor maps, function attributes and the launch itself belong
    to the current device); free when it already is."""
    if t.device.index is None or t.device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(t.device)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def status_publish(status: torch.Tensor, host_copy_ptr: int, stream=None) -> None:
    rc = load().rfa_status_publish(_ptr(status), host_copy_ptr, _stream(stream, status))
    _check(rc, "rfa_status_publish", kernels=0)


def seq_tile() -> int:
    return 128


def padded_seq(s: int) -> int:
    return (s + 127) // 128 * 128


def fwd_acc_elems(B: int, Sq: int, Hq: int, D: int) -> int:
    n = load().rfa_fwd_acc_elems(B, Sq, Hq, D)
    if n == 0:
        raise RuntimeError(f"unsupported shape for the forward state: B={B} S={Sq} H={Hq} D={D}")
    return n


def fwd_hop(q, k, v, acc, m, l, out, lse, softmax_scale: float, first: bool, last: bool, causal_diag: bool,
            status: torch.Tensor, stream=None, q_begin: int = 0, kv_len: Optional[int] = None, q_split: int = 0,
            last_lo: bool = False) -> None:
    """One forward hop; the keyword arguments restrict it to a window (zigzag layout, see the C header)."""
    B, Sq, Hq, D = q.shape
    _, Skv, Hkv, _ = k.shape
    with _on_device(q):
        rc = load().rfa_fwd_hop_window(
            _ptr(q), _ptr(k), _ptr(v), _ptr(acc), _ptr(m), _ptr(l), _ptr(out), _ptr(lse),
            B, Sq, Skv, Hq, Hkv, D, DTYPE_CODES[q.dtype], float(softmax_scale),
            int(first), int(last), int(causal_diag), int(q_begin), int(Skv if kv_len is None else kv_len),
            int(q_split), int(last_lo), _ptr(status), _stream(stream, q))
    _check(rc, "rfa_fwd_hop")


def bwd_prepare(out, dout, lse, delta, lse2, dq_acc, status, stream=None) -> None:
    B, Sq, Hq, D = out.shape
    with _on_device(out):
        rc = load().rfa_bwd_prepare(_ptr(out), _ptr(dout), _ptr(lse), _ptr(delta), _ptr(lse2), _ptr(dq_acc),
                                    B, Sq, Hq, D, DTYPE_CODES[out.dtype], _ptr(status), _stream(stream, out))
    _check(rc, "rfa_bwd_prepare")


def bwd_hop(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, softmax_scale: float, accumulate_prev: bool,
            causal_diag: bool, status, stream=None, q_begin: int = 0, kv_len: Optional[int] = None,
            dq_order: Optional[torch.Tensor] = None) -> None:
    """One backward hop; ``q_begin`` / ``kv_len`` restrict it to a window (zigzag layout, see the C header).
    With ``dq_order`` (int32 scratch of ``dq_order_elems``) the dQ reductions are added in K/V-tile order
    (bit-reproducible dQ, ``rfa_bwd_hop_ordered``)."""
    B, Sq, Hq, D = q.shape
    _, Skv, Hkv, _ = k.shape
    args = (_ptr(q), _ptr(k), _ptr(v), _ptr(dout), _ptr(lse2), _ptr(delta), _ptr(dq_acc), _ptr(dkdv_prev),
            _ptr(dkdv_out), B, Sq, Skv, Hq, Hkv, D, DTYPE_CODES[q.dtype], float(softmax_scale),
            int(accumulate_prev), int(causal_diag), int(q_begin), int(Skv if kv_len is None else kv_len))
    with _on_device(q):
        if dq_order is None:
            rc = load().rfa_bwd_hop_window(*args, _ptr(status), _stream(stream, q))
        else:
            assert dq_order.dtype == torch.int32 and dq_order.numel() >= dq_order_elems(B, Sq, Hq, D)
            rc = load().rfa_bwd_hop_ordered(*args, _ptr(dq_order), _ptr(status), _stream(stream, q))
    _check(rc, "rfa_bwd_hop")


def dq_order_elems(B: int, Sq: int, Hq: int, D: int) -> int:
    n = load().rfa_dq_order_elems(B, Sq, Hq, D)
    if n == 0:
        raise RuntimeError(f"unsupported shape for the dQ ordering counters: B={B} S={Sq} H={Hq} D={D}")
    return n


def bwd_hop_noalloc(q, k, v, dout, lse2, delta, dq, dkdv_prev, dkdv_out, softmax_scale: float,
                    accumulate_prev: bool, causal_diag: bool, status, stream=None) -> None:
    """One backward hop for callers that cannot allocate: no dQ accumulator is passed, ``dq`` (q's dtype)
    receives this hop's dQ.  The accumulator is a fixed array inside the library (see the C header for
    the size limit, the first-call set-up and the one-stream rule)."""
    B, Sq, Hq, D = q.shape
    _, Skv, Hkv, _ = k.shape
    with _on_device(q):
        rc = load().rfa_bwd_hop_noalloc(
            _ptr(q), _ptr(k), _ptr(v), _ptr(dout), _ptr(lse2), _ptr(delta), _ptr(dq), _ptr(dkdv_prev),
            _ptr(dkdv_out), B, Sq, Skv, Hq, Hkv, D, DTYPE_CODES[q.dtype], float(softmax_scale),
            int(accumulate_prev), int(causal_diag), _ptr(status), _stream(stream, q))
    _check(rc, "rfa_bwd_hop_noalloc", kernels=2)


def dq_acc_elems(B: int, Sq: int, Hq: int, D: int) -> int:
    n = load().rfa_dq_acc_elems(B, Sq, Hq, D)
    if n == 0:
        raise RuntimeError(f"unsupported shape for the dQ accumulator: B={B} S={Sq} H={Hq} D={D}")
    return n


def dq_finalize(dq_acc: torch.Tensor, dq: torch.Tensor, stream=None) -> None:
    B, Sq, Hq, D = dq.shape
    with _on_device(dq):
        rc = load().rfa_bwd_dq_finalize(_ptr(dq_acc), _ptr(dq), B, Sq, Hq, D, DTYPE_CODES[dq.dtype],
                                        _stream(stream, dq))
    _check(rc, "rfa_bwd_dq_finalize")


def dkdv_accumulate(prev: torch.Tensor, block: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    assert prev.dtype == block.dtype == out.dtype == torch.float32 and prev.numel() == block.numel() == out.numel()
    with _on_device(out):
        rc = load().rfa_dkdv_accumulate(_ptr(prev), _ptr(block), _ptr(out), prev.numel(), _stream(stream, out))
    _check(rc, "rfa_dkdv_accumulate")


def dkdv_accumulate_to16(prev: Optional[torch.Tensor], block: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    """``out = round16(float(prev) + block)``; ``prev=None`` writes ``round16(block)``.  16-bit dK/dV transport."""
    assert block.dtype == torch.float32 and out.dtype in DTYPE_CODES and block.numel() == out.numel()
    assert prev is None or (prev.dtype == out.dtype and prev.numel() == out.numel())
    with _on_device(out):
        rc = load().rfa_dkdv_accumulate_to16(_ptr(prev), _ptr(block), _ptr(out), block.numel(),
                                             DTYPE_CODES[out.dtype], _stream(stream, out))
    _check(rc, "rfa_dkdv_accumulate_to16")


def cast_from_f32(src: torch.Tensor, dst: torch.Tensor, stream=None) -> None:
    assert src.dtype == torch.float32 and src.numel() == dst.numel()
    with _on_device(dst):
        rc = load().rfa_cast_from_f32(_ptr(src), _ptr(dst), src.numel(), DTYPE_CODES[dst.dtype], _stream(stream, dst))
    _check(rc, "rfa_cast_from_f32")


def pack_kv(k: torch.Tensor, v: torch.Tensor, dst: torch.Tensor, stream=None) -> None:
    nbytes = k.numel() * k.element_size()
    with _on_device(dst):
        rc = load().rfa_pack_kv(_ptr(k), _ptr(v), _ptr(dst), nbytes, _stream(stream, dst))
    _check(rc, "rfa_pack_kv", kernels=0)


def mma_probe(mode: int, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, status: torch.Tensor, stream=None) -> None:
    with _on_device(c):
        rc = load().rfa_debug_mma_probe(mode, _ptr(a), _ptr(b), _ptr(c), _ptr(status), _stream(stream, c))
    _check(rc, "rfa_debug_mma_probe")


def wait_timeout_probe(status: torch.Tensor, stream=None) -> None:
    """Diagnostics: a kernel whose bounded wait runs out (about two seconds); it sets ``status`` and returns."""
    with _on_device(status):
        rc = load().rfa_debug_wait_timeout(_ptr(status), _stream(stream, status))
    _check(rc, "rfa_debug_wait_timeout")


def comm_unique_id() -> bytes:
    buf = ctypes.create_string_buffer(128)
    _check(load().rfa_comm_unique_id(buf), "rfa_comm_unique_id", kernels=0)
    return buf.raw


def comm_init(unique_id: bytes, rank: int, world: int) -> int:
    handle = ctypes.c_void_p()
    _check(load().rfa_comm_init(ctypes.c_char_p(unique_id), rank, world, ctypes.byref(handle)), "rfa_comm_init",
           kernels=0)
    return handle.value


def comm_destroy(handle: int) -> None:
    _check(load().rfa_comm_destroy(handle), "rfa_comm_destroy", kernels=0)


def ring_post(handle: int, send: torch.Tensor, recv: torch.Tensor, stream=None) -> int:
    nbytes = send.numel() * send.element_size()
    with _on_device(send):
        slot = load().rfa_ring_post(handle, _ptr(send), _ptr(recv), nbytes, _stream(stream, send))
    if slot < 0:
        _check(slot, "rfa_ring_post", kernels=0)
    return slot


def ring_wait(handle: int, slot: int, stream=None, device: Optional[torch.device] = None) -> None:
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    _check(load().rfa_ring_wait(handle, slot, s), "rfa_ring_wait", kernels=0)


def peer_create(rank: int, world: int) -> int:
    handle = ctypes.c_void_p()
    _check(load().rfa_peer_create(rank, world, ctypes.byref(handle)), "rfa_peer_create", kernels=0)
    return handle.value


def peer_alloc(handle: int, nbytes: int) -> int:
    ptr = ctypes.c_void_p()
    _check(load().rfa_peer_alloc(handle, nbytes, ctypes.byref(ptr)), "rfa_peer_alloc", kernels=0)
    return ptr.value


def peer_export(handle: int) -> bytes:
    n = load().rfa_peer_export_bytes()
    buf = ctypes.create_string_buffer(n)
    _check(load().rfa_peer_export(handle, buf, n), "rfa_peer_export", kernels=0)
    return buf.raw


def peer_connect(handle: int, prev_blob: bytes, next_blob: bytes) -> None:
    _check(load().rfa_peer_connect(handle, ctypes.c_char_p(prev_blob), ctypes.c_char_p(next_blob)), "rfa_peer_connect",
           kernels=0)


def peer_destroy(handle: int) -> None:
    _check(load().rfa_peer_destroy(handle), "rfa_peer_destroy", kernels=0)


def peer_post(handle: int, send: torch.Tensor, recv: torch.Tensor, stream=None) -> int:
    nbytes = send.numel() * send.element_size()
    with _on_device(send):
        slot = load().rfa_peer_post(handle, _ptr(send), _ptr(recv), nbytes, _stream(stream, send))
    if slot < 0:
        _check(slot, "rfa_peer_post", kernels=0)
    return slot


def peer_wait(handle: int, slot: int, stream=None, device: Optional[torch.device] = None) -> None:
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    _check(load().rfa_peer_wait(handle, slot, s), "rfa_peer_wait", kernels=0)


def peer_timing(handle: int, on: bool) -> None:
    _check(load().rfa_debug_peer_timing(handle, int(on)), "rfa_debug_peer_timing", kernels=0)


def peer_elapsed_ms(handle: int, slot: int) -> float:
    ms = ctypes.c_float()
    _check(load().rfa_debug_peer_elapsed(handle, slot, ctypes.byref(ms)), "rfa_debug_peer_elapsed", kernels=0)
    return float(ms.value)


def ring_timing(handle: int, on: bool) -> None:
    """Diagnostics: bracket every later post of this transport with timing events (see rfa_b200_debug.h)."""
    _check(load().rfa_debug_ring_timing(handle, int(on)), "rfa_debug_ring_timing", kernels=0)


def ring_elapsed_ms(handle: int, slot: int) -> float:
    ms = ctypes.c_float()
    _check(load().rfa_debug_ring_elapsed(handle, slot, ctypes.byref(ms)), "rfa_debug_ring_elapsed", kernels=0)
    return float(ms.value)


def set_trace(buf: Optional[torch.Tensor], n_ctas: int = 0, cap: int = 0) -> None:
    """Diagnostics: record pipeline events of the first ``n_ctas`` CTAs of later hop launches into ``buf``
    (int64/uint64 tensor of n_ctas*5*cap elements); ``None`` switches tracing off."""
    rc = load().rfa_debug_set_trace(_ptr(buf), n_ctas, cap)
    _check(rc, "rfa_debug_set_trace", kernels=0)


def check_status(status: torch.Tensor, what: str = "ring_flash_attn") -> None:
    """Read the device status word (synchronises) and raise if a kernel reported a problem."""
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: device status {code}: {STATUS_NAMES.get(code, 'unknown')}")
