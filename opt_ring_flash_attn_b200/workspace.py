"""Scratch buffers of the ring schedulers, allocated once per shape.

Mirrors ``_ForwardWorkspace`` / ``_BackwardWorkspace`` and their single-slot
caches (optimized_ring_flash_attn.py:211-303) with one deliberate difference:
tensors that outlive the call (``out``, ``lse``, the returned gradients) are
never part of the cache, so a second call with the same shapes cannot overwrite
what autograd saved for the first one.

All scratch is consumed inside the call that fills it, in stream order, so one
slot per (shape, dtype, device, world size) is enough as long as calls on one
device are issued on one stream.  A ring handle (several ranks driven by one
process) gets a slot of its own through ``owner``.

Each workspace also carries the device status word of its kernels and a pinned host copy of it.  A kernel
whose bounded pipeline wait runs out sets the word and every later kernel of that workspace returns at once, so
the word has to reach the host: :func:`publish_status` copies it out asynchronously at the end of a pass and
:func:`raise_if_failed` looks at the last copy at the start of the next one (no synchronisation; with
``RFA_B200_SYNC_STATUS=1`` every pass ends with a synchronising check instead).  :func:`check_all` does it on demand.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _native


def _padded_head_dim(d: int) -> int:
    return 64 if d <= 64 else (128 if d <= 128 else 256)


@dataclass
class ForwardWorkspace:
    acc: Optional[torch.Tensor]       # fp32 private tiled layout
    m: Optional[torch.Tensor]         # fp32 [B, Hq, Spad]
    l: Optional[torch.Tensor]         # fp32 [B, Hq, Spad]
    kv_send: Optional[torch.Tensor]   # dtype [2, B, S, Hkv, D]
    kv_recv: List[torch.Tensor]       # 2 x dtype [2, B, S, Hkv, D]
    status: torch.Tensor              # int32 [1]
    status_host: Optional[torch.Tensor] = None   # pinned int32 [1]: last published copy of ``status`` (-1: in flight)
    status_event: Any = None                     # host view (numpy) of status_host, None until something was published
    comms: Dict[str, Any] = field(default_factory=dict)  # ring name -> transport the ring buffers belong to
    last_publish: float = 0.0                    # host time of the last status copy


@dataclass
class BackwardWorkspace:
    delta: torch.Tensor               # fp32 [B, Hq, Spad]
    lse2: torch.Tensor                # fp32 [B, Hq, Spad]
    dq_acc: torch.Tensor              # fp32, private tiled layout (B*Hq*Spad*padded D elements)
    dkdv: List[torch.Tensor]          # 2 x [2, B, S, Hkv, D] in the transport dtype, fp32 by default (1 fp32 slot when world size is 1)
    block_dkdv: Optional[torch.Tensor]  # fp32 [2, B, S, Hkv, D]: this hop's own dK/dV before the ring accumulate
    kv_send: Optional[torch.Tensor]
    kv_recv: List[torch.Tensor]
    status: torch.Tensor
    dq_order: Optional[torch.Tensor] = None      # int32 counters of the ordered (deterministic) dQ reductions
    status_host: Optional[torch.Tensor] = None
    status_event: Any = None
    comms: Dict[str, Any] = field(default_factory=dict)
    last_publish: float = 0.0


# owner -> (key, workspace): one slot per owner (None = the process's own rank; a ring handle brings its own key)
_fwd_cache: Dict[Any, Tuple[Tuple, ForwardWorkspace]] = {}
_bwd_cache: Dict[Any, Tuple[Tuple, BackwardWorkspace]] = {}


def _key(q: torch.Tensor, k: torch.Tensor, world_size: int, extra=None) -> Tuple:
    return (tuple(q.shape), tuple(k.shape), q.dtype, str(q.device), world_size, extra)


def _new_status(dev: torch.device):
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    host = torch.zeros(1, dtype=torch.int32, pin_memory=True) if dev.type == "cuda" else None
    return status, host


def _ring_buffers(ring, tag: str, n: int, shape, dtype: torch.dtype, dev: torch.device):
    """``n`` packed ring buffers of ``shape``/``dtype`` and the transport they travel on.  ``ring(tag, sizes)``
    (given by the schedules) returns ``(transport, uint8 buffers)``: a peer-memory transport owns its buffers, the
    others take plain tensors.  Without a factory the buffers are plain tensors and no transport is attached."""
    nbytes = torch.empty(0, dtype=dtype).element_size()
    for d in shape:
        nbytes *= d
    if ring is None:
        return None, [torch.empty(shape, dtype=dtype, device=dev) for _ in range(n)]
    comm, raw = ring(tag, [nbytes] * n)
    return comm, [b.view(dtype).view(shape) for b in raw]


def _retire(ws) -> None:
    """A workspace leaves the cache: transports that own its ring buffers go with it (collective-free; every rank
    replaces its workspace at the same call, so neighbours unmap each other at the same point of the program)."""
    for comm in ws.comms.values():
        if comm is not None and getattr(comm, "owns_buffers", False):
            comm.close()
    ws.comms.clear()


def all_workspaces() -> List:
    return [ws for _, ws in list(_fwd_cache.values()) + list(_bwd_cache.values())]


def _fail(ws, code: int, what: str):
    ws.status.zero_()  # reported once; the workspace is usable again
    if ws.status_host is not None:
        ws.status_host.zero_()
    raise RuntimeError(f"{what}: device status {code}: {_native.STATUS_NAMES.get(code, 'unknown')}; the results of "
                       "the pass that hit it are invalid")


def _capturing(ws) -> bool:
    return ws.status.is_cuda and torch.cuda.is_current_stream_capturing()


def raise_if_failed(ws, what: str) -> None:
    """Start of a pass: if the copy published by the previous pass on this workspace has landed and is non-zero,
    clear the device word and raise.  Never blocks (a copy still in flight reads -1 and is looked at next time)."""
    view = ws.status_event
    if view is None:
        return
    code = int(view[0])
    if code > 0 and not _capturing(ws):
        _fail(ws, code, what)


_STATUS_CHECK = os.environ.get("RFA_B200_STATUS_CHECK", "1") != "0"


def publish_status(ws, what: str) -> None:
    """End of a pass: enqueue the 4-byte copy of the status word to pinned host memory (``rfa_status_publish``)."""
    if ws.status_host is None or not _STATUS_CHECK or _capturing(ws):
        return
    sync = os.environ.get("RFA_B200_SYNC_STATUS", "0") == "1"
    # The copy costs the host some 15 microseconds, which is a tenth of a short-shard step: passes that follow each
    # other within a millisecond share one copy (a failure then surfaces a few passes later instead of one).
    now = time.perf_counter()
    if not sync and now - ws.last_publish < 1e-3:
        return
    ws.last_publish = now
    if ws.status_event is None:
        ws.status_event = ws.status_host.numpy()  # shares the pinned memory
    _native.status_publish(ws.status, ws.status_host.data_ptr())
    if sync:
        torch.cuda.current_stream(ws.status.device).synchronize()
        raise_if_failed(ws, what)


def check_all(what: str = "ring_flash_attn") -> None:
    """Synchronising check of every cached workspace's status word; raises ``RuntimeError`` on the first failure."""
    for ws in all_workspaces():
        code = int(ws.status.item())
        if code != 0:
            _fail(ws, code, what)


def forward_workspace(q: torch.Tensor, k: torch.Tensor, world_size: int, owner=None, ring=None) -> ForwardWorkspace:
    key = _key(q, k, world_size)
    hit = _fwd_cache.get(owner)
    if hit is not None and hit[0] == key:
        return hit[1]
    if hit is not None:
        _retire(hit[1])
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    dev = q.device
    spad = _native.padded_seq(S)
    status, status_host = _new_status(dev)
    if world_size == 1:
        ws = ForwardWorkspace(None, None, None, None, [], status, status_host)
    else:
        acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
        m = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        l = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        comm, kv = _ring_buffers(ring, "fwd_kv", 3, (2, B, S, Hkv, D), q.dtype, dev)
        ws = ForwardWorkspace(acc, m, l, kv[0], kv[1:], status, status_host, comms={"fwd_kv": comm})
    _fwd_cache[owner] = (key, ws)  # single slot per owner, like the reference
    return ws


def backward_workspace(q: torch.Tensor, k: torch.Tensor, world_size: int,
                       comm_dtype: torch.dtype = torch.float32, owner=None, ring=None) -> BackwardWorkspace:
    """``comm_dtype`` is the dtype of the travelling dK/dV buffers (fp32, or the input dtype for 16-bit transport,
    optimized_ring_flash_attn.py:205-208, 271-272); this hop's own block is always fp32."""
    if world_size == 1:
        comm_dtype = torch.float32
    key = _key(q, k, world_size, comm_dtype)
    hit = _bwd_cache.get(owner)
    if hit is not None and hit[0] == key:
        return hit[1]
    if hit is not None:
        _retire(hit[1])
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    dev = q.device
    spad = _native.padded_seq(S)
    delta = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    lse2 = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    dq_acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
    comms = {}
    if world_size == 1:
        dkdv = [torch.empty(2, B, S, Hkv, D, dtype=comm_dtype, device=dev)]
        kv_send, kv_recv, block_dkdv = None, [], None
    else:
        comms["bwd_dkdv"], dkdv = _ring_buffers(ring, "bwd_dkdv", 2, (2, B, S, Hkv, D), comm_dtype, dev)
        comms["bwd_kv"], kv = _ring_buffers(ring, "bwd_kv", 3, (2, B, S, Hkv, D), q.dtype, dev)
        kv_send, kv_recv = kv[0], kv[1:]
        block_dkdv = torch.empty(2, B, S, Hkv, D, dtype=torch.float32, device=dev)
    status, status_host = _new_status(dev)
    # counters of the ordered dQ reductions: 8 per (batch, head, query tile of 64 rows) covers every head dim
    dq_order = torch.zeros(B * Hq * ((S + 63) // 64) * 2 * 8, dtype=torch.int32, device=dev)
    ws = BackwardWorkspace(delta, lse2, dq_acc, dkdv, block_dkdv, kv_send, kv_recv, status, dq_order, status_host,
                           comms=comms)
    _bwd_cache[owner] = (key, ws)
    return ws


def clear() -> None:
    for ws in all_workspaces():
        _retire(ws)
    _fwd_cache.clear()
    _bwd_cache.clear()
