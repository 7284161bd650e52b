"""Drives the product's ring schedules for W ranks inside ONE process (test helper).

``schedule.ring_forward`` / ``ring_backward`` / ``zigzag_*`` accept a *ring handle* in place of a process group.
Here every emulated rank is a Python thread with its own CUDA stream (or plain CPU tensors), its own scratch
(``workspace_key``) and transports that hand the packed buffers to the next rank through in-process mailboxes:

  post(send, recv)   puts (send buffer, "producer done" event) into the next rank's mailbox
  wait()             takes the oldest message from the own mailbox, copies it into ``recv`` on the caller's
                     stream, acknowledges it to the sender, then waits for the own message to be acknowledged
                     (a send completes when the peer has the data -- NCCL's semantics, which the double-buffer
                     rotation of the schedules relies on)

The kernels are the real ones (or any object with the ``_native`` call signatures); nothing of the schedule is
restated here.  Kernels of different ranks never wait on one another on the device: all ordering is host-side
hand-over plus stream events, so this is safe on a single GPU.
"""
from __future__ import annotations

import queue
import threading
from collections import deque
from typing import Callable, Dict, List, Tuple

import torch

_TIMEOUT_S = 120.0


class _Message:
    def __init__(self, buf: torch.Tensor, ready):
        self.buf = buf
        self.ready = ready              # CUDA event: the sender's stream has produced ``buf`` (None on CPU)
        self.acked = threading.Event()  # set by the receiver once its copy is enqueued
        self.copied = None              # CUDA event behind the receiver's copy


class InProcTransport:
    def __init__(self, ring: "InProcRing", rank: int, tag: str):
        self.ring, self.rank, self.tag = ring, rank, tag
        self.world_size = ring.world_size
        self._pending = deque()  # (recv buffer, own outgoing message)
        self.posted = 0
        self.bytes_sent = 0

    def post(self, send_buf: torch.Tensor, recv_buf: torch.Tensor) -> None:
        if send_buf.data_ptr() == recv_buf.data_ptr():
            raise RuntimeError("ring transport: send and receive buffers must differ")
        ready = None
        if send_buf.is_cuda:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(send_buf.device))
        msg = _Message(send_buf, ready)
        self.ring.mailbox(self.tag, (self.rank + 1) % self.world_size).put(msg)
        self._pending.append((recv_buf, msg))
        self.posted += 1
        self.bytes_sent += send_buf.numel() * send_buf.element_size()

    def wait(self) -> None:
        if not self._pending:
            raise RuntimeError("ring transport: wait() without a posted transfer")
        recv_buf, mine = self._pending.popleft()
        incoming = self.ring.mailbox(self.tag, self.rank).get(timeout=_TIMEOUT_S)
        if recv_buf.is_cuda:
            cur = torch.cuda.current_stream(recv_buf.device)
            cur.wait_event(incoming.ready)
            recv_buf.copy_(incoming.buf)
            incoming.copied = torch.cuda.Event()
            incoming.copied.record(cur)
        else:
            recv_buf.copy_(incoming.buf)
        incoming.acked.set()
        if not mine.acked.wait(_TIMEOUT_S):
            raise RuntimeError("ring transport: the next rank never took the message")
        if mine.copied is not None:
            torch.cuda.current_stream(recv_buf.device).wait_event(mine.copied)

    def drain(self) -> None:
        while self._pending:
            self.wait()

    def close(self) -> None:
        self._pending.clear()


class RankHandle:
    """What the schedules see instead of a process group."""

    def __init__(self, ring: "InProcRing", rank: int):
        self.ring = ring
        self.world_size = ring.world_size
        self.ring_rank = rank
        self.workspace_key = ("inproc", id(ring), rank)
        self._transports: Dict[str, InProcTransport] = {}

    def transport(self, tag: str) -> InProcTransport:
        t = self._transports.get(tag)
        if t is None:
            t = self._transports[tag] = InProcTransport(self.ring, self.ring_rank, tag)
        return t


class InProcRing:
    def __init__(self, world_size: int):
        self.world_size = world_size
        self._boxes: Dict[Tuple[str, int], "queue.Queue[_Message]"] = {}
        self._lock = threading.Lock()
        self.handles = [RankHandle(self, r) for r in range(world_size)]

    def mailbox(self, tag: str, rank: int) -> "queue.Queue[_Message]":
        with self._lock:
            box = self._boxes.get((tag, rank))
            if box is None:
                box = self._boxes[(tag, rank)] = queue.Queue()
            return box

    def run(self, fn: Callable[[RankHandle], object], device: torch.device) -> List[object]:
        """Runs ``fn(handle)`` for every rank concurrently (one thread and, on CUDA, one stream per rank) and
        returns the per-rank results; the first exception of any rank is re-raised."""
        results: List[object] = [None] * self.world_size
        errors: List[BaseException] = []

        def body(r: int):
            try:
                if device.type == "cuda":
                    torch.cuda.set_device(device)
                    stream = torch.cuda.Stream(device=device)
                    stream.wait_stream(torch.cuda.default_stream(device))
                    with torch.cuda.stream(stream):
                        results[r] = fn(self.handles[r])
                    stream.synchronize()
                else:
                    results[r] = fn(self.handles[r])
            except BaseException as e:  # noqa: BLE001 - handed to the caller
                errors.append(e)

        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.world_size)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(4 * _TIMEOUT_S)
        if errors:
            raise errors[0]
        if any(t.is_alive() for t in threads):
            raise RuntimeError("an emulated rank did not finish")
        return results


def drop_workspaces(ring: InProcRing) -> None:
    """Frees the scratch the schedules cached for this ring's ranks."""
    from opt_ring_flash_attn_b200 import workspace

    for h in ring.handles:
        workspace._fwd_cache.pop(h.workspace_key, None)
        workspace._bwd_cache.pop(h.workspace_key, None)


def run_ring(world_size: int, device: torch.device, qs, ks, vs, dos, scale: float, causal: bool, kernels=None,
             zigzag: bool = False, deterministic: bool = False):
    """Forward (+ backward when ``dos`` is given) of all ranks through the product schedules.
    Returns per-rank lists ``(outs, lses, dqs, dks, dvs)`` (the gradient lists are empty without ``dos``)."""
    from opt_ring_flash_attn_b200 import schedule

    ring = InProcRing(world_size)

    def one_rank(h: RankHandle):
        r = h.ring_rank
        S = qs[r].shape[1]
        if zigzag:
            out, lse = schedule.zigzag_forward(h, qs[r], ks[r], vs[r], scale, kernels=kernels)
        else:
            out, lse = schedule.ring_forward(h, qs[r], ks[r], vs[r], scale, causal, kernels=kernels)
        if dos is None:
            return out, lse[:, :, :S], None, None, None
        if zigzag:
            dq, dk, dv = schedule.zigzag_backward(h, dos[r], qs[r], ks[r], vs[r], out, lse, scale, kernels=kernels,
                                                  deterministic=deterministic)
        else:
            dq, dk, dv = schedule.ring_backward(h, dos[r], qs[r], ks[r], vs[r], out, lse, scale, causal,
                                                kernels=kernels, deterministic=deterministic)
        return out, lse[:, :, :S], dq, dk, dv

    try:
        res = ring.run(one_rank, device)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
            from opt_ring_flash_attn_b200 import workspace
            workspace.check_all("in-process ring")
    finally:
        drop_workspaces(ring)
    outs, lses, dqs, dks, dvs = (list(x) for x in zip(*res))
    if dos is None:
        dqs, dks, dvs = [], [], []
    return outs, lses, dqs, dks, dvs
