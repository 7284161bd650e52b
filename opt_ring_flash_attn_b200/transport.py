"""Ring transport: one packed buffer to the next rank, one from the previous rank, per hop.

Mirrors ``DoubleBufRingComm`` of the reference (optimized_ring_flash_attn.py:163-188):
``post(send, recv)`` issues one isend + one irecv as a single batch and returns
immediately; ``wait()`` completes the oldest outstanding batch.  Ranks are
group-local ring positions mapped to global ranks for sub-groups
(optimized_ring_flash_attn.py:168-172).

On CUDA the batch runs on the process group's NCCL stream: NCCL orders it after
everything already enqueued on the stream it was posted from, and ``wait()``
makes that stream wait for the transfer without blocking the host, so the
transfer of hop s+1's block overlaps the kernels of hop s.  With ``side_stream``
the post/wait pair is issued from a dedicated stream and fenced to the compute
stream with events, which keeps the compute stream free of transport waits
until the data is actually needed.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Deque, List, Optional

import torch
import torch.distributed as dist


class RingTransport:
    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, side_stream: bool = True):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        nxt = (self.rank + 1) % self.world_size
        prv = (self.rank - 1) % self.world_size
        if group is not None:
            nxt = dist.get_global_rank(group, nxt)
            prv = dist.get_global_rank(group, prv)
        self.send_rank = nxt
        self.recv_rank = prv
        self.device = device
        self._cuda = device.type == "cuda"
        self._stream = torch.cuda.Stream(device=device) if (self._cuda and side_stream) else None
        # FIFO of (requests, completion event or None)
        self._pending: Deque[List] = deque()
        self.posted = 0  # number of batches posted (for tests and the bench's byte accounting)
        self.bytes_sent = 0

    def post(self, send_buf: torch.Tensor, recv_buf: torch.Tensor) -> None:
        """Ship ``send_buf`` to the next rank and receive ``recv_buf`` from the previous one (async)."""
        if send_buf.data_ptr() == recv_buf.data_ptr():
            raise RuntimeError("ring transport: send and receive buffers must differ")
        ops = [
            dist.P2POp(dist.isend, send_buf, self.send_rank, group=self.group),
            dist.P2POp(dist.irecv, recv_buf, self.recv_rank, group=self.group),
        ]
        self.posted += 1
        self.bytes_sent += send_buf.numel() * send_buf.element_size()
        if self._stream is None:
            self._pending.append([dist.batch_isend_irecv(ops), None])
            return
        compute = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(compute)  # everything that produced send_buf / last read recv_buf
        self._stream.wait_event(ready)
        with torch.cuda.stream(self._stream):
            reqs = dist.batch_isend_irecv(ops)
            for r in reqs:
                r.wait()  # side stream waits for the NCCL stream; the host does not block
            done = torch.cuda.Event()
            done.record(self._stream)
        self._pending.append([reqs, done])

    def wait(self) -> None:
        """Make the current stream (or the host, on CPU) wait for the oldest outstanding batch."""
        if not self._pending:
            raise RuntimeError("ring transport: wait() without a posted transfer")
        reqs, done = self._pending.popleft()
        if done is None:
            for r in reqs:
                r.wait()
        else:
            torch.cuda.current_stream(self.device).wait_event(done)

    def drain(self) -> None:
        while self._pending:
            self.wait()

    def close(self) -> None:
        """Nothing of its own to release: the process group owns the communicator."""
        self._pending.clear()


class NativeRingTransport:
    """Same protocol on a private NCCL communicator inside ``librfa_b200.so`` (``rfa_ring_post`` / ``rfa_ring_wait``).

    One C call per post (event fence, grouped ncclSend + ncclRecv on the transport's own stream, completion
    event) instead of a ``batch_isend_irecv`` round trip through the process group: the per-hop host cost drops
    from roughly a hundred microseconds to about ten, which is what bounds short shards.  The communicator is
    created collectively on first use; its unique id travels over the given torch process group.
    """

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device):
        from . import _native

        self._native = _native
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.device = device
        src = dist.get_global_rank(group, 0) if group is not None else 0
        holder = [_native.comm_unique_id() if self.rank == 0 else None]
        dist.broadcast_object_list(holder, src=src, group=group, device=device)
        with torch.cuda.device(device):
            self._handle = _native.comm_init(holder[0], self.rank, self.world_size)
        self._pending: Deque[int] = deque()
        self.posted = 0
        self.bytes_sent = 0

    def post(self, send_buf: torch.Tensor, recv_buf: torch.Tensor) -> None:
        if send_buf.data_ptr() == recv_buf.data_ptr():
            raise RuntimeError("ring transport: send and receive buffers must differ")
        if len(self._pending) >= 6:
            raise RuntimeError("ring transport: too many transfers outstanding")
        self._pending.append(self._native.ring_post(self._handle, send_buf, recv_buf))
        self.posted += 1
        self.bytes_sent += send_buf.numel() * send_buf.element_size()

    def wait(self) -> None:
        if not self._pending:
            raise RuntimeError("ring transport: wait() without a posted transfer")
        self._native.ring_wait(self._handle, self._pending.popleft(), device=self.device)

    def drain(self) -> None:
        while self._pending:
            self.wait()

    def close(self) -> None:
        """Destroy the communicator, the transport stream and its events (collective-free, local)."""
        if self._handle is not None:
            handle, self._handle = self._handle, None
            self._pending.clear()
            with torch.cuda.device(self.device):
                self._native.comm_destroy(handle)

    # diagnostics: device time of each transfer (see rfa_b200_debug.h)
    def set_timing(self, on: bool) -> None:
        self._native.ring_timing(self._handle, on)

    def elapsed_ms(self, slot: int) -> float:
        return self._native.ring_elapsed_ms(self._handle, slot)

    def last_slot(self) -> int:
        return self._pending[-1]


class PeerUnavailable(RuntimeError):
    """The peer-memory transport could not be set up on some rank (no peer access between the GPUs, IPC refused);
    raised on every rank of the ring alike."""


class _DeviceMemory:
    """Lets torch wrap device memory that the transport library owns (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerRingTransport:
    """Same protocol over peer memory (``rfa_peer_*``): every transfer is a copy-engine copy out of the previous
    rank's buffer, ordered by flags in device memory; no SM takes part, so transfers neither wait for thread-block
    slots behind a hop kernel nor take SMs away from it.  The ring buffers belong to the transport (they must be
    exportable to the neighbours): ``buffers[i]`` are uint8 tensors over them, allocated for the sizes given at
    construction, in the same order on every rank.  Construction is collective over the group."""

    owns_buffers = True

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, sizes: List[int]):
        from . import _native

        self._native = _native
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.device = device
        self._handle = None
        self.buffers = []
        self._pending: Deque[int] = deque()
        # Every step that can fail on one rank only (allocation, export, mapping the neighbours) is followed by an
        # exchange of the outcome, so that all ranks keep the transport or all ranks give it up (PeerUnavailable).
        blob, ptrs, err = None, [], None
        try:
            with torch.cuda.device(device):
                self._handle = _native.peer_create(self.rank, self.world_size)
                ptrs = [_native.peer_alloc(self._handle, int(n)) for n in sizes]
                blob = _native.peer_export(self._handle)
        except RuntimeError as e:
            err = str(e)
        blobs = [None] * self.world_size
        dist.all_gather_object(blobs, blob, group=group)
        if err is None and all(b is not None for b in blobs):
            try:
                with torch.cuda.device(device):
                    _native.peer_connect(self._handle, blobs[(self.rank - 1) % self.world_size],
                                         blobs[(self.rank + 1) % self.world_size])
            except RuntimeError as e:
                err = str(e)
        elif err is None:
            err = "a neighbour could not export its buffers"
        outcomes = [None] * self.world_size
        dist.all_gather_object(outcomes, err, group=group)  # also: every rank has mapped its neighbours before anyone posts
        if any(o is not None for o in outcomes):
            self.close()
            raise PeerUnavailable("; ".join(f"rank {r}: {o}" for r, o in enumerate(outcomes) if o is not None))
        self.buffers = [torch.as_tensor(_DeviceMemory(p, int(n)), device=device) for p, n in zip(ptrs, sizes)]
        self.posted = 0
        self.bytes_sent = 0

    def post(self, send_buf: torch.Tensor, recv_buf: torch.Tensor) -> None:
        if send_buf.data_ptr() == recv_buf.data_ptr():
            raise RuntimeError("ring transport: send and receive buffers must differ")
        if len(self._pending) >= 6:
            raise RuntimeError("ring transport: too many transfers outstanding")
        self._pending.append(self._native.peer_post(self._handle, send_buf, recv_buf))
        self.posted += 1
        self.bytes_sent += send_buf.numel() * send_buf.element_size()

    def wait(self) -> None:
        if not self._pending:
            raise RuntimeError("ring transport: wait() without a posted transfer")
        self._native.peer_wait(self._handle, self._pending.popleft(), device=self.device)

    def drain(self) -> None:
        while self._pending:
            self.wait()

    def close(self) -> None:
        """Unmaps the neighbours' memory and frees the ring buffers.  The tensors in ``buffers`` die with it.
        Every rank must close before a neighbour's process exits (the mappings point into its memory)."""
        if self._handle is not None:
            handle, self._handle = self._handle, None
            self._pending.clear()
            self.buffers = []
            with torch.cuda.device(self.device):
                # the kernels that still read the buffers must have run; bounded, so that a rank whose neighbour is
                # gone (its compute stream then waits on a transfer that never completes) can still exit
                compute = torch.cuda.current_stream(self.device)
                deadline = time.monotonic() + 2.0
                while not compute.query() and time.monotonic() < deadline:
                    time.sleep(0.001)
                if compute.query():
                    self._native.peer_destroy(handle)  # (itself bounded on the transport's own stream)

    def set_timing(self, on: bool) -> None:
        self._native.peer_timing(self._handle, on)

    def elapsed_ms(self, slot: int) -> float:
        return self._native.peer_elapsed_ms(self._handle, slot)

    def last_slot(self) -> int:
        return self._pending[-1]


def transport_mode(group: Optional[dist.ProcessGroup], device: torch.device) -> str:
    """``peer`` (copy engines over mapped peer memory), ``native`` (private NCCL communicator) or ``torch`` (the
    process group's own send/recv).  CUDA ranks on an NCCL group default to ``peer``; ``RFA_B200_TRANSPORT``
    overrides; everything else (CPU ranks on gloo in the tests) uses ``torch``."""
    import os

    if device.type != "cuda" or dist.get_backend(group) != "nccl":
        return "torch"
    mode = os.environ.get("RFA_B200_TRANSPORT", "peer")
    return mode if mode in ("peer", "native", "torch") else "peer"


def make_transport(group: Optional[dist.ProcessGroup], device: torch.device):
    """A transport that works on caller-owned buffers: NCCL (``native``) or the process group (``torch``)."""
    if transport_mode(group, device) in ("peer", "native"):
        return NativeRingTransport(group, device)
    return RingTransport(group, device)
