"""Host-side ring schedules: which hop kernel runs on which K/V block, and when buffers move.

Forward follows ``_ring_forward_native`` (optimized_ring_flash_attn.py:818-867):
rank r holds K/V block ``(r - step) mod W`` at step ``step``; with ``causal`` a
rank computes only while ``step <= rank``, the elementwise mask applies only to
its own block (step 0), and its result is final at ``step == rank``.

Backward follows ``_ring_backward_native`` (optimized_ring_flash_attn.py:946-1029):
a second ring carries the fp32 partial dK/dV of the block a rank currently
holds; slot algebra ``prev_slot = (step - 1) & 1``, the W-th send returns the
sums to the block's owner (``final_slot = (W - 1) & 1``).  As in the reference, the hop kernel of a step
is launched before the partial sums of the previous rank are waited for, and a separate accumulate kernel
folds them in (optimized_ring_flash_attn.py:1001-1012), so the large kernel never waits on the ring.

Differences from the reference, on purpose: a world size of 1 runs with no
communication at all; the fp32 running state replaces the per-hop merge kernel;
dQ, dK and dV of a hop come from one fused kernel.
"""
from __future__ import annotations

import atexit
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _native, workspace
from .transport import PeerRingTransport, PeerUnavailable, make_transport, transport_mode


# (ring key, device, ring name) -> transport.  The key is the process-group object itself (not its id(), which
# Python may hand to another object once a group is gone); entries live until shutdown().
_transports = {}


def _is_ring_handle(group) -> bool:
    """A ring handle stands in for a process group: any object with ``world_size``, ``ring_rank``,
    ``transport(name)`` and ``workspace_key``.  It lets one process drive several ranks (each with its own
    scratch and its own transports), which is how the schedules are exercised on a single device."""
    return hasattr(group, "ring_rank")


def _ws_owner(group):
    return group.workspace_key if _is_ring_handle(group) else None


def _transport(group, device: torch.device, tag: str):
    """One transport (and side stream) per (group, device, ring) until :func:`shutdown`."""
    if _is_ring_handle(group):
        return group.transport(tag)
    ring = group if group is not None else dist.group.WORLD
    key = (ring, str(device), tag)
    t = _transports.get(key)
    if t is None or t.world_size != dist.get_world_size(group):
        if t is not None:
            t.close()
        t = make_transport(group, device)
        _transports[key] = t
    return t


def _ring_factory(group, device: torch.device):
    """``ring(name, sizes) -> (transport, uint8 buffers)`` for the workspaces: the peer-memory transport brings its
    own buffers (one transport per ring and workspace, created collectively); the others are cached per ring and
    work on plain tensors."""
    def ring(tag: str, sizes):
        if not _is_ring_handle(group) and transport_mode(group, device) == "peer":
            key = group if group is not None else dist.group.WORLD
            if key not in _no_peer:
                try:
                    comm = PeerRingTransport(group, device, sizes)
                    return comm, comm.buffers
                except PeerUnavailable as e:  # the same on every rank: all fall back to the NCCL transport together
                    _no_peer.add(key)
                    import warnings
                    warnings.warn(f"peer-memory ring transport unavailable, using the NCCL transport: {e}")
        return _transport(group, device, tag), [torch.empty(n, dtype=torch.uint8, device=device) for n in sizes]
    return ring


def shutdown() -> None:
    """Destroy every transport (mapped peer memory, NCCL communicators, streams, events) and the scratch that
    belongs to them.  Call it on every rank before destroying the process group the transports were created on; it
    also runs at interpreter exit."""
    workspace.clear()
    for t in list(_transports.values()):
        try:
            t.close()
        except Exception:
            pass
    _transports.clear()
    _shapes_agreed.clear()


atexit.register(shutdown)


_shapes_agreed = set()
_no_peer = set()  # process groups on which the peer-memory transport could not be set up


def _agree_on_shapes(group, q: torch.Tensor, k: torch.Tensor, W: int) -> None:
    """The ring needs the same local shapes and dtype on every rank (the reference's contract: equal contiguous
    shards).  A mismatch would otherwise show up as a transfer of the wrong size -- a hang or silent garbage -- so
    the first call with a new shape on a process group compares them across ranks (one small object all-gather,
    never repeated for that shape) and raises ``ValueError`` on every rank before any buffer moves.
    ``RFA_B200_CHECK_SHAPES=0`` skips it."""
    if W == 1 or _is_ring_handle(group) or os.environ.get("RFA_B200_CHECK_SHAPES", "1") == "0":
        return
    if q.is_cuda and torch.cuda.is_current_stream_capturing():
        return
    ring = group if group is not None else dist.group.WORLD
    mine = (tuple(q.shape), tuple(k.shape), str(q.dtype))
    key = (ring, mine)
    if key in _shapes_agreed:
        return
    everyone = [None] * W
    dist.all_gather_object(everyone, mine, group=group)
    if any(other != mine for other in everyone):
        raise ValueError(f"ring_flash_attn: ranks disagree on the local shapes/dtype (q, k, dtype) per rank: {everyone}")
    _shapes_agreed.add(key)


def _world(group) -> Tuple[int, int]:
    if _is_ring_handle(group):
        return group.world_size, group.ring_rank
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def ring_forward(group, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, causal: bool,
                 kernels=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(out [B,S,Hq,D] in q's dtype, lse_padded [B,Hq,Spad] fp32)``; both are fresh tensors."""
    kn = kernels if kernels is not None else _native
    W, rank = _world(group)
    B, S, Hq, D = q.shape
    _agree_on_shapes(group, q, k, W)
    ws = workspace.forward_workspace(q, k, W, owner=_ws_owner(group), ring=_ring_factory(group, q.device))
    workspace.raise_if_failed(ws, "ring_flash_attn forward")
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, _native.padded_seq(S), dtype=torch.float32, device=q.device)

    if W == 1:
        kn.fwd_hop(q, k, v, None, None, None, out, lse, softmax_scale, True, True, causal, ws.status)
        workspace.publish_status(ws, "ring_flash_attn forward")
        return out, lse

    comm = ws.comms["fwd_kv"]
    kn.pack_kv(k, v, ws.kv_send)
    cur = ws.kv_send
    k_cur, v_cur = k, v
    last_step = rank if causal else W - 1
    for step in range(W):
        if step + 1 < W:
            comm.post(cur, ws.kv_recv[step & 1])
        if (not causal) or step <= rank:
            kn.fwd_hop(q, k_cur, v_cur, ws.acc, ws.m, ws.l, out, lse, softmax_scale,
                       step == 0, step == last_step, causal and step == 0, ws.status)
        if step + 1 < W:
            comm.wait()
            cur = ws.kv_recv[step & 1]
            k_cur, v_cur = cur[0], cur[1]
    workspace.publish_status(ws, "ring_flash_attn forward")
    return out, lse


def backward_comm_dtype(local_dtype: torch.dtype) -> torch.dtype:
    """Dtype of the travelling dK/dV buffers: fp32, or the input dtype when ``OPTIMIZED_RING_BWD_COMM_BF16=1`` — the
    reference's own switch and semantics (optimized_ring_flash_attn.py:205-208): the partial sums are rounded to 16 bit
    once per hop and the backward wire bytes halve."""
    if os.getenv("OPTIMIZED_RING_BWD_COMM_BF16", "0") == "1" and local_dtype in (torch.bfloat16, torch.float16):
        return local_dtype
    return torch.float32


def _fold_block(kn, buf, block, first: bool) -> None:
    """Travelling buffer (+)= this hop's fp32 block, in the buffer's dtype."""
    if buf.dtype == torch.float32:
        if first:
            buf.copy_(block)
        else:
            kn.dkdv_accumulate(buf, block, buf)
    else:
        kn.dkdv_accumulate_to16(None if first else buf, block, buf)


def _finish_dkdv(kn, final, dk, dv) -> None:
    if final.dtype == torch.float32:
        kn.cast_from_f32(final[0], dk)
        kn.cast_from_f32(final[1], dv)
    else:  # already in the input dtype; copied because the buffer belongs to the cached workspace
        dk.copy_(final[0])
        dv.copy_(final[1])


def ring_backward(group, dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                  lse: torch.Tensor, softmax_scale: float, causal: bool, kernels=None, deterministic: bool = False):
    """Returns ``(dq, dk, dv)`` in the input dtypes.  ``deterministic`` adds the dQ contributions of the K/V tiles
    in a fixed order (bit-reproducible gradients, like the reference's tile-exclusive dQ update,
    optimized_ring_flash_attn.py:730-735) at some cost in speed."""
    kn = kernels if kernels is not None else _native
    W, rank = _world(group)
    ws = workspace.backward_workspace(q, k, W, backward_comm_dtype(q.dtype), owner=_ws_owner(group),
                                      ring=_ring_factory(group, q.device))
    workspace.raise_if_failed(ws, "ring_flash_attn backward")
    wire16 = ws.dkdv[0].dtype != torch.float32
    order = {"dq_order": ws.dq_order} if deterministic else {}
    dout = dout.contiguous()
    kn.bwd_prepare(out, dout, lse, ws.delta, ws.lse2, ws.dq_acc, ws.status)

    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)

    if W == 1:
        buf = ws.dkdv[0]
        kn.bwd_hop(q, k, v, dout, ws.lse2, ws.delta, ws.dq_acc, None, buf, softmax_scale, False, causal, ws.status,
                   **order)
        kn.dq_finalize(ws.dq_acc, dq)
        kn.cast_from_f32(buf[0], dk)
        kn.cast_from_f32(buf[1], dv)
        workspace.publish_status(ws, "ring_flash_attn backward")
        return dq, dk, dv

    kv_comm, dkv_comm = ws.comms["bwd_kv"], ws.comms["bwd_dkdv"]
    kn.pack_kv(k, v, ws.kv_send)
    cur = ws.kv_send
    k_cur, v_cur = k, v
    for step in range(W):
        if step + 1 < W:
            kv_comm.post(cur, ws.kv_recv[step & 1])
        prev_slot = (step - 1) & 1
        buf = ws.dkdv[prev_slot]
        active = (not causal) or step <= rank
        if active:
            # The hop kernel does not wait for the ring: on step 0 it writes the travelling buffer directly (fp32
            # transport), later it writes this rank's block and the partial sums are folded in once they have arrived.
            direct = step == 0 and not wire16
            kn.bwd_hop(q, k_cur, v_cur, dout, ws.lse2, ws.delta, ws.dq_acc, None, buf if direct else ws.block_dkdv,
                       softmax_scale, False, causal and step == 0, ws.status, **order)
            if step == 0 and wire16:
                _fold_block(kn, buf, ws.block_dkdv, first=True)
        if step > 0:
            dkv_comm.wait()  # partial dK/dV of the block now held has arrived in dkdv[prev_slot]
            if active:
                _fold_block(kn, buf, ws.block_dkdv, first=False)
        if step + 1 < W:
            kv_comm.wait()
            cur = ws.kv_recv[step & 1]
            k_cur, v_cur = cur[0], cur[1]
        dkv_comm.post(buf, ws.dkdv[step & 1])
    dkv_comm.wait()
    final = ws.dkdv[(W - 1) & 1]
    kn.dq_finalize(ws.dq_acc, dq)
    _finish_dkdv(kn, final, dk, dv)
    workspace.publish_status(ws, "ring_flash_attn backward")
    return dq, dk, dv


def _zigzag_half(S: int) -> int:
    # the kernels work on 128-row tiles: both halves of the local shard must be tile-aligned
    if S % 256 != 0:
        raise ValueError(f"zigzag needs S_local to be a multiple of 256, got {S}")
    return S // 2


def zigzag_forward(group, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, kernels=None):
    """Causal ring forward over the zigzag layout: rank r holds ``[chunk_r ; chunk_{2W-1-r}]`` of 2W chunks.

    Per-step rule of ``_zigzag_forward`` (optimized_ring_flash_attn.py:1130-1196): step 0 is causal attention on
    the local shard; while ``step <= rank`` all local queries see the FRONT half of the visiting K/V block; after
    that only the BACK half of the local queries sees the whole visiting block.  Every rank works on every step
    (about half a block each), which is what balances the causal load.  The front half of the local rows is
    final at ``step == rank`` (step 0 on rank 0), the back half at the last step.
    """
    kn = kernels if kernels is not None else _native
    W, rank = _world(group)
    B, S, Hq, D = q.shape
    _agree_on_shapes(group, q, k, W)
    ws = workspace.forward_workspace(q, k, W, owner=_ws_owner(group), ring=_ring_factory(group, q.device))
    workspace.raise_if_failed(ws, "ring_flash_attn forward")
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, _native.padded_seq(S), dtype=torch.float32, device=q.device)
    if W == 1:
        kn.fwd_hop(q, k, v, None, None, None, out, lse, softmax_scale, True, True, True, ws.status)
        workspace.publish_status(ws, "ring_flash_attn forward")
        return out, lse
    half = _zigzag_half(S)
    comm = ws.comms["fwd_kv"]
    kn.pack_kv(k, v, ws.kv_send)
    cur = ws.kv_send
    k_cur, v_cur = k, v
    lo_final_step = rank  # rank 0: its front half only ever sees its own block
    for step in range(W):
        if step + 1 < W:
            comm.post(cur, ws.kv_recv[step & 1])
        last_hi = step == W - 1
        last_lo = step == lo_final_step
        if step == 0:
            kn.fwd_hop(q, k_cur, v_cur, ws.acc, ws.m, ws.l, out, lse, softmax_scale, True, last_hi, True, ws.status,
                       q_begin=0, kv_len=S, q_split=half, last_lo=last_lo)
        elif step <= rank:
            kn.fwd_hop(q, k_cur, v_cur, ws.acc, ws.m, ws.l, out, lse, softmax_scale, False, last_hi, False,
                       ws.status, q_begin=0, kv_len=half, q_split=half, last_lo=last_lo)
        else:
            kn.fwd_hop(q, k_cur, v_cur, ws.acc, ws.m, ws.l, out, lse, softmax_scale, False, last_hi, False,
                       ws.status, q_begin=half, kv_len=S, q_split=half, last_lo=False)
        if step + 1 < W:
            comm.wait()
            cur = ws.kv_recv[step & 1]
            k_cur, v_cur = cur[0], cur[1]
    workspace.publish_status(ws, "ring_flash_attn forward")
    return out, lse


def zigzag_backward(group, dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                    lse: torch.Tensor, softmax_scale: float, kernels=None, deterministic: bool = False):
    """Backward of :func:`zigzag_forward`; same window rule per step (optimized_ring_flash_attn.py:1198-1275),
    same two rings and slot algebra as :func:`ring_backward`."""
    kn = kernels if kernels is not None else _native
    W, rank = _world(group)
    if W == 1:
        return ring_backward(group, dout, q, k, v, out, lse, softmax_scale, True, kernels=kernels,
                             deterministic=deterministic)
    S = q.shape[1]
    half = _zigzag_half(S)
    ws = workspace.backward_workspace(q, k, W, backward_comm_dtype(q.dtype), owner=_ws_owner(group),
                                      ring=_ring_factory(group, q.device))
    workspace.raise_if_failed(ws, "ring_flash_attn backward")
    order = {"dq_order": ws.dq_order} if deterministic else {}
    wire16 = ws.dkdv[0].dtype != torch.float32
    dout = dout.contiguous()
    kn.bwd_prepare(out, dout, lse, ws.delta, ws.lse2, ws.dq_acc, ws.status)
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    kv_comm, dkv_comm = ws.comms["bwd_kv"], ws.comms["bwd_dkdv"]
    kn.pack_kv(k, v, ws.kv_send)
    cur = ws.kv_send
    k_cur, v_cur = k, v
    for step in range(W):
        if step + 1 < W:
            kv_comm.post(cur, ws.kv_recv[step & 1])
        prev_slot = (step - 1) & 1
        buf = ws.dkdv[prev_slot]
        if step == 0:
            kn.bwd_hop(q, k_cur, v_cur, dout, ws.lse2, ws.delta, ws.dq_acc, None, ws.block_dkdv if wire16 else buf,
                       softmax_scale, False, True, ws.status, q_begin=0, kv_len=S, **order)
            if wire16:
                _fold_block(kn, buf, ws.block_dkdv, first=True)
        elif step <= rank:
            kn.bwd_hop(q, k_cur, v_cur, dout, ws.lse2, ws.delta, ws.dq_acc, None, ws.block_dkdv, softmax_scale, False,
                       False, ws.status, q_begin=0, kv_len=half, **order)
        else:
            kn.bwd_hop(q, k_cur, v_cur, dout, ws.lse2, ws.delta, ws.dq_acc, None, ws.block_dkdv, softmax_scale, False,
                       False, ws.status, q_begin=half, kv_len=S, **order)
        if step > 0:
            dkv_comm.wait()
            _fold_block(kn, buf, ws.block_dkdv, first=False)
        if step + 1 < W:
            kv_comm.wait()
            cur = ws.kv_recv[step & 1]
            k_cur, v_cur = cur[0], cur[1]
        dkv_comm.post(buf, ws.dkdv[step & 1])
    dkv_comm.wait()
    final = ws.dkdv[(W - 1) & 1]
    kn.dq_finalize(ws.dq_acc, dq)
    _finish_dkdv(kn, final, dk, dv)
    workspace.publish_status(ws, "ring_flash_attn backward")
    return dq, dk, dv


# ----------------------------------------------------------------------------------------------------------------
# Balanced execution of contiguous shards
# ----------------------------------------------------------------------------------------------------------------
# With contiguous causal shards rank r does (r + 1/2) of W block-equivalents of work and waits for the rest of the
# step: on 8 ranks the job runs at 8/15 of what the GPUs could do.  The zigzag layout (rank r holds chunks r and
# 2W-1-r of 2W) gives every rank the same work.  A caller that holds contiguous shards (the reference's default
# layout, optimized_ring_flash_attn.py:1346-1351) can still have it: the shards are regrouped into the zigzag
# arrangement with one exchange of half-shards, the zigzag schedules run, and the results are regrouped back.  The
# arithmetic per (query, key) pair is the same; only the rank that does it changes.

def _chunk_home_contiguous(c: int) -> Tuple[int, int]:
    """(rank, half) that holds chunk c of 2W in the contiguous layout."""
    return c // 2, c % 2


def _chunk_home_zigzag(c: int, W: int) -> Tuple[int, int]:
    """(rank, half) that holds chunk c of 2W in the zigzag layout (optimized_ring_flash_attn.py:1122-1124)."""
    return (c, 0) if c < W else (2 * W - 1 - c, 1)


def regroup(group, tensors, to_zigzag: bool):
    """Moves the two sequence halves of every ``[B, S_local, ...]`` tensor between the contiguous layout (rank r holds
    chunks 2r, 2r+1) and the zigzag layout (rank r holds chunks r, 2W-1-r): one batch of point-to-point transfers of
    half-shards on the process group (halves that stay on their rank are copied locally).  Returns new tensors."""
    W, rank = _world(group)
    outs = [torch.empty_like(t) for t in tensors]
    ops, staged = [], []

    def peer(r):
        return dist.get_global_rank(group, r) if group is not None else r

    for t, o in zip(tensors, outs):
        half = t.shape[1] // 2
        # what I hold -> where it goes
        for h in (0, 1):
            c = (2 * rank + h) if to_zigzag else (rank if h == 0 else 2 * W - 1 - rank)
            dst_rank, dst_half = _chunk_home_zigzag(c, W) if to_zigzag else _chunk_home_contiguous(c)
            src = t[:, h * half:(h + 1) * half]
            if dst_rank == rank:
                o[:, dst_half * half:(dst_half + 1) * half].copy_(src)
            else:
                buf = src.contiguous()
                staged.append(buf)
                ops.append(dist.P2POp(dist.isend, buf, peer(dst_rank), group=group))
        # what I need <- where it is
        for h in (0, 1):
            c = (rank if h == 0 else 2 * W - 1 - rank) if to_zigzag else (2 * rank + h)
            src_rank, _ = _chunk_home_contiguous(c) if to_zigzag else _chunk_home_zigzag(c, W)
            if src_rank == rank:
                continue
            dst = o[:, h * half:(h + 1) * half]
            if dst.is_contiguous():
                ops.append(dist.P2POp(dist.irecv, dst, peer(src_rank), group=group))
            else:
                buf = torch.empty(dst.shape, dtype=dst.dtype, device=dst.device)
                staged.append((buf, dst))
                ops.append(dist.P2POp(dist.irecv, buf, peer(src_rank), group=group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for item in staged:
        if isinstance(item, tuple):
            item[1].copy_(item[0])
    return outs


def balanced_forward(group, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, kernels=None):
    """Causal forward of contiguous shards, executed in the zigzag arrangement.  Returns ``(out, lse_padded, saved)``:
    ``out`` / ``lse`` in the caller's contiguous layout, ``saved`` = the zigzag-arranged ``(q, k, v, out, lse)`` that
    :func:`balanced_backward` needs."""
    S = q.shape[1]
    qz, kz, vz = regroup(group, [q, k, v], to_zigzag=True)
    out_z, lse_z = zigzag_forward(group, qz, kz, vz, softmax_scale, kernels=kernels)
    # lse is [B, Hq, S] (S % 256 == 0, so it carries no padding): regrouped along its last dimension
    out, lse_t = regroup(group, [out_z, lse_z[:, :, :S].transpose(1, 2).contiguous()], to_zigzag=False)
    return out, lse_t.transpose(1, 2).contiguous(), (qz, kz, vz, out_z, lse_z)


def balanced_backward(group, dout: torch.Tensor, saved, softmax_scale: float, kernels=None, deterministic: bool = False):
    qz, kz, vz, out_z, lse_z = saved
    (dout_z,) = regroup(group, [dout.contiguous()], to_zigzag=True)
    dq_z, dk_z, dv_z = zigzag_backward(group, dout_z, qz, kz, vz, out_z, lse_z, softmax_scale, kernels=kernels,
                                       deterministic=deterministic)
    dq, dk, dv = regroup(group, [dq_z, dk_z, dv_z], to_zigzag=False)
    return dq, dk, dv


def can_balance(group, S_local: int) -> bool:
    """Balanced execution needs a ring of at least two ranks and half-shards that are whole 128-row tiles."""
    W, _ = _world(group)
    return W > 1 and S_local % 256 == 0 and not _is_ring_handle(group)
