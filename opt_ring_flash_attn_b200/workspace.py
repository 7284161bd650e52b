"""Scratch buffers of the ring schedulers, allocated once per shape.

Mirrors ``_ForwardWorkspace`` / ``_BackwardWorkspace`` and their single-slot
caches (optimized_ring_flash_attn.py:211-303) with one deliberate difference:
tensors that outlive the call (``out``, ``lse``, the returned gradients) are
never part of the cache, so a second call with the same shapes cannot overwrite
what autograd saved for the first one.

All scratch is consumed inside the call that fills it, in stream order, so one
slot per (shape, dtype, device, world size) is enough as long as calls on one
device are issued on one stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

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


_fwd_cache: Dict[Tuple, ForwardWorkspace] = {}
_bwd_cache: Dict[Tuple, BackwardWorkspace] = {}


def _key(q: torch.Tensor, k: torch.Tensor, world_size: int, extra=None) -> Tuple:
    return (tuple(q.shape), tuple(k.shape), q.dtype, str(q.device), world_size, extra)


def forward_workspace(q: torch.Tensor, k: torch.Tensor, world_size: int) -> ForwardWorkspace:
    key = _key(q, k, world_size)
    ws = _fwd_cache.get(key)
    if ws is not None:
        return ws
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    dev = q.device
    spad = _native.padded_seq(S)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if world_size == 1:
        ws = ForwardWorkspace(None, None, None, None, [], status)
    else:
        acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
        m = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        l = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        kv_send = torch.empty(2, B, S, Hkv, D, dtype=q.dtype, device=dev)
        kv_recv = [torch.empty_like(kv_send) for _ in range(2)]
        ws = ForwardWorkspace(acc, m, l, kv_send, kv_recv, status)
    _fwd_cache.clear()  # single slot, like the reference
    _fwd_cache[key] = ws
    return ws


def backward_workspace(q: torch.Tensor, k: torch.Tensor, world_size: int,
                       comm_dtype: torch.dtype = torch.float32) -> BackwardWorkspace:
    """``comm_dtype`` is the dtype of the travelling dK/dV buffers (fp32, or the input dtype for 16-bit transport,
    optimized_ring_flash_attn.py:205-208, 271-272); this hop's own block is always fp32."""
    if world_size == 1:
        comm_dtype = torch.float32
    key = _key(q, k, world_size, comm_dtype)
    ws = _bwd_cache.get(key)
    if ws is not None:
        return ws
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    dev = q.device
    spad = _native.padded_seq(S)
    delta = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    lse2 = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    dq_acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
    nslots = 1 if world_size == 1 else 2
    dkdv = [torch.empty(2, B, S, Hkv, D, dtype=comm_dtype, device=dev) for _ in range(nslots)]
    if world_size == 1:
        kv_send, kv_recv, block_dkdv = None, [], None
    else:
        kv_send = torch.empty(2, B, S, Hkv, D, dtype=q.dtype, device=dev)
        kv_recv = [torch.empty_like(kv_send) for _ in range(2)]
        block_dkdv = torch.empty(2, B, S, Hkv, D, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = BackwardWorkspace(delta, lse2, dq_acc, dkdv, block_dkdv, kv_send, kv_recv, status)
    _bwd_cache.clear()
    _bwd_cache[key] = ws
    return ws


def clear() -> None:
    _fwd_cache.clear()
    _bwd_cache.clear()
