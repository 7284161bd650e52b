"""A hand-written walk over the W ranks of the contiguous-shard ring on ONE device, rank after rank.

The product schedules themselves are driven by tests/inproc_ring.py; this walk exists for the one code path they
do not take: the backward kernel's epilogue that adds the travelling partial dK/dV itself (``accumulate_prev``).
No two kernels wait on one another, so this is safe on a single GPU.  Test helper only.
"""
from __future__ import annotations

from typing import List

import torch

from opt_ring_flash_attn_b200 import _native


def _padded_head_dim(d):
    return 64 if d <= 64 else (128 if d <= 128 else 256)


def emulate_forward(qs: List[torch.Tensor], ks, vs, scale: float, causal: bool, kn=_native):
    W = len(qs)
    B, S, Hq, D = qs[0].shape
    dev = qs[0].device
    spad = _native.padded_seq(S)
    outs, lses, lses_padded = [], [], []
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for r in range(W):
        out = torch.empty_like(qs[r])
        lse = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
        m = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        l = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        last_step = r if causal else W - 1
        for step in range(W):
            kb = (r - step) % W
            if (not causal) or step <= r:
                single = (step == 0 and step == last_step)
                kn.fwd_hop(qs[r], ks[kb], vs[kb], None if single else acc, None if single else m,
                           None if single else l, out, lse, scale, step == 0, step == last_step,
                           causal and step == 0, status)
        outs.append(out)
        lses.append(lse[:, :, :S])
        lses_padded.append(lse)
    return outs, lses, lses_padded, status


def emulate_backward(douts, qs, ks, vs, outs, lses_padded, scale: float, causal: bool, kn=_native):
    """lses_padded: per-rank [B, Hq, Spad] fp32 as produced by the forward hop."""
    W = len(qs)
    B, S, Hq, D = qs[0].shape
    Hkv = ks[0].shape[2]
    dev = qs[0].device
    spad = _native.padded_seq(S)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    delta = [torch.empty(B, Hq, spad, dtype=torch.float32, device=dev) for _ in range(W)]
    lse2 = [torch.empty(B, Hq, spad, dtype=torch.float32, device=dev) for _ in range(W)]
    dq_acc = [torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev) for _ in range(W)]
    for r in range(W):
        kn.bwd_prepare(outs[r], douts[r], lses_padded[r], delta[r], lse2[r], dq_acc[r], status)
    # travelling dK/dV buffer of block kb; it starts at its owner (step 0) and moves to rank+1 each step
    travelling = {}
    for step in range(W):
        for r in range(W):
            kb = (r - step) % W
            if step == 0:
                travelling[kb] = torch.full((2, B, S, Hkv, D), float("nan"), dtype=torch.float32, device=dev)
            if (not causal) or step <= r:
                buf = travelling[kb]
                kn.bwd_hop(qs[r], ks[kb], vs[kb], douts[r], lse2[r], delta[r], dq_acc[r],
                           buf if step > 0 else None, buf, scale, step > 0, causal and step == 0, status)
    dqs, dks, dvs = [], [], []
    for r in range(W):
        dq = torch.empty_like(qs[r]); dk = torch.empty_like(ks[r]); dv = torch.empty_like(vs[r])
        kn.dq_finalize(dq_acc[r], dq)
        kn.cast_from_f32(travelling[r][0], dk)
        kn.cast_from_f32(travelling[r][1], dv)
        dqs.append(dq); dks.append(dk); dvs.append(dv)
    return dqs, dks, dvs, status
