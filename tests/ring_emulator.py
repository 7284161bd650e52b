"""Runs the W-rank ring schedule on ONE device by visiting the ranks one after another.

Each emulated rank issues exactly the hop-kernel calls that ``schedule.ring_forward`` /
``schedule.ring_backward`` issue for it (same first/last/causal flags, same buffer roles); the
transport is replaced by handing the packed buffers from one emulated rank to the next.  No two
kernels wait on one another, so this is safe on a single GPU.  Test helper only.
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


def emulate_zigzag(qs, ks, vs, douts, scale: float, kn=_native):
    """Zigzag schedule (schedule.zigzag_forward / zigzag_backward) rank by rank on one device.
    qs/ks/vs/douts are the zigzag-arranged shards.  Returns (outs, lses, dqs, dks, dvs, status)."""
    W = len(qs)
    B, S, Hq, D = qs[0].shape
    Hkv = ks[0].shape[2]
    dev = qs[0].device
    half = S // 2
    spad = _native.padded_seq(S)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    outs, lses_pad = [], []
    for r in range(W):
        out = torch.empty_like(qs[r])
        lse = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        acc = torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev)
        m = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        l = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        for step in range(W):
            kb = (r - step) % W
            last_hi, last_lo = step == W - 1, step == r
            if step == 0:
                kn.fwd_hop(qs[r], ks[kb], vs[kb], acc, m, l, out, lse, scale, True, last_hi, True, status,
                           q_begin=0, kv_len=S, q_split=half, last_lo=last_lo)
            elif step <= r:
                kn.fwd_hop(qs[r], ks[kb], vs[kb], acc, m, l, out, lse, scale, False, last_hi, False, status,
                           q_begin=0, kv_len=half, q_split=half, last_lo=last_lo)
            else:
                kn.fwd_hop(qs[r], ks[kb], vs[kb], acc, m, l, out, lse, scale, False, last_hi, False, status,
                           q_begin=half, kv_len=S, q_split=half, last_lo=False)
        outs.append(out)
        lses_pad.append(lse)
    delta = [torch.empty(B, Hq, spad, dtype=torch.float32, device=dev) for _ in range(W)]
    lse2 = [torch.empty(B, Hq, spad, dtype=torch.float32, device=dev) for _ in range(W)]
    dq_acc = [torch.empty(B * Hq * spad * _padded_head_dim(D), dtype=torch.float32, device=dev) for _ in range(W)]
    for r in range(W):
        kn.bwd_prepare(outs[r], douts[r], lses_pad[r], delta[r], lse2[r], dq_acc[r], status)
    travelling = {}
    block = torch.empty(2, B, S, Hkv, D, dtype=torch.float32, device=dev)
    for step in range(W):
        for r in range(W):
            kb = (r - step) % W
            if step == 0:
                travelling[kb] = torch.full((2, B, S, Hkv, D), float("nan"), dtype=torch.float32, device=dev)
                kn.bwd_hop(qs[r], ks[kb], vs[kb], douts[r], lse2[r], delta[r], dq_acc[r], None, travelling[kb], scale,
                           False, True, status, q_begin=0, kv_len=S)
                continue
            block.fill_(float("nan"))
            if step <= r:
                kn.bwd_hop(qs[r], ks[kb], vs[kb], douts[r], lse2[r], delta[r], dq_acc[r], None, block, scale, False,
                           False, status, q_begin=0, kv_len=half)
            else:
                kn.bwd_hop(qs[r], ks[kb], vs[kb], douts[r], lse2[r], delta[r], dq_acc[r], None, block, scale, False,
                           False, status, q_begin=half, kv_len=S)
            kn.dkdv_accumulate(travelling[kb], block, travelling[kb])
    dqs, dks, dvs = [], [], []
    for r in range(W):
        dq = torch.empty_like(qs[r]); dk = torch.empty_like(ks[r]); dv = torch.empty_like(vs[r])
        kn.dq_finalize(dq_acc[r], dq)
        kn.cast_from_f32(travelling[r][0], dk)
        kn.cast_from_f32(travelling[r][1], dv)
        dqs.append(dq); dks.append(dk); dvs.append(dv)
    return outs, [x[:, :, :S] for x in lses_pad], dqs, dks, dvs, status
