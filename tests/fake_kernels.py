"""Test double for the hop-kernel backend: same call signatures as ``_native``, fp32 torch math on any device.

It exists so that the HOST logic (ring schedules, slot algebra, transport) can run on CPU ranks over gloo.
It follows the oracle's arithmetic (it is test infrastructure; the product never imports it).
"""
import math

import torch

LOG2E = 1.4426950408889634


def _hf(x):
    return x.float().transpose(1, 2)  # [B, H, S, D]


def _expand(x, g):
    return x if g == 1 else x.repeat_interleave(g, dim=1)


def _scores(q, k, scale, causal_diag):
    g = q.shape[2] // k.shape[2]
    s = (_hf(q) @ _expand(_hf(k), g).transpose(-2, -1)) * scale
    if causal_diag:
        S = q.shape[1]
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    return s


def pack_kv(k, v, dst, stream=None):
    dst[0].copy_(k)
    dst[1].copy_(v)


def fwd_hop(q, k, v, acc, m, l, out, lse, scale, first, last, causal_diag, status, stream=None, q_begin=0,
            kv_len=None, q_split=0, last_lo=False):
    B, S, Hq, D = q.shape
    kv_len = k.shape[1] if kv_len is None else kv_len
    g = Hq // k.shape[2]
    s = _scores(q, k, scale, causal_diag)[:, :, q_begin:, :kv_len]
    vh = _expand(_hf(v), g)[:, :, :kv_len]
    rows = slice(q_begin, S)
    blk_max = s.max(-1).values
    if first:
        m_old = torch.full_like(blk_max, float("-inf"))
        l_old = torch.zeros_like(blk_max)
        a_old = torch.zeros(B, Hq, S - q_begin, D)
    else:
        m_old = m[:, :, rows].clone()
        l_old = l[:, :, rows].clone()
        a_old = acc[: B * Hq * S * D].view(B, Hq, S, D)[:, :, rows].clone()
    m_new = torch.maximum(m_old, blk_max)
    alpha = torch.exp(torch.where(torch.isfinite(m_old), m_old - m_new, torch.full_like(m_new, float("-inf"))))
    p = torch.exp(s - m_new.unsqueeze(-1))
    l_new = l_old * alpha + p.sum(-1)
    a_new = a_old * alpha.unsqueeze(-1) + p @ vh
    # rows below q_split finish with last_lo, the others with last
    pos = torch.arange(q_begin, S)
    fin = torch.where(pos < q_split, torch.tensor(bool(last_lo)), torch.tensor(bool(last)))
    if fin.any():
        idx = pos[fin]
        sel = fin.nonzero().squeeze(-1)
        out[:, idx] = (a_new[:, :, sel] / l_new[:, :, sel].unsqueeze(-1)).transpose(1, 2).to(out.dtype)
        lse[:, :, idx] = m_new[:, :, sel] + torch.log(l_new[:, :, sel])
    if (~fin).any():
        idx = pos[~fin]
        sel = (~fin).nonzero().squeeze(-1)
        m[:, :, idx] = m_new[:, :, sel]
        l[:, :, idx] = l_new[:, :, sel]
        acc[: B * Hq * S * D].view(B, Hq, S, D)[:, :, idx] = a_new[:, :, sel]


def bwd_prepare(out, dout, lse, delta, lse2, dq_acc, status, stream=None):
    B, S, Hq, D = out.shape
    delta.zero_()
    lse2.fill_(float("inf"))
    delta[:, :, :S] = (out.float() * dout.float()).sum(-1).transpose(1, 2)
    lse2[:, :, :S] = lse[:, :, :S] * LOG2E
    if dq_acc is not None:
        dq_acc.zero_()


def bwd_hop(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, scale, accumulate_prev, causal_diag, status,
            stream=None, q_begin=0, kv_len=None, dq_order=None):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    kv_len = k.shape[1] if kv_len is None else kv_len
    g = Hq // Hkv
    rows = slice(q_begin, S)
    s = _scores(q, k, scale, causal_diag)[:, :, rows, :kv_len]
    p = torch.exp2(s * LOG2E - lse2[:, :, rows].unsqueeze(-1))
    doh = _hf(dout)[:, :, rows]
    qh = _hf(q)[:, :, rows]
    kh = _expand(_hf(k), g)[:, :, :kv_len]
    vh = _expand(_hf(v), g)[:, :, :kv_len]
    dp = doh @ vh.transpose(-2, -1)
    ds = p * (dp - delta[:, :, rows].unsqueeze(-1))
    dq_acc[: B * Hq * S * D].view(B, Hq, S, D)[:, :, rows] += (ds @ kh) * scale
    dk = ((ds.transpose(-2, -1) @ qh) * scale).view(B, Hkv, g, kv_len, D).sum(2).transpose(1, 2)
    dv = (p.transpose(-2, -1) @ doh).view(B, Hkv, g, kv_len, D).sum(2).transpose(1, 2)
    full_dk = torch.zeros(B, k.shape[1], Hkv, D)
    full_dv = torch.zeros(B, k.shape[1], Hkv, D)
    full_dk[:, :kv_len] = dk
    full_dv[:, :kv_len] = dv
    if accumulate_prev:
        full_dk = full_dk + dkdv_prev[0]
        full_dv = full_dv + dkdv_prev[1]
    dkdv_out[0].copy_(full_dk)
    dkdv_out[1].copy_(full_dv)


def dq_finalize(dq_acc, dq, stream=None):
    B, S, Hq, D = dq.shape
    dq.copy_(dq_acc[: B * Hq * S * D].view(B, Hq, S, D).transpose(1, 2).to(dq.dtype))


def dkdv_accumulate(prev, block, out, stream=None):
    out.copy_(prev + block)


def dkdv_accumulate_to16(prev, block, out, stream=None):
    out.copy_((block if prev is None else prev.float() + block).to(out.dtype))


def cast_from_f32(src, dst, stream=None):
    dst.copy_(src.to(dst.dtype))
