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


def fwd_hop(q, k, v, acc, m, l, out, lse, scale, first, last, causal_diag, status, stream=None):
    B, S, Hq, D = q.shape
    g = Hq // k.shape[2]
    s = _scores(q, k, scale, causal_diag)
    vh = _expand(_hf(v), g)
    blk_max = s.max(-1).values
    if first:
        m_old = torch.full_like(blk_max, float("-inf"))
        l_old = torch.zeros_like(blk_max)
        a_old = torch.zeros(B, Hq, S, D)
    else:
        m_old = m[:, :, :S].clone()
        l_old = l[:, :, :S].clone()
        a_old = acc[: B * Hq * S * D].view(B, Hq, S, D).clone()
    m_new = torch.maximum(m_old, blk_max)
    alpha = torch.exp(torch.where(torch.isfinite(m_old), m_old - m_new, torch.full_like(m_new, float("-inf"))))
    p = torch.exp(s - m_new.unsqueeze(-1))
    l_new = l_old * alpha + p.sum(-1)
    a_new = a_old * alpha.unsqueeze(-1) + p @ vh
    if last:
        out.copy_((a_new / l_new.unsqueeze(-1)).transpose(1, 2).to(out.dtype))
        lse[:, :, :S] = m_new + torch.log(l_new)
    else:
        m[:, :, :S] = m_new
        l[:, :, :S] = l_new
        acc[: B * Hq * S * D].view(B, Hq, S, D).copy_(a_new)


def bwd_prepare(out, dout, lse, delta, lse2, dq_acc, status, stream=None):
    B, S, Hq, D = out.shape
    delta.zero_()
    lse2.fill_(float("inf"))
    delta[:, :, :S] = (out.float() * dout.float()).sum(-1).transpose(1, 2)
    lse2[:, :, :S] = lse[:, :, :S] * LOG2E
    if dq_acc is not None:
        dq_acc.zero_()


def bwd_hop(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, scale, accumulate_prev, causal_diag, status,
            stream=None):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    s = _scores(q, k, scale, causal_diag)
    p = torch.exp2(s * LOG2E - lse2[:, :, :S].unsqueeze(-1))
    doh = _hf(dout)
    dp = doh @ _expand(_hf(v), g).transpose(-2, -1)
    ds = p * (dp - delta[:, :, :S].unsqueeze(-1))
    dq_acc[: B * Hq * S * D].view(B, Hq, S, D).add_((ds @ _expand(_hf(k), g)) * scale)
    dk = ((ds.transpose(-2, -1) @ _hf(q)) * scale).view(B, Hkv, g, S, D).sum(2).transpose(1, 2)
    dv = (p.transpose(-2, -1) @ doh).view(B, Hkv, g, S, D).sum(2).transpose(1, 2)
    if accumulate_prev:
        dk = dk + dkdv_prev[0]
        dv = dv + dkdv_prev[1]
    dkdv_out[0].copy_(dk)
    dkdv_out[1].copy_(dv)


def dq_finalize(dq_acc, dq, stream=None):
    B, S, Hq, D = dq.shape
    dq.copy_(dq_acc[: B * Hq * S * D].view(B, Hq, S, D).transpose(1, 2).to(dq.dtype))


def dkdv_accumulate(prev, block, out, stream=None):
    out.copy_(prev + block)


def cast_from_f32(src, dst, stream=None):
    dst.copy_(src.to(dst.dtype))
