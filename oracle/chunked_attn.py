"""ORACLE (test infrastructure, not a product path): slice-wise fp32 restatement for shards too long to check whole.

``ring_attn_oracle`` materialises ``[B, H, S, S]`` score matrices, which stops being possible long before the
long-context workload (S_local = 131072: 4.4 TB).  This file restates the same arithmetic for *slices* of a causal
single-shard problem: a block of query rows against all keys they can see, or a block of keys against all queries
that can see them.  Same formulas as the reference's pure-PyTorch path:

  * scores, causal mask ``k_pos > q_pos``, softmax statistics      ring_attn.py:413-458
  * probs = exp(scores - max) / sum, dV, dP, dS = P o (dP - delta), dK, dQ      ring_attn.py:678-712
  * delta = rowsum(dO * O)                                          ring_attn.py:628-632

with the log-sum-exp ``max + log(sum)`` folded into one statistic.  ``tests/test_oracle.py`` holds it to the pinned
``ring_attn_oracle`` on small shapes; only tests import it.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _hf(x: torch.Tensor) -> torch.Tensor:
    return x.float().transpose(1, 2)  # [B, H, S, D]


def _expand(x: torch.Tensor, g: int) -> torch.Tensor:
    return x if g == 1 else x.repeat_interleave(g, dim=1)


def forward_rows(q, k, v, scale: float, row0: int, row1: int, causal: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows ``[row0, row1)`` of the attention output and of the LSE: ``(out [B, rows, Hq, D], lse [B, Hq, rows])``,
    fp32.  Scores of these rows against every key they can see are formed at once (ring_attn.py:413-458)."""
    g = q.shape[2] // k.shape[2]
    last_key = row1 if causal else k.shape[1]
    qh = _hf(q[:, row0:row1])
    kh = _expand(_hf(k[:, :last_key]), g)
    vh = _expand(_hf(v[:, :last_key]), g)
    s = (qh @ kh.transpose(-2, -1)) * scale
    if causal:
        qp = torch.arange(row0, row1, device=q.device).view(1, 1, -1, 1)
        kp = torch.arange(0, last_key, device=q.device).view(1, 1, 1, -1)
        s = s.masked_fill(kp > qp, float("-inf"))
    m = s.max(-1, keepdim=True).values
    e = torch.exp(s - m)
    l = e.sum(-1, keepdim=True)
    out = (e @ vh) / l
    return out.transpose(1, 2).contiguous(), (m + torch.log(l)).squeeze(-1)


def full_stats(q, k, v, dout, scale: float, causal: bool = True, row_block: int = 512):
    """``(lse [B, Hq, S], delta [B, Hq, S])`` for every row, block of rows by block of rows."""
    B, S, Hq, D = q.shape
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    for r0 in range(0, S, row_block):
        r1 = min(S, r0 + row_block)
        out, l = forward_rows(q, k, v, scale, r0, r1, causal)
        lse[:, :, r0:r1] = l
        delta[:, :, r0:r1] = (out * dout[:, r0:r1].float()).sum(-1).transpose(1, 2)
    return lse, delta


def _probs_and_dscores(q, k, v, dout, lse, delta, scale, r0, r1, k0, k1, causal):
    """P and dS for query rows [r0, r1) x keys [k0, k1) (ring_attn.py:678-705), heads first."""
    g = q.shape[2] // k.shape[2]
    qh = _hf(q[:, r0:r1])
    doh = _hf(dout[:, r0:r1])
    kh = _expand(_hf(k[:, k0:k1]), g)
    vh = _expand(_hf(v[:, k0:k1]), g)
    s = (qh @ kh.transpose(-2, -1)) * scale
    if causal:
        qp = torch.arange(r0, r1, device=q.device).view(1, 1, -1, 1)
        kp = torch.arange(k0, k1, device=q.device).view(1, 1, 1, -1)
        s = s.masked_fill(kp > qp, float("-inf"))
    p = torch.exp(s - lse[:, :, r0:r1].unsqueeze(-1))
    dp = doh @ vh.transpose(-2, -1)
    ds = p * (dp - delta[:, :, r0:r1].unsqueeze(-1))
    return p, ds, qh, doh, kh


def dq_rows(q, k, v, dout, lse, delta, scale: float, row0: int, row1: int, causal: bool = True) -> torch.Tensor:
    """dQ of rows ``[row0, row1)``: ``[B, rows, Hq, D]`` fp32."""
    last_key = row1 if causal else k.shape[1]
    _, ds, _, _, kh = _probs_and_dscores(q, k, v, dout, lse, delta, scale, row0, row1, 0, last_key, causal)
    return ((ds @ kh) * scale).transpose(1, 2).contiguous()


def dkdv_keys(q, k, v, dout, lse, delta, scale: float, key0: int, key1: int, causal: bool = True,
              row_block: int = 8192) -> Tuple[torch.Tensor, torch.Tensor]:
    """dK and dV of keys ``[key0, key1)``, summed over every query that can see them: two ``[B, keys, Hkv, D]`` fp32."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    n = key1 - key0
    dk = torch.zeros(B, Hq, n, D, dtype=torch.float32, device=q.device)
    dv = torch.zeros(B, Hq, n, D, dtype=torch.float32, device=q.device)
    first_row = key0 if causal else 0
    for r0 in range(first_row, S, row_block):
        r1 = min(S, r0 + row_block)
        p, ds, qh, doh, _ = _probs_and_dscores(q, k, v, dout, lse, delta, scale, r0, r1, key0, key1, causal)
        dv += p.transpose(-2, -1) @ doh
        dk += (ds.transpose(-2, -1) @ qh) * scale
    fold = lambda x: x.view(B, Hkv, g, n, D).sum(2).transpose(1, 2).contiguous()  # noqa: E731
    return fold(dk), fold(dv)
