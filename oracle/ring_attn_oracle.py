"""ORACLE (test infrastructure, not a product path).

fp32 restatement of the reference's pure-PyTorch ring attention, ``ring_attn.py``
(class ``RingAttentionFunction``), used only as the checker in ``tests/``, in
``__graft_entry__.smoke()`` and as the timed CPU baseline of ``bench.py``.
Nothing under ``opt_ring_flash_attn_b200/`` imports it.

What is restated, with the lines it follows:
  * block classification skip / mask / full      ring_attn.py:50-79
  * causal mask ``k_pos > q_pos``                 ring_attn.py:82-100
  * forward online softmax over K/V blocks        ring_attn.py:386-476
  * saved statistics (row max, row sum)           ring_attn.py:484
  * backward per (Q block, K block) pair          ring_attn.py:651-725
  * delta = rowsum(dO * O)                        ring_attn.py:628-632

The ring is simulated in one process: ``W`` shards are visited in the same
order as the reference's ranks visit them (own block first, then rank-1,
rank-2, ... with wrap-around), so the floating-point accumulation order of the
forward pass is the reference's.  Adaptations the reference's file needs to
serve as an oracle for the product path are built in: fp32 compute for 16-bit
inputs, GQA (kv head = q head // group), a free ``softmax_scale`` (the
reference hard-wires D**-0.5, ring_attn.py:336), and the log-sum-exp
``max + log(sum)`` exposed as a result.

Parity of this restatement is pinned against the reference itself: the
fixtures in ``tests/golden/`` were produced by importing ``ring_attn.py`` and
running it on gloo ranks (``tests/golden/make_golden.py``), and
``tests/test_oracle.py`` compares this file to them.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


def causal_block_info(q_block: int, k_block: int, q_len: int, k_len: int, causal: bool):
    """(skip, needs_mask, q_start, k_start) for one block pair -- ring_attn.py:50-79."""
    q_start, k_start = q_block * q_len, k_block * k_len
    if not causal:
        return False, False, q_start, k_start
    if k_start >= q_start + q_len:
        return True, False, q_start, k_start
    return False, (k_start + k_len) > q_start, q_start, k_start


def _mask(q_len: int, k_len: int, q_start: int, k_start: int, device) -> torch.Tensor:
    """True where the key lies in the query's future -- ring_attn.py:95-98."""
    qp = torch.arange(q_start, q_start + q_len, device=device).view(1, 1, q_len, 1)
    kp = torch.arange(k_start, k_start + k_len, device=device).view(1, 1, 1, k_len)
    return kp > qp


def _finite_or_zero(t: torch.Tensor) -> torch.Tensor:
    return torch.where(torch.isfinite(t), t, torch.zeros_like(t))


def _heads_first(x: torch.Tensor, dtype) -> torch.Tensor:
    return x.to(dtype).transpose(1, 2).contiguous()  # [B, H, S, D]


def _expand_kv(x: torch.Tensor, group: int) -> torch.Tensor:
    return x if group == 1 else x.repeat_interleave(group, dim=1)


def ring_attn_oracle(
    q_shards: Sequence[torch.Tensor],
    k_shards: Sequence[torch.Tensor],
    v_shards: Sequence[torch.Tensor],
    dout_shards: Optional[Sequence[torch.Tensor]] = None,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
    head_chunk: int = 0,
) -> Dict[str, List[torch.Tensor]]:
    """Ring attention over ``W = len(q_shards)`` contiguous sequence shards.

    Shards are ``[B, S_local, H, D]`` (k/v may have fewer heads: GQA).  Returns
    per-rank lists ``out`` [B,S,Hq,D], ``lse`` [B,Hq,S] and, when ``dout_shards``
    is given, ``dq``, ``dk``, ``dv``; everything in ``compute_dtype``.
    ``head_chunk`` > 0 processes that many query heads at a time (bounds the
    size of the score matrices; results are identical).
    """
    W = len(q_shards)
    B, S, Hq, D = q_shards[0].shape
    Hkv = k_shards[0].shape[2]
    assert Hq % Hkv == 0
    G = Hq // Hkv
    scale = float(D) ** -0.5 if softmax_scale is None else float(softmax_scale)
    step_h = Hq if head_chunk <= 0 else max(G, head_chunk // G * G)

    res: Dict[str, List[torch.Tensor]] = {"out": [], "lse": []}
    outs = [torch.empty(B, S, Hq, D, dtype=compute_dtype, device=q_shards[0].device) for _ in range(W)]
    lses = [torch.empty(B, Hq, S, dtype=compute_dtype, device=q_shards[0].device) for _ in range(W)]
    want_grad = dout_shards is not None
    if want_grad:
        dqs = [torch.zeros(B, S, Hq, D, dtype=compute_dtype, device=q_shards[0].device) for _ in range(W)]
        dks = [torch.zeros(B, S, Hkv, D, dtype=compute_dtype, device=q_shards[0].device) for _ in range(W)]
        dvs = [torch.zeros(B, S, Hkv, D, dtype=compute_dtype, device=q_shards[0].device) for _ in range(W)]

    for h0 in range(0, Hq, step_h):
        h1 = min(Hq, h0 + step_h)
        kv0, kv1 = h0 // G, (h1 + G - 1) // G
        qh = [_heads_first(q[:, :, h0:h1], compute_dtype) for q in q_shards]
        kh = [_expand_kv(_heads_first(k[:, :, kv0:kv1], compute_dtype), G) for k in k_shards]
        vh = [_expand_kv(_heads_first(v[:, :, kv0:kv1], compute_dtype), G) for v in v_shards]
        nh = h1 - h0
        dev = qh[0].device

        stats = []
        for r in range(W):
            # ---- forward: ring_attn.py:343-476 ----
            out_acc = torch.zeros(B, nh, S, D, dtype=compute_dtype, device=dev)
            sum_acc = torch.zeros(B, nh, S, 1, dtype=compute_dtype, device=dev)
            max_acc = torch.full((B, nh, S, 1), -float("inf"), dtype=compute_dtype, device=dev)
            for step in range(W):
                kb = (r - step) % W
                skip, needs_mask, q_start, k_start = causal_block_info(r, kb, S, S, causal)
                if skip:
                    continue
                scores = (qh[r] @ kh[kb].transpose(-2, -1)) * scale
                if needs_mask:
                    scores = scores.masked_fill(_mask(S, S, q_start, k_start, dev), -float("inf"))
                blk_max = scores.max(dim=-1, keepdim=True).values
                safe_blk = _finite_or_zero(blk_max)
                e = torch.exp(scores - safe_blk)
                new_max = torch.maximum(max_acc, blk_max)
                safe_old, safe_new = _finite_or_zero(max_acc), _finite_or_zero(new_max)
                out_acc = out_acc * torch.exp(safe_old - safe_new) + (e @ vh[kb]) * torch.exp(safe_blk - safe_new)
                sum_acc = sum_acc * torch.exp(safe_old - safe_new) + e.sum(-1, keepdim=True) * torch.exp(safe_blk - safe_new)
                max_acc = new_max
            sum_acc = torch.where(sum_acc == 0, torch.ones_like(sum_acc), sum_acc)
            out_head = out_acc / sum_acc
            outs[r][:, :, h0:h1] = out_head.transpose(1, 2)
            lses[r][:, h0:h1] = (max_acc + torch.log(sum_acc)).squeeze(-1)
            stats.append((out_head, sum_acc, max_acc))

        if not want_grad:
            continue
        # ---- backward: ring_attn.py:606-725 (K/V stay put, query-side state visits them) ----
        doh = [_heads_first(d[:, :, h0:h1], compute_dtype) for d in dout_shards]
        deltas = [(doh[r] * stats[r][0]).sum(-1, keepdim=True) for r in range(W)]
        dk_h = [torch.zeros(B, nh, S, D, dtype=compute_dtype, device=dev) for _ in range(W)]
        dv_h = [torch.zeros(B, nh, S, D, dtype=compute_dtype, device=dev) for _ in range(W)]
        dq_h = [torch.zeros(B, nh, S, D, dtype=compute_dtype, device=dev) for _ in range(W)]
        for kr in range(W):          # rank that owns the K/V block
            for step in range(W):    # query block (kr - step) visits it at this step
                qb = (kr - step) % W
                skip, needs_mask, q_start, k_start = causal_block_info(qb, kr, S, S, causal)
                if skip:
                    continue
                _, sum_q, max_q = stats[qb]
                scores = (qh[qb] @ kh[kr].transpose(-2, -1)) * scale
                if needs_mask:
                    scores = scores.masked_fill(_mask(S, S, q_start, k_start, dev), -float("inf"))
                probs = torch.exp(scores - max_q) / sum_q
                dv_h[kr] += probs.transpose(-2, -1) @ doh[qb]
                dprobs = doh[qb] @ vh[kr].transpose(-2, -1)
                dscores = probs * (dprobs - deltas[qb])
                dk_h[kr] += (dscores.transpose(-2, -1) @ qh[qb]) * scale
                dq_h[qb] += (dscores @ kh[kr]) * scale
        for r in range(W):
            dqs[r][:, :, h0:h1] = dq_h[r].transpose(1, 2)
            # fold the expanded heads back onto their kv head (autograd of repeat_interleave)
            dks[r][:, :, kv0:kv1] += dk_h[r].view(B, kv1 - kv0, G, S, D).sum(2).transpose(1, 2)
            dvs[r][:, :, kv0:kv1] += dv_h[r].view(B, kv1 - kv0, G, S, D).sum(2).transpose(1, 2)

    res["out"], res["lse"] = outs, lses
    if want_grad:
        res["dq"], res["dk"], res["dv"] = dqs, dks, dvs
    return res


def dense_attention(q, k, v, causal: bool, softmax_scale: Optional[float] = None, compute_dtype=torch.float32):
    """Plain softmax attention over the full sequence (the check the reference's own tests use,
    ring_attn.py:826-846).  Returns (out [B,S,Hq,D], lse [B,Hq,S])."""
    B, S, Hq, D = q.shape
    G = Hq // k.shape[2]
    scale = float(D) ** -0.5 if softmax_scale is None else float(softmax_scale)
    qh = _heads_first(q, compute_dtype)
    kh = _expand_kv(_heads_first(k, compute_dtype), G)
    vh = _expand_kv(_heads_first(v, compute_dtype), G)
    scores = (qh @ kh.transpose(-2, -1)) * scale
    if causal:
        scores = scores.masked_fill(_mask(S, S, 0, 0, q.device), -float("inf"))
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.softmax(scores, dim=-1) @ vh
    return out.transpose(1, 2).contiguous(), lse


def shard(x: torch.Tensor, world_size: int) -> List[torch.Tensor]:
    """Contiguous sequence shards in rank order (test_optimized_ring_flash_attn.py:55-56)."""
    return [c.contiguous() for c in x.chunk(world_size, dim=1)]


def zigzag_shard(x: torch.Tensor, world_size: int) -> List[torch.Tensor]:
    """Zigzag layout of the reference (optimized_ring_flash_attn.py:1122-1124): the sequence is cut into 2W chunks
    and rank r holds ``[chunk_r ; chunk_{2W-1-r}]``."""
    c = x.chunk(2 * world_size, dim=1)
    return [torch.cat([c[r], c[2 * world_size - 1 - r]], dim=1).contiguous() for r in range(world_size)]


def zigzag_oracle(q, k, v, dout, world_size: int, softmax_scale: Optional[float] = None,
                  compute_dtype: torch.dtype = torch.float32, head_chunk: int = 0) -> Dict[str, List[torch.Tensor]]:
    """Expected per-rank results of causal attention in the zigzag layout: the pinned contiguous-shard oracle is
    run over 2W chunks of the full sequence and its per-chunk results are regrouped rank by rank."""
    W2 = 2 * world_size
    res = ring_attn_oracle(shard(q, W2), shard(k, W2), shard(v, W2), shard(dout, W2) if dout is not None else None,
                           causal=True, softmax_scale=softmax_scale, compute_dtype=compute_dtype,
                           head_chunk=head_chunk)
    out: Dict[str, List[torch.Tensor]] = {}
    for key, parts in res.items():
        dim = 2 if key == "lse" else 1
        out[key] = [torch.cat([parts[r], parts[W2 - 1 - r]], dim=dim) for r in range(world_size)]
    return out


def make_inputs(seed: int, B: int, S_total: int, Hq: int, Hkv: int, D: int, std: float = 1.0,
                dtype: torch.dtype = torch.float32):
    """Seeded full-sequence q, k, v, dout drawn in that order on the CPU generator
    (the reference's harness: test_optimized_ring_flash_attn.py:143-153)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    q = torch.randn(B, S_total, Hq, D, generator=g) * std
    k = torch.randn(B, S_total, Hkv, D, generator=g) * std
    v = torch.randn(B, S_total, Hkv, D, generator=g) * std
    dout = torch.randn(B, S_total, Hq, D, generator=g)
    return q.to(dtype), k.to(dtype), v.to(dtype), dout.to(dtype)
