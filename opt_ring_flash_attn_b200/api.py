"""Public operator: ``ring_flash_attn(q, k, v, softmax_scale, causal, zigzag, group)``.

Same name, parameter order, defaults, return value and autograd behaviour as the
reference's entry point (optimized_ring_flash_attn.py:1297-1367): forward saves
``(q, k, v, out, lse)``, backward returns ``(dq, dk, dv, None, None, None, None)``.
"""
from __future__ import annotations

import contextlib
import os
import threading
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import schedule, workspace

_SUPPORTED = (torch.bfloat16, torch.float16)

_mode = threading.local()


def _deterministic_now() -> bool:
    v = getattr(_mode, "deterministic", None)
    return (os.environ.get("RFA_B200_DETERMINISTIC", "0") == "1") if v is None else bool(v)


@contextlib.contextmanager
def deterministic(enabled: bool = True):
    """Calls of :func:`ring_flash_attn` made inside this context compute bit-reproducible gradients: the dQ
    contributions of the K/V tiles are added in a fixed order instead of by unordered fp32 reductions (the
    reference's dQ kernel is deterministic by construction, optimized_ring_flash_attn.py:730-735).  The choice is
    taken at forward time and holds for that call's backward.  ``RFA_B200_DETERMINISTIC=1`` sets the default."""
    prev = getattr(_mode, "deterministic", None)
    _mode.deterministic = enabled
    try:
        yield
    finally:
        _mode.deterministic = prev


def _balanced_now() -> bool:
    v = getattr(_mode, "balanced", None)
    return (os.environ.get("RFA_B200_BALANCE", "0") == "1") if v is None else bool(v)


@contextlib.contextmanager
def balanced(enabled: bool = True):
    """Causal calls of :func:`ring_flash_attn` on *contiguous* shards made inside this context are executed in the
    zigzag arrangement: the shards are regrouped with one exchange of half-shards, every rank then does the same
    amount of work (instead of (r + 1/2)/W of it on rank r), and results and gradients are regrouped back.  Same
    call, same layout, same results to the tolerances of the operator; pays off once the ring is larger than two.
    Needs ``S_local % 256 == 0`` (otherwise the call runs as usual).  ``RFA_B200_BALANCE=1`` sets the default."""
    prev = getattr(_mode, "balanced", None)
    _mode.balanced = enabled
    try:
        yield
    finally:
        _mode.balanced = prev


def check(what: str = "ring_flash_attn") -> None:
    """Synchronise and raise ``RuntimeError`` if a kernel of any earlier call reported a failure through its device
    status word (a bounded pipeline wait that ran out).  Without this call such a failure surfaces at the start
    of the next forward or backward that uses the same scratch; ``RFA_B200_SYNC_STATUS=1`` checks after every pass."""
    workspace.check_all(what)


def _validate(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float) -> None:
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [B, S_local, H, D]")
    if q.dtype not in _SUPPORTED or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"q, k, v must share a dtype in {_SUPPORTED}, got {q.dtype}, {k.dtype}, {v.dtype}")
    if k.shape != v.shape:
        raise ValueError(f"k and v shapes differ: {tuple(k.shape)} vs {tuple(v.shape)}")
    B, S, Hq, D = q.shape
    if k.shape[0] != B or k.shape[1] != S or k.shape[3] != D:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} disagree in batch, local sequence or head dim")
    # same contract as the reference's assert (optimized_ring_flash_attn.py:822)
    assert Hq % k.shape[2] == 0, "H_q must be a multiple of H_kv"
    if D > 256 or D % 8 != 0:
        raise ValueError(f"head_dim must be a multiple of 8 and <= 256, got {D}")
    if not (softmax_scale > 0):
        raise ValueError("softmax_scale must be positive")
    if not q.is_cuda:
        raise RuntimeError("ring_flash_attn runs on CUDA tensors only (sm_100a kernels; there is no CPU path)")


class _RingFlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, zigzag, group):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** -0.5
        if zigzag:
            assert causal, "zigzag mode requires causal=True"
        _validate(q, k, v, softmax_scale)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        ctx.balanced = bool(causal and not zigzag and _balanced_now() and schedule.can_balance(group, q.shape[1]))
        if ctx.balanced:
            out, lse, saved = schedule.balanced_forward(group, q, k, v, softmax_scale)
            ctx.save_for_backward(*saved)  # the zigzag-arranged q, k, v, out, lse
        elif zigzag:
            out, lse = schedule.zigzag_forward(group, q, k, v, softmax_scale)
            ctx.save_for_backward(q, k, v, out, lse)
        else:
            out, lse = schedule.ring_forward(group, q, k, v, softmax_scale, causal)
            ctx.save_for_backward(q, k, v, out, lse)
        ctx.zigzag = zigzag
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        ctx.group = group
        ctx.deterministic = _deterministic_now()
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse=None):
        q, k, v, out, lse = ctx.saved_tensors
        if ctx.balanced:
            dq, dk, dv = schedule.balanced_backward(ctx.group, dout, (q, k, v, out, lse), ctx.softmax_scale,
                                                    deterministic=ctx.deterministic)
        elif ctx.zigzag:
            dq, dk, dv = schedule.zigzag_backward(ctx.group, dout, q, k, v, out, lse, ctx.softmax_scale,
                                                  deterministic=ctx.deterministic)
        else:
            dq, dk, dv = schedule.ring_backward(ctx.group, dout, q, k, v, out, lse, ctx.softmax_scale, ctx.causal,
                                                deterministic=ctx.deterministic)
        return dq, dk, dv, None, None, None, None


def ring_flash_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    zigzag: bool = False,
    group: Optional[dist.ProcessGroup] = None,
) -> torch.Tensor:
    """Sequence-parallel ring flash attention.

    Args:
      q:  [B, S_local, H_q, D]   bf16/fp16
      k:  [B, S_local, H_kv, D]  bf16/fp16 (H_kv may divide H_q: GQA)
      v:  [B, S_local, H_kv, D]
      softmax_scale: 1/sqrt(D) by default.
      causal: causal mask over the full (global) sequence; rank r holds tokens
              [r*S_local, (r+1)*S_local).
      zigzag: causal load balancing: the global sequence is cut into 2W chunks and rank r holds
              [chunk_r ; chunk_{2W-1-r}] concatenated along the sequence dim (requires causal=True and
              S_local % 256 == 0).
      group:  process group (default: WORLD).  Without an initialised process
              group the call is plain single-GPU flash attention.

    Returns: out [B, S_local, H_q, D] in q's dtype.
    """
    out, _ = _RingFlashAttnFunc.apply(q, k, v, softmax_scale, causal, zigzag, group)
    return out


def ring_flash_attn_with_lse(q, k, v, softmax_scale=None, causal=False, group=None,
                             zigzag=False) -> Tuple[torch.Tensor, torch.Tensor]:
    """As :func:`ring_flash_attn`, also returning the log-sum-exp ``[B, H_q, S_local]`` (fp32, not differentiable)."""
    out, lse = _RingFlashAttnFunc.apply(q, k, v, softmax_scale, causal, zigzag, group)
    return out, lse[:, :, : q.shape[1]]
