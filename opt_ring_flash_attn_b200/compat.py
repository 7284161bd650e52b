"""Wrappers with the call signatures of the reference's baseline file (the zhuzilin-style API,
ring_flash_attn.py:385-463), so that callers of ``ring_flash_attn_func`` / ``_kvpacked_func`` /
``_qkvpacked_func`` can switch without code changes.

Only what this build computes is accepted: dropout 0, no sliding window, no ALiBi.  Anything else raises
``NotImplementedError`` instead of being silently ignored.  ``return_attn_probs=True`` returns
``(out, softmax_lse, None)`` like the reference (ring_flash_attn.py:362).  ``deterministic=True``
(ring_flash_attn.py:179, 245) selects the ordered dQ reductions: gradients are bit-reproducible run to run.
"""
from __future__ import annotations

import contextlib

from .api import deterministic as _deterministic
from .api import ring_flash_attn, ring_flash_attn_with_lse


def _check_unsupported(dropout_p, window_size, alibi_slopes):
    if dropout_p != 0.0:
        raise NotImplementedError("dropout_p != 0 is not supported")
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("sliding-window attention is not supported")
    if alibi_slopes is not None:
        raise NotImplementedError("ALiBi is not supported")


def ring_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                         alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None):
    _check_unsupported(dropout_p, window_size, alibi_slopes)
    # False leaves the surrounding default (context manager or RFA_B200_DETERMINISTIC) in force
    with (_deterministic(True) if deterministic else contextlib.nullcontext()):
        if return_attn_probs:
            out, lse = ring_flash_attn_with_lse(q, k, v, softmax_scale=softmax_scale, causal=causal, group=group)
            return out, lse, None
        return ring_flash_attn(q, k, v, softmax_scale=softmax_scale, causal=causal, group=group)


def ring_flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                                  alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None):
    """``kv`` is ``[B, S_local, 2, H_kv, D]``."""
    return ring_flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale, causal, window_size,
                                alibi_slopes, deterministic, return_attn_probs, group)


def ring_flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                                   alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None):
    """``qkv`` is ``[B, S_local, 3, H, D]``."""
    return ring_flash_attn_func(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p, softmax_scale, causal,
                                window_size, alibi_slopes, deterministic, return_attn_probs, group)
