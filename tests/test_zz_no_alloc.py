"""The allocation-free backward hop against the regular one.

``rfa_bwd_hop_noalloc`` is for hosts that may not call cudaMalloc (a fully pre-assigned memory pool, a
plugin boundary that only hands tensors in and out).  It keeps its fp32 dQ accumulator in a fixed
array inside the library, so this test checks what that changes: the result must equal the regular
entry point's (``rfa_bwd_hop`` + ``rfa_bwd_dq_finalize`` with a caller-allocated accumulator) and the
oracle's, and a second call must not see what the first one left in the shared array.  Shapes beyond the array are
refused.  The file name sorts last so that a run stopping at the first failure has already covered
everything else.
"""
import pytest
import torch

from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle

pytestmark = pytest.mark.gpu

GRAD_REL_L2 = 2e-2  # tolerance of the parity tests for dQ/dK/dV


def _rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def _prepare(seed, B, S, Hq, Hkv, D, causal):
    from opt_ring_flash_attn_b200 import _native

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(seed, B, S, Hq, Hkv, D, dtype=torch.bfloat16))
    spad = _native.padded_seq(S)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    scale = D ** -0.5
    _native.fwd_hop(q, k, v, None, None, None, out, lse, scale, True, True, causal, status)
    delta = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
    lse2 = torch.empty_like(delta)
    _native.bwd_prepare(out, dout, lse, delta, lse2, None, status)
    return q, k, v, dout, lse2, delta, scale, status


def _regular(q, k, v, dout, lse2, delta, scale, causal, status):
    from opt_ring_flash_attn_b200 import _native

    B, S, Hq, D = q.shape
    acc = torch.zeros(_native.dq_acc_elems(B, S, Hq, D), dtype=torch.float32, device=q.device)
    dkdv = torch.empty(2, *k.shape, dtype=torch.float32, device=q.device)
    dq = torch.empty_like(q)
    _native.bwd_hop(q, k, v, dout, lse2, delta, acc, None, dkdv, scale, False, causal, status)
    _native.dq_finalize(acc, dq)
    return dq, dkdv


def test_noalloc_matches_regular_entry_point_twice():
    from opt_ring_flash_attn_b200 import _native

    # two different problems back to back: the second call must start from a cleared accumulator
    for seed, (B, S, Hq, Hkv, D, causal) in enumerate([(1, 384, 4, 2, 128, True), (2, 200, 2, 2, 64, False)]):
        q, k, v, dout, lse2, delta, scale, status = _prepare(40 + seed, B, S, Hq, Hkv, D, causal)
        dq_ref, dkdv_ref = _regular(q, k, v, dout, lse2, delta, scale, causal, status)
        dq = torch.full_like(q, float("nan"))
        dkdv = torch.full((2, *k.shape), float("nan"), dtype=torch.float32, device=q.device)
        _native.bwd_hop_noalloc(q, k, v, dout, lse2, delta, dq, None, dkdv, scale, False, causal, status)
        torch.cuda.synchronize()
        _native.check_status(status, "bwd_hop_noalloc")
        assert torch.isfinite(dq.float()).all() and torch.isfinite(dkdv).all()
        assert torch.equal(dkdv, dkdv_ref)                 # dK/dV do not touch the scratch: same bits
        assert _rel_l2(dq, dq_ref) <= GRAD_REL_L2          # dQ: fp32 reductions land in a different order
        # and directly against the oracle (one rank: this hop is the whole backward pass)
        ref = ring_attn_oracle([q], [k], [v], [dout], causal=causal)
        assert _rel_l2(dq, ref["dq"][0]) <= GRAD_REL_L2
        assert _rel_l2(dkdv[0], ref["dk"][0]) <= GRAD_REL_L2
        assert _rel_l2(dkdv[1], ref["dv"][0]) <= GRAD_REL_L2


def test_noalloc_rejects_shapes_beyond_the_array():
    from opt_ring_flash_attn_b200 import _native

    lib = _native.load()
    limit = lib.rfa_noalloc_scratch_bytes()
    B, S, Hq, D = 1, 16384, 16, 128
    assert _native.dq_acc_elems(B, S, Hq, D) * 4 > limit
    dev = torch.device("cuda:0")
    buf = torch.zeros(64, dtype=torch.float32, device=dev)  # never dereferenced: the call must refuse first
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = buf.data_ptr()
    rc = lib.rfa_bwd_hop_noalloc(p, p, p, p, p, p, p, None, p, B, S, S, Hq, Hq, D, 0, 0.1, 0, 1,
                                 status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -5, f"expected RFA_ERR_TOO_LARGE, got {rc}"
    torch.cuda.synchronize()
    assert int(status.item()) == 0
