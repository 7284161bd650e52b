"""The in-process ring (tests/inproc_ring.py) on CPU tensors with the fp32 test double for the kernels: the same
product schedules the GPU parity tests drive, so a fault in the hand-over protocol shows up here without a GPU."""
import pytest
import torch

from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle, shard, zigzag_oracle, zigzag_shard


def _rel(a, b):
    return ((a.float() - b).norm() / b.norm()).item()


@pytest.mark.parametrize("W,causal,Hq,Hkv,wire16", [(2, True, 2, 2, False), (3, True, 4, 2, False),
                                                    (3, False, 2, 1, False), (4, True, 2, 2, True)])
def test_contiguous_schedule_in_process(W, causal, Hq, Hkv, wire16, monkeypatch):
    import fake_kernels
    from inproc_ring import run_ring

    monkeypatch.setenv("OPTIMIZED_RING_BWD_COMM_BF16", "1" if wire16 else "0")
    B, S, D, scale = 1, 64, 16, 0.3
    q, k, v, dout = make_inputs(51, B, S * W, Hq, Hkv, D, dtype=torch.bfloat16)
    qs, ks, vs, dos = shard(q, W), shard(k, W), shard(v, W), shard(dout, W)
    outs, lses, dqs, dks, dvs = run_ring(W, torch.device("cpu"), qs, ks, vs, dos, scale, causal, kernels=fake_kernels)
    ref = ring_attn_oracle(qs, ks, vs, dos, causal=causal, softmax_scale=scale)
    for r in range(W):
        assert (outs[r].float() - ref["out"][r]).abs().max().item() <= 1e-2
        assert (lses[r] - ref["lse"][r]).abs().max().item() <= 1e-3
        assert _rel(dqs[r], ref["dq"][r]) <= 2e-2
        assert _rel(dks[r], ref["dk"][r]) <= 2e-2
        assert _rel(dvs[r], ref["dv"][r]) <= 2e-2


def test_zigzag_schedule_in_process():
    import fake_kernels
    from inproc_ring import run_ring

    W, B, S, Hq, Hkv, D, scale = 3, 1, 256, 2, 1, 16, 0.25
    q, k, v, dout = make_inputs(71, B, S * W, Hq, Hkv, D, dtype=torch.bfloat16)
    qs, ks, vs, dos = (zigzag_shard(x, W) for x in (q, k, v, dout))
    outs, lses, dqs, dks, dvs = run_ring(W, torch.device("cpu"), qs, ks, vs, dos, scale, True, kernels=fake_kernels,
                                         zigzag=True)
    ref = zigzag_oracle(q, k, v, dout, W, softmax_scale=scale)
    for r in range(W):
        assert (outs[r].float() - ref["out"][r]).abs().max().item() <= 1e-2
        assert (lses[r] - ref["lse"][r]).abs().max().item() <= 1e-3
        assert _rel(dqs[r], ref["dq"][r]) <= 2e-2
        assert _rel(dks[r], ref["dk"][r]) <= 2e-2
        assert _rel(dvs[r], ref["dv"][r]) <= 2e-2


def test_each_rank_has_its_own_scratch():
    """Ranks driven by one process must not share a workspace slot (they run concurrently)."""
    from inproc_ring import InProcRing
    from opt_ring_flash_attn_b200 import workspace

    ring = InProcRing(2)
    q = torch.zeros(1, 128, 2, 16, dtype=torch.bfloat16)
    a = workspace.forward_workspace(q, q, 2, owner=ring.handles[0].workspace_key)
    b = workspace.forward_workspace(q, q, 2, owner=ring.handles[1].workspace_key)
    try:
        assert a is not b and a.acc.data_ptr() != b.acc.data_ptr()
        assert workspace.forward_workspace(q, q, 2, owner=ring.handles[0].workspace_key) is a
    finally:
        workspace.clear()
