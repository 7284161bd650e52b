"""Tensor-core operand paths of the hop kernels, one 128x128x128 product each (bit patterns of bf16
inputs, fp32 accumulate; compared with a torch fp32 matmul of the same bf16 values)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
def test_mma_probe(mode):
    from opt_ring_flash_attn_b200 import _native

    torch.manual_seed(mode)
    dev = torch.device("cuda:0")
    a = torch.randn(128, 128, device=dev).to(torch.bfloat16)
    b = torch.randn(128, 128, device=dev).to(torch.bfloat16)
    c = torch.full((128, 128), float("nan"), device=dev, dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _native.mma_probe(mode, a, b, c, status)
    torch.cuda.synchronize()
    _native.check_status(status, f"mma probe mode {mode}")
    af, bf = a.float(), b.float()
    ref = {0: af @ bf.T, 1: af @ bf, 2: af @ bf, 3: af.T @ bf, 4: af @ bf.T}[mode]
    err = (c - ref).abs().max().item()
    assert err < 1e-3, f"mode {mode}: max abs err {err}"


def test_bounded_wait_runs_out_and_reports_through_the_status_word():
    """A pipeline wait that nothing satisfies: the kernel gives up after its time limit (about two seconds), writes the
    time-out code into the status word and returns -- no trap, no fault; later hop launches that share the word return
    at once, and once the word is cleared the same context computes correct results again."""
    import time

    from opt_ring_flash_attn_b200 import _native
    from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle

    dev = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    _native.wait_timeout_probe(status)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) == 1 and 1.0 < waited < 10.0
    with pytest.raises(RuntimeError, match="device status 1"):
        _native.check_status(status, "probe")
    # a hop launched with the word set does nothing
    q, k, v, _ = (x.to(dev) for x in make_inputs(3, 1, 256, 2, 2, 64, dtype=torch.bfloat16))
    out = torch.full_like(q, 7.0)
    lse = torch.empty(1, 2, 256, dtype=torch.float32, device=dev)
    _native.fwd_hop(q, k, v, None, None, None, out, lse, 0.125, True, True, True, status)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full_like(q, 7.0))
    # cleared: the context is intact
    status.zero_()
    _native.fwd_hop(q, k, v, None, None, None, out, lse, 0.125, True, True, True, status)
    torch.cuda.synchronize()
    ref = ring_attn_oracle([q], [k], [v], None, causal=True, softmax_scale=0.125)
    assert (out.float() - ref["out"][0]).abs().max().item() <= 1e-2 and int(status.item()) == 0
