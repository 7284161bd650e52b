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
