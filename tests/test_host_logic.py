"""Host-side pieces that need neither a GPU nor a process group."""
import torch


def test_backward_comm_dtype_follows_the_reference_switch(monkeypatch):
    """OPTIMIZED_RING_BWD_COMM_BF16=1 -> dK/dV travel in the input dtype, otherwise fp32
    (optimized_ring_flash_attn.py:205-208)."""
    from opt_ring_flash_attn_b200 import schedule

    monkeypatch.delenv("OPTIMIZED_RING_BWD_COMM_BF16", raising=False)
    assert schedule.backward_comm_dtype(torch.bfloat16) == torch.float32
    monkeypatch.setenv("OPTIMIZED_RING_BWD_COMM_BF16", "0")
    assert schedule.backward_comm_dtype(torch.float16) == torch.float32
    monkeypatch.setenv("OPTIMIZED_RING_BWD_COMM_BF16", "1")
    assert schedule.backward_comm_dtype(torch.bfloat16) == torch.bfloat16
    assert schedule.backward_comm_dtype(torch.float16) == torch.float16
    assert schedule.backward_comm_dtype(torch.float32) == torch.float32  # nothing to gain for fp32 inputs


def test_backward_workspace_buffers_by_transport_dtype():
    from opt_ring_flash_attn_b200 import workspace

    q = torch.zeros(1, 256, 4, 64, dtype=torch.bfloat16)
    k = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16)
    try:
        ws32 = workspace.backward_workspace(q, k, 2)
        assert ws32.dkdv[0].dtype == torch.float32 and ws32.block_dkdv.dtype == torch.float32
        ws16 = workspace.backward_workspace(q, k, 2, torch.bfloat16)
        assert ws16 is not ws32
        assert ws16.dkdv[0].dtype == torch.bfloat16 and ws16.dkdv[0].shape == (2, 1, 256, 2, 64)
        assert ws16.block_dkdv.dtype == torch.float32  # this hop's own block stays fp32
        assert workspace.backward_workspace(q, k, 2, torch.bfloat16) is ws16  # cached per (shapes, dtype, transport)
        ws1 = workspace.backward_workspace(q, k, 1, torch.bfloat16)
        assert ws1.dkdv[0].dtype == torch.float32 and ws1.block_dkdv is None  # one rank: nothing travels
    finally:
        workspace.clear()
