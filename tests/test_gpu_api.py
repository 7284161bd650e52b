"""The public operator on one GPU (no process group): autograd, repeated calls, argument checks."""
import pytest
import torch

from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle

pytestmark = pytest.mark.gpu


def _rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_autograd_single_gpu():
    from opt_ring_flash_attn_b200 import ring_flash_attn, ring_flash_attn_with_lse

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(21, 2, 384, 4, 2, 128, dtype=torch.bfloat16))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    out = ring_flash_attn(q, k, v, causal=True)
    out.backward(dout)
    ref = ring_attn_oracle([q.detach()], [k.detach()], [v.detach()], [dout], causal=True)
    assert (out.float() - ref["out"][0]).abs().max().item() <= 1e-2
    assert _rel_l2(q.grad, ref["dq"][0]) <= 2e-2
    assert _rel_l2(k.grad, ref["dk"][0]) <= 2e-2
    assert _rel_l2(v.grad, ref["dv"][0]) <= 2e-2
    _, lse = ring_flash_attn_with_lse(q.detach(), k.detach(), v.detach(), causal=True)
    assert (lse - ref["lse"][0]).abs().max().item() <= 1e-3


def test_two_calls_do_not_alias_saved_tensors():
    """Two same-shape calls (two layers) before either backward: the first call's saved out/lse must survive."""
    from opt_ring_flash_attn_b200 import ring_flash_attn

    dev = torch.device("cuda:0")
    a = [x.to(dev) for x in make_inputs(30, 1, 256, 2, 2, 64, dtype=torch.bfloat16)]
    b = [x.to(dev) for x in make_inputs(31, 1, 256, 2, 2, 64, dtype=torch.bfloat16)]
    for t in a[:3] + b[:3]:
        t.requires_grad_(True)
    out_a = ring_flash_attn(a[0], a[1], a[2], causal=True)
    out_b = ring_flash_attn(b[0], b[1], b[2], causal=True)
    (out_a.float() * a[3].float()).sum().backward()
    (out_b.float() * b[3].float()).sum().backward()
    for inp in (a, b):
        ref = ring_attn_oracle([inp[0].detach()], [inp[1].detach()], [inp[2].detach()], [inp[3]], causal=True)
        assert _rel_l2(inp[0].grad, ref["dq"][0]) <= 2e-2
        assert _rel_l2(inp[1].grad, ref["dk"][0]) <= 2e-2
        assert _rel_l2(inp[2].grad, ref["dv"][0]) <= 2e-2


def test_argument_errors():
    from opt_ring_flash_attn_b200 import ring_flash_attn

    dev = torch.device("cuda:0")
    q = torch.zeros(1, 128, 4, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(AssertionError):
        ring_flash_attn(q, q, q, causal=False, zigzag=True)
    with pytest.raises(AssertionError):
        ring_flash_attn(q, q[:, :, :3], q[:, :, :3])
    with pytest.raises(ValueError):
        ring_flash_attn(q.float(), q.float(), q.float())
    with pytest.raises(ValueError):
        ring_flash_attn(q[..., :60], q[..., :60], q[..., :60])


def test_zigzag_flag_single_gpu_equals_causal():
    """With one rank the zigzag layout is the plain sequence: zigzag=True must equal causal=True."""
    from opt_ring_flash_attn_b200 import ring_flash_attn

    dev = torch.device("cuda:0")
    q, k, v, _ = (x.to(dev) for x in make_inputs(34, 1, 256, 2, 2, 64, dtype=torch.bfloat16))
    assert torch.equal(ring_flash_attn(q, k, v, causal=True, zigzag=True), ring_flash_attn(q, k, v, causal=True))


def test_non_contiguous_inputs():
    from opt_ring_flash_attn_b200 import ring_flash_attn

    dev = torch.device("cuda:0")
    q, k, v, _ = (x.to(dev) for x in make_inputs(33, 1, 128, 2, 2, 64, dtype=torch.bfloat16))
    qt = q.transpose(1, 2).contiguous().transpose(1, 2)  # same values, permuted strides
    assert not qt.is_contiguous()
    o1 = ring_flash_attn(q, k, v)
    o2 = ring_flash_attn(qt, k, v)
    assert torch.equal(o1, o2)


def test_baseline_style_wrappers():
    """The zhuzilin-style entry points give the operator's results (packed inputs are strided views)."""
    import opt_ring_flash_attn_b200 as rfa

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(35, 1, 256, 4, 4, 64, dtype=torch.bfloat16))
    base = rfa.ring_flash_attn(q, k, v, causal=True)
    assert torch.equal(rfa.ring_flash_attn_func(q, k, v, causal=True), base)
    kv = torch.stack([k, v], dim=2)
    assert torch.equal(rfa.ring_flash_attn_kvpacked_func(q, kv, causal=True), base)
    qkv = torch.stack([q, k, v], dim=2).requires_grad_(True)
    out, lse, probs = rfa.ring_flash_attn_qkvpacked_func(qkv, causal=True, return_attn_probs=True)
    assert probs is None and lse.shape == (1, 4, 256) and torch.equal(out, base)
    out.backward(dout)
    assert qkv.grad is not None and torch.isfinite(qkv.grad.float()).all()
    with pytest.raises(NotImplementedError):
        rfa.ring_flash_attn_func(q, k, v, dropout_p=0.1)
    with pytest.raises(NotImplementedError):
        rfa.ring_flash_attn_func(q, k, v, window_size=(128, 0))


def test_cuda_graph_capture_single_gpu():
    """Forward + backward captured into a CUDA graph and replayed on new inputs: every launch of the path is
    asynchronous on the caller's stream and the library allocates nothing, so the whole step is capturable (the
    remedy for per-hop launch latency on short shards)."""
    from opt_ring_flash_attn_b200 import ring_flash_attn

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(23, 1, 256, 4, 2, 128, dtype=torch.bfloat16))
    sq, sk, sv = (x.clone().requires_grad_(True) for x in (q, k, v))
    sdo = dout.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: workspaces, function attributes
        for _ in range(2):
            sq.grad = sk.grad = sv.grad = None
            ring_flash_attn(sq, sk, sv, causal=True).backward(sdo)
    torch.cuda.current_stream().wait_stream(side)
    sq.grad = sk.grad = sv.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sout = ring_flash_attn(sq, sk, sv, causal=True)
        sout.backward(sdo)
    # replay on different data
    q2, k2, v2, do2 = (x.to(dev) for x in make_inputs(24, 1, 256, 4, 2, 128, dtype=torch.bfloat16))
    with torch.no_grad():
        sq.copy_(q2); sk.copy_(k2); sv.copy_(v2); sdo.copy_(do2)
    graph.replay()
    torch.cuda.synchronize()
    ref = ring_attn_oracle([q2], [k2], [v2], [do2], causal=True)
    assert (sout.float() - ref["out"][0]).abs().max().item() <= 1e-2
    assert _rel_l2(sq.grad, ref["dq"][0]) <= 2e-2
    assert _rel_l2(sk.grad, ref["dk"][0]) <= 2e-2
    assert _rel_l2(sv.grad, ref["dv"][0]) <= 2e-2


def test_device_status_word_surfaces_as_an_error(monkeypatch):
    """A kernel whose bounded wait runs out sets the workspace's status word and every later kernel returns at
    once.  The failure is made on the host here (the word is written from Python, nothing faults or times out on
    the GPU): the pass that ran with the word set publishes it, and the next call on that scratch raises and
    clears it; with RFA_B200_SYNC_STATUS=1 the failing call itself raises."""
    import time

    import opt_ring_flash_attn_b200 as rfa
    from opt_ring_flash_attn_b200 import workspace

    dev = torch.device("cuda:0")
    q, k, v, _ = (x.to(dev) for x in make_inputs(36, 1, 256, 2, 2, 64, dtype=torch.bfloat16))
    monkeypatch.setenv("RFA_B200_SYNC_STATUS", "0")
    good = rfa.ring_flash_attn(q, k, v, causal=True)
    torch.cuda.synchronize()
    ws = workspace.forward_workspace(q, k, 1)
    ws.status.fill_(1)                       # "a pipeline wait ran out" injected from the host
    time.sleep(0.002)                        # passes closer together than a millisecond share one status copy
    rfa.ring_flash_attn(q, k, v, causal=True)  # kernels return at once; the result of this call is invalid
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status 1"):
        rfa.ring_flash_attn(q, k, v, causal=True)
    assert int(ws.status.item()) == 0        # cleared once reported: the operator works again
    again = rfa.ring_flash_attn(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(again, good)
    # synchronous mode: the failing call raises itself
    monkeypatch.setenv("RFA_B200_SYNC_STATUS", "1")
    ws.status.fill_(1)
    with pytest.raises(RuntimeError, match="device status 1"):
        rfa.ring_flash_attn(q, k, v, causal=True)
    monkeypatch.setenv("RFA_B200_SYNC_STATUS", "0")
    ws.status.fill_(1)
    with pytest.raises(RuntimeError, match="device status 1"):
        rfa.check()
    assert torch.equal(rfa.ring_flash_attn(q, k, v, causal=True), good)


def test_deterministic_wrapper_flag_gives_identical_gradients():
    """`deterministic=True` of the baseline-style wrappers: two backward passes give the same bits."""
    import opt_ring_flash_attn_b200 as rfa

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(37, 1, 1024, 8, 2, 128, dtype=torch.bfloat16))
    grads = []
    for _ in range(2):
        a, b, c = (x.clone().requires_grad_(True) for x in (q, k, v))
        rfa.ring_flash_attn_func(a, b, c, causal=True, deterministic=True).backward(dout)
        grads.append((a.grad, b.grad, c.grad))
    for x, y in zip(*grads):
        assert torch.equal(x, y)
    ref = ring_attn_oracle([q], [k], [v], [dout], causal=True)
    assert _rel_l2(grads[0][0], ref["dq"][0]) <= 2e-2
