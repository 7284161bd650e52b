"""Parity of the sm_100a hop kernels (through the C ABI) with the oracle on the same seeded inputs.

Tolerances are the ones the task states for this path:
  out  max-abs <= 1e-2 (bf16/fp16 output),  LSE max-abs <= 1e-3,  dQ/dK/dV relative L2 <= 2e-2.
The W ranks run on one GPU through the product's own schedules (``schedule.ring_forward`` / ``ring_backward`` /
``zigzag_*`` with the native kernels; tests/inproc_ring.py hands the buffers from rank to rank inside the
process); tests/ring_emulator.py keeps one hand-written walk that exercises the accumulate-in-the-epilogue path
of the backward kernel.  The multi-process NCCL path is covered by tests/test_gpu_ring.py.
"""
import pytest
import torch

from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle, shard

pytestmark = pytest.mark.gpu

OUT_TOL, LSE_TOL, GRAD_REL_L2 = 1e-2, 1e-3, 2e-2


def _rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def run_case(B, S, Hq, Hkv, D, W, causal, dtype=torch.bfloat16, scale=None, seed=0, std=1.0, backward=True,
             path="schedule", head_chunk=4, deterministic=False):
    from opt_ring_flash_attn_b200 import _native
    from inproc_ring import run_ring
    from ring_emulator import emulate_backward, emulate_forward

    dev = torch.device("cuda:0")
    q, k, v, dout = make_inputs(seed, B, S * W, Hq, Hkv, D, std=std, dtype=dtype)
    q, k, v, dout = (x.to(dev) for x in (q, k, v, dout))
    qs, ks, vs, dos = shard(q, W), shard(k, W), shard(v, W), shard(dout, W)
    sc = D ** -0.5 if scale is None else scale

    if path == "schedule":
        outs, lses, dqs, dks, dvs = run_ring(W, dev, qs, ks, vs, dos if backward else None, sc, causal,
                                             deterministic=deterministic)
    else:  # hand-written walk over the ranks; the backward kernel's epilogue folds in the travelling partial sums
        outs, lses, lses_pad, status = emulate_forward(qs, ks, vs, sc, causal)
        torch.cuda.synchronize()
        _native.check_status(status, "forward hop")
        if backward:
            dqs, dks, dvs, status = emulate_backward(dos, qs, ks, vs, outs, lses_pad, sc, causal)
            torch.cuda.synchronize()
            _native.check_status(status, "backward hop")
    ref = ring_attn_oracle(qs, ks, vs, dos if backward else None, causal=causal, softmax_scale=sc,
                           head_chunk=head_chunk)
    for r in range(W):
        err_o = (outs[r].float() - ref["out"][r]).abs().max().item()
        err_l = (lses[r] - ref["lse"][r]).abs().max().item()
        assert err_o <= OUT_TOL, f"rank {r}: out max-abs {err_o}"
        assert err_l <= LSE_TOL, f"rank {r}: lse max-abs {err_l}"
    if not backward:
        return None
    for r in range(W):
        for name, got, want in (("dq", dqs[r], ref["dq"][r]), ("dk", dks[r], ref["dk"][r]), ("dv", dvs[r], ref["dv"][r])):
            assert torch.isfinite(got.float()).all(), f"rank {r}: {name} has non-finite values"
            e = _rel_l2(got, want)
            assert e <= GRAD_REL_L2, f"rank {r}: {name} rel-L2 {e}"
    return dqs, dks, dvs


def test_fwd_only_smallest():
    run_case(1, 128, 1, 1, 128, 1, False, backward=False)


def test_fwd_only_causal_two_tiles():
    run_case(1, 256, 2, 2, 128, 1, True, backward=False)


@pytest.mark.parametrize("causal", [False, True])
def test_w1_d128(causal):
    run_case(1, 256, 2, 2, 128, 1, causal, seed=1)


@pytest.mark.parametrize("causal", [False, True])
def test_w2_state_carry(causal):
    run_case(1, 256, 2, 2, 128, 2, causal, seed=2)


def test_w3_gqa_causal():
    run_case(1, 384, 4, 2, 128, 3, True, seed=3)


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_other_head_dims(D, causal):
    run_case(1, 256, 2, 1, D, 2, causal, seed=4)


@pytest.mark.parametrize("S", [72, 200, 328])
def test_ragged_sequence(S):
    run_case(1, S, 2, 2, 128, 2, True, seed=5)


def test_ragged_d256():
    run_case(1, 200, 2, 2, 256, 2, True, seed=5)


def test_fp16():
    run_case(1, 256, 2, 2, 128, 2, True, dtype=torch.float16, seed=6)


@pytest.mark.parametrize("D", [32, 96, 160])
def test_padded_head_dim(D):
    run_case(1, 192, 2, 2, D, 1, True, seed=7)


def test_batch_and_scale():
    run_case(2, 256, 4, 4, 128, 2, True, scale=0.05, seed=8)


def test_short_shard_mha_shape():
    # the short-shard workload (MHA, D=128, S_local=1024 per rank) with 8 of its 32 heads
    run_case(1, 1024, 8, 8, 128, 2, True, seed=1)


def test_gqa_shape_reduced():
    # the Llama-3-8B-shaped workload (GQA 4:1, D=128) at S_local=2048 with heads 8/2
    run_case(1, 2048, 8, 2, 128, 2, True, seed=2)


def test_gqa_shape_full_shard_one_rank():
    """One GQA group (H_q=4, H_kv=1) of the benchmarked workload at its full shard length S_local=8192, one rank:
    64 K/V tiles, several waves of CTAs.  The oracle's score matrices are 1 GB per chunk of four heads."""
    run_case(1, 8192, 4, 1, 128, 1, True, seed=2, head_chunk=4)


def test_gqa_shape_full_shard_two_ranks():
    """As above on a two-rank ring: rank 1 runs one diagonal and one full block of 8192 x 8192 through the product
    schedule (state carry, transport hand-over, separate dK/dV accumulate)."""
    run_case(1, 8192, 4, 1, 128, 2, True, seed=2, head_chunk=4)


def test_d256_shape_reduced():
    # the large-head-dim workload (B=2, D=256, scale 1/16) at S_local=1024 with 4 heads
    run_case(2, 1024, 4, 4, 256, 2, True, scale=1.0 / 16, seed=3)


def test_d256_shape_full_shard():
    """The large-head-dim workload at its real shard (B=2, S_local=4096, D=256, scale 1/16) with 4 of its 16 heads."""
    run_case(2, 4096, 4, 4, 256, 1, True, scale=1.0 / 16, seed=3, head_chunk=4)


def test_d256_shape_full_shard_two_ranks():
    run_case(2, 4096, 2, 2, 256, 2, True, scale=1.0 / 16, seed=3, head_chunk=2)


def test_long_context_distribution():
    # value distribution of the long-context workload (std 0.5, GQA 8:1) at reduced size
    run_case(1, 1024, 16, 2, 128, 2, True, seed=4, std=0.5)


def test_epilogue_accumulate_path():
    """The backward kernel's own `dkdv_out = dkdv_prev + block` epilogue (accumulate_prev=1), which the product
    schedule replaces by a separate accumulate kernel: a three-rank walk written out by hand."""
    run_case(1, 384, 4, 2, 128, 3, True, seed=3, path="emulator")
    run_case(1, 200, 2, 2, 256, 2, False, seed=5, path="emulator")


def test_bwd_window_ending_inside_a_tile():
    """kv_len that is not a multiple of the 128-row tile: the keys between kv_len and the end of the tile are real
    rows of K/V and must not reach dQ (they are masked out of P), and their dK/dV rows keep the previous sums."""
    from opt_ring_flash_attn_b200 import _native
    import fake_kernels

    dev = torch.device("cuda:0")
    B, S, Hq, Hkv, D, kv_len, q_begin = 1, 384, 4, 2, 128, 192, 128
    q, k, v, dout = (x.to(dev) for x in make_inputs(91, B, S, Hq, Hkv, D, dtype=torch.bfloat16))
    sc = D ** -0.5
    spad = _native.padded_seq(S)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # lse / delta of the windowed problem, from the fp32 test double (same arithmetic as the oracle)
    cq, ck, cv, cdo = (x.cpu() for x in (q, k, v, dout))
    out_c = torch.zeros(B, S, Hq, D)
    lse_c = torch.zeros(B, Hq, spad)
    fake_kernels.fwd_hop(cq, ck, cv, None, None, None, out_c, lse_c, sc, True, True, False, None, q_begin=q_begin,
                         kv_len=kv_len)
    delta_c, lse2_c = torch.zeros(B, Hq, spad), torch.zeros(B, Hq, spad)
    fake_kernels.bwd_prepare(out_c, cdo, lse_c, delta_c, lse2_c, None, None)
    dq_ref = torch.zeros(B * Hq * S * D)
    dkdv_ref = torch.zeros(2, B, S, Hkv, D)
    fake_kernels.bwd_hop(cq, ck, cv, cdo, lse2_c, delta_c, dq_ref, None, dkdv_ref, sc, False, False, None,
                         q_begin=q_begin, kv_len=kv_len)
    dq_ref = dq_ref.view(B, Hq, S, D).transpose(1, 2)
    # the kernel under test with the same statistics
    lse2, delta = lse2_c.to(dev), delta_c.to(dev)
    dq_acc = torch.zeros(_native.dq_acc_elems(B, S, Hq, D), dtype=torch.float32, device=dev)
    dkdv = torch.full((2, B, S, Hkv, D), float("nan"), dtype=torch.float32, device=dev)
    _native.bwd_hop(q, k, v, dout, lse2, delta, dq_acc, None, dkdv, sc, False, False, status, q_begin=q_begin,
                    kv_len=kv_len)
    dq = torch.empty_like(q)
    _native.dq_finalize(dq_acc, dq)
    torch.cuda.synchronize()
    _native.check_status(status, "windowed backward hop")
    assert torch.equal(dq[:, :q_begin].float().cpu(), torch.zeros(B, q_begin, Hq, D))  # rows before the window
    assert _rel_l2(dq.cpu(), dq_ref) <= GRAD_REL_L2
    assert torch.equal(dkdv[:, :, kv_len:].cpu(), torch.zeros(2, B, S - kv_len, Hkv, D))  # keys beyond the window
    assert _rel_l2(dkdv[0].cpu(), dkdv_ref[0]) <= GRAD_REL_L2
    assert _rel_l2(dkdv[1].cpu(), dkdv_ref[1]) <= GRAD_REL_L2


def test_deterministic_mode_is_bitwise_reproducible():
    """Ordered dQ reductions: two runs give identical bits for dq, dk and dv (and match the oracle); D=256 takes
    the two-CTAs-per-tile path, GQA 4:1 the path that would otherwise split the group over CTAs."""
    for (B, S, Hq, Hkv, D, W) in ((1, 1024, 8, 2, 128, 2), (1, 512, 2, 2, 256, 1), (1, 640, 4, 4, 64, 2)):
        a = run_case(B, S, Hq, Hkv, D, W, True, seed=12, deterministic=True)
        b = run_case(B, S, Hq, Hkv, D, W, True, seed=12, deterministic=True)
        for xs, ys in zip(a, b):
            for x, y in zip(xs, ys):
                assert torch.equal(x, y)


@pytest.mark.parametrize("W,S,Hq,Hkv,D", [(2, 256, 2, 2, 128), (3, 512, 4, 2, 128), (2, 256, 2, 1, 64), (2, 512, 2, 2, 256)])
def test_zigzag_layout(W, S, Hq, Hkv, D):
    """Zigzag schedule (window variants of the hop kernels) against the pinned oracle regrouped into the zigzag layout."""
    from inproc_ring import run_ring
    from oracle.ring_attn_oracle import zigzag_oracle, zigzag_shard

    dev = torch.device("cuda:0")
    q, k, v, dout = (x.to(dev) for x in make_inputs(80, 1, S * W, Hq, Hkv, D, dtype=torch.bfloat16))
    qs, ks, vs, dos = (zigzag_shard(x, W) for x in (q, k, v, dout))
    sc = D ** -0.5
    outs, lses, dqs, dks, dvs = run_ring(W, dev, qs, ks, vs, dos, sc, True, zigzag=True)
    ref = zigzag_oracle(q, k, v, dout, W, head_chunk=4)
    for r in range(W):
        assert (outs[r].float() - ref["out"][r]).abs().max().item() <= OUT_TOL
        assert (lses[r] - ref["lse"][r]).abs().max().item() <= LSE_TOL
        for name, got, want in (("dq", dqs[r], ref["dq"][r]), ("dk", dks[r], ref["dk"][r]), ("dv", dvs[r], ref["dv"][r])):
            assert torch.isfinite(got.float()).all(), f"rank {r}: {name} has non-finite values"
            e = _rel_l2(got, want)
            assert e <= GRAD_REL_L2, f"rank {r}: {name} rel-L2 {e}"


def test_wire16_through_the_product_schedule(monkeypatch):
    """16-bit dK/dV transport (the reference's OPTIMIZED_RING_BWD_COMM_BF16=1) on a three-rank ring."""
    monkeypatch.setenv("OPTIMIZED_RING_BWD_COMM_BF16", "1")
    run_case(1, 384, 4, 2, 128, 3, True, seed=14)


def test_run_twice_bitwise_forward():
    """Forward is deterministic: two runs give identical bits (cheap race detector)."""
    from ring_emulator import emulate_forward

    dev = torch.device("cuda:0")
    q, k, v, _ = make_inputs(10, 1, 512, 4, 2, 128, dtype=torch.bfloat16)
    qs, ks, vs = shard(q.to(dev), 2), shard(k.to(dev), 2), shard(v.to(dev), 2)
    o1, l1, _, _ = emulate_forward(qs, ks, vs, 128 ** -0.5, True)
    o2, l2, _, _ = emulate_forward(qs, ks, vs, 128 ** -0.5, True)
    torch.cuda.synchronize()
    for a, b in zip(o1 + l1, o2 + l2):
        assert torch.equal(a, b)


def test_dkdv_accumulate():
    from opt_ring_flash_attn_b200 import _native

    dev = torch.device("cuda:0")
    a = torch.randn(2, 1, 200, 2, 96, device=dev)
    b = torch.randn_like(a)
    out = torch.empty_like(a)
    _native.dkdv_accumulate(a, b, out)
    assert torch.equal(out, a + b)
    ref = a + b
    _native.dkdv_accumulate(a, b, a)  # in place, as the ring schedule uses it
    assert torch.equal(a, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dkdv_accumulate_to16(dtype):
    """16-bit dK/dV transport: out = round(float(prev) + block), bit-exact against torch (same rounding mode)."""
    from opt_ring_flash_attn_b200 import _native

    dev = torch.device("cuda:0")
    block = torch.randn(2, 1, 200, 2, 96, device=dev)
    out = torch.empty_like(block, dtype=dtype)
    _native.dkdv_accumulate_to16(None, block, out)  # first active hop
    assert torch.equal(out, block.to(dtype))
    prev = torch.randn_like(block).to(dtype)
    ref = (prev.float() + block).to(dtype)
    _native.dkdv_accumulate_to16(prev, block, prev)  # in place, as the ring schedule uses it
    assert torch.equal(prev, ref)


def test_abi_rejects_bad_arguments():
    from opt_ring_flash_attn_b200 import _native

    dev = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    q = torch.zeros(1, 128, 3, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(q)
    lse = torch.empty(1, 3, 128, dtype=torch.float32, device=dev)
    with pytest.raises(RuntimeError, match="RFA_ERR_INVALID_ARG"):  # 3 % 2 != 0
        _native.fwd_hop(q, k, k, None, None, None, out, lse, 0.1, True, True, False, status)
    q = torch.zeros(1, 128, 2, 100, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="RFA_ERR_UNSUPPORTED"):  # head dim not a multiple of 8
        _native.fwd_hop(q, q, q, None, None, None, torch.empty_like(q), lse, 0.1, True, True, False, status)
