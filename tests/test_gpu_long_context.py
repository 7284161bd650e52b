"""The long-context workload at its real shard length (S_local = 131072, GQA 8:1, D = 128, inputs ~ N(0, 0.5)),
one GQA group (H_q = 8, H_kv = 1), one rank, through the public operator.

The full score matrix of this problem is 0.5 TB per head, so parity is checked on slices against the slice-wise
fp32 restatement (oracle/chunked_attn.py, itself pinned to the oracle at small shapes): ``out``, ``lse`` and ``dq``
on sampled blocks of 128 query rows, ``dk`` and ``dv`` on sampled blocks of 128 keys -- early keys, which every
one of the 1024 query tiles of all eight heads adds into, and late ones.  Tolerances as everywhere else:
out max-abs 1e-2, LSE max-abs 1e-3, gradients relative L2 2e-2 (per slice).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

S_LOCAL, HQ, HKV, D, STD, SEED = 131072, 8, 1, 128, 0.5, 4
ROW_SLICES = (0, 128 * 37, 128 * 512, 128 * 1023)        # first, early, middle, last query tile
KEY_SLICES = (0, 128 * 300, 128 * 1000)                  # keys seen by all / most / the last 3 % of queries


def _rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def _draw(dev):
    g = torch.Generator(device="cpu")
    g.manual_seed(SEED)

    def one(h, std):
        t = torch.empty(1, S_LOCAL, h, D, dtype=torch.bfloat16, device=dev)
        for s0 in range(0, S_LOCAL, 16384):  # drawn in fp32 blocks to bound host memory
            t[0, s0:s0 + 16384] = (torch.randn(16384, h, D, generator=g) * std).to(torch.bfloat16).to(dev)
        return t

    return one(HQ, STD), one(HKV, STD), one(HKV, STD), one(HQ, 1.0)


def test_long_context_shard_on_sampled_slices():
    import opt_ring_flash_attn_b200 as rfa
    from oracle import chunked_attn as ca

    dev = torch.device("cuda:0")
    q, k, v, dout = _draw(dev)
    scale = D ** -0.5
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
    out, lse = rfa.ring_flash_attn_with_lse(qg, kg, vg, causal=True)
    out.backward(dout)
    torch.cuda.synchronize()
    rfa.check("long-context shard")
    assert torch.isfinite(out.float()).all() and torch.isfinite(qg.grad.float()).all()

    with torch.no_grad():
        lse_ref, delta_ref = ca.full_stats(q, k, v, dout, scale, row_block=512)
        assert (lse - lse_ref).abs().max().item() <= 1e-3  # every row of the LSE
        for r0 in ROW_SLICES:
            r1 = r0 + 128
            o_ref, _ = ca.forward_rows(q, k, v, scale, r0, r1)
            assert (out[:, r0:r1].float() - o_ref).abs().max().item() <= 1e-2, f"out rows {r0}"
            dq_ref = ca.dq_rows(q, k, v, dout, lse_ref, delta_ref, scale, r0, r1)
            assert _rel_l2(qg.grad[:, r0:r1], dq_ref) <= 2e-2, f"dq rows {r0}"
        for k0 in KEY_SLICES:
            k1 = k0 + 128
            dk_ref, dv_ref = ca.dkdv_keys(q, k, v, dout, lse_ref, delta_ref, scale, k0, k1, row_block=4096)
            assert _rel_l2(kg.grad[:, k0:k1], dk_ref) <= 2e-2, f"dk keys {k0}"
            assert _rel_l2(vg.grad[:, k0:k1], dv_ref) <= 2e-2, f"dv keys {k0}"
