"""Generates ``tests/golden/ring_attn_golden.npz`` by running the reference's own
``ring_attn.py`` (imported unchanged from the reference checkout) on gloo CPU
ranks.  The fixtures pin the oracle in ``oracle/ring_attn_oracle.py``.

Usage (only where the reference checkout exists):
    python tests/golden/make_golden.py /path/to/reference

The reference cannot travel with this repository, so the outputs are committed;
inputs are regenerated from the seed by ``oracle.ring_attn_oracle.make_inputs``
and guarded by a checksum stored next to the outputs.

Adaptations applied around the unchanged reference function (all outside it):
fp32 inputs; GQA by ``repeat_interleave`` of K/V heads before the call (autograd
folds dK/dV back); a non-default softmax scale by pre-multiplying q with
``scale * sqrt(D)``; LSE = max + log(sum) from the statistics the reference's
autograd node saves (read before backward frees them).
"""
from __future__ import annotations

import math
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle.ring_attn_oracle import make_inputs  # noqa: E402

# name, seed, B, S_total, Hq, Hkv, D, W, causal, softmax_scale (None = default), row_stride (output sampling)
CASES = [
    ("ref_test_shape_dense", 11, 2, 128, 4, 4, 8, 4, False, None, 1),
    ("ref_test_shape_causal", 11, 2, 128, 4, 4, 8, 4, True, None, 1),
    ("small_w4_dense", 0, 1, 256, 2, 2, 32, 4, False, None, 1),
    ("small_w4_causal", 0, 1, 256, 2, 2, 32, 4, True, None, 1),
    ("gqa_w2_causal", 5, 1, 128, 4, 2, 16, 2, True, None, 1),
    ("scaled_w2_causal", 6, 1, 128, 2, 2, 16, 2, True, 0.3, 1),
    # (no world-size-1 case: the reference's backward sends dQ to itself, which gloo rejects)
    # the reference's CPU configuration: B=1, S_total=2048 (8 x 256), H=8, D=64, causal, seed 0; every 37th row is stored
    ("config1_w8_causal", 0, 1, 2048, 8, 8, 64, 8, True, None, 37),
]


def _worker(rank: int, world: int, ref_dir: str, case, port: int, outdir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    sys.path.insert(0, ref_dir)
    import ring_attn as ref  # the reference, unchanged

    name, seed, B, S, Hq, Hkv, D, W, causal, scale, _ = case
    q, k, v, dout = make_inputs(seed, B, S, Hq, Hkv, D)
    G = Hq // Hkv
    sh = lambda x: x.chunk(W, dim=1)[rank].contiguous()
    ql = sh(q).clone().requires_grad_(True)
    kl = sh(k).clone().requires_grad_(True)
    vl = sh(v).clone().requires_grad_(True)
    q_in = ql if scale is None else ql * (scale * math.sqrt(D))
    k_in = kl if G == 1 else kl.repeat_interleave(G, dim=2)
    v_in = vl if G == 1 else vl.repeat_interleave(G, dim=2)
    out = ref.ring_attn(q_in, k_in, v_in, None, causal=causal)
    saved = out.grad_fn.saved_tensors
    s_sum, s_max = saved[4], saved[5]
    lse = (s_max + torch.log(s_sum)).squeeze(-1)
    lse = lse if causal else lse.transpose(1, 2)  # dense branch saves [B,S,H,1]
    lse = lse.detach().clone()
    out.backward(sh(dout))
    np.savez(os.path.join(outdir, f"{name}_{rank}.npz"), out=out.detach().numpy(), lse=lse.numpy(),
             dq=ql.grad.numpy(), dk=kl.grad.numpy(), dv=vl.grad.numpy())
    dist.barrier()
    dist.destroy_process_group()


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference-checkout")
    ref_dir = sys.argv[1]
    if not os.path.exists(os.path.join(ref_dir, "ring_attn.py")):
        raise SystemExit(f"{ref_dir}/ring_attn.py not found")
    fixtures = {}
    with tempfile.TemporaryDirectory() as tmp:
        for idx, case in enumerate(CASES):
            name, seed, B, S, Hq, Hkv, D, W, causal, scale, stride = case
            mp.spawn(_worker, args=(W, ref_dir, case, 29610 + idx, tmp), nprocs=W, join=True)
            parts = [np.load(os.path.join(tmp, f"{name}_{r}.npz")) for r in range(W)]
            q, k, v, dout = make_inputs(seed, B, S, Hq, Hkv, D)
            fixtures[f"{name}/meta"] = np.array([seed, B, S, Hq, Hkv, D, W, int(causal), stride], dtype=np.int64)
            fixtures[f"{name}/scale"] = np.array([-1.0 if scale is None else scale], dtype=np.float64)
            fixtures[f"{name}/input_checksum"] = np.array(
                [q.double().sum().item(), k.double().sum().item(), v.double().sum().item(), dout.double().sum().item()])
            for key in ("out", "dq", "dk", "dv"):
                full = np.concatenate([p[key] for p in parts], axis=1)  # [B, S_total, H, D]
                fixtures[f"{name}/{key}"] = full[:, ::stride].astype(np.float32)
            lse = np.concatenate([p["lse"] for p in parts], axis=2)  # [B, H, S_total]
            fixtures[f"{name}/lse"] = lse[:, :, ::stride].astype(np.float32)
            print(name, "done", {k2: fixtures[f'{name}/{k2}'].shape for k2 in ("out", "lse", "dk")})
    dst = Path(__file__).resolve().parent / "ring_attn_golden.npz"
    np.savez_compressed(dst, **fixtures)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
