"""The reference's 24-config correctness grid (test_optimized_ring_flash_attn.py:133-138, B = 1: head_dim {64, 128} x
(H_q, H_kv) {(8, 8), (16, 2)} x S_local {1024, 2048, 4096} x causal {False, True}), run through the C ABI as a
two-rank ring emulated on one GPU and held to the oracle with the tolerances of the other parity tests (the
reference compares against single-GPU flash-attn with max-abs 1e-3 .. 6e-2).
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(__file__))

pytestmark = pytest.mark.gpu

GRID = [(D, Hq, Hkv, S, causal)
        for D in (64, 128)
        for (Hq, Hkv) in ((8, 8), (16, 2))
        for S in (1024, 2048, 4096)
        for causal in (False, True)]


@pytest.mark.parametrize("D,Hq,Hkv,S,causal", GRID)
def test_reference_grid(D, Hq, Hkv, S, causal):
    from test_gpu_kernels import run_case

    run_case(1, S, Hq, Hkv, D, 2, causal, seed=100 + D + Hq + S // 1024 + int(causal))
