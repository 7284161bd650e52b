"""The real multi-process path: one process per GPU, public operator, both GPU transports (copy engines over mapped
peer memory, and the private NCCL communicator), compared with the oracle.
Skipped when fewer than two GPUs are visible (the single-GPU emulation in test_gpu_kernels.py covers the kernels)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cfg, errs, transport):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from opt_ring_flash_attn_b200 import _native, ring_flash_attn_with_lse, workspace
        from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle, shard

        from oracle.ring_attn_oracle import zigzag_oracle, zigzag_shard

        B, S, Hq, Hkv, D, causal, dtype = cfg[:7]
        os.environ["RFA_B200_TRANSPORT"] = transport
        zigzag = len(cfg) > 7 and cfg[7] is True
        balance = len(cfg) > 7 and cfg[7] == "balanced"  # contiguous shards, executed in the zigzag arrangement
        os.environ["RFA_B200_BALANCE"] = "1" if balance else "0"
        wire16 = len(cfg) > 8 and cfg[8]  # dK/dV travel in the input dtype (the reference's OPTIMIZED_RING_BWD_COMM_BF16)
        os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "1" if wire16 else "0"
        q, k, v, dout = (x.to(dev) for x in make_inputs(60, B, S * world, Hq, Hkv, D, dtype=dtype))
        if zigzag:
            qs, ks, vs, dos = (zigzag_shard(x, world) for x in (q, k, v, dout))
        else:
            qs, ks, vs, dos = shard(q, world), shard(k, world), shard(v, world), shard(dout, world)
        ql, kl, vl = (x[rank].clone().requires_grad_(True) for x in (qs, ks, vs))
        for it in range(2):  # second iteration reuses the cached workspaces and transports
            ql.grad = kl.grad = vl.grad = None
            out, lse = ring_flash_attn_with_lse(ql, kl, vl, causal=causal, group=dist.group.WORLD, zigzag=zigzag)
            out.backward(dos[rank])
        torch.cuda.synchronize()
        for ws in workspace.all_workspaces():
            _native.check_status(ws.status, "ring")
        if wire16:
            assert next(iter(workspace._bwd_cache.values()))[1].dkdv[0].dtype == dtype
        if zigzag:
            ref = zigzag_oracle(q, k, v, dout, world, head_chunk=4)
        else:
            ref = ring_attn_oracle(qs, ks, vs, dos, causal=causal, head_chunk=4)

        def rel(a, b):
            return ((a.float() - b).norm() / b.norm()).item()

        assert (out.float() - ref["out"][rank]).abs().max().item() <= 1e-2
        assert (lse - ref["lse"][rank]).abs().max().item() <= 1e-3
        assert rel(ql.grad, ref["dq"][rank]) <= 2e-2
        assert rel(kl.grad, ref["dk"][rank]) <= 2e-2
        assert rel(vl.grad, ref["dv"][rank]) <= 2e-2
        dist.barrier()
        from opt_ring_flash_attn_b200 import schedule
        schedule.shutdown()  # unmap the neighbours' memory before any of them exits
        dist.barrier()
    except Exception as e:
        errs.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [
    (1, 512, 4, 4, 128, True, torch.bfloat16),
    (1, 384, 8, 2, 128, False, torch.bfloat16),
    (2, 256, 4, 2, 64, True, torch.float16),
    (1, 320, 2, 2, 256, True, torch.bfloat16),
    (1, 512, 4, 2, 128, True, torch.bfloat16, True),  # zigzag layout
    (1, 384, 4, 2, 128, True, torch.bfloat16, False, True),  # 16-bit dK/dV transport
    (2, 512, 4, 2, 128, True, torch.bfloat16, "balanced"),  # contiguous shards regrouped internally (B = 2: strided halves)
])
@pytest.mark.parametrize("transport", ["peer", "native"])
def test_ring_nccl(cfg, transport):
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    errs = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, cfg, errs, transport)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
    msgs = []
    while not errs.empty():
        msgs.append(errs.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish in time")
    assert not msgs and all(p.exitcode == 0 for p in procs), msgs
