"""Host-side ring logic on CPU ranks (gloo): schedules, slot algebra and transport, with a test double
for the kernels.  Every rank's result is compared with the oracle on the full problem."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle, shard


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, Hq, Hkv, use_subgroup, errs, wire16=False):
    # 16-bit dK/dV transport is switched on like in the reference (optimized_ring_flash_attn.py:205-208)
    os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "1" if wire16 else "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(__file__))
        import fake_kernels
        from opt_ring_flash_attn_b200 import schedule

        group = None
        ring_world, ring_rank = world, rank
        if use_subgroup:
            # ranks {1, 2} form the ring; rank 0 sits out (tests group-local -> global rank mapping)
            group = dist.new_group([1, 2])
            if rank == 0:
                dist.barrier()
                return
            ring_world, ring_rank = 2, rank - 1
        B, S, D = 1, 96, 32
        q, k, v, dout = make_inputs(50, B, S * ring_world, Hq, Hkv, D, dtype=torch.bfloat16)
        qs, ks, vs, dos = shard(q, ring_world), shard(k, ring_world), shard(v, ring_world), shard(dout, ring_world)
        scale = 0.2
        out, lse = schedule.ring_forward(group, qs[ring_rank], ks[ring_rank], vs[ring_rank], scale, causal,
                                         kernels=fake_kernels)
        # a second forward before the first backward: results of call 1 must survive (no workspace aliasing)
        out2, _ = schedule.ring_forward(group, qs[ring_rank], ks[ring_rank], vs[ring_rank], scale, causal,
                                        kernels=fake_kernels)
        dq, dk, dv = schedule.ring_backward(group, dos[ring_rank], qs[ring_rank], ks[ring_rank], vs[ring_rank], out,
                                            lse, scale, causal, kernels=fake_kernels)
        ref = ring_attn_oracle(qs, ks, vs, dos, causal=causal, softmax_scale=scale)
        r = ring_rank

        def rel(a, b):
            return ((a.float() - b).norm() / b.norm()).item()

        if wire16 and ring_world > 1:
            from opt_ring_flash_attn_b200 import workspace
            ws = next(iter(workspace._bwd_cache.values()))[1]
            assert ws.dkdv[0].dtype == torch.bfloat16 and ws.block_dkdv.dtype == torch.float32
        assert torch.equal(out, out2)
        assert (out.float() - ref["out"][r]).abs().max().item() <= 1e-2
        assert (lse[:, :, :S] - ref["lse"][r]).abs().max().item() <= 1e-3
        assert rel(dq, ref["dq"][r]) <= 2e-2, rel(dq, ref["dq"][r])
        assert rel(dk, ref["dk"][r]) <= 2e-2, rel(dk, ref["dk"][r])
        assert rel(dv, ref["dv"][r]) <= 2e-2, rel(dv, ref["dv"][r])
        dist.barrier()
    except Exception as e:  # surface the failure to the parent
        errs.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,causal,Hq,Hkv,sub,wire16", [(2, True, 2, 2, False, False), (2, False, 4, 2, False, False),
                                                            (3, True, 4, 2, False, False), (3, True, 2, 1, True, False),
                                                            (3, True, 4, 2, False, True), (2, False, 2, 2, False, True)])
def test_ring_schedules_on_gloo(world, causal, Hq, Hkv, sub, wire16):
    ctx = mp.get_context("spawn")
    errs = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, causal, Hq, Hkv, sub, errs, wire16))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    msgs = []
    while not errs.empty():
        msgs.append(errs.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish in time")
    assert not msgs and all(p.exitcode == 0 for p in procs), msgs


def _zz_worker(rank, world, port, Hq, Hkv, errs, wire16=False):
    os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "1" if wire16 else "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(__file__))
        import fake_kernels
        from opt_ring_flash_attn_b200 import schedule
        from oracle.ring_attn_oracle import zigzag_oracle, zigzag_shard

        B, S, D = 1, 256, 16  # S_local = 256: two 128-row halves
        q, k, v, dout = make_inputs(70, B, S * world, Hq, Hkv, D, dtype=torch.bfloat16)
        qs, ks, vs, dos = (zigzag_shard(x, world) for x in (q, k, v, dout))
        scale = 0.25
        out, lse = schedule.zigzag_forward(None, qs[rank], ks[rank], vs[rank], scale, kernels=fake_kernels)
        dq, dk, dv = schedule.zigzag_backward(None, dos[rank], qs[rank], ks[rank], vs[rank], out, lse, scale,
                                              kernels=fake_kernels)
        ref = zigzag_oracle(q, k, v, dout, world, softmax_scale=scale)

        def rel(a, b):
            return ((a.float() - b).norm() / b.norm()).item()

        assert (out.float() - ref["out"][rank]).abs().max().item() <= 1e-2
        assert (lse[:, :, :S] - ref["lse"][rank]).abs().max().item() <= 1e-3
        assert rel(dq, ref["dq"][rank]) <= 2e-2, rel(dq, ref["dq"][rank])
        assert rel(dk, ref["dk"][rank]) <= 2e-2, rel(dk, ref["dk"][rank])
        assert rel(dv, ref["dv"][rank]) <= 2e-2, rel(dv, ref["dv"][rank])
        dist.barrier()
    except Exception as e:
        errs.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,Hq,Hkv,wire16", [(2, 2, 2, False), (3, 4, 2, False), (3, 4, 2, True)])
def test_zigzag_schedules_on_gloo(world, Hq, Hkv, wire16):
    ctx = mp.get_context("spawn")
    errs = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_zz_worker, args=(r, world, port, Hq, Hkv, errs, wire16)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    msgs = []
    while not errs.empty():
        msgs.append(errs.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish in time")
    assert not msgs and all(p.exitcode == 0 for p in procs), msgs


def test_transport_rejects_same_buffer_and_unposted_wait():
    """Error behaviour of the transport mirrors the reference's comm helpers (RuntimeError on misuse)."""
    port = _free_port()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        from opt_ring_flash_attn_b200.transport import RingTransport

        t = RingTransport(None, torch.device("cpu"))
        with pytest.raises(RuntimeError):
            t.wait()
        buf = torch.zeros(4)
        with pytest.raises(RuntimeError):
            t.post(buf, buf)
    finally:
        dist.destroy_process_group()


def _balanced_worker(rank, world, port, Hq, Hkv, errs):
    os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(__file__))
        import fake_kernels
        from opt_ring_flash_attn_b200 import schedule
        from oracle.ring_attn_oracle import zigzag_shard

        B, S, D = 2, 256, 16  # two 128-row halves per rank; B = 2 makes the half-shard views non-contiguous
        q, k, v, dout = make_inputs(72, B, S * world, Hq, Hkv, D, dtype=torch.bfloat16)
        qs, ks, vs, dos = shard(q, world), shard(k, world), shard(v, world), shard(dout, world)
        # the regrouping alone: contiguous -> zigzag gives the zigzag shards, and back is the identity
        (qz,) = schedule.regroup(None, [qs[rank]], to_zigzag=True)
        assert torch.equal(qz, zigzag_shard(q, world)[rank])
        (qc,) = schedule.regroup(None, [qz], to_zigzag=False)
        assert torch.equal(qc, qs[rank])
        scale = 0.25
        assert schedule.can_balance(None, S)
        out, lse, saved = schedule.balanced_forward(None, qs[rank], ks[rank], vs[rank], scale, kernels=fake_kernels)
        dq, dk, dv = schedule.balanced_backward(None, dos[rank], saved, scale, kernels=fake_kernels)
        ref = ring_attn_oracle(qs, ks, vs, dos, causal=True, softmax_scale=scale)  # contiguous layout

        def rel(a, b):
            return ((a.float() - b).norm() / b.norm()).item()

        assert (out.float() - ref["out"][rank]).abs().max().item() <= 1e-2
        assert (lse[:, :, :S] - ref["lse"][rank]).abs().max().item() <= 1e-3
        assert rel(dq, ref["dq"][rank]) <= 2e-2, rel(dq, ref["dq"][rank])
        assert rel(dk, ref["dk"][rank]) <= 2e-2, rel(dk, ref["dk"][rank])
        assert rel(dv, ref["dv"][rank]) <= 2e-2, rel(dv, ref["dv"][rank])
        dist.barrier()
    except Exception as e:
        errs.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,Hq,Hkv", [(2, 2, 2), (3, 4, 2), (4, 2, 1)])
def test_balanced_execution_of_contiguous_shards_on_gloo(world, Hq, Hkv):
    """Contiguous shards regrouped to the zigzag arrangement, zigzag schedules, results regrouped back: every rank
    must get the contiguous-layout results of the oracle (odd world sizes send both halves of one rank to one peer)."""
    ctx = mp.get_context("spawn")
    errs = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_balanced_worker, args=(r, world, port, Hq, Hkv, errs)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    msgs = []
    while not errs.empty():
        msgs.append(errs.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish in time")
    assert not msgs and all(p.exitcode == 0 for p in procs), msgs
