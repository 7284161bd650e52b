"""Failure behaviour of the host side, made on the host (CPU ranks on gloo, no GPU involved): a rank that leaves
between passes must end the others with an error instead of a hang, and ranks that disagree on their shard
shapes must be told so before any buffer moves."""
import os
import socket
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.ring_attn_oracle import make_inputs, shard


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup(rank, world, port, timeout_s):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "0"
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s))
    torch.set_num_threads(1)
    import sys
    sys.path.insert(0, os.path.dirname(__file__))


def _leaver_worker(rank, world, port, report):
    _setup(rank, world, port, 6)
    import fake_kernels
    from opt_ring_flash_attn_b200 import schedule

    q, k, v, dout = make_inputs(52, 1, 64 * world, 2, 2, 16, dtype=torch.bfloat16)
    qs, ks, vs, dos = shard(q, world), shard(k, world), shard(v, world), shard(dout, world)
    out, lse = schedule.ring_forward(None, qs[rank], ks[rank], vs[rank], 0.25, True, kernels=fake_kernels)
    if rank == world - 1:
        # leaves between the passes: nothing of it is in flight, it simply never joins the backward ring
        report.put((rank, "left"))
        dist.destroy_process_group()
        return
    t0 = time.time()
    try:
        schedule.ring_backward(None, dos[rank], qs[rank], ks[rank], vs[rank], out, lse, 0.25, True,
                               kernels=fake_kernels)
        report.put((rank, "no error"))
    except Exception as e:  # the process group's timeout or a closed connection, never a hang
        report.put((rank, f"raised {type(e).__name__} after {time.time() - t0:.1f}s"))
    # no collective here: the group is broken on purpose


def test_rank_that_leaves_ends_the_others_with_an_error():
    world = 2
    ctx = mp.get_context("spawn")
    report = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, world, port, report)) for r in range(world)]
    t0 = time.time()
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    msgs = {}
    while not report.empty():
        r, m = report.get()
        msgs[r] = m
    assert not hung, f"ranks still running after {time.time() - t0:.0f}s: {msgs}"
    assert msgs.get(world - 1) == "left"
    assert msgs.get(0, "").startswith("raised"), msgs


def _mismatch_worker(rank, world, port, report):
    _setup(rank, world, port, 30)
    import fake_kernels
    from opt_ring_flash_attn_b200 import schedule

    class Counting:
        calls = 0

        def __getattr__(self, name):
            fn = getattr(fake_kernels, name)

            def wrapped(*a, **kw):
                Counting.calls += 1
                return fn(*a, **kw)

            return wrapped

    S = 64 if rank == 0 else 128  # unequal shards
    q, k, v, _ = make_inputs(53, 1, S, 2, 2, 16, dtype=torch.bfloat16)
    try:
        schedule.ring_forward(None, q, k, v, 0.25, True, kernels=Counting())
        report.put((rank, "no error"))
    except ValueError as e:
        ok = "disagree" in str(e) and Counting.calls == 0 and not schedule._transports
        report.put((rank, "ok" if ok else f"late: calls={Counting.calls} transports={len(schedule._transports)}"))
    dist.barrier()
    dist.destroy_process_group()


def test_mismatched_shard_shapes_are_refused_before_any_transfer():
    world = 2
    ctx = mp.get_context("spawn")
    report = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_mismatch_worker, args=(r, world, port, report)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    for p in procs:
        if p.is_alive():
            p.terminate()
    msgs = {}
    while not report.empty():
        r, m = report.get()
        msgs[r] = m
    assert msgs == {0: "ok", 1: "ok"}, msgs


def test_status_word_reaches_the_host_without_a_gpu():
    """raise_if_failed / publish_status on a CPU workspace are inert (no pinned copy, no event) -- the GPU test
    injects a failure into the device word; here the bookkeeping itself is checked."""
    from opt_ring_flash_attn_b200 import workspace

    q = torch.zeros(1, 128, 2, 16, dtype=torch.bfloat16)
    try:
        ws = workspace.backward_workspace(q, q, 1)
        workspace.publish_status(ws, "x")       # CPU tensors: nothing to publish
        workspace.raise_if_failed(ws, "x")
        assert ws.status_event is None and int(ws.status.item()) == 0
        ws.status.fill_(1)
        with pytest.raises(RuntimeError, match="device status 1"):
            workspace.check_all("x")
        assert int(ws.status.item()) == 0       # reported once, then cleared
        workspace.check_all("x")
    finally:
        workspace.clear()
