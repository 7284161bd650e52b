#!/usr/bin/env python
"""Benchmark of the ring-flash-attention hot path: causal forward + backward per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2|c3|c4|c5] [--impl reference]
                    [--hops] [--grid speedup|ablation] [--graph] [--zigzag]

N > 1 is launched with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
One JSON line is printed by rank 0.

Workload (``config.workload``), by default: bf16 causal GQA attention shaped like Llama-3-8B, B=1,
S_local=8192 per rank, H_q=32, H_kv=8, D=128, q/k/v ~ N(0,1), dout ~ N(0,1) -- the configuration the
60%-of-peak target is quoted on.  Synthetic seeded inputs (the reference's harness also uses torch.randn).

FLOP accounting (algorithmic, causal FLOPs counted, not executed tiles):
  F_blk = 4*B*H_q*S_local^2*D per full block forward; the diagonal block counts 1/2; backward = 2.5x,
  forward+backward = 3.5x.  Rank r executes (r + 1/2) block-equivalents; the slowest rank is W-1.
  ``value`` is the whole-job rate (sum over ranks, W^2/2 block-equivalents) / slowest-rank time;
  ``slowest_rank_tflops_per_gpu`` is the per-GPU figure of the slowest rank, 3.5*(W-1/2)*F_blk / t.

Other modes
  --impl reference   the reference's own CPU path (its pure-PyTorch ring_attn.py, unchanged, on 8 gloo ranks on
                     the host cores) on its CPU-runnable configuration; rank 0 alone runs it.
  --hops             after the headline region, instrumented steps on every rank: CUDA events around every hop
                     kernel, accumulate kernel and transport wait, and around every transfer on the transport
                     stream; the slowest rank's table goes into the JSON line (``hops``).
  --grid speedup     the reference harness's speed-up grid (MHA causal, D in {64,128}, H in {8,16}, S_local
                     1024..8192, warm-up 3 / 10 iterations, MAX over ranks), with and without the three input clones
                     the reference times.
  --grid ablation    forward+backward with one host-side feature added per row: process-group transport, private
                     NCCL transport, peer-memory transport, 16-bit dK/dV transport, zigzag layout.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import socket
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: (B, S_local, Hq, Hkv, D, softmax_scale, std, seed, description)
    "c2": (1, 1024, 32, 32, 128, None, 1.0, 1, "short-shard MHA B=1 S_local=1024 H=32 D=128"),
    "c3": (1, 8192, 32, 8, 128, None, 1.0, 2, "Llama-3-8B-shaped GQA B=1 S_local=8192 Hq=32 Hkv=8 D=128"),
    "c4": (2, 4096, 16, 16, 256, 1.0 / 16, 1.0, 3, "large head_dim MHA B=2 S_local=4096 H=16 D=256"),
    "c5": (1, 131072, 64, 8, 128, None, 0.5, 4, "long-context GQA B=1 S_local=131072 Hq=64 Hkv=8 D=128"),
}
# The reference's CPU-runnable configuration: fp32 causal MHA, B=1, S_total=2048 as 8 shards of 256, H=8, D=64, seed 0.
REF_SAMPLE = {"B": 1, "S_total": 2048, "H": 8, "D": 64, "W": 8, "seed": 0}
REF_DIR = ROOT / "baseline" / "_ref"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def f_blk(B, S, Hq, D):
    return 4.0 * B * Hq * float(S) * float(S) * D


def kernel_digest(names=("bwd_hop.cu", "bwd_common.cuh", "tc05.cuh")) -> str:
    """Digest of the sources of the dominant kernel: the DRAM traffic figure captured under ncu is only emitted while
    the kernel it was captured from is the one being timed."""
    h = hashlib.sha256()
    for n in names:
        h.update((ROOT / "opt_ring_flash_attn_b200" / "csrc" / n).read_bytes())
    return h.hexdigest()[:16]


def captured_traffic(config: str):
    """(bytes per launch or None, note) from profiles/roofline_traffic.json."""
    p = ROOT / "profiles" / "roofline_traffic.json"
    if not p.exists():
        return None, "no ncu capture recorded"
    try:
        rec = json.loads(p.read_text()).get(f"bwd_hop_kernel/{config}/diagonal")
    except Exception:
        return None, "the recorded ncu capture is unreadable"
    if rec is None:
        return None, f"no ncu capture recorded for {config}"
    if rec.get("source_digest") != kernel_digest():
        return None, "kernel sources changed since the ncu capture"
    return int(rec["dram_bytes_per_launch"]), rec.get("note", "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 100):
        self.index = index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for n, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_shard(cfg, rank: int, device, dtype=torch.bfloat16, pinned=False):
    """Per-rank shards drawn from a per-rank seeded generator (seed*1009 + rank): q, k, v, dout."""
    B, S, Hq, Hkv, D, _, std, seed, _ = cfg
    g = torch.Generator(device="cpu")
    g.manual_seed(seed * 1009 + rank)

    def draw(h, s):
        t = torch.empty(B, S, h, D, dtype=dtype, pin_memory=pinned)
        # drawn in fp32 blocks to bound host memory, then cast
        for b in range(B):
            for s0 in range(0, S, 4096):
                s1 = min(S, s0 + 4096)
                t[b, s0:s1] = (torch.randn(s1 - s0, h, D, generator=g) * s).to(dtype)
        return t

    q, k, v = draw(Hq, std), draw(Hkv, std), draw(Hkv, std)
    dout = draw(Hq, 1.0)
    if device is not None:
        return [x.to(device) for x in (q, k, v, dout)]
    return [q, k, v, dout]


# ----------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own ring_attn.py on gloo ranks
# ----------------------------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ref_worker(rank, world, port, ref_dir, steps, warmup, threads, result):
    """One gloo rank of the CPU arm: the reference's ring_attn(q, k, v, None, causal=True) forward + backward
    (ring_attn.py:736-747) on its shard of the reference's CPU configuration."""
    import torch.distributed as dist

    # The arm may itself run under torchrun (rank 0 of an N-GPU launch): none of the launcher's rendezvous settings
    # may leak into these ranks (with TORCHELASTIC_USE_AGENT_STORE the env:// rendezvous expects the launcher's store).
    for k_ in list(os.environ):
        if k_.startswith(("TORCHELASTIC_", "TORCH_NCCL", "GROUP_", "ROLE_")) or k_ in (
                "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
            os.environ.pop(k_, None)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.set_num_threads(threads)
    sys.path.insert(0, ref_dir)
    import ring_attn as ref  # the reference's file, unchanged

    c = REF_SAMPLE
    torch.manual_seed(c["seed"])  # every rank draws the full tensors, as the reference's harness does
    full = [torch.randn(c["B"], c["S_total"], c["H"], c["D"]) for _ in range(4)]
    ql, kl, vl, dol = (x.chunk(world, dim=1)[rank].contiguous() for x in full)

    def step():
        qa, ka, va = (x.detach().clone().requires_grad_(True) for x in (ql, kl, vl))
        ref.ring_attn(qa, ka, va, None, causal=True).backward(dol)

    for _ in range(warmup):
        step()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    t = torch.tensor([dt], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        result.put(float(t.item()))
    dist.barrier()
    dist.destroy_process_group()


def _ref_flops():
    c = REF_SAMPLE
    W = c["W"]
    return 3.5 * (W * W / 2.0) * f_blk(c["B"], c["S_total"] // W, c["H"], c["D"])


def time_reference_cpu(steps: int, warmup: int):
    """Times the CPU arm.  Returns (seconds per step, cpu_baseline dict)."""
    import torch.multiprocessing as mp

    c = REF_SAMPLE
    W = c["W"]
    cores = os.cpu_count() or 1
    threads = max(1, cores // W)
    sample = (f"fp32 causal MHA B={c['B']} S_total={c['S_total']} ({W} contiguous shards of {c['S_total'] // W}) "
              f"H={c['H']} D={c['D']} seed {c['seed']}, forward+backward, {W} gloo ranks x {threads} threads, "
              f"{warmup} warm-up + {steps} timed steps, MAX over ranks")
    if (REF_DIR / "ring_attn.py").exists():
        ctx = mp.get_context("spawn")
        result = ctx.SimpleQueue()
        port = _free_port()
        procs = [ctx.Process(target=_ref_worker, args=(r, W, port, str(REF_DIR), steps, warmup, threads, result))
                 for r in range(W)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(600)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.terminate()
        if alive or result.empty() or any(p.exitcode != 0 for p in procs):
            raise RuntimeError("the CPU reference ranks did not finish")
        dt = result.get()
        kind = "reference"
        used = W * threads
    else:
        # the reference file did not travel: the oracle's restatement of it, all ranks simulated in one process
        from oracle.ring_attn_oracle import make_inputs, ring_attn_oracle, shard

        torch.set_num_threads(cores)
        q, k, v, do = make_inputs(c["seed"], c["B"], c["S_total"], c["H"], c["H"], c["D"])
        qs, ks, vs, dos = (shard(x, W) for x in (q, k, v, do))
        for _ in range(warmup):
            ring_attn_oracle(qs, ks, vs, dos, causal=True)
        t0 = time.perf_counter()
        for _ in range(steps):
            ring_attn_oracle(qs, ks, vs, dos, causal=True)
        dt = (time.perf_counter() - t0) / steps
        kind = "port"
        used = cores
        sample += " (baseline/_ref/ring_attn.py absent: oracle restatement, ranks simulated in one process)"
    val = _ref_flops() / dt / 1e12
    return dt, {"value": val, "unit": "TFLOP/s", "cores": used, "host_cores": cores, "kind": kind, "sample": sample,
                "ms_per_step": dt * 1e3}


def run_reference_arm(args, cfg, name):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    desc = cfg[8]
    steps = max(1, min(args.steps, 5))
    warmup = max(1, min(args.warmup, 1))
    dt, cb = time_reference_cpu(steps, warmup)
    line = {
        "impl": "reference", "metric": "causal_fwd_bwd_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name + ": " + desc, "sample": cb["sample"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------------
# Per-hop timeline
# ----------------------------------------------------------------------------------------------------------------
class HopRecorder:
    """Stands in for the kernel module of the schedules and brackets every call with CUDA events."""

    def __init__(self, native):
        self._n = native
        self.events = []  # (name, start event, end event)

    def __getattr__(self, name):
        fn = getattr(self._n, name)
        if not callable(fn) or name.startswith("_"):
            return fn

        def timed(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            self.events.append((name, e0, e1))
            return r

        return timed


def timeline_step(native, schedule, group, q, k, v, dout, scale, zigzag):
    """One instrumented forward + backward through the schedules.  Returns (rows, transfers): rows are
    {pass, what, ms} in issue order (hop kernels, accumulate kernels, exposed waits of the compute stream);
    transfers are the device times of the grouped send+recv on the transport streams."""
    rec = HopRecorder(native)
    dev = q.device
    tags = ("fwd_kv", "bwd_kv", "bwd_dkdv")
    transports = {}
    W = torch.distributed.get_world_size(group) if torch.distributed.is_initialized() else 1
    waits, posts = [], []
    if W > 1:
        from opt_ring_flash_attn_b200 import workspace

        # the transports of the scratch that earlier (untimed) steps of the same shape created
        cached = {}
        for ws_ in workspace.all_workspaces():
            cached.update(ws_.comms)
        for tag in tags:
            t = cached[tag]
            transports[tag] = t
            can_time = hasattr(t, "set_timing")
            if can_time:
                t.set_timing(True)
            orig_post, orig_wait = t.post, t.wait

            def post(send, recv, _t=t, _tag=tag, _orig=orig_post, _can=can_time):
                _orig(send, recv)
                posts.append((_tag, _t.last_slot() if _can else None, send.numel() * send.element_size()))

            def wait(_t=t, _tag=tag, _orig=orig_wait):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                _orig()
                e1.record()
                waits.append((_tag, len(rec.events), e0, e1))

            t.post, t.wait = post, wait
    try:
        if zigzag:
            out, lse = schedule.zigzag_forward(group, q, k, v, scale, kernels=rec)
            n_fwd = len(rec.events)
            schedule.zigzag_backward(group, dout, q, k, v, out, lse, scale, kernels=rec)
        else:
            out, lse = schedule.ring_forward(group, q, k, v, scale, True, kernels=rec)
            n_fwd = len(rec.events)
            schedule.ring_backward(group, dout, q, k, v, out, lse, scale, True, kernels=rec)
        torch.cuda.synchronize()
        rows = []
        wait_at = {}
        for tag, idx, e0, e1 in waits:
            wait_at.setdefault(idx, []).append((tag, e0.elapsed_time(e1)))
        for i, (name, e0, e1) in enumerate(rec.events):
            for tag, ms in wait_at.get(i, []):
                rows.append({"pass": "fwd" if tag == "fwd_kv" else "bwd", "what": f"wait {tag}", "ms": ms})
            rows.append({"pass": "fwd" if i < n_fwd else "bwd", "what": name, "ms": e0.elapsed_time(e1)})
        for tag, ms in wait_at.get(len(rec.events), []):
            rows.append({"pass": "bwd", "what": f"wait {tag}", "ms": ms})
        transfers = []
        for tag, slot, nbytes in posts:
            if slot is not None:
                ms = transports[tag].elapsed_ms(slot)
                transfers.append({"ring": tag, "bytes": nbytes, "ms": ms, "gb_s": nbytes / ms / 1e6 if ms > 0 else None})
        return rows, transfers
    finally:
        for tag, t in transports.items():
            t.__dict__.pop("post", None)
            t.__dict__.pop("wait", None)
            if hasattr(t, "set_timing"):
                t.set_timing(False)


def summarize_timeline(rows, transfers):
    def total(pred):
        return sum(r["ms"] for r in rows if pred(r))

    hop = ("fwd_hop", "bwd_hop")
    return {
        "fwd_hop_ms": [round(r["ms"], 4) for r in rows if r["what"] == "fwd_hop"],
        "bwd_hop_ms": [round(r["ms"], 4) for r in rows if r["what"] == "bwd_hop"],
        "kernel_ms": round(total(lambda r: not r["what"].startswith("wait")), 4),
        "hop_kernel_ms": round(total(lambda r: r["what"] in hop), 4),
        "accumulate_ms": round(total(lambda r: r["what"].startswith("dkdv_accumulate")), 4),
        "other_kernel_ms": round(total(lambda r: not r["what"].startswith("wait") and r["what"] not in hop
                                       and not r["what"].startswith("dkdv_accumulate")), 4),
        "exposed_wait_ms": {tag: round(total(lambda r, t=tag: r["what"] == f"wait {t}"), 4)
                            for tag in ("fwd_kv", "bwd_kv", "bwd_dkdv")},
        "exposed_waits": [{"what": r["what"], "ms": round(r["ms"], 4)} for r in rows if r["what"].startswith("wait")],
        "transfers": [{**t, "ms": round(t["ms"], 4), "gb_s": None if t["gb_s"] is None else round(t["gb_s"], 1)}
                      for t in transfers],
    }


# ----------------------------------------------------------------------------------------------------------------
# Timing helpers
# ----------------------------------------------------------------------------------------------------------------
def timed_region(step, steps, warmup, barrier, flush, dev, dist, world):
    """``warmup`` untimed steps, then exactly ``steps`` steps bracketed by barrier + synchronize on both sides, one
    CUDA-event pair per step, mean over the steps, MAX over ranks."""
    for _ in range(warmup):
        step()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    for i in range(steps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        ev[i][0].record()
        step()
        ev[i][1].record()
    barrier()
    ms = sum(a.elapsed_time(b) for a, b in ev) / steps
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def grid_mode(args, dist, dev, rank, world):
    """The reference harness's grids on this build (test_optimized_ring_flash_attn.py:59-84 protocol: warm-up 3,
    10 iterations, CUDA events, MAX over ranks)."""
    from opt_ring_flash_attn_b200 import ring_flash_attn, schedule, workspace

    group = dist.group.WORLD if world > 1 else None

    def reference_protocol(fn, warmup=3, iters=10):
        torch.cuda.synchronize()
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shards(hd, H, S_local):
        torch.manual_seed(0)
        S_full = S_local * world
        full = [torch.randn(1, S_full, H, hd, device=dev, dtype=torch.bfloat16) for _ in range(4)]
        return [x.chunk(world, dim=1)[rank].contiguous() for x in full]

    head_dims = tuple(int(x) for x in args.grid_head_dims.split(","))
    rows = []
    if args.grid == "speedup":
        for hd in head_dims:
            for H in (8, 16):
                for S_local in (1024, 2048, 4096, 8192):
                    ql, kl, vl, dol = shards(hd, H, S_local)

                    def fwd():
                        with torch.no_grad():
                            ring_flash_attn(ql, kl, vl, causal=True, group=group)

                    def fbw_with_clones():  # what the reference times (its three clone() calls included)
                        qa, ka, va = (x.detach().clone().requires_grad_(True) for x in (ql, kl, vl))
                        ring_flash_attn(qa, ka, va, causal=True, group=group).backward(dol)

                    qa, ka, va = (x.detach().clone().requires_grad_(True) for x in (ql, kl, vl))

                    def fbw():
                        qa.grad = ka.grad = va.grad = None
                        ring_flash_attn(qa, ka, va, causal=True, group=group).backward(dol)

                    fb = f_blk(1, S_local, H, hd)
                    t_fwd, t_fc, t_f = reference_protocol(fwd), reference_protocol(fbw_with_clones), reference_protocol(fbw)
                    rows.append({"head_dim": hd, "H": H, "S_local": S_local, "fwd_ms": round(t_fwd, 4),
                                 "fwd_bwd_ms_with_clones": round(t_fc, 4), "fwd_bwd_ms": round(t_f, 4),
                                 "slowest_rank_tflops_fwd_bwd": round(3.5 * (world - 0.5) * fb / (t_f * 1e-3) / 1e12, 1)})
    else:  # ablation: forward + backward, each row adds one host-side feature
        base = {"OPTIMIZED_RING_BWD_COMM_BF16": "0"}
        variants = [("A0 process-group transport", {**base, "RFA_B200_TRANSPORT": "torch"}, False),
                    ("A1 + private NCCL transport", {**base, "RFA_B200_TRANSPORT": "native"}, False),
                    ("A2 + peer-memory transport", {**base, "RFA_B200_TRANSPORT": "peer"}, False),
                    ("A3 + 16-bit dK/dV transport", {"RFA_B200_TRANSPORT": "peer", "OPTIMIZED_RING_BWD_COMM_BF16": "1"}, False),
                    ("A4 + zigzag layout", {"RFA_B200_TRANSPORT": "peer", "OPTIMIZED_RING_BWD_COMM_BF16": "1"}, True)]
        for hd in head_dims:
            for H in (8, 16):
                for S_local in (2048, 4096, 8192):
                    ql, kl, vl, dol = shards(hd, H, S_local)
                    qa, ka, va = (x.detach().clone().requires_grad_(True) for x in (ql, kl, vl))
                    row = {"head_dim": hd, "H": H, "S_local": S_local}
                    for name, env, zz in variants:
                        os.environ.update(env)
                        schedule.shutdown()  # transports are rebuilt for the new setting
                        workspace.clear()

                        def fbw():
                            qa.grad = ka.grad = va.grad = None
                            ring_flash_attn(qa, ka, va, causal=True, zigzag=zz, group=group).backward(dol)

                        row[name] = round(reference_protocol(fbw), 4)
                    rows.append(row)
        os.environ.pop("RFA_B200_TRANSPORT", None)
        os.environ["OPTIMIZED_RING_BWD_COMM_BF16"] = "0"
        schedule.shutdown()
    if rank == 0:
        print(json.dumps({"grid": args.grid, "n_gpus": world, "protocol": "warm-up 3, 10 iterations, CUDA events, MAX "
                          "over ranks; bf16, causal, MHA, B=1", "rows": rows}), flush=True)


def aux_mode(args, cfg, dev):
    """The bandwidth-bound kernels of the path at the workload's buffer sizes, alone: CUDA-event time and achieved
    HBM rate (algorithmic bytes / time) against the measured copy rate."""
    from opt_ring_flash_attn_b200 import _native

    B, S, Hq, Hkv, D, scale, std, seed, desc = cfg
    peaks, peak_kind = load_peaks()
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    q, k, v, dout = make_shard(cfg, 0, dev)
    spad = _native.padded_seq(S)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.randn_like(q)
    lse = torch.randn(B, Hq, spad, device=dev)
    delta, lse2 = torch.empty_like(lse), torch.empty_like(lse)
    dq_acc = torch.randn(_native.dq_acc_elems(B, S, Hq, D), device=dev)
    dq = torch.empty_like(q)
    a32 = torch.randn(2, B, S, Hkv, D, device=dev)
    b32 = torch.randn_like(a32)
    a16 = a32.to(q.dtype)
    dk = torch.empty_like(k)
    kv = torch.empty(2, B, S, Hkv, D, dtype=q.dtype, device=dev)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)
    e = q.element_size()
    n_q, n_kv = q.numel(), a32.numel()
    cases = [
        ("bwd_prepare (delta, lse2, accumulator cleared)", lambda: _native.bwd_prepare(out, dout, lse, delta, lse2, dq_acc, st),
         2 * n_q * e + 3 * lse.numel() * 4 + dq_acc.numel() * 4),
        ("dq_finalize (fp32 tiled accumulator -> dq)", lambda: _native.dq_finalize(dq_acc, dq), dq_acc.numel() * 4 + n_q * e),
        ("dkdv_accumulate (fp32 ring accumulate)", lambda: _native.dkdv_accumulate(a32, b32, a32), 3 * n_kv * 4),
        ("dkdv_accumulate_to16 (16-bit ring accumulate)", lambda: _native.dkdv_accumulate_to16(a16, b32, a16), n_kv * (4 + 2 * e)),
        ("cast_from_f32 (dK or dV)", lambda: _native.cast_from_f32(a32[0], dk), dk.numel() * (4 + e)),
        ("pack_kv (two device copies)", lambda: _native.pack_kv(k, v, kv), 2 * kv.numel() * e),
    ]
    rows = []
    for name, fn, nbytes in cases:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for i in range(10):
            flush.fill_(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = statistics.median(ts)
        rows.append({"kernel": name, "ms": round(ms, 4), "algorithmic_mb": round(nbytes / 1e6, 1),
                     "gb_s": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)})
    print(json.dumps({"aux_kernels": rows, "workload": f"{args.config}: {desc}", "hbm_peak_gb_s": hbm, "peak_kind": peak_kind,
                      "l2": "L2 flushed (256 MiB write) before every timed launch"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-zigzag-record", action="store_true", help="skip the zigzag sub-record at N > 1")
    ap.add_argument("--graph", action="store_true",
                    help="capture the step (forward + backward) into a CUDA graph and time replays (1 GPU only)")
    ap.add_argument("--zigzag", action="store_true",
                    help="zigzag layout (rank r holds chunks r and 2W-1-r) as the timed step; not the headline config")
    ap.add_argument("--hops", action="store_true", help="add the per-hop timeline of the slowest rank")
    ap.add_argument("--grid", default=None, choices=["speedup", "ablation"])
    ap.add_argument("--grid-head-dims", default="64,128", help="head dims of the grids, comma separated")
    ap.add_argument("--aux", action="store_true", help="time the bandwidth-bound kernels alone (1 GPU) and exit")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    B, S, Hq, Hkv, D, scale, std, seed, desc = cfg

    if args.impl == "reference":
        run_reference_arm(args, cfg, args.config)
        return

    import torch.distributed as dist

    from opt_ring_flash_attn_b200 import _native, ring_flash_attn, schedule, workspace

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _native.load()
    group = dist.group.WORLD if world > 1 else None

    if args.aux:
        aux_mode(args, cfg, dev)
        return

    if args.grid:
        grid_mode(args, dist, dev, rank, world)
        if world > 1:
            schedule.shutdown()
            dist.barrier()
            dist.destroy_process_group()
        return

    # at least three warm-up steps; the long-context workload (a step takes seconds) may run with fewer when asked to
    warmup = max(args.warmup, 1 if args.config == "c5" else 3)
    peaks, peak_kind = load_peaks()

    q, k, v, dout = make_shard(cfg, rank, dev)
    qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))

    def make_step(zigzag):
        def step_device():
            qg.grad = kg.grad = vg.grad = None
            out = ring_flash_attn(qg, kg, vg, softmax_scale=scale, causal=True, zigzag=zigzag, group=group)
            out.backward(dout)
            return out
        return step_device

    step_device = make_step(args.zigzag)

    if args.graph:
        if world > 1:
            raise SystemExit("--graph is measured on one GPU only")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # workspaces and function attributes are set up outside the capture
            for _ in range(2):
                step_device()
        torch.cuda.current_stream().wait_stream(side)
        qg.grad = kg.grad = vg.grad = None
        cuda_graph = torch.cuda.CUDAGraph()
        launches_c0 = _native.launch_count()
        with torch.cuda.graph(cuda_graph):
            ring_flash_attn(qg, kg, vg, softmax_scale=scale, causal=True, zigzag=args.zigzag).backward(dout)
        launches_per_replay = _native.launch_count() - launches_c0

        def step_device():  # noqa: F811 - the timed step is now one graph launch
            cuda_graph.replay()

    flush = None
    bytes_resident = sum(x.numel() * x.element_size() for x in (q, k, v, dout)) * 2 + q.numel() * 4
    if bytes_resident < 2 * 126 * 2 ** 20:
        flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from the warm-up on, so that short timed regions still get samples under load
    sampler = ClockSampler(local_rank, period_ms=100 if world == 1 else 25)
    sampler.start()
    for _ in range(warmup):
        step_device()
    barrier()
    launches0 = _native.launch_count()
    ms_max = timed_region(step_device, args.steps, 0, barrier, flush, dev, dist, world)
    launches = _native.launch_count() - launches0
    if args.graph:
        launches = launches_per_replay * args.steps  # the kernels run from the graph, not through the C ABI
    clocks = sampler.stop()
    if world > 1:  # the slowest rank is the one under sustained load: every rank's record goes into the line
        per_rank = [None] * world
        dist.all_gather_object(per_rank, {"sm_mhz": clocks.get("sm_mhz"), "sm_min_mhz": clocks.get("sm_min_mhz"),
                                          "power_w_max": clocks.get("power_w_max"), "reasons": clocks.get("reasons")})
        clocks["per_rank"] = per_rank
        clocks["reasons"] = sorted({r for c in per_rank for r in (c.get("reasons") or [])})

    # ---- zigzag layout beside the headline (same process; the same shards read as the zigzag arrangement) ----
    zigzag_rec = None
    if world > 1 and not args.zigzag and not args.no_zigzag_record and S % 256 == 0:
        zsteps = max(3, min(args.steps, 10))
        zz_ms = timed_region(make_step(True), zsteps, 3, barrier, flush, dev, dist, world)
        fb = f_blk(B, S, Hq, D)
        zigzag_rec = {"ms_per_step": zz_ms, "steps": zsteps,
                      "value": 3.5 * (world * world / 2.0) * fb / (zz_ms * 1e-3) / 1e12,
                      "tflops_per_gpu": 3.5 * (world / 2.0) * fb / (zz_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "note": "rank r holds chunks r and 2W-1-r of 2W: every rank does W/2 block-equivalents"}

    # ---- per-hop timeline (slowest rank's table) ----
    hops = None
    if args.hops:
        sc = D ** -0.5 if scale is None else scale
        hs = ClockSampler(local_rank, period_ms=20)  # started early: nvidia-smi needs a moment to deliver samples
        hs.start()
        for _ in range(3):
            timeline_step(_native, schedule, group, q, k, v, dout, sc, args.zigzag)
        barrier()
        tables = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            rows, transfers = timeline_step(_native, schedule, group, q, k, v, dout, sc, args.zigzag)
            e1.record()
            torch.cuda.synchronize()
            tb = summarize_timeline(rows, transfers)
            tb["step_ms"] = round(e0.elapsed_time(e1), 4)
            tables.append(tb)
        hclk = hs.stop()
        mine = sorted(tables, key=lambda x: x["step_ms"])[len(tables) // 2]
        mine["rank"] = rank
        mine["sm_mhz_median"] = hclk.get("sm_mhz")
        mine["reasons"] = hclk.get("reasons")
        if world > 1:
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
        else:
            everyone = [mine]
        slowest = max(everyone, key=lambda x: x["step_ms"])
        hops = {"slowest_rank": slowest,
                "per_rank_step_ms": [x["step_ms"] for x in everyone],
                "per_rank_hop_kernel_ms": [x["hop_kernel_ms"] for x in everyone],
                "per_rank_exposed_wait_ms": [round(sum(x["exposed_wait_ms"].values()), 4) for x in everyone],
                "per_rank_sm_mhz": [x["sm_mhz_median"] for x in everyone]}

    # ---- dominant kernel alone: backward hop on this rank's own (diagonal) block ----
    with torch.no_grad():
        # single-device forward of the diagonal block gives out/lse for the backward kernel
        spad = _native.padded_seq(S)
        out_d = torch.empty_like(q)
        lse_d = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        sc = D ** -0.5 if scale is None else scale
        _native.fwd_hop(q, k, v, None, None, None, out_d, lse_d, sc, True, True, True, st)
        delta = torch.empty(B, Hq, spad, dtype=torch.float32, device=dev)
        lse2 = torch.empty_like(delta)
        dq_acc = torch.empty(_native.dq_acc_elems(B, S, Hq, D), dtype=torch.float32, device=dev)
        dkdv = torch.empty(2, B, S, Hkv, D, dtype=torch.float32, device=dev)
        _native.bwd_prepare(out_d, dout, lse_d, delta, lse2, dq_acc, st)
        kreps = 3 if args.config == "c5" else max(3, min(args.steps, 10))

        def time_kernel(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(kreps)]
            for i in range(kreps):
                if flush is not None:
                    flush.fill_(i & 0xFF)
                evs[i][0].record()
                fn()
                evs[i][1].record()
            torch.cuda.synchronize()
            return sum(a.elapsed_time(b) for a, b in evs) / kreps

        bwd_ms = time_kernel(lambda: _native.bwd_hop(q, k, v, dout, lse2, delta, dq_acc, None, dkdv, sc, False, True, st))
        fwd_ms = time_kernel(lambda: _native.fwd_hop(q, k, v, None, None, None, out_d, lse_d, sc, True, True, True, st))
        bwd_full_ms = fwd_full_ms = None
        if args.config != "c5":
            bwd_full_ms = time_kernel(
                lambda: _native.bwd_hop(q, k, v, dout, lse2, delta, dq_acc, None, dkdv, sc, False, False, st))
            fwd_full_ms = time_kernel(
                lambda: _native.fwd_hop(q, k, v, None, None, None, out_d, lse_d, sc, True, True, False, st))
        _native.check_status(st, "bench kernels")
        del out_d, lse_d, delta, lse2, dq_acc, dkdv

    # ---- end to end through the public API with host buffers ----
    e2e_ms = None
    if not args.no_e2e:
        hq, hk, hv, hdo = make_shard(cfg, rank, None, pinned=True)
        # Two sets of device input buffers and pinned result buffers, one copy stream per direction: the H2D copy
        # of step i+1 and the D2H copy of step i-1 overlap the kernels of step i (PCIe is full duplex).  Every
        # step still copies its own inputs in and its own results out inside the timed region.
        host_in = (hq, hk, hv, hdo)
        dev_in = [[torch.empty_like(x, device=dev) for x in host_in] for _ in range(2)]
        host_out = [[torch.empty_like(x).pin_memory() for x in (hq, hq, hk, hv)] for _ in range(2)]
        h2d_s, d2h_s = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [torch.cuda.Event(), torch.cuda.Event()]
        ev_done = [torch.cuda.Event(), torch.cuda.Event()]
        cur = torch.cuda.current_stream(dev)
        for e in ev_done:
            e.record(cur)

        def step_e2e(i):
            sl = i & 1
            with torch.cuda.stream(h2d_s):
                h2d_s.wait_event(ev_done[sl])  # the step that last used this input set has finished
                for d_, h_ in zip(dev_in[sl], host_in):
                    d_.copy_(h_, non_blocking=True)
                ev_in[sl].record(h2d_s)
            cur.wait_event(ev_in[sl])
            a, b_, c = (x.detach().requires_grad_(True) for x in dev_in[sl][:3])
            o = ring_flash_attn(a, b_, c, softmax_scale=scale, causal=True, zigzag=args.zigzag, group=group)
            o.backward(dev_in[sl][3])
            ev_done[sl].record(cur)
            res = (o.detach(), a.grad, b_.grad, c.grad)
            with torch.cuda.stream(d2h_s):
                d2h_s.wait_event(ev_done[sl])
                for t_, h_ in zip(res, host_out[sl]):
                    h_.copy_(t_, non_blocking=True)
                    t_.record_stream(d2h_s)

        for i in range(2):
            step_e2e(i)
        cur.wait_stream(d2h_s)
        barrier()
        e_steps = 2 if args.config == "c5" else max(4, min(args.steps, 10))
        # Host-side copies share PCIe and host memory with whatever else runs on the machine: the region is timed
        # three times; the median pass is reported and all passes are listed beside it.
        e2e_passes = []
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(e_steps):
                step_e2e(i)
            cur.wait_stream(d2h_s)  # the last results have reached host memory
            e1.record()
            barrier()
            te = torch.tensor([e0.elapsed_time(e1) / e_steps], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            e2e_passes.append(float(te.item()))
        e2e_ms = statistics.median(e2e_passes)
        h2d = sum(x.numel() * x.element_size() for x in host_in)
        d2h = sum(x.numel() * x.element_size() for x in host_out[0])
    workspace.check_all("bench")

    line = None
    if rank == 0:
        W = world
        fb = f_blk(B, S, Hq, D)
        flops_job = 3.5 * (W * W / 2.0) * fb
        # contiguous shards: the last rank does W - 1/2 block-equivalents; zigzag: every rank does W/2
        flops_slowest = 3.5 * (W / 2.0 if args.zigzag else (W - 0.5)) * fb
        value = flops_job / (ms_max * 1e-3) / 1e12
        slowest = flops_slowest / (ms_max * 1e-3) / 1e12
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        peak_sus = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        bwd_flops = 2.5 * 0.5 * fb
        fwd_flops = 0.5 * fb
        achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
        traffic, traffic_note = captured_traffic(args.config) if W == 1 else (None, "reported at N=1 only")

        def rate(flops, ms):
            return None if ms is None else {"achieved": flops / (ms * 1e-3) / 1e12, "ms_per_launch": ms,
                                            "frac": flops / (ms * 1e-3) / 1e12 / peak}

        line = {
            "metric": "causal_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": W, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.config}: {desc}, causal, fwd+bwd, world size {W}"
                                   + (", zigzag layout" if args.zigzag else ", contiguous shards")
                                   + (", step replayed from a CUDA graph" if args.graph else ""),
                       "l2": "L2 flushed (256 MiB write) between timed steps" if flush is not None
                             else "per-step inputs+outputs exceed the 126 MB L2",
                       "flops": "algorithmic causal FLOPs: 3.5*(W^2/2)*4*B*Hq*S_local^2*D for the job"},
            "slowest_rank_tflops_per_gpu": slowest,
            "slowest_rank_frac_of_peak": slowest / peak_sus,
            "slowest_rank_frac_of_burst_peak": slowest / peak,
            "peak_used_for_step": {"bf16_tflops_sustained": peak_sus, "bf16_tflops_burst": peak, "kind": peak_kind},
            "roofline": {"bound": "tensor", "kernel": "bwd_hop_kernel (diagonal block)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_kind": peak_kind + " burst",
                         "traffic": traffic, "traffic_note": traffic_note, "ms_per_launch": bwd_ms,
                         "bwd_hop_full_block": rate(2.5 * fb, bwd_full_ms),
                         "fwd_hop": rate(fwd_flops, fwd_ms),
                         "fwd_hop_full_block": rate(fb, fwd_full_ms)},
            "gpu_launches": launches, "clocks": clocks,
        }
        if zigzag_rec is not None:
            line["zigzag"] = zigzag_rec
        if hops is not None:
            line["hops"] = hops
        if e2e_ms is not None:
            line["e2e"] = {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "passes_ms_per_step": e2e_passes, "reported": "median of the passes",
                           "pipelining": "per step: inputs copied from pinned host memory, out/dq/dk/dv copied back; "
                                         "copies of neighbouring steps overlap the kernels (2 buffer sets, 3 streams)"}
        if W == 1 and not args.no_cpu_baseline:
            try:
                _, line["cpu_baseline"] = time_reference_cpu(steps=3, warmup=1)
            except Exception as e:  # the GPU line stands without it
                line["cpu_baseline"] = {"unavailable": f"{type(e).__name__}: {e}"}

    # ---- balanced execution of the same contiguous shards (regroup to zigzag, run, regroup back), same process ----
    # Measured last and under a watchdog: its exchange of half-shards is the one part of this file that goes through
    # the process group's own point-to-point path.  If it does not come back in time, the line is printed without it.
    if world > 1 and not args.zigzag and not args.no_zigzag_record and S % 256 == 0 and args.config != "c5":
        done = threading.Event()

        def give_up():
            if not done.wait(90.0):
                if rank == 0:
                    line["balanced"] = {"unavailable": "did not finish within 90 s"}
                    print(json.dumps(line), flush=True)
                os._exit(0)

        threading.Thread(target=give_up, daemon=True).start()
        balanced_rec = None
        try:
            from opt_ring_flash_attn_b200 import balanced

            def step_balanced():
                qg.grad = kg.grad = vg.grad = None
                with balanced():
                    ring_flash_attn(qg, kg, vg, softmax_scale=scale, causal=True, group=group).backward(dout)

            bsteps = max(3, min(args.steps, 10))
            b_ms = timed_region(step_balanced, bsteps, 3, barrier, flush, dev, dist, world)
            workspace.check_all("bench, balanced")
            fb_ = f_blk(B, S, Hq, D)
            balanced_rec = {"ms_per_step": b_ms, "steps": bsteps,
                            "value": 3.5 * (world * world / 2.0) * fb_ / (b_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                            "note": "contiguous shards in and out; inside, the half-shards are exchanged so that every "
                                    "rank does W/2 block-equivalents (the exchange is inside the timed step)"}
        except Exception as e:  # the headline line stands without it
            balanced_rec = {"unavailable": f"{type(e).__name__}: {e}"}
        done.set()
        if rank == 0:
            line["balanced"] = balanced_rec
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        schedule.shutdown()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
