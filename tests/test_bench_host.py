"""Host-side pieces of bench.py that need no GPU: FLOP accounting, the traffic record keyed by the kernel's source
digest, and the summary of a per-hop timeline."""
import importlib.util
import json
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_flop_accounting_matches_the_stated_totals():
    b = _bench()
    B, S, Hq, Hkv, D = b.CONFIGS["c3"][:5]
    fb = b.f_blk(B, S, Hq, D)
    assert abs(fb / 1e12 - 1.0995) < 1e-3                      # one full block forward
    assert abs(3.5 * 7.5 * fb / 1e12 - 28.862) < 1e-2          # slowest rank of 8, forward + backward
    c = b.REF_SAMPLE
    assert abs(b._ref_flops() - 3.5 * 32 * b.f_blk(c["B"], 256, c["H"], c["D"])) < 1.0


def test_traffic_record_is_only_used_for_the_kernel_it_was_captured_from(tmp_path, monkeypatch):
    b = _bench()
    rec = json.loads((ROOT / "profiles" / "roofline_traffic.json").read_text())["bwd_hop_kernel/c3/diagonal"]
    traffic, note = b.captured_traffic("c3")
    if rec["source_digest"] == b.kernel_digest():
        assert traffic == rec["dram_bytes_per_launch"] and "dram__bytes" in note
    else:
        assert traffic is None and "changed" in note
    assert b.captured_traffic("c4")[0] is None               # nothing recorded for that workload
    monkeypatch.setattr(b, "kernel_digest", lambda *a, **k: "0" * 16)
    assert b.captured_traffic("c3") == (None, "kernel sources changed since the ncu capture")


def test_timeline_summary():
    b = _bench()
    rows = [{"pass": "fwd", "what": "pack_kv", "ms": 0.02}, {"pass": "fwd", "what": "fwd_hop", "ms": 0.5},
            {"pass": "fwd", "what": "wait fwd_kv", "ms": 0.003}, {"pass": "fwd", "what": "fwd_hop", "ms": 1.0},
            {"pass": "bwd", "what": "bwd_prepare", "ms": 0.06}, {"pass": "bwd", "what": "bwd_hop", "ms": 1.4},
            {"pass": "bwd", "what": "wait bwd_dkdv", "ms": 0.2}, {"pass": "bwd", "what": "dkdv_accumulate", "ms": 0.04}]
    s = b.summarize_timeline(rows, [{"ring": "fwd_kv", "bytes": 1000, "ms": 0.1, "gb_s": 0.01}])
    assert s["fwd_hop_ms"] == [0.5, 1.0] and s["bwd_hop_ms"] == [1.4]
    assert abs(s["hop_kernel_ms"] - 2.9) < 1e-9 and abs(s["accumulate_ms"] - 0.04) < 1e-9
    assert abs(s["other_kernel_ms"] - 0.08) < 1e-9 and abs(s["kernel_ms"] - 3.02) < 1e-9
    assert s["exposed_wait_ms"] == {"fwd_kv": 0.003, "bwd_kv": 0, "bwd_dkdv": 0.2}
