"""Host-side pieces of ``bench.py`` that need no GPU: the bounded reference leg, the host thread count,
and the ncu traffic record that is only reported while the kernel sources it was captured on are unchanged."""

import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def test_host_thread_count_is_positive_and_applied():
    n = bench._all_host_threads()
    assert n >= 1 and torch.get_num_threads() == n


def _stub_oracle(monkeypatch, seconds):
    from oracle import pi05_ref

    calls = []

    def fake(deq, shape, *inputs):
        calls.append(len(calls))
        time.sleep(seconds)
        return torch.zeros(1, 2, 3)

    monkeypatch.setattr(pi05_ref, "sample_actions", fake)
    monkeypatch.setattr(bench, "_oracle_inputs", lambda frames, cameras: ())
    return calls


def test_reference_leg_runs_the_requested_chunks_on_a_fast_host(monkeypatch):
    calls = _stub_oracle(monkeypatch, 0.0)
    times, out = bench._cpu_chunks(None, [[None]], ["cam"], None, warmup=3, reps=5, budget_s=240.0)
    assert len(times) == 5 and len(calls) == 8 and out.shape == (1, 2, 3)
    times, _ = bench._cpu_chunks(None, [[None]], ["cam"], None, warmup=1, reps=2)  # no budget: plain loop
    assert len(times) == 2


def test_reference_leg_stays_inside_its_budget_on_a_slow_host(monkeypatch):
    calls = _stub_oracle(monkeypatch, 0.05)
    t0 = time.perf_counter()
    times, _ = bench._cpu_chunks(None, [[None]], ["cam"], None, warmup=3, reps=50, budget_s=0.3)
    assert 1 <= len(times) < 50          # stopped by the budget, after at least one timed chunk
    assert len(calls) - len(times) <= 3  # slow warm-ups are cut short, never more than asked for
    assert time.perf_counter() - t0 < 1.0


def test_traffic_record_is_reported_only_for_the_sources_it_was_captured_on(monkeypatch, tmp_path):
    traffic, note = bench._traffic()
    rec = json.load(open(bench.TRAFFIC_FILE))
    if traffic is not None:  # the committed record matches the committed sources
        assert traffic == rec["dram_bytes_per_launch"] and str(rec["algorithmic_bytes"]) in note
    else:
        assert "stale" in note or "no ncu record" in note
    stale = dict(rec, source_sha256={k: "0" * 64 for k in rec["source_sha256"]})
    path = tmp_path / "record.json"
    path.write_text(json.dumps(stale))
    monkeypatch.setattr(bench, "TRAFFIC_FILE", str(path))
    traffic, note = bench._traffic()
    assert traffic is None and note.startswith("stale")
    monkeypatch.setattr(bench, "TRAFFIC_FILE", str(tmp_path / "missing.json"))
    assert bench._traffic()[0] is None
