"""Tracing ranges: off by default, recorded with names and durations when on, exported as Chrome-trace JSON."""

import json

import torch

from astrai_b200.utils import trace


def test_ranges_are_free_when_off_and_recorded_when_on(tmp_path):
    import sys

    sys.path.insert(0, str(__import__("pathlib").Path(__file__).parent))
    from helpers import tiny_config

    from astrai_b200.models import AutoRegressiveLM

    trace.disable()
    trace.clear()
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.tensor([[1, 2, 3, 4]])
    with torch.no_grad():
        model(ids)
    assert trace.events() == []
    trace.enable(record=True)
    try:
        with trace.range("step"):
            with torch.no_grad():
                model(ids)
            trace.mark("sampled")
        evs = trace.events()
        names = [e["name"] for e in evs]
        assert names[:len(model.layers)] == [f"layer{i}" for i in range(len(model.layers))]
        assert names[-2:] == ["sampled", "step"] and all(e["host_ms"] >= 0 for e in evs)
        step = evs[-1]
        assert step["host_ms"] >= sum(e["host_ms"] for e in evs[:len(model.layers)]) * 0.99  # the outer range covers the layers
        path = tmp_path / "trace.json"
        assert trace.export_chrome_trace(str(path), rank=3) == len(evs)
        doc = json.loads(path.read_text())
        assert {r["name"] for r in doc["traceEvents"]} >= {"step", "layer0"} and doc["traceEvents"][0]["pid"] == 3
    finally:
        trace.disable()
        trace.clear()
