"""Tests of the latency benchmark CLI (gdn2_sm120_b200/benchmark.py), the counterpart of the
reference's src/gdn2_sm120/benchmark.py: grid, record schema and, on a GPU, one measured point per mode."""

from __future__ import annotations

import json

import pytest
import torch

from gdn2_sm120_b200 import benchmark


def test_reference_grid_has_the_published_89_points():
    grid = benchmark.reference_grid()
    assert len(grid) == 89 and len(set(grid)) == 89
    by_mode = {mode: sum(1 for m, _, _ in grid if m == mode) for mode in benchmark.MODES}
    assert by_mode == {"chunk-forward": 33, "chunk-backward": 32, "chunk-training": 0, "token-forward": 24}
    assert ("chunk-backward", 4, 32768) not in grid and ("chunk-forward", 4, 32768) in grid


def test_algorithmic_bytes_per_mode():
    th = 2 * 64 * 3
    states = 2 * 3 * 65536
    assert benchmark.algorithmic_bytes("chunk-forward", 2, 64, 3) == 2048 * th + 2 * states
    assert benchmark.algorithmic_bytes("chunk-backward", 2, 64, 3) == 3840 * th + 2 * states
    assert benchmark.algorithmic_bytes("chunk-training", 2, 64, 3) == 5888 * th + 4 * states


def _fake_record(**over):
    rec = {"mode": "chunk-forward", "batch": 1, "time": 64, "heads": 16, "dtype": "bf16", "warmup": 5,
           "clock_stabilization_ms": 1000, "repeats": 50, "scale": 0.125, "device": "x",
           "b200": {"implementation": benchmark.IMPLEMENTATION, "median_us": 2.0, "minimum_us": 1.5}}
    rec.update(over)
    return rec


def test_document_envelope_and_validation():
    doc = benchmark.document([_fake_record()], suite_id="t")
    assert doc["schema_version"] == 2 and doc["results"][0]["b200"]["median_us"] == 2.0
    benchmark.validate_document(json.loads(json.dumps(doc)))
    with pytest.raises(ValueError, match="unknown mode"):
        benchmark.validate_document(benchmark.document([_fake_record(mode="nope")], "t"))
    with pytest.raises(ValueError, match="minimum_us"):
        bad = _fake_record()
        bad["b200"] = dict(bad["b200"], minimum_us=3.0)
        benchmark.validate_document(benchmark.document([bad], "t"))
    with pytest.raises(ValueError, match="schema-2"):
        benchmark.validate_document({"results": []})


def test_cli_refuses_to_run_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(SystemExit, match="no CPU path"):
        benchmark.main(["--mode", "token-forward", "--time", "1"])
    with pytest.raises(SystemExit, match="positive"):
        benchmark.main(["--batch", "0"])


@pytest.mark.gpu
@pytest.mark.parametrize("mode,time_", [("chunk-forward", 128), ("chunk-backward", 128), ("chunk-training", 64),
                                        ("token-forward", 4)])
def test_one_measured_point_per_mode(mode, time_, tmp_path):
    path = tmp_path / "r.json"
    benchmark.main(["--mode", mode, "--batch", "1", "--time", str(time_), "--heads", "2", "--warmup", "1",
                    "--repeats", "3", "--json", str(path)])
    doc = json.loads(path.read_text())
    benchmark.validate_document(doc)
    (record,) = doc["results"]
    assert record["mode"] == mode and record["time"] == time_ and record["triton"] is None
    assert record["tokens_per_s"] > 0 and record["algorithmic_gbs"] > 0
