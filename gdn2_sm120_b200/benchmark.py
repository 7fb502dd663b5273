"""Latency benchmark of the public operators, in the reference's result format.

    python -m gdn2_sm120_b200.benchmark --mode chunk-forward --batch 4 --time 8192 --heads 16
    python -m gdn2_sm120_b200.benchmark --suite reference --json results.json

Counterpart of the reference's benchmark CLI (src/gdn2_sm120/benchmark.py:33-60, 388-434):
same modes, same flags, same measurement (count-based warm-up, a clock-stabilisation phase of a
GEMM loop followed by the target itself, then ``repeats`` samples taken with CUDA events around
the public Python call; median and minimum are reported), and by default the same synthetic
inputs (seed 20260824: L2-normalised q/k, v = 0.2 N(0,1), g = -U(0, 0.03), sigmoid gates,
state = 0.03 N(0,1), scale 0.125; benchmark.py:99-126 there).  ``--inputs baseline`` draws the
stronger-decay distributions of this repository's own benchmark instead.

A result is one record of the reference's published schema (version 2,
docs/data/benchmark-results-sm120.json there): ``mode, batch, time, heads, dtype, warmup,
clock_stabilization_ms, repeats`` and a timing object ``{implementation, median_us, minimum_us,
process_medians_us, process_minimums_us}``.  The timing object is stored under ``b200`` (the
reference stores its own under ``cute``); ``triton``, ``speedup`` and ``validation_max_abs`` are
present and null, because the comparison against the official Triton implementation needs an
external checkout and is not part of this package.  Each record also carries what the reference's
lacks: tokens/s, the algorithmic HBM bandwidth and its fraction of the measured peak.

``--suite reference`` runs the grid of the reference's published table (33 forward, 32
backward-only and 24 token-forward points, B in {1, 2, 4}, H = 16) in this process and writes
one schema-2 document.
"""

from __future__ import annotations

import argparse
import datetime
import json
import math
import pathlib
import statistics
import time
from collections.abc import Callable

import torch

from .ops import chunk_gdn2, recurrent_gdn2

IMPLEMENTATION = "b200-sm100a"
SCHEMA_VERSION = 2
MODES = ("chunk-forward", "chunk-backward", "chunk-training", "token-forward")

_GEMM_CLOCK_STABILIZATION_SECONDS = 0.25
_TARGET_CLOCK_STABILIZATION_SECONDS = 0.75
_CLOCK_STABILIZATION_DIMENSION = 4096

# compulsory bytes per token-head: read q k v beta w (16-bit) + g (fp32), write o; backward reads
# the inputs and dO and writes six gradients
_FWD_BYTES = 5 * 256 + 512 + 256
_BWD_BYTES = (5 * 256 + 512 + 256) + (5 * 256 + 512)
_STATE_BYTES = 128 * 128 * 4


def reference_grid() -> list[tuple[str, int, int]]:
    """(mode, batch, time) of every point in the reference's published table (H = 16)."""

    lengths = [16, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768]
    grid = [("chunk-forward", b, t) for b in (1, 2, 4) for t in lengths]
    grid += [("chunk-backward", b, t) for b in (1, 2, 4) for t in lengths if not (b == 4 and t == 32768)]
    grid += [("token-forward", b, t) for b in (1, 2, 4) for t in (1, 2, 4, 8, 16, 32, 64, 128)]
    return grid


def make_inputs(batch: int, time_: int, heads: int, dtype: torch.dtype, *, kind: str = "reference",
                device: str | torch.device = "cuda"):
    """Synthetic q, k, v, g, beta, w, state on the device."""

    generator = torch.Generator(device=device).manual_seed(20260824)
    shape = (batch, time_, heads, 128)

    def randn(*size, dt=torch.float32):
        return torch.randn(*size, generator=generator, device=device, dtype=dt)

    q = torch.nn.functional.normalize(randn(*shape), dim=-1).to(dtype)
    k = torch.nn.functional.normalize(randn(*shape), dim=-1).to(dtype)
    if kind == "reference":
        v = randn(*shape, dt=dtype) * 0.2
        g = -torch.rand(shape, generator=generator, device=device, dtype=torch.float32) * 0.03
        beta = torch.sigmoid(randn(*shape, dt=dtype))
        w = torch.sigmoid(randn(*shape, dt=dtype))
        state = randn(batch, heads, 128, 128) * 0.03
    elif kind == "baseline":
        v = randn(*shape).to(dtype)
        beta = torch.sigmoid(randn(*shape)).to(dtype)
        w = torch.sigmoid(randn(*shape)).to(dtype)
        g = -torch.clamp(torch.nn.functional.softplus(randn(*shape) - 2.0), max=5.0)
        state = randn(batch, heads, 128, 128) * 0.02
    else:
        raise ValueError("inputs must be 'reference' or 'baseline'")
    return q, k, v, g, beta, w, state


def _stabilize_clocks() -> None:
    shape = (_CLOCK_STABILIZATION_DIMENSION, _CLOCK_STABILIZATION_DIMENSION)
    left = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    right = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    deadline = time.perf_counter() + _GEMM_CLOCK_STABILIZATION_SECONDS
    while time.perf_counter() < deadline:
        torch.mm(left, right, out=out)
        torch.cuda.synchronize()


def measure(call: Callable[[], object], warmup: int, repeats: int) -> tuple[float, float]:
    """Median and minimum latency of ``call`` in microseconds (CUDA events, one sync per sample)."""

    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    _stabilize_clocks()
    deadline = time.perf_counter() + _TARGET_CLOCK_STABILIZATION_SECONDS
    while time.perf_counter() < deadline:
        call()
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    samples = []
    for _ in range(repeats):
        start.record()
        call()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end) * 1000.0)
    return statistics.median(samples), min(samples)


def _build_call(mode: str, inputs, scale: float) -> Callable[[], object]:
    q, k, v, g, beta, w, state = inputs
    if mode == "chunk-forward":
        return lambda: chunk_gdn2(q, k, v, g, beta, w, state, scale=scale, output_final_state=True)
    if mode == "token-forward":
        return lambda: recurrent_gdn2(q, k, v, g, beta, w, state, scale=scale)
    if mode not in ("chunk-backward", "chunk-training"):
        raise ValueError(f"unknown mode {mode}")
    generator = torch.Generator(device=q.device).manual_seed(20260825)
    upstream_o = torch.randn(v.shape, generator=generator, device=v.device, dtype=v.dtype) * 0.2
    upstream_state = torch.randn(state.shape, generator=generator, device=v.device, dtype=torch.float32) * 0.1
    leaves = [t.detach().requires_grad_() for t in (q, k, v, g, beta, w)]
    state_leaf = state.detach().requires_grad_()
    grad_inputs = (*leaves, state_leaf)
    if mode == "chunk-backward":
        # backward only: the forward runs once, every sample differentiates the retained graph
        out, final = chunk_gdn2(*leaves, state_leaf, scale=scale, output_final_state=True)
        return lambda: torch.autograd.grad((out, final), grad_inputs, (upstream_o, upstream_state),
                                           retain_graph=True)

    def training():
        out, final = chunk_gdn2(*leaves, state_leaf, scale=scale, output_final_state=True)
        return torch.autograd.grad((out, final), grad_inputs, (upstream_o, upstream_state))

    return training


def _measured_hbm_peak() -> float | None:
    path = pathlib.Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return None


def algorithmic_bytes(mode: str, batch: int, time_: int, heads: int) -> int:
    """Compulsory HBM traffic of one call (sequence tensors plus the states that enter and leave)."""

    token_heads = batch * time_ * heads
    states = batch * heads * _STATE_BYTES
    if mode in ("chunk-forward", "token-forward"):
        return _FWD_BYTES * token_heads + 2 * states
    if mode == "chunk-backward":
        return _BWD_BYTES * token_heads + 2 * states
    return (_FWD_BYTES + _BWD_BYTES) * token_heads + 4 * states


def run_point(mode: str, batch: int, time_: int, heads: int, *, dtype: str = "bf16", scale: float = 0.125,
              warmup: int = 5, repeats: int = 50, inputs: str = "reference") -> dict:
    """Measure one point and return its schema-2 record."""

    if mode not in MODES:
        raise ValueError(f"mode must be one of {MODES}")
    if min(batch, time_, heads, warmup, repeats) <= 0:
        raise ValueError("batch, time, heads, warmup, and repeats must be positive")
    if not math.isfinite(scale):
        raise ValueError("benchmark scale must be finite")
    torch_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    tensors = make_inputs(batch, time_, heads, torch_dtype, kind=inputs)
    call = _build_call(mode, tensors, scale)
    median_us, minimum_us = measure(call, warmup, repeats)
    nbytes = algorithmic_bytes(mode, batch, time_, heads)
    gbs = nbytes / (median_us * 1e-6) / 1e9
    peak = _measured_hbm_peak()
    return {
        "mode": mode, "batch": batch, "time": time_, "heads": heads, "dtype": dtype,
        "warmup": warmup,
        "clock_stabilization_ms": round((_GEMM_CLOCK_STABILIZATION_SECONDS
                                         + _TARGET_CLOCK_STABILIZATION_SECONDS) * 1000),
        "repeats": repeats,
        "b200": {"implementation": IMPLEMENTATION, "median_us": median_us, "minimum_us": minimum_us,
                 "process_medians_us": [median_us], "process_minimums_us": [minimum_us]},
        "triton": None, "speedup": None, "validation_max_abs": None,
        "official_commit": None, "fla_commit": None,
        "qk_l2_normalized": True, "scale": scale,
        "device": torch.cuda.get_device_name(), "torch_version": str(torch.__version__),
        "cuda_runtime": str(torch.version.cuda), "process_repeats": 1,
        "inputs": inputs,
        "tokens_per_s": batch * time_ / (median_us * 1e-6),
        "algorithmic_bytes": nbytes, "algorithmic_gbs": gbs,
        "hbm_roofline_frac": (gbs / peak) if peak else None,
    }


def document(results: list[dict], suite_id: str) -> dict:
    """Wrap records in the schema-2 envelope of the reference's published file."""

    return {
        "schema_version": SCHEMA_VERSION,
        "suite_id": suite_id,
        "measured_at": datetime.date.today().isoformat(),
        "aggregation": {"unit": "single-process median", "default_process_repeats": 1},
        "hbm_peak_gbs": _measured_hbm_peak(),
        "results": results,
    }


def validate_document(doc: dict) -> None:
    """Check a document against the fields the reference's schema-2 consumers read."""

    if doc.get("schema_version") != SCHEMA_VERSION or not isinstance(doc.get("results"), list):
        raise ValueError("not a schema-2 benchmark document")
    for record in doc["results"]:
        for key in ("mode", "batch", "time", "heads", "dtype", "warmup", "clock_stabilization_ms", "repeats",
                    "b200", "scale", "device"):
            if key not in record:
                raise ValueError(f"record lacks {key!r}")
        if record["mode"] not in MODES:
            raise ValueError(f"unknown mode {record['mode']!r}")
        timing = record["b200"]
        if not (timing["minimum_us"] > 0 and timing["median_us"] >= timing["minimum_us"]):
            raise ValueError("timing must satisfy 0 < minimum_us <= median_us")


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--mode", choices=MODES, default="chunk-forward")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--time", type=int, default=16)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--dtype", choices=("bf16", "fp16"), default="bf16")
    parser.add_argument("--scale", type=float, default=0.125, help="explicit output scale")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--repeats", type=int, default=50)
    parser.add_argument("--inputs", choices=("reference", "baseline"), default="reference",
                        help="input distributions: the reference benchmark's, or this repository's benchmark's")
    parser.add_argument("--suite", choices=("reference",),
                        help="run every point of the reference's published table instead of one point")
    parser.add_argument("--max-time", type=int, default=None, help="with --suite: skip longer sequences")
    parser.add_argument("--json", type=pathlib.Path, help="also write the result(s) as a schema-2 document")
    return parser


def main(argv: list[str] | None = None) -> None:
    args = _parser().parse_args(argv)
    if min(args.batch, args.time, args.heads, args.warmup, args.repeats) <= 0:
        raise SystemExit("batch, time, heads, warmup, and repeats must be positive")
    if not torch.cuda.is_available():
        raise SystemExit("the benchmark needs a B200 GPU: there is no CPU path to time")
    if args.suite:
        points = [(m, b, t) for m, b, t in reference_grid() if args.max_time is None or t <= args.max_time]
        heads = 16
    else:
        points, heads = [(args.mode, args.batch, args.time)], args.heads
    results = []
    for mode, batch, time_ in points:
        record = run_point(mode, batch, time_, heads, dtype=args.dtype, scale=args.scale, warmup=args.warmup,
                           repeats=args.repeats, inputs=args.inputs)
        results.append(record)
        frac = record["hbm_roofline_frac"]
        print(f"{mode} B={batch} T={time_} H={heads} {args.dtype}: {IMPLEMENTATION}="
              f"{record['b200']['median_us']:.1f} us (min {record['b200']['minimum_us']:.1f}), "
              f"{record['tokens_per_s'] / 1e6:.2f} M tokens/s, {record['algorithmic_gbs']:.0f} GB/s"
              + (f" = {100 * frac:.1f} % of measured HBM peak" if frac else ""), flush=True)
        torch.cuda.empty_cache()
    if args.json is not None:
        doc = document(results, suite_id=f"b200-sm100a-{datetime.date.today().isoformat()}")
        validate_document(doc)
        args.json.parent.mkdir(parents=True, exist_ok=True)
        args.json.write_text(json.dumps(doc, indent=2) + "\n", encoding="utf-8")


if __name__ == "__main__":
    main()
