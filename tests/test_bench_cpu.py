"""CPU-side checks of bench.py: the reference arm's JSON contract, the fused loss, the clock
sampler's behaviour without a GPU, and that the GPU arm refuses to run without CUDA."""

from __future__ import annotations

import json
import pathlib
import subprocess
import sys

import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_reference_arm_prints_one_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]
    assert "workload" in line["config"]


def test_mean_square_loss_matches_autograd():
    torch.manual_seed(0)
    x = torch.randn(3, 5, 7, dtype=torch.bfloat16, requires_grad=True)
    loss = bench._MeanSquare.apply(x) * 3.0
    (grad,) = torch.autograd.grad(loss, x)
    y = x.detach().clone().requires_grad_(True)
    ref = y.float().square().mean() * 3.0
    (ref_grad,) = torch.autograd.grad(ref, y)
    torch.testing.assert_close(loss, ref, rtol=1e-6, atol=1e-7)
    torch.testing.assert_close(grad.float(), ref_grad.float(), rtol=2e-2, atol=1e-6)
    assert grad.dtype == torch.bfloat16


def test_clock_sampler_reports_without_a_gpu():
    sampler = bench.ClockSampler(0, period_s=0.001)
    sampler.start()
    sampler.mark()
    report = sampler.stop()
    assert {"sm_mhz", "sm_max_mhz", "samples", "reasons"} <= set(report)


def test_gpu_arm_fails_loudly_without_cuda():
    if torch.cuda.is_available():
        return
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0
    assert not any(ln.startswith("{") for ln in proc.stdout.splitlines())
