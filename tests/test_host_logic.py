"""CPU tests of the host side: dispatch tables, argument validation, overlap arithmetic,
autograd plumbing (with the kernels mocked out) and the C-ABI library's exports.
No kernel runs here.  Mirrors the CPU half of the reference's tests/test_ops.py,
tests/test_recurrent.py and tests/test_chunk.py."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest
import torch

import gdn2_sm120_b200 as pkg
from gdn2_sm120_b200 import _lib, _validate, chunk as chunk_module, ops as ops_module
from gdn2_sm120_b200 import recurrent as recurrent_module

ROOT = pathlib.Path(__file__).resolve().parent.parent


# ---- public surface -----------------------------------------------------------------
def test_public_names_match_reference_all():
    assert set(pkg.__all__) == {
        "chunk_backward", "chunk_forward", "chunk_gdn2", "chunkwise_forward_reference",
        "recurrent_forward_reference", "recurrent_gdn2", "token_forward", "MAX_BACKWARD_TOKENS",
    }
    assert pkg.MAX_BACKWARD_TOKENS == 128


# ---- dispatch -------------------------------------------------------------------------
@pytest.mark.parametrize(
    ("batch", "time", "heads", "chunk_api", "expected"),
    [
        (1, 1, 16, False, True), (1, 32, 16, False, True), (1, 48, 16, False, True),
        (4, 63, 16, False, True), (1, 64, 16, False, False), (1, 40, 16, True, True),
        (1, 48, 16, True, True), (1, 63, 1, True, True), (1, 64, 16, True, False),
        (4, 8192, 32, True, False), (64, 1, 32, False, True),
    ],
)
def test_forward_kernel_crossover_dispatch(batch, time, heads, chunk_api, expected):
    assert ops_module._use_recurrent_kernel(batch, time, heads, chunk_api=chunk_api) is expected


@pytest.mark.parametrize(
    ("batch", "time", "heads", "expected"),
    [(1, 63, 64, False), (1, 64, 1, True), (2, 64, 8, True), (1, 127, 16, True), (1, 128, 1, True),
     (4, 8200, 32, True), (1, 1, 1, False)],
)
def test_compact_wy_backward_dispatch(batch, time, heads, expected):
    assert ops_module._use_compact_wy_backward(batch, time, heads) is expected


# ---- overlap / stride / scale helpers -------------------------------------------------
def test_empty_byte_span_does_not_overlap():
    assert not recurrent_module._spans_overlap((128, 128), (0, 256))
    assert not recurrent_module._spans_overlap((0, 256), (128, 128))
    assert recurrent_module._spans_overlap((0, 256), (255, 300))
    assert not recurrent_module._spans_overlap((0, 256), (256, 300))


def test_scale_validation():
    assert _validate.float32_scale(None) == pytest.approx(128 ** -0.5, rel=1e-7)
    assert _validate.float32_scale(-0.0) == 0.0
    with pytest.raises(ValueError, match="scale must be finite"):
        _validate.float32_scale(float("nan"))
    with pytest.raises(ValueError, match="representable as float32"):
        _validate.float32_scale(1e100)


# ---- validation happens before any device work ------------------------------------------
def _cpu_inputs(shape=(1, 4, 2, 128), dtype=torch.bfloat16):
    seq = [torch.zeros(shape, dtype=dtype) for _ in range(6)]
    seq[3] = torch.zeros(shape, dtype=torch.float32)
    return seq


def test_rejections_in_reference_order():
    q, k, v, g, beta, w = _cpu_inputs()
    with pytest.raises(TypeError, match="torch.Tensor"):
        pkg.token_forward(q, k, v, g, beta, None)
    with pytest.raises(ValueError, match="rank-4"):
        pkg.token_forward(q[0], k, v, g, beta, w)
    with pytest.raises(ValueError, match="identical"):
        pkg.token_forward(q[:, :2], k, v, g, beta, w)
    with pytest.raises(ValueError, match="K == V == 128"):
        pkg.token_forward(*_cpu_inputs((1, 4, 2, 64)))
    with pytest.raises(NotImplementedError, match="K == V == 128"):
        pkg.chunk_forward(*_cpu_inputs((1, 4, 2, 64)))
    with pytest.raises(ValueError, match="batch and heads must be positive"):
        pkg.token_forward(*_cpu_inputs((0, 4, 2, 128)))
    with pytest.raises(ValueError, match="must be positive"):
        pkg.chunk_forward(*_cpu_inputs((1, 0, 2, 128)))
    with pytest.raises(TypeError, match="float16 or torch.bfloat16"):
        pkg.token_forward(*[t.float() for t in _cpu_inputs()])
    with pytest.raises(TypeError, match="same dtype"):
        pkg.token_forward(q, k.half(), v, g, beta, w)
    with pytest.raises(TypeError, match="g must have"):
        pkg.token_forward(q, k, v, g.half(), beta, w)
    with pytest.raises(ValueError, match="CUDA tensors"):
        pkg.token_forward(q, k, v, g, beta, w)
    with pytest.raises(ValueError, match="CUDA tensors"):
        pkg.chunk_backward(q, k, v, g, beta, w, torch.zeros(1, 2, 128, 128), v, torch.zeros(1, 2, 128, 128))


def test_chunk_gdn2_rejects_non_finite_scale_first():
    with pytest.raises(ValueError, match="scale must be finite"):
        pkg.chunk_gdn2(*_cpu_inputs(), scale=float("inf"))


# ---- autograd plumbing with the kernels replaced by fakes ---------------------------------
def test_inference_bypasses_autograd_function(monkeypatch):
    calls = []

    def fake_token_forward(q, k, v, g, beta, w, state=None, scale=None, **_):
        calls.append(("token", q.requires_grad))
        return v.clone(), torch.zeros(q.shape[0], q.shape[2], 128, 128)

    def fake_chunk_forward(q, k, v, g, beta, w, state=None, *, scale=None, return_aux=False, **_):
        calls.append(("chunk", return_aux))
        return v.clone(), torch.zeros(q.shape[0], q.shape[2], 128, 128)

    def boom(*args, **kwargs):
        raise AssertionError("autograd.Function must not be entered for inference")

    monkeypatch.setattr(ops_module, "token_forward", fake_token_forward)
    monkeypatch.setattr(ops_module, "chunk_forward", fake_chunk_forward)
    monkeypatch.setattr(ops_module._ChunkGDN2, "apply", staticmethod(boom))

    short = _cpu_inputs((1, 8, 1, 128))
    long = _cpu_inputs((1, 128, 1, 128))
    out, state = pkg.chunk_gdn2(*short)
    assert state is None and out.shape == short[2].shape
    _, state = pkg.chunk_gdn2(*long, output_final_state=True)
    assert state is not None
    with torch.no_grad():
        pkg.chunk_gdn2(*[t.requires_grad_(t.is_floating_point()) for t in _cpu_inputs((1, 128, 1, 128))])
    with torch.inference_mode():
        pkg.chunk_gdn2(*_cpu_inputs((1, 128, 1, 128)))
    assert calls == [("token", False), ("chunk", False), ("chunk", False), ("chunk", False)]


def test_training_enters_function_once_per_call(monkeypatch):
    seen = []

    def fake_apply(q, k, v, g, beta, w, state, scale, prepare_backward):
        seen.append((q.shape[0], prepare_backward, scale))
        return v.clone(), torch.zeros(q.shape[0], q.shape[2], 128, 128)

    monkeypatch.setattr(ops_module._ChunkGDN2, "apply", staticmethod(fake_apply))
    seq = torch.zeros((3, 128, 1, 128), dtype=torch.bfloat16, requires_grad=True)
    out, state = pkg.chunk_gdn2(*([seq] * 6), output_final_state=True)
    assert out.shape == seq.shape and state.shape == (3, 1, 128, 128)
    assert seen == [(3, True, pytest.approx(128 ** -0.5))]
    # a state that requires grad is enough to need the backward edge
    seq2 = torch.zeros((1, 4, 1, 128), dtype=torch.bfloat16)
    s0 = torch.zeros((1, 1, 128, 128), requires_grad=True)
    pkg.chunk_gdn2(*([seq2] * 6), s0)
    assert len(seen) == 2


def test_hidden_final_state_reaches_backward_as_none(monkeypatch):
    """When the loss ignores S_T no zero cotangent may be materialised
    (reference: src/gdn2_sm120/ops.py:136-148, tests/test_ops.py:167-215)."""

    captured = {}

    def fake_sequence_inputs(q, *rest, **kwargs):
        return q.shape[0], q.shape[1], q.shape[2]

    def fake_launch(q, k, v, g, beta, w, state, output, final_state, boundaries, *rest):
        output.zero_()
        final_state.zero_()

    def fake_backward(q, k, v, g, beta, w, aux, d_out, d_final_state, scale):
        captured["d_final_state"] = d_final_state
        captured["aux"] = aux
        return (*[torch.zeros_like(x) for x in (q, k, v, g, beta, w)],
                torch.zeros(q.shape[0], q.shape[2], 128, 128))

    monkeypatch.setattr(_validate, "sequence_inputs", fake_sequence_inputs)
    monkeypatch.setattr(ops_module, "_launch_token_forward", fake_launch)
    monkeypatch.setattr(ops_module, "backward_from_aux", fake_backward)
    seq = [torch.zeros((1, 8, 1, 128), dtype=torch.bfloat16, requires_grad=True) for _ in range(6)]
    out, state = pkg.chunk_gdn2(*seq, output_final_state=False)
    assert state is None
    grads = torch.autograd.grad(out.float().sum(), seq)
    assert captured["d_final_state"] is None
    assert captured["aux"].full_tokens == 0 and captured["aux"].tail_boundaries.shape == (1, 2, 1, 128, 128)
    assert all(g.shape == s.shape for g, s in zip(grads, seq))


def test_token_slot_arithmetic():
    assert chunk_module._token_slots(1) == 2
    assert chunk_module._token_slots(16) == 2
    assert chunk_module._token_slots(17) == 3
    assert chunk_module._token_slots(63) == 5


# ---- the C-ABI library ----------------------------------------------------------------------
def test_library_loads_and_exports_every_declared_symbol():
    header = (ROOT / "include" / "gdn2_b200.h").read_text()
    declared = set(re.findall(r"\b(gdn2_[a-z0-9_]+)\s*\(", header))
    declared -= {"gdn2_status", "gdn2_dtype"}
    handle = _lib.lib()
    assert declared, "no declarations parsed from the header"
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.exported_symbols())
    assert handle.gdn2_version() >= 100
    assert handle.gdn2_status_string(0) == b"ok"
    assert b"NULL" in handle.gdn2_status_string(-1)


def test_entry_points_reject_bad_arguments_without_a_gpu():
    """Host-side validation of the C ABI returns before any CUDA call."""

    handle = _lib.lib()
    null = None
    assert handle.gdn2_token_forward(null, null, null, null, null, null, null, null, null, null,
                                     1, 1, 1, 0, 1, 0, 2, 1.0, null) == -1
    one = ctypes.c_void_p(16)
    args = [one] * 6 + [null, one, null, null]
    assert handle.gdn2_token_forward(*args, 0, 1, 1, 0, 1, 0, 2, 1.0, null) == -2
    assert handle.gdn2_token_forward(*args, 1, 4, 1, 2, 1, 0, 2, 1.0, null) == -4
    assert handle.gdn2_token_forward(*args, 1, 4, 1, 0, 5, 0, 2, 1.0, null) == -4
    assert handle.gdn2_token_forward(*args, 1, 4, 1, 0, 4, 2, 2, 1.0, null) == -3
    assert handle.gdn2_token_forward(*args, 1, 4, 1, 0, 4, 0, 1, 1.0, null) == -3
    bad_state = [one] * 6 + [ctypes.c_void_p(18), one, null, null]
    assert handle.gdn2_token_forward(*bad_state, 1, 4, 1, 0, 4, 0, 2, 1.0, null) == -5


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_handle", None)
    monkeypatch.setenv("GDN2_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_wave_plan_sizes_training_waves_for_the_backward_transients():
    """The workspace of a wave is what backward consumes, so backward runs over the forward's waves: a
    training plan must keep the backward scratch of a wave (dZ tiles + cotangent checkpoints) inside the
    budget, not only the smaller forward scratch.  B=32, T=16384, H=32 is the one-GPU point of the
    8-GPU configuration."""

    from gdn2_sm120_b200 import chunk_kernels

    batch, tokens, heads = 32, 16384, 32
    waves = chunk_kernels.plan_waves(batch, tokens, heads, training=True)
    assert waves[0][0] == 0 and waves[-1][1] == batch
    assert all(a[1] == b[0] for a, b in zip(waves, waves[1:]))
    rows = max(b1 - b0 for b0, b1 in waves)
    assert chunk_kernels._backward_wave_bytes(rows, tokens, heads) <= chunk_kernels.SCRATCH_BUDGET_BYTES
    assert len(waves) >= 3
    # scratch sizes by kind: a training forward keeps the tiles both scans read in its workspace
    units = batch * (tokens // 64) * heads
    assert chunk_kernels.scratch_bytes(batch, tokens, heads, False) == units * 144 * 1024
    assert chunk_kernels.scratch_bytes(batch, tokens, heads, False, training=True) == units * 32 * 1024
    assert chunk_kernels.scratch_bytes(batch, tokens, heads, True) == units * 36 * 1024
    assert chunk_kernels.workspace_bytes(batch, tokens, heads, True) == units * (160 * 1024 + 512) + 256
    # an inference plan is sized by its own scratch alone
    assert len(chunk_kernels.plan_waves(batch, tokens, heads)) == 4
