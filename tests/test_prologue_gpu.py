"""GPU tests of the fused layer prologue (q/k L2 normalisation + gate activations) and of the
``use_qk_l2norm_in_kernel`` / ``use_gate_in_kernel`` keywords of the public operators.

Ground truth: the oracle's float64 prologue composed with its float64 recurrence.  The kernels hand
16-bit activated tensors to the primitive, so the comparison is made the way a caller of the unfused
API would see it: activations evaluated exactly, rounded to the sequence dtype, fed to the recurrence;
cotangents of those rounded tensors pulled back through the exact Jacobian of the activations."""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from gdn2_sm120_b200 import chunk_gdn2, recurrent_gdn2
from gdn2_sm120_b200.prologue import gate_prologue

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(cpu, d_out, d_fin, normalize_qk, activate_gates, scale=None):
    q, k, v, g, beta, w, s0 = cpu
    act = oracle.gate_prologue(q, k, g, beta, w, normalize_qk=normalize_qk, activate_gates=activate_gates)
    qa, ka, ga, ba, wa = (a.to(t.dtype) for a, t in zip(act, (q, k, g, beta, w)))   # what the primitive sees
    if d_out is None and d_fin is None:
        out, fin = oracle.recurrence(qa, ka, v, ga, ba, wa, s0, scale=scale)
        return (qa, ka, ga, ba, wa), out, fin, None
    out, fin, grads = oracle.recurrence_grads(qa, ka, v, ga, ba, wa, s0, d_out, d_fin, scale=scale)
    dq, dk, dv, dg, dbeta, dw, ds0 = grads
    dq, dk, dg, dbeta, dw = oracle.gate_prologue_vjp(q, k, g, beta, w, dq, dk, dg, dbeta, dw,
                                                     normalize_qk=normalize_qk, activate_gates=activate_gates)
    return (qa, ka, ga, ba, wa), out, fin, (dq, dk, dv, dg, dbeta, dw, ds0)


@pytest.mark.parametrize("dtype,g_dtype", [(torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
def test_prologue_kernel_matches_exact_activations(dtype, g_dtype):
    q, k, v, g, beta, w, _ = oracle.make_raw_inputs(2, 37, 3, seed=5, dtype=dtype, g_dtype=g_dtype)
    want = oracle.gate_prologue(q, k, g, beta, w)
    got = gate_prologue(*(t.to(DEV) for t in (q, k, g, beta, w)))
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    tiny = 0.0 if dtype == torch.bfloat16 else 2.0 ** -24   # spacing of fp16 subnormals (|x| < 6.1e-5)
    for name, a, b, raw in zip(("q", "k", "g", "beta", "w"), got, want, (q, k, g, beta, w)):
        assert a.dtype == raw.dtype and a.shape == raw.shape
        # fp32 arithmetic rounded once to the tensor's dtype: within one unit in the last place
        err = (a.double().cpu() - b).abs()
        assert (err <= ulp * b.abs() + tiny + 1e-30).all(), name
    # either group can be switched off and then leaves its tensors alone
    dq, dk, dg, dbeta, dw = (t.to(DEV) for t in (q, k, g, beta, w))
    only_norm = gate_prologue(dq, dk, dg, dbeta, dw, activate_gates=False)
    assert only_norm[2] is dg and only_norm[3] is dbeta and torch.equal(only_norm[0], got[0])
    only_gate = gate_prologue(dq, dk, dg, dbeta, dw, normalize_qk=False)
    assert only_gate[0] is dq and torch.equal(only_gate[3], got[3]) and torch.equal(only_gate[2], got[2])


@pytest.mark.parametrize("time", [19, 200])
@pytest.mark.parametrize("normalize_qk,activate_gates", [(True, True), (True, False), (False, True)])
def test_fused_flags_forward_and_backward_against_oracle(time, normalize_qk, activate_gates):
    raw = oracle.make_raw_inputs(1, time, 2, seed=40 + time)
    cpu = list(raw)
    if not normalize_qk:   # un-normalised keys would leave the operating range of the primitive
        act = oracle.gate_prologue(*[cpu[i] for i in (0, 1, 3, 4, 5)], activate_gates=False)
        cpu[0], cpu[1] = act[0].to(torch.bfloat16), act[1].to(torch.bfloat16)
    if not activate_gates:
        act = oracle.gate_prologue(*[cpu[i] for i in (0, 1, 3, 4, 5)], normalize_qk=False)
        cpu[3], cpu[4], cpu[5] = act[2].float(), act[3].to(torch.bfloat16), act[4].to(torch.bfloat16)
    gen = torch.Generator().manual_seed(7)
    d_out = (torch.randn(cpu[2].shape, generator=gen) * 0.1).bfloat16()
    d_fin = torch.randn(cpu[6].shape, generator=gen) * 0.01
    _, ref_out, ref_fin, ref_grads = _reference(cpu, d_out, d_fin, normalize_qk, activate_gates)

    leaves = [t.to(DEV).requires_grad_(True) for t in cpu]
    out, fin = chunk_gdn2(*leaves[:6], leaves[6], output_final_state=True,
                          use_qk_l2norm_in_kernel=normalize_qk, use_gate_in_kernel=activate_gates)
    grads = torch.autograd.grad((out.float() * d_out.to(DEV).float()).sum() + (fin * d_fin.to(DEV)).sum(), leaves)
    torch.testing.assert_close(out.float().cpu(), ref_out.float(), rtol=2e-2, atol=1e-2)
    # the kernel's fp32 activations may round differently from the exact ones in the last bit of a few
    # elements, hence twice the usual fp32 tolerance on the state and the fp32 gradients
    assert oracle.rel_l2(fin, ref_fin) < 2e-3
    for name, got, want in zip(("dq", "dk", "dv", "dg", "dbeta", "dw", "dS0"), grads, ref_grads):
        limit = 2e-3 if got.dtype == torch.float32 else 5e-3
        err = oracle.rel_l2(got, want)
        assert err < limit, f"{name}: {err:.3e}"


def _exact_reference(cpu, normalize_qk, activate_gates, scale=None):
    """Recurrence on the exactly activated (un-rounded, float64) tensors: what the in-kernel prologue of
    the forward kernels approximates in fp32."""

    q, k, v, g, beta, w, s0 = cpu
    qa, ka, ga, ba, wa = oracle.gate_prologue(q, k, g, beta, w, normalize_qk=normalize_qk,
                                              activate_gates=activate_gates)
    return oracle.recurrence(qa, ka, v.double(), ga, ba, wa, None if s0 is None else s0.double(), scale=scale)


@pytest.mark.parametrize("time", [1, 19, 64, 200])
@pytest.mark.parametrize("normalize_qk,activate_gates", [(True, True), (True, False), (False, True)])
def test_inference_applies_the_prologue_inside_the_forward_kernels(time, normalize_qk, activate_gates):
    """Without gradients no activated tensor is materialised: the prep kernel (full chunks), the token
    kernel (short sequences and the ragged tail) apply the flags as they load the raw inputs."""

    raw = list(oracle.make_raw_inputs(2, time, 3, seed=300 + time))
    if not normalize_qk:
        act = oracle.gate_prologue(*[raw[i] for i in (0, 1, 3, 4, 5)], activate_gates=False)
        raw[0], raw[1] = act[0].to(torch.bfloat16), act[1].to(torch.bfloat16)
    if not activate_gates:
        act = oracle.gate_prologue(*[raw[i] for i in (0, 1, 3, 4, 5)], normalize_qk=False)
        raw[3], raw[4], raw[5] = act[2].float(), act[3].to(torch.bfloat16), act[4].to(torch.bfloat16)
    ref_out, ref_fin = _exact_reference(raw, normalize_qk, activate_gates)
    args = [t.to(DEV) for t in raw]
    from gdn2_sm120_b200 import _lib
    _lib.KERNEL_EVENTS = {}
    try:
        with torch.no_grad():
            out, fin = chunk_gdn2(*args[:6], args[6], output_final_state=True,
                                  use_qk_l2norm_in_kernel=normalize_qk, use_gate_in_kernel=activate_gates)
        called = set(_lib.KERNEL_EVENTS)
    finally:
        _lib.KERNEL_EVENTS = None
    assert "gdn2_gate_prologue" not in called and any(name.endswith("_fused") for name in called)
    torch.testing.assert_close(out.float().cpu(), ref_out.float(), rtol=2e-2, atol=1e-2)
    assert oracle.rel_l2(fin, ref_fin) < (1e-3 if time >= 64 else 1e-5)


@pytest.mark.parametrize("with_state", [True, False])
def test_decode_kernels_apply_the_prologue(with_state):
    """T = 1 with 288 heads: the persistent decode kernel (with a state) and the closed form (without)."""

    raw = list(oracle.make_raw_inputs(9, 1, 32, seed=91))
    if not with_state:
        raw[6] = None
    ref_out, ref_fin = _exact_reference(raw, True, True, scale=0.2)
    args = [None if t is None else t.to(DEV) for t in raw]
    out, fin = recurrent_gdn2(*args[:6], args[6], scale=0.2, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True)
    torch.testing.assert_close(out.float().cpu(), ref_out.float(), rtol=2e-3, atol=2e-3)
    assert oracle.rel_l2(fin, ref_fin) < 1e-5
    # the flags off: bit-identical to the plain entry points (the fused kernels are the same kernels)
    plain = [t.to(DEV) for t in oracle.make_inputs(9, 1, 32, seed=92)]
    a = recurrent_gdn2(*plain[:6], plain[6] if with_state else None)
    from gdn2_sm120_b200.recurrent import token_forward
    b = token_forward(*plain[:6], plain[6] if with_state else None, prologue=0)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_recurrent_api_accepts_the_flags():
    cpu = oracle.make_raw_inputs(2, 1, 3, seed=77)
    ref_out, ref_fin = _exact_reference(cpu, True, True)
    args = [t.to(DEV) for t in cpu]
    out, fin = recurrent_gdn2(*args[:6], args[6], use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True)
    torch.testing.assert_close(out.float().cpu(), ref_out.to(out.dtype).float(), rtol=2e-3, atol=2e-3)
    assert oracle.rel_l2(fin, ref_fin) < 1e-5
    # the materialising route (prologue kernel, then the plain operator) agrees within the rounding of
    # the activated tensors to the sequence dtype
    qa, ka, ga, ba, wa = gate_prologue(args[0], args[1], args[3], args[4], args[5])
    out2, fin2 = recurrent_gdn2(qa, ka, args[2], ga, ba, wa, args[6])
    torch.testing.assert_close(out.float(), out2.float(), rtol=2e-2, atol=1e-2)
    assert oracle.rel_l2(fin, fin2) < 5e-3
