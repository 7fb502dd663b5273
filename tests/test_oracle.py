"""CPU tests of the oracle: pinned to the reference-generated golden vectors, plus the
self-consistency identities the reference checks (tests/test_reference.py:11-113 there)."""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from conftest import load_golden

GOLDEN_CASES = [
    "config0_b1_t64_h2",
    "decode_b1_t5_h2_bf16",
    "decode_b1_t5_h2_fp16_lowg",
    "decode_b2_t1_h3_zero",
    "short_b2_t19_h3",
    "chunk_b1_t129_h2_nostate",
]


def _inputs(rec):
    return (rec["q"], rec["k"], rec["v"], rec["g"], rec["beta"], rec["w"], rec.get("initial_state"))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_fp32_oracle_reproduces_reference_forward_bit_exactly(name):
    """Same op order in float32 => identical bits to reference.py:47-99."""

    torch.set_num_threads(1)
    rec = load_golden(name)
    q, k, v, g, beta, w, s0 = _inputs(rec)
    o, s = oracle.recurrence(q, k, v, g, beta, w, s0, scale=rec["scale"], dtype=torch.float32)
    assert torch.equal(o.to(rec["dtype"]).view(torch.int16), rec["out"].view(torch.int16))
    torch.testing.assert_close(s, rec["final_state"], rtol=0, atol=0)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_fp64_oracle_agrees_with_reference_within_fp32_rounding(name):
    rec = load_golden(name)
    q, k, v, g, beta, w, s0 = _inputs(rec)
    o, s = oracle.recurrence(q, k, v, g, beta, w, s0, scale=rec["scale"])
    assert oracle.rel_l2(s, rec["final_state"]) < 2e-6
    torch.testing.assert_close(o.to(rec["dtype"]).float(), rec["out"].float(), rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_chunkwise_restatement_matches_reference_chunk16(name):
    rec = load_golden(name)
    q, k, v, g, beta, w, s0 = _inputs(rec)
    o, s = oracle.chunkwise(q, k, v, g, beta, w, s0, scale=rec["scale"], chunk_size=16)
    assert oracle.rel_l2(s, rec["final_state_chunk16"]) < 5e-6
    assert oracle.rel_l2(o, rec["out_chunk16"].double()) < 6e-3  # reference output is 16-bit


@pytest.mark.parametrize("name", [n for n in GOLDEN_CASES if n != "decode_b1_t5_h2_fp16_lowg"])
def test_gradients_match_reference_autograd(name):
    """Reference gradients are fp32 autograd results rounded to the leaf dtypes."""

    rec = load_golden(name)
    q, k, v, g, beta, w, s0 = _inputs(rec)
    o, s = oracle.recurrence(q, k, v, g, beta, w, s0, scale=rec["scale"])
    # the reference loss squares the *rounded* output and autograd carries the cotangent
    # back through the cast in the 16-bit type: d/do = round(2*round(o)/n)
    o_rounded = o.to(rec["dtype"]).float()
    d_out = (2.0 * o_rounded / o.numel()).to(rec["dtype"]).double()
    d_state = 2.0 * s / s.numel()
    grads = oracle.token_vjp(q, k, v, g, beta, w, s0, d_out, d_state, scale=rec["scale"])
    for label, grad in zip(("dq", "dk", "dv", "dg", "dbeta", "dw"), grads):
        tol = 6e-3 if rec[label].dtype != torch.float32 else 2e-5
        assert oracle.rel_l2(grad, rec[label].double()) < tol, label
    if s0 is not None:
        assert oracle.rel_l2(grads[6], rec["dS0"]) < 2e-5


@pytest.mark.parametrize("time", [1, 3, 4, 5, 9])
@pytest.mark.parametrize("chunk", [1, 2, 4])
def test_chunkwise_equals_recurrence_small_dims(time, chunk):
    gen = torch.Generator().manual_seed(17)
    shape_k, shape_v = (2, time, 3, 4), (2, time, 3, 5)
    q, k, beta = (torch.randn(shape_k, generator=gen, dtype=torch.float64) for _ in range(3))
    v, w = (torch.randn(shape_v, generator=gen, dtype=torch.float64) for _ in range(2))
    g = -torch.rand(shape_k, generator=gen, dtype=torch.float64)
    s0 = torch.randn((2, 3, 4, 5), generator=gen, dtype=torch.float64)
    o_r, s_r = oracle.recurrence(q, k, v, g, beta, w, s0)
    o_c, s_c = oracle.chunkwise(q, k, v, g, beta, w, s0, chunk_size=chunk)
    torch.testing.assert_close(o_c, o_r, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(s_c, s_r, rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("with_state", [True, False])
@pytest.mark.parametrize("with_final_grad", [True, False])
def test_token_vjp_equals_autograd(with_state, with_final_grad):
    gen = torch.Generator().manual_seed(23)
    shape_k, shape_v = (2, 5, 2, 7), (2, 5, 2, 5)
    q, k, beta = (torch.randn(shape_k, generator=gen, dtype=torch.float64) for _ in range(3))
    v, w = (torch.randn(shape_v, generator=gen, dtype=torch.float64) for _ in range(2))
    g = -torch.rand(shape_k, generator=gen, dtype=torch.float64)
    s0 = torch.randn((2, 2, 7, 5), generator=gen, dtype=torch.float64) if with_state else None
    d_out = torch.randn(shape_v, generator=gen, dtype=torch.float64)
    d_fin = torch.randn((2, 2, 7, 5), generator=gen, dtype=torch.float64) if with_final_grad else None
    _, _, auto = oracle.recurrence_grads(q, k, v, g, beta, w, s0, d_out, d_fin)
    manual = oracle.token_vjp(q, k, v, g, beta, w, s0, d_out, d_fin)
    for a, m in zip(auto, manual):
        if a is None:
            assert m is None
        else:
            torch.testing.assert_close(m, a, rtol=1e-10, atol=1e-12)


def test_zero_key_known_answer():
    """k = 0 => o = 0 and S_T = S_0 * exp(sum g) (reference tests/test_reference.py:11-24)."""

    gen = torch.Generator().manual_seed(3)
    shape = (1, 6, 2, 4)
    q, v, beta, w = (torch.randn(shape, generator=gen, dtype=torch.float64) for _ in range(4))
    k = torch.zeros(shape, dtype=torch.float64)
    g = -torch.rand(shape, generator=gen, dtype=torch.float64)
    s0 = torch.randn((1, 2, 4, 4), generator=gen, dtype=torch.float64)
    o, s = oracle.recurrence(q, k, v, g, beta, w, s0)
    expected = s0 * g.sum(dim=1).exp().unsqueeze(-1)
    torch.testing.assert_close(s, expected, rtol=1e-12, atol=1e-12)
    # with k == 0 nothing is written, the output only reads the decayed initial state
    decayed = s0.clone()
    for t in range(6):
        decayed = g[:, t].exp().unsqueeze(-1) * decayed
        ref = torch.einsum("bhk,bhkv->bhv", q[:, t] * 0.5, decayed)
        torch.testing.assert_close(o[:, t], ref, rtol=1e-12, atol=1e-12)


def test_t1_zero_state_closed_form():
    q, k, v, g, beta, w, _ = oracle.make_inputs(2, 1, 3, seed=611, with_state=False)
    o, s = oracle.recurrence(q, k, v, g, beta, w, None, scale=0.0625)
    o_cf, s_cf = oracle.t1_zero_closed_form(q, k, v, w, scale=0.0625)
    torch.testing.assert_close(o_cf, o, rtol=1e-12, atol=1e-14)
    torch.testing.assert_close(s_cf, s, rtol=1e-12, atol=1e-14)


def test_empty_sequence():
    q, k, v, g, beta, w, s0 = oracle.make_inputs(1, 0, 2)
    o, s = oracle.recurrence(q, k, v, g, beta, w, s0)
    assert o.shape == (1, 0, 2, 128)
    torch.testing.assert_close(s, s0.double(), rtol=0, atol=0)


def test_input_distribution_respects_decay_contract():
    *_, g, _, _, _ = oracle.make_inputs(1, 256, 2, seed=0)[:4] + (None, None, None)
    g = oracle.make_inputs(1, 256, 2, seed=0)[3]
    assert g.max() <= 0 and g.min() >= -5.0
    windows = g.unfold(1, 16, 16).sum(-1)
    assert windows.min() > -87.0


@pytest.mark.parametrize("chunk,kdim,vdim", [(4, 7, 5), (7, 7, 5), (16, 8, 8)])
def test_chunk_wy_stage_oracle_matches_recurrence_and_autograd(chunk, kdim, vdim):
    """Compact-WY chunk form and its hand-derived VJP against the token recurrence and
    torch.autograd in float64 (same role as the reference's tests/test_backward_wy.py:257-317)."""

    gen = torch.Generator().manual_seed(91 + chunk)
    dt = torch.float64
    q, k, beta = (torch.randn(chunk, kdim, generator=gen, dtype=dt) for _ in range(3))
    v, w = (torch.randn(chunk, vdim, generator=gen, dtype=dt) for _ in range(2))
    g = -torch.rand(chunk, kdim, generator=gen, dtype=dt)
    s0 = torch.randn(kdim, vdim, generator=gen, dtype=dt)
    d_o = torch.randn(chunk, vdim, generator=gen, dtype=dt)
    d_s1 = torch.randn(kdim, vdim, generator=gen, dtype=dt)
    scale = 0.37

    def batched(x):
        return x[None, :, None]

    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta, w, s0)]
    o, s1 = oracle.recurrence(*[batched(t) for t in leaves[:6]], leaves[6][None, None], scale=scale)
    fwd = oracle.chunk_wy_forward(q, k, v, g, beta, w, s0, scale=scale)
    torch.testing.assert_close(fwd["o"], o[0, :, 0].detach(), rtol=1e-10, atol=1e-12)
    torch.testing.assert_close(fwd["s1"], s1[0, 0].detach(), rtol=1e-10, atol=1e-12)
    want = torch.autograd.grad((o[0, :, 0] * d_o).sum() + (s1[0, 0] * d_s1).sum(), leaves)
    got = oracle.chunk_wy_vjp(q, k, v, g, beta, w, s0, d_o, d_s1, scale=scale)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-11)


# ---- the package's public reference functions (same two names the reference exports) --------
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_public_reference_functions_reproduce_the_reference(name):
    """``gdn2_sm120_b200.recurrent_forward_reference`` in its default float32 mode gives the bits
    the reference's reference.py:47-99 gave; the chunkwise form agrees with reference.py:102-179."""

    from gdn2_sm120_b200 import chunkwise_forward_reference, recurrent_forward_reference

    torch.set_num_threads(1)
    rec = load_golden(name)
    q, k, v, g, beta, w, s0 = _inputs(rec)
    out, state = recurrent_forward_reference(q, k, v, g, beta, w, s0, scale=rec["scale"])
    assert out.dtype == rec["dtype"] and state.dtype == torch.float32
    assert torch.equal(out.view(torch.int16), rec["out"].view(torch.int16))
    torch.testing.assert_close(state, rec["final_state"], rtol=0, atol=0)
    out_c, state_c = chunkwise_forward_reference(q, k, v, g, beta, w, s0, scale=rec["scale"], chunk_size=16)
    assert oracle.rel_l2(state_c, rec["final_state_chunk16"]) < 5e-6
    assert oracle.rel_l2(out_c.double(), rec["out_chunk16"].double()) < 6e-3


# ---- stage-level oracles pinned to the reference's executable proofs ---------------------------
def _stage_record():
    rec = load_golden("stage_chunk64")
    seq = tuple(rec[n][0, :, 0] for n in ("q", "k", "v", "g", "beta", "w"))
    return rec, seq, rec["initial_state"][0, 0], rec["d_out"][0, :, 0], rec["d_s1"][0, 0]


def test_stage_oracle_boundary_step_matches_reference_proof():
    """dR = A^T dO + Kt dS1 and dS0 of one 64-token chunk against
    boundary_dstate_wy_reference (backward_parallel.py:315-373 of the reference)."""

    rec, seq, s0, d_o, d_s1 = _stage_record()
    f = oracle.chunk_wy_forward(*seq, s0, scale=rec["scale"])
    d_r = f["A"].T @ d_o.double() + f["Kt"] @ d_s1.double()
    d_s0 = f["d"][:, None] * d_s1.double() + f["Qg"].T @ d_o.double() - f["Y"].T @ d_r
    assert oracle.rel_l2(d_r, rec["d_residual"][0, :, 0]) < 2e-5
    assert oracle.rel_l2(d_s0, rec["d_s0"][0, 0]) < 2e-5
    assert oracle.rel_l2(f["s1"], rec["final_state"][0, 0]) < 2e-5


def test_stage_oracle_chunk_vjp_matches_reference_proof():
    """All six sequence gradients of one 64-token chunk against
    compact_wy_chunk_vjp_reference (backward_wy.py:62-223 of the reference)."""

    rec, seq, s0, d_o, d_s1 = _stage_record()
    grads = oracle.chunk_wy_vjp(*seq, s0, d_o, d_s1, scale=rec["scale"])
    for name, got in zip(("dq", "dk", "dv", "dg", "dbeta", "dw"), grads[:6]):
        assert oracle.rel_l2(got, rec["stage_" + name][0, :, 0]) < 2e-5, name
    assert oracle.rel_l2(grads[6], rec["d_s0"][0, 0]) < 2e-5


# ---- layer prologue (normalisation + gate activations) -------------------------------------------
def test_prologue_oracle_vjp_matches_autograd():
    torch.manual_seed(3)
    raw = [torch.randn(2, 5, 3, 16, dtype=torch.float64, requires_grad=True) for _ in range(5)]
    outs = oracle.gate_prologue(*raw)
    cots = [torch.randn_like(o) for o in outs]
    want = torch.autograd.grad(outs, raw, cots)
    got = oracle.gate_prologue_vjp(*[r.detach() for r in raw], *cots)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, rtol=1e-10, atol=1e-12)
    # activated values follow the primitive's contract: unit-norm q/k, gates in (0, 1), g <= 0
    q, k, g, beta, w = (o.detach() for o in outs)
    torch.testing.assert_close(q.norm(dim=-1), torch.ones_like(q[..., 0]), rtol=1e-5, atol=1e-5)
    assert (g <= 0).all() and ((beta > 0) & (beta < 1)).all() and ((w > 0) & (w < 1)).all()
