"""GPU tests of packed variable-length sequences (``chunk_gdn2_varlen``) and grouped value heads
(``expand_grouped_heads``): every packed sequence must give exactly what a separate call gives."""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from gdn2_sm120_b200 import chunk_gdn2
from gdn2_sm120_b200.varlen import chunk_gdn2_varlen, expand_grouped_heads

DEV = "cuda"


def _packed_case(lengths, heads, seed):
    cases = [oracle.make_inputs(1, n, heads, seed=seed + i) for i, n in enumerate(lengths)]
    packed = [torch.cat([c[j] for c in cases], dim=1) for j in range(6)]
    states = torch.cat([c[6] for c in cases], dim=0)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return cases, packed, states, cu


@pytest.mark.gpu
def test_packed_sequences_equal_separate_calls_forward_and_backward():
    lengths = [70, 5, 0, 200, 64]
    cases, packed, states, cu = _packed_case(lengths, 2, seed=900)
    gen = torch.Generator().manual_seed(1)
    d_out = (torch.randn(packed[2].shape, generator=gen) * 0.1).bfloat16().to(DEV)
    d_fin = (torch.randn(states.shape, generator=gen) * 0.01).to(DEV)

    leaves = [t.to(DEV).requires_grad_(True) for t in packed]
    s0 = states.to(DEV).requires_grad_(True)
    out, fin = chunk_gdn2_varlen(*leaves, torch.tensor(cu, dtype=torch.int32), s0, output_final_state=True)
    assert out.shape == packed[2].shape and fin.shape == states.shape
    grads = torch.autograd.grad((out.float() * d_out.float()).sum() + (fin * d_fin).sum(), (*leaves, s0))

    for i, n in enumerate(lengths):
        lo, hi = cu[i], cu[i + 1]
        if n == 0:
            assert torch.equal(fin[i], s0[i]) and torch.equal(grads[6][i], d_fin[i])
            continue
        single = [t[:, lo:hi].detach().clone().requires_grad_(True) for t in leaves]
        s_single = s0[i:i + 1].detach().clone().requires_grad_(True)
        o, f = chunk_gdn2(*single, s_single, output_final_state=True)
        gr = torch.autograd.grad((o.float() * d_out[:, lo:hi].float()).sum() + (f * d_fin[i:i + 1]).sum(),
                                 (*single, s_single))
        assert torch.equal(o, out[:, lo:hi]) and torch.equal(f, fin[i:i + 1])
        for a, b in zip(gr[:6], grads[:6]):
            assert torch.equal(a, b[:, lo:hi])
        assert torch.equal(gr[6], grads[6][i:i + 1])
    # one sequence against the oracle as well
    ref_out, ref_state = oracle.recurrence(*cases[3])
    torch.testing.assert_close(out[:, cu[3]:cu[4]].float().cpu(), ref_out.float(), rtol=2e-2, atol=1e-2)
    assert oracle.rel_l2(fin[3:4], ref_state) < 1e-3


@pytest.mark.gpu
def test_packed_inference_without_states_and_with_fused_flags():
    lengths = [33, 130]
    raws = [oracle.make_raw_inputs(1, n, 2, seed=50 + i) for i, n in enumerate(lengths)]
    packed = [torch.cat([c[j] for c in raws], dim=1).to(DEV) for j in range(6)]
    with torch.no_grad():
        out, fin = chunk_gdn2_varlen(*packed, [0, 33, 163], use_qk_l2norm_in_kernel=True,
                                     use_gate_in_kernel=True, output_final_state=True)
        for i, (lo, hi) in enumerate(((0, 33), (33, 163))):
            o, f = chunk_gdn2(*(t[:, lo:hi] for t in packed), use_qk_l2norm_in_kernel=True,
                              use_gate_in_kernel=True, output_final_state=True)
            assert torch.equal(o, out[:, lo:hi]) and torch.equal(f, fin[i:i + 1])
        assert chunk_gdn2_varlen(*packed, [0, 33, 163])[1] is None


def test_cu_seqlens_and_group_validation():
    q = torch.zeros(1, 10, 2, 128)
    with pytest.raises(ValueError, match="start at 0 and end"):
        chunk_gdn2_varlen(q, q, q, q, q, q, [0, 4, 9])
    with pytest.raises(ValueError, match="non-decreasing"):
        chunk_gdn2_varlen(q, q, q, q, q, q, [0, 7, 4, 10])
    with pytest.raises(TypeError, match="int32 or int64"):
        chunk_gdn2_varlen(q, q, q, q, q, q, torch.tensor([0.0, 10.0]))
    with pytest.raises(ValueError, match=r"\[1, total, H, 128\]"):
        chunk_gdn2_varlen(torch.zeros(2, 5, 2, 128), q, q, q, q, q, [0, 5])
    with pytest.raises(ValueError, match="multiple"):
        expand_grouped_heads(q, q, q, q, 3)
    a = torch.arange(2 * 3 * 2 * 4, dtype=torch.float32).view(2, 3, 2, 4).requires_grad_(True)
    wide = expand_grouped_heads(a, a, a, a, 6)[0]
    assert wide.shape == (2, 3, 6, 4) and wide.is_contiguous()
    assert torch.equal(wide[:, :, 0], a[:, :, 0]) and torch.equal(wide[:, :, 2], a[:, :, 0])
    assert torch.equal(wide[:, :, 3], a[:, :, 1])
    (grad,) = torch.autograd.grad(wide.sum(), a)
    assert torch.equal(grad, torch.full_like(a, 3.0))
