"""GPU parity tests of the tensor-core chunk forward (64-token chunks + token-path tail).

Tolerances: outputs |x - ref| <= 1e-2 + 2e-2 |ref| (16-bit output), final state relative L2
<= 1e-3 against the float64 recurrence on identical inputs (benchmark specification).
Shapes follow the reference's tests/test_chunk.py:111-144, 311-385 (T on both sides of every
chunk boundary, several batch/head grids, with and without initial state).
"""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from conftest import load_golden
from gdn2_sm120_b200 import chunk_forward, chunk_gdn2, chunk_kernels, recurrent_gdn2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(*tensors):
    return tuple(None if t is None else t.to(DEV) for t in tensors)


def check(out, state, ref_out, ref_state):
    torch.testing.assert_close(out.float().cpu(), ref_out.float(), rtol=2e-2, atol=1e-2)
    err = oracle.rel_l2(state, ref_state)
    assert err < 1e-3, f"final state rel-L2 {err:.3e}"


@pytest.mark.parametrize("time", [64, 65, 127, 128, 129, 192, 512, 1024])
@pytest.mark.parametrize("with_state", [True, False])
def test_chunk_forward_matches_oracle(time, with_state):
    cpu = oracle.make_inputs(2, time, 3, seed=2026 + time, with_state=with_state)
    ref_out, ref_state = oracle.recurrence(*cpu)
    out, state = chunk_gdn2(*dev(*cpu), output_final_state=True)
    check(out, state, ref_out, ref_state)


@pytest.mark.parametrize("batch,heads", [(1, 2), (2, 1), (2, 6), (1, 12), (2, 16)])
def test_chunk_forward_grids(batch, heads):
    cpu = oracle.make_inputs(batch, 256, heads, seed=31 + batch + heads)
    ref_out, ref_state = oracle.recurrence(*cpu)
    out, state = chunk_forward(*dev(*cpu))
    check(out, state, ref_out, ref_state)


def test_both_ways_of_handling_a_ragged_length_agree():
    """The C ABI takes a ragged length either way: whole chunks on the chunk kernels plus the tail on the
    token kernels (full_tokens = 64 * floor(T / 64)), or everything on the chunk kernels with a partial
    last chunk (64 * ceil(T / 64), what chunk_gdn2 does).  Same inputs, both against the oracle."""

    from gdn2_sm120_b200 import chunk_kernels
    from gdn2_sm120_b200.recurrent import _launch_token_forward

    batch, time, heads = 2, 150, 3
    cpu = oracle.make_inputs(batch, time, heads, seed=150)
    ref_out, ref_state = oracle.recurrence(*cpu)
    q, k, v, g, beta, w, s0 = dev(*cpu)
    out_pad, fin_pad = chunk_gdn2(q, k, v, g, beta, w, s0, output_final_state=True)
    check(out_pad, fin_pad, ref_out, ref_state)
    out_split, fin_split = torch.empty_like(v), torch.empty_like(s0)
    scale = 128 ** -0.5
    chunk_kernels.forward(q, k, v, g, beta, w, s0, out_split, fin_split, None, batch, time, heads, 128, scale)
    _launch_token_forward(q, k, v, g, beta, w, fin_split, out_split, fin_split, None, batch, time, heads, 128,
                          time, scale)
    check(out_split, fin_split, ref_out, ref_state)
    # the first two chunks are the same computation either way
    assert torch.equal(out_split[:, :128], out_pad[:, :128])


def test_a_sequence_shorter_than_one_chunk_runs_as_one_partial_chunk():
    """The Python API sends fewer than 64 tokens to the token kernels, but the C ABI takes them as one
    partial chunk too (full_tokens = 64 > T): 40 real tokens, 24 identity steps."""

    from gdn2_sm120_b200 import chunk_kernels

    batch, time, heads = 2, 40, 2
    cpu = oracle.make_inputs(batch, time, heads, seed=40)
    ref_out, ref_state = oracle.recurrence(*cpu)
    q, k, v, g, beta, w, s0 = dev(*cpu)
    out, fin = torch.empty_like(v), torch.empty_like(s0)
    chunk_kernels.forward(q, k, v, g, beta, w, s0, out, fin, None, batch, time, heads, 64, 128 ** -0.5)
    check(out, fin, ref_out, ref_state)


def test_chunk_forward_more_units_than_sms():
    """An inference call whose units (batch x chunks x heads = 256) outnumber the SMs: the persistent prep
    kernel walks over several units per CTA with the next unit's inputs arriving under the current one."""

    cpu = oracle.make_inputs(2, 2048, 4, seed=4096)
    ref_out, ref_state = oracle.recurrence(*cpu)
    out, state = chunk_gdn2(*dev(*cpu), output_final_state=True)
    check(out, state, ref_out, ref_state)


@pytest.mark.parametrize("dtype,g_dtype", [(torch.float16, torch.float32), (torch.float16, torch.float16),
                                           (torch.bfloat16, torch.bfloat16)])
def test_chunk_forward_dtypes(dtype, g_dtype):
    cpu = oracle.make_inputs(1, 192, 2, seed=77, dtype=dtype, g_dtype=g_dtype)
    ref_out, ref_state = oracle.recurrence(*cpu, scale=0.125)
    out, state = chunk_forward(*dev(*cpu), scale=0.125)
    assert out.dtype == dtype
    check(out, state, ref_out, ref_state)


def test_weak_decay_distribution_of_the_reference_benchmark():
    """g = -U(0, 0.03), v * 0.2, state * 0.03, scale 0.125 (src/gdn2_sm120/benchmark.py:99-126):
    with almost no decay the state operand matters in every chunk."""

    gen = torch.Generator().manual_seed(20260824)
    shape = (1, 1024, 2, 128)
    q = torch.nn.functional.normalize(torch.randn(shape, generator=gen), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(shape, generator=gen), dim=-1).bfloat16()
    v = (torch.randn(shape, generator=gen) * 0.2).bfloat16()
    g = -torch.rand(shape, generator=gen) * 0.03
    beta = torch.sigmoid(torch.randn(shape, generator=gen)).bfloat16()
    w = torch.sigmoid(torch.randn(shape, generator=gen)).bfloat16()
    s0 = torch.randn((1, 2, 128, 128), generator=gen) * 0.03
    ref_out, ref_state = oracle.recurrence(q, k, v, g, beta, w, s0, scale=0.125)
    out, state = chunk_forward(*dev(q, k, v, g, beta, w, s0), scale=0.125)
    check(out, state, ref_out, ref_state)


def test_strongest_decay_allowed_by_the_contract():
    """g = -5 on every channel: 16-token prefix sums reach -80 (the contract's floor is -87) and
    64-token sums -320; the block-anchored normalisation must not overflow."""

    cpu = list(oracle.make_inputs(1, 128, 2, seed=9))
    cpu[3] = torch.full_like(cpu[3], -5.0)
    ref_out, ref_state = oracle.recurrence(*cpu)
    out, state = chunk_forward(*dev(*cpu))
    assert torch.isfinite(out.float()).all() and torch.isfinite(state).all()
    check(out, state, ref_out, ref_state)


def test_golden_t129_without_state():
    rec = load_golden("chunk_b1_t129_h2_nostate")
    args = dev(rec["q"], rec["k"], rec["v"], rec["g"], rec["beta"], rec["w"])
    out, state = chunk_gdn2(*args, output_final_state=True)
    torch.testing.assert_close(out.float().cpu(), rec["out"].float(), rtol=2e-2, atol=1e-2)
    assert oracle.rel_l2(state, rec["final_state"]) < 1e-3


def test_preallocated_outputs_and_exact_state_alias():
    cpu = oracle.make_inputs(1, 130, 2, seed=404)
    ref_out, ref_state = oracle.recurrence(*cpu)
    q, k, v, g, beta, w, s0 = dev(*cpu)
    out_buf = torch.empty_like(v)
    out, state = chunk_forward(q, k, v, g, beta, w, s0, out=out_buf, final_state_out=s0)
    assert out is out_buf and state is s0
    check(out, state, ref_out, ref_state)
    s0 = cpu[6].to(DEV)
    with pytest.raises(ValueError, match="must not partially overlap"):
        doubled = torch.cat([s0.view(-1), s0.view(-1)])
        doubled[: s0.numel()].copy_(s0.view(-1))
        first = doubled[: s0.numel()].view_as(s0)
        shifted = doubled[64: 64 + s0.numel()].view_as(s0)
        chunk_forward(q, k, v, g, beta, w, first, final_state_out=shifted)
    with pytest.raises(ValueError, match="out must not overlap"):
        chunk_forward(q, k, v, g, beta, w, s0, out=v)
    with pytest.raises(ValueError, match="16-byte aligned"):
        backing = torch.empty(q.numel() + 8, device=DEV, dtype=q.dtype)
        chunk_forward(backing[1:1 + q.numel()].view_as(q), k, v, g, beta, w, s0)
    with pytest.raises(ValueError, match="return_aux=False"):
        chunk_forward(q, k, v, g, beta, w, s0, return_aux=True, out=out_buf)


def test_recurrent_api_crosses_into_chunk_path_and_keeps_buffers():
    cpu = oracle.make_inputs(1, 200, 2, seed=808)
    ref_out, ref_state = oracle.recurrence(*cpu)
    q, k, v, g, beta, w, s0 = dev(*cpu)
    out_buf, fin_buf = torch.empty_like(q), torch.empty_like(s0)
    out, state = recurrent_gdn2(q, k, v, g, beta, w, s0, out=out_buf, final_state_out=fin_buf)
    assert out is out_buf and state is fin_buf
    check(out, state, ref_out, ref_state)
    out, state = recurrent_gdn2(q, k, v, g, beta, w, s0, inplace_final_state=True)
    assert state is s0
    check(out, state, ref_out, ref_state)


def test_chunk_boundaries_are_the_chunk_start_states():
    cpu = oracle.make_inputs(1, 256, 2, seed=12)
    _, _, states = oracle.recurrence(*cpu, return_states=True)
    q, k, v, g, beta, w, s0 = dev(*cpu)
    out, fin = torch.empty_like(v), torch.empty_like(s0)
    bnd = torch.empty((1, 5, 2, 128, 128), device=DEV)
    ws = chunk_kernels.forward(q, k, v, g, beta, w, s0, out, fin, bnd, 1, 256, 2, 256, 128 ** -0.5)
    assert chunk_kernels.read_status(ws, 1, 256, 2) == 0
    assert torch.equal(bnd[:, 0], s0)
    for c in range(5):
        assert oracle.rel_l2(bnd[:, c], states[64 * c]) < 1e-3
    assert torch.equal(bnd[:, 4], fin)


def test_non_default_stream():
    cpu = oracle.make_inputs(1, 320, 2, seed=55)
    ref_out, ref_state = oracle.recurrence(*cpu)
    args = dev(*cpu)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        out, state = chunk_forward(*args)
    side.synchronize()
    check(out, state, ref_out, ref_state)


@pytest.mark.slow
def test_prefill_configuration_properties():
    """Benchmark prefill configuration B=8, T=4096, H=16: too large for the CPU oracle in full, so
    check (i) two heads of one batch row against the oracle and (ii) that the same rows computed
    as a small standalone problem give identical bits (shard independence)."""

    cpu = oracle.make_inputs(8, 4096, 16, seed=0)
    args = dev(*cpu)
    out, state = chunk_gdn2(*args, output_final_state=True)
    sub = tuple(t[3:4, :, 5:7].contiguous() for t in cpu[:6]) + (cpu[6][3:4, 5:7].contiguous(),)
    ref_out, ref_state = oracle.recurrence(*sub)
    check(out[3:4, :, 5:7], state[3:4, 5:7], ref_out, ref_state)
    out_sub, state_sub = chunk_gdn2(*dev(*sub), output_final_state=True)
    assert torch.equal(out_sub, out[3:4, :, 5:7]) and torch.equal(state_sub, state[3:4, 5:7])


def test_per_kernel_profile_events():
    """`gdn2_profile_enable` / `gdn2_profile_chunk_kernels`: four positive durations after a
    training forward + backward, nothing once profiling is switched off again."""

    from gdn2_sm120_b200 import _lib

    cpu = oracle.make_inputs(1, 256, 2, seed=21)
    leaves = [t.to(DEV).requires_grad_(True) for t in cpu]
    _lib.profile_enable(True)
    try:
        out, fin = chunk_gdn2(*leaves[:6], leaves[6], output_final_state=True)
        torch.autograd.grad(out.float().sum() + fin.sum(), leaves)
        times = _lib.profile_chunk_kernels()
    finally:
        _lib.profile_enable(False)
    assert set(times) == {"chunk_prep_kernel", "chunk_scan_kernel", "chunk_bwd_scan_kernel", "chunk_bwd_vjp_kernel"}
    assert all(0.0 < value < 100.0 for value in times.values())
    assert _lib.profile_chunk_kernels() == {}


def test_two_host_threads_on_their_own_streams():
    """Launches are lock-free and the library keeps no per-call state: two Python threads, each on its
    own stream with its own problem, get the results a single thread gets."""

    import threading

    problems = [oracle.make_inputs(1, 192 + 64 * i, 2, seed=300 + i) for i in range(2)]
    expected = [chunk_gdn2(*dev(*cpu), output_final_state=True) for cpu in problems]
    torch.cuda.synchronize()
    results = [None, None]
    errors = []

    def worker(index):
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                tensors = dev(*problems[index])
                for _ in range(5):
                    results[index] = chunk_gdn2(*tensors, output_final_state=True)
            stream.synchronize()
        except Exception as exc:  # noqa: BLE001 - reported by the main thread
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for (out, state), (ref_out, ref_state) in zip(results, expected):
        assert torch.equal(out, ref_out) and torch.equal(state, ref_state)
