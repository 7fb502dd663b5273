"""GPU test of gdn2_chunk_forward_static, the chunk forward whose workspace is a fixed array
inside the library (for hosts that may not allocate device memory per call, e.g. a server
that plans all GPU memory at start-up).  Collected last on purpose: if it fails under
``pytest -x`` every other test has already run.

It calls the new entry point through the C ABI twice in a row, with different inputs, and
compares each result with the ordinary entry point (caller-allocated workspace) on the same
inputs, within the chunk path's tolerances.  The second call checks that nothing left in the
shared array by the first call leaks into the result.
"""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from gdn2_sm120_b200 import _lib, chunk_kernels

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call_static(q, k, v, g, beta, w, s0, batch, time, heads, full, scale):
    out = torch.zeros_like(v)
    fin = torch.empty((batch, heads, 128, 128), device=DEV)
    handle = _lib.lib()
    status = handle.gdn2_chunk_forward_static(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
        None if s0 is None else s0.data_ptr(), out.data_ptr(), fin.data_ptr(),
        batch, time, heads, full, _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale,
        torch.cuda.current_stream().cuda_stream)
    return status, out, fin


def _call_ordinary(q, k, v, g, beta, w, s0, batch, time, heads, full, scale):
    out = torch.zeros_like(v)
    fin = torch.empty((batch, heads, 128, 128), device=DEV)
    ws = chunk_kernels.forward(q, k, v, g, beta, w, s0, out, fin, None, batch, time, heads, full, scale)
    assert chunk_kernels.read_status(ws, batch, full, heads) == 0
    return out, fin


@pytest.mark.parametrize("shapes", [[(1, 256, 4, 501, True), (2, 128, 3, 502, False), (1, 200, 3, 503, True)]])
def test_static_workspace_entry_matches_ordinary_entry_twice(shapes):
    scale = 128 ** -0.5
    for batch, time, heads, seed, with_state in shapes:
        cpu = oracle.make_inputs(batch, time, heads, seed=seed, with_state=with_state)
        q, k, v, g, beta, w = (t.to(DEV) for t in cpu[:6])
        s0 = cpu[6].to(DEV) if with_state else None
        full = -(-time // 64) * 64  # 200 tokens: four chunks, the last one with 8 of its 64 tokens
        status, out_s, fin_s = _call_static(q, k, v, g, beta, w, s0, batch, time, heads, full, scale)
        assert status == 0, _lib.lib().gdn2_status_string(status)
        # no bounded wait ran out inside the kernels (status word of the fixed array)
        assert _lib.lib().gdn2_chunk_static_read_status(torch.cuda.current_stream().cuda_stream) == 0
        out_o, fin_o = _call_ordinary(q, k, v, g, beta, w, s0, batch, time, heads, full, scale)
        torch.cuda.synchronize()
        torch.testing.assert_close(out_s.float(), out_o.float(), rtol=2e-2, atol=1e-2)
        assert oracle.rel_l2(fin_s, fin_o) < 1e-3
        # and against the oracle, like every other chunk-path test
        ref_out, ref_state = oracle.recurrence(*cpu)
        torch.testing.assert_close(out_s.float().cpu(), ref_out.float(), rtol=2e-2, atol=1e-2)
        assert oracle.rel_l2(fin_s, ref_state) < 1e-3


def test_static_workspace_entry_rejects_sizes_beyond_its_array():
    batch, time, heads = 2, 512, 8  # 2 * 8 * 8 = 128 chunk-heads > 64
    cpu = oracle.make_inputs(batch, time, heads, seed=9)
    q, k, v, g, beta, w, s0 = (t.to(DEV) for t in cpu)
    status, _, _ = _call_static(q, k, v, g, beta, w, s0, batch, time, heads, time, 0.1)
    assert status == -9
    assert b"exceeds" in _lib.lib().gdn2_status_string(status)
