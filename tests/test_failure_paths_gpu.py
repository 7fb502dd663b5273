"""GPU tests of the failure paths of the chunk kernels, without faulting anything.

Every asynchronous wait inside the kernels (bulk copies, tensor-core commits) is bounded: when it
gives up, the kernel records status 1 in the workspace, keeps going to its end (so that tensor
memory is released) and writes NaN instead of results.  The test entry point
``gdn2_debug_wait_expires`` makes such a wait run out in the only harmless way there is: a small
kernel polls, at most 1024 times, an mbarrier that nothing arms, and returns by itself.
"""

from __future__ import annotations

import pytest
import torch

import gdn2_oracle as oracle
from gdn2_sm120_b200 import _lib, chunk_kernels
from gdn2_sm120_b200.chunk import chunk_forward

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _forward_into(workspace, scratch, tensors, batch, time, heads, scale):
    q, k, v, g, beta, w, s0 = tensors
    out = torch.zeros_like(v)
    fin = torch.empty_like(s0)
    _lib.call("gdn2_chunk_forward", q.device, q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(),
              beta.data_ptr(), w.data_ptr(), s0.data_ptr(), out.data_ptr(), fin.data_ptr(), None,
              workspace.data_ptr(), scratch.data_ptr(), batch, time, heads, time, 0,
              _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale, _lib.stream_ptr(q.device))
    return out, fin


def _expire_a_wait(workspace, batch, time, heads, polls=1024):
    status = _lib.lib().gdn2_debug_wait_expires(workspace.data_ptr(), batch, time, heads, polls,
                                                torch.cuda.current_stream().cuda_stream)
    assert status == 0, _lib.lib().gdn2_status_string(status)


def test_expired_wait_sets_the_status_word_and_the_next_call_clears_it():
    batch, time, heads, scale = 1, 128, 2, 128 ** -0.5
    tensors = [t.to(DEV) for t in oracle.make_inputs(batch, time, heads, seed=70)]
    workspace = torch.empty(chunk_kernels.workspace_bytes(batch, time, heads, False), device=DEV, dtype=torch.uint8)
    scratch = torch.empty(chunk_kernels.scratch_bytes(batch, time, heads, False), device=DEV, dtype=torch.uint8)
    out, fin = _forward_into(workspace, scratch, tensors, batch, time, heads, scale)
    assert chunk_kernels.read_status(workspace, batch, time, heads) == 0

    _expire_a_wait(workspace, batch, time, heads)
    assert chunk_kernels.read_status(workspace, batch, time, heads) == 1   # the kernel came back by itself

    # the context is intact and the same workspace serves the next call, which starts from status 0
    out2, fin2 = _forward_into(workspace, scratch, tensors, batch, time, heads, scale)
    assert chunk_kernels.read_status(workspace, batch, time, heads) == 0
    assert torch.equal(out, out2) and torch.equal(fin, fin2)


def test_a_failure_recorded_in_the_workspace_turns_the_gradients_into_nan():
    """Backward starts from the status word the forward left: a wait that expired anywhere upstream
    shows in the gradients themselves, not only in a word that nobody reads."""

    batch, time, heads, scale = 1, 128, 2, 128 ** -0.5
    q, k, v, g, beta, w, s0 = (t.to(DEV) for t in oracle.make_inputs(batch, time, heads, seed=71))
    _, _, aux = chunk_forward(q, k, v, g, beta, w, s0, scale=scale, return_aux=True)
    assert chunk_kernels.read_status(aux.workspace, batch, time, heads) == 0
    d_out = torch.ones_like(v)
    d_fin = torch.ones_like(s0)

    def backward():
        grads = tuple(torch.zeros_like(x) for x in (q, k, v, g, beta, w))
        d_s0 = torch.zeros_like(s0)
        chunk_kernels.backward(q, k, v, g, beta, w, aux.workspace, aux.chunk_boundaries, d_out, d_fin, grads,
                               d_s0, batch, time, heads, time, scale)
        torch.cuda.synchronize()
        return (*grads, d_s0)

    assert all(torch.isfinite(x.float()).all() for x in backward())
    _expire_a_wait(aux.workspace[0], batch, time, heads)
    assert chunk_kernels.read_status(aux.workspace, batch, time, heads) == 1
    assert all(torch.isnan(x.float()).all() for x in backward())


def test_debug_wait_entry_validates_its_arguments():
    handle = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert handle.gdn2_debug_wait_expires(None, 1, 64, 1, 16, stream) == -1
    buf = torch.empty(4096, device=DEV, dtype=torch.uint8)
    assert handle.gdn2_debug_wait_expires(buf.data_ptr(), 1, 65, 1, 16, stream) == -2
