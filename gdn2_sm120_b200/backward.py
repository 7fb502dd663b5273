"""Checkpointed backward: host wrapper.

``chunk_backward`` keeps the public signature of the reference
(src/gdn2_sm120/backward.py:1264-1349) and returns
``dq, dk, dv, dg, dbeta, dw, d_initial_state``.  One deliberate difference: the
reference reconstructs earlier states from ``final_state`` by inverting the
recurrence (Sherman-Morrison, docs/design.md:125-145 of the reference), whose error
grows like exp(sum |g|).  Here the forward is re-run from ``initial_state`` (``None`` =
zero) with fp32 checkpoints -- on the tensor-core chunk kernels from 64 tokens on, on the
token kernels below -- and nothing is inverted, so callers whose forward started from a
non-zero state must pass it, at every length (the reference needs it only above 128 tokens,
backward.py:1286-1298).  ``final_state`` is used as a consistency check: the state the re-run
arrives at is compared with it on the device, and a mismatch raises ``ValueError`` instead of
returning gradients of a different forward.  The check cannot see a wrong starting state whose
influence has decayed away by the end of the sequence.

``backward_from_aux`` is what the autograd wrapper calls: it consumes the checkpoints
that ``chunk_forward(return_aux=True)`` saved.  The ragged tail is differentiated first
(it yields the cotangent of the state after the last full chunk), then the full chunks,
mirroring the order of the reference (backward_parallel.py:1493-1522).
"""

from __future__ import annotations

import torch

from . import _lib, _validate
from .chunk import ChunkForwardAux, _token_slots, chunk_forward
from .recurrent import _chunk_forward_compatible, _launch_token_forward, _use_recurrent_kernel

_DIM = _validate.DIM
# Kept for callers that imported the reference's constant (backward.py:57): there it is
# the longest sequence the final-state-only inverse path accepts; here no cap exists.
MAX_BACKWARD_TOKENS = 128
# Largest relative L2 distance between the caller's final_state and the recomputed one that still
# counts as "the same forward": the chunk kernels' tf32 contractions differ from an exact fp32
# recurrence by up to ~5e-4, a wrong starting state by O(1).
_FINAL_STATE_REL_TOL = 5e-3


def _token_backward(q, k, v, g, beta, w, d_out, d_final_state, boundaries, grads,
                    batch, time, heads, t_begin, t_end, scale, d_state_before):
    """Token-path VJP over tokens [t_begin, t_end); writes ``d_state_before``."""

    dq, dk, dv, dg, dbeta, dw = grads
    d_boundaries = torch.empty_like(boundaries)
    dtype, g_dtype = _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype)
    stream = _lib.stream_ptr(q.device)
    _lib.call(
        "gdn2_token_dstate_scan", q.device,
        q.data_ptr(), k.data_ptr(), g.data_ptr(), beta.data_ptr(), d_out.data_ptr(),
        _lib.ptr(d_final_state), d_boundaries.data_ptr(), _lib.ptr(d_state_before),
        batch, time, heads, t_begin, t_end, dtype, g_dtype, scale, stream,
    )
    _lib.call(
        "gdn2_token_chunk_vjp", q.device,
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
        d_out.data_ptr(), boundaries.data_ptr(), d_boundaries.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), dbeta.data_ptr(),
        dw.data_ptr(), batch, time, heads, t_begin, t_end, dtype, g_dtype, scale, stream,
    )


def backward_from_aux(q, k, v, g, beta, w, aux: ChunkForwardAux, d_out, d_final_state, scale, *,
                      grads_out=None, d_initial_state_out=None):
    """Gradients from saved checkpoints; ``d_final_state`` may be ``None`` (zero).

    ``grads_out`` (six contiguous tensors shaped like the inputs) and ``d_initial_state_out`` let a
    caller have the kernels write into buffers it owns (slices of packed tensors, for instance)."""

    batch, time, heads, _ = q.shape
    grads = grads_out if grads_out is not None else tuple(torch.empty_like(x) for x in (q, k, v, g, beta, w))
    d_initial_state = d_initial_state_out if d_initial_state_out is not None else torch.empty(
        (batch, heads, _DIM, _DIM), device=q.device, dtype=torch.float32)
    full = aux.full_tokens
    d_state = d_final_state
    if time > full:
        # tail first: its scan produces the cotangent of the state after the last full chunk
        target = d_initial_state if full == 0 else torch.empty_like(d_initial_state)
        _token_backward(q, k, v, g, beta, w, d_out, d_state, aux.tail_boundaries, grads,
                        batch, time, heads, full, time, scale, target)
        d_state = target
    if full:
        from . import chunk_kernels

        chunk_kernels.backward(q, k, v, g, beta, w, aux.workspace, aux.chunk_boundaries, d_out,
                               d_state, grads, d_initial_state, batch, time, heads, full, scale)
    return (*grads, d_initial_state)


def chunk_backward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    w: torch.Tensor,
    final_state: torch.Tensor,
    do: torch.Tensor,
    d_final_state: torch.Tensor,
    scale: float | None = None,
    initial_state: torch.Tensor | None = None,
):
    """Return ``dq, dk, dv, dg, dbeta, dw, d_initial_state`` (see module docstring)."""

    batch, time, heads = _validate.sequence_inputs(q, k, v, g, beta, w)
    if not isinstance(do, torch.Tensor) or do.shape != v.shape:
        raise ValueError("do must match v's [B, T, H, 128] shape")
    if do.dtype != q.dtype:
        raise TypeError("q, k, v, beta, w, and do must have the same dtype")
    if do.device != q.device or not do.is_contiguous():
        raise ValueError("do must be a contiguous CUDA tensor on q's device")
    _validate.state("final_state", final_state, batch, heads, q.device)
    _validate.state("d_final_state", d_final_state, batch, heads, q.device)
    if initial_state is not None:
        _validate.state("initial_state", initial_state, batch, heads, q.device)
    output_scale = _validate.float32_scale(scale)

    args = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
    do_arg, dfs_arg = _validate.detached(do), _validate.detached(d_final_state)
    s0 = _validate.detached(initial_state)
    given_final = _validate.detached(final_state)
    if time == 0:
        grads = tuple(torch.empty_like(x) for x in args)
        return (*grads, dfs_arg.clone())

    # recompute the forward with checkpoints, then differentiate
    buffers = (*args, do_arg, dfs_arg) + (() if s0 is None else (s0,))
    if not _use_recurrent_kernel(batch, time, heads) and _chunk_forward_compatible(buffers):
        _, reached, aux = chunk_forward(*args, s0, scale=output_scale, return_aux=True)
    else:
        boundaries = torch.empty((batch, _token_slots(time), heads, _DIM, _DIM), device=q.device,
                                 dtype=torch.float32)
        reached = torch.empty((batch, heads, _DIM, _DIM), device=q.device, dtype=torch.float32)
        scratch_out = torch.empty_like(v)
        _launch_token_forward(*args, s0, scratch_out, reached, boundaries, batch, time, heads, 0, time,
                              output_scale)
        aux = ChunkForwardAux(None, boundaries, 0)
    # one small reduction on the device, read back after the backward kernels have been queued
    mismatch = torch.stack([(reached - given_final).square().sum(), given_final.square().sum()])
    result = backward_from_aux(*args, aux, do_arg, dfs_arg, output_scale)
    diff2, ref2 = mismatch.tolist()
    if not diff2 <= _FINAL_STATE_REL_TOL ** 2 * max(ref2, 1e-30):
        raise ValueError(
            "final_state does not match the state the forward reaches from initial_state "
            f"(relative L2 difference {(diff2 / max(ref2, 1e-30)) ** 0.5:.3e}): chunk_backward re-runs the "
            "forward from initial_state (None = zero) and never inverts the recurrence, so a forward that "
            "started from a non-zero state needs initial_state passed here"
        )
    return result


__all__ = ["MAX_BACKWARD_TOKENS", "chunk_backward"]
