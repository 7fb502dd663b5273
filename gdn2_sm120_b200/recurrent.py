"""Recurrent / decode forward: host wrapper over the token-path kernels.

Mirrors ``token_forward`` of the reference (src/gdn2_sm120/recurrent.py:704-891):
same signature, same ownership rules for ``out`` / ``final_state_out`` /
``inplace_final_state``, same overlap rejections and T == 0 behaviour, and the same
shape-based crossover into the chunk path for long sequences.  The device work is
``gdn2_token_forward`` / ``gdn2_token_forward_t1_zero`` of the C ABI.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from . import _lib, _validate

_DIM = _validate.DIM
# Sequences up to this length always run on the token kernel.
_SHORT_RECURRENT_MAX_TOKENS = 32
# From here on the chunk path is used (one full 64-token tensor-core chunk exists).
_CHUNK_ALWAYS_MIN_TOKENS = 64


def _use_recurrent_kernel(batch: int, time: int, heads: int, *, chunk_api: bool = False) -> bool:
    """Shape-based forward dispatch (reference: src/gdn2_sm120/recurrent.py:59-84).

    The structure of the reference's selector is kept -- always recurrent up to 32
    tokens, always chunked from 64 tokens, an API-dependent window in between -- but on
    B200 the chunk kernels work on 64-token chunks, so nothing below 64 tokens holds a
    full chunk and the window resolves to the token kernel for both APIs.
    """

    del batch, heads  # the B200 crossover does not depend on the grid size
    if time <= _SHORT_RECURRENT_MAX_TOKENS:
        return True
    if time >= _CHUNK_ALWAYS_MIN_TOKENS:
        return False
    # 33..63 tokens: the reference sends the chunk API to its chunk kernel at 48 tokens (three of its
    # 16-token chunks); here the window holds no full chunk for either API
    del chunk_api
    return True


def _chunk_forward_compatible(tensors: Sequence[torch.Tensor]) -> bool:
    """The chunk path needs every buffer 16-byte aligned (TMA / 128-bit access)."""

    return all(t.data_ptr() % 16 == 0 for t in tensors)


_byte_span = _validate.byte_span
_spans_overlap = _validate.spans_overlap


def _launch_token_forward(q, k, v, g, beta, w, initial_state, output, final_state, boundaries,
                          batch, time, heads, t_begin, t_end, scale, prologue: int = 0) -> None:
    if prologue:
        if boundaries is not None:
            raise ValueError("the fused prologue is forward-only: no checkpoints")
        _lib.call(
            "gdn2_token_forward_fused", q.device,
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
            _lib.ptr(initial_state), output.data_ptr(), _lib.ptr(final_state),
            batch, time, heads, t_begin, t_end,
            _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale, prologue, _lib.stream_ptr(q.device),
        )
        return
    _lib.call(
        "gdn2_token_forward", q.device,
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
        _lib.ptr(initial_state), output.data_ptr(), _lib.ptr(final_state), _lib.ptr(boundaries),
        batch, time, heads, t_begin, t_end,
        _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale, _lib.stream_ptr(q.device),
    )


def _launch_t1_zero(q, k, v, w, output, final_state, batch, heads, scale, prologue: int = 0) -> None:
    if prologue:
        _lib.call(
            "gdn2_token_forward_t1_zero_fused", q.device,
            q.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), output.data_ptr(),
            final_state.data_ptr(), batch, heads, _lib.dtype_code(q.dtype), scale, prologue,
            _lib.stream_ptr(q.device),
        )
        return
    _lib.call(
        "gdn2_token_forward_t1_zero", q.device,
        q.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), output.data_ptr(),
        final_state.data_ptr(), batch, heads, _lib.dtype_code(q.dtype), scale,
        _lib.stream_ptr(q.device),
    )


def token_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    w: torch.Tensor,
    initial_state: torch.Tensor | None = None,
    scale: float | None = None,
    *,
    out: torch.Tensor | None = None,
    final_state_out: torch.Tensor | None = None,
    inplace_final_state: bool = False,
    prologue: int = 0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Evaluate the GDN2 recurrence; returns ``(output, final_state)``.

    ``prologue`` (not part of the reference's signature; bit 0 = L2-normalise raw q / k, bit 1 =
    activate raw beta / w / g) makes the forward kernels apply a layer's input prologue themselves.

    Inputs are contiguous ``[B, T, H, 128]``; q/k/v/beta/w fp16 or bf16, ``g`` the same
    type or fp32; ``initial_state`` optional fp32 ``[B, H, 128, 128]``.  By default fresh
    tensors are allocated and no input is modified.  ``out`` / ``final_state_out`` are
    caller-owned buffers that are returned by identity; ``inplace_final_state=True``
    updates and returns ``initial_state`` itself.
    """

    batch, time, heads = _validate.sequence_inputs(q, k, v, g, beta, w)
    if initial_state is not None:
        _validate.state("initial_state", initial_state, batch, heads, q.device)
    output_scale = _validate.float32_scale(scale)

    if out is None:
        output = torch.empty_like(q)
    else:
        _validate.buffer("out", out, q.shape, q.dtype, q.device)
        output = out

    state_shape = (batch, heads, _DIM, _DIM)
    if inplace_final_state:
        if initial_state is None:
            raise ValueError("inplace_final_state=True requires initial_state")
        if final_state_out is not None:
            raise ValueError("final_state_out cannot be used with inplace_final_state=True")
        final_state = initial_state
    elif final_state_out is not None:
        _validate.buffer("final_state_out", final_state_out, state_shape, torch.float32, q.device)
        final_state = final_state_out
    else:
        final_state = torch.empty(state_shape, device=q.device, dtype=torch.float32)

    sequence = (q, k, v, g, beta, w)
    if out is not None or final_state_out is not None or inplace_final_state:
        seq_spans = [_byte_span(t) for t in sequence]
        init_span = _byte_span(initial_state) if initial_state is not None else None
        final_span = _byte_span(final_state)
        if out is not None and output.numel():
            out_span = _byte_span(output)
            if any(_spans_overlap(out_span, s) for s in seq_spans) or (
                init_span is not None and _spans_overlap(out_span, init_span)
            ):
                raise ValueError("out must not overlap an input tensor")
            if _spans_overlap(out_span, final_span):
                raise ValueError("out and final_state must not overlap")
        if final_state_out is not None:
            if any(_spans_overlap(final_span, s) for s in seq_spans) or (
                init_span is not None and _spans_overlap(final_span, init_span)
            ):
                raise ValueError("final_state_out must not overlap an input tensor")
        if inplace_final_state and any(_spans_overlap(final_span, s) for s in seq_spans):
            raise ValueError("initial_state must not overlap sequence inputs for in-place update")

    if time == 0:
        if initial_state is None:
            final_state.zero_()
        elif final_state is not initial_state:
            final_state.copy_(initial_state)
        return output, final_state

    if not _use_recurrent_kernel(batch, time, heads) and _chunk_forward_compatible(
        (*sequence, output, final_state) + (() if initial_state is None else (initial_state,))
    ):
        from .chunk import chunk_forward  # lazy: decode never pays for the chunk module

        return chunk_forward(q, k, v, g, beta, w, initial_state, scale=output_scale,
                             out=output, final_state_out=final_state, prologue=prologue)

    if time == 1 and initial_state is None:
        _launch_t1_zero(q, k, v, w, output, final_state, batch, heads, output_scale, prologue)
    else:
        _launch_token_forward(q, k, v, g, beta, w, initial_state, output, final_state, None,
                              batch, time, heads, 0, time, output_scale, prologue)
    return output, final_state


__all__ = ["token_forward"]
