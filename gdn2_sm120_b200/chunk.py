"""Chunkwise forward: host wrapper.

Mirrors ``chunk_forward`` / ``ChunkForwardAux`` of the reference
(src/gdn2_sm120/chunk.py:1056-1075, 1160-1419): same signature, validation, ``out`` /
``final_state_out`` rules (``final_state_out`` may alias ``initial_state`` exactly,
never partially) and the ``return_aux`` contract used by the autograd wrapper.

From 64 tokens on the tensor-core chunk kernels process the whole sequence:
``full_tokens = 64 * ceil(T / 64)``, the last chunk of a ragged length being partial (the
kernels read its missing tokens as zeros, the identity step of the recurrence; the reference
runs a scalar tail scan instead, chunk.py:1021-1053).  Shorter sequences
(``full_tokens = 0``) go to the exact fp32 token kernels as one tail.

Activation checkpoints for backward are the fp32 states at chunk / span starts plus,
for the chunk kernels, the workspaces of per-chunk WY factors that the forward prep kernel
wrote, one per wave of batch rows (the reference saves the same factors, chunk.py:1056-1075).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib, _validate
from .recurrent import _byte_span, _launch_token_forward, _spans_overlap

_DIM = _validate.DIM
_CHUNK = 64           # tokens per tensor-core chunk
_TOKEN_INTERVAL = 16  # tokens between two token-path boundary slots


@dataclass(frozen=True)
class ChunkForwardAux:
    """State checkpoints consumed by the checkpointed backward.

    ``chunk_boundaries``  fp32 ``[B, full_tokens/64 + 1, H, 128, 128]``: state before every
                          64-token chunk and after the last one, or ``None``.
    ``tail_boundaries``   fp32 ``[B, ceil(tail/16) + 1, H, 128, 128]``: state before every
                          16-token span of the tail ``[full_tokens, T)`` and after it, or
                          ``None`` when there is no tail (any sequence of 64 tokens or more).
    ``full_tokens``       tokens covered by ``chunk_boundaries`` (``T`` rounded up to whole chunks).
    ``workspace``         the chunk kernels' per-chunk WY factors (operand-ready tiles written
                          by the forward prep kernel and reused by backward), a tuple with one
                          tensor per wave of batch rows, or ``None``.
    """

    chunk_boundaries: torch.Tensor | None
    tail_boundaries: torch.Tensor | None
    full_tokens: int
    workspace: tuple[torch.Tensor, ...] | None = None


def _token_slots(tokens: int) -> int:
    return -(-tokens // _TOKEN_INTERVAL) + 1


def _chunk_kernel_tokens(time: int) -> int:
    """Tokens handed to the tensor-core chunk kernels, a multiple of 64: none below 64 tokens, else the
    whole sequence rounded up (the kernels treat the missing tokens of a partial last chunk as identity
    steps, so a ragged length costs one more chunk instead of a pass through the token kernels)."""

    if time < _CHUNK:
        return 0
    return -(-time // _CHUNK) * _CHUNK


def chunk_forward(
    q,
    k,
    v,
    g,
    beta,
    w,
    initial_state=None,
    *,
    scale: float | None = None,
    return_aux: bool = False,
    out=None,
    final_state_out=None,
    prologue: int = 0,
):
    """Run the chunkwise forward; returns ``(output, final_state[, aux])``.

    ``prologue`` (not in the reference's signature): bit flags of the layer prologue the forward
    kernels apply themselves to raw inputs (see ``prologue.py``); forward-only, so it excludes
    ``return_aux``."""

    batch, time, heads = _validate.sequence_inputs(
        q, k, v, g, beta, w, dim_error=NotImplementedError, need_tokens=True, need_alignment=True
    )
    if initial_state is not None:
        _validate.state("initial_state", initial_state, batch, heads, q.device, need_alignment=True)
    output_scale = _validate.float32_scale(scale)
    if return_aux and (out is not None or final_state_out is not None):
        raise ValueError("preallocated outputs are supported only when return_aux=False")
    if return_aux and prologue:
        raise ValueError("the fused prologue is forward-only: activate with gate_prologue when training")

    state_shape = (batch, heads, _DIM, _DIM)
    if out is None:
        output = torch.empty_like(v)
    else:
        _validate.buffer("out", out, v.shape, v.dtype, q.device, need_alignment=True)
        output = out
    if final_state_out is None:
        final_state = torch.empty(state_shape, device=q.device, dtype=torch.float32)
    else:
        _validate.buffer("final_state_out", final_state_out, state_shape, torch.float32, q.device,
                         need_alignment=True)
        final_state = final_state_out

    if out is not None or final_state_out is not None:
        seq_spans = [_byte_span(t) for t in (q, k, v, g, beta, w)]
        init_span = _byte_span(initial_state) if initial_state is not None else None
        out_span, final_span = _byte_span(output), _byte_span(final_state)
        if out is not None:
            if any(_spans_overlap(out_span, s) for s in seq_spans) or (
                init_span is not None and _spans_overlap(out_span, init_span)
            ):
                raise ValueError("out must not overlap an input tensor")
            if _spans_overlap(out_span, final_span):
                raise ValueError("out and final_state_out must not overlap")
        if final_state_out is not None:
            if any(_spans_overlap(final_span, s) for s in seq_spans):
                raise ValueError("final_state_out must not overlap a sequence input")
            if init_span is not None and final_span != init_span and _spans_overlap(final_span, init_span):
                raise ValueError(
                    "final_state_out may exactly alias initial_state but must not partially overlap it"
                )

    full_tokens = _chunk_kernel_tokens(time)
    tail = max(0, time - full_tokens)  # only sequences shorter than one chunk have one
    chunk_boundaries = tail_boundaries = None
    if return_aux:
        if full_tokens:
            from . import chunk_kernels

            chunk_kernels.check_memory(
                batch * (full_tokens // _CHUNK + 1) * heads * _DIM * _DIM * 4
                + chunk_kernels.workspace_bytes(batch, full_tokens, heads, True),
                q.device, "chunk forward with checkpoints")
            chunk_boundaries = torch.empty(
                (batch, full_tokens // _CHUNK + 1, heads, _DIM, _DIM), device=q.device, dtype=torch.float32
            )
        if tail:
            tail_boundaries = torch.empty(
                (batch, _token_slots(tail), heads, _DIM, _DIM), device=q.device, dtype=torch.float32
            )

    state = initial_state
    workspace = None
    if full_tokens:
        from . import chunk_kernels

        workspace = chunk_kernels.forward(q, k, v, g, beta, w, state, output, final_state,
                                          chunk_boundaries, batch, time, heads, full_tokens,
                                          output_scale, prologue=prologue)
        state = final_state
    if tail:
        _launch_token_forward(q, k, v, g, beta, w, state, output, final_state, tail_boundaries,
                              batch, time, heads, full_tokens, time, output_scale, prologue)
    if not return_aux:
        return output, final_state
    return output, final_state, ChunkForwardAux(chunk_boundaries, tail_boundaries, full_tokens,
                                                workspace if return_aux else None)


__all__ = ["ChunkForwardAux", "chunk_forward"]
