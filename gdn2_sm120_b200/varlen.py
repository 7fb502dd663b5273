"""Packed variable-length sequences and grouped value heads on top of the primitive.

The reference lists both as not yet part of its specialisation (README.md:128-130, 297-299 of
the reference); callers that batch ragged sequences need them next to the operator:

``chunk_gdn2_varlen``    several sequences packed along the time axis of ``[1, total, H, 128]``
                         tensors, delimited by ``cu_seqlens`` (``[N + 1]`` cumulative lengths, as
                         in flash-attention style APIs), each with its own initial / final state
                         (``[N, H, 128, 128]``).  Every sequence is an independent recurrence, so
                         the implementation walks over the sequences and runs the same
                         shape-dispatched kernels on each slice of the packed buffers (a slice of
                         consecutive tokens of a batch-1 tensor is itself a contiguous
                         ``[1, L, H, 128]`` tensor: nothing is copied on the way in).  One
                         ``autograd.Function`` spans the whole call, so backward writes every
                         sequence's gradients straight into the packed gradient tensors.
``expand_grouped_heads`` key-shaped tensors given for fewer heads than the value-shaped ones
                         (every group of value heads shares one q / k / g / beta head) expanded
                         to the value heads; gradients of the shared heads are summed by autograd.

The kernels themselves are unchanged: one launch sequence per packed sequence, which is efficient
for long sequences (prefill, training on documents) and launch-bound for many very short ones.
"""

from __future__ import annotations

import math

import torch

from . import _validate
from .backward import backward_from_aux
from .ops import _aux_from_tensors, _aux_tensors, _forward_with_aux, _prologue_flags
from .prologue import gate_prologue

_DIM = 128


def _bounds(cu_seqlens, total: int) -> tuple[int, ...]:
    if isinstance(cu_seqlens, torch.Tensor):
        if cu_seqlens.ndim != 1 or cu_seqlens.dtype not in (torch.int32, torch.int64):
            raise TypeError("cu_seqlens must be a rank-1 int32 or int64 tensor")
        values = [int(x) for x in cu_seqlens.tolist()]
    else:
        values = [int(x) for x in cu_seqlens]
    if len(values) < 2 or values[0] != 0 or values[-1] != total:
        raise ValueError("cu_seqlens must start at 0 and end at the packed length of the tensors")
    if any(b < a for a, b in zip(values, values[1:])):
        raise ValueError("cu_seqlens must be non-decreasing")
    return tuple(values)


def _packed_forward(seq, state, bounds, scale: float, prepare_backward: bool, prologue: int = 0):
    """Forward over every packed sequence; returns output, final states and the saved checkpoints."""

    q = seq[0]
    n_seq, heads = len(bounds) - 1, q.shape[2]
    output = torch.empty_like(seq[2])
    final_state = torch.empty((n_seq, heads, _DIM, _DIM), device=q.device, dtype=torch.float32)
    saved, layouts = [], []
    for i, (start, stop) in enumerate(zip(bounds, bounds[1:])):
        state_i = None if state is None else state[i:i + 1]
        if stop == start:   # an empty sequence leaves its state as it is
            if state_i is None:
                final_state[i].zero_()
            else:
                final_state[i:i + 1].copy_(state_i)
            layouts.append((0, 0, 0, 0))
            continue
        piece = tuple(t[:, start:stop] for t in seq)
        out_i, final_i, aux = _forward_with_aux(piece, state_i, scale, prepare_backward, prologue)
        output[:, start:stop].copy_(out_i)
        final_state[i:i + 1].copy_(final_i)
        tensors, layout = _aux_tensors(aux)
        saved.extend(tensors)
        layouts.append(layout)
    return output, final_state, saved, tuple(layouts)


class _ChunkGDN2Varlen(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, w, initial_state, bounds, scale: float):
        seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
        output, final_state, saved, layouts = _packed_forward(seq, _validate.detached(initial_state), bounds,
                                                              scale, True)
        ctx.save_for_backward(q, k, v, g, beta, w, *saved)
        ctx.set_materialize_grads(False)
        ctx.bounds, ctx.layouts, ctx.scale = bounds, layouts, scale
        ctx.has_initial_state = initial_state is not None
        return output, final_state

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_output, d_final_state):
        q, k, v, g, beta, w, *saved = ctx.saved_tensors
        seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
        n_seq, heads = len(ctx.bounds) - 1, q.shape[2]
        if d_output is None:
            d_output = torch.zeros_like(v)
        elif not d_output.is_contiguous():
            d_output = d_output.contiguous()
        if d_final_state is not None and not d_final_state.is_contiguous():
            d_final_state = d_final_state.contiguous()
        grads = tuple(torch.empty_like(x) for x in seq)
        d_state = torch.empty((n_seq, heads, _DIM, _DIM), device=q.device, dtype=torch.float32)
        scale = _validate.float32_scale(ctx.scale)
        cursor = 0
        for i, (start, stop) in enumerate(zip(ctx.bounds, ctx.bounds[1:])):
            layout = ctx.layouts[i]
            d_final_i = None if d_final_state is None else d_final_state[i:i + 1]
            if stop == start:
                if d_final_i is None:
                    d_state[i].zero_()
                else:
                    d_state[i:i + 1].copy_(d_final_i)
                continue
            count = layout[0] + layout[1] + layout[2]
            aux = _aux_from_tensors(saved[cursor:cursor + count], layout)
            cursor += count
            backward_from_aux(*(t[:, start:stop] for t in seq), aux, d_output[:, start:stop], d_final_i, scale,
                              grads_out=tuple(gr[:, start:stop] for gr in grads),
                              d_initial_state_out=d_state[i:i + 1])
        return (*grads, d_state if ctx.has_initial_state else None, None, None)


def chunk_gdn2_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    w: torch.Tensor,
    cu_seqlens,
    initial_state: torch.Tensor | None = None,
    *,
    scale: float | None = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    use_gate_in_kernel: bool = False,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``chunk_gdn2`` over ``N`` sequences packed along time.

    Sequence tensors are contiguous ``[1, total, H, 128]`` (same dtype rules as ``chunk_gdn2``);
    ``cu_seqlens`` holds ``N + 1`` cumulative lengths (tensor or sequence of ints, read on the host);
    ``initial_state`` is ``None`` or fp32 ``[N, H, 128, 128]``.  Returns the packed output and,
    when asked for, the ``[N, H, 128, 128]`` final states.  Differentiable like ``chunk_gdn2``.
    """

    if not isinstance(q, torch.Tensor) or q.ndim != 4 or q.shape[0] != 1:
        raise ValueError("packed sequence tensors must have shape [1, total, H, 128]")
    bounds = _bounds(cu_seqlens, q.shape[1])
    output_scale = float(scale) if scale is not None else 1.0 / math.sqrt(_DIM)
    if not math.isfinite(output_scale):
        raise ValueError("scale must be finite")
    _validate.sequence_inputs(q, k, v, g, beta, w, need_alignment=True)
    n_seq, heads = len(bounds) - 1, q.shape[2]
    if initial_state is not None:
        _validate.state("initial_state", initial_state, n_seq, heads, q.device, need_alignment=True)
    wants_grad = torch.is_grad_enabled() and any(
        isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v, g, beta, w, initial_state)
    )
    if wants_grad:
        # training: materialise the activated tensors once for the whole packed batch
        if use_qk_l2norm_in_kernel or use_gate_in_kernel:
            q, k, g, beta, w = gate_prologue(q, k, g, beta, w, normalize_qk=use_qk_l2norm_in_kernel,
                                             activate_gates=use_gate_in_kernel)
        output, final_state = _ChunkGDN2Varlen.apply(q, k, v, g, beta, w, initial_state, bounds, output_scale)
    else:
        seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
        output, final_state, _, _ = _packed_forward(
            seq, _validate.detached(initial_state), bounds, output_scale, False,
            _prologue_flags(use_qk_l2norm_in_kernel, use_gate_in_kernel))
    return output, final_state if output_final_state else None


def expand_grouped_heads(q, k, g, beta, value_heads: int):
    """Expand key-shaped tensors ``[B, T, Hk, 128]`` to ``value_heads = Hk * r`` heads.

    Value head ``j`` uses key head ``j // r``.  Returns contiguous ``[B, T, value_heads, 128]``
    tensors; under autograd the gradients of the ``r`` value heads of a group add up in the shared
    key head."""

    key_heads = q.shape[2]
    if value_heads <= 0 or value_heads % key_heads:
        raise ValueError("value_heads must be a positive multiple of the number of key heads")
    repeat = value_heads // key_heads
    if repeat == 1:
        return q, k, g, beta
    return tuple(t.repeat_interleave(repeat, dim=2) for t in (q, k, g, beta))


__all__ = ["chunk_gdn2_varlen", "expand_grouped_heads"]
