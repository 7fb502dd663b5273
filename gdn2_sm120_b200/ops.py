"""Public PyTorch operators: ``chunk_gdn2`` and ``recurrent_gdn2``.

Drop-in for src/gdn2_sm120/ops.py:224-327 of the reference: identical signatures,
defaults, return conventions, grad-mode detection (inference bypasses the
``autograd.Function``), hidden-final-state handling (no zero cotangent is materialised
when the loss ignores ``S_T``) and T == 0 behaviour.  Device work goes through the C ABI
on the current PyTorch stream of the tensors' device.
"""

from __future__ import annotations

import math

import torch

from . import _validate
from .backward import backward_from_aux
from .chunk import ChunkForwardAux, _token_slots, chunk_forward
from .prologue import gate_prologue
from .recurrent import _launch_token_forward, _use_recurrent_kernel, token_forward

_DIM = 128
_CHUNK_SIZE = 64
_PARALLEL_BACKWARD_MIN_TOKENS = 64


def _prologue_flags(normalize_qk: bool, activate_gates: bool) -> int:
    """Bit flags of the fused prologue (GDN2_PROLOGUE_NORMALIZE_QK = 1, GDN2_PROLOGUE_ACTIVATE_GATES = 2)."""

    return (1 if normalize_qk else 0) | (2 if activate_gates else 0)


def _use_compact_wy_backward(batch: int, time: int, heads: int) -> bool:
    """True when backward runs the tensor-core compact-WY chunk VJP for the leading
    full chunks (reference selector: src/gdn2_sm120/ops.py:22-28).

    The reference needs T >= 128, or T == 64 on a grid large enough to fill its GPU,
    because its VJP is a 10-12 launch graph.  The B200 VJP is a fused kernel per
    direction, so one full 64-token chunk is enough regardless of the grid.
    """

    del batch, heads
    return time >= _PARALLEL_BACKWARD_MIN_TOKENS


def _forward_with_aux(seq, state, scale: float, prepare_backward: bool, prologue: int = 0):
    """Forward of one (detached) problem on the shape-dispatched kernels.

    Returns ``(output, final_state, aux)``; ``aux`` (the checkpoints backward consumes) is ``None``
    unless ``prepare_backward`` and the sequence is not empty.  ``prologue`` (inference only) makes
    the forward kernels apply the layer prologue to raw inputs."""

    q = seq[0]
    batch, time, heads = q.shape[0], q.shape[1], q.shape[2]
    aux = None
    if _use_recurrent_kernel(batch, time, heads, chunk_api=True):
        if prepare_backward and time > 0:
            # token path with fp32 checkpoints every 16 tokens
            batch, time, heads = _validate.sequence_inputs(*seq)
            if state is not None:
                _validate.state("initial_state", state, batch, heads, q.device)
            output = torch.empty_like(seq[2])
            final_state = torch.empty((batch, heads, _DIM, _DIM), device=q.device, dtype=torch.float32)
            boundaries = torch.empty((batch, _token_slots(time), heads, _DIM, _DIM),
                                     device=q.device, dtype=torch.float32)
            _launch_token_forward(*seq, state, output, final_state, boundaries, batch, time,
                                  heads, 0, time, _validate.float32_scale(scale))
            aux = ChunkForwardAux(None, boundaries, 0)
        else:
            output, final_state = token_forward(*seq, state, scale=scale, prologue=prologue)
    elif prepare_backward:
        output, final_state, aux = chunk_forward(*seq, state, scale=scale, return_aux=True)
    else:
        output, final_state = chunk_forward(*seq, state, scale=scale, prologue=prologue)
    return output, final_state, aux


def _aux_tensors(aux) -> tuple[list, tuple[int, int, int, int]]:
    """Flatten an aux bundle for ``save_for_backward``: tensors and (counts..., full_tokens)."""

    if aux is None:
        return [], (0, 0, 0, 0)
    tensors, counts = [], []
    for item in (aux.chunk_boundaries, aux.tail_boundaries):
        counts.append(0 if item is None else 1)
        if item is not None:
            tensors.append(item)
    workspaces = aux.workspace or ()
    tensors.extend(workspaces)
    return tensors, (counts[0], counts[1], len(workspaces), aux.full_tokens)


def _aux_from_tensors(tensors: list, layout: tuple[int, int, int, int]) -> ChunkForwardAux:
    n_chunk, n_tail, n_ws, full_tokens = layout
    tensors = list(tensors)
    chunk_boundaries = tensors.pop(0) if n_chunk else None
    tail_boundaries = tensors.pop(0) if n_tail else None
    workspace = tuple(tensors[:n_ws]) if n_ws else None
    return ChunkForwardAux(chunk_boundaries, tail_boundaries, full_tokens, workspace)


class _ChunkGDN2(torch.autograd.Function):
    """Connects the forward kernels, their state checkpoints and the backward kernels."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, w, initial_state, scale: float, prepare_backward: bool):
        seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
        state = _validate.detached(initial_state)
        output, final_state, aux = _forward_with_aux(seq, state, scale, prepare_backward)
        tensors, ctx.aux_layout = _aux_tensors(aux)
        ctx.save_for_backward(q, k, v, g, beta, w, *tensors)
        ctx.set_materialize_grads(False)
        ctx.has_initial_state = initial_state is not None
        ctx.scale = scale
        return output, final_state

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_output, d_final_state):
        q, k, v, g, beta, w, *saved = ctx.saved_tensors
        if q.shape[1] == 0:
            empty = tuple(torch.empty_like(x) for x in (q, k, v, g, beta, w))
            d_state = None
            if ctx.has_initial_state:
                d_state = (
                    torch.zeros((q.shape[0], q.shape[2], _DIM, _DIM), device=q.device,
                                dtype=torch.float32)
                    if d_final_state is None
                    else d_final_state.contiguous().clone()
                )
            return (*empty, d_state, None, None)
        if d_output is None:
            d_output = torch.zeros_like(v)
        elif not d_output.is_contiguous():
            d_output = d_output.contiguous()
        if d_final_state is not None and not d_final_state.is_contiguous():
            d_final_state = d_final_state.contiguous()
        aux = _aux_from_tensors(saved, ctx.aux_layout)
        seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
        *sequence_grads, d_initial_state = backward_from_aux(
            *seq, aux, d_output, d_final_state, _validate.float32_scale(ctx.scale)
        )
        return (*sequence_grads, d_initial_state if ctx.has_initial_state else None, None, None)


def chunk_gdn2(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    w: torch.Tensor,
    initial_state: torch.Tensor | None = None,
    *,
    scale: float | None = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    use_gate_in_kernel: bool = False,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Gated DeltaNet-2 with shape-dispatched forward and native backward.

    Sequence tensors are contiguous ``[B, T, H, 128]``; q/k/v/beta/w fp16 or bf16, ``g``
    additionally fp32; states fp32 ``[B, H, 128, 128]``.  By default (as in the reference) gate
    activations and q/k normalisation stay with the caller and ``g`` must be finite and
    non-positive with every 16-token prefix sum above ln(FLT_MIN).  With
    ``use_qk_l2norm_in_kernel`` q and k are the raw projections and are L2-normalised first; with
    ``use_gate_in_kernel`` beta, w and g are pre-activations (beta = sigmoid, w = sigmoid,
    g = -softplus).  Without gradients the forward kernels apply both themselves as they load the
    inputs; a call that needs gradients runs them as one fused kernel in front of the primitive
    and one behind its backward (``prologue.gate_prologue``).  Returns ``(o, S_T)`` or ``(o, None)``.
    """

    output_scale = float(scale) if scale is not None else 1.0 / math.sqrt(_DIM)
    if not math.isfinite(output_scale):
        raise ValueError("scale must be finite")
    wants_grad = torch.is_grad_enabled() and any(
        isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v, g, beta, w, initial_state)
    )
    if wants_grad:
        # training: the activated tensors are what backward differentiates, so they are materialised
        if use_qk_l2norm_in_kernel or use_gate_in_kernel:
            q, k, g, beta, w = gate_prologue(q, k, g, beta, w, normalize_qk=use_qk_l2norm_in_kernel,
                                             activate_gates=use_gate_in_kernel)
        output, final_state = _ChunkGDN2.apply(q, k, v, g, beta, w, initial_state, output_scale, True)
        return output, final_state if output_final_state else None

    # inference: the forward kernels apply the prologue themselves
    prologue = _prologue_flags(use_qk_l2norm_in_kernel, use_gate_in_kernel)
    seq = tuple(_validate.detached(x) for x in (q, k, v, g, beta, w))
    state = _validate.detached(initial_state)
    if _use_recurrent_kernel(q.shape[0], q.shape[1], q.shape[2], chunk_api=True):
        output, final_state = token_forward(*seq, state, scale=output_scale, prologue=prologue)
    else:
        output, final_state = chunk_forward(*seq, state, scale=output_scale, return_aux=False, prologue=prologue)
    return output, final_state if output_final_state else None


def recurrent_gdn2(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    w: torch.Tensor,
    initial_state: torch.Tensor | None = None,
    *,
    scale: float | None = None,
    out: torch.Tensor | None = None,
    final_state_out: torch.Tensor | None = None,
    inplace_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    use_gate_in_kernel: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Forward-only GDN2 for serving, with the recurrent/chunk crossover.

    With the two ``use_*_in_kernel`` keywords (default off) the inputs are raw projections / gate
    pre-activations and the decode and prefill kernels apply the prologue as they load them."""

    return token_forward(q, k, v, g, beta, w, initial_state, scale=scale, out=out,
                         final_state_out=final_state_out, inplace_final_state=inplace_final_state,
                         prologue=_prologue_flags(use_qk_l2norm_in_kernel, use_gate_in_kernel))


__all__ = ["chunk_gdn2", "recurrent_gdn2"]
