"""Fused input prologue: q/k L2 normalisation and gate activations in one kernel, with its VJP.

The reference's primitive expects already-normalised q/k and already-activated gates and leaves
those steps to the caller (README.md:127-131, docs/design.md:32-34 of the reference); the official
implementation it is benchmarked against takes them as ``use_qk_l2norm_in_kernel`` /
``use_gate_in_kernel`` (src/gdn2_sm120/benchmark.py:230-231).  ``chunk_gdn2`` and
``recurrent_gdn2`` accept the same two keywords here (default off): the raw tensors then go through
``gate_prologue`` -- one memory-bound pass instead of a dozen elementwise launches -- before the
primitive, and the cotangents through its VJP kernel afterwards (in place).

    q = q_raw / sqrt(sum(q_raw^2) + 1e-6)       k likewise
    beta = sigmoid(beta_raw)    w = sigmoid(w_raw)    g = -softplus(g_raw)
"""

from __future__ import annotations

import torch

from . import _lib, _validate


def _launch_forward(q, k, g, beta, w, normalize_qk, activate_gates):
    batch, time, heads, _ = q.shape
    rows = (batch, time, heads)
    outs = [torch.empty_like(t) if on else t for t, on in
            ((q, normalize_qk), (k, normalize_qk), (g, activate_gates), (beta, activate_gates), (w, activate_gates))]
    inv_q = inv_k = None
    if normalize_qk:
        inv_q = torch.empty(rows, device=q.device, dtype=torch.float32)
        inv_k = torch.empty(rows, device=q.device, dtype=torch.float32)
    if time > 0:
        n, a = normalize_qk, activate_gates
        _lib.call(
            "gdn2_gate_prologue", q.device,
            q.data_ptr() if n else None, k.data_ptr() if n else None, g.data_ptr() if a else None,
            beta.data_ptr() if a else None, w.data_ptr() if a else None,
            outs[0].data_ptr() if n else None, outs[1].data_ptr() if n else None,
            outs[2].data_ptr() if a else None, outs[3].data_ptr() if a else None, outs[4].data_ptr() if a else None,
            _lib.ptr(inv_q), _lib.ptr(inv_k), batch, time, heads,
            _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), _lib.stream_ptr(q.device),
        )
    return outs, inv_q, inv_k


class _GatePrologue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, g, beta, w, normalize_qk: bool, activate_gates: bool):
        raw = tuple(_validate.detached(t) for t in (q, k, g, beta, w))
        outs, inv_q, inv_k = _launch_forward(*raw, normalize_qk, activate_gates)
        ctx.normalize_qk, ctx.activate_gates = normalize_qk, activate_gates
        saved = [q, k, g, beta, w]
        if normalize_qk:
            saved += [inv_q, inv_k]
        ctx.save_for_backward(*saved)
        ctx.set_materialize_grads(False)
        # tensors the prologue leaves alone are returned as they came
        return tuple(o if on else t for o, t, on in zip(
            outs, (q, k, g, beta, w), (normalize_qk, normalize_qk, activate_gates, activate_gates, activate_gates)))

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dq, dk, dg, dbeta, dw):
        q, k, g, beta, w, *inv = ctx.saved_tensors
        n, a = ctx.normalize_qk, ctx.activate_gates
        batch, time, heads, _ = q.shape

        def ready(grad, like):
            if grad is None:
                return torch.zeros_like(like)
            return grad if grad.is_contiguous() else grad.contiguous()

        grads = [ready(dq, q), ready(dk, k), ready(dg, g), ready(dbeta, beta), ready(dw, w)]
        outs = [torch.empty_like(x) for x in grads]
        if time > 0:
            raw = tuple(_validate.detached(t) for t in (q, k, g, beta, w))
            _lib.call(
                "gdn2_gate_prologue_vjp", q.device,
                raw[0].data_ptr() if n else None, raw[1].data_ptr() if n else None,
                raw[2].data_ptr() if a else None, raw[3].data_ptr() if a else None, raw[4].data_ptr() if a else None,
                inv[0].data_ptr() if n else None, inv[1].data_ptr() if n else None,
                grads[0].data_ptr() if n else None, grads[1].data_ptr() if n else None,
                grads[2].data_ptr() if a else None, grads[3].data_ptr() if a else None,
                grads[4].data_ptr() if a else None,
                outs[0].data_ptr() if n else None, outs[1].data_ptr() if n else None,
                outs[2].data_ptr() if a else None, outs[3].data_ptr() if a else None,
                outs[4].data_ptr() if a else None,
                batch, time, heads, _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), _lib.stream_ptr(q.device),
            )
        result = [o if on else gr for o, gr, on in zip(outs, grads, (n, n, a, a, a))]
        return (*result, None, None)


def gate_prologue(q, k, g, beta, w, *, normalize_qk: bool = True, activate_gates: bool = True):
    """Return ``(q, k, g, beta, w)`` normalised / activated as the flags say (differentiable).

    Inputs are the raw projections of a layer: contiguous ``[B, T, H, 128]``; q/k/beta/w fp16 or
    bf16, ``g`` the same type or fp32.  With both flags off the inputs are returned unchanged."""

    if not (normalize_qk or activate_gates):
        return q, k, g, beta, w
    # beta / w / v share the value-shaped layout checks of the primitive; v is not touched here
    _validate.sequence_inputs(q, k, w, g, beta, w, need_alignment=True)
    wants_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, g, beta, w))
    if wants_grad:
        return _GatePrologue.apply(q, k, g, beta, w, bool(normalize_qk), bool(activate_gates))
    raw = tuple(_validate.detached(t) for t in (q, k, g, beta, w))
    outs, _, _ = _launch_forward(*raw, bool(normalize_qk), bool(activate_gates))
    return tuple(outs)


__all__ = ["gate_prologue"]
