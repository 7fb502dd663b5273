"""Readable PyTorch definitions of the primitive (device-agnostic, differentiable).

Part of the public surface because the reference exports the same two names
(src/gdn2_sm120/__init__.py:9-18, reference.py:47-179).  They are *not* used by any
kernel path of this package; they exist so that user code which calls
``recurrent_forward_reference`` / ``chunkwise_forward_reference`` keeps working.

Conventions: ``g <= 0`` is a log-decay (the decay is ``exp(g)``), sequence tensors are
``[B, T, H, D]``, states ``[B, H, K, V]``.  Like the reference the arithmetic runs in
float32 by default whatever the input type; ``compute_dtype=torch.float64`` gives a
double-precision evaluation.  The output is cast to ``q.dtype``; the state keeps the
compute type.
"""

from __future__ import annotations

import math

import torch


def _dims(q, k, v, g, beta, w, initial_state):
    if q.ndim != 4 or v.ndim != 4:
        raise ValueError("q/k/g/beta and v/w must be rank-4 [B, T, H, D] tensors")
    if not (q.shape == k.shape == g.shape == beta.shape):
        raise ValueError("q, k, g, and beta must have identical shapes")
    if v.shape != w.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError("v and w must match each other and q's [B, T, H] dimensions")
    if any(x.device != q.device for x in (k, v, g, beta, w)):
        raise ValueError("all inputs must be on the same device")
    b, t, h, kd = q.shape
    vd = v.shape[-1]
    if initial_state is not None and tuple(initial_state.shape) != (b, h, kd, vd):
        raise ValueError(f"initial_state must have shape [B, H, K, V] = {(b, h, kd, vd)}")
    return b, t, h, kd, vd


def _start_state(initial_state, b, h, kd, vd, device, dtype):
    if initial_state is None:
        return torch.zeros((b, h, kd, vd), device=device, dtype=dtype)
    return initial_state.to(dtype)


def recurrent_forward_reference(q, k, v, g, beta, w, initial_state=None, *, scale=None,
                                return_final_state=True, compute_dtype=torch.float32):
    """Token recurrence: X = exp(g) S; S = X + k (w v - X^T (beta k))^T; o = S^T (scale q)."""

    b, t, h, kd, vd = _dims(q, k, v, g, beta, w, initial_state)
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(kd)
    ct = compute_dtype
    s = _start_state(initial_state, b, h, kd, vd, q.device, ct)
    rows = []
    for i in range(t):
        k_i = k[:, i].to(ct)
        x = g[:, i].to(ct).exp()[..., None] * s
        erased = torch.einsum("bhk,bhkv->bhv", beta[:, i].to(ct) * k_i, x)
        s = x + k_i[..., None] * (w[:, i].to(ct) * v[:, i].to(ct) - erased)[..., None, :]
        rows.append(torch.einsum("bhk,bhkv->bhv", q[:, i].to(ct) * sc, s))
    out = (
        torch.stack(rows, dim=1).to(q.dtype)
        if rows
        else torch.empty((b, 0, h, vd), device=q.device, dtype=q.dtype)
    )
    return out, (s if return_final_state else None)


def chunkwise_forward_reference(q, k, v, g, beta, w, initial_state=None, *, scale=None,
                                chunk_size=64, return_final_state=True,
                                compute_dtype=torch.float32):
    """Compact-WY chunk form of the same recurrence (one triangular solve per chunk)."""

    b, t, h, kd, vd = _dims(q, k, v, g, beta, w, initial_state)
    if chunk_size <= 0:
        raise ValueError("chunk_size must be positive")
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(kd)
    ct = compute_dtype
    s = _start_state(initial_state, b, h, kd, vd, q.device, ct)
    blocks = []
    for lo in range(0, t, chunk_size):
        hi = min(t, lo + chunk_size)
        qc, kc, vc, gc, bc, wc = (z[:, lo:hi].permute(0, 2, 1, 3).to(ct) for z in (q, k, v, g, beta, w))
        log_gamma = torch.cumsum(gc, dim=2)
        gamma = log_gamma.exp()
        k_over = kc * (-log_gamma).exp()
        erase = bc * kc * gamma
        strict = torch.tril(erase @ k_over.mT, diagonal=-1)
        system = strict + torch.eye(hi - lo, device=q.device, dtype=ct)
        rhs = torch.cat([erase, wc * vc], dim=-1)
        sol = torch.linalg.solve_triangular(system, rhs, upper=False, unitriangular=True)
        y, u = sol[..., :kd], sol[..., kd:]
        resid = u - y @ s
        q_gamma = qc * gamma * sc
        blocks.append((q_gamma @ s + torch.tril(q_gamma @ k_over.mT) @ resid).permute(0, 2, 1, 3))
        end = gamma[:, :, -1]
        s = end[..., None] * s + (k_over * end[:, :, None]).mT @ resid
    out = (
        torch.cat(blocks, dim=1).to(q.dtype)
        if blocks
        else torch.empty((b, 0, h, vd), device=q.device, dtype=q.dtype)
    )
    return out, (s if return_final_state else None)


__all__ = ["chunkwise_forward_reference", "recurrent_forward_reference"]
