"""Host-side argument checks shared by the token, chunk and backward wrappers.

The exception types and the key phrases of the messages follow the reference
(src/gdn2_sm120/recurrent.py:374-433, 451-478; chunk.py:1183-1229, 1265-1316;
backward.py:953-1009) because its tests match on them: everything is rejected in
Python, before any launch, and nothing falls back silently.
"""

from __future__ import annotations

import math
import struct

import torch

from . import _lib

DIM = 128
_SEQ_NAMES = ("q", "k", "v", "g", "beta", "w")
_LOW_PRECISION = (torch.float16, torch.bfloat16)


def sequence_inputs(q, k, v, g, beta, w, *, dim_error=ValueError, need_tokens=False,
                    need_alignment=False):
    """Validate the six ``[B, T, H, 128]`` tensors; return ``(B, T, H)``."""

    seq = (q, k, v, g, beta, w)
    if not all(isinstance(x, torch.Tensor) for x in seq):
        raise TypeError("q, k, v, g, beta, and w must be torch.Tensor objects")
    if any(x.ndim != 4 for x in seq):
        raise ValueError("q, k, v, g, beta, and w must be rank-4 [B, T, H, D] tensors")
    if not (q.shape == k.shape == g.shape == beta.shape):
        raise ValueError("q, k, g, and beta must have identical [B, T, H, K] shapes")
    if v.shape != w.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError("v and w must match each other and q's [B, T, H] dimensions")
    batch, time, heads, key_dim = q.shape
    if key_dim != DIM or v.shape[-1] != DIM:
        raise dim_error("the B200 GDN2 kernels require K == V == 128")
    if batch <= 0 or heads <= 0 or (need_tokens and time <= 0):
        what = "batch, time, and heads" if need_tokens else "batch and heads"
        raise ValueError(f"{what} must be positive")
    if q.dtype not in _LOW_PRECISION:
        raise TypeError("q/k/v/beta/w must use torch.float16 or torch.bfloat16")
    if any(x.dtype != q.dtype for x in (k, v, beta, w)):
        raise TypeError("q, k, v, beta, and w must have the same dtype")
    if g.dtype not in (q.dtype, torch.float32):
        raise TypeError("g must have the input dtype or torch.float32")
    if not all(x.is_cuda for x in seq):
        raise ValueError("all inputs must be CUDA tensors")
    if any(x.device != q.device for x in seq):
        raise ValueError("all inputs must be on the same CUDA device")
    if not all(x.is_contiguous() for x in seq):
        raise ValueError("all inputs must be contiguous")
    if need_alignment and any(x.data_ptr() % 16 for x in seq):
        raise ValueError("all inputs must be 16-byte aligned")
    _lib.require_b200(q.device)
    return batch, time, heads


def state(name: str, tensor, batch: int, heads: int, device, *, need_alignment=False):
    """Validate an fp32 ``[B, H, 128, 128]`` state tensor."""

    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor or None")
    expected = (batch, heads, DIM, DIM)
    if tuple(tensor.shape) != expected:
        raise ValueError(f"{name} must have shape {expected}")
    if tensor.dtype != torch.float32:
        raise TypeError(f"{name} must use torch.float32")
    if tensor.device != device:
        raise ValueError(f"{name} must be on the same CUDA device as q")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if need_alignment and tensor.data_ptr() % 16:
        raise ValueError(f"{name} must be 16-byte aligned")


def buffer(name: str, tensor, shape, dtype, device, *, need_alignment=False):
    """Validate a caller-provided output buffer."""

    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor or None")
    if tuple(tensor.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}")
    if tensor.dtype != dtype:
        raise TypeError(f"{name} must use {dtype}")
    if tensor.device != device:
        raise ValueError(f"{name} must be on the same CUDA device as q")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if need_alignment and tensor.data_ptr() % 16:
        raise ValueError(f"{name} must be 16-byte aligned for the chunk path")


def float32_scale(scale, dim: int = DIM) -> float:
    """Default 1/sqrt(dim); reject values that are not finite once rounded to fp32."""

    value = float(scale) if scale is not None else 1.0 / math.sqrt(dim)
    if not math.isfinite(value):
        raise ValueError("scale must be finite")
    try:
        rounded = struct.unpack("=f", struct.pack("=f", value))[0]
    except OverflowError as exc:
        raise ValueError("scale must be representable as float32") from exc
    if not math.isfinite(rounded):
        raise ValueError("scale must be representable as float32 (finite after rounding)")
    return rounded


def byte_span(tensor: torch.Tensor) -> tuple[int, int]:
    """Half-open byte interval of a contiguous tensor."""

    lo = tensor.data_ptr()
    return lo, lo + tensor.numel() * tensor.element_size()


def spans_overlap(left: tuple[int, int], right: tuple[int, int]) -> bool:
    """True when two non-empty half-open intervals intersect."""

    if left[0] >= left[1] or right[0] >= right[1]:
        return False
    return left[0] < right[1] and right[0] < left[1]


def detached(tensor):
    """Storage-sharing view without an autograd edge (``None`` passes through)."""

    if tensor is None or not tensor.requires_grad:
        return tensor
    return tensor.detach()
