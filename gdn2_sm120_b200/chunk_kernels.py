"""Launch glue for the 64-token tensor-core chunk kernels (forward and backward).

``supported_tokens`` tells the host wrappers how many leading tokens of a sequence the
chunk kernels take; the remaining ragged tail goes to the token kernels.  The workspace
that holds the per-chunk WY factors is allocated here with torch (so the caching
allocator and stream semantics apply) after asking the C ABI for its size.
"""

from __future__ import annotations

import torch

from . import _lib

_CHUNK = 64

# Set to False to force whole sequences onto the exact fp32 token kernels.
FORWARD_ENABLED = True
BACKWARD_ENABLED = True


def _has(symbol: str) -> bool:
    return hasattr(_lib.lib(), symbol)


def supported_tokens(time: int, *, training: bool = False) -> int:
    """Leading tokens the chunk kernels process (a multiple of 64, possibly 0)."""

    if not FORWARD_ENABLED or not _has("gdn2_chunk_forward"):
        return 0
    if training and not (BACKWARD_ENABLED and _has("gdn2_chunk_backward")):
        return 0
    return (time // _CHUNK) * _CHUNK


def workspace_bytes(batch: int, full_tokens: int, heads: int, training: bool = False) -> int:
    size = _lib.lib().gdn2_chunk_workspace_bytes(batch, full_tokens, heads, int(training))
    if size <= 0:
        raise RuntimeError(f"gdn2_chunk_workspace_bytes failed with status {size}")
    return int(size)


def forward(q, k, v, g, beta, w, initial_state, output, final_state, chunk_boundaries,
            batch, time, heads, full_tokens, scale) -> torch.Tensor:
    """Run the chunk forward over tokens [0, full_tokens); returns the workspace."""

    training = chunk_boundaries is not None
    workspace = torch.empty(workspace_bytes(batch, full_tokens, heads, training), device=q.device,
                            dtype=torch.uint8)
    _lib.call(
        "gdn2_chunk_forward", q.device,
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
        _lib.ptr(initial_state), output.data_ptr(), _lib.ptr(final_state), _lib.ptr(chunk_boundaries),
        workspace.data_ptr(), batch, time, heads, full_tokens, int(training),
        _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale, _lib.stream_ptr(q.device),
    )
    return workspace


def read_status(workspace: torch.Tensor, batch: int, full_tokens: int, heads: int) -> int:
    """Synchronise the current stream and return the workspace's device status word."""

    with torch.cuda.device(workspace.device):
        return int(_lib.lib().gdn2_chunk_read_status(
            workspace.data_ptr(), batch, full_tokens, heads, _lib.stream_ptr(workspace.device)))


def backward(q, k, v, g, beta, w, workspace, chunk_boundaries, d_out, d_final_state, grads,
             d_initial_state, batch, time, heads, full_tokens, scale) -> None:
    """Chunk backward over tokens [0, full_tokens): fills rows of ``grads`` and ``d_initial_state``."""

    dq, dk, dv, dg, dbeta, dw = grads
    d_boundaries = torch.empty_like(chunk_boundaries)
    _lib.call(
        "gdn2_chunk_backward", q.device,
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), w.data_ptr(),
        d_out.data_ptr(), _lib.ptr(d_final_state), chunk_boundaries.data_ptr(), d_boundaries.data_ptr(),
        workspace.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(),
        dbeta.data_ptr(), dw.data_ptr(), _lib.ptr(d_initial_state),
        batch, time, heads, full_tokens,
        _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype), scale, _lib.stream_ptr(q.device),
    )
