"""Launch glue for the 64-token tensor-core chunk kernels (forward and backward).

Buffers are allocated here with torch (so the caching allocator and stream semantics apply)
after asking the C ABI for their sizes:

  workspace   what a training forward leaves for backward (160 KiB per 64-token chunk and head;
              an inference call's holds the chunk-end decays and a status word only)
  scratch     tiles that live inside one call (forward 144 KiB, backward 36 KiB per chunk-head)
  cotangent checkpoints of backward (64 KiB per chunk-head), also dead when the call returns

A large batch is processed as *waves* of consecutive batch rows: every wave is one call of the
entry point on a batch slice, all waves of a pass share one scratch buffer (they run one after
another on the stream), and each wave keeps a workspace of its own for backward.  The wave size
is the largest one whose scratch stays under ``SCRATCH_BUDGET_BYTES``; a batch that fits runs as
a single wave, which is the fastest form.  The reference has no counterpart: its intermediates
are sequence-sized allocations per call (src/gdn2_sm120/chunk.py:1317-1362) and a shape whose
checkpoints pass 4 GiB is rejected (chunk.py:1236-1248).
"""

from __future__ import annotations

import torch

from . import _lib

_CHUNK = 64
_STATE_BYTES = 128 * 128 * 4

# Upper bound on the scratch of one wave (forward tiles, or backward tiles plus cotangent checkpoints).
SCRATCH_BUDGET_BYTES = 12 << 30
# Requests below this size skip the free-memory check.
CHECK_MEMORY_MIN_BYTES = 16 << 30


def supported_tokens(time: int, *, training: bool = False) -> int:
    """Tokens the chunk kernels process (a multiple of 64: 0 below 64 tokens, else ``time`` rounded up)."""

    del training
    return 0 if time < _CHUNK else -(-time // _CHUNK) * _CHUNK


def workspace_bytes(batch: int, full_tokens: int, heads: int, training: bool = False) -> int:
    size = _lib.lib().gdn2_chunk_workspace_bytes(batch, full_tokens, heads, int(training))
    if size <= 0:
        raise RuntimeError(f"gdn2_chunk_workspace_bytes failed with status {size}")
    return int(size)


def scratch_bytes(batch: int, full_tokens: int, heads: int, backward: bool = False, *,
                  training: bool = False) -> int:
    """Per-call scratch: of a backward pass, or of the forward of an inference / a training call (a
    training forward keeps the tiles both scans read in its workspace, so its scratch is smaller)."""

    kind = 1 if backward else (2 if training else 0)
    size = _lib.lib().gdn2_chunk_scratch_bytes(batch, full_tokens, heads, kind)
    if size <= 0:
        raise RuntimeError(f"gdn2_chunk_scratch_bytes failed with status {size}")
    return int(size)


def _backward_wave_bytes(batch: int, full_tokens: int, heads: int) -> int:
    """Scratch of one backward wave: dZ tiles plus the cotangent checkpoints."""

    return scratch_bytes(batch, full_tokens, heads, True) + batch * (full_tokens // _CHUNK + 1) * heads * _STATE_BYTES


def plan_waves(batch: int, full_tokens: int, heads: int, *, backward: bool = False, training: bool = False,
               budget: int | None = None) -> list[tuple[int, int]]:
    """Batch ranges ``[(b0, b1), ...]`` of the waves of one pass."""

    budget = SCRATCH_BUDGET_BYTES if budget is None else budget
    if backward:
        per_row = _backward_wave_bytes(1, full_tokens, heads)
    elif training:
        # backward runs over the same waves (a workspace belongs to one wave): the larger of the two
        # transients, the backward one (dZ tiles and cotangent checkpoints), sets the wave size
        per_row = max(scratch_bytes(1, full_tokens, heads, False, training=True),
                      _backward_wave_bytes(1, full_tokens, heads))
    else:
        per_row = scratch_bytes(1, full_tokens, heads, False)
    rows = max(1, min(batch, budget // per_row))
    # equal-sized waves (the last one may be smaller by at most one row per wave)
    n_waves = -(-batch // rows)
    rows = -(-batch // n_waves)
    return [(b0, min(batch, b0 + rows)) for b0 in range(0, batch, rows)]


def check_memory(needed: int, device: torch.device, what: str) -> None:
    """Fail with a clear message instead of an out-of-memory error in the middle of a pass."""

    # Asking the driver for the free memory costs about a millisecond: only requests large enough for
    # that not to matter are checked, the rest is left to the allocator.  Nothing may be queried
    # while a stream is being captured.
    if needed < CHECK_MEMORY_MIN_BYTES or torch.cuda.is_current_stream_capturing():
        return
    free, _ = torch.cuda.mem_get_info(device)
    if needed <= free:
        return
    # memory torch's caching allocator holds but does not use counts as free too
    free += max(0, torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device))
    if needed > free:
        raise ValueError(
            f"{what} needs {needed} bytes ({needed / 2**30:.1f} GiB) of device memory for workspaces and "
            f"state checkpoints but only {free} bytes ({free / 2**30:.1f} GiB) are free; "
            "reduce the batch or the sequence length, or shard over more GPUs"
        )


def forward(q, k, v, g, beta, w, initial_state, output, final_state, chunk_boundaries,
            batch, time, heads, full_tokens, scale, *, prologue: int = 0) -> tuple[torch.Tensor, ...]:
    """Run the chunk forward over tokens [0, full_tokens); returns one workspace per wave.

    ``prologue`` != 0 (inference only) selects the entry point whose prep kernel activates raw inputs."""

    training = chunk_boundaries is not None
    if prologue and training:
        raise ValueError("the fused prologue is forward-only")
    waves = plan_waves(batch, full_tokens, heads, training=training)
    rows = waves[0][1] - waves[0][0]
    scratch_size = scratch_bytes(rows, full_tokens, heads, False, training=training)
    needed = scratch_size + sum(workspace_bytes(b1 - b0, full_tokens, heads, training) for b0, b1 in waves)
    check_memory(needed, q.device, "chunk forward")
    scratch = torch.empty(scratch_size, device=q.device, dtype=torch.uint8)
    dtype, g_dtype = _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype)
    stream = _lib.stream_ptr(q.device)
    workspaces = []
    for b0, b1 in waves:
        workspace = torch.empty(workspace_bytes(b1 - b0, full_tokens, heads, training), device=q.device,
                                dtype=torch.uint8)
        common = [
            q[b0:b1].data_ptr(), k[b0:b1].data_ptr(), v[b0:b1].data_ptr(), g[b0:b1].data_ptr(),
            beta[b0:b1].data_ptr(), w[b0:b1].data_ptr(),
            None if initial_state is None else initial_state[b0:b1].data_ptr(),
            output[b0:b1].data_ptr(), None if final_state is None else final_state[b0:b1].data_ptr(),
        ]
        if prologue:
            _lib.call("gdn2_chunk_forward_fused", q.device, *common, workspace.data_ptr(), scratch.data_ptr(),
                      b1 - b0, time, heads, full_tokens, dtype, g_dtype, scale, prologue, stream)
        else:
            _lib.call(
                "gdn2_chunk_forward", q.device, *common,
                None if chunk_boundaries is None else chunk_boundaries[b0:b1].data_ptr(),
                workspace.data_ptr(), scratch.data_ptr(), b1 - b0, time, heads, full_tokens, int(training),
                dtype, g_dtype, scale, stream,
            )
        workspaces.append(workspace)
    return tuple(workspaces)


def read_status(workspace, batch: int, full_tokens: int, heads: int) -> int:
    """Synchronise the current stream and return the device status word (the largest one over the
    waves when given the tuple ``forward`` returned)."""

    if isinstance(workspace, torch.Tensor):
        with torch.cuda.device(workspace.device):
            return int(_lib.lib().gdn2_chunk_read_status(
                workspace.data_ptr(), batch, full_tokens, heads, _lib.stream_ptr(workspace.device)))
    worst = 0
    waves = plan_waves(batch, full_tokens, heads)
    if len(waves) != len(workspace):  # the workspaces of a training call
        waves = plan_waves(batch, full_tokens, heads, training=True)
    for (b0, b1), ws in zip(waves, workspace):
        worst = max(worst, read_status(ws, b1 - b0, full_tokens, heads))
    return worst


def backward(q, k, v, g, beta, w, workspaces, chunk_boundaries, d_out, d_final_state, grads,
             d_initial_state, batch, time, heads, full_tokens, scale, *, f32_grads: bool = False,
             keep_d_boundaries: bool = False):
    """Chunk backward over tokens [0, full_tokens): fills rows of ``grads`` and ``d_initial_state``.

    ``workspaces`` is what ``forward`` returned.  ``f32_grads`` selects the test entry point that
    writes fp32 dq, dk, dv, dbeta, dw; ``keep_d_boundaries`` returns the cotangent checkpoints and
    the backward scratch of the (single) wave for inspection by tests."""

    dq, dk, dv, dg, dbeta, dw = grads
    forward_waves = plan_waves(batch, full_tokens, heads, training=True)
    if len(forward_waves) != len(workspaces):
        raise ValueError("workspaces do not match the wave plan of this shape")
    n_slots = full_tokens // _CHUNK + 1
    # backward runs over the forward's waves (a workspace belongs to one wave; plan_waves sized them
    # for the backward transients)
    dtype, g_dtype = _lib.dtype_code(q.dtype), _lib.dtype_code(g.dtype)
    stream = _lib.stream_ptr(q.device)
    rows = max(b1 - b0 for b0, b1 in forward_waves)
    check_memory(_backward_wave_bytes(rows, full_tokens, heads), q.device, "chunk backward")
    scratch = torch.empty(scratch_bytes(rows, full_tokens, heads, True), device=q.device, dtype=torch.uint8)
    d_boundaries = torch.empty((rows, n_slots, heads, 128, 128), device=q.device, dtype=torch.float32)
    name = "gdn2_chunk_backward_f32grads" if f32_grads else "gdn2_chunk_backward"
    for (b0, b1), workspace in zip(forward_waves, workspaces):
        args = [
            q[b0:b1].data_ptr(), k[b0:b1].data_ptr(), v[b0:b1].data_ptr(), g[b0:b1].data_ptr(),
            beta[b0:b1].data_ptr(), w[b0:b1].data_ptr(), d_out[b0:b1].data_ptr(),
            None if d_final_state is None else d_final_state[b0:b1].data_ptr(),
            chunk_boundaries[b0:b1].data_ptr(), d_boundaries.data_ptr(), workspace.data_ptr(),
            scratch.data_ptr(), dq[b0:b1].data_ptr(), dk[b0:b1].data_ptr(), dv[b0:b1].data_ptr(),
            dg[b0:b1].data_ptr(), dbeta[b0:b1].data_ptr(), dw[b0:b1].data_ptr(),
            None if d_initial_state is None else d_initial_state[b0:b1].data_ptr(),
            b1 - b0, time, heads, full_tokens,
        ]
        if not f32_grads:
            args += [dtype, g_dtype]
        _lib.call(name, q.device, *args, scale, stream)
    if keep_d_boundaries:
        return d_boundaries, scratch
    return None
