"""Launch glue for the 64-token tensor-core chunk kernels (forward and backward).

``supported_tokens`` tells the host wrappers how many leading tokens of a sequence the
chunk kernels take; the remaining tail goes to the token kernels.
"""

from __future__ import annotations

_CHUNK = 64

# Entry points of the C ABI that implement the chunk path.  Until they exist in the
# loaded library the token kernels process whole sequences.
FORWARD_AVAILABLE = False
BACKWARD_AVAILABLE = False


def supported_tokens(time: int) -> int:
    if not FORWARD_AVAILABLE:
        return 0
    return (time // _CHUNK) * _CHUNK


def forward(q, k, v, g, beta, w, initial_state, output, final_state, chunk_boundaries,
            batch, time, heads, full_tokens, scale) -> None:
    raise RuntimeError("the tensor-core chunk forward is not built into this library")


def backward(*args, **kwargs) -> None:
    raise RuntimeError("the tensor-core chunk backward is not built into this library")
