"""B200 (sm_100a) Gated DeltaNet-2 kernels behind the gdn2-sm120 Python API."""

from .backward import MAX_BACKWARD_TOKENS, chunk_backward
from .chunk import chunk_forward
from .ops import chunk_gdn2, recurrent_gdn2
from .recurrent import token_forward
from .reference import chunkwise_forward_reference, recurrent_forward_reference

__all__ = [
    "chunk_backward",
    "chunk_forward",
    "chunk_gdn2",
    "chunkwise_forward_reference",
    "recurrent_forward_reference",
    "recurrent_gdn2",
    "token_forward",
    "MAX_BACKWARD_TOKENS",
]
__version__ = "0.1.0"
