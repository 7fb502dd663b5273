"""ctypes binding of ``libgdn2_b200.so`` (the C ABI declared in include/gdn2_b200.h).

This replaces the reference's TVM-FFI executor cache
(src/gdn2_sm120/recurrent.py:510-573, chunk.py:1089-1157): there is no JIT, shapes
are run-time arguments, and the only thing cached is the loaded library handle.
There is deliberately no fallback: if the shared object is missing or a call
fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import pathlib
import threading

import torch

_PACKAGE_DIR = pathlib.Path(__file__).resolve().parent
_LIB_ENV = "GDN2_B200_LIB"
_lock = threading.Lock()
_handle: ctypes.CDLL | None = None

BF16, FP16, FP32 = 0, 1, 2
_DTYPE_CODES = {torch.bfloat16: BF16, torch.float16: FP16, torch.float32: FP32}

_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_INT = ctypes.c_int
_F32 = ctypes.c_float

# name -> argument types (return type is always int unless listed in _RESTYPES)
_PROTOTYPES: dict[str, list] = {
    "gdn2_version": [],
    "gdn2_status_string": [_INT],
    "gdn2_last_cuda_error": [],
    "gdn2_device_supported": [],
    "gdn2_token_forward": [_P] * 10 + [_I64] * 5 + [_INT, _INT, _F32, _P],
    "gdn2_token_forward_t1_zero": [_P] * 6 + [_I64] * 2 + [_INT, _F32, _P],
    "gdn2_token_dstate_scan": [_P] * 8 + [_I64] * 5 + [_INT, _INT, _F32, _P],
    "gdn2_token_chunk_vjp": [_P] * 15 + [_I64] * 5 + [_INT, _INT, _F32, _P],
    "gdn2_chunk_workspace_bytes": [_I64] * 3 + [_INT],
    "gdn2_chunk_scratch_bytes": [_I64] * 3 + [_INT],
    "gdn2_chunk_forward": [_P] * 12 + [_I64] * 4 + [_INT, _INT, _INT, _F32, _P],
    "gdn2_chunk_backward": [_P] * 19 + [_I64] * 4 + [_INT, _INT, _F32, _P],
    "gdn2_chunk_backward_f32grads": [_P] * 19 + [_I64] * 4 + [_F32, _P],
    "gdn2_chunk_read_status": [_P] + [_I64] * 3 + [_P],
    "gdn2_debug_wait_expires": [_P] + [_I64] * 4 + [_P],
    "gdn2_token_forward_fused": [_P] * 9 + [_I64] * 5 + [_INT, _INT, _F32, _INT, _P],
    "gdn2_token_forward_t1_zero_fused": [_P] * 6 + [_I64] * 2 + [_INT, _F32, _INT, _P],
    "gdn2_chunk_forward_fused": [_P] * 11 + [_I64] * 4 + [_INT, _INT, _F32, _INT, _P],
    "gdn2_gate_prologue": [_P] * 12 + [_I64] * 3 + [_INT, _INT, _P],
    "gdn2_gate_prologue_vjp": [_P] * 17 + [_I64] * 3 + [_INT, _INT, _P],
    "gdn2_chunk_forward_static": [_P] * 9 + [_I64] * 4 + [_INT, _INT, _F32, _P],
    "gdn2_chunk_static_read_status": [_P],
    "gdn2_profile_enable": [_INT],
    "gdn2_profile_chunk_kernels": [_P] * 4,
}
_RESTYPES = {"gdn2_status_string": ctypes.c_char_p, "gdn2_last_cuda_error": ctypes.c_char_p,
             "gdn2_chunk_workspace_bytes": ctypes.c_int64, "gdn2_chunk_scratch_bytes": ctypes.c_int64}


def library_path() -> pathlib.Path:
    override = os.environ.get(_LIB_ENV)
    return pathlib.Path(override) if override else _PACKAGE_DIR / "libgdn2_b200.so"


def exported_symbols() -> tuple[str, ...]:
    """Every entry point the header declares (used by the load test)."""

    return tuple(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """Load the shared object once; raise if it has not been built."""

    global _handle
    if _handle is not None:
        return _handle
    with _lock:
        if _handle is None:
            path = library_path()
            if not path.exists():
                raise RuntimeError(
                    f"{path} is missing: build the CUDA kernels first with "
                    "`python -m gdn2_sm120_b200.build` (there is no CPU or PyTorch fallback)"
                )
            handle = ctypes.CDLL(str(path))
            for name, argtypes in _PROTOTYPES.items():
                fn = getattr(handle, name)  # AttributeError if the symbol is absent
                fn.argtypes = argtypes
                fn.restype = _RESTYPES.get(name, ctypes.c_int)
            _handle = handle
    return _handle


def dtype_code(dtype: torch.dtype) -> int:
    return _DTYPE_CODES[dtype]


def ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# Number of kernels launched through successful entry-point calls.
LAUNCHES = [0]
# When set to a dict, every call is bracketed by CUDA events on the current stream and
# the pair is appended under the entry point's name (used by bench.py to time individual
# kernels live; never enabled on the normal path).
KERNEL_EVENTS: dict[str, list] | None = None


# kernels launched by one successful call of each entry point (default 1)
_KERNELS_PER_CALL = {"gdn2_chunk_forward": 2, "gdn2_chunk_forward_fused": 2, "gdn2_chunk_backward": 2, "gdn2_chunk_backward_f32grads": 2,
                     "gdn2_chunk_forward_static": 2}


def check(status: int, what: str) -> None:
    """Turn a negative gdn2_status into a RuntimeError; count successful launches."""

    if status == 0:
        LAUNCHES[0] += _KERNELS_PER_CALL.get(what, 1)
        return
    handle = lib()
    text = handle.gdn2_status_string(status).decode()
    detail = handle.gdn2_last_cuda_error().decode()
    suffix = f" [{detail}]" if detail and status == -7 else ""
    raise RuntimeError(f"{what} failed with status {status}: {text}{suffix}")


def call(name: str, device: torch.device, *args) -> None:
    """Invoke entry point ``name`` with ``device`` current; raise on a non-zero status."""

    fn = getattr(lib(), name)
    with torch.cuda.device(device):
        if KERNEL_EVENTS is None:
            status = fn(*args)
        else:
            begin = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            begin.record()
            status = fn(*args)
            end.record()
            KERNEL_EVENTS.setdefault(name, []).append((begin, end))
    check(status, name)


_capability_ok: dict[int, bool] = {}


def require_b200(device: torch.device) -> None:
    """Reject any GPU that is not compute capability 10.x (no silent fallback)."""

    index = device.index if device.index is not None else torch.cuda.current_device()
    ok = _capability_ok.get(index)
    if ok is None:
        ok = torch.cuda.get_device_capability(index)[0] == 10
        _capability_ok[index] = ok
    if not ok:
        raise RuntimeError("these kernels are built for sm_100a (B200) GPUs only")


def profile_enable(on: bool) -> None:
    """Switch the per-kernel event timing of the chunk entry points on or off."""

    lib().gdn2_profile_enable(1 if on else 0)


def profile_chunk_kernels() -> dict[str, float]:
    """Durations (ms) of the four kernels of the most recent chunk forward / backward calls.

    Waits for the recorded events.  Kernels whose call has not run since profiling was switched on
    are left out."""

    values = [ctypes.c_float(-1.0) for _ in range(4)]
    status = lib().gdn2_profile_chunk_kernels(*[ctypes.byref(v) for v in values])
    if status != 0:
        raise RuntimeError(f"gdn2_profile_chunk_kernels failed with status {status}")
    names = ("chunk_prep_kernel", "chunk_scan_kernel", "chunk_bwd_scan_kernel", "chunk_bwd_vjp_kernel")
    return {n: v.value for n, v in zip(names, values) if v.value >= 0.0}
