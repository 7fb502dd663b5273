"""Generate the golden fixtures from the reference project's own PyTorch oracle.

Run once, in a container where the reference source tree is present:

    python tests/golden/make_golden.py /path/to/reference/src

It imports ``gdn2_sm120.reference`` (src/gdn2_sm120/reference.py) and records,
for a handful of small seeded cases, the inputs (as raw 16-bit / 32-bit
patterns) together with what the reference computes: the output, the final
state and -- through ``torch.autograd`` over ``recurrent_forward_reference`` --
the seven gradients of the benchmark loss ``mean(o^2) + mean(S_T^2)``.
The reference keeps no stored vectors of its own (its tests draw seeded random
inputs), so these files are the committed anchor of the parity chain:

    reference.py  ==(this script)==>  tests/golden/*.npz
    tests/golden/*.npz  <==(tests/test_oracle.py)==  oracle/gdn2_oracle.py
    oracle/gdn2_oracle.py  <==(tests -m gpu)==  CUDA kernels

A second kind of fixture, ``stage_chunk64.npz``, pins the stage-level oracles: for one
64-token chunk (K = V = 128) it records what the reference's own executable proofs return --
``boundary_dstate_wy_reference`` (src/gdn2_sm120/backward_parallel.py:315-373: the chunk's
residual cotangent dR and the state cotangent at the chunk start) and
``compact_wy_chunk_vjp_reference`` (src/gdn2_sm120/backward_wy.py:62-223: the six sequence
gradients of the chunk), both evaluated in float64 on auxiliaries built by
``build_wy_boundary_aux_reference`` (backward_parallel.py:193-270).

Inputs are drawn by ``oracle.gdn2_oracle.make_inputs`` (pure torch CPU RNG) so
the generator of the inputs is committed too; the arrays are stored anyway so
that the fixtures do not depend on RNG stability.
"""

from __future__ import annotations

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent / "oracle"))

import gdn2_oracle as oracle  # noqa: E402

# name -> (B, T, H, seed, dtype, g_dtype, with_state, scale, want_grads)
CASES = {
    # benchmark configuration 0: the reference's CPU-runnable case
    "config0_b1_t64_h2": (1, 64, 2, 0, torch.bfloat16, torch.float32, True, None, True),
    # decode-shaped cases mirroring tests/test_recurrent.py:195-226
    "decode_b1_t5_h2_bf16": (1, 5, 2, 1234, torch.bfloat16, torch.float32, True, 0.125, True),
    "decode_b1_t5_h2_fp16_lowg": (1, 5, 2, 1235, torch.float16, torch.float16, True, 0.125, False),
    "decode_b2_t1_h3_zero": (2, 1, 3, 611, torch.bfloat16, torch.float32, False, 0.0625, True),
    # short sequences on both sides of the dispatch thresholds, ragged tail
    "short_b2_t19_h3": (2, 19, 3, 2045, torch.bfloat16, torch.float32, True, None, True),
    "chunk_b1_t129_h2_nostate": (1, 129, 2, 2155, torch.bfloat16, torch.float32, False, None, True),
}


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().copy()
    return t.contiguous().numpy().copy()


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    from gdn2_sm120.reference import (  # type: ignore
        chunkwise_forward_reference,
        recurrent_forward_reference,
    )

    torch.set_num_threads(1)  # fixed summation order
    for name, (b, t, h, seed, dtype, g_dtype, with_state, scale, want_grads) in CASES.items():
        q, k, v, g, beta, w, s0 = oracle.make_inputs(
            b, t, h, seed=seed, dtype=dtype, g_dtype=g_dtype, with_state=with_state
        )
        record = {
            "dtype": np.array(str(dtype)),
            "g_dtype": np.array(str(g_dtype)),
            "scale": np.array(-1.0 if scale is None else scale),
            "q": _bits(q), "k": _bits(k), "v": _bits(v), "g": _bits(g),
            "beta": _bits(beta), "w": _bits(w),
        }
        if s0 is not None:
            record["initial_state"] = s0.numpy().copy()
        out, final = recurrent_forward_reference(q, k, v, g, beta, w, s0, scale=scale)
        record["out"] = _bits(out)
        record["final_state"] = final.numpy().copy()
        out_c, final_c = chunkwise_forward_reference(q, k, v, g, beta, w, s0, scale=scale, chunk_size=16)
        record["out_chunk16"] = _bits(out_c)
        record["final_state_chunk16"] = final_c.numpy().copy()
        if want_grads:
            leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, g, beta, w)]
            s0_leaf = None if s0 is None else s0.detach().clone().requires_grad_(True)
            out_g, final_g = recurrent_forward_reference(*leaves, s0_leaf, scale=scale)
            loss = out_g.float().square().mean() + final_g.square().mean()
            wanted = leaves + ([s0_leaf] if s0_leaf is not None else [])
            grads = torch.autograd.grad(loss, wanted)
            for label, grad in zip(("dq", "dk", "dv", "dg", "dbeta", "dw", "dS0"), grads):
                record[label] = _bits(grad)
            record["loss"] = np.array(loss.item())
        np.savez_compressed(HERE / f"{name}.npz", **record)
        print(name, {key: getattr(val, "shape", None) for key, val in record.items() if key in ("q", "out", "final_state")})


def stage_fixture(reference_src: str) -> None:
    """One 64-token chunk through the reference's stage-level proofs, in float64."""

    sys.path.insert(0, reference_src)
    from types import SimpleNamespace

    from gdn2_sm120.backward_parallel import (  # type: ignore
        boundary_dstate_wy_reference,
        build_wy_boundary_aux_reference,
    )
    from gdn2_sm120.backward_wy import compact_wy_chunk_vjp_reference  # type: ignore
    from gdn2_sm120.reference import recurrent_forward_reference  # type: ignore

    torch.set_num_threads(1)
    chunk = 64
    q, k, v, g, beta, w, s0 = oracle.make_inputs(1, chunk, 1, seed=6464)
    gen = torch.Generator().manual_seed(6465)
    d_out = (torch.randn(v.shape, generator=gen) * 0.1).to(torch.bfloat16)
    d_s1 = torch.randn(s0.shape, generator=gen) * 0.01
    scale = 1.0 / 128 ** 0.5
    q64, k64, v64, g64, beta64, w64 = (x.double() for x in (q, k, v, g, beta, w))
    s0_64, do64, ds1_64 = s0.double(), d_out.double(), d_s1.double()

    # auxiliaries: the reference's own builder (fp32 inside), U by the same triangular solve in float64
    aux32 = build_wy_boundary_aux_reference(q64, k64, g64, beta64, scale=scale, chunk_size=chunk)
    gamma = g64[:, :, 0].cumsum(dim=1).exp()                       # [1, 64, 128]
    erase = gamma * beta64[:, :, 0] * k64[:, :, 0]
    k_bar = k64[:, :, 0] / gamma
    lower = torch.tril(erase @ k_bar.transpose(-1, -2), diagonal=-1)
    system = lower + torch.eye(chunk, dtype=torch.float64)
    u = torch.linalg.solve_triangular(system, w64[:, :, 0] * v64[:, :, 0], upper=False, unitriangular=True)
    aux = SimpleNamespace(y=aux32.y.double(), u=u.unsqueeze(2), q_gamma=aux32.q_gamma.double(),
                          k_tail=aux32.k_tail.double(), decay_end=aux32.decay_end.double(),
                          aqk=aux32.aqk.double())
    _, s1 = recurrent_forward_reference(q, k, v, g, beta, w, s0, scale=scale)
    d_bnd, d_residual = boundary_dstate_wy_reference(aux, do64, ds1_64, chunk_size=chunk,
                                                     return_d_residual=True)
    state_bnd = torch.stack([s0_64, s1.double()], dim=1)
    grads, _ = compact_wy_chunk_vjp_reference(q64, k64, v64, g64, beta64, w64, state_bnd, d_bnd.double(),
                                              aux, do64, scale=scale, chunk_size=chunk,
                                              verify_boundaries=True)
    record = {
        "dtype": np.array(str(torch.bfloat16)), "g_dtype": np.array(str(torch.float32)),
        "scale": np.array(scale),
        "q": _bits(q), "k": _bits(k), "v": _bits(v), "g": _bits(g), "beta": _bits(beta), "w": _bits(w),
        "initial_state": s0.numpy().copy(), "d_out": _bits(d_out), "d_s1": d_s1.numpy().copy(),
        "d_residual": d_residual.float().numpy().copy(),
        "d_s0": d_bnd[:, 0].float().numpy().copy(),
        "final_state": s1.numpy().copy(),
    }
    for label, grad in zip(("dq", "dk", "dv", "dg", "dbeta", "dw"), grads[:6]):
        record["stage_" + label] = grad.float().numpy().copy()
    np.savez_compressed(HERE / "stage_chunk64.npz", **record)
    print("stage_chunk64", {key: val.shape for key, val in record.items() if hasattr(val, "shape") and val.ndim})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout's src directory>")
    main(sys.argv[1])
    stage_fixture(sys.argv[1])
