"""Helpers shared by the GPU parity tests: torch <-> numpy (bf16 as bit patterns)
and tolerance checks stated once.

Tolerances (relative to the largest magnitude of the reference result):
  fp32  1e-5   bf16/fp16  2e-2
The planned (gather) kernels sum in the oracle's order with separate multiply and
add, so their fp32 results are additionally required to be bit-exact.
"""

import numpy as np
import torch

import oracle

REL_TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def to_np(t: torch.Tensor) -> np.ndarray:
    """fp32 view of a tensor's values (bf16/fp16 are widened exactly)."""
    return t.detach().float().cpu().numpy()


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_combine(experts, indices, weights, T, out0=None):
    """fp32-arithmetic oracle on the tensors' exact values (bf16 inputs are widened, not re-rounded)."""
    ex = [to_np(e) for e in experts]
    out = None if out0 is None else np.ascontiguousarray(to_np(out0))
    return oracle.combine(ex, indices.cpu().numpy().astype(np.int64), to_np(weights), T, out=out)


def assert_close(actual: torch.Tensor, expected: np.ndarray, dtype, what=""):
    a = to_np(actual)
    scale = max(float(np.abs(expected).max()), 1e-30)
    err = float(np.abs(a - expected).max()) / scale
    assert err <= REL_TOL[dtype], f"{what}: relative error {err:.3e} > {REL_TOL[dtype]:.0e}"
    return err


def split_rows(rows, sizes):
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
    return [rows[offs[e] : offs[e + 1]] for e in range(len(sizes))]
