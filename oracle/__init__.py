"""CPU oracle of the MoE dispatch/combine hot path — TEST INFRASTRUCTURE, not product.

A restatement of the reference's CPU/PyTorch arithmetic (polkadot21/fastmoe) in
plain C (`combine_oracle.c`, loaded through ctypes) and numpy (`routing.py`,
`layer.py`). Only tests/, `__graft_entry__.smoke()` and bench.py's CPU-baseline
legs may import it; nothing under fastmoe_b200/ does.

Pinned: every function here is checked against fixtures produced by importing the
reference itself (tests/golden/make_golden.py, tests/test_oracle_golden.py). Where a
checkout of the reference is at hand, `install_ref.py` installs the unmodified package
into oracle/_ref/ (untracked) and `reference_ops()` hands out its operator module, which
bench.py times as the CPU baseline and tests compare the C port with.

bf16 data crosses this interface as numpy uint16 bit patterns.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

from .layer import moe_layer_forward  # noqa: F401
from .routing import build_index, prepare_metadata, topk_softmax  # noqa: F401

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compiles combine_oracle.c with gcc (see the Makefile beside it)."""
    src = _DIR / "combine_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        proc = subprocess.run(["make", "-C", str(_DIR), "-B", "liboracle.so"], capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"building the oracle failed:\n{proc.stdout}\n{proc.stderr}")
    return _LIB_PATH


def _c():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def reference_ops():
    """The reference's own operator module (`fastmoe.kernels.ops`, unmodified), if
    oracle/install_ref.py has installed the package into oracle/_ref/; None where it has not
    (or where its imports fail). Used to time the reference's CPU path
    (src/fastmoe/kernels/ops.py:373-384) beside this build's kernels, and to check the C port
    of that path against the real thing."""
    ref_dir = _DIR / "_ref"
    if not (ref_dir / "fastmoe" / "kernels" / "ops.py").exists():
        return None
    import importlib
    import sys

    sys.path.insert(0, str(ref_dir))
    try:
        return importlib.import_module("fastmoe.kernels.ops")
    except Exception:  # a dependency of the package (settings, logging) is missing on this machine
        return None
    finally:
        sys.path.remove(str(ref_dir))


def num_threads() -> int:
    return int(_c().oracle_num_threads())


def use_all_cores() -> int:
    """Lets the C oracle use every core this process may run on (an inherited
    OMP_NUM_THREADS=1, as torchrun sets it, would otherwise pin it to one). Returns the count."""
    import os

    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    _c().oracle_set_num_threads(ctypes.c_int(n))
    return num_threads()


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _ptr_array(arrays):
    arr = (ctypes.c_void_p * max(len(arrays), 1))()
    for i, a in enumerate(arrays):
        arr[i] = a.ctypes.data
    return arr


def _prep(experts, idx, dtype):
    experts = [np.ascontiguousarray(e, dtype=dtype) for e in experts]
    sizes = np.array([e.shape[0] for e in experts], dtype=np.int64)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    if idx.shape[0] != int(sizes.sum()):
        raise ValueError("one index per expert row is required")
    return experts, sizes, idx


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, as torch's .to(torch.bfloat16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def combine(experts, idx, w, T, out=None) -> np.ndarray:
    """fp32 combine, src/fastmoe/kernels/ops.py:373-384. Accumulates into `out` if given."""
    experts, sizes, idx = _prep(experts, idx, np.float32)
    D = experts[0].shape[1]
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.zeros((T, D), np.float32) if out is None else out
    assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (T, D)
    if len(idx) and (idx.min() < 0 or idx.max() >= T):
        raise IndexError("index out of range")
    _c().oracle_combine_f32(_ptr_array(experts), _ptr(sizes), ctypes.c_int64(len(experts)), _ptr(idx),
                            _ptr(w), _ptr(out), ctypes.c_int64(T), ctypes.c_int64(D))  # fmt: skip
    return out


def combine_bf16(experts_bits, idx, w_bits, T, out_bits=None) -> np.ndarray:
    """The reference's own bf16 CPU arithmetic (bf16 product, bf16 accumulation), on bit patterns."""
    experts, sizes, idx = _prep(experts_bits, idx, np.uint16)
    D = experts[0].shape[1]
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    out = np.zeros((T, D), np.uint16) if out_bits is None else out_bits
    assert out.dtype == np.uint16 and out.flags.c_contiguous and out.shape == (T, D)
    if len(idx) and (idx.min() < 0 or idx.max() >= T):
        raise IndexError("index out of range")
    _c().oracle_combine_bf16(_ptr_array(experts), _ptr(sizes), ctypes.c_int64(len(experts)), _ptr(idx),
                             _ptr(w), _ptr(out), ctypes.c_int64(T), ctypes.c_int64(D))  # fmt: skip
    return out


def combine_bf16_in_f32(experts_bits, idx, w_bits, T, out=None) -> np.ndarray:
    """bf16 inputs, fp32 arithmetic and result: the yardstick for the kernels' bf16 runs."""
    experts, sizes, idx = _prep(experts_bits, idx, np.uint16)
    D = experts[0].shape[1]
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    out = np.zeros((T, D), np.float32) if out is None else out
    assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (T, D)
    if len(idx) and (idx.min() < 0 or idx.max() >= T):
        raise IndexError("index out of range")
    _c().oracle_combine_bf16_in_f32(_ptr_array(experts), _ptr(sizes), ctypes.c_int64(len(experts)),
                                    _ptr(idx), _ptr(w), _ptr(out), ctypes.c_int64(T),
                                    ctypes.c_int64(D))  # fmt: skip
    return out


def combine_bwd(rows, idx, w, grad_out, with_grad_w=True):
    """(grad_rows [N, D], grad_w [N]) as autograd derives them from ops.py:380-382."""
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    w = np.ascontiguousarray(w, dtype=np.float32)
    grad_out = np.ascontiguousarray(grad_out, dtype=np.float32)
    N, D = rows.shape
    grad_rows = np.empty((N, D), np.float32)
    grad_w = np.empty(N, np.float32) if with_grad_w else None
    _c().oracle_combine_bwd_f32(_ptr(rows), _ptr(idx), _ptr(w), _ptr(grad_out), _ptr(grad_rows),
                                _ptr(grad_w) if with_grad_w else None, ctypes.c_int64(N),
                                ctypes.c_int64(D))  # fmt: skip
    return grad_rows, grad_w


def permute(x, reverse_map) -> np.ndarray:
    """permuted = x[reverse_map], src/fastmoe/models/tiny_model.py:133 (any 2- or 4-byte dtype)."""
    x = np.ascontiguousarray(x)
    rm = np.ascontiguousarray(reverse_map, dtype=np.int64)
    out = np.empty((rm.shape[0], x.shape[1]), x.dtype)
    _c().oracle_permute(_ptr(x), _ptr(rm), _ptr(out), ctypes.c_int64(rm.shape[0]),
                        ctypes.c_int64(x.shape[1]), ctypes.c_int64(x.dtype.itemsize))  # fmt: skip
    return out


def permute_bwd(grad_permuted, reverse_map, T) -> np.ndarray:
    """grad_x = zeros.index_put_(reverse_map, grad_permuted, accumulate=True)."""
    gp = np.ascontiguousarray(grad_permuted, dtype=np.float32)
    rm = np.ascontiguousarray(reverse_map, dtype=np.int64)
    out = np.zeros((T, gp.shape[1]), np.float32)
    _c().oracle_permute_bwd_f32(_ptr(gp), _ptr(rm), _ptr(out), ctypes.c_int64(gp.shape[0]),
                                ctypes.c_int64(gp.shape[1]))  # fmt: skip
    return out
