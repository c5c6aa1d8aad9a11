"""Expert FFN as grouped GEMMs on the tcgen05 tensor cores.

`grouped_gemm` multiplies every expert's contiguous block of rows by that expert's
weight matrix in ONE persistent launch, reading the per-expert row ranges from device
memory, and `grouped_swiglu_ffn` chains two of them into down(silu(gate(x)) * up(x)).
They replace the Python loop over `self.experts` in `MoEFeedForward.compute_experts` of
polkadot21/fastmoe (src/fastmoe/models/tiny_model.py:282-294).

Forward, data gradient and weight gradient all run on the hand-written tcgen05 kernels
(`csrc/grouped_gemm.cu`) with the per-expert row ranges read from device memory; the
SwiGLU derivative between them is one streaming kernel over recomputed pre-activations.
Shapes the kernels do not tile (N or K not a multiple of 64/128/256) fall back to
per-expert library products.
"""

from __future__ import annotations

import torch

from . import ops
from .ops import _require_cuda, _status_word, _stream_ptr


def _check(a, w, offsets, counts):
    _require_cuda(a, "a")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError("grouped_gemm runs in bfloat16")
    if a.dim() != 2 or w.dim() != 3 or w.shape[2] != a.shape[1]:
        raise ValueError(f"a must be [R, K] and w [E, N, K]; got {tuple(a.shape)} and {tuple(w.shape)}")
    if offsets.dtype != torch.int64 or counts.dtype != torch.int64:
        raise ValueError("offsets and counts must be int64 device tensors")
    if offsets.numel() != w.shape[0] or counts.numel() != w.shape[0]:
        raise ValueError("offsets and counts need one entry per expert")


def _launch(a, w, offsets, counts, swiglu, row_map=None, covers_all_rows=False, row_ptrs=None):
    a, w = a.contiguous(), w.contiguous()
    R, K = a.shape
    E, N, _ = w.shape
    cols = N // 2 if swiglu else N
    if row_ptrs is not None:
        c = None  # every row goes where its table entry points
    elif covers_all_rows or R == 0:
        c = torch.empty(R, cols, dtype=torch.bfloat16, device=a.device)
    else:  # rows that belong to no expert are never written: start from zeros so they are defined
        c = torch.zeros(R, cols, dtype=torch.bfloat16, device=a.device)
    ops._call(
        "fmoe_grouped_gemm", 1, a.data_ptr(), w.data_ptr(), c.data_ptr() if c is not None else None,
        offsets.data_ptr(), counts.data_ptr(), row_map.data_ptr() if row_map is not None else None,
        row_ptrs.data_ptr() if row_ptrs is not None else None, E, R, N, K,
        1 if swiglu else 0, _status_word(a.device).data_ptr(), _stream_ptr(a.device),
    )  # fmt: skip
    return c


class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, offsets, counts, swiglu, row_map, covers_all_rows):
        _check(a, w, offsets, counts)
        if row_map is not None and (row_map.dtype != torch.int64 or row_map.numel() != a.shape[0]):
            raise ValueError("row_map must be an int64 device tensor with one entry per row of a")
        ctx.save_for_backward(a, w, offsets, counts, row_map)
        ctx.swiglu, ctx.covers_all_rows = swiglu, covers_all_rows
        return _launch(a, w, offsets, counts, swiglu, row_map, covers_all_rows)

    @staticmethod
    def backward(ctx, grad_c):
        a, w, offsets, counts, row_map = ctx.saved_tensors
        if row_map is not None:
            grad_c = grad_c.index_select(0, row_map)  # back to the row order of `a`
        grad_c = grad_c.contiguous()
        if ctx.swiglu:
            # recompute the pre-activations with the plain kernel, then the SwiGLU derivative
            ff = w.shape[1] // 2
            h = _launch(a, w, offsets, counts, False, covers_all_rows=ctx.covers_all_rows)
            grad_h = torch.empty_like(h)
            ops._call("fmoe_swiglu_bwd", 1, h.data_ptr(), grad_c.data_ptr(), grad_h.data_ptr(), h.shape[0], ff,
                      _stream_ptr(h.device))  # fmt: skip
            grad_c = grad_h
            del h
        need_a, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        grad_a = _dgrad(grad_c, w, offsets, counts, ctx.covers_all_rows) if need_a else None
        grad_w = _wgrad(grad_c, a, w.shape, offsets, counts) if need_w else None
        return grad_a, grad_w, None, None, None, None, None


def _dgrad(grad_c, w, offsets, counts, covers_all_rows=False, row_ptrs=None):
    """grad_a[rows of e] = grad_c[rows of e] @ w[e] on the tensor cores; rows owned by no
    expert get zero. With `row_ptrs` (int64 [R] addresses) every result row is stored where
    its entry points and nothing is returned."""
    R, N = grad_c.shape
    E, _, K = w.shape
    if row_ptrs is None and (N % 64 or K % 256):
        return _dgrad_library(grad_c, w, offsets, counts)
    grad_a = None
    if row_ptrs is None:
        alloc = torch.empty if covers_all_rows else torch.zeros
        grad_a = alloc(R, K, dtype=torch.bfloat16, device=grad_c.device)
    ops._call(
        "fmoe_grouped_gemm_dgrad", 1, grad_c.data_ptr(), w.contiguous().data_ptr(),
        grad_a.data_ptr() if grad_a is not None else None, offsets.data_ptr(), counts.data_ptr(),
        row_ptrs.data_ptr() if row_ptrs is not None else None, E, R, N, K,
        _status_word(grad_c.device).data_ptr(), _stream_ptr(grad_c.device),
    )  # fmt: skip
    return grad_a


def _wgrad(grad_c, a, w_shape, offsets, counts):
    """grad_w[e] = grad_c[rows of e].T @ a[rows of e] on the tensor cores."""
    E, N, K = w_shape
    R = a.shape[0]
    if N % 128 or K % 256:
        return _wgrad_library(grad_c, a, w_shape, offsets, counts)
    grad_w = torch.empty(E, N, K, dtype=torch.bfloat16, device=a.device)
    ops._call(
        "fmoe_grouped_gemm_wgrad", 1, grad_c.data_ptr(), a.contiguous().data_ptr(), grad_w.data_ptr(),
        offsets.data_ptr(), counts.data_ptr(), E, R, N, K, _status_word(a.device).data_ptr(), _stream_ptr(a.device),
    )  # fmt: skip
    return grad_w


def _dgrad_library(grad_c, w, offsets, counts):
    """Shapes the kernels do not tile: per-expert library products (needs the counts on the host)."""
    grad_a = torch.zeros(grad_c.shape[0], w.shape[2], dtype=grad_c.dtype, device=grad_c.device)
    for e, (o, n) in enumerate(zip(offsets.tolist(), counts.tolist())):
        if n:
            grad_a[o : o + n] = grad_c[o : o + n] @ w[e]
    return grad_a


def _wgrad_library(grad_c, a, w_shape, offsets, counts):
    grad_w = torch.zeros(w_shape, dtype=a.dtype, device=a.device)
    for e, (o, n) in enumerate(zip(offsets.tolist(), counts.tolist())):
        if n:
            grad_w[e] = grad_c[o : o + n].t() @ a[o : o + n]
    return grad_w


def grouped_gemm(a, w, offsets, counts, swiglu=False, row_map=None, covers_all_rows=False):
    """C[rows of e] = A[rows of e] @ w[e].T (or the fused SwiGLU of its two halves).

    a [R, K] bf16; w [E, N, K] bf16; offsets, counts int64 [E] on the device (rows
    [offsets[e], offsets[e]+counts[e]) belong to expert e). Returns bf16 [R, N] (or [R, N/2]).
    `row_map` (int64 [R], a permutation) stores the result of row r at row row_map[r].
    `covers_all_rows=True` promises that every row belongs to an expert, which saves the
    zero-fill of the output.
    """
    return _GroupedGemm.apply(a, w, offsets, counts, bool(swiglu), row_map, bool(covers_all_rows))


def grouped_swiglu_ffn(x, w_gate_up, w_down, offsets, counts, row_map=None, covers_all_rows=False):
    """down(silu(gate(x)) * up(x)) per expert. w_gate_up [E, 2*ff, D] (gate rows first), w_down [E, D, ff].
    `row_map` reorders the rows of the result (see grouped_gemm)."""
    hidden = grouped_gemm(x, w_gate_up, offsets, counts, swiglu=True, covers_all_rows=covers_all_rows)
    return grouped_gemm(hidden, w_down, offsets, counts, swiglu=False, row_map=row_map,
                        covers_all_rows=covers_all_rows)  # fmt: skip


def grouped_gemm_to_rows(a, w, offsets, counts, row_ptrs):
    """Plain grouped GEMM (no autograd) whose output row r is stored at the ADDRESS row_ptrs[r]
    (int64 [R] on the device; the rows may live in other GPUs' memory). Returns nothing."""
    _check(a, w, offsets, counts)
    if row_ptrs.dtype != torch.int64 or row_ptrs.numel() < a.shape[0]:
        raise ValueError("row_ptrs must be an int64 device tensor with one entry per row of a")
    _launch(a, w, offsets, counts, False, row_ptrs=row_ptrs)
