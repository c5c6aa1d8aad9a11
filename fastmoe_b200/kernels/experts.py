"""Expert FFN as grouped GEMMs on the tcgen05 tensor cores.

`grouped_gemm` multiplies every expert's contiguous block of rows by that expert's
weight matrix in ONE persistent launch, reading the per-expert row ranges from device
memory. `grouped_swiglu_ffn` chains two of them into down(silu(gate(x)) * up(x)) and
`grouped_gelu_ffn` into fc2(gelu(fc1(x))), the reference's own expert
(src/fastmoe/models/tiny_model.py:68-77). They replace the Python loop over `self.experts`
in `MoEFeedForward.compute_experts` of polkadot21/fastmoe (tiny_model.py:282-294).

Forward, data gradient and weight gradient all run on the hand-written tcgen05 kernels
(`csrc/grouped_gemm.cu`) with the per-expert row ranges read from device memory; the
activation's derivative between them is one streaming kernel over the pre-activations,
which a forward that will be differentiated stores from its epilogue beside the result. Shapes the kernels do not tile raise ValueError, forward and backward
alike: there is no library fallback.
"""

from __future__ import annotations

import torch

from .. import _lib
from . import ops
from .ops import _require_cuda, _status_word, _stream_ptr

ACT_NONE, ACT_SWIGLU, ACT_GELU = _lib.ACT_NONE, _lib.ACT_SWIGLU, _lib.ACT_GELU


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


def check_shapes(N: int, K: int, act: int = ACT_NONE, training: bool = False):
    """Raises ValueError unless the kernels tile a [*, K] x [E, N, K] product (and, with
    `training`, its two gradients): the forward needs K % 64 == 0 and N % 256 == 0, the
    gradients K % 256 == 0 and N % 128 == 0."""
    if K % 64 or N % 256:
        raise ValueError(f"grouped_gemm needs K a multiple of 64 and N a multiple of 256, got K={K}, N={N}")
    if training and (K % 256 or N % 128):
        raise ValueError(f"the grouped GEMM's gradients need K a multiple of 256 and N of 128, got K={K}, N={N}")
    if act == ACT_SWIGLU and (N // 2) % 128:
        raise ValueError(f"SwiGLU needs N = 2*ff with ff a multiple of 128, got N={N}")


def supported(N: int, K: int, act: int = ACT_NONE, training: bool = False) -> bool:
    try:
        check_shapes(N, K, act, training)
    except ValueError:
        return False
    return True


def _after_launch(device, what):
    """With checking switched on (FASTMOE_B200_CHECK=1) reads the status word after the launch
    and raises if a bounded device-side wait gave up or rows were cut off."""
    if ops._check:
        value = ops.read_status(device)
        if value:
            raise RuntimeError(f"{what}: device status word = {value}"
                               + (" (a bounded wait gave up)" if value & _lib.STATUS_WAIT_TIMEOUT else ""))  # fmt: skip


def _launch(a, w, offsets, counts, act, row_map=None, covers_all_rows=False, row_ptrs=None, out=None, pre=None):
    """One grouped GEMM launch. `act` is ACT_NONE / ACT_SWIGLU / ACT_GELU (False / True also
    mean the first two). `out` ([R, cols], bf16, contiguous) receives the result instead of a
    fresh tensor; with `row_ptrs` every row goes where its table entry points. `pre` ([R, N],
    bf16, contiguous) also receives the product before the activation, row r of `a` in row r."""
    a, w = a.contiguous(), w.contiguous()
    act = int(act)
    R, K = a.shape
    E, N, _ = w.shape
    cols = N // 2 if act == ACT_SWIGLU else N
    if row_ptrs is not None:
        c = None  # every row goes where its table entry points
    elif out is not None:
        if out.shape != (R, cols) or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous bfloat16 [{R}, {cols}] tensor")
        c = out
    elif covers_all_rows or R == 0:
        c = torch.empty(R, cols, dtype=torch.bfloat16, device=a.device)
    else:  # rows that belong to no expert are never written: start from zeros so they are defined
        c = torch.zeros(R, cols, dtype=torch.bfloat16, device=a.device)
    tail = (offsets.data_ptr(), counts.data_ptr(), row_map.data_ptr() if row_map is not None else None,
            row_ptrs.data_ptr() if row_ptrs is not None else None, E, R, N, K,
            act, _status_word(a.device).data_ptr(), _stream_ptr(a.device))  # fmt: skip
    c_ptr = c.data_ptr() if c is not None else None
    if pre is None:
        ops._call("fmoe_grouped_gemm", 1, a.data_ptr(), w.data_ptr(), c_ptr, *tail)
    else:
        if pre.shape != (R, N) or pre.dtype != torch.bfloat16 or not pre.is_contiguous():
            raise ValueError(f"pre must be a contiguous bfloat16 [{R}, {N}] tensor")
        ops._call("fmoe_grouped_gemm_keep_pre", 1, a.data_ptr(), w.data_ptr(), c_ptr, pre.data_ptr(), *tail)
    _after_launch(a.device, "fmoe_grouped_gemm")
    return c


class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, offsets, counts, act, row_map, covers_all_rows, keep_pre):
        # a forward that will be differentiated keeps the product before the activation (the
        # epilogue stores it beside the result), so that the backward needs no second product
        pre = None
        if keep_pre and act != ACT_NONE:
            pre = torch.empty(a.shape[0], w.shape[1], dtype=torch.bfloat16, device=a.device)
        out = _launch(a, w, offsets, counts, act, row_map, covers_all_rows, pre=pre)
        ctx.save_for_backward(a, w, offsets, counts, row_map, pre)
        ctx.act, ctx.covers_all_rows = act, covers_all_rows
        return out

    @staticmethod
    def backward(ctx, grad_c):
        a, w, offsets, counts, row_map, h = ctx.saved_tensors
        if row_map is not None:
            grad_c = grad_c.index_select(0, row_map)  # back to the row order of `a`
        grad_c = grad_c.contiguous()
        if ctx.act != ACT_NONE:
            if h is None:  # the forward ran without keeping them: recompute with the plain kernel
                h = _launch(a, w, offsets, counts, ACT_NONE, covers_all_rows=ctx.covers_all_rows)
            grad_h = torch.empty_like(h)
            if ctx.act == ACT_SWIGLU:
                ops._call("fmoe_swiglu_bwd", 1, h.data_ptr(), grad_c.data_ptr(), grad_h.data_ptr(), h.shape[0],
                          w.shape[1] // 2, _stream_ptr(h.device))  # fmt: skip
            else:
                ops._call("fmoe_gelu_bwd", 1, h.data_ptr(), grad_c.data_ptr(), grad_h.data_ptr(), h.shape[0],
                          w.shape[1], _stream_ptr(h.device))  # fmt: skip
            grad_c = grad_h
            del h
        need_a, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        grad_a = _dgrad(grad_c, w, offsets, counts, ctx.covers_all_rows) if need_a else None
        grad_w = _wgrad(grad_c, a, w.shape, offsets, counts) if need_w else None
        return grad_a, grad_w, None, None, None, None, None, None


def _apply(a, w, offsets, counts, act, row_map, covers_all_rows):
    """Checks the arguments, then runs the product through autograd. Whether gradients will be
    asked for is decided here, where the caller's grad mode is still visible: a width whose
    gradients the kernels do not tile raises now rather than in the middle of a backward pass."""
    _check(a, w, offsets, counts)
    if row_map is not None and (row_map.dtype != torch.int64 or row_map.numel() != a.shape[0]):
        raise ValueError("row_map must be an int64 device tensor with one entry per row of a")
    training = torch.is_grad_enabled() and (a.requires_grad or w.requires_grad)
    check_shapes(w.shape[1], w.shape[2], act, training)
    return _GroupedGemm.apply(a, w, offsets, counts, act, row_map, covers_all_rows, training)


def _dgrad(grad_c, w, offsets, counts, covers_all_rows=False, row_ptrs=None):
    """grad_a[rows of e] = grad_c[rows of e] @ w[e] on the tensor cores; rows owned by no
    expert get zero. With `row_ptrs` (int64 [R] addresses) every result row is stored where
    its entry points and nothing is returned."""
    R, N = grad_c.shape
    E, _, K = w.shape
    if N % 64 or K % 256:
        raise ValueError(f"the grouped GEMM's data gradient needs N a multiple of 64 and K of 256, got N={N}, K={K}")
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
    _after_launch(grad_c.device, "fmoe_grouped_gemm_dgrad")
    return grad_a


def _wgrad(grad_c, a, w_shape, offsets, counts):
    """grad_w[e] = grad_c[rows of e].T @ a[rows of e] on the tensor cores."""
    E, N, K = w_shape
    R = a.shape[0]
    if N % 128 or K % 256:
        raise ValueError(f"the grouped GEMM's weight gradient needs N a multiple of 128 and K of 256, got N={N}, K={K}")
    grad_w = torch.empty(E, N, K, dtype=torch.bfloat16, device=a.device)
    ops._call(
        "fmoe_grouped_gemm_wgrad", 1, grad_c.data_ptr(), a.contiguous().data_ptr(), grad_w.data_ptr(),
        offsets.data_ptr(), counts.data_ptr(), E, R, N, K, _status_word(a.device).data_ptr(), _stream_ptr(a.device),
    )  # fmt: skip
    _after_launch(a.device, "fmoe_grouped_gemm_wgrad")
    return grad_w


def grouped_gemm(a, w, offsets, counts, swiglu=False, row_map=None, covers_all_rows=False, activation=None):
    """C[rows of e] = A[rows of e] @ w[e].T, optionally followed by an activation in the epilogue.

    a [R, K] bf16; w [E, N, K] bf16; offsets, counts int64 [E] on the device (rows
    [offsets[e], offsets[e]+counts[e]) belong to expert e). Returns bf16 [R, N] (or [R, N/2]
    for SwiGLU, which pairs the first N/2 weight rows as gate with the last N/2 as up).
    `activation`: ACT_NONE, ACT_SWIGLU or ACT_GELU (`swiglu=True` is the older spelling of
    ACT_SWIGLU). `row_map` (int64 [R], a permutation) stores the result of row r at row
    row_map[r]. `covers_all_rows=True` promises that every row belongs to an expert, which
    saves the zero-fill of the output.
    """
    act = int(activation) if activation is not None else (ACT_SWIGLU if swiglu else ACT_NONE)
    return _apply(a, w, offsets, counts, act, row_map, bool(covers_all_rows))


def grouped_swiglu_ffn(x, w_gate_up, w_down, offsets, counts, row_map=None, covers_all_rows=False):
    """down(silu(gate(x)) * up(x)) per expert. w_gate_up [E, 2*ff, D] (gate rows first), w_down [E, D, ff].
    `row_map` reorders the rows of the result (see grouped_gemm)."""
    hidden = grouped_gemm(x, w_gate_up, offsets, counts, activation=ACT_SWIGLU, covers_all_rows=covers_all_rows)
    return grouped_gemm(hidden, w_down, offsets, counts, row_map=row_map, covers_all_rows=covers_all_rows)


def grouped_gelu_ffn(x, w1, w2, offsets, counts, row_map=None, covers_all_rows=False):
    """fc2(gelu(fc1(x))) per expert, bias-free: the reference's expert (tiny_model.py:68-77).
    w1 [E, ff, D], w2 [E, D, ff], both in nn.Linear layout."""
    hidden = grouped_gemm(x, w1, offsets, counts, activation=ACT_GELU, covers_all_rows=covers_all_rows)
    return grouped_gemm(hidden, w2, offsets, counts, row_map=row_map, covers_all_rows=covers_all_rows)


def grouped_gemm_to_rows(a, w, offsets, counts, row_ptrs):
    """Plain grouped GEMM (no autograd) whose output row r is stored at the ADDRESS row_ptrs[r]
    (int64 [R] on the device; the rows may live in other GPUs' memory). Returns nothing."""
    _check(a, w, offsets, counts)
    if row_ptrs.dtype != torch.int64 or row_ptrs.numel() < a.shape[0]:
        raise ValueError("row_ptrs must be an int64 device tensor with one entry per row of a")
    _launch(a, w, offsets, counts, ACT_NONE, row_ptrs=row_ptrs)
