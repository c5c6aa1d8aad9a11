"""Grouped pointer-table combine: the operator layer of polkadot21/fastmoe on B200.

Same public names, argument order and semantics as the reference module
`src/fastmoe/kernels/ops.py`:

  grouped_weighted_scatter_add (ops.py:365-394), weighted_scatter_add (ops.py:397),
  prepare_grouped_metadata (ops.py:200-271), GroupedWeightedScatterAdd (ops.py:316-359)

Behind them sit hand-written sm_100a CUDA kernels reached through the C ABI of
`libfastmoe_b200.so`. There is no Triton and no CPU path: CPU tensors raise.

Differences from the reference that a caller can observe:
  * the gate weights receive a gradient (the reference's CUDA backward returns
    None for them, ops.py:358-359; its CPU path produces one through autograd);
  * arguments are validated and bad ones raise ValueError before any launch;
  * results are bit-reproducible from run to run in the default "gather" mode.
"""

from __future__ import annotations

import itertools
import operator
import os

import numpy as np
import torch

from .. import _lib

__all__ = [
    "grouped_weighted_scatter_add",
    "weighted_scatter_add",
    "prepare_grouped_metadata",
    "GroupedWeightedScatterAdd",
    "GroupedMetadata",
    "CombinePlan",
    "build_combine_plan",
    "routed_combine",
    "combine_mode",
    "set_combine_mode",
    "read_status",
    "HAS_TRITON",
]

_is_contiguous = torch.Tensor.is_contiguous
_size = torch.Tensor.size
_data_ptr = torch.Tensor.data_ptr
_dtype = operator.attrgetter("dtype")
_get_device = torch.Tensor.get_device
_requires_grad = operator.attrgetter("requires_grad")
_head = operator.itemgetter(0)

# The reference exports this flag (ops.py:10,12); this build never uses Triton.
HAS_TRITON = False

_DTYPES = {torch.float32: _lib.FMOE_F32, torch.bfloat16: _lib.FMOE_BF16, torch.float16: _lib.FMOE_F16}
_ITYPES = {torch.int64: _lib.FMOE_I64, torch.int32: _lib.FMOE_I32}

# "gather": plan (inverse map) + token-major gather, one write per output element.
# "scatter": one launch with vector red.global.add, no scratch memory.
_mode = os.environ.get("FASTMOE_B200_COMBINE", "gather")
_check = os.environ.get("FASTMOE_B200_CHECK", "0") == "1"

_status_words: dict[int, torch.Tensor] = {}
# (device, addresses + offsets + sizes) -> device arrays of prepare_grouped_metadata, a few entries
_table_cache: dict = {}


def combine_mode() -> str:
    return _mode


def set_combine_mode(mode: str) -> None:
    """Selects the combine algorithm: "gather" (default) or "scatter"."""
    global _mode
    if mode not in ("gather", "scatter"):
        raise ValueError(f"combine mode must be 'gather' or 'scatter', got {mode!r}")
    _mode = mode


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels OR error bits into (bad index, null pointer ...)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = word
    return word


def read_status(device=None, reset: bool = True) -> int:
    """Reads (synchronising) and optionally clears the device status word.

    Non-zero means a kernel skipped rows: bit 1 = index outside [0, T),
    bit 2 = row outside its expert, bit 4 = null pointer-table entry.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(device)
    value = int(word.item())
    if reset and value:
        word.zero_()
    return value


def _maybe_check(device: torch.device, what: str) -> None:
    if _check:
        value = read_status(device)
        if value:
            raise RuntimeError(f"{what}: device status word = {value} (rows were skipped)")


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"fastmoe_b200 has no CPU path: `{name}` lives on {t.device}; move it to a CUDA device"
        )


class GroupedMetadata(tuple):
    """The reference's 5-tuple (ptr_table, chunk_sizes, expert_offsets, max_rows, num_experts)
    (ops.py:271), plus what the launch needs to know about the matrices behind the table:
    `num_rows` (sum of the chunk sizes), `dim`, `dtype`, and `keepalive` (contiguous copies
    made for row-strided inputs, so the addresses in the table stay valid)."""

    def __new__(cls, ptr_table, chunk_sizes, expert_offsets, max_rows, num_experts,
                num_rows=None, dim=None, dtype=None, keepalive=None):  # fmt: skip
        self = super().__new__(cls, (ptr_table, chunk_sizes, expert_offsets, max_rows, num_experts))
        self.num_rows, self.dim, self.dtype, self.keepalive = num_rows, dim, dtype, keepalive
        return self


def prepare_grouped_metadata(expert_tensors, device):
    """Pointer table, per-expert row counts and their exclusive prefix sum.

    Same result as the reference (ops.py:200-271): `ptr_table` int64 [E] of raw
    addresses, `chunk_sizes` int32 [E], `expert_offsets` int64 [E], and the Python
    ints `max_rows` and `num_experts`. The table borrows the addresses: it is valid
    only while the same tensors stay alive at the same place (row-strided inputs are
    copied to contiguous rows first, and the copies are kept alive by the result).
    All three arrays travel in one host-to-device copy.
    """
    num_experts = len(expert_tensors)
    if num_experts == 0:
        empty64 = torch.zeros(0, dtype=torch.int64, device=device)
        return GroupedMetadata(empty64, torch.zeros(0, dtype=torch.int32, device=device), empty64, 0, 0, 0)
    ref = expert_tensors[0]
    if ref.dim() != 2:
        raise ValueError(f"expert tensors must be 2-D [rows, D], got shape {tuple(ref.shape)}")
    dim, dtype, dev = ref.shape[1], ref.dtype, ref.device
    keep = None
    # one C-level pass per property: this runs for every MoE layer call with E tensors
    if not all(map(_is_contiguous, expert_tensors)):
        # the kernels read rows at stride D, as the reference kernel does (ops.py:138)
        expert_tensors = [t if t.is_contiguous() else t.contiguous() for t in expert_tensors]
        keep = expert_tensors
    shapes = list(map(_size, expert_tensors))
    if ({len(sh) == 2 and sh[1] for sh in shapes} != {dim} or set(map(_dtype, expert_tensors)) != {dtype}
            or set(map(_get_device, expert_tensors)) != {ref.get_device()}):  # fmt: skip
        for i, t in enumerate(expert_tensors):
            if t.dim() != 2 or t.shape[1] != dim or t.dtype != dtype or t.device != dev:
                raise ValueError(
                    f"expert_tensors[{i}] ({tuple(t.shape)}, {t.dtype}, {t.device}) does not match "
                    f"expert_tensors[0] ([rows, {dim}], {dtype}, {dev})"
                )
    ptrs = list(map(_data_ptr, expert_tensors))
    sizes = list(map(_head, shapes))
    offsets = list(itertools.accumulate(sizes, initial=0))
    run = offsets.pop()
    device = torch.device(device)
    table = ptrs + offsets + sizes
    if device.type == "cuda":
        # The device arrays are a pure function of (addresses, sizes): when the same matrices
        # come back (the caching allocator hands out the same blocks step after step) the
        # arrays of the previous call are reused and nothing is copied.
        key = (device.index, tuple(table))
        cached = _table_cache.get(key)
        if cached is None:
            # pinned staging + asynchronous copy: the host never waits for the stream to drain
            staging = torch.empty(3 * num_experts, dtype=torch.int64, pin_memory=True)
            staging.numpy()[:] = table
            packed = staging.to(device, non_blocking=True)
            cached = (packed[:num_experts], packed[2 * num_experts :].to(torch.int32),
                      packed[num_experts : 2 * num_experts], torch.cuda.current_stream(device), packed)  # fmt: skip
            if len(_table_cache) >= 8:
                _table_cache.pop(next(iter(_table_cache)))
            _table_cache[key] = cached
        elif cached[3] != torch.cuda.current_stream(device):
            # built on another stream: order this stream after the copy that filled it
            current = torch.cuda.current_stream(device)
            current.wait_stream(cached[3])
            cached[4].record_stream(current)  # keep the allocator from recycling it under this stream
            cached[1].record_stream(current)
        ptr_table, chunk_sizes, expert_offsets = cached[:3]
    else:
        packed = torch.from_numpy(np.array(table, dtype=np.int64))
        ptr_table = packed[:num_experts]
        expert_offsets = packed[num_experts : 2 * num_experts]
        chunk_sizes = packed[2 * num_experts :].to(torch.int32)
    return GroupedMetadata(ptr_table, chunk_sizes, expert_offsets, max(sizes), num_experts,
                           run, dim, dtype, keep)  # fmt: skip


def _metadata_for(expert_tensors, indices, metadata):
    """Validated metadata for a launch: built here, or the caller's (trusted, as in the reference)."""
    if metadata is None:
        if len(expert_tensors) == 0:
            raise ValueError("expert_tensors is empty")
        ref = expert_tensors[0]
        _require_cuda(ref, "expert_tensors[0]")
        metadata = prepare_grouped_metadata(expert_tensors, ref.device)
    elif not isinstance(metadata, GroupedMetadata) or metadata.dim is None:
        ref = expert_tensors[0]
        metadata = GroupedMetadata(*metadata, num_rows=int(indices.shape[0]), dim=int(ref.shape[1]), dtype=ref.dtype)
    if metadata.dtype not in _DTYPES:
        raise ValueError(f"unsupported expert dtype {metadata.dtype}; use float32, bfloat16 or float16")
    return metadata


def _check_routing(indices, weights, n_rows):
    _require_cuda(indices, "indices")
    _require_cuda(weights, "weights")
    if indices.dtype not in _ITYPES:
        raise ValueError(f"indices must be int64 or int32, got {indices.dtype}")
    if weights.dtype not in _DTYPES:
        raise ValueError(f"unsupported weights dtype {weights.dtype}")
    if indices.dim() != 1 or weights.dim() != 1:
        raise ValueError("indices and weights must be 1-D")
    if indices.shape[0] != n_rows or weights.shape[0] != n_rows:
        raise ValueError(
            f"indices ({indices.shape[0]}) and weights ({weights.shape[0]}) must have one entry per "
            f"expert row ({n_rows})"
        )
    return indices.contiguous(), weights.contiguous()


class CombinePlan:
    """Device-side inverse of `indices`: per output row, its source rows in ascending
    global row order with resolved addresses and fp32 weights. Holds references to
    everything the stored addresses point into."""

    def __init__(self, buf, n_rows, n_out, dim, dtype, keepalive):
        self.buf, self.n_rows, self.n_out, self.dim, self.dtype = buf, n_rows, n_out, dim, dtype
        self._keepalive = keepalive


def build_combine_plan(expert_tensors, indices, weights, n_out, metadata=None) -> CombinePlan:
    """Builds the plan for out[n_out, D]: one cooperative launch on the current stream (four
    small ones where the sizes rule that out)."""
    metadata = _metadata_for(expert_tensors, indices, metadata)
    ptr_table, chunk_sizes, expert_offsets, _, num_experts = metadata
    n_rows, dim, dtype = metadata.num_rows, metadata.dim, metadata.dtype
    indices, weights = _check_routing(indices, weights, n_rows)
    device = indices.device
    nbytes = _lib.lib().fmoe_combine_plan_bytes(n_rows, n_out)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    # one cooperative launch when the piece totals of the scan fit (see csrc/combine_plan.cu)
    pieces = (n_out + 511) // 512
    _call(
        "fmoe_combine_plan", 1 if 0 < pieces <= min(n_rows, 2048) else 4,
        ptr_table.data_ptr(), chunk_sizes.data_ptr(), expert_offsets.data_ptr(),
        indices.data_ptr(), _ITYPES[indices.dtype], weights.data_ptr(), _DTYPES[weights.dtype],
        num_experts, n_rows, n_out, dim, _DTYPES[dtype],
        buf.data_ptr(), nbytes, _status_word(device).data_ptr(), _stream_ptr(device),
    )  # fmt: skip
    return CombinePlan(buf, n_rows, n_out, dim, dtype, (expert_tensors, metadata, indices, weights))


def _check_out(out, dim, dtype, what="out"):
    _require_cuda(out, what)
    if out.dim() != 2 or out.shape[1] != dim:
        raise ValueError(f"{what} must be [T, {dim}], got {tuple(out.shape)}")
    if out.dtype != dtype:
        raise ValueError(f"{what} dtype {out.dtype} differs from the expert dtype {dtype}")
    if out.shape[1] > 1 and out.stride(1) != 1:
        raise ValueError(f"{what} must have unit column stride")


# Benchmark hooks: number of kernels this package has launched, and (when set to a
# dict) per entry point a list of CUDA event pairs recorded around every call, on the
# stream the kernels are launched on.
launch_count = 0
kernel_events = None


def _call(fn_name, n_kernels, *args):
    """Calls a C-ABI entry point; counts its kernels and, if asked, brackets it with events."""
    global launch_count
    launch_count += n_kernels
    if kernel_events is None:
        return _lib.call(fn_name, *args)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    rc = _lib.call(fn_name, *args)
    ev1.record()
    kernel_events.setdefault(fn_name, []).append((ev0, ev1))
    return rc


def _combine_into(expert_tensors, indices, weights, out, metadata, accumulate, mode=None):
    """Runs the combine into `out` ([T, D], any row stride). Returns the plan (or None)."""
    mode = _mode if mode is None else mode
    metadata = _metadata_for(expert_tensors, indices, metadata)
    dim, dtype = metadata.dim, metadata.dtype
    _check_out(out, dim, dtype)
    device = out.device
    n_out = int(out.shape[0])
    row_stride = int(out.stride(0)) if n_out > 1 else dim
    if mode == "gather":
        plan = build_combine_plan(expert_tensors, indices, weights, n_out, metadata)
        _call(
            "fmoe_combine_gather", 1, plan.buf.data_ptr(), out.data_ptr(), row_stride, plan.n_rows,
            n_out, dim, _DTYPES[dtype], 1 if accumulate else 0, _stream_ptr(device),
        )  # fmt: skip
        _maybe_check(device, "grouped_weighted_scatter_add")
        return plan
    ptr_table, chunk_sizes, expert_offsets, _, num_experts = metadata
    n_rows = metadata.num_rows
    indices, weights = _check_routing(indices, weights, n_rows)
    if not accumulate:
        out.zero_()
    _call(
        "fmoe_combine_scatter", 1,
        ptr_table.data_ptr(), chunk_sizes.data_ptr(), expert_offsets.data_ptr(),
        indices.data_ptr(), _ITYPES[indices.dtype], weights.data_ptr(), _DTYPES[weights.dtype],
        out.data_ptr(), row_stride, num_experts, n_rows, n_out, dim, _DTYPES[dtype],
        _status_word(device).data_ptr(), _stream_ptr(device),
    )  # fmt: skip
    _maybe_check(device, "grouped_weighted_scatter_add")
    return None


class GroupedWeightedScatterAdd(torch.autograd.Function):
    """out[indices[g]] += expert_row_g * weights[g] with gradients for the expert rows
    and the gate weights. Argument order as in the reference (ops.py:318):
    (indices, weights, out_shape, *expert_tensors)."""

    @staticmethod
    def forward(ctx, indices, weights, out_shape, *expert_tensors):
        if len(expert_tensors) == 0:
            raise ValueError("expert_tensors is empty")
        ref = expert_tensors[0]
        _require_cuda(ref, "expert_tensors[0]")
        out_shape = tuple(int(s) for s in out_shape)
        if len(out_shape) != 2:
            raise ValueError(f"out_shape must be (T, D), got {out_shape}")
        # the gather kernel writes every row itself; only the scatter form needs zeros first
        out = torch.empty(out_shape, device=ref.device, dtype=ref.dtype)
        ctx.plan = _combine_into(expert_tensors, indices, weights, out, None, accumulate=False)
        ctx.n_out = out_shape[0]
        ctx.save_for_backward(indices, weights, *expert_tensors)
        ctx.expert_sizes = list(map(_head, map(_size, expert_tensors)))
        ctx.weights_dtype = weights.dtype
        ctx.dim = out_shape[1]
        return out

    @staticmethod
    def backward(ctx, grad_output):
        plan = ctx.plan
        if plan is None:  # forward ran in scatter mode: the backward still wants the inverse map
            indices, weights, *experts = ctx.saved_tensors
            plan = build_combine_plan(experts, indices, weights, ctx.n_out)
        n_rows, dim = plan.n_rows, ctx.dim
        if grad_output.dim() != 2 or (dim > 1 and grad_output.stride(1) != 1):
            grad_output = grad_output.contiguous()
        if grad_output.dtype != plan.dtype:
            grad_output = grad_output.to(plan.dtype)
        device = grad_output.device
        grad_rows = torch.empty(n_rows, dim, device=device, dtype=plan.dtype)
        want_gw = ctx.needs_input_grad[1]
        grad_w = torch.empty(n_rows, device=device, dtype=torch.float32) if want_gw else None
        row_stride = int(grad_output.stride(0)) if grad_output.shape[0] > 1 else dim
        _call(
            "fmoe_combine_bwd", 1, plan.buf.data_ptr(), grad_output.data_ptr(), row_stride,
            grad_rows.data_ptr(), grad_w.data_ptr() if want_gw else None, n_rows, plan.n_out, dim,
            _DTYPES[plan.dtype], _stream_ptr(device),
        )  # fmt: skip
        grad_experts = torch.split(grad_rows, ctx.expert_sizes)
        if want_gw:
            grad_w = grad_w.to(ctx.weights_dtype)
        return None, grad_w, None, *grad_experts


class _RoutedCombine(torch.autograd.Function):
    """out[t] = sum_k rows[slot_of[t*K+k]] * sorted_w[slot_of[t*K+k]]: the combine fed by the
    routing index itself (no plan), with gradients for the rows and the gate weights."""

    @staticmethod
    def forward(ctx, rows, slot_of, sorted_w, K):
        T = slot_of.numel() // K
        D = rows.shape[1]
        out = torch.empty(T, D, dtype=rows.dtype, device=rows.device)
        _call("fmoe_combine_routed", 1, rows.data_ptr(), slot_of.data_ptr(), sorted_w.data_ptr(),
              _DTYPES[sorted_w.dtype], out.data_ptr(), D, T, K, D, _DTYPES[rows.dtype], 0, _stream_ptr(rows.device))  # fmt: skip
        ctx.save_for_backward(rows, slot_of, sorted_w)
        ctx.K = K
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rows, slot_of, sorted_w = ctx.saved_tensors
        K, (N, D) = ctx.K, rows.shape
        T = N // K
        if grad_out.dim() != 2 or (D > 1 and grad_out.stride(1) != 1):
            grad_out = grad_out.contiguous()
        if grad_out.dtype != rows.dtype:
            grad_out = grad_out.to(rows.dtype)
        grad_rows = torch.empty_like(rows)
        want_gw = ctx.needs_input_grad[2]
        grad_w = torch.empty(N, device=rows.device, dtype=torch.float32) if want_gw else None
        row_stride = int(grad_out.stride(0)) if T > 1 else D
        _call("fmoe_combine_routed_bwd", 1, rows.data_ptr(), slot_of.data_ptr(), sorted_w.data_ptr(),
              _DTYPES[sorted_w.dtype], grad_out.data_ptr(), row_stride, grad_rows.data_ptr(),
              grad_w.data_ptr() if want_gw else None, T, K, D, _DTYPES[rows.dtype], _stream_ptr(rows.device))  # fmt: skip
        return grad_rows, None, grad_w.to(sorted_w.dtype) if want_gw else None, None


def routed_combine(rows, slot_of, sorted_w, top_k):
    """The combine for rows that are ONE matrix in the index builder's sorted-slot order:
    out[t] = sum over k of rows[slot_of[t*K+k]] * sorted_w[slot_of[t*K+k]], [T, D] in the rows'
    dtype. `slot_of` (int32 [T*K]) is `build_index`'s inverse map, `sorted_w` the gate weight per
    sorted slot. Equal to `grouped_weighted_scatter_add([rows], reverse_map, sorted_w, (T, D))`
    up to the order of the K additions per token, without building a plan: inside the layer
    the index is already in hand (MoEFeedForward.unpermute, src/fastmoe/models/tiny_model.py:
    396-409). Differentiable in `rows` and `sorted_w`."""
    _require_cuda(rows, "rows")
    _require_cuda(slot_of, "slot_of")
    _require_cuda(sorted_w, "sorted_w")
    if rows.dim() != 2 or rows.dtype not in _DTYPES or sorted_w.dtype not in _DTYPES:
        raise ValueError("rows must be a 2-D float32/bfloat16/float16 matrix and sorted_w a float vector")
    K = int(top_k)
    N = rows.shape[0]
    if slot_of.dtype != torch.int32 or slot_of.numel() != N or sorted_w.numel() != N or K < 1 or N % K:
        raise ValueError(f"slot_of (int32) and sorted_w need one entry per row ({N}), a multiple of top_k={K}")
    D = rows.shape[1]
    if D % (16 // rows.element_size()):
        raise ValueError(f"routed_combine needs a row width that is a multiple of 16 bytes, got D={D}")
    return _RoutedCombine.apply(rows.contiguous(), slot_of.contiguous(), sorted_w.contiguous(), K)


def _needs_grad(expert_tensors, weights):
    if not torch.is_grad_enabled():
        return False
    return weights.requires_grad or any(map(_requires_grad, expert_tensors))


def grouped_weighted_scatter_add(expert_tensors, indices, weights, out_shape, out=None, metadata=None):
    """Sums weighted rows of disjoint per-expert matrices into token rows.

    Same contract as the reference (ops.py:365-394): with `out` given, rows are
    accumulated into it in place (no autograd, no zero-fill, graph-capturable with
    cached `metadata`); otherwise a fresh tensor in the experts' dtype is returned
    through autograd.
    """
    _require_cuda(indices, "indices")
    if out is not None:
        _combine_into(expert_tensors, indices, weights, out, metadata, accumulate=True)
        return out
    if not _needs_grad(expert_tensors, weights):
        # nothing to differentiate: the same launches without handing E tensors to autograd
        if len(expert_tensors) == 0:
            raise ValueError("expert_tensors is empty")
        ref = expert_tensors[0]
        _require_cuda(ref, "expert_tensors[0]")
        out_shape = tuple(int(s) for s in out_shape)
        if len(out_shape) != 2:
            raise ValueError(f"out_shape must be (T, D), got {out_shape}")
        out = torch.empty(out_shape, device=ref.device, dtype=ref.dtype)
        _combine_into(expert_tensors, indices, weights, out, metadata, accumulate=False)
        return out
    return GroupedWeightedScatterAdd.apply(indices, weights, out_shape, *expert_tensors)


def weighted_scatter_add(src, indices, weights, out_shape, out=None):
    """Single-matrix form (ops.py:397-398)."""
    return grouped_weighted_scatter_add([src], indices, weights, out_shape, out)
