"""Router top-k/softmax, index-offset builder and dispatch permute on the GPU.

Host wrappers (with autograd) over the C-ABI kernels that replace the routing half
of `MoEFeedForward.gate_and_sort` in polkadot21/fastmoe
(src/fastmoe/models/tiny_model.py:94-153):

  route_topk        torch.topk + softmax(dtype=fp32).type_as(x)        (:97-100)
  build_index       argsort + gathers + bincount + per-rank sums       (:105-153)
  permute_rows      x_flat[reverse_map]                                (:133)

The sorted order is the stable one (expert id, then flat routed position t*K+k);
the reference's own order inside an expert segment is whatever an unstable
torch.argsort returns (:112).
"""

from __future__ import annotations

from typing import NamedTuple

import torch

from .. import _lib
from . import ops
from .ops import _DTYPES, _require_cuda, _status_word, _stream_ptr


class RoutingIndex(NamedTuple):
    reverse_map: torch.Tensor  # int64 [N] token of each sorted slot
    sorted_w: torch.Tensor  # [N] gate weight of each sorted slot
    counts: torch.Tensor  # int64 [E] rows per expert
    offsets: torch.Tensor  # int64 [E] exclusive prefix sum of counts
    rank_counts: torch.Tensor  # int64 [world] rows per owning rank
    slot_of: torch.Tensor  # int32 [N] sorted position of routed slot t*K+k


class _RouteTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, K, w_dtype):
        _require_cuda(logits, "logits")
        if logits.dim() != 2:
            raise ValueError(f"logits must be [T, E], got {tuple(logits.shape)}")
        if logits.dtype not in _DTYPES:
            raise ValueError(f"unsupported logits dtype {logits.dtype}")
        logits = logits.contiguous()
        T, E = logits.shape
        topk_idx = torch.empty(T, K, dtype=torch.int64, device=logits.device)
        topk_w = torch.empty(T, K, dtype=w_dtype, device=logits.device)
        ops._call(
            "fmoe_route_topk", 1, logits.data_ptr(), _DTYPES[logits.dtype], T, E, K,
            topk_idx.data_ptr(), topk_w.data_ptr(), _DTYPES[w_dtype], _stream_ptr(logits.device),
        )  # fmt: skip
        ctx.save_for_backward(topk_w, topk_idx)
        ctx.shape, ctx.logits_dtype = (T, E), logits.dtype
        ctx.mark_non_differentiable(topk_idx)
        return topk_w, topk_idx

    @staticmethod
    def backward(ctx, grad_w, _grad_idx):
        # softmax over the K selected logits: dv = w * (g - sum(g * w)); everything else gets 0
        topk_w, topk_idx = ctx.saved_tensors
        w = topk_w.float()
        g = grad_w.float()
        dv = w * (g - (g * w).sum(-1, keepdim=True))
        grad_logits = torch.zeros(ctx.shape, dtype=torch.float32, device=grad_w.device)
        grad_logits.scatter_(1, topk_idx, dv)
        return grad_logits.to(ctx.logits_dtype), None, None


def route_topk(logits: torch.Tensor, K: int, w_dtype: torch.dtype | None = None):
    """(topk_weights [T, K], topk_indices int64 [T, K]): the K largest logits per token in
    descending order (ties: lower expert first) and their softmax, computed in fp32 and
    rounded to `w_dtype` (default: the logits' dtype)."""
    return _RouteTopK.apply(logits, int(K), logits.dtype if w_dtype is None else w_dtype)


class _BuildIndex(torch.autograd.Function):
    @staticmethod
    def forward(ctx, topk_w, topk_idx, E, world):
        _require_cuda(topk_idx, "topk_idx")
        if topk_idx.dtype != torch.int64 or topk_idx.dim() != 2 or topk_w.shape != topk_idx.shape:
            raise ValueError("topk_idx must be int64 [T, K] and topk_w must have the same shape")
        if topk_w.dtype not in _DTYPES:
            raise ValueError(f"unsupported weight dtype {topk_w.dtype}")
        topk_idx, topk_w = topk_idx.contiguous(), topk_w.contiguous()
        T, K = topk_idx.shape
        N, dev = T * K, topk_idx.device
        reverse_map = torch.empty(N, dtype=torch.int64, device=dev)
        sorted_w = torch.empty(N, dtype=topk_w.dtype, device=dev)
        meta = torch.empty(2 * E + world, dtype=torch.int64, device=dev)
        counts, offsets, rank_counts = meta[:E], meta[E : 2 * E], meta[2 * E :]
        slot_of = torch.empty(N, dtype=torch.int32, device=dev)
        nbytes = _lib.lib().fmoe_build_index_bytes(T, E, K)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        ops._call(
            "fmoe_build_index", 3, topk_idx.data_ptr(), topk_w.data_ptr(), _DTYPES[topk_w.dtype], T, E, K,
            world, reverse_map.data_ptr(), sorted_w.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
            rank_counts.data_ptr(), slot_of.data_ptr(), scratch.data_ptr(), nbytes,
            _status_word(dev).data_ptr(), _stream_ptr(dev),
        )  # fmt: skip
        ctx.save_for_backward(slot_of)
        ctx.shape = (T, K)
        ctx.mark_non_differentiable(reverse_map, counts, offsets, rank_counts, slot_of)
        return sorted_w, reverse_map, counts, offsets, rank_counts, slot_of

    @staticmethod
    def backward(ctx, grad_sorted_w, *_):
        (slot_of,) = ctx.saved_tensors
        return grad_sorted_w[slot_of.long()].view(ctx.shape), None, None, None


def build_index(topk_idx: torch.Tensor, topk_w: torch.Tensor, E: int, world: int = 1) -> RoutingIndex:
    """Stable counting sort of the routed slots by expert (histogram + prefix sum + placement)."""
    if E % world != 0:
        raise ValueError(f"E={E} is not divisible by world={world}")
    sorted_w, reverse_map, counts, offsets, rank_counts, slot_of = _BuildIndex.apply(
        topk_w, topk_idx, int(E), int(world)
    )
    return RoutingIndex(reverse_map, sorted_w, counts, offsets, rank_counts, slot_of)


class _PermuteRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, slot_of, K):
        _require_cuda(x, "x")
        if x.dim() != 2 or x.dtype not in _DTYPES:
            raise ValueError(f"x must be a 2-D float32/bfloat16/float16 tensor, got {tuple(x.shape)} {x.dtype}")
        if x.shape[1] > 1 and x.stride(1) != 1:
            x = x.contiguous()
        T, D = x.shape
        if slot_of.dtype != torch.int32 or slot_of.numel() != T * K:
            raise ValueError("slot_of must be int32 with T*K entries")
        out = torch.empty(T * K, D, dtype=x.dtype, device=x.device)
        row_stride = int(x.stride(0)) if T > 1 else D
        ops._call(
            "fmoe_permute_fwd", 1, x.data_ptr(), row_stride, slot_of.data_ptr(), out.data_ptr(), T, K, D,
            _DTYPES[x.dtype], _stream_ptr(x.device),
        )  # fmt: skip
        ctx.save_for_backward(slot_of)
        ctx.dims = (T, K, D)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (slot_of,) = ctx.saved_tensors
        T, K, D = ctx.dims
        grad_out = grad_out.contiguous()
        grad_x = torch.empty(T, D, dtype=grad_out.dtype, device=grad_out.device)
        ops._call(
            "fmoe_permute_bwd", 1, grad_out.data_ptr(), slot_of.data_ptr(), grad_x.data_ptr(), D, T, K, D,
            _DTYPES[grad_out.dtype], _stream_ptr(grad_out.device),
        )  # fmt: skip
        return grad_x, None, None


def permute_rows(x: torch.Tensor, slot_of: torch.Tensor, K: int) -> torch.Tensor:
    """permuted[slot_of[t*K+k]] = x[t]: the dispatch permute, each token row read once.
    Backward sums the K routed gradient rows of a token in fp32."""
    return _PermuteRows.apply(x, slot_of, int(K))
