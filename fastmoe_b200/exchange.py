"""Expert-parallel token exchange: counts, payload all-to-all (with gradients) and the
rank-major <-> expert-major bookkeeping on the receiving side.

Pure torch.distributed plumbing (NCCL over NVLink on GPUs, gloo in CPU tests); the
data kernels live elsewhere. Replaces `MoEFeedForward.dispatch_exchange` and
`combine_exchange` of polkadot21/fastmoe (src/fastmoe/models/tiny_model.py:166-218,
:308-339) and corrects two things the reference gets wrong with more than one rank:

  * the receive buffer arrives ordered by (source rank, local expert), but the
    reference splits it as if it were ordered by local expert (:187, :282-294), which
    is only right with one expert per rank; here the rows are regrouped by expert
    before the expert FFN and put back before the return trip;
  * `dist.all_to_all_single` carries no gradient (:210-216, :332-338); here the
    exchange is an autograd Function whose backward is the mirrored exchange.

Only one host synchronisation is needed per layer call (the reference has two,
:187 and :198-199): send and receive counts are read back together.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAllRows(torch.autograd.Function):
    """y = all_to_all_single(x) over dim 0 with uneven splits; backward swaps the splits."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        x = x.contiguous()
        y = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(y, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        grad_y = grad_y.contiguous()
        grad_x = grad_y.new_empty((sum(ctx.in_splits),) + tuple(grad_y.shape[1:]))
        dist.all_to_all_single(
            grad_x, grad_y, output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group
        )
        return grad_x, None, None, None


def all_to_all_rows(x, out_splits, in_splits, group=None):
    """Row exchange with gradient. `in_splits[r]` rows go to rank r, `out_splits[r]` come from it."""
    return _AllToAllRows.apply(x, list(out_splits), list(in_splits), group)


class SplitList(list):
    """A plain list of per-rank row counts (what the reference returns) that also carries
    the receive-side regrouping, so `combine_exchange` can undo it."""

    to_expert_major = None  # int64 [R]: expert-major row i comes from rank-major row to_expert_major[i]
    to_rank_major = None  # its inverse
    counts_by_source = None  # int64 [world, E_local] on the host side as nested lists
    device_counts = None  # the same counts as an int64 device tensor, when one exists


def exchange_counts(send_expert_counts: torch.Tensor, send_rank_counts: torch.Tensor, group=None):
    """One small all-to-all of the per-(rank, local expert) counts, then ONE device-to-host read.

    send_expert_counts: int64 [world, E_local] rows this rank routes to each remote expert.
    Returns (recv_counts device tensor [world(source), E_local], recv_counts as nested lists,
    send_list, recv_list).
    """
    recv_counts = torch.empty_like(send_expert_counts)
    dist.all_to_all_single(recv_counts, send_expert_counts.contiguous(), group=group)
    world = send_expert_counts.shape[0]
    both = torch.cat([recv_counts.reshape(-1), send_rank_counts.reshape(-1)]).tolist()  # the one sync
    flat, send_list = both[: -world], both[-world:]
    e_local = send_expert_counts.shape[1]
    nested = [flat[s * e_local : (s + 1) * e_local] for s in range(world)]
    recv_list = [sum(row) for row in nested]
    return recv_counts, nested, send_list, recv_list


def regroup_indices(counts_by_source, device):
    """Row permutations between the arrival order (source rank, then local expert) and the
    order the expert FFN wants (local expert, then source rank).

    counts_by_source[s][e] rows came from rank s for local expert e. Returns
    (to_expert_major, to_rank_major, tokens_per_local_expert).
    """
    world = len(counts_by_source)
    e_local = len(counts_by_source[0]) if world else 0
    starts, run = [[0] * e_local for _ in range(world)], 0
    for s in range(world):
        for e in range(e_local):
            starts[s][e] = run
            run += counts_by_source[s][e]
    pieces, tokens_per_expert = [], []
    for e in range(e_local):
        total = 0
        for s in range(world):
            n = counts_by_source[s][e]
            if n:
                pieces.append(torch.arange(starts[s][e], starts[s][e] + n))
            total += n
        tokens_per_expert.append(total)
    to_expert_major = torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.int64)
    to_rank_major = torch.empty_like(to_expert_major)
    to_rank_major[to_expert_major] = torch.arange(to_expert_major.numel())
    return to_expert_major.to(device), to_rank_major.to(device), tokens_per_expert
