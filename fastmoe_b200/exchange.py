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
    """Row exchange with gradient. `in_splits[r]` rows go to rank r, `out_splits[r]` come from it.

    The split lists are checked on the host before anything is enqueued: a list of the wrong
    length, a negative count or send counts that do not add up to the rows of `x` raise
    ValueError here, on this rank, instead of surfacing as a mismatched collective that the
    other ranks wait on.
    """
    out_splits, in_splits = [int(n) for n in out_splits], [int(n) for n in in_splits]
    world = dist.get_world_size(group)
    if len(in_splits) != world or len(out_splits) != world:
        raise ValueError(
            f"all_to_all_rows needs one send and one receive count per rank ({world}), got "
            f"{len(in_splits)} and {len(out_splits)}"
        )
    if min(in_splits + out_splits, default=0) < 0:
        raise ValueError(f"negative split size in {in_splits} / {out_splits}")
    if sum(in_splits) != x.shape[0]:
        raise ValueError(f"send counts {in_splits} add up to {sum(in_splits)}, but there are {x.shape[0]} rows to send")
    return _AllToAllRows.apply(x, out_splits, in_splits, group)


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


def regroup_indices(counts_by_source, device, host_counts=None):
    """Row permutations between the arrival order (source rank, then local expert) and the
    order the expert FFN wants (local expert, then source rank).

    counts_by_source: [world, E_local] counts (nested lists or a tensor); counts_by_source[s][e]
    rows came from rank s for local expert e. Returns (to_expert_major, to_rank_major,
    tokens_per_local_expert as a list). A handful of vectorised tensor operations on
    `device`, independent of world * E_local in launch count. Pass the counts as a device
    tensor together with `host_counts` (the same numbers as nested lists) to avoid both a
    host-to-device copy and a read-back.
    """
    if host_counts is not None:  # the caller already holds the counts on the host: no read-back
        host = host_counts
    else:
        host = counts_by_source.tolist() if torch.is_tensor(counts_by_source) else counts_by_source
    world = len(host)
    e_local = len(host[0]) if world else 0
    tokens_per_expert = [sum(host[s][e] for s in range(world)) for e in range(e_local)]
    total = sum(tokens_per_expert)
    if torch.is_tensor(counts_by_source):
        counts = counts_by_source.to(device=device, dtype=torch.int64)
    else:
        counts = torch.tensor(host, dtype=torch.int64).reshape(world, e_local).to(device)
    if total == 0:
        empty = torch.zeros(0, dtype=torch.int64, device=device)
        return empty, empty.clone(), tokens_per_expert
    flat_rm = counts.reshape(-1)  # segments in arrival order (s, e)
    rm_start = torch.cumsum(flat_rm, 0) - flat_rm
    counts_em = counts.t().reshape(-1)  # segments in expert-major order (e, s)
    em_start = torch.cumsum(counts_em, 0) - counts_em
    rm_start_em = rm_start.reshape(world, e_local).t().reshape(-1)  # arrival start of each (e, s) segment
    seg = torch.repeat_interleave(torch.arange(counts_em.numel(), device=device), counts_em, output_size=total)
    to_expert_major = rm_start_em[seg] + (torch.arange(total, device=device) - em_start[seg])
    to_rank_major = torch.empty_like(to_expert_major)
    to_rank_major[to_expert_major] = torch.arange(total, device=device)
    return to_expert_major, to_rank_major, tokens_per_expert


def fused_layout(C: torch.Tensor, rank: int, cap_rows: int, row_bytes: int):
    """Placement arithmetic of the fused (peer-store) exchange, from everybody's per-expert
    counts C[s, e] (rows that rank s routes to global expert e; experts sharded contiguously).
    The statement in tensor operations of what `fmoe_ep_layout` computes on the GPU in two
    small launches: the CUDA path is checked against it, and CPU tests emulate the exchange
    with it.

    Every rank lays out what it receives expert-major, sources in rank order inside an expert.
    Rows that would land at or beyond `cap_rows` do not exist: their senders drop them, and the
    counts the experts see stop there. Returns, all on C's device and with sizes that do not
    depend on the data:
      dst_row0       int64 [E]         row on expert e's owner where THIS rank's rows for e begin
      counts_local   int64 [E_local]   rows this rank receives per local expert (cut off at cap_rows)
      offsets_local  int64 [E_local]   their first rows
      src_rank       int64 [cap_rows]  source rank of every receive-buffer row
      origin_byte    int64 [cap_rows]  byte offset, in the source's sorted-slot buffer, of the slot the
                                       row came from (entries from rows_used on are meaningless)
      rows_used      int64 [1]         rows of the receive buffer in use
    """
    world, E = C.shape
    el = E // world
    C = C.clamp(min=0)
    per_dest = C.view(world, world, el).permute(1, 2, 0).reshape(world, el * world)  # [d, (e, s)]
    seg_start = torch.cumsum(per_dest, 1) - per_dest
    # contiguous: the kernel indexes it by global expert
    dst_row0 = seg_start.view(world, el, world)[:, :, rank].reshape(E).contiguous()
    mine = per_dest[rank]  # sizes of the (e, s) segments this rank receives
    received = mine.view(el, world).sum(1)
    first = torch.cumsum(received, 0) - received
    counts_local = torch.minimum(received, (cap_rows - first).clamp(min=0)).contiguous()
    offsets_local = first.clamp(max=cap_rows).contiguous()
    rows_used = received.sum().clamp(max=cap_rows).reshape(1)
    rows = torch.arange(cap_rows, device=C.device)
    my_start = seg_start[rank]
    seg = torch.searchsorted(my_start + mine, rows, right=True).clamp_(max=el * world - 1)
    src_rank = seg % world
    origin_offsets = torch.cumsum(C, 1) - C  # [s, e]: start of expert e in rank s's sorted rows
    origin_slot = origin_offsets[src_rank, rank * el + seg // world] + (rows - my_start[seg])
    return dst_row0, counts_local, offsets_local, src_rank, (origin_slot * row_bytes).contiguous(), rows_used
