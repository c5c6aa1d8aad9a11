"""MoE layer and pipelined block with the module API of polkadot21/fastmoe
(src/fastmoe/models/tiny_model.py), running the dispatch/combine hot path on the
sm_100a kernels of this package.

`MoEFeedForward` keeps the reference's constructor, attributes and stage methods
(gate_and_sort -> dispatch_exchange -> compute_experts -> combine_exchange ->
unpermute, tiny_model.py:42-420). What differs, on purpose:

  * routing is a fused top-k/softmax kernel plus a stable counting sort instead of
    torch.topk/softmax/argsort/bincount, and the dispatch permute and the combine
    are token-major kernels (see fastmoe_b200/kernels);
  * with more than one rank the received rows are regrouped by expert and gradients
    flow through the exchange (the reference does neither, see fastmoe_b200/exchange.py);
  * FAST `forward` hands the per-expert outputs to the grouped combine as separate
    tensors: no torch.cat of expert results;
  * `expert_type="swiglu"` gives bias-free SwiGLU experts (gate/up/down) instead of
    Linear-GELU-Linear;
  * in bf16 with the FAST implementation both expert types run as two grouped tcgen05 GEMM
    launches (activation fused in the first one's epilogue) instead of a Python loop of
    per-expert library calls.

There is no CPU path: inputs must live on a CUDA device.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.profiler import record_function

from .. import consts, exchange
from ..kernels import experts as expert_kernels
from ..kernels import routing
from ..kernels.experts import grouped_gelu_ffn, grouped_swiglu_ffn
from ..kernels.ops import grouped_weighted_scatter_add, routed_combine


class MultiheadSelfAttention(nn.Module):
    """Plain full self-attention (the shell around the MoE layer; tiny_model.py:12-28)."""

    def __init__(self, dim, n_heads):
        super().__init__()
        if dim % n_heads:
            raise ValueError("dim must be divisible by n_heads")
        self.dim, self.n_heads, self.hd = dim, n_heads, dim // n_heads
        self.qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.proj = nn.Linear(dim, dim, bias=False)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(x).view(B, T, 3, self.n_heads, self.hd).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=False)
        return self.proj(y.transpose(1, 2).reshape(B, T, D))


class RoutedShape(tuple):
    """The (B, T) that `gate_and_sort` returns as its last element (tiny_model.py:155-164),
    carrying the index builder's inverse map `slot_of` (int32 [B*T*top_k]: the sorted slot of
    routed copy k of token t) to `unpermute`, which can then combine without building a plan."""

    slot_of = None

    def __new__(cls, shape, slot_of=None):
        self = super().__new__(cls, shape)
        self.slot_of = slot_of
        return self


class GroupedSwiGLUExperts(nn.Module):
    """All local SwiGLU experts as two stacked weight tensors, the layout the grouped GEMM
    reads: `w_gate_up` [E, 2*ff, D] (gate rows, then up rows) and `w_down` [E, D, ff],
    bias-free. Iterating or indexing yields one callable per expert that computes
    down(silu(gate(x)) * up(x)) with plain matrix products."""

    def __init__(self, num_experts, dim, ff_dim):
        super().__init__()
        self.num_experts, self.dim, self.ff_dim = num_experts, dim, ff_dim
        self.w_gate_up = nn.Parameter(torch.empty(num_experts, 2 * ff_dim, dim))
        self.w_down = nn.Parameter(torch.empty(num_experts, dim, ff_dim))
        for w in (self.w_gate_up, self.w_down):  # nn.Linear's default range, without a 22 GB temporary
            bound = 1.0 / w.shape[-1] ** 0.5
            nn.init.uniform_(w, -bound, bound)

    def __len__(self):
        return self.num_experts

    def expert(self, e):
        def run(x):
            h = x @ self.w_gate_up[e].t()
            return (F.silu(h[:, : self.ff_dim]) * h[:, self.ff_dim :]) @ self.w_down[e].t()

        return run

    def __getitem__(self, e):
        return self.expert(e)

    def __iter__(self):
        return (self.expert(e) for e in range(self.num_experts))

    def forward(self, x, offsets, counts, row_map=None):
        """x rows grouped by expert (device-side `offsets`/`counts`, int64 [E], covering every
        row) -> FFN output rows, stored at `row_map[r]` instead of r when a map is given."""
        return grouped_swiglu_ffn(x, self.w_gate_up, self.w_down, offsets, counts, row_map, covers_all_rows=True)


class MoEFeedForward(nn.Module):
    grouped_gelu_min_experts = 16  # local GELU experts from which the FAST bf16 path runs them grouped

    def __init__(self, dim, ff_dim, num_experts, top_k, implementation, group=None, expert_type="gelu"):
        super().__init__()
        self.dim, self.num_experts, self.top_k = dim, num_experts, top_k
        self.implementation, self.group = implementation, group
        if dist.is_initialized():
            self.world_size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world_size, self.rank = 1, 0
        if num_experts % self.world_size:
            raise ValueError(f"num_experts={num_experts} is not divisible by world size {self.world_size}")
        self.num_local_experts = num_experts // self.world_size
        self.router = nn.Linear(dim, num_experts, bias=False)
        self.expert_type = expert_type
        if expert_type == "gelu":
            self.experts = nn.ModuleList(
                nn.Sequential(nn.Linear(dim, ff_dim, bias=False), nn.GELU(), nn.Linear(ff_dim, dim, bias=False))
                for _ in range(self.num_local_experts)
            )
        elif expert_type == "swiglu":
            self.experts = GroupedSwiGLUExperts(self.num_local_experts, dim, ff_dim)
        else:
            raise ValueError(f"expert_type must be 'gelu' or 'swiglu', got {expert_type!r}")

    # -- stage 1 ---------------------------------------------------------------------------
    def gate_and_sort(self, x):
        """Router, top-k gate, expert-major index and the dispatch permute (tiny_model.py:79-164).

        Returns the reference's 6-tuple: (permuted [N, D], rank_counts int64 [world],
        expert_counts_by_rank int64 [world, E_local], reverse_map int64 [N],
        sorted_weights [N], (B, T)).
        """
        B, T, D = x.shape
        x_flat = x.reshape(-1, D)
        logits = self.router(x_flat)
        topk_w, topk_idx = routing.route_topk(logits, self.top_k, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, self.num_experts, self.world_size)
        permuted = routing.permute_rows(x_flat, ix.slot_of, self.top_k)
        by_rank = ix.counts.view(self.world_size, self.num_local_experts)
        return permuted, ix.rank_counts, by_rank, ix.reverse_map, ix.sorted_w, RoutedShape((B, T), ix.slot_of)

    # -- stage 2 ---------------------------------------------------------------------------
    def dispatch_exchange(self, permuted_data, send_rank_counts, send_expert_counts):
        """Sends every routed row to the rank that owns its expert (tiny_model.py:166-218).

        Returns (rows grouped by local expert, recv_splits, send_splits,
        tokens_per_local_expert). One host synchronisation (the counts).
        """
        if self.world_size == 1:
            device_counts = send_expert_counts.view(-1)
            counts = exchange.SplitList(device_counts.tolist())
            counts.device_counts = device_counts
            total = [sum(counts)]
            return permuted_data, total, list(total), counts
        recv_counts, nested, send_list, recv_list = exchange.exchange_counts(
            send_expert_counts, send_rank_counts, self.group
        )
        recv = exchange.all_to_all_rows(permuted_data, recv_list, send_list, self.group)
        splits = exchange.SplitList(recv_list)
        splits.counts_by_source = nested
        tokens_per_expert = exchange.SplitList(sum(nested[s][e] for s in range(self.world_size))
                                               for e in range(self.num_local_experts))  # fmt: skip
        tokens_per_expert.device_counts = recv_counts.sum(dim=0)
        if self.num_local_experts > 1:
            to_expert_major, to_rank_major, _ = exchange.regroup_indices(recv_counts, recv.device, nested)
            splits.to_expert_major, splits.to_rank_major = to_expert_major, to_rank_major
            tokens_per_expert.to_expert_major, tokens_per_expert.to_rank_major = to_expert_major, to_rank_major
            recv = recv.index_select(0, to_expert_major)
        return recv, splits, send_list, tokens_per_expert

    def _pad_per_rank(self, rows, padded_per_rank, real_per_rank):
        """[world * real, D] -> [world * padded, D]: every rank's block is followed by zero rows."""
        block = rows.new_zeros(self.world_size, padded_per_rank, rows.shape[1])
        block[:, :real_per_rank] = rows.view(self.world_size, real_per_rank, rows.shape[1])
        return block.view(-1, rows.shape[1])

    def _static_exchange(self, rows, static_splits, real_tokens_per_rank):
        """Uniform all-to-all of `rows` (the same count to and from every rank, known on the
        host, so nothing is read back). With splits larger than the real count the blocks are
        padded with zero rows before the trip and the padding is cut off after it."""
        splits = list(static_splits)
        padded = splits[0]
        if any(s != padded for s in splits) or len(splits) != self.world_size:
            raise ValueError(f"static_splits must hold one equal count per rank, got {splits}")
        if rows.shape[0] != real_tokens_per_rank * self.world_size or padded < real_tokens_per_rank:
            raise ValueError(
                f"{rows.shape[0]} rows do not make {self.world_size} blocks of {real_tokens_per_rank} "
                f"(padded to {padded})"
            )
        if padded > real_tokens_per_rank:
            rows = self._pad_per_rank(rows, padded, real_tokens_per_rank)
        got = exchange.all_to_all_rows(rows, splits, splits, self.group)
        if padded > real_tokens_per_rank:
            got = got.view(self.world_size, padded, -1)[:, :real_tokens_per_rank].reshape(-1, got.shape[1])
        return got

    def dispatch_exchange_static(self, permuted_data, static_splits, real_tokens_per_rank):
        """Exchange with host-known uniform splits (tiny_model.py:220-280): every rank sends
        `real_tokens_per_rank` rows to every rank, padded to `static_splits[r]` rows on the
        wire. Only meaningful when routing really is uniform over ranks; routed rows beyond a
        rank's block land on the wrong rank, here as in the reference. The exact path is
        `dispatch_exchange`. Returns (rows, static_splits, static_splits)."""
        if self.world_size == 1:
            return permuted_data, static_splits, static_splits
        recv = self._static_exchange(permuted_data, static_splits, real_tokens_per_rank)
        return recv, static_splits, static_splits

    def combine_exchange_static(self, expert_output, static_splits, real_tokens_per_rank):
        """Return trip of `dispatch_exchange_static` (tiny_model.py:341-394). Unlike the
        reference, which copies the real rows to the front of the padded buffer and so hands
        most ranks padding, the padding here follows each rank's block: the round trip
        dispatch -> combine returns every row to where it started, with the same bytes on the wire."""
        if self.world_size == 1:
            return expert_output
        return self._static_exchange(expert_output, static_splits, real_tokens_per_rank)

    # -- stage 3 ---------------------------------------------------------------------------
    def expert_outputs(self, recv_data, tokens_per_expert):
        """One output tensor per local expert, left where each expert wrote it."""
        outs = []
        for chunk, expert in zip(recv_data.split(tokens_per_expert, dim=0), self.experts, strict=False):
            outs.append(expert(chunk) if chunk.shape[0] > 0 else chunk.new_empty(0, self.dim))
        return outs

    def _grouped_ffn(self, recv_data, tokens_per_expert, arrival_order_out=False):
        """Experts on the FAST path in bf16: two grouped-GEMM launches, no per-expert loop.
        With `arrival_order_out` (several ranks, rows regrouped by expert on arrival) the second
        GEMM's epilogue stores every result row at its ARRIVAL position, so that the return
        exchange needs no reordering copy."""
        counts = getattr(tokens_per_expert, "device_counts", None)
        if counts is None:
            staging = torch.tensor(list(tokens_per_expert), dtype=torch.int64, pin_memory=True)
            counts = staging.to(recv_data.device, non_blocking=True)
        offsets = torch.cumsum(counts, 0) - counts
        row_map = getattr(tokens_per_expert, "to_expert_major", None) if arrival_order_out else None
        if self.expert_type == "swiglu":
            return self.experts(recv_data, offsets, counts, row_map)
        # the reference's experts (nn.ModuleList of Linear-GELU-Linear, tiny_model.py:68-77): their
        # weights are stacked into the [E, N, K] layout the grouped GEMM reads; gradients flow
        # back to the individual modules through the stack
        w1 = torch.stack([expert[0].weight for expert in self.experts])
        w2 = torch.stack([expert[2].weight for expert in self.experts])
        if w1.dtype != torch.bfloat16:  # bf16 autocast over fp32 modules: cast as autocast's linear would
            recv_data, w1, w2 = recv_data.bfloat16(), w1.bfloat16(), w2.bfloat16()
        return grouped_gelu_ffn(recv_data, w1, w2, offsets, counts, row_map, covers_all_rows=True)

    @staticmethod
    def _autocast_bf16():
        return torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16

    def _use_grouped(self, recv_data):
        if self.implementation != consts.MoEImplementation.FAST or not recv_data.is_cuda:
            return False
        if self.expert_type == "swiglu":
            return recv_data.dtype == torch.bfloat16
        # GELU experts: bf16 modules and rows, or any under bf16 autocast, only widths the
        # kernels tile (forward and, when training, backward), and only with many experts, where
        # the reference's loop is bound by its 2 x E launches (256 experts of width 256: 243 ->
        # 192 ms per training step). A handful of large experts (8 of 8192 x 8192) run as fast
        # as per-expert library products and need no stacked copy of the weights (measured 259 ms
        # per step in the loop against 282 ms grouped), so everything else keeps the modules,
        # exactly as the reference runs them
        if len(self.experts) < self.grouped_gelu_min_experts:
            return False
        fc1 = self.experts[0][0].weight
        in_bf16 = fc1.dtype == torch.bfloat16 and recv_data.dtype == torch.bfloat16
        if not fc1.is_cuda or not (in_bf16 or self._autocast_bf16()):
            return False
        ff, dim = fc1.shape
        training = torch.is_grad_enabled() and (fc1.requires_grad or recv_data.requires_grad)
        return (expert_kernels.supported(ff, dim, expert_kernels.ACT_GELU, training)
                and expert_kernels.supported(dim, ff, expert_kernels.ACT_NONE, training))  # fmt: skip

    def compute_experts(self, recv_data, tokens_per_expert, arrival_order_out=False):
        """Concatenated expert outputs, rows in the order of recv_data (tiny_model.py:282-294).

        `arrival_order_out=True` (used by `forward` and the pipelined schedule together with
        `combine_exchange(..., rows_in_arrival_order=True)`) returns the rows in the order they
        ARRIVED from the other ranks instead, where that saves a copy; both calls must agree."""
        if self._use_grouped(recv_data):
            return self._grouped_ffn(recv_data, tokens_per_expert, arrival_order_out)
        outs = self.expert_outputs(recv_data, tokens_per_expert)
        out = torch.cat(outs, dim=0) if outs else recv_data.new_empty(0, self.dim)
        to_rank_major = getattr(tokens_per_expert, "to_rank_major", None)
        if arrival_order_out and to_rank_major is not None:
            out = out.index_select(0, to_rank_major)
        return out

    def compute_experts_static(self, recv_data):
        """Experts over equal shares of the rows (tiny_model.py:296-306): local expert e gets
        the e-th of `num_local_experts` chunks, sized as torch.chunk sizes them."""
        n, rows = self.num_local_experts, recv_data.shape[0]
        size = -(-rows // n) if rows else 0
        shares = [max(0, min(size, rows - e * size)) for e in range(n)]
        return self.compute_experts(recv_data, shares)

    # -- stage 4 ---------------------------------------------------------------------------
    def combine_exchange(self, expert_output, recv_splits, send_splits, rows_in_arrival_order=False):
        """Returns expert outputs to the ranks that own the tokens (tiny_model.py:308-339).
        `expert_output` has the row order of what `dispatch_exchange` returned (grouped by local
        expert) unless `rows_in_arrival_order` says that `compute_experts` already put the rows
        back in the order they arrived in (see there)."""
        if self.world_size == 1:
            return expert_output
        to_rank_major = getattr(recv_splits, "to_rank_major", None)
        if to_rank_major is not None and self.num_local_experts > 1 and not rows_in_arrival_order:
            expert_output = expert_output.index_select(0, to_rank_major)
        return exchange.all_to_all_rows(expert_output, list(send_splits), list(recv_splits), self.group)

    # -- stage 5 ---------------------------------------------------------------------------
    def unpermute(self, x_out, reverse_map_indices, sorted_weights, original_shape):
        """Weights every routed row by its gate and sums it into its token (tiny_model.py:396-409)."""
        B, T = original_shape
        D = self.dim
        if self.implementation == consts.MoEImplementation.STANDARD:
            x_out = x_out * sorted_weights.unsqueeze(-1)
            out = torch.zeros(B * T, D, device=x_out.device, dtype=x_out.dtype)
            out.index_add_(0, reverse_map_indices, x_out)
            return out.view(B, T, D)
        if self.implementation == consts.MoEImplementation.FAST:
            slot_of = getattr(original_shape, "slot_of", None)
            if (torch.is_tensor(x_out) and slot_of is not None and x_out.is_cuda and x_out.dim() == 2
                    and x_out.shape[0] == slot_of.numel() == sorted_weights.numel()
                    and x_out.shape[1] % (16 // x_out.element_size()) == 0):  # fmt: skip
                # one matrix in sorted-slot order and the inverse map in hand: no plan to build
                return routed_combine(x_out, slot_of, sorted_weights, self.top_k).view(B, T, D)
            experts = list(x_out) if isinstance(x_out, (list, tuple)) else [x_out]
            out = grouped_weighted_scatter_add(experts, reverse_map_indices, sorted_weights, (B * T, D))
            return out.view(B, T, D)
        raise NotImplementedError

    def enable_fused_exchange(self, max_tokens, capacity_factor=2.0, expert_groups=None):
        """With several ranks and SwiGLU experts: from now on EVERY `forward` of this module,
        with or without gradients, runs with the exchange fused into the permute kernel and
        the GEMM epilogue (peer stores over NVLink, no all-to-all, no host synchronisation; see
        fastmoe_b200/ep_fused.py). Collective: every rank of the group must call it, and from
        then on all ranks take the same path by construction: the choice is made here, once,
        not per call from rank-local conditions. A call the fused path cannot serve (more than
        `max_tokens` tokens, a dtype other than bfloat16) raises ValueError on the rank that
        makes it instead of silently falling back to the all-to-all path, whose collectives
        the other ranks would not match. `disable_fused_exchange()` returns to the NCCL path
        (again on every rank)."""
        from ..ep_fused import FusedExpertParallel

        self._fused_exchange = FusedExpertParallel(self, max_tokens, capacity_factor, self.group, expert_groups)
        return self

    def disable_fused_exchange(self):
        self._fused_exchange = None
        return self

    def forward(self, x):
        fused = getattr(self, "_fused_exchange", None)
        if fused is not None:
            needs_grad = torch.is_grad_enabled() and (
                x.requires_grad or any(p.requires_grad for p in self.parameters()))  # fmt: skip
            return fused.forward_with_grad(x) if needs_grad else fused(x)
        permuted, send_rank_counts, send_exp_counts, rev_idx, weights, shape = self.gate_and_sort(x)
        recv, recv_splits, send_splits, tokens_per_expert = self.dispatch_exchange(
            permuted, send_rank_counts, send_exp_counts
        )
        if (self.world_size == 1 and self.implementation == consts.MoEImplementation.FAST
                and not self._use_grouped(recv)):  # fmt: skip
            # "no-cat": the combine reads the disjoint expert outputs through its pointer table
            return self.unpermute(self.expert_outputs(recv, tokens_per_expert), rev_idx, weights, shape)
        expert_out = self.compute_experts(recv, tokens_per_expert, arrival_order_out=True)
        final = self.combine_exchange(expert_out, recv_splits, send_splits, rows_in_arrival_order=True)
        return self.unpermute(final, rev_idx, weights, shape)


class FeedForward(nn.Module):
    """Dense GELU feed-forward of the non-MoE block (tiny_model.py:32-39)."""

    def __init__(self, dim, ff_dim):
        super().__init__()
        self.fc1 = nn.Linear(dim, ff_dim, bias=False)
        self.fc2 = nn.Linear(ff_dim, dim, bias=False)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


class _ResidualBlock(nn.Module):
    """Pre-norm attention and feed-forward with residual connections; `self.ff` is set by the subclass."""

    def __init__(self, dim, n_heads):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = MultiheadSelfAttention(dim, n_heads)
        self.norm2 = nn.LayerNorm(dim)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.ff(self.norm2(x))


class Block(_ResidualBlock):
    """Dense transformer block (tiny_model.py:424-435)."""

    def __init__(self, dim, n_heads, ff_dim):
        super().__init__(dim, n_heads)
        self.ff = FeedForward(dim, ff_dim)


class MoEBlock(_ResidualBlock):
    """Transformer block whose feed-forward is a `MoEFeedForward` (tiny_model.py:438-463)."""

    def __init__(self, dim, n_heads, ff_dim, num_experts, top_k, implementation, expert_type="gelu"):
        super().__init__(dim, n_heads)
        self.ff = MoEFeedForward(dim, ff_dim, num_experts, top_k, implementation, expert_type=expert_type)


class PipelinedMoEBlock(nn.Module):
    """Attention + MoE block that splits the batch into micro-batches and overlaps one
    micro-batch's token exchange with another's compute on separate CUDA streams
    (tiny_model.py:466-630 uses two micro-batches on `stream0`/`stream1`; here
    `num_micro_batches` may be larger and further streams are created on demand).
    Exchanges are the exact, dynamically sized ones. Left at None, the number of micro-batches
    is 2 with several ranks and 1 with a single rank: without an exchange there is nothing to
    overlap, and splitting the batch only doubles the per-expert launches."""

    def __init__(self, dim, n_heads, ff_dim, num_experts, top_k, stream0, stream1,
                 comm_balance_factor=1, num_micro_batches=None, expert_type="gelu"):  # fmt: skip
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = MultiheadSelfAttention(dim, n_heads)
        self.norm2 = nn.LayerNorm(dim)
        self.moe = MoEFeedForward(dim, ff_dim, num_experts, top_k, consts.MoEImplementation.FAST,
                                  expert_type=expert_type)  # fmt: skip
        self.stream0, self.stream1 = stream0, stream1
        self.comm_balance_factor = comm_balance_factor  # kept for signature parity; padding is never sent
        self.num_micro_batches = num_micro_batches
        self._extra_streams = []

    def _streams(self, n):
        if self.stream0 is None:  # a caller without streams of its own gets two from the block
            self.stream0 = torch.cuda.Stream()
        if self.stream1 is None:
            self.stream1 = torch.cuda.Stream()
        streams = [self.stream0, self.stream1]
        while len(streams) + len(self._extra_streams) < n:
            self._extra_streams.append(torch.cuda.Stream())
        return (streams + self._extra_streams)[:n]

    def forward(self, x):
        n_mb = self.num_micro_batches
        if n_mb is None:
            n_mb = 2 if self.moe.world_size > 1 else 1
        if n_mb == 1 or getattr(self.moe, "_fused_exchange", None) is not None:
            # nothing to overlap here: one micro-batch, or the fused exchange, which overlaps the
            # dispatch of one expert group with the GEMMs of the previous one inside the layer
            x = x + self.attn(self.norm1(x))
            return x + self.moe(self.norm2(x))
        chunks = x.chunk(n_mb, dim=0)
        streams = self._streams(len(chunks))
        main = torch.cuda.current_stream()
        resid, moe_in = [], []
        prev_attn_done = None
        # attention per micro-batch, staggered: micro-batch i+1's attention overlaps i's exchange
        for i, (mb, s) in enumerate(zip(chunks, streams)):
            s.wait_stream(main)
            with torch.cuda.stream(s):
                if prev_attn_done is not None:
                    s.wait_event(prev_attn_done)
                with record_function(f"S{i}: Attn {i}"):
                    r = mb + self.attn(self.norm1(mb))
                    resid.append(r)
                    moe_in.append(self.norm2(r))
                prev_attn_done = torch.cuda.Event()
                prev_attn_done.record()
        moe_out = pipelined_moe_forward(self.moe, moe_in, streams)
        outs = []
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                y = moe_out[i] + resid[i]
                y.record_stream(main)  # read by the concatenation on the caller's stream
                outs.append(y)
            main.wait_stream(s)
        return torch.cat(outs, dim=0)


def pipelined_moe_forward(moe, inputs, streams):
    """Runs `moe` on several micro-batches, one CUDA stream each, issuing the work so that
    the token exchange of micro-batch i+1 is in flight while micro-batch i's experts compute:

        gate(0..n-1) ; dispatch(0) ; for i: dispatch(i+1), experts(i), combine(i)

    (the software-pipelined form of the two-stream zig-zag of polkadot21/fastmoe,
    src/fastmoe/models/tiny_model.py:506-630, for any number of micro-batches). Collectives
    of one process group execute in issue order, which is why dispatch(i+1) is issued before
    combine(i). Returns the per-micro-batch outputs, each produced on its own stream.
    """
    n = len(inputs)
    gated, dispatched, outs = [None] * n, [None] * n, [None] * n
    for i in range(n):
        with torch.cuda.stream(streams[i]), record_function(f"S{i}: Gate {i}"):
            gated[i] = moe.gate_and_sort(inputs[i])

    def dispatch(i):
        with torch.cuda.stream(streams[i]), record_function(f"S{i}: Dispatch {i}"):
            perm, rank_counts, exp_counts, _, _, _ = gated[i]
            dispatched[i] = moe.dispatch_exchange(perm, rank_counts, exp_counts)

    if n:
        dispatch(0)
    experts_done = None
    for i in range(n):
        if i + 1 < n:
            dispatch(i + 1)
        with torch.cuda.stream(streams[i]):
            _, _, _, rev, w, shape = gated[i]
            recv, recv_splits, send_splits, tokens = dispatched[i]
            if experts_done is not None:
                # one micro-batch's experts at a time: two persistent GEMMs sharing the SMs
                # finish later than either alone and delay the return exchange they feed
                streams[i].wait_event(experts_done)
            with record_function(f"S{i}: Experts {i}"):
                eo = moe.compute_experts(recv, tokens, arrival_order_out=True)
            experts_done = torch.cuda.Event()
            experts_done.record()
            with record_function(f"S{i}: Combine {i}"):
                fd = moe.combine_exchange(eo, recv_splits, send_splits, rows_in_arrival_order=True)
            with record_function(f"S{i}: Finalize {i}"):
                outs[i] = moe.unpermute(fd, rev, w, shape)
        gated[i] = dispatched[i] = None
    return outs


class TinyModel(nn.Module):
    """Input projection, `n_layers` blocks, output projection (tiny_model.py:634-699).

    The block type follows the reference: dense `Block` without MoE, `MoEBlock` for the
    STANDARD implementation, `PipelinedMoEBlock` for FAST. `top_k`, `stream0` and `stream1`
    may be left out (the reference's own training benchmark calls the constructor without
    them, run_on_cloud.py:111-121, which its signature rejects): top_k then defaults to 2
    and the pipelined blocks create their streams on first use.
    """

    def __init__(self, in_dim, dim, n_heads, ff_dim, n_layers, num_experts=None, top_k=None,
                 implementation=None, stream0=None, stream1=None, comm_balance_factor=1, *,
                 use_moe, expert_type="gelu", num_micro_batches=None):  # fmt: skip
        super().__init__()
        self.inp = nn.Linear(in_dim, dim, bias=False)
        if use_moe:
            if num_experts is None:
                raise ValueError("use_moe=True needs num_experts")
            top_k = 2 if top_k is None else top_k
        if not use_moe:
            blocks = [Block(dim, n_heads, ff_dim) for _ in range(n_layers)]
        elif implementation == consts.MoEImplementation.STANDARD:
            blocks = [MoEBlock(dim, n_heads, ff_dim, num_experts, top_k, implementation, expert_type)
                      for _ in range(n_layers)]  # fmt: skip
        elif implementation == consts.MoEImplementation.FAST:
            blocks = [PipelinedMoEBlock(dim, n_heads, ff_dim, num_experts, top_k, stream0, stream1,
                                        comm_balance_factor, num_micro_batches, expert_type)
                      for _ in range(n_layers)]  # fmt: skip
        else:
            raise NotImplementedError(f"implementation {implementation!r}")
        self.blocks = nn.ModuleList(blocks)
        self.out = nn.Linear(dim, in_dim, bias=False)

    def forward(self, x):
        x = self.inp(x)
        for block in self.blocks:
            x = block(x)
        return self.out(x)
