"""Expert-parallel MoE layer with the token exchange fused into the compute kernels.

The NCCL path of `MoEFeedForward` (fastmoe_b200/models/tiny_model.py) moves tokens with
`all_to_all_single` before and after the experts. Here no payload collective runs at all:

  dispatch   the permute kernel stores every routed copy of a token row straight into the
             receive buffer of the GPU that owns its expert, already in expert-major order
             (`fmoe_permute_peer_fwd`, plain peer stores over NVLink);
  return     the down-projection's epilogue stores every output row straight into the
             buffer of the GPU that owns the token, at the slot its combine expects
             (`fmoe_grouped_gemm` with a table of row addresses).

Only the per-expert counts travel through NCCL (one all-gather of world x E integers); the
placement arithmetic (`fmoe_ep_layout`) and the barriers that order consumers after writers
(`fmoe_peer_barrier`, flags in symmetric memory, bounded waits) are small kernels of this
library. Nothing is read back to the host, so a call enqueues without ever waiting for the
GPU. It replaces dispatch_exchange / compute_experts / combine_exchange of polkadot21/fastmoe
(src/fastmoe/models/tiny_model.py:166-218, :282-294, :308-339) for SwiGLU experts in bf16.

Overlap. The reference hides the exchange behind compute by splitting the TOKENS into two
micro-batches on two streams (tiny_model.py:506-630). Here each rank's local EXPERTS are
split into `expert_groups` groups instead: the rows of group g+1 cross NVLink (on a side
stream; the copy kernel shares the SMs with the persistent GEMM) while the tensor cores work
on group g, and the down-projection of group g sends its results home from its epilogue.
Rows per expert and weight traffic stay what they are with one group, which token
micro-batches do not achieve (every micro-batch streams all local weights again).

`forward` is the gradient-free call; `forward_with_grad` is the training call, whose backward
sends the gradients the same way (peer-store dispatch of the slot gradients, the gate/up data
gradient's epilogue storing each row back at its owner). Buffers are symmetric allocations
(`torch.distributed._symmetric_memory`) mapped into every rank of the group; multicast is not
used.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib
from .kernels import experts, ops, routing
from .kernels.ops import _DTYPES, _status_word, _stream_ptr, routed_combine


@dataclass
class _Layout:
    """Device-side placement of one call (see `fmoe_ep_layout`)."""

    dst_row0: torch.Tensor  # int64 [E]
    counts_local: torch.Tensor  # int64 [E_local]
    offsets_local: torch.Tensor  # int64 [E_local]
    rows_used: torch.Tensor  # int64 [1]
    row_ptrs: torch.Tensor  # int64 [cap_rows]: where the result of each received row goes
    grad_row_ptrs: torch.Tensor | None  # the same into the gradients' return buffers


class FusedExpertParallel:
    """Symmetric buffers and peer tables for one `MoEFeedForward` with SwiGLU experts.

    max_tokens: the largest number of tokens a call will bring on any rank.
    capacity_factor: rows a rank can receive, as a multiple of max_tokens * top_k (its own
    share when routing is even); world_size is always enough. Copies beyond it are dropped:
    they add zero to their tokens (and get zero gradient), bit 1 of the device status word is
    set on the sender and on the receiver, and `check_status()` turns that into an exception
    at a step boundary of the caller's choice.
    expert_groups: groups the local experts are split into for the overlap described in the
    module docstring (None = 4 with several ranks, fewer if the rank holds fewer experts; 1 in
    a group of one rank, where nothing crosses NVLink). The first group is half an even share.
    barrier_timeout_ms: bound of every wait for the other ranks inside `fmoe_peer_barrier`.
    """

    def __init__(self, moe, max_tokens: int, capacity_factor: float = 2.0, group=None, expert_groups=None,
                 barrier_timeout_ms: int = 20000):  # fmt: skip
        if not dist.is_initialized():
            raise RuntimeError("FusedExpertParallel needs an initialised process group")
        if moe.expert_type != "swiglu":
            raise ValueError("the fused path serves SwiGLU experts (expert_type='swiglu')")
        if capacity_factor <= 0:
            raise ValueError("capacity_factor must be positive")
        # plain peer stores only: keep the allocator from binding the buffers to a multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.moe, self.group = moe, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = moe.router.weight.device
        self.dim, self.top_k = moe.dim, moe.top_k
        self.max_rows = int(max_tokens) * moe.top_k
        self._generation = 0  # forwards run so far: a backward checks that it belongs to the latest
        self.cap_rows = int(min(capacity_factor, self.world) * self.max_rows)
        self.cap_rows = max(128, (self.cap_rows + 127) // 128 * 128)
        el = moe.num_local_experts
        if expert_groups is None:
            expert_groups = min(4, el) if self.world > 1 else 1
        if expert_groups < 1 or expert_groups > el:
            raise ValueError(f"expert_groups={expert_groups} must lie between 1 and the {el} local experts")
        self.expert_groups = int(expert_groups)
        self.group_bounds = self._group_bounds(el, self.expert_groups)
        self.stagger_copies = True  # see _exchange_and_experts
        self.barrier_timeout_ms = int(barrier_timeout_ms)
        self._recv = symm_mem.empty(self.cap_rows * self.dim, dtype=torch.bfloat16, device=self.device)
        self._ret = symm_mem.empty(self.max_rows * self.dim, dtype=torch.bfloat16, device=self.device)
        # barrier flags: two channels (main stream, side stream) of `world` slots each
        self._flags = symm_mem.empty(2 * 32, dtype=torch.int32, device=self.device)
        self._flags.zero_()
        h_recv = symm_mem.rendezvous(self._recv, self.group)
        h_ret = symm_mem.rendezvous(self._ret, self.group)
        h_flags = symm_mem.rendezvous(self._flags, self.group)
        self._handles = (h_recv, h_ret, h_flags)
        self.recv_bases = self._peer_addresses(h_recv, self._recv)
        self.ret_bases = self._peer_addresses(h_ret, self._ret)
        flag_bases = self._peer_addresses(h_flags, self._flags)
        self._flag_bases = (flag_bases, flag_bases + 32 * 4)
        self._seq = [0, 0]
        # group overlap: dispatches on a side stream, the GEMMs on a stream of higher priority, so
        # that the GEMM's CTAs are placed first and the copy kernel's fill what is left of the SMs
        self._side = torch.cuda.Stream(device=self.device)
        self._gemm_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._grad = None
        torch.cuda.synchronize(self.device)  # the flags are zero before anybody's first barrier
        dist.barrier(self.group)

    @staticmethod
    def _group_bounds(el, groups):
        """First local expert of every group, and `el` at the end. The first group is half the
        size of an even share: its rows cross NVLink before any GEMM can start, so it is the one
        part of the exchange that nothing hides; the others share the rest evenly."""
        if groups == 1:
            return [0, el]
        first = max(1, el // (2 * groups))
        rest = el - first
        return [0] + [first + rest * g // (groups - 1) for g in range(groups)]

    def _peer_addresses(self, handle, tensor):
        """Device array with the address of `tensor`'s first byte in every rank's mapping. The
        allocator may place the tensor at an offset inside a larger symmetric segment; the
        layout is the same on every rank, so the local offset applies to all of them."""
        bases = list(handle.buffer_ptrs)
        offset = tensor.data_ptr() - bases[self.rank]
        if offset < 0 or offset + tensor.numel() * tensor.element_size() > handle.buffer_size:
            raise RuntimeError("symmetric allocation does not lie inside its rendezvous buffer")
        return torch.tensor([b + offset for b in bases], dtype=torch.int64, device=self.device)

    def _barrier(self, channel: int = 0):
        """Every rank's earlier work on the current stream is complete before anyone's later
        work on it starts. Channel 0 belongs to the caller's stream, channel 1 to the side
        stream: each channel's flags are written in one stream's order, so they only grow."""
        self._seq[channel] = (self._seq[channel] + 1) & 0x7FFFFFFF
        ops._call("fmoe_peer_barrier", 1, self._flag_bases[channel].data_ptr(), self.world, self.rank,
                  self._seq[channel], self.barrier_timeout_ms, _status_word(self.device).data_ptr(),
                  _stream_ptr(self.device))  # fmt: skip

    def check_status(self) -> None:
        """Reads the device status word (this waits for the GPU) and raises if a call since the
        last check dropped rows for lack of receive capacity or gave up waiting for a peer."""
        value = ops.read_status(self.device)
        if value & _lib.STATUS_WAIT_TIMEOUT:
            raise RuntimeError(f"FusedExpertParallel: a wait for another rank ran out (status word {value})")
        if value:
            raise RuntimeError(
                f"FusedExpertParallel: rows were dropped, the receive buffer of {self.cap_rows} rows was too "
                f"small for the routing skew (status word {value}); raise capacity_factor"
            )

    # -- placement and transport ----------------------------------------------------------------
    def _layout(self, counts, with_grad_ptrs=False) -> _Layout:
        """From everybody's per-expert counts: where my rows go, what my experts receive and
        where every received row came from. All on the device, fixed-size outputs."""
        world, E, el, dev = self.world, self.moe.num_experts, self.moe.num_local_experts, counts.device
        C = torch.empty(world, E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(C, counts.contiguous(), group=self.group)
        i64 = dict(dtype=torch.int64, device=dev)
        out = torch.empty(E + 2 * el + 1, **i64)
        dst_row0, counts_local, offsets_local, rows_used = out[:E], out[E : E + el], out[E + el : E + 2 * el], out[-1:]
        row_ptrs = torch.empty(self.cap_rows, **i64)
        grad_ptrs = torch.empty(self.cap_rows, **i64) if with_grad_ptrs else None
        grad_bases = self._grad_buffers()[3] if with_grad_ptrs else None
        scratch = torch.empty(2 * E, **i64)
        ops._call(
            "fmoe_ep_layout", 2, C.data_ptr(), world, E, self.rank, self.cap_rows, self.dim * 2,
            self.ret_bases.data_ptr(), grad_bases.data_ptr() if with_grad_ptrs else None, dst_row0.data_ptr(),
            counts_local.data_ptr(), offsets_local.data_ptr(), rows_used.data_ptr(), row_ptrs.data_ptr(),
            grad_ptrs.data_ptr() if with_grad_ptrs else None, scratch.data_ptr(),
            _status_word(dev).data_ptr(), _stream_ptr(dev),
        )  # fmt: skip
        return _Layout(dst_row0, counts_local, offsets_local, rows_used, row_ptrs, grad_ptrs)

    def _send_rows(self, rows, expert_of_row, slot_of_row, k, offsets, dst_row0, bases, ret_local, lo=0, hi=None):
        """Peer-store dispatch of `rows` ([n, D]; row i carries k routed copies) into `bases`:
        the copies for local experts [lo, hi) of every rank. A dropped copy's row of `ret_local`
        (this rank's own return buffer) is zeroed."""
        dev = rows.device
        el = self.moe.num_local_experts
        ops._call(
            "fmoe_permute_peer_fwd", 1, rows.data_ptr(), int(rows.stride(0)), expert_of_row.data_ptr(),
            slot_of_row.data_ptr(), offsets.data_ptr(), dst_row0.data_ptr(), bases.data_ptr(),
            rows.shape[0], k, self.dim, self.moe.num_experts, el, self.cap_rows, ret_local.data_ptr(),
            lo, el if hi is None else hi, _DTYPES[rows.dtype], _status_word(dev).data_ptr(), _stream_ptr(dev),
        )  # fmt: skip

    def _grad_buffers(self):
        """Second pair of symmetric buffers, for the gradients' trip (allocated on first use)."""
        if self._grad is None:
            import torch.distributed._symmetric_memory as symm_mem

            g_recv = symm_mem.empty(self.cap_rows * self.dim, dtype=torch.bfloat16, device=self.device)
            g_ret = symm_mem.empty(self.max_rows * self.dim, dtype=torch.bfloat16, device=self.device)
            h1, h2 = symm_mem.rendezvous(g_recv, self.group), symm_mem.rendezvous(g_ret, self.group)
            self._grad = (g_recv, g_ret, self._peer_addresses(h1, g_recv), self._peer_addresses(h2, g_ret), h1, h2)
        return self._grad[:4]

    def _exchange_and_experts(self, x_flat, topk_idx, ix, lay: _Layout, keep_pre=False):
        """Dispatch, both grouped GEMMs and the return trip for all expert groups; ends with the
        barrier after which this rank's return buffer holds every expert output for its tokens.
        Returns the activations between the two GEMMs ([cap_rows, ff]) and, with `keep_pre`, the
        gate/up products before the activation ([cap_rows, 2*ff]): what a backward needs."""
        moe, K, D, G = self.moe, self.top_k, self.dim, self.expert_groups
        el = moe.num_local_experts
        recv = self._recv.view(self.cap_rows, D)
        w_gate_up, w_down = moe.experts.w_gate_up, moe.experts.w_down
        hidden = torch.empty(self.cap_rows, w_down.shape[2], dtype=torch.bfloat16, device=x_flat.device)
        pre = None
        if keep_pre:
            pre = torch.empty(self.cap_rows, w_gate_up.shape[1], dtype=torch.bfloat16, device=x_flat.device)

        def send(lo, hi):
            self._send_rows(x_flat, topk_idx, ix.slot_of, K, ix.offsets, lay.dst_row0, self.recv_bases, self._ret,
                            lo, hi)  # fmt: skip

        def run_experts(lo, hi):
            off, cnt = lay.offsets_local[lo:hi], lay.counts_local[lo:hi]
            experts._launch(recv, w_gate_up[lo:hi], off, cnt, True, out=hidden, pre=pre)
            experts._launch(hidden, w_down[lo:hi], off, cnt, False, row_ptrs=lay.row_ptrs)

        if G == 1:
            send(0, el)
            self._barrier()  # all rows for my experts have landed
            run_experts(0, el)
        else:
            main, side, hi = torch.cuda.current_stream(self.device), self._side, self._gemm_stream
            bounds = self.group_bounds
            side.wait_stream(main)
            hi.wait_stream(main)

            def send_group(g):
                with torch.cuda.stream(side):
                    send(bounds[g], bounds[g + 1])
                    self._barrier(1)  # group g's rows have landed on every rank
                    return side.record_event()

            arrived = send_group(0)
            for g in range(G):
                with torch.cuda.stream(hi):
                    hi.wait_event(arrived)
                    gemm_starts = hi.record_event()
                if g + 1 < G:
                    # the next group's copy starts with this group's gate/up GEMM (which does not
                    # touch NVLink) rather than as soon as the previous copy is done: it then
                    # competes less with the down-projection's stores to the other GPUs
                    if self.stagger_copies:
                        side.wait_event(gemm_starts)
                    arrived = send_group(g + 1)
                with torch.cuda.stream(hi):
                    run_experts(bounds[g], bounds[g + 1])
            with torch.cuda.stream(hi):
                self._barrier()  # every expert output for my tokens has landed
            main.wait_stream(hi)
            return hidden, pre
        self._barrier()  # every expert output for my tokens has landed
        return hidden, pre

    def experts_over_peers(self, x_flat, topk_idx, ix):
        """Expert outputs for the routed rows of `x_flat`, in this rank's sorted-slot order
        ([T*K, D], a view of the return buffer), differentiable in x_flat and the expert weights."""
        return _FusedExperts.apply(x_flat, self.moe.experts.w_gate_up, self.moe.experts.w_down, topk_idx,
                                   ix.slot_of, ix.offsets, ix.counts, self)  # fmt: skip

    def _check_input(self, x):
        n_tok = x.shape[0] * x.shape[1]
        if n_tok * self.top_k > self.max_rows:
            raise ValueError(f"{n_tok} tokens exceed max_tokens={self.max_rows // self.top_k} of this FusedExpertParallel")
        if x.dtype != torch.bfloat16:
            raise ValueError("the fused path runs in bfloat16")
        return n_tok

    def forward_with_grad(self, x: torch.Tensor) -> torch.Tensor:
        """The layer with gradients for tokens, router and experts; the forward exchange and
        the gradients' exchange both ride on peer stores. One forward/backward pair may be in
        flight per instance (the buffers keep the forward's rows for the backward)."""
        moe, K = self.moe, self.top_k
        B, T, D = x.shape
        n_tok = self._check_input(x)
        self._grad_buffers()  # collective on first use: here, not inside the backward pass
        self._generation += 1  # a backward of an earlier forward now refuses to run
        x_flat = x.reshape(n_tok, D)
        topk_w, topk_idx = routing.route_topk(moe.router(x_flat), K, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, moe.num_experts, self.world)
        rows = self.experts_over_peers(x_flat, topk_idx, ix)
        return routed_combine(rows, ix.slot_of, ix.sorted_w, K).view(B, T, D)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        moe, D, K = self.moe, self.dim, self.top_k
        B, T, _ = x.shape
        n_tok = self._check_input(x)
        x_flat = x.reshape(n_tok, D)
        self._generation += 1  # overwrites the buffers a pending backward would read

        # routing, as in gate_and_sort
        topk_w, topk_idx = routing.route_topk(moe.router(x_flat), K, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, moe.num_experts, self.world)
        lay = self._layout(ix.counts)
        self._exchange_and_experts(x_flat, topk_idx, ix, lay)
        ret = self._ret.view(self.max_rows, D)[: n_tok * K]
        return routed_combine(ret, ix.slot_of, ix.sorted_w, K).view(B, T, D)

    __call__ = forward


class _FusedExperts(torch.autograd.Function):
    """rows[slot] = expert(slot)(x[token(slot)]) with both directions of the exchange done by
    peer stores, forward and backward (see FusedExpertParallel)."""

    @staticmethod
    def forward(ctx, x_flat, w_gate_up, w_down, topk_idx, slot_of, offsets, counts, fx):
        D, K = fx.dim, fx.top_k
        n_rows = x_flat.shape[0] * K
        lay = fx._layout(counts, with_grad_ptrs=True)
        ix = routing.RoutingIndex(None, None, counts, offsets, None, slot_of)
        hidden, pre = fx._exchange_and_experts(x_flat, topk_idx, ix, lay, keep_pre=True)
        ctx.fx, ctx.k = fx, K
        ctx.generation = fx._generation
        ctx.save_for_backward(w_gate_up, w_down, slot_of, offsets, counts, lay.dst_row0, lay.counts_local,
                              lay.offsets_local, lay.rows_used, lay.grad_row_ptrs, hidden, pre)  # fmt: skip
        return fx._ret.view(fx.max_rows, D)[:n_rows]

    @staticmethod
    def backward(ctx, grad_rows):
        (w_gate_up, w_down, slot_of, offsets, counts, dst_row0, counts_local, offsets_local, rows_used,
         back_ptrs, hidden, pre) = ctx.saved_tensors  # fmt: skip
        fx, K = ctx.fx, ctx.k
        if ctx.generation != fx._generation:
            raise RuntimeError(
                "FusedExpertParallel: another forward ran on this layer before the backward of an earlier "
                "one; the exchange buffers keep one forward's rows, so those gradients would be wrong. "
                "Run each forward's backward before the next forward (or use the NCCL path)."
            )
        D = fx.dim
        dev = grad_rows.device
        n_rows = grad_rows.shape[0]
        g_recv, g_ret, g_recv_bases, _ = fx._grad_buffers()
        grad_rows = grad_rows.contiguous()

        # 1. every slot's gradient row goes to the GPU of its expert, at the row its forward copy took
        #    (a copy the forward dropped is dropped again, and its gradient row is zeroed)
        slots = torch.arange(n_rows, device=dev)
        expert_of_slot = torch.searchsorted(offsets + counts, slots, right=True).clamp_(max=offsets.numel() - 1)
        fx._send_rows(grad_rows, expert_of_slot.contiguous(), slots.to(torch.int32), 1, offsets, dst_row0,
                      g_recv_bases, g_ret)  # fmt: skip
        fx._barrier()

        # 2. the experts' backward on the rows this rank received (still in the receive buffer)
        recv = fx._recv.view(fx.cap_rows, D)
        grad_y = g_recv.view(fx.cap_rows, D)
        ff = w_down.shape[2]
        grad_hidden = experts._dgrad(grad_y, w_down, offsets_local, counts_local, covers_all_rows=True)
        grad_w_down = experts._wgrad(grad_y, hidden, w_down.shape, offsets_local, counts_local)
        grad_pre = torch.empty_like(pre)  # `pre`: the gate/up products the forward's epilogue kept
        ops._call("fmoe_swiglu_bwd_ragged", 1, pre.data_ptr(), grad_hidden.data_ptr(), grad_pre.data_ptr(),
                  pre.shape[0], ff, rows_used.data_ptr(), _stream_ptr(dev))  # fmt: skip
        grad_w_gate_up = experts._wgrad(grad_pre, recv, w_gate_up.shape, offsets_local, counts_local)
        # 3. the data gradient's epilogue stores every row back at its owner's slot
        experts._dgrad(grad_pre, w_gate_up, offsets_local, counts_local, row_ptrs=back_ptrs)
        fx._barrier()

        # 4. sum the K routed gradients of every token
        T = n_rows // K
        grad_x = torch.empty(T, D, dtype=grad_rows.dtype, device=dev)
        ops._call(
            "fmoe_permute_bwd", 1, g_ret.data_ptr(), slot_of.data_ptr(), grad_x.data_ptr(), D, T, K, D,
            _DTYPES[grad_rows.dtype], _stream_ptr(dev),
        )  # fmt: skip
        return grad_x, grad_w_gate_up, grad_w_down, None, None, None, None, None
