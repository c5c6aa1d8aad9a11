"""Expert-parallel MoE layer with the token exchange fused into the compute kernels.

The NCCL path of `MoEFeedForward` (fastmoe_b200/models/tiny_model.py) moves tokens with
`all_to_all_single` before and after the experts. Here no payload collective runs at all:

  dispatch   the permute kernel stores every routed copy of a token row straight into the
             receive buffer of the GPU that owns its expert, already in expert-major order
             (`fmoe_permute_peer_fwd`, plain peer stores over NVLink);
  return     the down-projection's epilogue stores every output row straight into the
             buffer of the GPU that owns the token, at the slot its combine expects
             (`fmoe_grouped_gemm` with a table of row addresses).

Only the per-expert counts travel through NCCL (one all-gather of world x E integers), and
two one-element all-reduces order the consumers after the writers. Nothing is read back to
the host, so a call enqueues without ever waiting for the GPU. It replaces
dispatch_exchange / compute_experts / combine_exchange of polkadot21/fastmoe
(src/fastmoe/models/tiny_model.py:166-218, :282-294, :308-339) for SwiGLU experts in bf16.

`forward` is the gradient-free call; `forward_with_grad` is the training call, whose backward
sends the gradients the same way (peer-store dispatch of the slot gradients, the gate/up data
gradient's epilogue storing each row back at its owner). Buffers are symmetric allocations (`torch.distributed._symmetric_memory`) mapped
into every rank of the group; multicast is not used.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import exchange
from .kernels import experts, ops, routing
from .kernels.ops import _DTYPES, _status_word, _stream_ptr, grouped_weighted_scatter_add


class FusedExpertParallel:
    """Symmetric buffers and peer tables for one `MoEFeedForward` with SwiGLU experts.

    max_tokens: the largest number of tokens a call will bring on any rank.
    capacity_factor: rows a rank can receive, as a multiple of max_tokens * top_k (its own
    share when routing is even). Rows beyond it are dropped and flagged in the device
    status word (bit 1), so choose it for the skew you expect; world_size is always enough.
    """

    def __init__(self, moe, max_tokens: int, capacity_factor: float = 2.0, group=None):
        if not dist.is_initialized():
            raise RuntimeError("FusedExpertParallel needs an initialised process group")
        if moe.expert_type != "swiglu":
            raise ValueError("the fused path serves SwiGLU experts (expert_type='swiglu')")
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
        self.cap_rows = (self.cap_rows + 127) // 128 * 128
        self._recv = symm_mem.empty(self.cap_rows * self.dim, dtype=torch.bfloat16, device=self.device)
        self._ret = symm_mem.empty(self.max_rows * self.dim, dtype=torch.bfloat16, device=self.device)
        h_recv = symm_mem.rendezvous(self._recv, self.group)
        h_ret = symm_mem.rendezvous(self._ret, self.group)
        self._handles = (h_recv, h_ret)
        self.recv_bases = self._peer_addresses(h_recv, self._recv)
        self.ret_bases = self._peer_addresses(h_ret, self._ret)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._grad = None
        dist.barrier(self.group)

    def _peer_addresses(self, handle, tensor):
        """Device array with the address of `tensor`'s first byte in every rank's mapping. The
        allocator may place the tensor at an offset inside a larger symmetric segment; the
        layout is the same on every rank, so the local offset applies to all of them."""
        bases = list(handle.buffer_ptrs)
        offset = tensor.data_ptr() - bases[self.rank]
        if offset < 0 or offset + tensor.numel() * tensor.element_size() > handle.buffer_size:
            raise RuntimeError("symmetric allocation does not lie inside its rendezvous buffer")
        return torch.tensor([b + offset for b in bases], dtype=torch.int64, device=self.device)

    def _barrier(self):
        """Every rank's earlier work on this stream is complete before anyone's later work starts."""
        dist.all_reduce(self._token, group=self.group)

    # -- the exchange + experts as one differentiable step -------------------------------------
    def _layout(self, counts):
        """From everybody's per-expert counts: where my rows go, what my experts receive and
        where every received row came from. All on the device, fixed-size outputs."""
        world, E = self.world, self.moe.num_experts
        C = torch.empty(world, E, dtype=torch.int64, device=counts.device)
        dist.all_gather_into_tensor(C, counts.contiguous(), group=self.group)
        return exchange.fused_layout(C, self.rank, self.cap_rows, self.dim * 2)

    def _send_rows(self, rows, expert_of_row, slot_of_row, k, offsets, dst_row0, bases):
        """Peer-store dispatch of `rows` ([n, D]; row i carries k routed copies) into `bases`."""
        dev = rows.device
        ops._call(
            "fmoe_permute_peer_fwd", 1, rows.data_ptr(), int(rows.stride(0)), expert_of_row.data_ptr(),
            slot_of_row.data_ptr(), offsets.data_ptr(), dst_row0.data_ptr(), bases.data_ptr(),
            rows.shape[0], k, self.dim, self.moe.num_experts, self.moe.num_local_experts, self.cap_rows,
            _DTYPES[rows.dtype], _status_word(dev).data_ptr(), _stream_ptr(dev),
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

    def experts_over_peers(self, x_flat, topk_idx, ix):
        """Expert outputs for the routed rows of `x_flat`, in this rank's sorted-slot order
        ([T*K, D], a view of the return buffer), differentiable in x_flat and the expert weights."""
        return _FusedExperts.apply(x_flat, self.moe.experts.w_gate_up, self.moe.experts.w_down, topk_idx,
                                   ix.slot_of, ix.offsets, ix.counts, self)  # fmt: skip

    def forward_with_grad(self, x: torch.Tensor) -> torch.Tensor:
        """The layer with gradients for tokens, router and experts; the forward exchange and
        the gradients' exchange both ride on peer stores. One forward/backward pair may be in
        flight per instance (the buffers keep the forward's rows for the backward)."""
        moe, K = self.moe, self.top_k
        B, T, D = x.shape
        n_tok = B * T
        if n_tok * K > self.max_rows or x.dtype != torch.bfloat16:
            raise ValueError("the fused path needs bfloat16 input of at most max_tokens tokens")
        self._grad_buffers()  # collective on first use: here, not inside the backward pass
        self._generation += 1  # a backward of an earlier forward now refuses to run
        x_flat = x.reshape(n_tok, D)
        topk_w, topk_idx = routing.route_topk(moe.router(x_flat), K, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, moe.num_experts, self.world)
        rows = self.experts_over_peers(x_flat, topk_idx, ix)
        out = grouped_weighted_scatter_add([rows], ix.reverse_map, ix.sorted_w, (n_tok, D))
        return out.view(B, T, D)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        moe, world, D, K = self.moe, self.world, self.dim, self.top_k
        B, T, _ = x.shape
        n_tok = B * T
        if n_tok * K > self.max_rows:
            raise ValueError(f"{n_tok} tokens exceed max_tokens={self.max_rows // K} of this FusedExpertParallel")
        if x.dtype != torch.bfloat16:
            raise ValueError("the fused path runs in bfloat16")
        E = moe.num_experts
        x_flat = x.reshape(n_tok, D)
        self._generation += 1  # overwrites the buffers a pending backward would read

        # routing, as in gate_and_sort
        topk_w, topk_idx = routing.route_topk(moe.router(x_flat), K, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, E, world)

        dst_row0, counts_local, offsets_local, src_rank, origin_byte = self._layout(ix.counts)
        self._send_rows(x_flat, topk_idx, ix.slot_of, K, ix.offsets, dst_row0, self.recv_bases)
        self._barrier()  # all rows for my experts have landed

        row_ptrs = (self.ret_bases[src_rank] + origin_byte).contiguous()
        recv = self._recv.view(self.cap_rows, D)
        hidden = experts.grouped_gemm(recv, moe.experts.w_gate_up, offsets_local, counts_local, swiglu=True,
                                      covers_all_rows=True)  # fmt: skip
        experts.grouped_gemm_to_rows(hidden, moe.experts.w_down, offsets_local, counts_local, row_ptrs)
        self._barrier()  # every expert output for my tokens has landed

        ret = self._ret.view(self.max_rows, D)[: n_tok * K]
        out = grouped_weighted_scatter_add([ret], ix.reverse_map, ix.sorted_w, (n_tok, D))
        return out.view(B, T, D)

    __call__ = forward


class _FusedExperts(torch.autograd.Function):
    """rows[slot] = expert(slot)(x[token(slot)]) with both directions of the exchange done by
    peer stores, forward and backward (see FusedExpertParallel)."""

    @staticmethod
    def forward(ctx, x_flat, w_gate_up, w_down, topk_idx, slot_of, offsets, counts, fx):
        D, K = fx.dim, fx.top_k
        n_rows = x_flat.shape[0] * K
        dst_row0, counts_local, offsets_local, src_rank, origin_byte = fx._layout(counts)
        fx._send_rows(x_flat, topk_idx, slot_of, K, offsets, dst_row0, fx.recv_bases)
        fx._barrier()
        recv = fx._recv.view(fx.cap_rows, D)
        hidden = experts._launch(recv, w_gate_up, offsets_local, counts_local, True, covers_all_rows=True)
        row_ptrs = (fx.ret_bases[src_rank] + origin_byte).contiguous()
        experts._launch(hidden, w_down, offsets_local, counts_local, False, row_ptrs=row_ptrs)
        fx._barrier()
        ctx.fx, ctx.k = fx, K
        ctx.generation = fx._generation
        ctx.save_for_backward(w_gate_up, w_down, slot_of, offsets, counts, dst_row0, counts_local,
                              offsets_local, src_rank, origin_byte, hidden)  # fmt: skip
        return fx._ret.view(fx.max_rows, D)[:n_rows]

    @staticmethod
    def backward(ctx, grad_rows):
        (w_gate_up, w_down, slot_of, offsets, counts, dst_row0, counts_local, offsets_local, src_rank,
         origin_byte, hidden) = ctx.saved_tensors  # fmt: skip
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
        g_recv, g_ret, g_recv_bases, g_ret_bases = fx._grad_buffers()
        grad_rows = grad_rows.contiguous()

        # 1. every slot's gradient row goes to the GPU of its expert, at the row its forward copy took
        slots = torch.arange(n_rows, device=dev)
        expert_of_slot = torch.searchsorted(offsets + counts, slots, right=True).clamp_(max=offsets.numel() - 1)
        fx._send_rows(grad_rows, expert_of_slot.contiguous(), slots.to(torch.int32), 1, offsets, dst_row0, g_recv_bases)
        fx._barrier()

        # 2. the experts' backward on the rows this rank received (still in the receive buffer)
        recv = fx._recv.view(fx.cap_rows, D)
        grad_y = g_recv.view(fx.cap_rows, D)
        ff = w_down.shape[2]
        grad_hidden = experts._dgrad(grad_y, w_down, offsets_local, counts_local, covers_all_rows=True)
        grad_w_down = experts._wgrad(grad_y, hidden, w_down.shape, offsets_local, counts_local)
        pre = experts._launch(recv, w_gate_up, offsets_local, counts_local, False, covers_all_rows=True)
        grad_pre = torch.empty_like(pre)
        rows_used = counts_local.sum(dtype=torch.int64).reshape(1)  # the buffers are sized for the worst case
        ops._call("fmoe_swiglu_bwd_ragged", 1, pre.data_ptr(), grad_hidden.data_ptr(), grad_pre.data_ptr(),
                  pre.shape[0], ff, rows_used.data_ptr(), _stream_ptr(dev))  # fmt: skip
        grad_w_gate_up = experts._wgrad(grad_pre, recv, w_gate_up.shape, offsets_local, counts_local)
        # 3. the data gradient's epilogue stores every row back at its owner's slot
        back_ptrs = (g_ret_bases[src_rank] + origin_byte).contiguous()
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
