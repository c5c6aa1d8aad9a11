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

Forward only (inference or activation recomputation); the autograd-capable path is the
NCCL one. Buffers are symmetric allocations (`torch.distributed._symmetric_memory`) mapped
into every rank of the group; multicast is not used.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

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
        self._rows = torch.arange(self.cap_rows, device=self.device)
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

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        moe, world, rank, D, K = self.moe, self.world, self.rank, self.dim, self.top_k
        B, T, _ = x.shape
        n_tok = B * T
        if n_tok * K > self.max_rows:
            raise ValueError(f"{n_tok} tokens exceed max_tokens={self.max_rows // K} of this FusedExpertParallel")
        if x.dtype != torch.bfloat16:
            raise ValueError("the fused path runs in bfloat16")
        E, el = moe.num_experts, moe.num_local_experts
        x_flat = x.reshape(n_tok, D)
        dev = x_flat.device

        # routing, as in gate_and_sort
        topk_w, topk_idx = routing.route_topk(moe.router(x_flat), K, w_dtype=x.dtype)
        ix = routing.build_index(topk_idx, topk_w, E, world)

        # everybody's per-expert counts: C[s, e] rows go from rank s to expert e
        C = torch.empty(world, E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(C, ix.counts.contiguous(), group=self.group)
        # receive layout of rank d: expert-major, sources in rank order inside an expert
        per_dest = C.view(world, world, el).permute(1, 2, 0).reshape(world, el * world)  # [d, (e, s)]
        seg_start = torch.cumsum(per_dest, 1) - per_dest
        # where MY rows of expert e begin on its owner (contiguous: the kernel indexes it by expert)
        dst_row0 = seg_start.view(world, el, world)[:, :, rank].reshape(E).contiguous()

        ops._call(
            "fmoe_permute_peer_fwd", 1, x_flat.data_ptr(), int(x_flat.stride(0)), topk_idx.data_ptr(),
            ix.slot_of.data_ptr(), ix.offsets.data_ptr(), dst_row0.data_ptr(), self.recv_bases.data_ptr(),
            n_tok, K, D, E, el, self.cap_rows, _DTYPES[x.dtype], _status_word(dev).data_ptr(), _stream_ptr(dev),
        )  # fmt: skip
        self._barrier()  # all rows for my experts have landed

        # my experts' problem sizes, from the same counts
        mine = per_dest[rank]  # [(e, s)] sizes of my segments
        counts_local = mine.view(el, world).sum(1).contiguous()
        offsets_local = (torch.cumsum(counts_local, 0) - counts_local).contiguous()
        # return address of every received row: the slot it came from, in its owner's buffer
        my_start = seg_start[rank]
        seg = torch.searchsorted(my_start + mine, self._rows, right=True).clamp_(max=el * world - 1)
        src_rank = seg % world
        origin_offsets = torch.cumsum(C, 1) - C  # [s, e]: start of expert e in rank s's sorted rows
        origin_slot = origin_offsets[src_rank, rank * el + seg // world] + (self._rows - my_start[seg])
        row_ptrs = (self.ret_bases[src_rank] + origin_slot * (D * 2)).contiguous()

        recv = self._recv.view(self.cap_rows, D)
        hidden = experts.grouped_gemm(recv, moe.experts.w_gate_up, offsets_local, counts_local, swiglu=True,
                                      covers_all_rows=True)  # fmt: skip
        experts.grouped_gemm_to_rows(hidden, moe.experts.w_down, offsets_local, counts_local, row_ptrs)
        self._barrier()  # every expert output for my tokens has landed

        ret = self._ret.view(self.max_rows, D)[: n_tok * K]
        out = grouped_weighted_scatter_add([ret], ix.reverse_map, ix.sorted_w, (n_tok, D))
        return out.view(B, T, D)

    __call__ = forward
