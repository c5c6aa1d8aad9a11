"""Seeded synthetic workloads with the shapes and value distributions of the
benchmark configurations (combine microbenchmark, skewed combine, dispatch+combine
under autograd). Routing is drawn on the CPU generator so that it is identical on
every machine; payload rows are drawn on the device generator.

The reference's microbenchmark builds its inputs the same way, at a smaller scale
(polkadot21/fastmoe, src/fastmoe/benchmarks/run_on_cloud.py:207-226).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


def routing_softmax(T: int, E: int, K: int, seed: int):
    """Router logits N(0,1) -> top-K -> softmax over the selected logits in fp32."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    vals, idx = torch.topk(logits, K, dim=-1)
    return idx, torch.softmax(vals, dim=-1, dtype=torch.float32)


def routing_zipf(T: int, E: int, K: int, seed: int, s: float = 1.2):
    """K distinct experts per token with p(e) ~ (e+1)^-s; gate weights Dirichlet(1)."""
    g = torch.Generator().manual_seed(seed)
    p = (torch.arange(E, dtype=torch.float64) + 1.0) ** (-s)
    idx = torch.multinomial((p / p.sum()).expand(T, E), K, replacement=False, generator=g)
    expo = -torch.log(torch.rand(T, K, generator=g, dtype=torch.float64).clamp_min(1e-300))
    return idx, (expo / expo.sum(-1, keepdim=True)).float()


def routing_uniform(T: int, E: int, K: int, seed: int):
    """K distinct experts per token, uniformly; softmax of N(0,1) gate logits."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.rand(T, E, generator=g).topk(K, dim=-1).indices
    return idx, torch.softmax(torch.randn(T, K, generator=g), dim=-1)


ROUTINGS = {"softmax": routing_softmax, "zipf": routing_zipf, "uniform": routing_uniform}


def sort_routing(topk_idx: torch.Tensor, topk_w: torch.Tensor, E: int):
    """Expert-major stable order of the T*K routed slots: (reverse_map, sorted_w, counts)."""
    T, K = topk_idx.shape
    flat = topk_idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    reverse_map = torch.arange(T).repeat_interleave(K)[order]
    return reverse_map, topk_w.reshape(-1)[order], torch.bincount(flat, minlength=E)


@dataclass
class CombineWorkload:
    experts: list  # E separately allocated [n_e, D] tensors on the device
    indices: torch.Tensor  # int64 [N] target token of each routed row
    weights: torch.Tensor  # [N] gate weights in the payload dtype
    counts: list  # rows per expert
    T: int
    D: int
    topk_idx: torch.Tensor  # CPU int64 [T, K]
    topk_w: torch.Tensor  # CPU fp32 [T, K]
    spacers: list = field(default_factory=list)  # keep the expert tensors apart in memory

    @property
    def N(self) -> int:
        return int(self.indices.shape[0])

    def algorithmic_bytes(self) -> int:
        """Bytes a perfect combine moves: every source row read once, every output
        element written once, plus the index, weight and table entries."""
        es = self.experts[0].element_size()
        return (self.N * self.D * es + self.T * self.D * es
                + self.N * (self.indices.element_size() + self.weights.element_size())
                + len(self.experts) * 20)  # fmt: skip


def make_combine_workload(T, D, E, K, dtype=torch.bfloat16, routing="softmax", seed=0, device="cuda"):
    """E disjoint expert output matrices with N(0,1) rows plus expert-major routing.

    routing="random_targets" reproduces the reference microbenchmark's inputs instead
    (src/fastmoe/benchmarks/run_on_cloud.py:207-214): T*K rows split evenly over the experts,
    every row aimed at a uniformly random token (duplicates and untouched tokens included),
    uniform(0,1) weights."""
    if routing == "random_targets":
        g = torch.Generator().manual_seed(seed)
        n = T * K
        reverse_map = torch.randint(0, T, (n,), generator=g)
        sorted_w = torch.rand(n, generator=g)
        counts = torch.tensor([len(c) for c in torch.arange(n).chunk(E)] + [0] * max(0, E - n), dtype=torch.int64)[:E]
        topk_idx = torch.zeros(0, K, dtype=torch.int64)
        topk_w = torch.zeros(0, K)
    else:
        topk_idx, topk_w = ROUTINGS[routing](T, E, K, seed)
        reverse_map, sorted_w, counts = sort_routing(topk_idx, topk_w, E)
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    experts, spacers = [], []
    for e, n in enumerate(counts.tolist()):
        experts.append(torch.randn(n, D, generator=gen, device=device, dtype=dtype))
        # an odd-sized allocation between neighbours keeps the matrices non-contiguous
        spacers.append(torch.empty(4096 + 512 * (e % 7), dtype=torch.uint8, device=device))
    return CombineWorkload(
        experts=experts,
        indices=reverse_map.to(device),
        weights=sorted_w.to(dtype).to(device),
        counts=counts.tolist(),
        T=T,
        D=D,
        topk_idx=topk_idx,
        topk_w=topk_w,
        spacers=spacers,
    )
