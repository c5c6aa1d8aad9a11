"""Generates the golden fixtures in this directory by running the REFERENCE's own
CPU/PyTorch path (polkadot21/fastmoe, imported unchanged from a source checkout).

    python tests/golden/make_golden.py /path/to/reference

The reference checkout exists only where the fixtures are made; tests read the
committed .npz files and never import the reference. Inputs are stored in the
fixtures (they are small); the config-1 layer fixture stores its weights' seed
and a checksum instead, and regenerates them with numpy's PCG64.

bf16 tensors are stored as uint16 bit patterns.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/a/checkout/of/polkadot21/fastmoe")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "src"))

sys.path.insert(0, str(HERE))

from fastmoe.consts import MoEImplementation  # noqa: E402
from make_inputs import layer_cfg1_weights  # noqa: E402
from fastmoe.kernels.ops import (  # noqa: E402
    grouped_weighted_scatter_add,
    prepare_grouped_metadata,
    weighted_scatter_add,
)
from fastmoe.models.tiny_model import MoEFeedForward  # noqa: E402

torch.set_num_threads(1)  # one thread: summation orders are the sequential ones


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def scatter_add_small():
    """The shape of the reference's only numeric test (tests/test_cpu_moe.py:94-114)."""
    rng = np.random.default_rng(1)
    N, D, T = 10, 4, 5
    src = rng.standard_normal((N, D)).astype(np.float32)
    w = rng.random(N).astype(np.float32)
    idx = rng.integers(0, T, N).astype(np.int64)
    out = weighted_scatter_add(torch.from_numpy(src), torch.from_numpy(idx), torch.from_numpy(w), (T, D))
    loop = torch.zeros(T, D)  # the test's own per-row ground truth
    for i in range(N):
        loop[int(idx[i])] += torch.from_numpy(src[i]) * float(w[i])
    np.savez(HERE / "scatter_add_small.npz", src=src, w=w, idx=idx, out=out.numpy(), out_loop=loop.numpy())


def grouped(name, sizes, D, T, seed, idx_mode="random"):
    rng = np.random.default_rng(seed)
    N = int(sum(sizes))
    rows = rng.standard_normal((N, D)).astype(np.float32)
    w = rng.random(N).astype(np.float32)
    idx = rng.integers(0, T, N).astype(np.int64)
    if idx_mode == "one_target":
        idx[:] = T // 2
    grad_out = rng.standard_normal((T, D)).astype(np.float32)
    out0 = rng.standard_normal((T, D)).astype(np.float32)
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)

    def run(dtype):
        ex = [torch.from_numpy(rows[offs[e] : offs[e + 1]]).to(dtype).requires_grad_(True) for e in range(len(sizes))]
        wt = torch.from_numpy(w).to(dtype).requires_grad_(True)
        it = torch.from_numpy(idx)
        out = grouped_weighted_scatter_add(ex, it, wt, (T, D))
        out.backward(torch.from_numpy(grad_out).to(dtype))
        acc = torch.from_numpy(out0).to(dtype).clone()
        with torch.no_grad():
            grouped_weighted_scatter_add([e.detach() for e in ex], it, wt.detach(), (T, D), out=acc)
        g_rows = torch.cat([e.grad if e.grad is not None else torch.zeros_like(e) for e in ex], 0)
        return out.detach(), g_rows, wt.grad, acc

    out, g_rows, g_w, acc = run(torch.float32)
    d = dict(sizes=np.array(sizes, np.int64), rows=rows, w=w, idx=idx, grad_out=grad_out, out0=out0,
             out=out.numpy(), grad_rows=g_rows.numpy(), grad_w=g_w.numpy(), out_acc=acc.numpy())  # fmt: skip
    # the reference's own bf16 CPU arithmetic on the bf16-rounded inputs
    outb, g_rowsb, g_wb, accb = run(torch.bfloat16)
    d.update(out_bf16=bits(outb), grad_rows_bf16=bits(g_rowsb), grad_w_bf16=bits(g_wb), out_acc_bf16=bits(accb))
    # metadata, as the reference builds it (device = cpu)
    ex = [torch.from_numpy(rows[offs[e] : offs[e + 1]]) for e in range(len(sizes))]
    _, chunk_sizes, expert_offsets, max_rows, num_experts = prepare_grouped_metadata(ex, "cpu")
    d.update(chunk_sizes=chunk_sizes.numpy(), expert_offsets=expert_offsets.numpy(),
             max_rows=np.int64(max_rows), num_experts=np.int64(num_experts))  # fmt: skip
    np.savez(HERE / f"{name}.npz", **d)


def routing(name, T, D, E, K, seed, dtype=torch.float32):
    """gate_and_sort with torch.argsort forced stable: the canonical order."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((1, T, D)).astype(np.float32)
    router = (rng.standard_normal((E, D)) * 0.5).astype(np.float32)
    moe = MoEFeedForward(D, 2 * D, E, K, MoEImplementation.FAST)
    with torch.no_grad():
        moe.router.weight.copy_(torch.from_numpy(router))
    moe = moe.to(dtype)
    xt = torch.from_numpy(x).to(dtype)
    real_argsort = torch.argsort
    torch.argsort = lambda t, *a, **k: real_argsort(t, *a, stable=True, **k)
    try:
        with torch.no_grad():
            permuted, rank_counts, by_rank, rev, sw, shape = moe.gate_and_sort(xt)
            logits = moe.router(xt.view(-1, D))
            tw, ti = torch.topk(logits, K, dim=-1)
            tw = torch.softmax(tw, dim=-1, dtype=torch.float32).type_as(xt)
    finally:
        torch.argsort = real_argsort
    # the unpatched call: same multiset per expert segment, order implementation-defined
    with torch.no_grad():
        _, _, _, rev_unstable, _, _ = moe.gate_and_sort(xt)
    f = (lambda t: bits(t)) if dtype == torch.bfloat16 else (lambda t: t.numpy())
    np.savez(HERE / f"{name}.npz", x=f(xt[0]), router=f(moe.router.weight.detach()), logits=f(logits),
             topk_idx=ti.numpy(), topk_w=f(tw), permuted=f(permuted), rank_counts=rank_counts.numpy(),
             expert_counts_by_rank=by_rank.numpy(), reverse_map=rev.numpy(), sorted_w=f(sw),
             reverse_map_unstable=rev_unstable.numpy(), K=np.int64(K), E=np.int64(E))  # fmt: skip


def layer_cfg1():
    """Config 1: T=256, D=128, E=8, top-2, ff=512, fp32, weights N(0,0.02); forward+backward
    through the reference's CPU combine path (FAST implementation, world size 1)."""
    router, w1, w2, x, target = layer_cfg1_weights()
    moe = MoEFeedForward(128, 512, 8, 2, MoEImplementation.FAST)
    with torch.no_grad():
        moe.router.weight.copy_(torch.from_numpy(router))
        for e in range(8):
            moe.experts[e][0].weight.copy_(torch.from_numpy(w1[e]))
            moe.experts[e][2].weight.copy_(torch.from_numpy(w2[e]))
    real_argsort = torch.argsort
    torch.argsort = lambda t, *a, **k: real_argsort(t, *a, stable=True, **k)
    try:
        xt = torch.from_numpy(x).view(1, 256, 128).requires_grad_(True)
        out = moe(xt)
        loss = ((out - torch.from_numpy(target).view(1, 256, 128)) ** 2).sum()
        loss.backward()
    finally:
        torch.argsort = real_argsort
    checksum = np.float64(router.astype(np.float64).sum() + w1.astype(np.float64).sum() + w2.astype(np.float64).sum() + x.astype(np.float64).sum())
    np.savez(HERE / "layer_cfg1.npz", out=out.detach().numpy()[0], x_grad=xt.grad.numpy()[0],
             router_grad=moe.router.weight.grad.numpy(),
             w1_grad_e0=moe.experts[0][0].weight.grad.numpy(), w2_grad_e7=moe.experts[7][2].weight.grad.numpy(),
             loss=np.float64(loss.item()), input_checksum=checksum)  # fmt: skip


if __name__ == "__main__":
    scatter_add_small()
    grouped("grouped_ragged", [3, 0, 7, 1, 0, 5], D=24, T=6, seed=2)
    grouped("grouped_one_target", [4, 4], D=8, T=3, seed=3, idx_mode="one_target")
    grouped("grouped_single", [16], D=40, T=9, seed=4)
    routing("routing_fp32", T=64, D=16, E=8, K=2, seed=5)
    routing("routing_bf16", T=96, D=32, E=16, K=4, seed=6, dtype=torch.bfloat16)
    layer_cfg1()
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)
