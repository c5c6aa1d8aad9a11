"""The MoE layer module on the GPU against the reference's CPU layer (fixture) and the oracle:
config 1 (fp32 layer forward+backward), the dispatch+combine pair under autograd (config 4's
path), and the size-independent identity property at config 4's full size."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200.consts import MoEImplementation
from fastmoe_b200.kernels import ops, routing
from fastmoe_b200.models.tiny_model import MoEFeedForward
from fastmoe_b200.workloads import routing_uniform
from util import assert_close, to_np

sys.path.insert(0, str(Path(__file__).parent / "golden"))
from make_inputs import layer_cfg1_weights  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cfg1_layer(impl):
    router, w1, w2, x, target = layer_cfg1_weights()
    moe = MoEFeedForward(128, 512, 8, 2, impl).to(DEV)
    with torch.no_grad():
        moe.router.weight.copy_(torch.from_numpy(router))
        for e in range(8):
            moe.experts[e][0].weight.copy_(torch.from_numpy(w1[e]))
            moe.experts[e][2].weight.copy_(torch.from_numpy(w2[e]))
    xt = torch.from_numpy(x).to(DEV).view(1, 256, 128).requires_grad_(True)
    return moe, xt, torch.from_numpy(target).to(DEV).view(1, 256, 128)


@pytest.mark.parametrize("impl", [MoEImplementation.FAST, MoEImplementation.STANDARD])
def test_config1_layer_forward_backward(golden, impl):
    """T=256, D=128, E=8, top-2, fp32, weights N(0, 0.02): forward and backward of the whole layer
    against what the reference's CPU layer produced. 1e-4 of the largest magnitude: the two
    GEMMs per expert run on cuBLAS with another summation order than the CPU's."""
    g = golden("layer_cfg1")
    moe, x, target = _cfg1_layer(impl)
    out = moe(x)
    loss = ((out - target) ** 2).sum()
    loss.backward()
    tol = 1e-4

    def rel(a, b):
        return float(np.abs(to_np(a) - b).max()) / float(np.abs(b).max())

    assert rel(out[0], g["out"]) <= tol
    assert rel(x.grad[0], g["x_grad"]) <= tol
    assert rel(moe.router.weight.grad, g["router_grad"]) <= tol
    assert rel(moe.experts[0][0].weight.grad, g["w1_grad_e0"]) <= tol
    assert rel(moe.experts[7][2].weight.grad, g["w2_grad_e7"]) <= tol
    assert abs(float(loss.detach()) - float(g["loss"])) <= tol * float(g["loss"])
    assert ops.read_status() == 0


def test_gate_and_sort_contract():
    moe, x, _ = _cfg1_layer(MoEImplementation.FAST)
    permuted, rank_counts, by_rank, rev, w, shape = moe.gate_and_sort(x)
    assert shape == (1, 256) and permuted.shape == (512, 128)
    assert rank_counts.dtype == torch.int64 and rank_counts.tolist() == [512]
    assert by_rank.dtype == torch.int64 and by_rank.shape == (1, 8) and int(by_rank.sum()) == 512
    assert rev.dtype == torch.int64 and w.dtype == x.dtype
    logits = to_np(moe.router(x.view(-1, 128)))
    o_idx, o_w = oracle.topk_softmax(logits, 2)
    ix = oracle.build_index(o_idx, o_w, 8)
    assert np.array_equal(rev.cpu().numpy(), ix["reverse_map"])
    assert np.array_equal(by_rank.cpu().numpy().reshape(-1), ix["counts"])
    np.testing.assert_allclose(to_np(w), ix["sorted_w"], rtol=2e-6, atol=1e-7)
    assert np.array_equal(to_np(permuted), to_np(x.view(-1, 128))[ix["reverse_map"]])
    recv, recv_splits, send_splits, tokens = moe.dispatch_exchange(permuted, rank_counts, by_rank)
    assert recv is permuted and recv_splits == [512] and send_splits == [512] and tokens == ix["counts"].tolist()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dispatch_combine_autograd_against_oracle(dtype):
    """Config 4's path at a size the oracle handles in a blink: uniform top-8 routing over 256
    experts, permute -> per-expert scale (stands in for the FFN) -> combine; checks permuted,
    out, dx and d(gate)."""
    T, D, E, K = 512, 7168, 256, 8
    idx, w = routing_uniform(T, E, K, seed=4)
    rng = np.random.default_rng(4)
    x = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32)).to(DEV).to(dtype).requires_grad_(True)
    gate = w.to(DEV).to(dtype).requires_grad_(True)
    grad_out = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32)).to(DEV).to(dtype)
    scale = torch.linspace(0.5, 1.5, E, device=DEV)

    ix = routing.build_index(idx.to(DEV), gate, E)
    permuted = routing.permute_rows(x, ix.slot_of, K)
    counts = ix.counts.tolist()
    outs = [c * scale[e].to(dtype) for e, c in enumerate(permuted.split(counts))]
    out = ops.grouped_weighted_scatter_add(outs, ix.reverse_map, ix.sorted_w, (T, D))
    out.backward(grad_out)

    o = oracle.build_index(idx.numpy(), to_np(gate), E)
    assert np.array_equal(ix.reverse_map.cpu().numpy(), o["reverse_map"])
    assert np.array_equal(ix.counts.cpu().numpy(), o["counts"]) and np.array_equal(ix.offsets.cpu().numpy(), o["offsets"])
    rm = o["reverse_map"]
    perm_ref = oracle.permute(to_np(x), rm)
    assert np.array_equal(to_np(permuted), perm_ref)
    rows_ref = np.concatenate([to_np(t) for t in outs], 0)  # the kernels' actual inputs
    out_ref = oracle.combine([rows_ref], rm, o["sorted_w"], T)
    assert_close(out, out_ref, dtype, "out")
    g_rows, g_w = oracle.combine_bwd(rows_ref, rm, o["sorted_w"], to_np(grad_out))
    s_of_row = np.repeat(to_np(scale), o["counts"])
    if dtype == torch.bfloat16:  # the scale multiply's backward rounds to bf16 once more
        g_rows = to_np(torch.from_numpy(g_rows).to(dtype)) * np.repeat(to_np(scale.to(dtype)), o["counts"])[:, None]
    else:
        g_rows = g_rows * s_of_row[:, None]
    dx_ref = oracle.permute_bwd(g_rows, rm, T)
    assert_close(x.grad, dx_ref, dtype, "dx")
    dgate_ref = np.empty(T * K, np.float32)
    dgate_ref[:] = g_w[o["slot_of"]]
    assert_close(gate.grad.reshape(-1), dgate_ref, dtype, "d(gate)")


def test_config4_full_size_identity_property():
    """T=16384, D=7168, E=256, top-8, bf16. With identity experts and gate weights that sum to one,
    combine(permute(x)) must return x, and the backward must return the upstream gradient."""
    T, D, E, K = 16384, 7168, 256, 8
    idx, w = routing_uniform(T, E, K, seed=9)
    gen = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(T, D, generator=gen, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    grad_out = torch.randn(T, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    gate = w.to(DEV)  # fp32 weights: they sum to 1 to fp32 accuracy
    ix = routing.build_index(idx.to(DEV), gate, E)
    assert int(ix.counts.sum()) == T * K and bool((ix.counts == torch.bincount(idx.reshape(-1), minlength=E).to(DEV)).all())
    permuted = routing.permute_rows(x, ix.slot_of, K)
    assert torch.equal(permuted, x.detach()[ix.reverse_map])
    outs = list(permuted.split(ix.counts.tolist()))
    out = ops.grouped_weighted_scatter_add(outs, ix.reverse_map, ix.sorted_w, (T, D))
    out.backward(grad_out)
    err = float((out.float() - x.detach().float()).abs().max() / x.detach().float().abs().max())
    assert err <= 2e-2, err
    gerr = float((x.grad.float() - grad_out.float()).abs().max() / grad_out.float().abs().max())
    assert gerr <= 2e-2, gerr
    assert ops.read_status() == 0


def test_config4_full_size_gate_gradient_against_oracle():
    """The same full-size configuration with the gate weights as a leaf: d(gate) of every routed
    copy of a sample of tokens against the oracle's combine backward (the row-wise dot of the
    upstream gradient with the expert row, which the reference's CPU path yields through
    autograd), and d(rows) of the same copies, for the planned and for the plan-free combine."""
    T, D, E, K = 16384, 7168, 256, 8
    idx, w = routing_uniform(T, E, K, seed=11)
    gen = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(T, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    grad_out = torch.randn(T, D, generator=gen, device=DEV, dtype=torch.bfloat16)
    sample = torch.randperm(T, generator=torch.Generator().manual_seed(12))[:96].sort().values
    for routed in (False, True):
        gate = w.to(DEV).bfloat16().requires_grad_(True)
        ix = routing.build_index(idx.to(DEV), gate, E)
        permuted = routing.permute_rows(x, ix.slot_of, K).requires_grad_(True)
        if routed:
            out = ops.routed_combine(permuted, ix.slot_of, ix.sorted_w, K)
        else:
            out = ops.grouped_weighted_scatter_add([permuted], ix.reverse_map, ix.sorted_w, (T, D))
        out.backward(grad_out)
        assert ops.read_status() == 0
        # oracle on the sampled tokens alone: their K rows each, re-indexed to 0..95
        slots = ix.slot_of.view(T, K)[sample.to(DEV)].reshape(-1).long()
        rows_s = to_np(permuted.detach()[slots])
        rm_s = np.repeat(np.arange(sample.numel()), K)
        w_s = to_np(ix.sorted_w.detach()[slots])
        g_rows, g_w = oracle.combine_bwd(rows_s, rm_s, w_s, to_np(grad_out[sample.to(DEV)]))
        assert_close(gate.grad.view(T, K)[sample.to(DEV)].reshape(-1), g_w, torch.bfloat16, f"d(gate), routed={routed}")
        assert_close(permuted.grad[slots], g_rows, torch.bfloat16, f"d(rows), routed={routed}")
        out_s = oracle.combine([rows_s], rm_s, w_s, sample.numel())
        assert_close(out[sample.to(DEV)], out_s, torch.bfloat16, f"out, routed={routed}")
        del permuted, out


@pytest.mark.parametrize("impl", [MoEImplementation.FAST, MoEImplementation.STANDARD])
def test_swiglu_layer_matches_fp32_reference(impl):
    """SwiGLU experts (the expert-parallel benchmark's FFN): the FAST path runs the tcgen05
    grouped GEMM, the STANDARD path per-expert matrix products; both against a plain PyTorch
    fp32 evaluation of the same layer with the same routing."""
    torch.manual_seed(0)
    T, D, FF, E, K = 512, 256, 256, 8, 2
    moe = MoEFeedForward(D, FF, E, K, impl, expert_type="swiglu").to(DEV).bfloat16()
    with torch.no_grad():
        for prm in moe.parameters():
            prm.normal_(0, 0.05)
    x = torch.randn(1, T, D, device=DEV).bfloat16().requires_grad_(True)
    out = moe(x)
    out.float().pow(2).sum().backward()
    assert ops.read_status() == 0
    # fp32 reference with the layer's own routing decision
    xf = x.detach().float().view(T, D)
    logits = moe.router(x.detach().view(T, D))
    w, idx = routing.route_topk(logits, K, w_dtype=torch.bfloat16)
    ref = torch.zeros(T, D, device=DEV)
    wgu, wd = moe.experts.w_gate_up.detach().float(), moe.experts.w_down.detach().float()
    for k in range(K):
        for e in range(E):
            m = idx[:, k] == e
            h = xf[m] @ wgu[e].t()
            a = (torch.nn.functional.silu(h[:, :FF]) * h[:, FF:]).bfloat16().float()  # hidden is stored in bf16
            ref[m] += (a @ wd[e].t()).bfloat16().float() * w[m, k].float()[:, None]
    err = float((out.float().view(T, D) - ref).abs().max() / ref.abs().max())
    assert err <= 2e-2, err
    assert x.grad is not None and moe.experts.w_gate_up.grad is not None and moe.router.weight.grad is not None
    assert torch.isfinite(x.grad.float()).all()


def test_gelu_experts_run_grouped_in_bf16_and_match_the_per_expert_modules():
    """The reference's own experts (nn.ModuleList of Linear-GELU-Linear, tiny_model.py:68-77):
    in bf16 the FAST layer runs them as two grouped tcgen05 launches over the stacked weights,
    the STANDARD layer as a loop of per-expert modules. Same parameters, same inputs: outputs
    and every gradient (tokens, router, each expert's two matrices) agree within bf16 bounds,
    the state dict keeps the reference's keys, and an fp32 layer keeps the per-expert path."""
    torch.manual_seed(3)
    T, D, FF, E, K = 384, 256, 512, 8, 2
    fast = MoEFeedForward(D, FF, E, K, MoEImplementation.FAST).to(DEV).bfloat16()
    std = MoEFeedForward(D, FF, E, K, MoEImplementation.STANDARD).to(DEV).bfloat16()
    assert not fast._use_grouped(torch.zeros(4, D, device=DEV).bfloat16())  # 8 experts: below the threshold
    fast.grouped_gelu_min_experts = 1  # the layer takes the grouped path from this many local experts on
    assert "experts.3.0.weight" in fast.state_dict() and "experts.3.2.weight" in fast.state_dict()
    with torch.no_grad():
        for prm in fast.parameters():
            prm.normal_(0, 0.05)
    std.load_state_dict(fast.state_dict())
    x = torch.randn(1, T, D, device=DEV).bfloat16()
    coeff = torch.randn(1, T, D, device=DEV)
    assert fast._use_grouped(x.view(T, D)) and not std._use_grouped(x.view(T, D))
    assert not MoEFeedForward(D, FF, E, K, MoEImplementation.FAST).to(DEV)._use_grouped(x.view(T, D).float())
    results = []
    for moe in (fast, std):
        xi = x.clone().requires_grad_(True)
        before = ops.launch_count
        out = moe(xi)
        (out.float() * coeff).sum().backward()
        results.append((out.detach(), xi.grad, moe.router.weight.grad, moe.experts[0][0].weight.grad,
                        moe.experts[E - 1][2].weight.grad, ops.launch_count - before))  # fmt: skip
    assert ops.read_status() == 0
    for got, want, what in zip(results[0][:5], results[1][:5], ("out", "dx", "d router", "d fc1[0]", "d fc2[-1]")):
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= 3e-2, (what, err)  # two bf16 pipelines against each other
    assert results[0][5] > results[1][5]  # the FAST layer's kernels are this library's


def test_pipelined_block_matches_unpipelined_computation():
    """PipelinedMoEBlock (micro-batches on side streams) against the same block evaluated in one
    piece on the current stream; also with 4 micro-batches and SwiGLU experts."""
    from fastmoe_b200.models.tiny_model import PipelinedMoEBlock

    torch.manual_seed(1)
    for n_mb, expert_type, dtype in ((2, "gelu", torch.float32), (4, "swiglu", torch.bfloat16)):
        s0, s1 = torch.cuda.Stream(), torch.cuda.Stream()
        blk = PipelinedMoEBlock(256, 4, 128, 8, 2, s0, s1, num_micro_batches=n_mb, expert_type=expert_type)
        blk = blk.to(DEV).to(dtype)
        x = torch.randn(8, 32, 256, device=DEV, dtype=dtype)
        with torch.no_grad():
            out = blk(x)
            torch.cuda.synchronize()
            r = x + blk.attn(blk.norm1(x))
            ref = torch.cat([blk.moe(c) for c in blk.norm2(r).chunk(n_mb, 0)], 0) + r
        assert out.shape == x.shape
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err <= tol, (n_mb, expert_type, err)
    assert ops.read_status() == 0
