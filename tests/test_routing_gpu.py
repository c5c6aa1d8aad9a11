"""GPU parity of the router top-k/softmax, the index-offset builder and the dispatch
permute: indices, counts and offsets bit-exact against the oracle and the reference
fixtures; weights within fp32 rounding."""

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200.kernels import ops, routing
from util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=None):
    if a.dtype == np.uint16:  # bf16 bit patterns
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(DEV)
    t = torch.from_numpy(a.copy()).to(DEV)
    return t if dtype is None else t.to(dtype)


def _bits_or_values(t):
    if t.dtype == torch.bfloat16:
        return t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.cpu().numpy()


@pytest.mark.parametrize("name", ["routing_fp32", "routing_bf16"])
def test_reference_fixture(golden, name):
    g = golden(name)
    K, E = int(g["K"]), int(g["E"])
    logits = _t(g["logits"])
    w, idx = routing.route_topk(logits, K)
    l32 = to_np(logits)
    srt = np.sort(l32, -1)[:, ::-1]
    ties = (srt[:, :K] == srt[:, 1 : K + 1]).any(-1)
    assert np.array_equal(idx.cpu().numpy()[~ties], g["topk_idx"][~ties])
    o_idx, o_w = oracle.topk_softmax(l32, K)
    assert np.array_equal(idx.cpu().numpy(), o_idx)  # ties too: lower expert id first
    if logits.dtype == torch.bfloat16:
        d = np.abs(_bits_or_values(w).astype(np.int32) - g["topk_w"].astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 0.01
    else:
        np.testing.assert_allclose(to_np(w), g["topk_w"], rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(to_np(w), o_w, rtol=2e-6, atol=1e-7)
    # the builder, fed the reference's own top-k, must reproduce its (stable) outputs bit for bit
    ix = routing.build_index(_t(g["topk_idx"]), _t(g["topk_w"]), E)
    assert np.array_equal(ix.reverse_map.cpu().numpy(), g["reverse_map"])
    assert np.array_equal(_bits_or_values(ix.sorted_w), g["sorted_w"].reshape(-1))
    assert np.array_equal(ix.counts.cpu().numpy().reshape(1, E), g["expert_counts_by_rank"])
    assert np.array_equal(ix.rank_counts.cpu().numpy(), g["rank_counts"])
    permuted = routing.permute_rows(_t(g["x"]), ix.slot_of, K)
    assert np.array_equal(_bits_or_values(permuted), g["permuted"])


SHAPES = [(1, 8, 1), (33, 8, 2), (1000, 256, 8), (257, 100, 3), (64, 1000, 32), (4096, 64, 6), (16384, 256, 8), (5, 3, 3)]


@pytest.mark.parametrize("T,E,K", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_and_index_against_oracle(T, E, K, dtype):
    rng = np.random.default_rng(T * 131 + E * 7 + K)
    logits = torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(DEV).to(dtype)
    w, idx = routing.route_topk(logits, K)
    o_idx, o_w = oracle.topk_softmax(to_np(logits), K)
    assert idx.dtype == torch.int64 and np.array_equal(idx.cpu().numpy(), o_idx)
    tol = 2e-6 if dtype == torch.float32 else 2.0**-8
    np.testing.assert_allclose(to_np(w), o_w, rtol=tol, atol=1e-7)
    for world in (1, 2) if E % 2 == 0 else (1,):
        ix = routing.build_index(idx, w, E, world)
        o = oracle.build_index(o_idx, to_np(w), E, world)
        assert np.array_equal(ix.reverse_map.cpu().numpy(), o["reverse_map"])
        assert np.array_equal(to_np(ix.sorted_w), o["sorted_w"])
        assert ix.counts.dtype == torch.int64 and np.array_equal(ix.counts.cpu().numpy(), o["counts"])
        assert np.array_equal(ix.offsets.cpu().numpy(), o["offsets"])
        assert np.array_equal(ix.rank_counts.cpu().numpy(), o["rank_counts"])
        assert ix.slot_of.dtype == torch.int32 and np.array_equal(ix.slot_of.cpu().numpy(), o["slot_of"])
    assert ops.read_status() == 0


def test_ties_nan_and_rank_counts():
    logits = torch.zeros(4, 16, device=DEV)
    logits[1, 5] = 1.0
    logits[2, 3] = float("nan")
    logits[3] = torch.arange(16, device=DEV).float() * -1.0
    w, idx = routing.route_topk(logits, 3)
    assert idx[0].tolist() == [0, 1, 2]  # equal values: lower expert id first
    assert idx[1].tolist() == [5, 0, 1]
    assert idx[2].tolist()[0] == 3  # NaN ranks above everything, as in torch.topk
    assert idx[3].tolist() == [0, 1, 2]
    np.testing.assert_allclose(to_np(w[0]), [1 / 3] * 3, rtol=1e-6)
    clean = torch.tensor([[0, 15, 7], [8, 9, 1], [15, 14, 13], [3, 2, 1]], device=DEV)
    ix = routing.build_index(clean, torch.ones(4, 3, device=DEV), 16, world=4)
    assert ix.rank_counts.tolist() == [5, 1, 2, 4] and int(ix.counts.sum()) == 12


def test_bad_expert_id_is_flagged_not_fatal():
    idx = torch.tensor([[0, 99], [1, -2]], device=DEV)
    ix = routing.build_index(idx, torch.ones(2, 2, device=DEV), 4)
    assert ops.read_status() & 2
    assert ix.counts.tolist() == [1, 1, 0, 0] and ix.slot_of.tolist() == [0, -1, 1, -1]
    with pytest.raises(ValueError):
        routing.build_index(idx, torch.ones(2, 2, device=DEV), 6, world=4)
    with pytest.raises(ValueError):
        routing.route_topk(torch.zeros(2, 4, device=DEV), 5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,E,K", [(37, 24, 8, 2), (128, 7168, 32, 8), (64, 1001, 8, 4), (300, 16, 16, 1)])
def test_permute_forward_backward(T, D, E, K, dtype):
    rng = np.random.default_rng(T + D)
    x = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32)).to(DEV).to(dtype).requires_grad_(True)
    logits = torch.from_numpy(rng.standard_normal((T, E)).astype(np.float32)).to(DEV)
    w, idx = routing.route_topk(logits, K)
    ix = routing.build_index(idx, w, E)
    permuted = routing.permute_rows(x, ix.slot_of, K)
    rm = ix.reverse_map.cpu().numpy()
    assert np.array_equal(to_np(permuted), oracle.permute(to_np(x), rm))  # a copy: bit-exact in any dtype
    g = torch.from_numpy(rng.standard_normal((T * K, D)).astype(np.float32)).to(DEV).to(dtype)
    permuted.backward(g)
    ref = oracle.permute_bwd(to_np(g), rm, T)
    if dtype == torch.float32 and K <= 2:
        assert np.array_equal(to_np(x.grad), ref)  # two addends: order cannot matter
    assert_close(x.grad, ref, dtype, "grad_x")


def test_topk_backward_matches_torch_autograd():
    torch.manual_seed(0)
    logits = torch.randn(200, 64, device=DEV, requires_grad=True)
    w, idx = routing.route_topk(logits, 6)
    ix = routing.build_index(idx, w, 64)
    coeff = torch.randn_like(ix.sorted_w)
    (ix.sorted_w * coeff).sum().backward()
    ref_logits = logits.detach().clone().requires_grad_(True)
    vals, ridx = torch.topk(ref_logits, 6, dim=-1)
    rw = torch.softmax(vals, -1, dtype=torch.float32)
    order = torch.argsort(ridx.reshape(-1), stable=True)
    (rw.reshape(-1)[order] * coeff).sum().backward()
    assert torch.equal(idx, ridx)
    torch.testing.assert_close(logits.grad, ref_logits.grad, rtol=1e-5, atol=1e-7)
