"""GPU parity of the combine (forward, out= accumulation, backward) against the
CPU oracle and the reference-generated fixtures. Every call goes through the
public operator, which reaches the kernels through the C ABI."""

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200.kernels import ops
from fastmoe_b200.workloads import make_combine_workload
from util import REL_TOL, assert_close, oracle_combine, split_rows, to_np

pytestmark = pytest.mark.gpu

DEV = "cuda"
GROUPED = ["grouped_ragged", "grouped_one_target", "grouped_single"]
MODES = ["gather", "scatter"]


@pytest.fixture(autouse=True)
def _mode_guard():
    prev = ops.combine_mode()
    yield
    ops.set_combine_mode(prev)
    assert ops.read_status() == 0, "a kernel flagged skipped rows"


def _experts(rows, sizes, dtype):
    return [torch.from_numpy(r.copy()).to(DEV).to(dtype) for r in split_rows(rows, sizes)]


@pytest.mark.parametrize("mode", MODES)
def test_reference_unit_test_shape(golden, mode):
    """tests/test_cpu_moe.py:94-114 of the reference, against its per-row loop and its own output."""
    g = golden("scatter_add_small")
    ops.set_combine_mode(mode)
    src = torch.from_numpy(g["src"]).to(DEV)
    idx = torch.from_numpy(g["idx"]).to(DEV)
    w = torch.from_numpy(g["w"]).to(DEV)
    out = ops.weighted_scatter_add(src, idx, w, (5, 4))
    assert (to_np(out) - g["out_loop"]).__abs__().max() < 1e-5
    out2 = torch.zeros(5, 4, device=DEV)
    ops.weighted_scatter_add(src, idx, w, (5, 4), out=out2)
    assert_close(out2, g["out"], torch.float32)
    if mode == "gather":
        assert np.array_equal(to_np(out2), g["out"])


@pytest.mark.parametrize("name", GROUPED)
@pytest.mark.parametrize("mode", MODES)
def test_golden_fp32(golden, name, mode):
    g = golden(name)
    ops.set_combine_mode(mode)
    T, D = g["out"].shape
    ex = _experts(g["rows"], g["sizes"], torch.float32)
    idx = torch.from_numpy(g["idx"]).to(DEV)
    w = torch.from_numpy(g["w"]).to(DEV)
    out = torch.zeros(T, D, device=DEV)
    ops.grouped_weighted_scatter_add(ex, idx, w, (T, D), out=out)
    assert_close(out, g["out"], torch.float32, "out")
    acc = torch.from_numpy(g["out0"].copy()).to(DEV)
    ops.grouped_weighted_scatter_add(ex, idx, w, (T, D), out=acc)  # accumulates, never clears
    assert_close(acc, g["out_acc"], torch.float32, "out_acc")
    if mode == "gather":
        assert np.array_equal(to_np(out), g["out"]) and np.array_equal(to_np(acc), g["out_acc"])


@pytest.mark.parametrize("name", GROUPED)
@pytest.mark.parametrize("mode", MODES)
def test_golden_bf16(golden, name, mode):
    """bf16 run against the fp32-arithmetic oracle on the same bf16-rounded inputs (2e-2), and
    against what the reference's own bf16 CPU arithmetic returned (same bound)."""
    g = golden(name)
    ops.set_combine_mode(mode)
    T, D = g["out"].shape
    ex = _experts(g["rows"], g["sizes"], torch.bfloat16)
    idx = torch.from_numpy(g["idx"]).to(DEV)
    w = torch.from_numpy(g["w"]).to(DEV).bfloat16()
    out = torch.zeros(T, D, device=DEV, dtype=torch.bfloat16)
    ops.grouped_weighted_scatter_add(ex, idx, w, (T, D), out=out)
    ref32 = oracle_combine(ex, idx, w, T)
    assert_close(out, ref32, torch.bfloat16)
    assert_close(out, oracle.bf16_bits_to_f32(g["out_bf16"]), torch.bfloat16)
    if mode == "gather":  # one rounding of the fp32 sum: half a bf16 ulp
        assert np.all(np.abs(to_np(out) - ref32) <= np.abs(ref32) * 2.0**-8 + 1e-30)


@pytest.mark.parametrize("name", GROUPED)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_golden_backward(golden, name, dtype):
    g = golden(name)
    T, D = g["out"].shape
    ex = [e.requires_grad_(True) for e in _experts(g["rows"], g["sizes"], dtype)]
    idx = torch.from_numpy(g["idx"]).to(DEV)
    w = torch.from_numpy(g["w"]).to(DEV).to(dtype).requires_grad_(True)
    out = ops.grouped_weighted_scatter_add(ex, idx, w, (T, D))
    assert out.dtype == dtype  # the experts' dtype (ops.py:327)
    grad_out = torch.from_numpy(g["grad_out"]).to(DEV).to(dtype)
    out.backward(grad_out)
    if dtype == torch.float32:
        assert np.array_equal(to_np(out), g["out"])
        g_rows = torch.cat([e.grad for e in ex], 0)
        assert np.array_equal(to_np(g_rows), g["grad_rows"])
        np.testing.assert_allclose(to_np(w.grad), g["grad_w"], rtol=1e-5, atol=1e-6)
    else:
        rows32 = np.concatenate([to_np(e) for e in ex], 0)
        gr, gw = oracle.combine_bwd(rows32, g["idx"], to_np(w), to_np(grad_out))
        g_rows = torch.cat([e.grad for e in ex], 0)
        assert_close(g_rows, gr, dtype, "grad_rows")
        assert_close(w.grad, gw, dtype, "grad_w")
    for e, n in zip(ex, g["sizes"]):  # empty experts get an empty gradient, not None
        assert e.grad is not None and e.grad.shape == (int(n), D)


CASES = [
    # T, D, sizes, dtype, idx dtype
    (7, 8, [5], torch.float32, torch.int64),
    (16, 128, [9, 0, 14], torch.float32, torch.int32),
    (33, 1000, [40, 1, 25], torch.bfloat16, torch.int64),
    (64, 7168, [100, 0, 0, 156], torch.bfloat16, torch.int64),
    (12, 2048, [30], torch.float16, torch.int64),
    (5, 6, [4, 4], torch.float32, torch.int64),  # D not a multiple of the vector width
    (9, 1001, [20, 3], torch.bfloat16, torch.int32),  # odd width, element-wise path
    (4, 16, [0, 0, 0], torch.float32, torch.int64),  # no rows at all
    (300, 256, [1] * 64, torch.bfloat16, torch.int64),  # many one-row experts
    (3, 512, [2000], torch.float32, torch.int64),  # long segments: 2000 rows into 3 tokens
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"T{c[0]}-D{c[1]}-E{len(c[2])}-{str(c[3])[6:]}")
def test_random_cases_against_oracle(case, mode):
    T, D, sizes, dtype, itype = case
    ops.set_combine_mode(mode)
    rng = np.random.default_rng(abs(hash((T, D, len(sizes)))) % (1 << 31))
    N = sum(sizes)
    ex = [torch.from_numpy(rng.standard_normal((n, D)).astype(np.float32)).to(DEV).to(dtype) for n in sizes]
    idx = torch.from_numpy(rng.integers(0, T, N)).to(DEV).to(itype)
    w = torch.from_numpy(rng.random(N).astype(np.float32)).to(DEV).to(dtype)
    out0 = torch.from_numpy(rng.standard_normal((T, D)).astype(np.float32)).to(DEV).to(dtype)
    ref = oracle_combine(ex, idx, w, T)
    fresh = ops.grouped_weighted_scatter_add(ex, idx, w, (T, D))
    assert fresh.shape == (T, D) and fresh.dtype == dtype
    assert_close(fresh, ref, dtype, "fresh")
    acc = out0.clone()
    ops.grouped_weighted_scatter_add(ex, idx, w, (T, D), out=acc)
    ref_acc = oracle_combine(ex, idx, w, T, out0=out0)
    if dtype == torch.float32 and mode == "gather":
        assert np.array_equal(to_np(fresh), ref) and np.array_equal(to_np(acc), ref_acc)
    else:
        assert_close(acc, ref_acc, dtype, "acc")


def test_strided_out_and_metadata_reuse():
    """`out` may be a row-strided view (ops.py:304 passes its strides); cached metadata is reused."""
    rng = np.random.default_rng(11)
    T, D, sizes = 10, 64, [6, 2, 9]
    ex = [torch.from_numpy(rng.standard_normal((n, D)).astype(np.float32)).to(DEV) for n in sizes]
    idx = torch.from_numpy(rng.integers(0, T, sum(sizes))).to(DEV)
    w = torch.from_numpy(rng.random(sum(sizes)).astype(np.float32)).to(DEV)
    meta = ops.prepare_grouped_metadata(ex, ex[0].device)
    ptr_table, chunk_sizes, expert_offsets, max_rows, num_experts = meta
    assert ptr_table.dtype == torch.int64 and chunk_sizes.dtype == torch.int32
    assert expert_offsets.dtype == torch.int64 and (max_rows, num_experts) == (9, 3)
    assert ptr_table.tolist() == [e.data_ptr() for e in ex]
    ref = oracle_combine(ex, idx, w, T)
    for mode in MODES:
        ops.set_combine_mode(mode)
        wide = torch.zeros(T, 2 * D, device=DEV)
        view = wide[:, :D]
        ops.grouped_weighted_scatter_add(ex, idx, w, (T, D), out=view, metadata=meta)
        assert_close(view, ref, torch.float32)
        assert float(wide[:, D:].abs().max()) == 0.0


def test_bit_reproducible_and_fp32_weights_with_bf16_rows():
    wl = make_combine_workload(T=256, D=1024, E=16, K=4, dtype=torch.bfloat16, seed=3)
    a = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (wl.T, wl.D))
    b = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (wl.T, wl.D))
    assert torch.equal(a, b)
    w32 = wl.weights.float()
    c = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, w32, (wl.T, wl.D))
    assert c.dtype == torch.bfloat16
    assert_close(c, oracle_combine(wl.experts, wl.indices, w32, wl.T), torch.bfloat16)


def test_bad_arguments_raise_before_launch():
    src = torch.zeros(4, 8, device=DEV)
    idx = torch.zeros(4, dtype=torch.int64, device=DEV)
    w = torch.ones(4, device=DEV)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.weighted_scatter_add(src.cpu(), idx.cpu(), w.cpu(), (2, 8))
    with pytest.raises(ValueError):
        ops.grouped_weighted_scatter_add([], idx, w, (2, 8))
    with pytest.raises(ValueError):
        ops.weighted_scatter_add(src, idx[:3], w, (2, 8))
    with pytest.raises(ValueError):
        ops.weighted_scatter_add(src, idx.float(), w, (2, 8))
    with pytest.raises(ValueError):
        ops.weighted_scatter_add(src, idx, w, (2, 8), out=torch.zeros(2, 8, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.grouped_weighted_scatter_add([src, torch.zeros(2, 4, device=DEV)], idx, w, (2, 8))


@pytest.mark.parametrize("mode", MODES)
def test_out_of_range_index_is_skipped_and_flagged(mode):
    """A bad index must not fault the GPU: the row is skipped and the status word says so."""
    ops.set_combine_mode(mode)
    src = torch.ones(3, 8, device=DEV)
    idx = torch.tensor([0, 99, -1], device=DEV)
    w = torch.ones(3, device=DEV)
    out = torch.zeros(2, 8, device=DEV)
    ops.weighted_scatter_add(src, idx, w, (2, 8), out=out)
    assert ops.read_status() & 1
    assert to_np(out)[0].tolist() == [1.0] * 8 and float(out[1].abs().max()) == 0.0
    assert ops.read_status() == 0  # cleared by the read above


@pytest.mark.parametrize("routing", ["softmax", "zipf"])
def test_medium_workload_all_dtypes(routing):
    for dtype in (torch.float32, torch.bfloat16):
        wl = make_combine_workload(T=512, D=2048, E=64, K=8, dtype=dtype, routing=routing, seed=5)
        ref = oracle_combine(wl.experts, wl.indices, wl.weights, wl.T)
        for mode in MODES:
            ops.set_combine_mode(mode)
            out = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (wl.T, wl.D))
            err = assert_close(out, ref, dtype, f"{routing}/{mode}/{dtype}")
            assert err <= REL_TOL[dtype]


def test_cuda_graph_capture_and_replay_like_the_reference_benchmark():
    """The reference's microbenchmark captures `grouped_weighted_scatter_add(..., out=, metadata=)`
    in a CUDA graph and replays it after zeroing `out` (run_on_cloud.py:64-91). The same flow must
    work here, in both combine modes, and give the oracle's result on every replay."""
    wl = make_combine_workload(T=256, D=2048, E=32, K=4, dtype=torch.float32, seed=9)
    shape = (wl.T, wl.D)
    ref = oracle_combine(wl.experts, wl.indices, wl.weights, wl.T)
    for mode in MODES:
        ops.set_combine_mode(mode)
        out_static = torch.zeros(shape, device=DEV)
        metadata = ops.prepare_grouped_metadata(wl.experts, out_static.device)
        ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, shape, out=out_static, metadata=metadata)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        out_static.zero_()
        with torch.cuda.graph(graph):
            ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, shape, out=out_static, metadata=metadata)
        for _ in range(3):
            out_static.zero_()
            graph.replay()
        torch.cuda.synchronize()
        assert_close(out_static, ref, torch.float32, f"graph replay / {mode}")
        if mode == "gather":
            assert np.array_equal(to_np(out_static), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,D,E,K", [(64, 128, 8, 2), (257, 1000, 16, 4), (128, 7168, 32, 8), (33, 8, 4, 1)])
def test_routed_combine_matches_oracle(dtype, T, D, E, K):
    """The plan-free combine (one matrix in sorted-slot order + the index builder's inverse map)
    against the oracle's combine and its backward on the same values: forward, d(rows) and
    d(gate). It adds a token's K rows in routed order k rather than in ascending row order, so
    fp32 is held to 1e-5, not to bit equality."""
    from fastmoe_b200.kernels import routing
    from fastmoe_b200.workloads import routing_uniform

    idx, w = routing_uniform(T, E, K, seed=T + K)
    gen = torch.Generator(device=DEV).manual_seed(D)
    gate = w.to(DEV).to(dtype).requires_grad_(True)
    ix = routing.build_index(idx.to(DEV), gate, E)
    rows = torch.randn(T * K, D, generator=gen, device=DEV).to(dtype).requires_grad_(True)
    grad_out = torch.randn(T, D, generator=gen, device=DEV).to(dtype)
    out = ops.routed_combine(rows, ix.slot_of, ix.sorted_w, K)
    out.backward(grad_out)
    rm = ix.reverse_map.cpu().numpy()
    sw = to_np(ix.sorted_w)
    ref = oracle.combine([to_np(rows)], rm, sw, T)
    assert_close(out, ref, dtype, "out")
    g_rows, g_w = oracle.combine_bwd(to_np(rows), rm, sw, to_np(grad_out))
    assert_close(rows.grad, g_rows, dtype, "d(rows)")
    dgate = np.empty(T * K, np.float32)
    dgate[:] = g_w[ix.slot_of.cpu().numpy()]
    assert_close(gate.grad.reshape(-1), dgate, dtype, "d(gate)")
    # the same numbers as the planned operator gives for this matrix
    planned = ops.grouped_weighted_scatter_add([rows.detach()], ix.reverse_map, ix.sorted_w.detach(), (T, D))
    assert_close(out, to_np(planned), dtype, "routed vs planned")


def test_routed_combine_refuses_bad_arguments():
    rows = torch.zeros(8, 16, device=DEV)
    slot_of = torch.arange(8, device=DEV, dtype=torch.int32)
    w = torch.ones(8, device=DEV)
    with pytest.raises(ValueError):
        ops.routed_combine(rows, slot_of.long(), w, 2)
    with pytest.raises(ValueError):
        ops.routed_combine(rows, slot_of[:6], w[:6], 2)
    with pytest.raises(ValueError):
        ops.routed_combine(rows, slot_of, w, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.routed_combine(rows.cpu(), slot_of, w, 2)


def test_no_grad_call_skips_autograd_but_not_the_work():
    """Without anything to differentiate the operator launches the same kernels directly
    (no autograd node holding E tensors); results are identical to the autograd path."""
    wl = make_combine_workload(T=96, D=256, E=12, K=3, dtype=torch.bfloat16, seed=3, device=DEV)
    before = ops.launch_count
    plain = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (wl.T, wl.D))
    assert ops.launch_count - before == 2 and not plain.requires_grad
    tracked = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights.clone().requires_grad_(True), (wl.T, wl.D))
    assert tracked.requires_grad and torch.equal(plain, tracked.detach())
