"""Pins the CPU oracle against fixtures produced by the reference's own CPU path
(tests/golden/make_golden.py). If these pass, the oracle may stand in for the
reference in the GPU parity tests."""

import numpy as np
import pytest

import oracle

GROUPED = ["grouped_ragged", "grouped_one_target", "grouped_single"]


def _split(rows, sizes):
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
    return [rows[offs[e] : offs[e + 1]] for e in range(len(sizes))]


def test_scatter_add_small_matches_reference_and_its_loop(golden):
    g = golden("scatter_add_small")
    out = oracle.combine([g["src"]], g["idx"], g["w"], 5)
    assert np.array_equal(out, g["out"])  # bit-exact with the reference's CPU path
    assert np.abs(out - g["out_loop"]).max() < 1e-5  # the reference test's own bound


@pytest.mark.parametrize("name", GROUPED)
def test_grouped_fp32_bit_exact(golden, name):
    g = golden(name)
    T = g["out"].shape[0]
    out = oracle.combine(_split(g["rows"], g["sizes"]), g["idx"], g["w"], T)
    assert np.array_equal(out, g["out"])
    acc = oracle.combine(_split(g["rows"], g["sizes"]), g["idx"], g["w"], T, out=g["out0"].copy())
    assert np.array_equal(acc, g["out_acc"])  # out= accumulates, never clears


@pytest.mark.parametrize("name", GROUPED)
def test_grouped_bf16_native_bit_exact(golden, name):
    g = golden(name)
    T = g["out"].shape[0]
    rows = oracle.f32_to_bf16_bits(g["rows"])
    w = oracle.f32_to_bf16_bits(g["w"])
    out = oracle.combine_bf16(_split(rows, g["sizes"]), g["idx"], w, T)
    assert np.array_equal(out, g["out_bf16"])
    acc = oracle.combine_bf16(_split(rows, g["sizes"]), g["idx"], w, T, out_bits=oracle.f32_to_bf16_bits(g["out0"]))
    assert np.array_equal(acc, g["out_acc_bf16"])
    # the fp32-arithmetic yardstick stays within bf16 accumulation error of it
    ref32 = oracle.combine_bf16_in_f32(_split(rows, g["sizes"]), g["idx"], w, T)
    scale = np.abs(ref32).max()
    assert np.abs(oracle.bf16_bits_to_f32(out) - ref32).max() <= 2e-2 * scale


@pytest.mark.parametrize("name", GROUPED)
def test_grouped_backward(golden, name):
    g = golden(name)
    grad_rows, grad_w = oracle.combine_bwd(g["rows"], g["idx"], g["w"], g["grad_out"])
    assert np.array_equal(grad_rows, g["grad_rows"])
    np.testing.assert_allclose(grad_w, g["grad_w"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", GROUPED)
def test_metadata(golden, name):
    g = golden(name)
    chunk_sizes, offsets, max_rows, E = oracle.prepare_metadata(g["sizes"])
    assert chunk_sizes.dtype == np.int32 and np.array_equal(chunk_sizes, g["chunk_sizes"])
    assert offsets.dtype == np.int64 and np.array_equal(offsets, g["expert_offsets"])
    assert max_rows == int(g["max_rows"]) and E == int(g["num_experts"])


def _as_f32(a):
    return oracle.bf16_bits_to_f32(a) if a.dtype == np.uint16 else a


@pytest.mark.parametrize("name", ["routing_fp32", "routing_bf16"])
def test_routing_bit_exact(golden, name):
    g = golden(name)
    K, E = int(g["K"]), int(g["E"])
    bf16 = g["x"].dtype == np.uint16
    logits = _as_f32(g["logits"])
    # torch.topk leaves the order of equal values open: compare the tokens whose
    # selection is tie-free (all of them in fp32, most of them in bf16)
    srt = np.sort(logits, axis=-1)[:, ::-1]
    idx, w = oracle.topk_softmax(logits, K)
    ties = (srt[:, :K] == srt[:, 1 : K + 1]).any(axis=-1)
    assert ties.mean() < 0.5 and (bf16 or not ties.any())
    assert np.array_equal(idx[~ties], g["topk_idx"][~ties])
    # with ties the selected VALUES still agree
    assert np.array_equal(np.take_along_axis(logits, idx, -1), np.take_along_axis(logits, g["topk_idx"], -1))
    if bf16:
        w_cmp, w_ref = oracle.f32_to_bf16_bits(w), g["topk_w"]
        # exp() may differ in the last fp32 bit between libraries: allow one bf16 ulp on < 1% of entries
        diff = np.abs(w_cmp.astype(np.int32) - w_ref.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 0.01
        w_in = g["topk_w"]
    else:
        np.testing.assert_allclose(w, g["topk_w"], rtol=2e-6, atol=1e-7)
        w_in = g["topk_w"]
    ix = oracle.build_index(g["topk_idx"], w_in, E, world=1)
    assert np.array_equal(ix["reverse_map"], g["reverse_map"])
    assert np.array_equal(ix["sorted_w"], g["sorted_w"].reshape(-1))
    assert np.array_equal(ix["expert_counts_by_rank"], g["expert_counts_by_rank"])
    assert np.array_equal(ix["rank_counts"], g["rank_counts"])
    assert np.array_equal(oracle.permute(g["x"], ix["reverse_map"]), g["permuted"])
    # slot_of inverts the sort
    T = g["x"].shape[0]
    assert np.array_equal(ix["reverse_map"][ix["slot_of"]], np.repeat(np.arange(T), K))
    # the reference's unstable argsort yields a per-expert permutation of the same rows
    off = np.concatenate([ix["offsets"], [T * K]])
    for e in range(E):
        a, b = off[e], off[e + 1]
        assert np.array_equal(np.sort(g["reverse_map_unstable"][a:b]), np.sort(ix["reverse_map"][a:b]))
    # world > 1 bookkeeping (tiny_model.py:144-150)
    ix2 = oracle.build_index(g["topk_idx"], w_in, E, world=2)
    assert np.array_equal(ix2["expert_counts_by_rank"].reshape(-1), ix["counts"])
    assert ix2["rank_counts"].sum() == T * K


def test_layer_cfg1_forward(golden):
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).parent / "golden"))
    from make_inputs import layer_cfg1_weights

    g = golden("layer_cfg1")
    router, w1, w2, x, _ = layer_cfg1_weights()
    checksum = sum(float(a.astype(np.float64).sum()) for a in (router, w1, w2, x))
    assert abs(checksum - float(g["input_checksum"])) < 1e-9
    out, _ = oracle.moe_layer_forward(x, router, list(w1), list(w2), K=2)
    np.testing.assert_allclose(out, g["out"], rtol=1e-5, atol=1e-6)


def test_c_port_matches_the_installed_reference_package():
    """Where oracle/install_ref.py has installed the unmodified reference package, the C port
    of its CPU combine is compared with the package itself on fresh random inputs: fp32 to
    1e-6 of the largest magnitude, bf16 bit for bit (same per-call fp32 accumulation and
    rounding). Skipped where the package is not installed (it does not travel with the repo)."""
    import pytest
    import torch

    import oracle

    ref = oracle.reference_ops()
    if ref is None:
        pytest.skip("the reference package is not installed under oracle/_ref")
    g = torch.Generator().manual_seed(5)
    T, D, sizes = 37, 24, [5, 0, 11, 3, 20]
    experts = [torch.randn(n, D, generator=g) for n in sizes]
    idx = torch.randint(0, T, (sum(sizes),), generator=g)
    w = torch.rand(sum(sizes), generator=g)
    want = ref.grouped_weighted_scatter_add(experts, idx, w, (T, D)).numpy()
    got = oracle.combine([e.numpy() for e in experts], idx.numpy(), w.numpy(), T)
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max()
    ex16, w16 = [e.bfloat16() for e in experts], w.bfloat16()
    want16 = ref.grouped_weighted_scatter_add(ex16, idx, w16, (T, D))
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    got16 = oracle.combine_bf16([bits(e) for e in ex16], idx.numpy(), bits(w16), T)
    assert np.array_equal(got16, bits(want16))
