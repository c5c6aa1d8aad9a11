"""Size-independent properties of the CPU oracle (the checker of every GPU parity test).

The golden fixtures pin the oracle to the reference on fixed inputs; these tests hold it to the
algebra of the operation on seeded random inputs of ragged shapes: linearity, the plain
per-row definition, adjointness of forward and backward, and the empty cases.
"""

import numpy as np
import pytest

import oracle


def _case(seed, T, D, sizes):
    rng = np.random.default_rng(seed)
    experts = [rng.standard_normal((n, D)).astype(np.float32) for n in sizes]
    N = int(sum(sizes))
    idx = rng.integers(0, T, size=N).astype(np.int64)
    w = rng.random(N).astype(np.float32)
    return experts, idx, w, N


CASES = [(1, 1, [1]), (7, 4, [0, 3, 0, 5]), (33, 8, [10, 0, 1, 40, 2]), (64, 128, [17] * 8), (5, 3, [0, 0, 0])]


@pytest.mark.parametrize("T,D,sizes", CASES)
def test_combine_is_the_per_row_definition(T, D, sizes):
    """out[idx[g]] += rows[g] * w[g], rows taken expert after expert (ops.py:373-384)."""
    experts, idx, w, N = _case(1, T, D, sizes)
    got = oracle.combine(experts, idx, w, T)
    rows = np.concatenate(experts, 0) if N else np.zeros((0, D), np.float32)
    want = np.zeros((T, D), np.float64)
    for g in range(N):
        want[idx[g]] += rows[g].astype(np.float64) * float(w[g])
    assert got.shape == (T, D) and got.dtype == np.float32
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    untouched = np.setdiff1d(np.arange(T), idx)
    assert not got[untouched].any()


@pytest.mark.parametrize("T,D,sizes", CASES[1:4])
def test_combine_is_linear_in_weights_and_rows_and_accumulates_into_out(T, D, sizes):
    experts, idx, w, N = _case(2, T, D, sizes)
    rng = np.random.default_rng(3)
    w2 = rng.random(N).astype(np.float32)
    a = oracle.combine(experts, idx, w, T)
    b = oracle.combine(experts, idx, w2, T)
    both = oracle.combine(experts, idx, w + w2, T)
    assert np.allclose(both, a + b, rtol=1e-5, atol=1e-5)
    doubled = oracle.combine([2 * e for e in experts], idx, w, T)
    assert np.allclose(doubled, 2 * a, rtol=1e-6, atol=1e-6)
    base = rng.standard_normal((T, D)).astype(np.float32)
    out = base.copy()
    oracle.combine(experts, idx, w, T, out=out)  # `out` given: accumulated into, never zeroed
    assert np.allclose(out, base + a, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("T,D,sizes", CASES[1:4])
def test_backward_is_the_adjoint_of_forward(T, D, sizes):
    """<grad_out, combine(rows, w)> differentiated: grad_rows[g] = grad_out[idx[g]] * w[g] and
    grad_w[g] = <grad_out[idx[g]], rows[g]>; checked by the inner-product identity too."""
    experts, idx, w, N = _case(4, T, D, sizes)
    rows = np.concatenate(experts, 0)
    rng = np.random.default_rng(5)
    grad_out = rng.standard_normal((T, D)).astype(np.float32)
    grad_rows, grad_w = oracle.combine_bwd(rows, idx, w, grad_out)
    assert np.allclose(grad_rows, grad_out[idx] * w[:, None], rtol=1e-6, atol=1e-6)
    assert np.allclose(grad_w, (grad_out[idx].astype(np.float64) * rows).sum(1), rtol=1e-5, atol=1e-5)
    # adjointness in the rows: <grad_out, J v> == <J^T grad_out, v> for a random direction v
    v = rng.standard_normal(rows.shape).astype(np.float32)
    splits = np.cumsum(sizes)[:-1]
    Jv = oracle.combine(np.split(v, splits), idx, w, T)
    lhs = float((grad_out.astype(np.float64) * Jv).sum())
    rhs = float((grad_rows.astype(np.float64) * v).sum())
    assert abs(lhs - rhs) <= 1e-4 * max(1.0, abs(lhs))
    only_rows, none = oracle.combine_bwd(rows, idx, w, grad_out, with_grad_w=False)
    assert none is None and np.array_equal(only_rows, grad_rows)


def test_permute_round_trip_sums_the_copies_of_every_token():
    """permute_bwd(permute(x)) = x times the number of routed copies of each token."""
    rng = np.random.default_rng(6)
    T, D, K = 19, 12, 3
    x = rng.standard_normal((T, D)).astype(np.float32)
    reverse_map = np.repeat(np.arange(T), K)
    rng.shuffle(reverse_map)
    permuted = oracle.permute(x, reverse_map)
    assert np.array_equal(permuted, x[reverse_map])
    back = oracle.permute_bwd(permuted, reverse_map, T)
    assert np.allclose(back, K * x, rtol=1e-6, atol=1e-6)
    halves = oracle.permute(x.astype(np.float16), reverse_map)  # a 2-byte dtype moves bit for bit
    assert np.array_equal(halves, x.astype(np.float16)[reverse_map])


def test_bf16_paths_agree_with_fp32_arithmetic_within_the_bf16_bound():
    """The reference's own bf16 arithmetic and the fp32 yardstick on the same bf16 values differ by
    rounding only; the yardstick equals the fp32 oracle on the widened values exactly."""
    experts, idx, w, N = _case(7, 16, 32, [9, 0, 23, 4])
    e_bits = [oracle.f32_to_bf16_bits(e) for e in experts]
    w_bits = oracle.f32_to_bf16_bits(w)
    wide = oracle.combine([oracle.bf16_bits_to_f32(b) for b in e_bits], idx, oracle.bf16_bits_to_f32(w_bits), 16)
    yard = oracle.combine_bf16_in_f32(e_bits, idx, w_bits, 16)
    assert np.array_equal(yard, wide)
    native = oracle.bf16_bits_to_f32(oracle.combine_bf16(e_bits, idx, w_bits, 16))
    assert float(np.abs(native - yard).max()) <= 2e-2 * float(np.abs(yard).max())
    # the conversion itself: round to nearest even, exact on values that bf16 holds
    exact = np.array([0.0, 1.0, -2.5, 2.0**127, 2.0**-126], np.float32)
    assert np.array_equal(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(exact)), exact)
    assert oracle.f32_to_bf16_bits(np.array([1.00390625], np.float32))[0] == 0x3F80  # tie -> even mantissa
    assert oracle.f32_to_bf16_bits(np.array([1.01171875], np.float32))[0] == 0x3F82  # tie -> even mantissa


def test_bad_inputs_are_refused():
    experts, idx, w, _ = _case(8, 4, 2, [2, 1])
    with pytest.raises(IndexError):
        oracle.combine(experts, np.array([0, 4, 1]), w, 4)
    with pytest.raises(IndexError):
        oracle.combine(experts, np.array([0, -1, 1]), w, 4)
    with pytest.raises(ValueError):
        oracle.combine(experts, idx[:2], w[:2], 4)


@pytest.mark.parametrize("T,E,K,world", [(1, 1, 1, 1), (37, 8, 2, 1), (64, 16, 4, 4), (200, 256, 8, 8)])
def test_routing_oracle_invariants(T, E, K, world):
    """Top-k picks the K largest logits in descending order (equal values: lower expert id
    first), the gate weights are a softmax over the selected values, and the index is the stable
    expert-major sort of the T*K routed slots with its exact inverse."""
    from oracle import routing

    rng = np.random.default_rng(11)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    if E > 2:
        logits[0, 1] = logits[0, 2] = logits[0].max() + 1.0  # a tie at the top of token 0
    idx, w = routing.topk_softmax(logits, K)
    assert idx.shape == (T, K) and idx.dtype == np.int64 and w.dtype == np.float32
    picked = np.take_along_axis(logits, idx, -1)
    assert (np.diff(picked, axis=-1) <= 0).all()
    assert (np.sort(logits, -1)[:, ::-1][:, :K] == picked).all()
    assert all(len(set(row)) == K for row in idx.tolist())
    if E > 2 and K >= 2:
        assert idx[0, 0] == 1 and idx[0, 1] == 2
    assert np.allclose(w.sum(-1), 1.0, atol=1e-6) and (w > 0).all()
    want = np.exp(picked - picked.max(-1, keepdims=True))
    assert np.allclose(w, want / want.sum(-1, keepdims=True), rtol=1e-6, atol=1e-7)

    ix = routing.build_index(idx, w, E, world)
    N = T * K
    flat_e, flat_w = idx.reshape(-1), w.reshape(-1)
    order = np.argsort(flat_e, kind="stable")
    assert np.array_equal(ix["reverse_map"], order // K)
    assert np.array_equal(ix["sorted_w"], flat_w[order])
    assert np.array_equal(ix["counts"], np.bincount(flat_e, minlength=E))
    assert np.array_equal(ix["offsets"], np.cumsum(ix["counts"]) - ix["counts"])
    assert int(ix["counts"].sum()) == N
    assert np.array_equal(ix["expert_counts_by_rank"], ix["counts"].reshape(world, E // world))
    assert np.array_equal(ix["rank_counts"], ix["counts"].reshape(world, -1).sum(1))
    assert ix["slot_of"].dtype == np.int32 and np.array_equal(order[ix["slot_of"]], np.arange(N))
    # every expert's segment of the sorted order holds its own slots in ascending routed position
    sorted_e = flat_e[order]
    assert (np.diff(sorted_e) >= 0).all()
    same = np.diff(sorted_e) == 0
    assert (np.diff(order)[same] > 0).all()


def test_metadata_oracle_handles_empty_and_ragged_experts():
    from oracle import routing

    sizes, offsets, max_rows, n = routing.prepare_metadata([3, 0, 5, 0])
    assert sizes.dtype == np.int32 and offsets.dtype == np.int64
    assert sizes.tolist() == [3, 0, 5, 0] and offsets.tolist() == [0, 3, 3, 8] and (max_rows, n) == (5, 4)
    sizes, offsets, max_rows, n = routing.prepare_metadata([])
    assert len(sizes) == 0 and len(offsets) == 0 and (max_rows, n) == (0, 0)
