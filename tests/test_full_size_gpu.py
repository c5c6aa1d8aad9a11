"""Parity at the benchmark configurations' FULL sizes: the bf16 combine of the microbenchmark
(T=8192, D=16384, E=256, top-8) with softmax routing and with Zipf-skewed routing, against the
C oracle's fp32 arithmetic on the very same bf16 inputs (2.1 GB of rows copied to the host),
plus the size-independent properties: bit-reproducibility and linearity in the gate weights."""

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200.kernels import ops
from fastmoe_b200.workloads import make_combine_workload
from util import to_np

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("routing", ["softmax", "zipf"])
def test_combine_full_size_against_oracle(routing):
    T, D, E, K = 8192, 16384, 256, 8
    wl = make_combine_workload(T, D, E, K, torch.bfloat16, routing, seed=0)
    assert wl.N == T * K and sum(wl.counts) == wl.N
    if routing == "zipf":
        assert max(wl.counts) > 0.9 * T and min(wl.counts) < 64  # one hot expert, many nearly idle ones
    out = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (T, D))
    again = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (T, D))
    assert torch.equal(out, again)  # no atomics: bit-reproducible
    assert ops.read_status() == 0

    oracle.use_all_cores()
    ref = oracle.combine_bf16_in_f32([_bits(e) for e in wl.experts], wl.indices.cpu().numpy(), _bits(wl.weights), T)
    got = to_np(out)
    scale = float(np.abs(ref).max())
    err = float(np.abs(got - ref).max()) / scale
    assert err <= 2e-2, err
    # fp32 accumulation and ONE rounding: within half a bf16 ulp of the fp32 result, element by element
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0**-8 + 1e-30)

    # linearity in the gate weights: combine(2w) == 2 * combine(w) exactly (a power of two)
    doubled = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights * 2, (T, D))
    assert torch.equal(doubled.float(), out.float() * 2)

    # the scatter form (atomics in bf16) stays inside the 2e-2 bound as well
    acc = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    ops.set_combine_mode("scatter")
    try:
        ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, (T, D), out=acc)
    finally:
        ops.set_combine_mode("gather")
    assert float(np.abs(to_np(acc) - ref).max()) / scale <= 2e-2
