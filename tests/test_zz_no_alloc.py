"""fmoe_combine_fwd_static — the combine for hosts that cannot allocate device memory
(a plugin inside a framework that owns all of HBM, a serving loop that cannot take
cudaMalloc's device-wide stall): its plan lives in a fixed array inside the library.

Checked through the C ABI against the regular pair fmoe_combine_plan +
fmoe_combine_gather (caller-provided scratch) on two calls in a row with different
inputs, so that anything left over from the first call would show in the second.
Both paths run the same kernels in the same order: the outputs must be identical.
The first call's output is also held against the CPU oracle's fp32 arithmetic on the
same bf16 values, so the test stands on its own if the regular path were wrong too.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200 import _lib
from fastmoe_b200.kernels import ops
from fastmoe_b200.workloads import make_combine_workload

pytestmark = pytest.mark.gpu

STATIC_BYTES = 4194304  # FMOE_STATIC_SCRATCH_BYTES in include/fastmoe_b200.h


def _both_paths(wl, accumulate, out0):
    meta = ops.prepare_grouped_metadata(wl.experts, wl.experts[0].device)
    ptr_table, chunk_sizes, expert_offsets, _, E = meta
    dev = wl.indices.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    common = (ptr_table.data_ptr(), chunk_sizes.data_ptr(), expert_offsets.data_ptr(),
              wl.indices.data_ptr(), _lib.FMOE_I64, wl.weights.data_ptr(), _lib.FMOE_BF16)  # fmt: skip

    out_static = out0.clone()
    _lib.call("fmoe_combine_fwd_static", *common, out_static.data_ptr(), wl.D, E, wl.N, wl.T, wl.D,
              _lib.FMOE_BF16, accumulate, status.data_ptr(), stream)  # fmt: skip

    nbytes = _lib.lib().fmoe_combine_plan_bytes(wl.N, wl.T)
    plan = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out_ref = out0.clone()
    _lib.call("fmoe_combine_plan", *common, E, wl.N, wl.T, wl.D, _lib.FMOE_BF16, plan.data_ptr(), nbytes,
              status.data_ptr(), stream)  # fmt: skip
    _lib.call("fmoe_combine_gather", plan.data_ptr(), out_ref.data_ptr(), wl.D, wl.N, wl.T, wl.D,
              _lib.FMOE_BF16, accumulate, stream)  # fmt: skip
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0
    return out_static, out_ref


def test_static_entry_point_matches_regular_path_twice_in_a_row():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    # first call: larger problem, fresh output; second call: smaller problem with other routing,
    # accumulating into a non-zero output -- stale plan entries from call one would corrupt it
    first = make_combine_workload(T=512, D=1024, E=32, K=8, dtype=torch.bfloat16, routing="softmax", seed=21, device=dev)
    second = make_combine_workload(T=300, D=1024, E=16, K=4, dtype=torch.bfloat16, routing="zipf", seed=22, device=dev)
    garbage = torch.full((first.T, first.D), 7.0, dtype=torch.bfloat16, device=dev)
    a_static, a_ref = _both_paths(first, accumulate=0, out0=garbage)
    assert torch.equal(a_static, a_ref)
    assert float(a_ref.float().abs().max()) > 0 and not bool((a_ref == 7.0).all())
    want = oracle.combine([e.float().cpu().numpy() for e in first.experts], first.indices.cpu().numpy(),
                          first.weights.float().cpu().numpy(), first.T)  # fmt: skip
    err = float(np.abs(a_static.float().cpu().numpy() - want).max()) / float(np.abs(want).max())
    assert err <= 2e-2, err  # the bf16 bound of the other parity tests
    base = torch.randn(second.T, second.D, device=dev).to(torch.bfloat16)
    b_static, b_ref = _both_paths(second, accumulate=1, out0=base)
    assert torch.equal(b_static, b_ref)
    # and the first problem again, to see that call two left nothing behind either
    c_static, c_ref = _both_paths(first, accumulate=0, out0=garbage)
    assert torch.equal(c_static, c_ref) and torch.equal(c_static, a_static)


def test_static_entry_point_refuses_what_does_not_fit():
    lib = _lib.lib()
    assert lib.fmoe_combine_plan_bytes(131072, 16384) <= STATIC_BYTES  # the documented size that fits
    too_many = 1 << 20
    assert lib.fmoe_combine_plan_bytes(too_many, 16384) > STATIC_BYTES
    with pytest.raises(ValueError, match="built-in array holds"):
        _lib.call("fmoe_combine_fwd_static", None, None, None, None, 0, None, 0, None, 8, 4, too_many, 16384, 8,
                  _lib.FMOE_BF16, 0, None, None)  # fmt: skip
