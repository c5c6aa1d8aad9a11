"""The tcgen05 grouped GEMM against a plain PyTorch fp32 reference of the same product
(bf16 inputs, fp32 accumulation, one rounding to bf16): tolerance 2e-2 of the largest
magnitude, stated once in util.REL_TOL."""

import pytest
import torch

from fastmoe_b200.kernels import experts, ops
from util import REL_TOL

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(a, w, counts, swiglu):
    out, o = [], 0
    for e, n in enumerate(counts):
        h = a[o : o + n].float() @ w[e].float().t()
        if swiglu:
            ff = h.shape[1] // 2
            h = torch.nn.functional.silu(h[:, :ff]) * h[:, ff:]
        out.append(h)
        o += n
    return torch.cat(out, 0)


def _case(counts, K, N, swiglu, seed=0):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    R, E = sum(counts), len(counts)
    a = torch.randn(R, K, generator=gen, device=DEV).bfloat16()
    w = (torch.randn(E, N, K, generator=gen, device=DEV) / K**0.5).bfloat16()
    cnt = torch.tensor(counts, dtype=torch.int64, device=DEV)
    off = torch.cumsum(cnt, 0) - cnt
    return a, w, off, cnt


CASES = [
    ([128], 64, 256, False),  # one tile, one k-block
    ([128], 256, 256, False),  # pipeline wraps once
    ([128], 64, 256, True),
    ([200, 0, 5, 300], 512, 512, False),  # ragged, an empty expert, several column blocks
    ([200, 0, 5, 300], 512, 512, True),
    ([1] * 40, 128, 256, False),  # many one-row experts
    ([700, 33], 7168, 256, False),  # deep K: the pipeline wraps many times
    ([513, 127, 129], 1024, 1024, True),
    ([256, 257, 16, 17, 270, 0, 255], 256, 512, True),  # around the row-block boundaries
    ([256, 257, 16, 17, 270, 0, 255], 256, 512, False),
]


@pytest.mark.parametrize("counts,K,N,swiglu", CASES)
def test_grouped_gemm_matches_fp32_reference(counts, K, N, swiglu):
    a, w, off, cnt = _case(counts, K, N, swiglu)
    c = experts.grouped_gemm(a, w, off, cnt, swiglu=swiglu)
    torch.cuda.synchronize()
    assert ops.read_status() == 0, "a bounded wait timed out inside the kernel"
    ref = _reference(a, w, counts, swiglu)
    assert c.shape == ref.shape and c.dtype == torch.bfloat16
    err = float((c.float() - ref).abs().max() / ref.abs().max())
    assert err <= REL_TOL[torch.bfloat16], err
    assert err <= 1e-2  # fp32 accumulation + one bf16 rounding is far inside the bound


def test_rows_outside_every_expert_stay_zero_and_backward_runs():
    a, w, off, cnt = _case([100, 60], 128, 256, False, seed=3)
    pad = torch.randn(40, 128, device=DEV).bfloat16()
    a2 = torch.cat([a[:100], pad, a[100:]], 0).requires_grad_(True)  # 40 unowned rows in the middle
    off2 = torch.tensor([0, 140], dtype=torch.int64, device=DEV)
    w2 = w.clone().requires_grad_(True)
    c = experts.grouped_gemm(a2, w2, off2, cnt)
    assert float(c[100:140].abs().max()) == 0.0
    ref = torch.cat([a[:100].float() @ w[0].float().t(), a[100:].float() @ w[1].float().t()], 0)
    got = torch.cat([c[:100], c[140:]], 0).float()
    assert float((got - ref).abs().max() / ref.abs().max()) <= 1e-2
    c.sum().backward()
    assert a2.grad is not None and w2.grad is not None and float(a2.grad[100:140].abs().max()) == 0.0


def test_swiglu_ffn_end_to_end():
    counts = [300, 17, 0, 200]
    a, w_gu, off, cnt = _case(counts, 256, 512, True, seed=5)
    gen = torch.Generator(device=DEV).manual_seed(6)
    w_down = (torch.randn(4, 256, 256, generator=gen, device=DEV) / 16).bfloat16()
    y = experts.grouped_swiglu_ffn(a, w_gu, w_down, off, cnt)
    hidden = _reference(a, w_gu, counts, True).bfloat16()
    ref = _reference(hidden, w_down, counts, False)
    assert float((y.float() - ref).abs().max() / ref.abs().max()) <= REL_TOL[torch.bfloat16]
    assert ops.read_status() == 0


def test_unsupported_shapes_raise():
    a, w, off, cnt = _case([16], 64, 256, False)
    with pytest.raises(ValueError):
        experts.grouped_gemm(a[:, :48].contiguous(), w[:, :, :48].contiguous(), off, cnt)  # K % 64
    with pytest.raises(ValueError):
        experts.grouped_gemm(a, w[:, :100].contiguous(), off, cnt)  # N % 256
    with pytest.raises(ValueError):
        experts.grouped_gemm(a.float(), w.float(), off, cnt)


def test_row_map_scatters_the_output_rows():
    counts = [150, 0, 90, 260]
    a, w, off, cnt = _case(counts, 256, 512, False, seed=8)
    R = sum(counts)
    perm = torch.randperm(R, device=DEV)
    plain = experts.grouped_gemm(a, w, off, cnt, covers_all_rows=True)
    mapped = experts.grouped_gemm(a, w, off, cnt, row_map=perm, covers_all_rows=True)
    expect = torch.empty_like(plain)
    expect[perm] = plain
    assert torch.equal(mapped, expect)
    wgu = w
    fused = experts.grouped_gemm(a, wgu, off, cnt, swiglu=True, row_map=perm, covers_all_rows=True)
    ref = torch.empty_like(fused)
    ref[perm] = experts.grouped_gemm(a, wgu, off, cnt, swiglu=True)
    assert torch.equal(fused, ref)


def test_bounded_waits_give_up_and_report_instead_of_hanging():
    """Failure detection without a fault: with the producer told to load nothing, the MMA and
    epilogue roles' mbarrier waits run out (short limit), the kernel sets the WAIT_TIMEOUT status
    bit, releases its tensor memory and returns; the context stays usable and the next launch is
    correct."""
    from fastmoe_b200 import _lib

    a, w, off, cnt = _case([300, 100], 256, 256, False, seed=11)
    _lib.tune("gemm_spin_limit", 1 << 12)
    _lib.tune("gemm_skip_loads", 1)
    try:
        experts.grouped_gemm(a, w, off, cnt)
        torch.cuda.synchronize()
        assert ops.read_status() & 8
    finally:
        _lib.tune("gemm_skip_loads", 0)
        _lib.tune("gemm_spin_limit", 1 << 24)
    c = experts.grouped_gemm(a, w, off, cnt)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    ref = _reference(a, w, [300, 100], False)
    assert float((c.float() - ref).abs().max() / ref.abs().max()) <= 1e-2


@pytest.mark.parametrize("counts,K,N,swiglu", [
    ([128], 256, 256, False),
    ([200, 0, 5, 300], 512, 512, False),
    ([200, 0, 5, 300], 512, 512, True),
    ([700, 33, 64], 768, 1024, True),
])  # fmt: skip
def test_backward_on_tensor_cores_matches_fp32_autograd(counts, K, N, swiglu):
    """Data and weight gradients (tcgen05 kernels with the contiguous dimension as MN, ragged
    row reduction masked in shared memory) against fp32 autograd of the same products."""
    a, w, off, cnt = _case(counts, K, N, swiglu, seed=21)
    a.requires_grad_(True)
    w.requires_grad_(True)
    c = experts.grouped_gemm(a, w, off, cnt, swiglu=swiglu)
    gen = torch.Generator(device=DEV).manual_seed(22)
    g = torch.randn(c.shape, generator=gen, device=DEV).bfloat16()
    c.backward(g)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    a32 = a.detach().float().requires_grad_(True)
    w32 = w.detach().float().requires_grad_(True)
    _reference(a32, w32, counts, swiglu).backward(g.float())
    for got, want, what in ((a.grad, a32.grad, "grad_a"), (w.grad, w32.grad, "grad_w")):
        err = float((got.float() - want).abs().max() / want.abs().max())
        assert err <= REL_TOL[torch.bfloat16], (what, err)
    assert float(w.grad[1].abs().max()) == 0.0 if counts[1:2] == [0] else True  # an expert without rows


def test_swiglu_derivative_over_a_capacity_sized_buffer():
    """fmoe_swiglu_bwd_ragged touches only the rows a device-side count names; the plain entry
    point is the same kernel over all rows. Checked against autograd of silu(gate) * up in fp32."""
    from fastmoe_b200.kernels.ops import _stream_ptr

    rows, used, ff = 96, 41, 256
    gen = torch.Generator(device=DEV).manual_seed(3)
    h = torch.randn(rows, 2 * ff, generator=gen, device=DEV).bfloat16()
    g = torch.randn(rows, ff, generator=gen, device=DEV).bfloat16()
    hf = h.float().requires_grad_(True)
    (torch.nn.functional.silu(hf[:, :ff]) * hf[:, ff:] * g.float()).sum().backward()
    want = hf.grad
    sentinel = 7.0
    for count in (used, None):
        out = torch.full_like(h, sentinel)
        if count is None:
            ops._call("fmoe_swiglu_bwd", 1, h.data_ptr(), g.data_ptr(), out.data_ptr(), rows, ff, _stream_ptr(h.device))
            n = rows
        else:
            cnt = torch.tensor([count], dtype=torch.int64, device=DEV)
            ops._call("fmoe_swiglu_bwd_ragged", 1, h.data_ptr(), g.data_ptr(), out.data_ptr(), rows, ff,
                      cnt.data_ptr(), _stream_ptr(h.device))  # fmt: skip
            n = count
        torch.cuda.synchronize()
        err = float((out[:n].float() - want[:n]).abs().max() / want.abs().max())
        assert err <= REL_TOL[torch.bfloat16], err
        assert bool((out[n:] == sentinel).all()), "rows past the count were written"
