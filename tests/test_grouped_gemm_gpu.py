"""The tcgen05 grouped GEMM against a plain PyTorch fp32 reference of the same product
(bf16 inputs, fp32 accumulation, one rounding to bf16): tolerance 2e-2 of the largest
magnitude, stated once in util.REL_TOL."""

import pytest
import torch

from fastmoe_b200.kernels import experts, ops
from util import REL_TOL

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=["tokens_as_m", "tokens_as_n"], autouse=True)
def forward_kernel(request):
    """Every test of this file runs with each of the two forward kernels behind fmoe_grouped_gemm:
    tokens in 128-row blocks as the MMA's M dimension, and tokens in 16-row steps as its N
    dimension (left to itself the library picks by the average rows per expert)."""
    from fastmoe_b200 import _lib

    _lib.tune("gemm_tokens_as_n", 1 if request.param == "tokens_as_n" else 0)
    yield request.param
    _lib.tune("gemm_tokens_as_n", -1)


def _reference(a, w, counts, swiglu, gelu=False):
    out, o = [], 0
    for e, n in enumerate(counts):
        h = a[o : o + n].float() @ w[e].float().t()
        if swiglu:
            ff = h.shape[1] // 2
            h = torch.nn.functional.silu(h[:, :ff]) * h[:, ff:]
        if gelu:
            h = torch.nn.functional.gelu(h)  # the exact (erf) form, nn.GELU()'s default
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
    ([511, 513, 15, 31, 33, 1023, 1], 128, 256, False),  # equal shares of 2, 3 and 4 tiles; sub-box experts
    ([511, 513, 15, 31, 33, 1023, 1], 128, 256, True),
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
    a, w, off, cnt = _case([100, 60], 256, 256, False, seed=3)
    pad = torch.randn(40, 256, device=DEV).bfloat16()
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
    # a width only the forward tiles: asking for gradients raises too, up front (no library fallback)
    experts.grouped_gemm(a, w, off, cnt)
    with pytest.raises(ValueError, match="gradients"):
        experts.grouped_gemm(a.clone().requires_grad_(True), w, off, cnt)  # K = 64 is not a multiple of 256


@pytest.mark.parametrize("counts,K,N", [([128], 64, 256), ([200, 0, 5, 300], 512, 512), ([513, 127, 129], 256, 1024)])
def test_gelu_epilogue_matches_fp32_reference(counts, K, N):
    """The reference's own expert is Linear-GELU-Linear: the first product with the exact GELU
    fused into the epilogue."""
    a, w, off, cnt = _case(counts, K, N, False, seed=31)
    c = experts.grouped_gemm(a, w, off, cnt, activation=experts.ACT_GELU)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    ref = _reference(a, w, counts, False, gelu=True)
    err = float((c.float() - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, err


def test_gelu_ffn_forward_and_backward_match_fp32_autograd():
    counts, D, FF = [300, 17, 0, 200], 256, 512
    a, w1, off, cnt = _case(counts, D, FF, False, seed=33)
    gen = torch.Generator(device=DEV).manual_seed(34)
    w2 = (torch.randn(len(counts), D, FF, generator=gen, device=DEV) / FF**0.5).bfloat16()
    g = torch.randn(sum(counts), D, generator=gen, device=DEV).bfloat16()
    a.requires_grad_(True), w1.requires_grad_(True), w2.requires_grad_(True)
    y = experts.grouped_gelu_ffn(a, w1, w2, off, cnt, covers_all_rows=True)
    y.backward(g)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    a32, w1_32, w2_32 = (t.detach().float().requires_grad_(True) for t in (a, w1, w2))
    hidden = _reference(a32, w1_32, counts, False, gelu=True)
    ref = _reference(hidden, w2_32, counts, False)
    ref.backward(g.float())
    tol = REL_TOL[torch.bfloat16]
    assert float((y.float() - ref).abs().max() / ref.abs().max()) <= tol
    for got, want, what in ((a.grad, a32.grad, "dx"), (w1.grad, w1_32.grad, "dw1"), (w2.grad, w2_32.grad, "dw2")):
        err = float((got.float() - want).abs().max() / want.abs().max())
        assert err <= tol, (what, err)


def test_counts_that_run_past_the_rows_are_cut_off():
    """Counts that claim more rows than A has (what an overflowing receive buffer would hand
    over): the last expert is cut at A's end, nothing beyond A or C is read or written, and
    the status word says so."""
    real = [200, 100]
    a, w, off, _ = _case(real, 256, 256, False, seed=41)
    claimed = torch.tensor([200, 260], dtype=torch.int64, device=DEV)  # 160 rows more than exist
    guard = torch.full((64, 256), 7.0, dtype=torch.bfloat16, device=DEV)
    c = torch.cat([torch.zeros(300, 256, dtype=torch.bfloat16, device=DEV), guard], 0)  # C with a canary behind it
    experts._launch(a, w, off, claimed, experts.ACT_NONE, out=c[:300])
    torch.cuda.synchronize()
    assert ops.read_status() & 2
    assert bool((c[300:] == 7.0).all()), "rows behind C were written"
    ref = _reference(a, w, real, False)
    assert float((c[:300].float() - ref).abs().max() / ref.abs().max()) <= 1e-2
    # the same through a table of row addresses that has exactly one entry per row of A
    out = torch.zeros(300 + 64, 256, dtype=torch.bfloat16, device=DEV)
    ptrs = out.data_ptr() + torch.arange(300, device=DEV, dtype=torch.int64) * 512
    experts._launch(a, w, off, claimed, experts.ACT_NONE, row_ptrs=ptrs)
    torch.cuda.synchronize()
    assert ops.read_status() & 2
    assert float(out[300:].abs().max()) == 0.0
    assert float((out[:300].float() - ref).abs().max() / ref.abs().max()) <= 1e-2


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


def test_weight_gradient_ignores_nan_rows_behind_the_last_expert():
    """Capacity-sized operands: rows behind the last expert's end hold whatever the allocator
    left there, NaN bit patterns included. The ragged last chunk is cleared in BOTH operands
    before the MMAs, so none of it reaches the weight gradient (0 x NaN would be NaN)."""
    counts = [130, 70]  # 200 rows in use; the last 64-row chunk of expert 1 reaches rows 200..255
    a, w, off, cnt = _case(counts, 256, 256, False, seed=51)
    gen = torch.Generator(device=DEV).manual_seed(52)
    g = torch.randn(200, 256, generator=gen, device=DEV).bfloat16()
    nan_tail = torch.full((120, 256), float("nan"), dtype=torch.bfloat16, device=DEV)
    inf_tail = torch.full((120, 256), float("inf"), dtype=torch.bfloat16, device=DEV)
    for a_tail, g_tail in ((nan_tail, nan_tail), (inf_tail, torch.zeros_like(nan_tail)), (nan_tail, inf_tail)):
        a_cap, g_cap = torch.cat([a, a_tail], 0), torch.cat([g, g_tail], 0)
        grad_w = experts._wgrad(g_cap, a_cap, w.shape, off, cnt)
        torch.cuda.synchronize()
        assert ops.read_status() == 0
        assert bool(torch.isfinite(grad_w.float()).all())
        for e, (o, n) in enumerate(zip([0, 130], counts)):
            ref = g[o : o + n].float().t() @ a[o : o + n].float()
            assert float((grad_w[e].float() - ref).abs().max() / ref.abs().max()) <= REL_TOL[torch.bfloat16]


def test_expert_parallel_layer_sized_products():
    """The sizes the expert-parallel layer runs: one rank of eight (32 experts x 2048 rows,
    7168 -> 2 x 2048 SwiGLU and 2048 -> 7168) and a single rank (256 experts x 256 rows, where
    the weight tensor map has 1,048,576 rows). Checked on whole experts at the front, the
    middle and the end against fp32 products of the same bf16 values."""
    D, FF = 7168, 2048
    for E, per in ((32, 2048), (256, 256)):
        R = E * per
        gen = torch.Generator(device=DEV).manual_seed(60 + E)
        cnt = torch.full((E,), per, dtype=torch.int64, device=DEV)
        jitter = torch.randint(-(per // 8), per // 8 + 1, (E // 2,), generator=gen, device=DEV)
        cnt[: E // 2] += jitter
        cnt[E // 2 :] -= jitter.flip(0)
        off = torch.cumsum(cnt, 0) - cnt
        x = torch.randn(R, D, generator=gen, device=DEV, dtype=torch.bfloat16)
        wgu = torch.empty(E, 2 * FF, D, device=DEV, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        wd = torch.empty(E, D, FF, device=DEV, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        with torch.no_grad():
            hidden = experts.grouped_gemm(x, wgu, off, cnt, swiglu=True, covers_all_rows=True)
            y = experts.grouped_gemm(hidden, wd, off, cnt, covers_all_rows=True)
        torch.cuda.synchronize()
        assert ops.read_status() == 0
        for e in (0, E // 2 - 1, E // 2, E - 1):
            o, n = int(off[e]), int(cnt[e])
            h = x[o : o + n].float() @ wgu[e].float().t()
            ref_h = torch.nn.functional.silu(h[:, :FF]) * h[:, FF:]
            err_h = float((hidden[o : o + n].float() - ref_h).abs().max() / ref_h.abs().max())
            ref_y = hidden[o : o + n].float() @ wd[e].float().t()
            err_y = float((y[o : o + n].float() - ref_y).abs().max() / ref_y.abs().max())
            assert err_h <= 1e-2 and err_y <= 1e-2, (E, e, err_h, err_y)
        del x, wgu, wd, hidden, y
        torch.cuda.empty_cache()


@pytest.mark.parametrize("act", ["swiglu", "gelu"])
def test_training_forward_keeps_the_products_before_the_activation(act):
    """fmoe_grouped_gemm_keep_pre: the result is what the plain entry point gives, and `pre`
    holds the product before the activation (gate columns, then up columns, for SwiGLU), row r of
    A in row r of `pre` even when the result rows are scattered through a row map; rows that
    belong to no expert are left alone."""
    counts, K, N = [200, 0, 5, 300], 256, 512
    a, w, off, cnt = _case(counts, K, N, act == "swiglu", seed=71)
    pad = torch.zeros(24, K, device=DEV, dtype=torch.bfloat16)
    a = torch.cat([a, pad], 0)  # 24 rows behind the last expert
    R = a.shape[0]
    code = experts.ACT_SWIGLU if act == "swiglu" else experts.ACT_GELU
    perm = torch.randperm(R, device=DEV)
    want = experts._launch(a, w, off, cnt, code, row_map=perm)
    pre = torch.full((R, N), 3.0, dtype=torch.bfloat16, device=DEV)
    got = experts._launch(a, w, off, cnt, code, row_map=perm, pre=pre)
    plain = experts._launch(a, w, off, cnt, experts.ACT_NONE)
    torch.cuda.synchronize()
    assert ops.read_status() == 0
    used = sum(counts)
    assert torch.equal(got[perm[:used]], want[perm[:used]])
    assert torch.equal(pre[:used], plain[:used])
    assert bool((pre[used:] == 3.0).all()), "rows of no expert were written"
    with pytest.raises(ValueError):
        experts._launch(a, w, off, cnt, code, pre=pre[:, : N // 2].contiguous())
