"""The host-buffer entry point of the C ABI (fmoe_combine_host): copies in, plans, gathers and
copies out, in one piece or pipelined over slices of columns. Checked against the CPU oracle
(bit-exact in fp32) and against the device-resident operator on the same values."""

import ctypes

import numpy as np
import pytest
import torch

from fastmoe_b200 import _lib
from fastmoe_b200.kernels import ops
from util import assert_close, oracle_combine

pytestmark = pytest.mark.gpu

DEV = "cuda"
TAGS = {torch.float32: _lib.FMOE_F32, torch.bfloat16: _lib.FMOE_BF16, torch.float16: _lib.FMOE_F16}

# (T, D, rows per expert, dtype, index dtype, host_chunks knob (0 = library's choice), pinned)
CASES = [
    (40, 64, [5, 0, 7, 3], torch.float32, torch.int64, 0, True),  # short rows: one piece
    (33, 4352, [9, 0, 17, 1, 30], torch.float32, torch.int32, 3, True),  # three slices, last one narrower
    (64, 8192, [100, 50, 0, 106], torch.bfloat16, torch.int64, 0, True),  # 16 KB rows: sliced by default
    (64, 8192, [100, 50, 0, 106], torch.bfloat16, torch.int64, 1, True),  # the same in one piece
    (16, 8196, [20, 12], torch.bfloat16, torch.int64, 2, True),  # rows that rule out 16-byte stores
    (24, 8192, [31, 33], torch.float16, torch.int64, 4, False),  # pageable host memory
]


def _host(t, pinned):
    t = t.cpu().contiguous()
    return t.pin_memory() if pinned else t


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"T{c[0]}-D{c[1]}-E{len(c[2])}-{str(c[3])[6:]}-chunks{c[5]}")
def test_host_call_matches_oracle_and_device_operator(case):
    T, D, sizes, dtype, itype, chunks, pinned = case
    g = torch.Generator().manual_seed(T * 131 + D)
    N, E = sum(sizes), len(sizes)
    experts = [_host(torch.randn(n, D, generator=g).to(dtype), pinned) for n in sizes]
    idx = _host(torch.randint(0, T, (N,), generator=g).to(itype), pinned)
    w = _host(torch.rand(N, generator=g).to(dtype), pinned)
    out_host = _host(torch.full((T, D), float("nan")).to(dtype), pinned)

    lib = _lib.lib()
    c_sizes = (ctypes.c_int64 * E)(*sizes)
    c_ptrs = (ctypes.c_void_p * E)(*[e.data_ptr() if e.numel() else None for e in experts])
    arena_bytes = lib.fmoe_combine_host_arena_bytes(c_sizes, E, N, T, D, TAGS[dtype])
    assert arena_bytes > N * D * experts[0].element_size()
    arena = torch.empty(arena_bytes, dtype=torch.uint8, device=DEV)
    _lib.tune("host_chunks", chunks)
    try:
        for _ in range(2):  # the second call reuses the arena and the library's helper stream
            out_host.fill_(float("nan"))
            _lib.call("fmoe_combine_host", c_ptrs, c_sizes, idx.data_ptr(),
                      _lib.FMOE_I32 if itype == torch.int32 else _lib.FMOE_I64, w.data_ptr(), TAGS[dtype],
                      out_host.data_ptr(), E, N, T, D, TAGS[dtype], arena.data_ptr(), arena_bytes,
                      torch.cuda.current_stream().cuda_stream)  # fmt: skip
            want = oracle_combine(experts, idx, w, T)
            assert_close(out_host, want, dtype, "host call vs oracle")
            if dtype == torch.float32:
                assert np.array_equal(out_host.numpy(), want), "fp32 host call is not bit-exact"
    finally:
        _lib.tune("host_chunks", 1)  # the library default
    on_device = ops.grouped_weighted_scatter_add(
        [e.to(DEV) for e in experts], idx.to(DEV), w.to(DEV), (T, D)
    )
    assert torch.equal(on_device.cpu(), out_host), "host call and device operator disagree"


def test_host_call_rejects_bad_arguments_before_copying():
    lib = _lib.lib()
    sizes = (ctypes.c_int64 * 2)(3, 4)
    rows = [torch.zeros(3, 8), torch.zeros(4, 8)]
    ptrs = (ctypes.c_void_p * 2)(*[r.data_ptr() for r in rows])
    idx, w, out = torch.zeros(7, dtype=torch.int64), torch.zeros(7), torch.zeros(5, 8)
    need = lib.fmoe_combine_host_arena_bytes(sizes, 2, 7, 5, 8, _lib.FMOE_F32)
    arena = torch.empty(need, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    with pytest.raises(ValueError, match="sum to"):  # sizes do not add up to N
        _lib.call("fmoe_combine_host", ptrs, sizes, idx.data_ptr(), _lib.FMOE_I64, w.data_ptr(), _lib.FMOE_F32,
                  out.data_ptr(), 2, 8, 5, 8, _lib.FMOE_F32, arena.data_ptr(), need, stream)  # fmt: skip
    with pytest.raises(ValueError, match="arena"):  # arena too small
        _lib.call("fmoe_combine_host", ptrs, sizes, idx.data_ptr(), _lib.FMOE_I64, w.data_ptr(), _lib.FMOE_F32,
                  out.data_ptr(), 2, 7, 5, 8, _lib.FMOE_F32, arena.data_ptr(), need - 256, stream)  # fmt: skip
    idx[3] = 5  # outside [0, T): the row is skipped and the call says so
    with pytest.raises(ValueError, match="outside"):
        _lib.call("fmoe_combine_host", ptrs, sizes, idx.data_ptr(), _lib.FMOE_I64, w.data_ptr(), _lib.FMOE_F32,
                  out.data_ptr(), 2, 7, 5, 8, _lib.FMOE_F32, arena.data_ptr(), need, stream)  # fmt: skip
