"""Host-side logic that needs no GPU: metadata builder against the reference fixture,
argument checking, the synthetic workloads' routing, and the no-CPU-path rule."""

import numpy as np
import pytest
import torch

import oracle
from fastmoe_b200.consts import MoEImplementation
from fastmoe_b200.kernels import ops
from fastmoe_b200.workloads import ROUTINGS, sort_routing


@pytest.mark.parametrize("name", ["grouped_ragged", "grouped_one_target", "grouped_single"])
def test_prepare_grouped_metadata_matches_reference(golden, name):
    g = golden(name)
    offs = np.concatenate([[0], np.cumsum(g["sizes"])]).astype(int)
    ex = [torch.from_numpy(g["rows"][offs[e] : offs[e + 1]].copy()) for e in range(len(g["sizes"]))]
    meta = ops.prepare_grouped_metadata(ex, "cpu")
    ptr_table, chunk_sizes, expert_offsets, max_rows, num_experts = meta  # unpacks like the reference's tuple
    assert ptr_table.dtype == torch.int64 and ptr_table.tolist() == [t.data_ptr() for t in ex]
    assert chunk_sizes.dtype == torch.int32 and np.array_equal(chunk_sizes.numpy(), g["chunk_sizes"])
    assert expert_offsets.dtype == torch.int64 and np.array_equal(expert_offsets.numpy(), g["expert_offsets"])
    assert max_rows == int(g["max_rows"]) and num_experts == int(g["num_experts"])
    assert meta.num_rows == int(g["sizes"].sum()) and meta.dim == g["rows"].shape[1]


def test_metadata_keeps_contiguous_copies_alive():
    wide = torch.randn(6, 16)
    meta = ops.prepare_grouped_metadata([wide[:, :8], torch.randn(2, 8)], "cpu")
    assert meta.keepalive is not None and meta[0][0].item() == meta.keepalive[0].data_ptr()
    with pytest.raises(ValueError):
        ops.prepare_grouped_metadata([torch.randn(2, 8), torch.randn(2, 4)], "cpu")
    empty = ops.prepare_grouped_metadata([], "cpu")
    assert empty[3] == 0 and empty[4] == 0


def test_cpu_tensors_are_refused():
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.weighted_scatter_add(torch.zeros(2, 4), torch.zeros(2, dtype=torch.int64), torch.ones(2), (2, 4))
    with pytest.raises(ValueError):
        ops.set_combine_mode("triton")
    assert MoEImplementation.FAST == "fast" and MoEImplementation.STANDARD == "standard"
    assert ops.HAS_TRITON is False


@pytest.mark.parametrize("routing", sorted(ROUTINGS))
def test_workload_routing_is_valid_and_sorted(routing):
    T, E, K = 64, 16, 4
    idx, w = ROUTINGS[routing](T, E, K, seed=1)
    assert idx.shape == (T, K) and all(len(set(r)) == K for r in idx.tolist())  # K distinct experts
    assert torch.allclose(w.sum(-1), torch.ones(T), atol=1e-5)
    rev, sw, counts = sort_routing(idx, w, E)
    ix = oracle.build_index(idx.numpy(), w.numpy(), E)
    assert np.array_equal(rev.numpy(), ix["reverse_map"]) and np.array_equal(counts.numpy(), ix["counts"])
    assert np.array_equal(sw.numpy(), ix["sorted_w"])


def test_expert_and_exchange_wrappers_refuse_cpu_and_bad_shapes():
    from fastmoe_b200 import ep_fused, exchange
    from fastmoe_b200.kernels import experts, routing

    a, w = torch.zeros(4, 64, dtype=torch.bfloat16), torch.zeros(1, 256, 64, dtype=torch.bfloat16)
    cnt = torch.tensor([4])
    with pytest.raises(RuntimeError, match="no CPU path"):
        experts.grouped_gemm(a, w, cnt - 4, cnt)
    with pytest.raises(RuntimeError, match="no CPU path"):
        routing.route_topk(torch.zeros(4, 8), 2)
    with pytest.raises(RuntimeError, match="process group"):
        ep_fused.FusedExpertParallel(object(), 16)
    # the layout arithmetic of the fused exchange is plain tensor code and runs anywhere
    C = torch.tensor([[3, 0, 2, 1], [1, 4, 0, 2]])
    dst_row0, counts_local, offsets_local, src_rank, origin_byte, used = exchange.fused_layout(
        C, rank=1, cap_rows=16, row_bytes=8)  # fmt: skip
    assert counts_local.tolist() == [2, 3] and offsets_local.tolist() == [0, 2]  # rank 1 owns experts 2 and 3
    assert used.tolist() == [5]
    # on the owner, experts follow each other and rank 0's rows of an expert precede mine
    assert dst_row0.tolist() == [3, 4, 2, 3]
    assert src_rank[:5].tolist() == [0, 0, 0, 1, 1]
    assert origin_byte[:5].tolist() == [3 * 8, 4 * 8, 5 * 8, 5 * 8, 6 * 8]


@pytest.mark.parametrize("cap", [0, 1, 3, 4, 5, 9])
def test_fused_layout_stops_at_the_receive_capacity(cap):
    """More rows routed to a rank than its receive buffer holds: the counts handed to the
    experts stop at the capacity (offsets + counts never pass it), the senders' placement is
    unchanged (they drop what lands beyond it), and the rows in use are the capacity."""
    from fastmoe_b200 import exchange

    C = torch.tensor([[3, 0, 2, 1], [1, 4, 0, 2]])  # rank 0 receives 3+1+0+4 = 8 rows, rank 1 receives 5
    for rank, received in ((0, [4, 4]), (1, [2, 3])):
        dst_row0, counts, offsets, _, _, used = exchange.fused_layout(C, rank, cap, 8)
        full = exchange.fused_layout(C, rank, 64, 8)
        assert dst_row0.tolist() == full[0].tolist()
        assert bool(((offsets + counts) <= cap).all()) and bool((counts >= 0).all())
        assert int(used) == min(sum(received), cap) == int(counts.sum())
        first = 0
        for e, n in enumerate(received):  # what fits of each expert, in expert order
            assert int(counts[e]) == max(0, min(n, cap - first))
            first += n


def test_swiglu_expert_container_behaves_like_a_module_list():
    from fastmoe_b200.models.tiny_model import GroupedSwiGLUExperts

    ex = GroupedSwiGLUExperts(3, 8, 4)
    assert len(ex) == 3 and len(list(ex)) == 3 and ex.w_gate_up.shape == (3, 8, 8) and ex.w_down.shape == (3, 8, 4)
    x = torch.randn(5, 8)
    h = x @ ex.w_gate_up[1].t()
    want = (torch.nn.functional.silu(h[:, :4]) * h[:, 4:]) @ ex.w_down[1].t()
    assert torch.allclose(ex[1](x), want)


def test_expert_groups_cover_the_local_experts_with_a_small_first_group():
    """Group boundaries of the fused exchange's overlap: contiguous, non-empty, covering every
    local expert once; the first group (whose transfer nothing hides) is about half an even share."""
    from fastmoe_b200.ep_fused import FusedExpertParallel

    for el, groups in ((64, 4), (32, 4), (128, 4), (4, 4), (8, 4), (8, 2), (1, 1), (3, 2), (256, 1), (5, 5)):
        b = FusedExpertParallel._group_bounds(el, groups)
        assert b[0] == 0 and b[-1] == el and len(b) == groups + 1
        assert all(b[i] < b[i + 1] for i in range(groups))
        if groups > 1 and el >= 4 * groups:
            assert b[1] - b[0] <= (el // groups + 1) // 2 + 1 <= b[2] - b[1]
    assert FusedExpertParallel._group_bounds(64, 4) == [0, 8, 26, 45, 64]


@pytest.mark.parametrize("world,el,seed", [(1, 1, 0), (1, 5, 1), (2, 3, 2), (4, 2, 3), (8, 4, 4), (3, 7, 5)])
def test_fused_layout_against_a_row_by_row_simulation_of_the_exchange(world, el, seed):
    """The placement arithmetic of the fused exchange, held against the exchange done one row at a
    time in plain Python: every rank's rows (expert-major, as the index builder leaves them) are
    appended to the owner's receive list in (local expert, source rank) order."""
    from fastmoe_b200 import exchange

    E, row_bytes = world * el, 16
    gen = torch.Generator().manual_seed(seed)
    C = torch.randint(0, 6, (world, E), generator=gen)
    C[torch.rand(world, E, generator=gen) < 0.3] = 0  # experts that a rank sends nothing to
    starts = torch.cumsum(C, 1) - C  # first sorted slot of expert e on rank s
    received = {d: [] for d in range(world)}  # (source rank, source slot, local expert) per receive row
    first_row = {}  # (source rank, global expert) -> row on the owner where that source's rows begin
    for d in range(world):
        for le in range(el):
            g = d * el + le
            for s in range(world):
                first_row[(s, g)] = len(received[d])
                received[d] += [(s, int(starts[s, g]) + i, le) for i in range(int(C[s, g]))]
    for rank in range(world):
        total = len(received[rank])
        for cap in (total + 3, max(total - 2, 0)):
            dst_row0, counts, offsets, src_rank, origin_byte, used = exchange.fused_layout(C, rank, cap, row_bytes)
            assert dst_row0.tolist() == [first_row[(rank, g)] for g in range(E)]
            kept = received[rank][:cap]
            assert int(used) == len(kept)
            assert counts.tolist() == [sum(1 for r in kept if r[2] == le) for le in range(el)]
            assert offsets.tolist() == [min(sum(1 for r in received[rank] if r[2] < le), cap) for le in range(el)]
            assert src_rank[: len(kept)].tolist() == [r[0] for r in kept]
            assert origin_byte[: len(kept)].tolist() == [r[1] * row_bytes for r in kept]
