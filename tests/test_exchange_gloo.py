"""Expert-parallel exchange bookkeeping on CPU ranks over gloo (world size 2 and 4):
counts, uneven all-to-all with gradients, regrouping by expert and the return trip.
Ground truth is the single-rank computation over all experts."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastmoe_b200 import exchange
from fastmoe_b200.workloads import routing_uniform, sort_routing


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_fn(rows, expert_id):
    """A stand-in expert with a distinct, non-linear action per expert."""
    return torch.tanh(rows * (0.5 + 0.1 * expert_id)) * (1.0 + expert_id)


def _worker(rank, world, port, E, K, T, D, fail_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        e_local = E // world
        torch.manual_seed(100 + rank)
        x = torch.randn(T, D, dtype=torch.float64, requires_grad=True)
        idx, w = routing_uniform(T, E, K, seed=100 + rank)
        rev, sw, counts = sort_routing(idx, w.double(), E)
        permuted = x[rev]
        by_rank = counts.view(world, e_local)
        rank_counts = by_rank.sum(1)

        recv_counts, nested, send_list, recv_list = exchange.exchange_counts(by_rank, rank_counts)
        assert send_list == rank_counts.tolist() and recv_list == [sum(r) for r in nested]
        assert recv_counts.tolist() == nested
        recv = exchange.all_to_all_rows(permuted, recv_list, send_list)
        to_em, to_rm, tokens = exchange.regroup_indices(nested, recv.device)
        assert tokens == [sum(nested[s][e] for s in range(world)) for e in range(e_local)]
        assert torch.equal(to_em[to_rm], torch.arange(recv.shape[0]))
        grouped = recv.index_select(0, to_em)
        outs = [
            _expert_fn(chunk, rank * e_local + e) for e, chunk in enumerate(grouped.split(tokens))
        ]
        back = exchange.all_to_all_rows(torch.cat(outs).index_select(0, to_rm), send_list, recv_list)
        out = torch.zeros(T, D, dtype=torch.float64).index_add(0, rev, back * sw[:, None])
        coeff = torch.randn(T, D, dtype=torch.float64)
        (out * coeff).sum().backward()

        # single-rank ground truth over all experts
        x2 = x.detach().clone().requires_grad_(True)
        p2 = x2[rev]
        o2 = torch.cat([_expert_fn(c, e) for e, c in enumerate(p2.split(counts.tolist()))])
        out2 = torch.zeros(T, D, dtype=torch.float64).index_add(0, rev, o2 * sw[:, None])
        (out2 * coeff).sum().backward()
        assert torch.allclose(out, out2, rtol=1e-12, atol=1e-12)
        assert torch.allclose(x.grad, x2.grad, rtol=1e-12, atol=1e-12)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure in the parent
        import traceback

        fail_q.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


@pytest.mark.parametrize("world,E", [(2, 2), (2, 8), (4, 8)])
def test_exchange_matches_single_rank(world, E):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, _free_port_cached(world, E), E, 3 if E > 2 else 2, 24, 5, q))
             for r in range(world)]  # fmt: skip
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


_ports = {}


def _free_port_cached(world, E):
    key = (world, E)
    if key not in _ports:
        _ports[key] = _free_port()
    return _ports[key]


def test_regroup_indices_small():
    # 2 source ranks, 3 local experts; arrival order is (source, expert)
    nested = [[2, 0, 1], [1, 2, 0]]
    to_em, to_rm, tokens = exchange.regroup_indices(nested, "cpu")
    assert tokens == [3, 2, 1]
    # rank-major rows: s0e0 s0e0 s0e2 | s1e0 s1e1 s1e1 -> expert-major: e0(s0,s0,s1) e1(s1,s1) e2(s0)
    assert to_em.tolist() == [0, 1, 3, 4, 5, 2]
    assert np.array_equal(to_rm.numpy(), np.argsort(to_em.numpy()))
    empty = exchange.regroup_indices([[0, 0], [0, 0]], "cpu")
    assert empty[0].numel() == 0 and empty[2] == [0, 0]


@pytest.mark.parametrize("world,E,K,cap_share", [(2, 8, 2, 1.0), (4, 8, 3, 1.0), (4, 16, 4, 1.0),
                                                 (2, 8, 2, 0.4), (4, 16, 4, 0.2)])  # fmt: skip
def test_fused_layout_routes_every_row_there_and_back(world, E, K, cap_share):
    """The placement arithmetic of the peer-store exchange, emulated with plain tensors: every
    rank's rows reach the right expert's owner in expert-major order, and the return addresses
    bring each result back to the slot it came from. With a receive buffer smaller than the
    rows routed to a rank (cap_share < 1) the copies that do not fit are dropped by their
    senders, the experts see only rows that arrived, and a dropped copy's result is zero."""
    T, D = 40, 3
    el = E // world
    cap = int(world * T * K * cap_share)
    torch.manual_seed(world * 100 + E)
    ranks = []
    for r in range(world):
        x = torch.randn(T, D)
        idx, w = routing_uniform(T, E, K, seed=10 + r)
        rev, _, counts = sort_routing(idx, w, E)
        order = torch.argsort(idx.reshape(-1), stable=True)
        slot_of = torch.empty(T * K, dtype=torch.int64)
        slot_of[order] = torch.arange(T * K)
        ranks.append(dict(x=x, idx=idx, rev=rev, counts=counts, offsets=torch.cumsum(counts, 0) - counts, slot_of=slot_of))
    C = torch.stack([r["counts"] for r in ranks])
    recv = [torch.full((cap, D), float("nan")) for _ in range(world)]
    ret = [torch.full((T * K, D), float("nan")) for _ in range(world)]
    kept = [torch.ones(T * K, dtype=torch.bool) for _ in range(world)]
    layouts = [exchange.fused_layout(C, r, cap, D) for r in range(world)]  # row_bytes = D "bytes" per row
    for r, rk in enumerate(ranks):  # dispatch: what the permute kernel computes per routed copy
        dst_row0 = layouts[r][0]
        for t in range(T):
            for k in range(K):
                e = int(rk["idx"][t, k])
                slot = int(rk["slot_of"][t * K + k])
                row = int(dst_row0[e]) + slot - int(rk["offsets"][e])
                if row >= cap:  # no room: dropped, and the owner's return row is cleared
                    ret[r][slot] = 0.0
                    kept[r][slot] = False
                    continue
                assert torch.isnan(recv[e // el][row]).all()  # nobody else writes this row
                recv[e // el][row] = rk["x"][t]
    for d in range(world):  # experts: scale by (global expert id + 1), then the return stores
        _, counts_local, offsets_local, src_rank, origin_byte, used = layouts[d]
        routed_here = int(C[:, d * el : (d + 1) * el].sum())
        assert int(counts_local.sum()) == min(routed_here, cap) == int(used)
        assert bool(((offsets_local + counts_local) <= cap).all())
        for e in range(el):
            for i in range(int(offsets_local[e]), int(offsets_local[e] + counts_local[e])):
                assert not torch.isnan(recv[d][i]).any()
                ret[int(src_rank[i])][int(origin_byte[i]) // D] = recv[d][i] * (d * el + e + 1)
    assert cap_share >= 1.0 or not all(bool(k.all()) for k in kept)  # the small buffers did overflow
    for r, rk in enumerate(ranks):
        expert_of_slot = torch.repeat_interleave(torch.arange(E), rk["counts"])
        want = rk["x"][rk["rev"]] * (expert_of_slot + 1).float()[:, None] * kept[r][:, None]
        assert torch.equal(ret[r], want)


def _static_worker(rank, world, port, factor, fail_q):
    """The host-known uniform exchange of the module: every row reaches the rank whose block it
    sits in, padding never shows, and the return trip undoes the dispatch, gradients included."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from fastmoe_b200 import consts
        from fastmoe_b200.models.tiny_model import MoEFeedForward

        D, real = 6, 5
        moe = MoEFeedForward(D, 8, 2 * world, 2, consts.MoEImplementation.STANDARD)
        rows = (torch.arange(world * real * D, dtype=torch.float64).view(world * real, D) + 1000 * rank)
        rows.requires_grad_(True)
        splits = [real * factor] * world
        recv, s_in, s_out = moe.dispatch_exchange_static(rows, splits, real)
        assert s_in is splits and s_out is splits and recv.shape == (world * real, D)
        for src in range(world):  # block `rank` of every source, in source order
            want = torch.arange(world * real * D, dtype=torch.float64).view(world, real, D)[rank] + 1000 * src
            assert torch.equal(recv[src * real : (src + 1) * real].detach(), want)
        shares = moe.compute_experts_static(recv.detach().float())
        assert shares.shape == (world * real, D)
        back = moe.combine_exchange_static(recv * 2.0, splits, real)
        assert torch.equal(back.detach(), rows.detach() * 2.0)
        coeff = torch.randn(world * real, D, dtype=torch.float64)
        (back * coeff).sum().backward()
        assert torch.equal(rows.grad, coeff * 2.0)
        with pytest.raises(ValueError):
            moe.dispatch_exchange_static(rows.detach(), [real, real + 1][:world] + [real] * (world - 2), real)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:
        import traceback

        fail_q.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


@pytest.mark.parametrize("factor", [1, 3])
def test_static_exchange_round_trip(factor):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_static_worker, args=(r, world, port, factor, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


def test_static_exchange_single_rank_is_identity():
    from fastmoe_b200 import consts
    from fastmoe_b200.models.tiny_model import MoEFeedForward

    moe = MoEFeedForward(4, 8, 3, 2, consts.MoEImplementation.STANDARD)
    rows = torch.randn(7, 4)
    got, a, b = moe.dispatch_exchange_static(rows, [14], 7)
    assert got is rows and a == [14] and b == [14]
    assert moe.combine_exchange_static(rows, [14], 7) is rows
    out = moe.compute_experts_static(rows)  # shares of 3, 3, 1 rows
    want = torch.cat([moe.experts[0](rows[:3]), moe.experts[1](rows[3:6]), moe.experts[2](rows[6:])])
    assert torch.equal(out, want)


def _bad_split_worker(rank, world, port, fail_q):
    """A rank whose send counts do not match its rows learns so on the host, before any
    collective is enqueued: no rank is left waiting inside a mismatched all-to-all."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        rows = torch.randn(6, 3)
        for out_splits, in_splits in (([3, 3], [3, 4]), ([3, 3], [3]), ([3, -1], [3, 3])):
            with pytest.raises(ValueError):
                exchange.all_to_all_rows(rows, out_splits, in_splits)
        got = exchange.all_to_all_rows(rows, [3, 3], [3, 3])  # the group is still usable afterwards
        assert got.shape == (6, 3)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:
        import traceback

        fail_q.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


def test_mismatched_splits_raise_before_the_collective():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_bad_split_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)
