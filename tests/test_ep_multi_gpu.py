"""Expert-parallel MoE layer on 2, 4 and 8 GPUs over NCCL against the single-rank computation
over all experts (the ground truth: the reference's own multi-rank path is wrong for more than
one expert per rank and carries no gradients). A world size is skipped on boxes with fewer
GPUs; the pieces that need no second GPU (the fused path in a one-rank group, the placement
kernel, the barrier's give-up path, receive-buffer overflow) run everywhere."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_weights(e, D, FF, device):
    g = torch.Generator(device=device).manual_seed(500 + e)
    wgu = torch.empty(2 * FF, D, device=device).normal_(0, 0.05, generator=g).bfloat16()
    wd = torch.empty(D, FF, device=device).normal_(0, 0.05, generator=g).bfloat16()
    return wgu, wd


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from fastmoe_b200.consts import MoEImplementation
        from fastmoe_b200.kernels import ops, routing
        from fastmoe_b200.models.tiny_model import MoEFeedForward, pipelined_moe_forward

        T, D, FF, E, K = 384, 256, 256, 8, 2
        moe = MoEFeedForward(D, FF, E, K, MoEImplementation.FAST, expert_type="swiglu").to(dev).bfloat16()
        assert moe.world_size == world and moe.num_local_experts == E // world
        g = torch.Generator(device=dev).manual_seed(7)
        with torch.no_grad():
            moe.router.weight.copy_(torch.empty(E, D, device=dev).normal_(0, 0.3, generator=g))
            for e in range(moe.num_local_experts):
                wgu, wd = _expert_weights(rank * moe.num_local_experts + e, D, FF, dev)
                moe.experts.w_gate_up[e].copy_(wgu)
                moe.experts.w_down[e].copy_(wd)
        gx = torch.Generator(device=dev).manual_seed(100 + rank)
        x = torch.randn(1, T, D, generator=gx, device=dev).bfloat16().requires_grad_(True)
        out = moe(x)
        coeff = torch.randn(1, T, D, generator=gx, device=dev)
        (out.float() * coeff).sum().backward()
        assert ops.read_status() == 0

        # ground truth on this rank's tokens with ALL experts, fp32 math on the same bf16 values
        xf = x.detach().float().view(T, D).requires_grad_(True)
        logits = moe.router(x.detach().view(T, D))
        _, idx = routing.route_topk(logits, K, w_dtype=torch.bfloat16)  # the layer's routing decision
        # gate weights recomputed in fp32 with autograd, so the router path carries gradient too
        w = torch.softmax(torch.gather(xf @ moe.router.weight.detach().float().t(), 1, idx), dim=-1)
        ref = torch.zeros(T, D, device=dev)
        for e in range(E):
            wgu, wd = _expert_weights(e, D, FF, dev)
            for k in range(K):
                m = idx[:, k] == e
                h = xf[m] @ wgu.float().t()
                a = torch.nn.functional.silu(h[:, :FF]) * h[:, FF:]
                ref = ref.index_add(0, m.nonzero().view(-1), (a @ wd.float().t()) * w[m, k].float()[:, None])
        (ref * coeff.view(T, D)).sum().backward()
        err = float((out.float().view(T, D) - ref).abs().max() / ref.abs().max())
        assert err <= 2e-2, f"forward rel err {err}"
        # gradient w.r.t. the tokens: through experts living on both ranks and through the router
        gerr = float((x.grad.float().view(T, D) - xf.grad).abs().max() / xf.grad.abs().max())
        assert gerr <= 5e-2, f"grad rel err {gerr}"
        assert moe.experts.w_down.grad is not None and float(moe.experts.w_down.grad.abs().max()) > 0

        # the pipelined schedule gives the same result as the plain forward
        chunks = [c.contiguous() for c in x.detach().view(4, T // 4, D).unsqueeze(1)]
        streams = [torch.cuda.Stream(device=dev) for _ in chunks]
        for s in streams:
            s.wait_stream(torch.cuda.current_stream())
        with torch.no_grad():
            outs = pipelined_moe_forward(moe, chunks, streams)
        torch.cuda.synchronize()
        piped = torch.cat(outs, 1).view(T, D)
        perr = float((piped.float() - ref.detach()).abs().max() / ref.abs().max())
        assert perr <= 2e-2, f"pipelined rel err {perr}"
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:
        import traceback

        q.put(f"rank {rank}: {exc}\n{traceback.format_exc()}")
        raise


def _fused_worker(rank, world, port, q):
    failure = None
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                          TORCH_SYMM_MEM_DISABLE_MULTICAST="1")  # fmt: skip
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from fastmoe_b200.consts import MoEImplementation
        from fastmoe_b200.ep_fused import FusedExpertParallel
        from fastmoe_b200.kernels import ops
        from fastmoe_b200.models.tiny_model import MoEFeedForward

        T, D, FF, E, K = 640, 256, 256, 8, 2
        moe = MoEFeedForward(D, FF, E, K, MoEImplementation.FAST, expert_type="swiglu").to(dev).bfloat16()
        g = torch.Generator(device=dev).manual_seed(7)
        with torch.no_grad():
            moe.router.weight.copy_(torch.empty(E, D, device=dev).normal_(0, 0.3, generator=g))
            for e in range(moe.num_local_experts):
                wgu, wd = _expert_weights(rank * moe.num_local_experts + e, D, FF, dev)
                moe.experts.w_gate_up[e].copy_(wgu)
                moe.experts.w_down[e].copy_(wd)
        fused = FusedExpertParallel(moe, max_tokens=T)
        results = []
        for call in range(3):  # repeated calls reuse the same symmetric buffers
            gx = torch.Generator(device=dev).manual_seed(100 + rank + 10 * call)
            n = T if call != 1 else T // 2  # a smaller batch in between
            x = torch.randn(1, n, D, generator=gx, device=dev).bfloat16()
            with torch.no_grad():
                results.append((fused(x), moe(x)))
        torch.cuda.synchronize()
        # training call: forward and backward over peer stores against the NCCL path's autograd
        xg = torch.randn(1, T, D, generator=torch.Generator(device=dev).manual_seed(900 + rank), device=dev).bfloat16()
        coeff = torch.randn(1, T, D, generator=torch.Generator(device=dev).manual_seed(901 + rank), device=dev)
        grads = []
        for path in (fused.forward_with_grad, moe):
            for prm in moe.parameters():
                prm.grad = None
            xi = xg.clone().requires_grad_(True)
            yo = path(xi)
            (yo.float() * coeff).sum().backward()
            grads.append((yo.detach(), xi.grad, moe.router.weight.grad.clone(), moe.experts.w_gate_up.grad.clone(),
                          moe.experts.w_down.grad.clone()))  # fmt: skip
        torch.cuda.synchronize()
        grad_errs = []
        for got, want in zip(*grads):
            scale = float(want.float().abs().max())
            grad_errs.append(float((got.float() - want.float()).abs().max()) / max(scale, 1e-30))

        # the buffers keep ONE forward's rows: the backward of an overtaken forward must refuse
        y_old = fused.forward_with_grad(xg.clone().requires_grad_(True))
        y_new = fused.forward_with_grad(xg.clone().requires_grad_(True))
        try:
            y_old.float().sum().backward()
            stale_refused = False
        except RuntimeError as exc:
            stale_refused = "another forward" in str(exc)
        y_new.float().sum().backward()  # the latest forward's backward still runs
        torch.cuda.synchronize()

        # the module-level switch routes every forward through the fused path, the training
        # call included; a call it cannot serve raises instead of taking another path
        moe.enable_fused_exchange(max_tokens=T)
        with torch.no_grad():
            via_module = moe(x)
        results.append((via_module, results[-1][1]))
        for prm in moe.parameters():
            prm.grad = None
        xi = xg.clone().requires_grad_(True)
        ym = moe(xi)
        (ym.float() * coeff).sum().backward()
        module_grad_errs = [float((got.float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-30)
                            for got, want in zip((ym.detach(), xi.grad, moe.experts.w_down.grad),
                                                 (grads[0][0], grads[0][1], grads[0][4]))]  # fmt: skip
        try:
            moe(torch.zeros(1, T + 8, D, device=dev, dtype=torch.bfloat16))
            too_big_refused = False
        except ValueError:
            too_big_refused = True
        moe.disable_fused_exchange()
        fused.check_status()  # raises if a row was dropped or a wait ran out
        torch.cuda.synchronize()
        status = ops.read_status()
        dist.barrier()  # every rank has finished its GPU work before anyone may fail and leave
        assert status == 0
        assert stale_refused, "a backward ran on exchange buffers that a later forward had overwritten"
        assert too_big_refused, "a call beyond max_tokens did not raise"
        assert max(module_grad_errs) == 0.0, module_grad_errs  # the module's training call IS forward_with_grad
        # out, d x, d router, d w_gate_up, d w_down: same kernels on both paths, bf16 rounding at most
        assert max(grad_errs) <= 2e-2, grad_errs
        for got, want in results:
            # same kernels, same row order inside every expert: the two paths must agree exactly
            assert torch.equal(got, want), float((got.float() - want.float()).abs().max())
    except Exception as exc:
        import traceback

        failure = f"rank {rank}: {exc}\n{traceback.format_exc()}"
    finally:
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception:
            pass
    if failure:
        q.put(failure)
        raise SystemExit(1)


def test_fused_exchange_single_rank_group():
    """The same fused path in a process group of ONE rank (its "peer" stores go to its own
    symmetric buffers): runs on a single-GPU box and covers the forward, the backward and the
    buffer reuse without a second GPU."""
    _run_ranks(_fused_worker, 1)


def _run_ranks(target, world, extra=()):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q, *extra)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    for p in procs:
        if p.is_alive():
            p.kill()
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchange_matches_nccl_path(world):
    """Dispatch by peer stores + return trip in the GEMM epilogue against the NCCL all-to-all path."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_fused_worker, world)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_layer_matches_single_rank_ground_truth(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker, world)


def _overflow_worker(rank, world, port, q):
    """More rows routed to a rank than its receive buffer holds (capacity_factor 0.5 in a group
    of one rank: the upper half of the sorted rows does not fit). Nothing faults: the copies
    that do not fit are dropped, the status word says so on sender and receiver, the dropped
    copies add exactly zero, gradients included, and the next call with room is clean."""
    failure = None
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                          TORCH_SYMM_MEM_DISABLE_MULTICAST="1")  # fmt: skip
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from fastmoe_b200.consts import MoEImplementation
        from fastmoe_b200.ep_fused import FusedExpertParallel
        from fastmoe_b200.kernels import experts, ops, routing
        from fastmoe_b200.kernels.ops import routed_combine
        from fastmoe_b200.models.tiny_model import MoEFeedForward

        T, D, FF, E, K = 512, 256, 256, 8, 2
        moe = MoEFeedForward(D, FF, E, K, MoEImplementation.FAST, expert_type="swiglu").to(dev).bfloat16()
        g = torch.Generator(device=dev).manual_seed(7)
        with torch.no_grad():
            moe.router.weight.copy_(torch.empty(E, D, device=dev).normal_(0, 0.3, generator=g))
            for e in range(E):
                wgu, wd = _expert_weights(e, D, FF, dev)
                moe.experts.w_gate_up[e].copy_(wgu)
                moe.experts.w_down[e].copy_(wd)
        small = FusedExpertParallel(moe, max_tokens=T, capacity_factor=0.5, expert_groups=2)
        cap = small.cap_rows
        assert cap == T * K // 2
        # poison what an earlier call could have left in the buffers: a dropped copy must not read it
        small._ret.fill_(float("nan"))
        small._recv.fill_(float("nan"))
        x = torch.randn(1, T, D, generator=g, device=dev).bfloat16()

        def expected(xin):
            """The layer with the gate weight of every copy that does not fit set to zero. In a
            one-rank group a copy's receive row is its sorted slot, so slots >= cap are dropped."""
            xf = xin.view(T, D)
            topk_w, topk_idx = routing.route_topk(moe.router(xf), K, w_dtype=xf.dtype)
            ix = routing.build_index(topk_idx, topk_w, E, 1)
            rows = routing.permute_rows(xf, ix.slot_of, K)
            y = experts.grouped_swiglu_ffn(rows, moe.experts.w_gate_up, moe.experts.w_down, ix.offsets, ix.counts,
                                           covers_all_rows=True)  # fmt: skip
            keep = (torch.arange(T * K, device=dev) < cap).to(y.dtype)
            return routed_combine(y * keep[:, None], ix.slot_of, ix.sorted_w * keep, K).view(1, T, D)

        with torch.no_grad():
            got = small(x)
            want = expected(x)
        torch.cuda.synchronize()
        status_after_overflow = ops.read_status()
        forward_ok = torch.equal(got, want) and bool(torch.isfinite(got.float()).all())

        # training call: dropped copies carry no gradient, everything stays finite
        coeff = torch.randn(1, T, D, generator=g, device=dev)
        grads = []
        for path in (small.forward_with_grad, expected):
            for prm in moe.parameters():
                prm.grad = None
            xi = x.clone().requires_grad_(True)
            (path(xi).float() * coeff).sum().backward()
            grads.append((xi.grad, moe.experts.w_down.grad.clone(), moe.experts.w_gate_up.grad.clone(),
                          moe.router.weight.grad.clone()))  # fmt: skip
        torch.cuda.synchronize()
        status_after_training = ops.read_status()
        grad_errs = []
        for a, b in zip(*grads):
            assert bool(torch.isfinite(a.float()).all())
            grad_errs.append(float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-30))
        try:
            small(x)
            small.check_status()
            check_raised = False
        except RuntimeError as exc:
            check_raised = "dropped" in str(exc)

        # the same buffers, half the tokens: everything fits, the call is clean and exact
        with torch.no_grad():
            half = x[:, : T // 2].contiguous()
            clean, ref = small(half), moe(half)
        torch.cuda.synchronize()
        status_clean = ops.read_status()
        dist.barrier()
        assert status_after_overflow & 1, status_after_overflow
        assert status_after_training & 1, status_after_training
        assert forward_ok, float((got.float() - want.float()).abs().max())
        assert max(grad_errs) <= 2e-2, grad_errs
        assert check_raised, "check_status() did not report the dropped rows"
        assert status_clean == 0 and torch.equal(clean, ref)
    except Exception as exc:
        import traceback

        failure = f"rank {rank}: {exc}\n{traceback.format_exc()}"
    finally:
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception:
            pass
    if failure:
        q.put(failure)
        raise SystemExit(1)


def test_receive_buffer_overflow_drops_rows_cleanly():
    _run_ranks(_overflow_worker, 1)


@pytest.mark.parametrize("world,E,rank,cap", [(1, 8, 0, 4096), (2, 8, 1, 1024), (4, 64, 2, 4096), (8, 256, 5, 2048),
                                              (8, 256, 0, 300), (4, 64, 3, 0)])  # fmt: skip
def test_layout_kernel_matches_the_tensor_statement(world, E, rank, cap):
    """`fmoe_ep_layout` (two small launches) against `exchange.fused_layout` (the same arithmetic
    as tensor operations) on random counts, with and without overflow of the receive buffer."""
    from fastmoe_b200 import exchange
    from fastmoe_b200.kernels import ops
    from fastmoe_b200.kernels.ops import _status_word, _stream_ptr

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(world * 1000 + E + rank)
    C = torch.randint(0, 40, (world, E), generator=gen, device=dev, dtype=torch.int64)
    C[:, ::5] = 0  # experts nobody routes to
    el, row_bytes = E // world, 512
    bases = torch.arange(1, world + 1, device=dev, dtype=torch.int64) * (1 << 32)
    gbases = bases + (1 << 40)
    i64 = dict(dtype=torch.int64, device=dev)
    dst_row0, counts_local, offsets_local = torch.empty(E, **i64), torch.empty(el, **i64), torch.empty(el, **i64)
    used, ptrs, gptrs = torch.empty(1, **i64), torch.full((max(cap, 1),), -1, **i64), torch.full((max(cap, 1),), -1, **i64)
    scratch = torch.empty(2 * E, **i64)
    ops.read_status()
    ops._call("fmoe_ep_layout", 2, C.data_ptr(), world, E, rank, cap, row_bytes, bases.data_ptr(), gbases.data_ptr(),
              dst_row0.data_ptr(), counts_local.data_ptr(), offsets_local.data_ptr(), used.data_ptr(), ptrs.data_ptr(),
              gptrs.data_ptr(), scratch.data_ptr(), _status_word(dev).data_ptr(), _stream_ptr(dev))  # fmt: skip
    torch.cuda.synchronize()
    want = exchange.fused_layout(C, rank, cap, row_bytes)
    assert torch.equal(dst_row0, want[0]) and torch.equal(counts_local, want[1]) and torch.equal(offsets_local, want[2])
    assert torch.equal(used, want[5])
    n = int(used)
    want_ptrs = bases[want[3]] + want[4]
    assert torch.equal(ptrs[:n], want_ptrs[:n]) and torch.equal(gptrs[:n], want_ptrs[:n] + (1 << 40))
    assert bool((ptrs[n:cap] == 0).all()) and bool((gptrs[n:cap] == 0).all())
    overflowed = int(C[:, rank * el : (rank + 1) * el].sum()) > cap
    assert bool(ops.read_status() & 1) == overflowed


def test_peer_barrier_gives_up_on_a_peer_that_never_arrives():
    """Failure detection without a fault: a "peer" whose flag nothing ever sets. The wait runs
    out after its time limit, the status word gets the WAIT_TIMEOUT bit and the kernel returns;
    the context stays usable, and a barrier whose peers are all present passes at once."""
    from fastmoe_b200.kernels import ops
    from fastmoe_b200.kernels.ops import _status_word, _stream_ptr

    dev = torch.device("cuda")
    mine = torch.zeros(32, dtype=torch.int32, device=dev)
    absent = torch.zeros(32, dtype=torch.int32, device=dev)  # stands for a rank that never runs its barrier
    bases = torch.tensor([mine.data_ptr(), absent.data_ptr()], dtype=torch.int64, device=dev)
    ops.read_status()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ops._call("fmoe_peer_barrier", 1, bases.data_ptr(), 2, 0, 1, 50, _status_word(dev).data_ptr(), _stream_ptr(dev))
    t1.record()
    torch.cuda.synchronize()
    assert ops.read_status() & 8
    assert 40.0 <= t0.elapsed_time(t1) <= 2000.0  # gave up after about the 50 ms it was allowed
    assert int(absent[0]) == 1 and int(mine[0]) == 1  # it did announce itself to both
    # the same rank alone in its group: its own flag is the only one it waits for
    solo = torch.tensor([mine.data_ptr()], dtype=torch.int64, device=dev)
    ops._call("fmoe_peer_barrier", 1, solo.data_ptr(), 1, 0, 2, 50, _status_word(dev).data_ptr(), _stream_ptr(dev))
    torch.cuda.synchronize()
    assert ops.read_status() == 0 and int(mine[0]) == 2
