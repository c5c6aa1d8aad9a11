"""Expert-parallel MoE layer on 2 GPUs over NCCL against the single-rank computation over all
experts (the ground truth: the reference's own multi-rank path is wrong for more than one
expert per rank and carries no gradients). Skipped on boxes with fewer than 2 GPUs."""

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

        T, D, FF, E, K = 384, 256, 128, 8, 2
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

        T, D, FF, E, K = 640, 256, 128, 8, 2
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

        # the module-level switch routes gradient-free forwards through the same fused path
        moe.enable_fused_exchange(max_tokens=T)
        with torch.no_grad():
            via_module = moe(x)
        results.append((via_module, results[-1][1]))
        assert moe(x.requires_grad_(True)).requires_grad  # with gradients: the NCCL path, as before
        torch.cuda.synchronize()
        status = ops.read_status()
        dist.barrier()  # every rank has finished its GPU work before anyone may fail and leave
        assert status == 0
        assert stale_refused, "a backward ran on exchange buffers that a later forward had overwritten"
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
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    p = ctx.Process(target=_fused_worker, args=(0, 1, _free_port(), q))
    p.start()
    p.join(300)
    msgs = []
    while not q.empty():
        msgs.append(q.get())
    if p.is_alive():
        p.kill()
    assert not msgs, "\n".join(msgs)
    assert p.exitcode == 0


def test_fused_exchange_matches_nccl_path_on_two_gpus():
    """Dispatch by peer stores + return trip in the GEMM epilogue against the NCCL all-to-all path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_worker, args=(r, 2, port, q)) for r in range(2)]
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


def test_ep_layer_two_gpus_matches_single_rank_ground_truth():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
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
