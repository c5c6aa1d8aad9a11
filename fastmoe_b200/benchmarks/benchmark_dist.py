"""Expert-parallel benchmark driver with the entry points of polkadot21/fastmoe
(src/fastmoe/benchmarks/benchmark_dist.py): one process per GPU over NCCL, a 2-layer
`TinyModel` in bf16 at the GIGACHAT_10B preset, forward + backward, STANDARD blocks against
the FAST pipelined blocks. Rank 0 prints the result as one JSON line.

    python -m fastmoe_b200.benchmarks.benchmark_dist             # spawns one worker per visible GPU
    torchrun --nproc-per-node N -m fastmoe_b200.benchmarks.benchmark_dist
"""

from __future__ import annotations

import json
import logging
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.profiler import ProfilerActivity, profile, record_function

from ..config import MoEScale, MoESetup, get_config
from ..consts import MoEImplementation
from ..models.tiny_model import TinyModel

log = logging.getLogger("fastmoe_b200.bench")


def setup():
    """Joins the NCCL process group described by the environment and selects this rank's GPU."""
    local_rank = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", 0)))
    torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", init_method="env://", device_id=torch.device("cuda", local_rank))


def cleanup():
    if dist.is_initialized():
        dist.destroy_process_group()


def benchmark_step(model, x, desc, profile_trace=False, steps=10, warmup=5) -> tuple[float, float]:
    """(ms per forward+backward, peak MiB) over `steps` iterations after `warmup` forwards
    (benchmark_dist.py:36-68). With `profile_trace` the iterations run under the torch profiler
    instead, a trace is written to ./logs/<desc>, and (0.0, 0.0) is returned."""
    for _ in range(warmup):
        model(x)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()

    def iteration():
        model(x).mean().backward()

    if profile_trace:
        path = os.path.join(".", "logs", desc)
        os.makedirs(path, exist_ok=True)
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True,
                     on_trace_ready=torch.profiler.tensorboard_trace_handler(path)) as prof:  # fmt: skip
            for i in range(steps):
                with record_function(f"Model Step: {i}"):
                    iteration()
                prof.step()
        return 0.0, 0.0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        iteration()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps, torch.cuda.max_memory_allocated() / 2**20


def _build(cfg: MoESetup, implementation, device, streams=(None, None)):
    return TinyModel(
        in_dim=cfg.hidden_dim, dim=cfg.hidden_dim, n_heads=cfg.n_heads, ff_dim=cfg.ff_dim,
        n_layers=cfg.n_layers, num_experts=cfg.num_experts, top_k=cfg.top_k, implementation=implementation,
        stream0=streams[0], stream1=streams[1], comm_balance_factor=cfg.comm_balance_factor, use_moe=True,
    ).to(device).to(torch.bfloat16)  # fmt: skip


def _worker_entrypoint(cfg: MoESetup | None = None, profile_trace: bool = False):
    setup()
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = cfg or get_config(MoEScale.GIGACHAT_10B)
    device = torch.device("cuda", torch.cuda.current_device())
    if rank == 0:
        logging.basicConfig(level=logging.INFO, format="%(asctime)s | %(levelname)-7s | %(message)s")
        log.info("%d GPUs | hidden %d | batch %d x %d tokens | %d layers | %d experts top-%d", world,
                 cfg.hidden_dim, cfg.batch_size, cfg.seq_len, cfg.n_layers, cfg.num_experts, cfg.top_k)  # fmt: skip
    torch.manual_seed(100 + rank)
    x = torch.randn(cfg.batch_size, cfg.seq_len, cfg.hidden_dim, device=device, dtype=torch.bfloat16,
                    requires_grad=True)  # fmt: skip

    torch.manual_seed(0)
    model = _build(cfg, MoEImplementation.STANDARD, device)
    ms_std, mem_std = benchmark_step(model, x, "standard_moe_timing")
    if profile_trace:
        benchmark_step(model, x, "standard_moe", profile_trace=True)
    del model
    torch.cuda.empty_cache()

    streams = (torch.cuda.Stream(device=device, priority=-1), torch.cuda.Stream(device=device, priority=-1))
    torch.manual_seed(0)
    model = _build(cfg, MoEImplementation.FAST, device, streams)
    ms_fast, mem_fast = benchmark_step(model, x, "fast_moe_timing")
    if profile_trace:
        benchmark_step(model, x, "fast_moe", profile_trace=True)
    del model

    # the slowest rank sets the pace
    times = torch.tensor([ms_std, ms_fast, mem_std, mem_fast], dtype=torch.float64, device=device)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    report = None
    if rank == 0:
        ms_std, ms_fast, mem_std, mem_fast = times.tolist()
        tokens = cfg.batch_size * cfg.seq_len * world
        report = {
            "scale": cfg.scale.value, "n_gpus": world, "dtype": "bf16", "tokens_per_step": tokens,
            "standard_ms": ms_std, "pipelined_ms": ms_fast, "speedup": ms_std / ms_fast,
            "standard_tokens_per_s": tokens / ms_std * 1e3, "pipelined_tokens_per_s": tokens / ms_fast * 1e3,
            "standard_peak_mib": mem_std, "pipelined_peak_mib": mem_fast,
        }  # fmt: skip
        print(json.dumps(report), flush=True)
    cleanup()
    return report


def _spawn_worker(rank, world_size, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world_size), LOCAL_RANK=str(rank))  # fmt: skip
    _worker_entrypoint()


def run_benchmark():
    """Under a launcher (RANK and WORLD_SIZE set) runs this rank; otherwise spawns one worker per
    visible GPU (benchmark_dist.py:182-190)."""
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return _worker_entrypoint()
    world_size = torch.cuda.device_count()
    if world_size < 1:
        log.warning("no CUDA device: nothing to run")
        return None
    if world_size < 2:
        log.warning("one GPU: the exchange is a no-op, only the compute path is timed")
    mp.spawn(_spawn_worker, args=(world_size, int(os.environ.get("MASTER_PORT", 12355))), nprocs=world_size, join=True)
    return None


if __name__ == "__main__":
    run_benchmark()
