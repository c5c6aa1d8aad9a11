"""Single-GPU benchmark driver with the entry points of polkadot21/fastmoe
(src/fastmoe/benchmarks/run_on_cloud.py): the combine microbenchmark (cat -> scale ->
index_add_ against the grouped pointer-table combine under CUDA-graph replay) and a short
mixed-precision training loop of `TinyModel`, STANDARD against FAST. `run_on_cloud()`
returns its results as a dict and prints them as one JSON line.

    python -m fastmoe_b200.benchmarks.run_on_cloud [debug|gigachat-10b|gigachat-700b] [--no-training]
"""

from __future__ import annotations

import gc
import json
import logging
import sys

import torch

from .. import consts
from ..config import MoEScale, MoESetup, get_config
from ..kernels.ops import grouped_weighted_scatter_add, prepare_grouped_metadata
from ..models.tiny_model import TinyModel

log = logging.getLogger("fastmoe_b200.bench")
MIB, GIB = 2**20, 2**30


def _standard_combine(expert_outputs, indices, weights, out_shape):
    rows = torch.cat(expert_outputs, dim=0) * weights.unsqueeze(-1)
    out = torch.zeros(out_shape, device=rows.device, dtype=rows.dtype)
    return out.index_add_(0, indices, rows)


def verify_correctness(expert_outputs, indices, weights, out_shape, tol=1e-4) -> float:
    """Largest absolute difference between the grouped combine and cat -> scale -> index_add_
    on the same inputs (run_on_cloud.py:13-32); logs a warning above `tol`."""
    want = _standard_combine(expert_outputs, indices, weights, out_shape)
    got = torch.zeros(out_shape, device=want.device, dtype=want.dtype)
    grouped_weighted_scatter_add(expert_outputs, indices, weights, out_shape, out=got)
    diff = float((want - got).abs().max()) if want.numel() else 0.0
    (log.warning if diff > tol else log.info)("combine check: max |difference| %.3e (tolerance %.0e)", diff, tol)
    return diff


def _timed(steps, body):
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        body()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / max(steps, 1), torch.cuda.max_memory_allocated() / MIB


def benchmark_standard(expert_outputs, indices, weights, out_shape, steps):
    """(ms per step, peak MiB) of cat -> scale -> zeros -> index_add_ (run_on_cloud.py:35-53)."""
    return _timed(steps, lambda: _standard_combine(expert_outputs, indices, weights, out_shape))


def benchmark_fastmoe_grouped(expert_outputs, indices, weights, out_shape, steps):
    """(ms per step, peak MiB) of the grouped combine with prebuilt metadata, captured once in
    a CUDA graph and replayed; the output is zeroed before every replay (run_on_cloud.py:56-96)."""
    device = expert_outputs[0].device
    out = torch.zeros(out_shape, device=device, dtype=expert_outputs[0].dtype)
    metadata = prepare_grouped_metadata(expert_outputs, device)

    def launch():
        grouped_weighted_scatter_add(expert_outputs, indices, weights, out_shape, out=out, metadata=metadata)

    launch()  # loads the library and warms the allocator outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    out.zero_()
    with torch.cuda.graph(graph):
        launch()

    def step():
        out.zero_()
        graph.replay()

    return _timed(steps, step)


def run_training_experiment(implementation, cfg: MoESetup, warmup=5):
    """(ms per step, peak GiB) of a bf16-autocast SGD loop on a 2-layer `TinyModel` with narrow
    experts (ff 256) and the preset's wide rows (run_on_cloud.py:99-192): forward, MSE loss,
    backward, gradient clipping, step."""
    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    device = torch.device("cuda")
    model = TinyModel(
        in_dim=cfg.hidden_dim, dim=cfg.hidden_dim, n_heads=16, ff_dim=256, n_layers=2,
        num_experts=cfg.num_experts, top_k=cfg.top_k, implementation=implementation,
        comm_balance_factor=cfg.comm_balance_factor, use_moe=True,
    ).to(device)  # fmt: skip
    optimizer = torch.optim.SGD(model.parameters(), lr=0.5)
    x = torch.randn(cfg.batch_size, cfg.seq_len, cfg.hidden_dim, device=device)
    target = x.clone()

    def step():
        with torch.amp.autocast("cuda", dtype=torch.bfloat16):
            loss = ((model(x) - target) ** 2).mean()
        loss.backward()
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        optimizer.step()
        optimizer.zero_grad()
        return loss, norm

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(cfg.active_steps):
        loss, norm = step()
        if i % 10 == 0 or i == cfg.active_steps - 1:
            log.info("step %03d/%d | loss %.4f | grad norm %.4f | %.2f GiB", i, cfg.active_steps,
                     float(loss), float(norm), torch.cuda.memory_allocated() / GIB)  # fmt: skip
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / max(cfg.active_steps, 1)
    peak = torch.cuda.max_memory_allocated() / GIB
    del model, optimizer, x, target
    return ms, peak


def run_on_cloud(scale: MoEScale = MoEScale.GIGACHAT_700B, training: bool = True, cfg: MoESetup | None = None):
    """Kernel microbenchmark, then the training comparison, at `scale` (run_on_cloud.py:195-273).
    Returns the report and prints it as one JSON line; without a GPU returns None."""
    logging.basicConfig(level=logging.INFO, format="%(asctime)s | %(levelname)-7s | %(message)s")
    cfg = cfg or get_config(scale)
    if not torch.cuda.is_available():
        log.warning("no CUDA device: nothing to run")
        return None
    device = torch.device("cuda")
    rows = cfg.total_tokens
    per_expert = rows // cfg.num_experts
    rows = per_expert * cfg.num_experts
    tokens = cfg.batch_size * cfg.seq_len
    experts = [torch.randn(per_expert, cfg.hidden_dim, device=device) for _ in range(cfg.num_experts)]
    indices = torch.randint(0, tokens, (rows,), device=device)
    weights = torch.rand(rows, device=device)
    out_shape = (tokens, cfg.hidden_dim)
    base = torch.cuda.memory_allocated() / MIB

    report = {"scale": cfg.scale.value, "experts": cfg.num_experts, "hidden_dim": cfg.hidden_dim,
              "tokens": tokens, "top_k": cfg.top_k, "dtype": "fp32", "steps": cfg.active_steps}  # fmt: skip
    report["max_abs_diff"] = verify_correctness(experts, indices, weights, out_shape)
    std_ms, std_mem = benchmark_standard(experts, indices, weights, out_shape, cfg.active_steps)
    fast_ms, fast_mem = benchmark_fastmoe_grouped(experts, indices, weights, out_shape, cfg.active_steps)
    report["kernel"] = {
        "standard_ms": std_ms, "grouped_ms": fast_ms, "speedup": std_ms / fast_ms,
        "standard_extra_mib": std_mem - base, "grouped_extra_mib": fast_mem - base,
    }  # fmt: skip
    log.info("combine: standard %.3f ms, grouped %.3f ms (%.2fx); extra memory %.0f vs %.0f MiB",
             std_ms, fast_ms, std_ms / fast_ms, std_mem - base, fast_mem - base)  # fmt: skip
    del experts, indices, weights
    torch.cuda.empty_cache()

    if training:
        train = {}
        try:
            train["standard_ms"], train["standard_peak_gib"] = run_training_experiment(
                consts.MoEImplementation.STANDARD, cfg
            )
        except torch.cuda.OutOfMemoryError:
            log.error("standard implementation ran out of memory")
            train["standard_ms"] = train["standard_peak_gib"] = None
        train["fast_ms"], train["fast_peak_gib"] = run_training_experiment(consts.MoEImplementation.FAST, cfg)
        if train["standard_ms"]:
            train["speedup"] = train["standard_ms"] / train["fast_ms"]
        report["training"] = train
        log.info("training: %s", train)
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    run_on_cloud(MoEScale(args[0]) if args else MoEScale.GIGACHAT_700B, training="--no-training" not in sys.argv)
