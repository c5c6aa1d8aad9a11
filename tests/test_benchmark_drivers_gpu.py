"""The benchmark drivers end to end at the smallest preset, on one GPU."""

import dataclasses

import pytest
import torch

from fastmoe_b200 import consts
from fastmoe_b200.benchmarks import benchmark_dist, run_on_cloud
from fastmoe_b200.config import MoEScale, get_config
from fastmoe_b200.models.tiny_model import TinyModel

pytestmark = pytest.mark.gpu


def test_run_on_cloud_report_at_debug_scale(capsys):
    cfg = dataclasses.replace(get_config(MoEScale.DEBUG), active_steps=3)
    report = run_on_cloud.run_on_cloud(cfg=cfg)
    assert report["max_abs_diff"] <= 1e-4
    assert report["kernel"]["grouped_ms"] > 0 and report["kernel"]["standard_ms"] > 0
    train = report["training"]
    assert train["standard_ms"] > 0 and train["fast_ms"] > 0 and train["fast_peak_gib"] > 0
    assert '"kernel"' in capsys.readouterr().out  # the JSON line


@pytest.mark.parametrize(
    "implementation,micro_batches",
    [(consts.MoEImplementation.STANDARD, None), (consts.MoEImplementation.FAST, None), (consts.MoEImplementation.FAST, 2)],
)
def test_benchmark_step_single_rank(implementation, micro_batches):
    """Forward + backward of the model shells; FAST both as the plain block a single rank gets by
    default and with two micro-batches on side streams (gradients cross the streams)."""
    cfg = get_config(MoEScale.DEBUG)
    torch.manual_seed(0)
    model = TinyModel(cfg.hidden_dim, cfg.hidden_dim, 8, 256, 2, cfg.num_experts, cfg.top_k, implementation,
                      None, None, use_moe=True, num_micro_batches=micro_batches).cuda().to(torch.bfloat16)  # fmt: skip
    x = torch.randn(cfg.batch_size, cfg.seq_len, cfg.hidden_dim, device="cuda", dtype=torch.bfloat16,
                    requires_grad=True)  # fmt: skip
    ms, mib = benchmark_dist.benchmark_step(model, x, "test", steps=2, warmup=1)
    assert ms > 0 and mib > 0
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()
    grads = [p.grad for p in model.parameters()]
    assert all(g is not None and torch.isfinite(g.float()).all() for g in grads)
