"""Benchmark presets, model shells and driver entry points: names, signatures and the host-side
arithmetic that needs no GPU."""

import inspect

import pytest
import torch

from fastmoe_b200 import consts
from fastmoe_b200.benchmarks import benchmark_dist, run_on_cloud
from fastmoe_b200.config import MoEScale, MoESetup, get_config
from fastmoe_b200.models.tiny_model import Block, FeedForward, MoEBlock, PipelinedMoEBlock, TinyModel


def test_presets_match_the_reference_sizes():
    debug, mid, big = (get_config(s) for s in (MoEScale.DEBUG, MoEScale.GIGACHAT_10B, MoEScale.GIGACHAT_700B))
    assert (debug.batch_size, debug.seq_len, debug.hidden_dim, debug.num_experts, debug.top_k) == (2, 128, 512, 4, 2)
    assert (mid.batch_size, mid.seq_len, mid.hidden_dim, mid.ff_dim, mid.num_experts, mid.top_k,
            mid.comm_balance_factor) == (16, 2048, 8192, 8192, 8, 2, 8)  # fmt: skip
    assert (big.batch_size, big.seq_len, big.hidden_dim, big.num_experts, big.top_k) == (2, 2048, 16384, 256, 4)
    assert big.total_tokens == 16384 and big.activation_volume_mb == 1024.0
    assert (big.warmup_steps, big.active_steps, big.n_layers, big.n_heads) == (10, 50, 2, 32)
    assert get_config("gigachat-10b") == mid and get_config() == debug
    assert MoESetup().seq_len == 4096


def test_entry_points_keep_the_reference_names_and_arguments():
    def names(fn):
        return list(inspect.signature(fn).parameters)

    assert names(run_on_cloud.verify_correctness)[:4] == ["expert_outputs", "indices", "weights", "out_shape"]
    for fn in (run_on_cloud.benchmark_standard, run_on_cloud.benchmark_fastmoe_grouped):
        assert names(fn) == ["expert_outputs", "indices", "weights", "out_shape", "steps"]
    assert names(run_on_cloud.run_training_experiment)[:2] == ["implementation", "cfg"]
    assert names(benchmark_dist.benchmark_step)[:4] == ["model", "x", "desc", "profile_trace"]
    for fn in (benchmark_dist.setup, benchmark_dist.cleanup, benchmark_dist.run_benchmark, run_on_cloud.run_on_cloud):
        assert callable(fn)
    assert names(TinyModel.__init__)[1:12] == ["in_dim", "dim", "n_heads", "ff_dim", "n_layers", "num_experts", "top_k",
                                               "implementation", "stream0", "stream1", "comm_balance_factor"]  # fmt: skip
    assert inspect.signature(TinyModel.__init__).parameters["use_moe"].kind is inspect.Parameter.KEYWORD_ONLY


def test_drivers_do_nothing_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert run_on_cloud.run_on_cloud(MoEScale.DEBUG) is None
    assert benchmark_dist.run_benchmark() is None


def test_dense_model_trains_on_cpu():
    torch.manual_seed(0)
    model = TinyModel(12, 16, 4, 32, 2, None, None, None, None, None, use_moe=False)
    assert all(isinstance(b, Block) and isinstance(b.ff, FeedForward) for b in model.blocks)
    x = torch.randn(2, 5, 12)
    y = model(x)
    assert y.shape == x.shape
    y.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


def test_moe_models_build_with_and_without_the_optional_arguments():
    std = TinyModel(8, 16, 4, 32, 2, 4, 2, consts.MoEImplementation.STANDARD, None, None, use_moe=True)
    assert all(isinstance(b, MoEBlock) and b.ff.top_k == 2 and len(b.ff.experts) == 4 for b in std.blocks)
    # the call the reference's training benchmark makes: no top_k, no streams
    fast = TinyModel(in_dim=8, dim=16, n_heads=4, ff_dim=32, n_layers=2, num_experts=4,
                     implementation=consts.MoEImplementation.FAST, comm_balance_factor=1, use_moe=True)  # fmt: skip
    assert all(isinstance(b, PipelinedMoEBlock) and b.moe.top_k == 2 for b in fast.blocks)
    with pytest.raises(ValueError):
        TinyModel(8, 16, 4, 32, 1, use_moe=True)
    with pytest.raises(NotImplementedError):
        TinyModel(8, 16, 4, 32, 1, 4, 2, "other", use_moe=True)
