"""Benchmark presets with the names and sizes of polkadot21/fastmoe (src/fastmoe/config.py:9-92).

Plain dataclasses: the presets are code, not environment-driven settings, and the package
needs no settings library. Any field can be overridden with `dataclasses.replace`.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class MoEScale(str, Enum):
    DEBUG = "debug"
    GIGACHAT_10B = "gigachat-10b"
    GIGACHAT_700B = "gigachat-700b"


@dataclass(frozen=True)
class MoESetup:
    scale: MoEScale = MoEScale.DEBUG
    # model
    batch_size: int = 4
    seq_len: int = 4096
    hidden_dim: int = 4096
    n_heads: int = 32
    ff_dim: int = 4096
    n_layers: int = 2
    # MoE
    num_experts: int = 8
    top_k: int = 2
    # timing
    warmup_steps: int = 10
    active_steps: int = 50
    comm_balance_factor: int = 1

    @property
    def total_tokens(self) -> int:
        """Routed rows of one batch: batch * sequence * top_k."""
        return self.batch_size * self.seq_len * self.top_k

    @property
    def activation_volume_mb(self) -> float:
        """MiB of the fp32 [routed rows, hidden] tensor that the combine reads."""
        return self.total_tokens * self.hidden_dim * 4 / 2**20


_PRESETS = {
    MoEScale.DEBUG: dict(batch_size=2, seq_len=128, hidden_dim=512, num_experts=4, top_k=2),
    # wide layers, few experts: the expert-parallel overlap benchmark
    MoEScale.GIGACHAT_10B: dict(batch_size=16, seq_len=2048, hidden_dim=8192, ff_dim=8192, num_experts=8,
                                top_k=2, comm_balance_factor=8),  # fmt: skip
    # very wide rows, many small experts: the combine microbenchmark
    MoEScale.GIGACHAT_700B: dict(batch_size=2, seq_len=2048, hidden_dim=16384, num_experts=256, top_k=4),
}


def get_config(scale: MoEScale = MoEScale.DEBUG) -> MoESetup:
    """The preset for `scale` (defaults for anything else)."""
    scale = MoEScale(scale)
    return MoESetup(scale=scale, **_PRESETS.get(scale, {}))
