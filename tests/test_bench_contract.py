"""bench.py's reference arm runs without a GPU (it times the reference's CPU path: the
unmodified package where oracle/install_ref.py has installed it, else the C port of it):
here on a small workload, checking the JSON line the driver parses."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("extra,kinds", [((), ("reference", "port")), (("--cpu-port",), ("port",))])
def test_reference_arm_prints_one_json_line_with_the_contract_keys(extra, kinds):
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
         "--workload", "combine_small_bf16_T1024_D4096_E64_top8", *extra],
        capture_output=True, text=True, timeout=300, env={"CUDA_VISIBLE_DEVICES": "", "PATH": "/usr/bin:/bin"},
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "combine_hbm_gbs" and d["unit"] == "GB/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype",
                "data", "config", "cpu_baseline", "e2e"):  # fmt: skip
        assert key in d, key
    assert d["steps"] == 2 and d["value"] > 0 and d["config"]["workload"].startswith("combine_small")
    assert d["cpu_baseline"]["kind"] in kinds and d["cpu_baseline"]["cores"] >= 1
    assert set(d["config"]) == {"workload", "T", "D", "E", "top_k", "routing"}  # the same keys as the GPU arm's
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]


def test_reference_arm_on_another_rank_exits_quietly():
    """Under a multi-rank launch only rank 0 times the CPU path; the others print nothing and exit 0."""
    env = {"CUDA_VISIBLE_DEVICES": "", "PATH": "/usr/bin:/bin", "RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
        capture_output=True, text=True, timeout=120, env=env,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert not [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
