"""Installs the UNMODIFIED reference package (polkadot21/fastmoe, pure Python) into
oracle/_ref/ so that its own CPU path can be timed beside this build's kernels.

    python oracle/install_ref.py /path/to/reference/checkout

TEST INFRASTRUCTURE, like everything under oracle/: only bench.py's CPU-baseline legs and
tests use what this installs, and only as the thing measured against, never as a compute
path of the product. oracle/_ref/ is not tracked (no reference source enters the history);
it is produced by this recipe wherever a checkout of the reference exists, and found by
`oracle.reference_ops()` where it was installed.

The install is pip's, offline, without dependency resolution (torch and the settings
libraries the package imports are already in the image). pip builds the wheel inside the
source tree, so the checkout is copied to a temporary directory first.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

TARGET = Path(__file__).resolve().parent / "_ref"


def install(checkout: str | Path, wheelhouse: str | Path | None = "/opt/wheelhouse") -> Path:
    checkout = Path(checkout)
    if not (checkout / "pyproject.toml").exists():
        raise FileNotFoundError(f"{checkout} is not a checkout of the reference (no pyproject.toml)")
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "fastmoe_src"
        shutil.copytree(checkout, src, ignore=shutil.ignore_patterns(".git", "assets", "uv.lock"))
        if TARGET.exists():
            shutil.rmtree(TARGET)
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--target", str(TARGET)]  # fmt: skip
        if wheelhouse and Path(wheelhouse).is_dir():
            cmd += ["--find-links", str(wheelhouse)]
        proc = subprocess.run(cmd + [str(src)], capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"installing the reference failed:\n{proc.stdout}\n{proc.stderr}")
    if not (TARGET / "fastmoe" / "kernels" / "ops.py").exists():
        raise RuntimeError(f"the install did not produce {TARGET}/fastmoe/kernels/ops.py")
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(install(sys.argv[1]))
