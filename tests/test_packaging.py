"""The package builds into a wheel offline, the wheel carries the native libraries and the lighthouse
console scripts, and an installed copy works away from the source tree (the reference ships a
maturin-built wheel with a ``torchft_lighthouse`` script, pyproject.toml:43-48)."""

import os
import shutil
import subprocess
import sys
import zipfile
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def _pip(*args, tmp):
    env = dict(os.environ, TMPDIR=str(tmp), PIP_DISABLE_PIP_VERSION_CHECK="1")
    return subprocess.run([sys.executable, "-m", "pip", *args, "--no-index", "--no-deps", "--no-cache-dir"],
                          cwd=REPO, env=env, capture_output=True, text=True, timeout=1200)


@pytest.fixture
def clean_setuptools_leftovers():
    """``pip wheel .`` builds in the source tree; remove what setuptools leaves next to the native build's objects."""
    yield
    for d in (REPO / "build").glob("lib.*"):
        shutil.rmtree(d, ignore_errors=True)
    for d in (REPO / "build").glob("bdist.*"):
        shutil.rmtree(d, ignore_errors=True)
    shutil.rmtree(REPO / "torchft_b200.egg-info", ignore_errors=True)


@pytest.mark.timeout(1500)
def test_wheel_builds_installs_and_runs(tmp_path, clean_setuptools_leftovers):
    out = tmp_path / "wheel"
    r = _pip("wheel", ".", "--no-build-isolation", "-w", str(out), tmp=tmp_path)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    (whl,) = list(out.glob("torchft_b200-*.whl"))
    assert "linux" in whl.name and "none-any" not in whl.name  # platform wheel: it holds shared objects
    names = zipfile.ZipFile(whl).namelist()
    assert "torchft_b200/_lib/libftb200_kernels.so" in names
    assert any(n.startswith("torchft_b200/_ftcp") and n.endswith(".so") for n in names)
    assert "torchft_b200/csrc/kernels/gemm_tcgen05_2cta.cu" in names  # sources travel: the package can rebuild itself
    assert not any(n.startswith(("tests/", "_work/", "baseline/")) for n in names)
    entry = next(n for n in names if n.endswith("entry_points.txt"))
    text = zipfile.ZipFile(whl).read(entry).decode()
    assert "torchft_lighthouse = torchft_b200.lighthouse_cli:main" in text
    assert "torchft_b200_lighthouse = torchft_b200.lighthouse_cli:main" in text

    site = tmp_path / "site"
    r = _pip("install", str(whl), "--target", str(site), tmp=tmp_path)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    # run from another directory so that the source tree is not importable by accident
    code = (
        "import torchft_b200, sys\n"
        f"assert torchft_b200.__file__.startswith({str(site)!r}), torchft_b200.__file__\n"
        "from torchft_b200 import Manager, DistributedDataParallel, Optimizer\n"
        "from torchft_b200.coordination import LighthouseServer\n"
        "from torchft_b200.local_sgd import DiLoCo, LocalSGD\n"
        "from torchft_b200.ops import _native\n"
        "_native.lib()\n"
        "lh = LighthouseServer(bind='[::]:0', min_replicas=1)\n"
        "assert lh.address().startswith('http://')\n"
        "lh.shutdown()\n"
        "print('installed ok')\n"
    )
    env = dict(os.environ, PYTHONPATH=str(site), FTB200_NO_AUTOBUILD="1")
    r = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "installed ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    r = subprocess.run([str(site / "bin" / "torchft_lighthouse"), "--help"], cwd=tmp_path, env=env, capture_output=True, text=True,
                       timeout=120)
    assert "--min_replicas" in (r.stdout + r.stderr)
