"""The documentation stays in step with the code: the generated API reference is current, every environment
variable the sources read is described, and the pages the index links to exist."""

import re
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent
DOCS = REPO / "docs"


def test_api_reference_is_current():
    r = subprocess.run([sys.executable, str(DOCS / "gen_api.py"), "--check"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr


def test_every_environment_variable_is_documented():
    text = (DOCS / "environment.md").read_text()
    pat = re.compile(r"""(?:environ(?:\.get|\.setdefault)?[\(\[]\s*|getenv\()["']([A-Z][A-Z_0-9]+)["']""")
    sources = list((REPO / "torchft_b200").rglob("*.py")) + list((REPO / "torchft_b200" / "csrc").rglob("*.*"))
    sources += [REPO / n for n in ("train_ddp.py", "train_diloco.py", "train_hsdp.py")]
    names = set()
    for p in sources:
        if p.suffix in (".py", ".h", ".cpp", ".cu", ".cuh"):
            names.update(pat.findall(p.read_text()))
    # constants that hold a variable's name (NAME = "TORCHFT_…") are read through the constant
    for p in (REPO / "torchft_b200").rglob("*.py"):
        names.update(re.findall(r"""^[A-Z_]+\s*(?::\s*str\s*)?=\s*["']((?:TORCHFT|TORCH_NCCL)_[A-Z_0-9]+)["']""", p.read_text(), re.M))
    names -= {"CUDA_VISIBLE_DEVICES", "PATH", "HOME", "TORCH_NCCL_DEBUG_INFO_PIPE_FILE_ENV_VAR"}
    missing = sorted(n for n in names if f"`{n}" not in text and f"`{n}=" not in text)
    assert not missing, f"not described in docs/environment.md: {missing}"
    assert len(names) > 20


def test_index_links_resolve():
    for page in DOCS.glob("*.md"):
        for target in re.findall(r"\]\(([^)#]+\.md)\)", page.read_text()):
            assert (DOCS / target).is_file(), f"{page.name} links to missing {target}"
