"""Makes ``oracle/_ref/grilly``: a runnable copy of the reference's Python package, taken from its source tree.

    python oracle/make_ref.py /path/to/grilly-source

TEST INFRASTRUCTURE ONLY, like everything under oracle/. The copy is not part of this repository's history
(``oracle/_ref/`` is git-ignored); it exists so that the machine that runs the GPU tests and the benchmark, which has
no reference source tree, can still execute the reference's own CPU code: ``bench.py --impl reference`` times
``VulkanSentenceTransformer._forward_layer`` from it, and tests/test_gpu_reference_dropin.py runs that same method
unchanged on top of ``grilly_b200.Compute()``. Only ``*.py`` files are copied (no shaders, docs or tests); nothing
is edited.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

DEST = Path(__file__).resolve().parent / "_ref" / "grilly"
SKIP_DIRS = {"tests", "docs", "examples", "tutorials", "scripts", "shaders", ".git", "__pycache__"}


def make(src: str | Path) -> Path:
    src = Path(src).resolve()
    if not (src / "__init__.py").exists() or not (src / "backend").is_dir():
        raise SystemExit(f"{src} does not look like the grilly source tree")
    if DEST.exists():
        shutil.rmtree(DEST)
    n = 0
    for path in sorted(src.rglob("*.py")):
        rel = path.relative_to(src)
        if any(part in SKIP_DIRS for part in rel.parts[:-1]):
            continue
        out = DEST / rel
        out.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(path, out)
        n += 1
    (DEST.parent / "SOURCE.txt").write_text(f"copied {n} .py files from {src} by oracle/make_ref.py; not edited\n")
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/make_ref.py <path to the grilly source tree>")
    print(make(sys.argv[1]))
