"""Stages the reference's own implementation of the path under oracle/_ref/ (git-ignored, travels to the GPU box).

    python oracle/make_ref.py [REFERENCE_ROOT]        # default: the checkout named by DEFAULT_ROOT below

The reference (angryslavemerchant/QuantExperiments, package `shapequant`) is pure Python, so there is nothing to
compile: the recipe copies, unmodified, the four modules that define and execute the packed format -
shapequant/codebook.py, masks.py, packed.py and kernels/gemv.py (the Triton batch-1 kernel) - plus the two package
__init__ files, into oracle/_ref/shapequant/.  Nothing of it enters the repository's history or the product: only
tests/, __graft_entry__.smoke() and bench.py's reference legs may import it, as the checker and as the timed baseline.
A file MANIFEST.json records the source paths and sizes."""
from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path

FILES = ["shapequant/__init__.py", "shapequant/codebook.py", "shapequant/masks.py", "shapequant/packed.py",
         "shapequant/kernels/__init__.py", "shapequant/kernels/gemv.py"]
HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
DEFAULT_ROOT = Path("/root/reference")


def make(ref_root: str | Path = DEFAULT_ROOT) -> Path | None:
    """Copy the files if the reference is present; returns the destination (or None when it is absent)."""
    root = Path(ref_root)
    if not (root / FILES[1]).exists():
        return None
    manifest = {}
    for rel in FILES:
        dst = DEST / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(root / rel, dst)
        manifest[rel] = (root / rel).stat().st_size
    (DEST / "MANIFEST.json").write_text(json.dumps({"source": "angryslavemerchant/QuantExperiments", "files": manifest}, indent=1))
    return DEST


def load():
    """Import the staged package (`shapequant` from oracle/_ref); None when it has not been staged."""
    if not (DEST / FILES[3]).exists():
        return None
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    import importlib
    return importlib.import_module("shapequant")


if __name__ == "__main__":
    out = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT)
    print(out if out else "reference not found: nothing staged")
