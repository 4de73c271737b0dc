#!/usr/bin/env python3
"""Test infrastructure: stage the reference's own CPU implementation of the path for timing.

The reference's decode path is pure Python over torch (speccheck/specimpl.py, speccheck/mtp.py), so
"building" it means placing those two modules, unmodified, where a machine without the reference
checkout can import them:

    python oracle/make_ref.py [--reference /path/to/reference]

copies them byte for byte into oracle/_ref/speccheck/ (kept out of version control, never edited)
and prints their SHA-256.  Only the benchmark's reference arm and the tests import from there;
nothing of the product does.  `load()` returns the reference's (specimpl, mtp) modules or None when
the copy is absent, and `make_forward()` builds a reference Forward over seeded weights with the
checkpoint reader bypassed (the reader wants a safetensors shard that does not exist here).
"""
from __future__ import annotations

import argparse
import hashlib
import importlib
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
FILES = ("__init__.py", "specimpl.py", "mtp.py")


def stage(reference: Path) -> dict:
    src = reference / "speccheck"
    if not (src / "specimpl.py").exists():
        raise FileNotFoundError(f"{src}/specimpl.py not found")
    out = DEST / "speccheck"
    out.mkdir(parents=True, exist_ok=True)
    sums = {}
    for name in FILES:
        if (src / name).exists():
            shutil.copyfile(src / name, out / name)
            sums[name] = hashlib.sha256((out / name).read_bytes()).hexdigest()
        elif name == "__init__.py":
            (out / name).write_text("")
    return sums


def load():
    """(specimpl, mtp) modules of the staged reference, or None."""
    if not (DEST / "speccheck" / "specimpl.py").exists():
        return None
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    try:
        return importlib.import_module("speccheck.specimpl"), importlib.import_module("speccheck.mtp")
    except Exception:           # a dependency of the reference (safetensors) is missing on this machine
        return None


def make_forward(ref, params: dict, gdn_form: str = "chunk"):
    """The reference's Forward over a dict of seeded tensors (its checkpoint reader is bypassed)."""
    import torch
    w = ref.Weights.__new__(ref.Weights)
    w.dtype = torch.bfloat16
    w.p = params
    return ref.Forward(w, gdn_form=gdn_form)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    a = ap.parse_args()
    for k, v in stage(Path(a.reference)).items():
        print(v, k)
