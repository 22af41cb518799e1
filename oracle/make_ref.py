"""Place an UNMODIFIED copy of the reference's Python packages under oracle/_ref/.

    python oracle/make_ref.py [--ref /path/to/MatchAttention]

TEST INFRASTRUCTURE ONLY.  oracle/_ref/ is a build output: it is listed in
.gitignore and never committed.  It exists so that the machine that runs the
GPU tests and the benchmark, which has no checkout of the reference, can still
run the reference's own code next to this library:

* tests/test_gpu_model.py builds the reference's MatchStereo twice (its
  'pytorch' branch and its 'cuda' branch with this library behind the module
  name ``match_attention``) and compares them;
* bench.py --mode model times that model; bench.py's CPU baseline times the
  reference's own models/mat_pytorch_impl.py on the host cores.

Only ``models/*.py`` and ``utils/*.py`` are copied, byte for byte (their CUDA
sources, demos and assets are not needed).  A MANIFEST with the SHA-256 of every
copied file is written beside them; oracle.ref_loader checks it before importing.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")
PACKAGES = ("models", "utils")


def default_source() -> str | None:
    """$MATCHATTN_REF, else a directory named 'reference' next to this repository."""
    cand = os.environ.get("MATCHATTN_REF") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "models", "mat_pytorch_impl.py")) else None


def sha256(path: str) -> str:
    with open(path, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def make_ref(src: str | None = None, force: bool = False) -> str | None:
    """Copy the packages; returns the output directory, or None when no reference checkout is found."""
    src = src or default_source()
    if src is None:
        return None
    manifest_path = os.path.join(REF_OUT, "MANIFEST.json")
    wanted = {}
    for pkg in PACKAGES:
        for name in sorted(os.listdir(os.path.join(src, pkg))):
            if name.endswith(".py"):
                wanted[f"{pkg}/{name}"] = sha256(os.path.join(src, pkg, name))
    if not force and os.path.exists(manifest_path):
        with open(manifest_path) as f:
            if json.load(f).get("files") == wanted:
                return REF_OUT
    if os.path.isdir(REF_OUT):
        shutil.rmtree(REF_OUT)
    for rel in wanted:
        dst = os.path.join(REF_OUT, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(src, rel), dst)
        os.chmod(dst, 0o644)
    with open(manifest_path, "w") as f:
        json.dump({"source": "TingmanYan/MatchAttention, models/*.py and utils/*.py, unmodified", "files": wanted}, f,
                  indent=1)
    return REF_OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = make_ref(a.ref, a.force)
    print(out if out else "no reference checkout found (set MATCHATTN_REF)")
