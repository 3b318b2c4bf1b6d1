"""Stage the reference's own CPU routing benchmark under oracle/_ref/ (git-ignored).

TEST / BENCHMARK INFRASTRUCTURE ONLY (see the package docstring).

    python -m oracle.build_ref --reference /path/to/moe-routers

The reference's CPU path is pure Python (`bench_router.py --device cpu`, lines 484-505, with
`models/decoder_moe.py` for the routers), so "building" it means placing its four unmodified files
where the benchmark's reference arm can run them on a machine that has no checkout of the
reference.  Nothing is edited, and nothing lands in the version-controlled tree: oracle/_ref/ is
ignored by git.  `oracle.ref_runner` runs the staged files.
"""
from __future__ import annotations

import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = ["bench_router.py", "models/__init__.py", "models/decoder_moe.py", "models/transformer_decoder_model.py"]


def stage(reference_root: str) -> str | None:
    """Copy the files if the checkout has them all; returns the staged directory or None."""
    if not all(os.path.isfile(os.path.join(reference_root, f)) for f in FILES):
        return None
    for f in FILES:
        dst = os.path.join(REF_DIR, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference_root, f), dst)
    return REF_DIR


def staged() -> bool:
    return all(os.path.isfile(os.path.join(REF_DIR, f)) for f in FILES)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of santiweide/moe-routers")
    a = ap.parse_args()
    out = stage(a.reference)
    print(out if out else f"reference checkout not found at {a.reference}: nothing staged")
