"""Stage the reference project's own CPU-runnable files under ``oracle/_ref/`` (test infrastructure).

    python -m oracle.make_ref [<checkout of HKUSTDial/omni-moe>]      # default: $OMNI_MOE_REFERENCE

The reference is pure Python, so "building" it is a copy: the files listed in ``FILES`` are taken
byte for byte from the checkout, with a manifest of their SHA-256 digests.  ``oracle/_ref/`` is
listed in ``.gitignore`` - the files never enter this repository's history - but it travels with the
working tree to the machine that runs the GPU tests and the benchmark, where no checkout exists.

What uses it (and nothing else does):

* ``bench.py --impl reference`` and the ``cpu_baseline`` leg time ``OmniMoE_Torch``
  (omni_moe/modules/omni_moe.py:109-194), the reference's own PyTorch layer, on the host cores;
* ``tests/test_oracle_golden.py`` checks the restatement in ``omni_oracle.py`` against it directly;
* ``tests/test_gpu_reference_files.py`` runs the reference's own test files against this library
  through the ``omni_moe.ops.triton`` import path they use.

Without a checkout this is a no-op and every user falls back (the benchmark to the restatement in
``omni_oracle.py``, labelled as such; the tests skip).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = [
    "omni_moe/modules/omni_moe.py",             # OmniMoEConfig, OmniMoE_Torch: the CPU path that is timed
    "omni_moe/ops/triton/omni_scheduler.py",    # get_scheduling_info (torch ops only)
    "tests/testing.py",                         # the reference's benchmark / validation harness
    "tests/test_router.py",
    "tests/test_expert.py",
    "tests/test_mlp.py",
]


def default_checkout() -> str | None:
    cand = os.environ.get("OMNI_MOE_REFERENCE")
    if cand and os.path.isfile(os.path.join(cand, FILES[0])):
        return cand
    return None


def stage(checkout: str | None = None, quiet: bool = False) -> str | None:
    """Copy the files; returns the destination, or None when there is no checkout to copy from."""
    src = checkout or default_checkout()
    if src is None:
        if not quiet:
            print("oracle/_ref: no reference checkout found (set OMNI_MOE_REFERENCE); nothing staged")
        return None
    manifest = {}
    for rel in FILES:
        a, b = os.path.join(src, rel), os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(b), exist_ok=True)
        shutil.copyfile(a, b)
        manifest[rel] = hashlib.sha256(open(b, "rb").read()).hexdigest()
    with open(os.path.join(DEST, "MANIFEST.json"), "w") as f:
        json.dump({"source": "HKUSTDial/omni-moe (files copied unmodified)", "sha256": manifest}, f, indent=1)
    if not quiet:
        print(f"oracle/_ref: staged {len(FILES)} files from {src}")
    return DEST


if __name__ == "__main__":
    stage(sys.argv[1] if len(sys.argv) > 1 else None)
