"""Build recipe for the CPU checker (TEST INFRASTRUCTURE ONLY).

Two products:

* ``oracle/liboracle.so`` -- the plain-C restatement in ``oracle_ops.c`` (always built;
  a second copy ``liboracle_fast.so`` is built with ``-O3 -march=native -fopenmp`` for the
  benchmark's CPU-baseline leg).
* ``oracle/_ref/libref_stories.so`` and ``oracle/_ref/libref_dynamic.so`` -- the reference's
  own ``training/stories_cpu_ops.h`` and ``training/training_dynamic/cpu_ops.h`` compiled from
  where they lie (only when the reference tree is present).  The header text is piped to
  gcc on standard input followed by a small file of exported wrappers, so that its quoted
  ``#include "stories_config.h"`` / ``"config.h"`` resolves to the stand-in headers under
  ``oracle/shim`` instead of the Objective-C originals, and no reference source is copied
  into this repository.  ``-ffp-contract=off`` keeps the arithmetic as written.

Usage: ``python oracle/build_oracle.py [--ref-root DIR] [--force]``
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REF_ROOT = os.environ.get("ANE_REFERENCE_ROOT", "/root/reference")


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_restatement(force: bool = False) -> list[str]:
    src = os.path.join(HERE, "oracle_ops.c")
    outs = []
    for name, flags in (
        ("liboracle.so", ["-O2", "-ffp-contract=off"]),
        ("liboracle_fast.so", ["-O3", "-march=native", "-fopenmp"]),
    ):
        out = os.path.join(HERE, name)
        if force or not _newer(out, [src]):
            cmd = ["gcc", "-std=c11", "-shared", "-fPIC", "-fvisibility=hidden", *flags, src, "-o", out, "-lm"]
            subprocess.run(cmd, check=True)
        outs.append(out)
    return outs


def _build_ref_one(header: str, exports: str, shim_dir: str, out: str, flags: list[str]) -> None:
    with open(header, "rb") as f:
        text = f.read()
    with open(exports, "rb") as f:
        text += b"\n" + f.read()
    cmd = ["gcc", "-std=gnu11", "-shared", "-fPIC", *flags, "-w", "-x", "c", "-", "-o", out, "-lm"]
    # cwd = the stand-in directory: a quoted include read from stdin is searched there first.
    subprocess.run(cmd, input=text, check=True, cwd=shim_dir)


def build_reference(ref_root: str = DEFAULT_REF_ROOT, force: bool = False) -> list[str]:
    """Compile the reference's two operator headers into oracle/_ref/.  Returns the
    libraries built (empty list when the reference tree is not there)."""
    stories_h = os.path.join(ref_root, "training", "stories_cpu_ops.h")
    dynamic_h = os.path.join(ref_root, "training", "training_dynamic", "cpu_ops.h")
    if not (os.path.exists(stories_h) and os.path.exists(dynamic_h)):
        return []
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    outs = []
    jobs = [
        (stories_h, "ref_stories_exports.c", "stories", "libref_stories"),
        (dynamic_h, "ref_dynamic_exports.c", "dynamic", "libref_dynamic"),
    ]
    for header, exports, shim, stem in jobs:
        exp = os.path.join(HERE, exports)
        shim_dir = os.path.join(HERE, "shim", shim)
        deps = [header, exp, os.path.join(HERE, "shim", "accelerate_shim.h")]
        for suffix, flags in (("", ["-O2", "-ffp-contract=off"]), ("_fast", ["-O3", "-march=native"])):
            out = os.path.join(out_dir, f"{stem}{suffix}.so")
            if force or not _newer(out, deps):
                _build_ref_one(header, exp, shim_dir, out, flags)
            outs.append(out)
    return outs


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=DEFAULT_REF_ROOT)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print("\n".join(build_restatement(a.force)))
    refs = build_reference(a.ref_root, a.force)
    print("\n".join(refs) if refs else "reference tree not present: oracle/_ref not rebuilt")
    return 0


if __name__ == "__main__":
    sys.exit(main())
