"""Build recipe for the CPU checker (TEST INFRASTRUCTURE ONLY).

Two products:

* ``oracle/liboracle.so`` -- the plain-C restatement in ``oracle_ops.c`` (always built;
  a second copy ``liboracle_fast.so`` is built with ``-O3 -march=native -fopenmp`` for the
  benchmark's CPU-baseline leg).
* ``oracle/_ref/libref_stories.so``, ``oracle/_ref/libref_dynamic.so`` and
  ``oracle/_ref/libref_inline.so`` -- the reference's
  own ``training/stories_cpu_ops.h`` and ``training/training_dynamic/cpu_ops.h``, and the inline
  operator blocks of ``training/training_dynamic/train.m`` / helpers of ``training/forward.h``
  (extracted by line range into the wrappers of ``ref_inline_exports.c.in``), compiled from
  where they lie (only when the reference tree is present).  The header text is piped to
  gcc on standard input followed by a small file of exported wrappers, so that its quoted
  ``#include "stories_config.h"`` / ``"config.h"`` resolves to the stand-in headers under
  ``oracle/shim`` instead of the Objective-C originals, and no reference source is copied
  into this repository.  ``-ffp-contract=off`` keeps the arithmetic as written.

The reference tree is looked for in ``--ref-root``, else in the environment variable
``ANE_REFERENCE_ROOT``, else in a directory ``reference`` beside this repository; where none of
them holds it, only the restatement is built.

Usage: ``python oracle/build_oracle.py [--ref-root DIR] [--force]``
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REF_ROOT = os.environ.get("ANE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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


def expand_inline_template(template: str, ref_root: str) -> bytes:
    """Replace every `//@REF path first last` line of the template by those lines of the reference file, after
    checking the first and last of them against the `//@EXPECT_FIRST` / `//@EXPECT_LAST` lines that follow."""
    out: list[str] = []
    lines = open(template, encoding="utf-8").read().split("\n")
    i = 0
    cache: dict[str, list[str]] = {}
    while i < len(lines):
        ln = lines[i]
        if ln.startswith("//@REF "):
            _, rel, first, last = ln.split()
            first, last = int(first), int(last)
            want_first = lines[i + 1].removeprefix("//@EXPECT_FIRST ").strip()
            want_last = lines[i + 2].removeprefix("//@EXPECT_LAST ").strip()
            if not (lines[i + 1].startswith("//@EXPECT_FIRST ") and lines[i + 2].startswith("//@EXPECT_LAST ")):
                raise RuntimeError(f"{template}:{i + 1}: //@REF must be followed by //@EXPECT_FIRST and //@EXPECT_LAST")
            if rel not in cache:
                cache[rel] = open(os.path.join(ref_root, rel), encoding="utf-8", errors="replace").read().split("\n")
            src = cache[rel]
            got_first, got_last = src[first - 1].strip(), src[last - 1].strip()
            if got_first != want_first or got_last != want_last:
                raise RuntimeError(f"{rel}:{first}-{last} no longer holds the expected block "
                                   f"(first line {got_first!r}, last line {got_last!r}): the reference moved")
            out.append(f'#line {first} "{rel}"')
            out.extend(src[first - 1:last])
            out.append(f'#line {i + 4} "{os.path.basename(template)}"')
            i += 3
        else:
            out.append(ln)
            i += 1
    return "\n".join(out).encode("utf-8")


def build_reference_inline(ref_root: str = DEFAULT_REF_ROOT, force: bool = False) -> list[str]:
    """Compile the inline operator blocks of train.m and the plain-C helpers of forward.h into
    oracle/_ref/libref_inline.so (see ref_inline_exports.c.in)."""
    train_m = os.path.join(ref_root, "training", "training_dynamic", "train.m")
    forward_h = os.path.join(ref_root, "training", "forward.h")
    if not (os.path.exists(train_m) and os.path.exists(forward_h)):
        return []
    template = os.path.join(HERE, "ref_inline_exports.c.in")
    shim_dir = os.path.join(HERE, "shim")
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libref_inline.so")
    deps = [train_m, forward_h, template, os.path.join(shim_dir, "accelerate_shim.h")]
    if force or not _newer(out, deps):
        text = expand_inline_template(template, ref_root)
        cmd = ["gcc", "-std=gnu11", "-shared", "-fPIC", "-O2", "-ffp-contract=off", "-w", "-I", shim_dir, "-x", "c", "-", "-o", out, "-lm"]
        subprocess.run(cmd, input=text, check=True, cwd=shim_dir)
    return [out]


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
    outs += build_reference_inline(ref_root, force)
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
