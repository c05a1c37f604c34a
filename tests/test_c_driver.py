"""A plain C program calls libane_cuda through include/ane_cuda.h in the order of the reference's training step
(tests/c_driver/train_step_driver.c) and checks every operator against the C oracle.  Without a GPU the test
checks that the driver compiles and links against the header and the library; with one it runs it."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_driver", "train_step_driver.c")


def _build(tmp_path):
    from ane_b200 import lib
    from oracle.oracle import ensure_built
    lib.load()                       # raises if libane_cuda.so has not been built
    ensure_built()
    exe = str(tmp_path / "train_step_driver")
    cmd = ["gcc", "-O1", "-Wall", "-Werror", SRC, "-I", os.path.join(ROOT, "include"),
           "-L", os.path.join(ROOT, "ane_b200", "lib"), "-lane_cuda", "-L", os.path.join(ROOT, "oracle"), "-loracle", "-lm",
           "-Wl,-rpath," + os.path.join(ROOT, "ane_b200", "lib"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_driver_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    assert os.path.getsize(exe) > 0


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_driver_runs_the_training_step_order(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all operators agree with the oracle" in r.stdout
    assert r.stdout.count(" ok\n") == 19 and "MISMATCH" not in r.stdout
