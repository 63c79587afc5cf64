"""The checked build (-DB200EMB_BOUNDS=1: every index a kernel reads from device memory is range-checked
by the kernel, csrc/bounds.cuh) runs the tiny models of every architecture and weight format, gives the
normal build's rows bit for bit, and reports a planted out-of-range sequence boundary as a status instead
of reading past the token stream. It is the stand-in for a memory checker where none may be run. A library
is loaded once per process, so both variants run as child processes (tests/checked_build_cases.py)."""
import os
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def test_checked_build_matches_the_normal_build_and_reports_a_bad_boundary(tmp_path):
    from infinity_b200 import build as b
    checked = b.build(checked=True)   # a no-op when the library travelled with the tree
    script = str(ROOT / "tests" / "checked_build_cases.py")
    env = dict(os.environ)
    env.pop("B200EMB_LIBRARY", None)
    r = subprocess.run([sys.executable, script, str(tmp_path), "normal"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    env["B200EMB_LIBRARY"] = str(checked)
    r = subprocess.run([sys.executable, script, str(tmp_path), "checked"], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "checked: " in r.stdout
