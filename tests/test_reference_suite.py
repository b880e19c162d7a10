"""Runs the reference project's own CPU unit tests (its known-answer vectors for plans, signals,
generated programs and lowered schedules) against THIS package, by aliasing the ``syncopate``
import name.  The reference checkout is looked for where the environment variable
SYNCOPATE_REFERENCE points, else in a directory called ``reference`` next to this repository;
without one the test is skipped (the same vectors are then covered through
tests/golden/frontend_golden.json)."""
import os
import subprocess
import sys

import pytest

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("SYNCOPATE_REFERENCE") or os.path.join(os.path.dirname(_REPO), "reference")
FILES = [
    "tests/test_comm_plan.py",
    "tests/test_descriptor.py",
    "tests/test_tile_schedule.py",
    "tests/test_plan_compute_signal.py",
    "tests/test_allgather_schedule.py",
    "tests/test_lowering.py",
    "tests/test_codegen_all_gather.py",
    "tests/test_ring_allgather_codegen.py",
    "tests/test_double_ring_allgather_codegen.py",
    "tests/test_reduce_scatter_codegen.py",
    "tests/test_all_reduce_descriptor.py",
]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests")), reason="reference checkout not mounted")
def test_reference_cpu_suite_passes_on_this_front_end(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([root, here])
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    cmd = [
        sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "-p", "alias_reference_imports",
        "--rootdir", str(tmp_path), "-c", os.devnull,
    ] + [os.path.join(REF, f) for f in FILES]
    res = subprocess.run(cmd, cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0, tail
    assert " passed" in res.stdout, tail
