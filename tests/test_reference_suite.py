"""Runs the reference project's own CPU unit tests (its known-answer vectors for plans, signals,
generated programs and lowered schedules) against THIS package, by aliasing the ``syncopate``
import name.  Only possible where the reference checkout is mounted; skipped elsewhere (the same
vectors are then covered through tests/golden/frontend_golden.json)."""
import os
import subprocess
import sys

import pytest

REF = os.environ.get("SYNCOPATE_REFERENCE", "/root/reference")
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
