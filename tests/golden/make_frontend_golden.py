"""Generates ``frontend_golden.json`` by running the REFERENCE front end over the case grid.

    PYTHONPATH=<reference checkout> python tests/golden/make_frontend_golden.py

Needs the reference checkout on PYTHONPATH (it is pure Python: torch + triton.cdiv).  The JSON is
committed; the tests only read it.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from frontend_cases import cases, split_cases  # noqa: E402
from frontend_run import compact, run_case  # noqa: E402


def main():
    import syncopate  # noqa: F401  (fails loudly when the reference is not importable)

    golden = {}
    for name, builder, world, kw, codegen in cases():
        golden[name] = compact(run_case("syncopate", builder, world, kw, codegen))
    for name, builder, world, kw, n in split_cases():
        golden[name] = compact(run_case("syncopate", builder, world, kw, "ce", num_splits=n))
    path = os.path.join(HERE, "frontend_golden.json")
    with open(path, "w") as f:
        json.dump(golden, f, sort_keys=True, separators=(",", ":"))
    print(f"wrote {path}: {len(golden)} cases, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
