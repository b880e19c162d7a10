"""Front end vs the golden vectors produced by the reference implementation
(tests/golden/make_frontend_golden.py): plans, planned signals, generated op programs and lowered
schedules must be identical, bit for bit, for every case of the grid."""
import json
import os

import pytest

from frontend_cases import cases, split_cases
from frontend_run import compact, run_case

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "frontend_golden.json")))


def _check(name, got_full):
    want = GOLDEN[name]
    got = compact(got_full)
    # compare the readable parts first so that a mismatch points at something
    for key in ("lowered", "lowered_error", "counters", "comm_info", "comm_info_error"):
        if key in want:
            assert json.loads(json.dumps(got_full.get(key))) == want[key], f"{name}: {key} differs"
    if "full" in want:
        got_norm = json.loads(json.dumps(got_full))
        for key in want["full"]:
            assert got_norm.get(key) == want["full"][key], f"{name}: {key} differs"
    assert got["sha256"] == want["sha256"], f"{name}: digest of the complete canonical form differs"


@pytest.mark.parametrize("case", cases(), ids=lambda c: c[0])
def test_case_matches_reference_golden(case):
    name, builder, world, kw, codegen = case
    _check(name, run_case("syncopate_b200", builder, world, kw, codegen))


@pytest.mark.parametrize("case", split_cases(), ids=lambda c: c[0])
def test_split_case_matches_reference_golden(case):
    name, builder, world, kw, n = case
    _check(name, run_case("syncopate_b200", builder, world, kw, "ce", num_splits=n))


def test_golden_covers_every_case():
    names = {c[0] for c in cases()} | {c[0] for c in split_cases()}
    assert names == set(GOLDEN)
