"""pytest plugin: makes ``import syncopate...`` resolve to this package's front end, so that the
reference project's own CPU test files can be run, unmodified and in place, against this
implementation (see test_reference_suite.py)."""
import importlib
import sys

import syncopate_b200

_SUBMODULES = [
    "communication",
    "communication.descriptor",
    "communication.code_gen",
    "communication.common_descriptors",
    "communication.common_descriptors.utils",
    "communication.common_descriptors.all_gather",
    "communication.common_descriptors.all_reduce",
    "communication.common_descriptors.all_to_all",
    "communication.common_descriptors.reduce_scatter",
    "communication.comm_runtime",
    "communication.comm_runtime.operations",
    "interface",
    "interface.tile_schedule",
    "interface.lowering",
]

sys.modules["syncopate"] = syncopate_b200
for _name in _SUBMODULES:
    sys.modules[f"syncopate.{_name}"] = importlib.import_module(f"syncopate_b200.{_name}")
