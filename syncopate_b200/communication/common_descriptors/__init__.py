"""Plan builders for the common collectives (same names as
syncopate/communication/common_descriptors/__init__.py:3-28), plus ``split_transfers_along_axis``
(chunk-size tuning for plans that are lowered to kernel schedules)."""

from .all_gather import (
    build_all_gather_plan_1d_swizzle,
    build_double_ring_all_gather_plan,
    build_ring_all_gather_plan,
)
from .all_reduce import build_all_reduce_nvsharp_plan, build_all_reduce_plan
from .all_to_all import (
    build_all_to_all_plan,
    build_all_to_all_plan_axis,
    build_all_to_all_plan_dim,
    build_all_to_all_plan_dim_waves,
)
from .chunk_split import split_transfers_along_axis
from .reduce_scatter import build_reduce_scatter_collective_plan, build_reduce_scatter_direct_reduce_plan

__all__ = [
    "build_all_gather_plan_1d_swizzle",
    "build_ring_all_gather_plan",
    "build_double_ring_all_gather_plan",
    "build_all_to_all_plan",
    "build_all_to_all_plan_dim",
    "build_all_to_all_plan_dim_waves",
    "build_all_to_all_plan_axis",
    "build_reduce_scatter_collective_plan",
    "build_reduce_scatter_direct_reduce_plan",
    "build_all_reduce_plan",
    "build_all_reduce_nvsharp_plan",
    "split_transfers_along_axis",
]
