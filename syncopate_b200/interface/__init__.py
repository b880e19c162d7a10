"""Bridge between communication and computation: ordered block schedules
(same exports as syncopate/interface/__init__.py)."""
from .lowering import lower_comm_plan_to_raw_schedules
from .tile_schedule import Mod1DSchedule, RawSchedule, SimplifiedSchedule, TileBlock, TileCoord

__all__ = [
    "TileCoord",
    "TileBlock",
    "RawSchedule",
    "SimplifiedSchedule",
    "Mod1DSchedule",
    "lower_comm_plan_to_raw_schedules",
]
