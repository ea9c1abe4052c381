"""Architectures this framework ships.  Importing the package registers them."""
from . import qwen3  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry"]
