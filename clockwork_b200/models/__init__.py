"""Architectures.  Importing this package registers each of them by name."""

from . import gamesun, kapolorn, nuzulorn, qwen2, rapitar  # noqa: F401
from .qwen2 import Qwen2Architecture, Qwen2Config
from .rapitar import RapitarArchitecture, RapitarConfig

__all__ = ["Qwen2Architecture", "Qwen2Config", "RapitarArchitecture", "RapitarConfig"]
