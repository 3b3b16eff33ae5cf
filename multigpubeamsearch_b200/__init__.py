"""B200-native beam-search step behind the MultiGPUBeamSearch engine API."""

from . import puzzles  # noqa: F401

__all__ = ["puzzles", "beam_engine", "records"]
