"""The step function and, above it, the generation loop and trace replay."""
from .engine import Engine, StepEntry, Workspace

__all__ = ["Engine", "StepEntry", "Workspace"]
