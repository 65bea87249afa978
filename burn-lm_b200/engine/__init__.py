"""The step function and, above it, the generation loop and trace replay."""
from .engine import Engine, StepEntry, Workspace
from .generate import (GenerateOptions, GenerationLoop, GenerationOutput, GenerationStats, RequestResult,
                       plan_batches)

__all__ = ["Engine", "StepEntry", "Workspace", "GenerateOptions", "GenerationLoop", "GenerationOutput",
           "GenerationStats", "RequestResult", "plan_batches"]
