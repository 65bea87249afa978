"""burn-lm_b200: a small, whole, B200-native library for generating with the dense Llama decoder.

From a model folder (config.json, model.safetensors) to next tokens on one GPU: typed configuration
and registry, weights by name, layers put together from parts, a paged cache with a slot per
sequence, one step function, a generation loop, sampling, and hand-written sm_100a kernels.
"""
from . import architectures  # noqa: F401  (registers the architectures)
from . import parts  # noqa: F401  (registers the parts)
from .config import ConfigError, LlamaConfig, preset, preset_names, read_config_json
from .registry import (Architecture, architecture, architecture_of, architectures as list_architectures,
                       register_architecture, register_part)
from .weights import TensorSpec, WeightsError, write_random_model
from .model import Model, load_model, plan_of, random_model
from .cache import Cache, CacheError, CacheFull, ContextLengthExceeded
from .engine import Engine, GenerateOptions, GenerationLoop, StepEntry
from .sampling import Sampler, SamplingParams
from .api import LanguageModel, load, load_random

__version__ = "0.1.0"
