"""A B200-native inference engine for the LFM2 architecture.

The public names follow the reference's (``lalamo/__init__.py``): ``LanguageModel`` with
``load`` / ``generate_tokens`` / ``stream_tokens``, ``GenerationConfig``, ``SamplingPolicy``,
``ModelRegistry``; the engine-level interface (``Engine``, ``StepEntry``) is this engine's own.
"""

from .config import Lfm2Config, ModelPlan, load_config, register_architecture
from .engine import Engine, EngineConfig, StepEntry
from .language_model import LanguageModel
from .model_registry import ModelRegistry, ModelSpec
from .sampling import GenerationConfig, SamplingPolicy
from .weights import WeightsError, load_weights, write_random_model

__version__ = "0.1.0"

__all__ = [
    "Engine",
    "EngineConfig",
    "GenerationConfig",
    "LanguageModel",
    "Lfm2Config",
    "ModelPlan",
    "ModelRegistry",
    "ModelSpec",
    "SamplingPolicy",
    "StepEntry",
    "WeightsError",
    "load_config",
    "load_weights",
    "register_architecture",
    "write_random_model",
]
