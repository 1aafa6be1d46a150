"""The engine: a loaded model with its cache manager and step function.

``Engine.load`` goes from a model folder (``config.json`` + safetensors) to something that can
be stepped; the model class is chosen by ``config.json`` through the architecture registry.
Generation (scheduler, sampling) builds on this in :mod:`lalamo_b200.engine.generation`.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import torch

from .. import native, ops
from ..cache.manager import CacheManager
from ..config.plan import ModelPlan
from ..config.registry import ArchitectureConfig, load_config
from ..parts.base import Runtime
from ..parts.model import DecoderModel, TensorKey
from ..weights.loader import load_weights
from .executor import Executor, StepEntry

__all__ = ["Engine", "EngineConfig", "NoDeviceError", "resolve_dtype"]


class NoDeviceError(RuntimeError):
    pass


def resolve_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
        raise ValueError(f"the engine computes in bfloat16 or float32, not {name}")
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise ValueError(f"unknown dtype {name!r}; known: {sorted(table)}")
    return table[name]


@dataclass(frozen=True)
class EngineConfig:
    """Sizes of the engine that do not come from the model."""

    dtype: str = "bfloat16"
    page_size: int = 16
    max_tokens: int = 65536  # tokens all live requests may hold (the page pools are made for this)
    max_requests: int = 64  # live requests (state slots)
    max_batch_tokens: int = 2048  # tokens one step may run (the scheduler's budget)
    device: str = "cuda:0"
    cuda_graphs: bool = True  # replay decode steps from CUDA graphs
    freeze_gc: bool = True  # after loading, exempt the objects alive so far from garbage collection passes
    poison_freed: bool = False  # tests: overwrite pages and state slots with NaN when they are given back


def _require_device(device: str) -> torch.device:
    if not torch.cuda.is_available():
        raise NoDeviceError("lalamo_b200 runs on a CUDA device (sm_100a) only; none is visible and there is no CPU path")
    return torch.device(device)


class Engine:
    def __init__(
        self,
        plan: ModelPlan,
        tensors: dict[TensorKey, torch.Tensor],
        engine_config: EngineConfig = EngineConfig(),
        architecture_config: ArchitectureConfig | None = None,
    ) -> None:
        device = _require_device(engine_config.device)
        native.library()  # fails loudly if the kernels cannot be built or loaded
        ops.configure_matmul_precision()
        torch.cuda.set_device(device)
        self.engine_config = engine_config
        self.architecture_config = architecture_config
        self.plan = plan
        self.runtime = Runtime(device=device, dtype=resolve_dtype(engine_config.dtype))
        self.model = DecoderModel(plan, tensors, self.runtime)
        page_size = engine_config.page_size
        self.cache = CacheManager(
            self.model.cache_needs(),
            [entry.cache_from for entry in plan.schedule],
            self.runtime,
            page_size=page_size,
            num_pages=-(-engine_config.max_tokens // page_size),
            num_slots=engine_config.max_requests,
            poison_freed=engine_config.poison_freed,
        )
        self.executor = Executor(self.model, self.cache, self.runtime, use_graphs=engine_config.cuda_graphs)
        self._request_numbers = 0
        if engine_config.freeze_gc:
            # A full collection walks every live object; with a loaded model that costs milliseconds in
            # the middle of a decode step.  What is alive now stays alive for the engine's lifetime.
            gc.collect()
            gc.freeze()

    @classmethod
    def load(cls, model_dir: str | Path, engine_config: EngineConfig = EngineConfig(), **overrides: object) -> "Engine":
        """Loads the model in ``model_dir``.  Keyword arguments override fields of ``engine_config``."""
        if overrides:
            engine_config = EngineConfig(**{**engine_config.__dict__, **overrides})  # type: ignore[arg-type]
        _require_device(engine_config.device)
        config = load_config(model_dir)
        plan = config.to_plan()
        tensors = load_weights(model_dir, config, plan)
        return cls(plan, tensors, engine_config, config)

    @classmethod
    def random(cls, config: ArchitectureConfig | dict, seed: int, std: float = 0.02, engine_config: EngineConfig = EngineConfig(),
               **overrides: object) -> "Engine":
        """An engine with random weights made in memory (no model folder): ``config`` is a typed
        configuration or a raw ``config.json`` mapping.  The tensors are those the random-weights
        mode would write for the same configuration, seed and spread."""
        from ..config.registry import config_from_dict
        from ..parts.model import plan_tensor_decls
        from ..weights.random_init import random_tensors

        if overrides:
            engine_config = EngineConfig(**{**engine_config.__dict__, **overrides})  # type: ignore[arg-type]
        _require_device(engine_config.device)
        typed = config_from_dict(config) if isinstance(config, dict) else config
        plan = typed.to_plan()
        storage = "float32" if resolve_dtype(engine_config.dtype) == torch.float32 else "bfloat16"
        named = random_tensors(typed, seed=seed, std=std, dtype=storage)
        tensors = {key: named[typed.checkpoint_names(*key)[0]].reshape(decl.shape) for key, decl in plan_tensor_decls(plan).items()}
        return cls(plan, tensors, engine_config, typed)

    # ------------------------------------------------------------- step-level interface
    @property
    def vocab_size(self) -> int:
        return self.plan.vocab_size

    def new_request_number(self) -> int:
        """A number no other request of this engine has had (generators name their requests with it)."""
        self._request_numbers += 1
        return self._request_numbers - 1

    def admit(self, request_id: object) -> None:
        self.cache.admit(request_id)

    def release(self, request_id: object) -> None:
        self.cache.release(request_id)

    def step(self, entries: Sequence[StepEntry], previous_sampled: torch.Tensor | None = None) -> torch.Tensor:
        return self.executor.step(entries, previous_sampled)
