"""The Python entry point, in the reference's manner.

``LanguageModel.load(path)`` then ``generate_tokens`` / ``stream_tokens`` /
``generate_tokens_many`` mirror ``lalamo/models/language_model.py:274-287``, ``:444-568`` and
``lalamo/inference/batch_scheduler.py:770-778``.  Token ids go in and come out as Python lists on the
host; outputs are trimmed after the first stop token, which is kept
(``language_model.py:142-150``).
"""

from __future__ import annotations

import json
from dataclasses import replace
from pathlib import Path
from typing import Callable, Iterator, Sequence

from .engine.engine import Engine, EngineConfig
from .engine.generation import GeneratedSequence, Generator
from .model_registry import PRESETS, ModelRegistry
from .sampling.policy import GenerationConfig

__all__ = ["LanguageModel", "load_generation_config"]


def _merge_token_ids(*sources: int | Sequence[int] | None) -> tuple[int, ...]:
    merged: set[int] = set()
    for source in sources:
        if source is None:
            continue
        if isinstance(source, int):
            merged.add(source)
        else:
            merged.update(int(token) for token in source)
    return tuple(sorted(merged))


def load_generation_config(model_dir: str | Path | None, eos_token_id: int | Sequence[int] | None, spec: str | None = None) -> GenerationConfig:
    """The model's default generation options, as the reference settles them at import
    (``lalamo/model_import/common.py:251-271``): ``generation_config.json`` if the folder has one
    (its sampling keys are taken over, ``lalamo/model_import/huggingface_generation_config.py:13-78``);
    else the options the model registry gives the model (``lalamo/model_import/model_specs/lfm2.py:30,58``),
    found by ``spec`` (a repository name) or by the folder's name; else neutral options.  In every case
    the stop tokens are merged with ``config.json``'s ``eos_token_id``."""
    stop = _merge_token_ids(eos_token_id)
    path = Path(model_dir) / "generation_config.json" if model_dir is not None else None
    if path is None or not path.is_file():
        registry = ModelRegistry.build()
        known = registry.find(spec) if spec is not None else (registry.find(Path(model_dir).resolve().name) if model_dir is not None else None)
        if spec is not None and known is None:
            raise ValueError(f"{spec!r} is not a known model; known: {sorted(registry.repo_to_model)}")
        if known is None:
            return GenerationConfig(stop_token_ids=stop)
        return replace(known.generation_config, stop_token_ids=_merge_token_ids(stop, known.generation_config.stop_token_ids))
    raw = json.loads(path.read_text())
    return GenerationConfig(
        stop_token_ids=_merge_token_ids(stop, raw.get("eos_token_id")),
        temperature=raw.get("temperature"),
        top_k=raw.get("top_k"),
        top_p=raw.get("top_p"),
        min_p=raw.get("min_p"),
        repetition_penalty=raw.get("repetition_penalty"),
    )


class LanguageModel:
    def __init__(self, engine: Engine, generation_config: GenerationConfig) -> None:
        self.engine = engine
        self.generation_config = generation_config

    @classmethod
    def load(cls, path: str | Path, engine_config: EngineConfig = EngineConfig(), spec: str | None = None, **overrides: object) -> "LanguageModel":
        """Loads the model folder ``path`` (``config.json`` + safetensors [+ ``generation_config.json``]).
        ``spec`` names the model in the registry (``"LiquidAI/LFM2-1.2B"``) whose default generation
        options apply when the folder brings none; without it the folder's name is looked up."""
        engine = Engine.load(path, engine_config, **overrides)
        eos = getattr(engine.architecture_config, "eos_token_id", None)
        return cls(engine, load_generation_config(path, eos, spec))

    @classmethod
    def random(cls, config: str | Path | dict, seed: int, std: float = 0.02, engine_config: EngineConfig = EngineConfig(),
               spec: str | None = None, **overrides: object) -> "LanguageModel":
        """A model with random weights made in memory.  ``config``: the name of a preset shape
        (``"lfm2-1.2b"`` ...), a ``config.json`` file, a folder holding one, or the mapping itself."""
        if isinstance(config, dict):
            raw = config
        elif isinstance(config, str) and config in PRESETS:
            raw = PRESETS[config]
        else:
            file = Path(config) / "config.json" if Path(config).is_dir() else Path(config)
            if not file.is_file():
                raise FileNotFoundError(f"{config!r} is neither a preset ({sorted(PRESETS)}) nor a config.json or a folder with one")
            raw = json.loads(file.read_text())
        engine = Engine.random(raw, seed, std, engine_config, **overrides)
        eos = getattr(engine.architecture_config, "eos_token_id", None)
        folder = Path(config) if not isinstance(config, dict) and Path(str(config)).is_dir() else None
        return cls(engine, load_generation_config(folder, eos, spec))

    # ------------------------------------------------------------------- generation
    def _config(self, generation_config: GenerationConfig | None, eos_token_ids: Sequence[int] | None) -> GenerationConfig:
        config = self.generation_config if generation_config is None else generation_config
        if generation_config is not None and not config.stop_token_ids:
            config = replace(config, stop_token_ids=self.generation_config.stop_token_ids)
        if eos_token_ids is not None:
            config = replace(config, stop_token_ids=tuple(int(token) for token in eos_token_ids))
        return config

    def generate_tokens_many(
        self,
        prompt_token_ids: Sequence[Sequence[int]],
        generation_config: GenerationConfig | Sequence[GenerationConfig] | None = None,
        max_output_length: int = 8192,
        eos_token_ids: Sequence[int] | None = None,
        seed: int = 0,
        chunk_size: int | None = None,
        on_step: Callable[[Generator], None] | None = None,
    ) -> Iterator[GeneratedSequence]:
        """Continuous batching over any number of prompts; sequences are yielded as they finish.
        ``chunk_size`` caps the portion of one prompt in a step; ``on_step`` is called with the
        generator after every step (for statistics)."""
        if max_output_length < 1:
            raise ValueError("max_output_length must be at least 1.")
        if generation_config is None or isinstance(generation_config, GenerationConfig):
            configs: GenerationConfig | list[GenerationConfig] = self._config(generation_config, eos_token_ids)
        else:
            configs = [self._config(config, eos_token_ids) for config in generation_config]
        generator = Generator(self.engine, seed=seed, chunk_size=chunk_size)
        yield from generator.generate_many(prompt_token_ids, configs, max_output_length, on_step)

    def generate_tokens(
        self,
        prompt_token_ids: Sequence[Sequence[int]],
        generation_config: GenerationConfig | None = None,
        prompt_lengths_without_padding: Sequence[int] | None = None,
        max_output_length: int = 8192,
        eos_token_ids: Sequence[int] | None = None,
        seed: int = 0,
    ) -> list[list[int]]:
        """Generated token ids for every prompt, in the order of the prompts.  Rows of a padded batch
        are cut to ``prompt_lengths_without_padding`` first."""
        prompts = [list(row) for row in prompt_token_ids]
        if prompt_lengths_without_padding is not None:
            prompts = [row[: int(length)] for row, length in zip(prompts, prompt_lengths_without_padding)]
        results: list[list[int]] = [[] for _ in prompts]
        for sequence in self.generate_tokens_many(prompts, generation_config, max_output_length, eos_token_ids, seed):
            results[sequence.index] = sequence.token_ids
        return results

    def stream_tokens(
        self,
        prompt_token_ids: Sequence[int],
        generation_config: GenerationConfig | None = None,
        max_output_length: int = 8192,
        eos_token_ids: Sequence[int] | None = None,
        seed: int = 0,
    ) -> Iterator[int]:
        """Yields the tokens of one reply as they are sampled."""
        config = self._config(generation_config, eos_token_ids)
        generator = Generator(self.engine, seed=seed)
        try:
            request = generator.add(prompt_token_ids, config.default_policy(), config.stop_token_ids, max_output_length, key_number=0)
            sent = len(request.prompt)
            while generator.has_work():
                generator.step()
                while sent < len(request.tokens) - request.unresolved:  # tokens whose ids have reached the host
                    yield request.tokens[sent]
                    sent += 1
        finally:
            generator.close()  # a consumer that stops early leaves nothing in the cache
