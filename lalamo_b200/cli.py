"""The command line, in the reference's manner (``lalamo/main.py``): ``chat``, ``convert`` and
``list-models`` keep the reference's option names and meanings; ``generate`` (token ids in, token
ids out), ``random-weights`` and ``trace`` are this engine's own.
"""

from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path
from typing import Annotated, Optional

from rich.console import Console
from rich.table import Table
from typer import Argument, Exit, Option, Typer

from .model_registry import PRESETS, ModelRegistry

app = Typer(add_completion=False, pretty_exceptions_show_locals=False, no_args_is_help=True)
console = Console()
err_console = Console(stderr=True)


def _error(message: str) -> None:
    err_console.print(f"[red]Error:[/red] {message}")
    raise Exit(1)


def _parse_ids(text: str) -> list[int]:
    return [int(item) for item in text.replace(",", " ").split()]


@app.command(name="list-models", help="List the supported models.")
def list_models(
    plain: Annotated[bool, Option(help="Only list repo names without fancy formatting.")] = False,
) -> None:
    specs = ModelRegistry.build().sorted_specs()
    if plain:
        for spec in specs:
            console.print(spec.description)
        return
    table = Table(show_header=True, header_style="bold", show_lines=True)
    for column in ("Vendor", "Family", "Size", "Origin"):
        table.add_column(column)
    for spec in specs:
        table.add_row(spec.vendor, spec.family, spec.size, spec.description)
    console.print(table)


@app.command(help="Generate token ids for prompts given as token ids (or as text, if the model folder has a tokenizer).")
def generate(
    model_path: Annotated[Optional[Path], Argument(help="Path to the model directory (with --random-weights: a directory holding config.json, or a config.json).",
                                                   metavar="MODEL_PATH", show_default="none: give --preset")] = None,
    prompt_ids: Annotated[Optional[str], Option(help="One prompt as comma- or space-separated token ids.")] = None,
    prompt_ids_file: Annotated[Optional[Path], Option(help="A file with one prompt (token ids) per line.")] = None,
    prompt: Annotated[Optional[str], Option(help="One prompt as text (needs tokenizer.json in the model directory); the reply is printed as text too.")] = None,
    max_tokens: Annotated[int, Option(help="Maximum number of tokens to generate per reply.")] = 64,
    temperature: Annotated[Optional[float], Option(help="Sampling temperature. Use 0 for greedy decoding.", show_default="model default")] = None,
    top_k: Annotated[Optional[int], Option(help="Keep the k most likely tokens.")] = None,
    top_p: Annotated[Optional[float], Option(help="Nucleus sampling threshold.")] = None,
    min_p: Annotated[Optional[float], Option(help="Drop tokens less likely than min_p times the most likely one.")] = None,
    repetition_penalty: Annotated[Optional[float], Option(help="Penalty on tokens already seen.")] = None,
    seed: Annotated[int, Option(help="Seed of the sampling random stream.")] = 0,
    dtype: Annotated[str, Option(help="Compute type: bfloat16 or float32.")] = "bfloat16",
    random_weights: Annotated[Optional[int], Option(help="Make random weights from this seed in memory instead of reading safetensors.", metavar="SEED")] = None,
    preset: Annotated[Optional[str], Option(help=f"With random weights: one of the shapes {sorted(PRESETS)} instead of MODEL_PATH.")] = None,
    std: Annotated[float, Option(help="Standard deviation of the random weights.")] = 0.02,
    spec: Annotated[Optional[str], Option(help="The model's name in `list-models`, whose default generation options apply if the folder brings none.")] = None,
    page_size: Annotated[int, Option(help="Tokens per cache page.")] = 16,
    max_cache_tokens: Annotated[int, Option(help="Tokens the cache holds for all live requests together.")] = 65536,
    max_batch_tokens: Annotated[int, Option(help="Tokens one step may run.")] = 2048,
    max_requests: Annotated[int, Option(help="Requests live at a time.")] = 64,
    chunk_size: Annotated[Optional[int], Option(help="Longest portion of one prompt in a step.", show_default="max-batch-tokens")] = None,
    stats: Annotated[bool, Option(help="Print scheduler statistics to standard error.")] = False,
) -> None:
    from dataclasses import replace

    from .engine.engine import EngineConfig
    from .language_model import LanguageModel

    if preset is not None and preset not in PRESETS:
        _error(f"unknown preset {preset!r}; known: {sorted(PRESETS)}")
    if (model_path is None) == (preset is None):
        _error("give MODEL_PATH or --preset (not both)")
    tokenizer = None
    prompts: list[list[int]] = []
    if prompt is not None:
        tokenizer_path = (model_path if model_path is not None and model_path.is_dir() else Path(".")) / "tokenizer.json"
        if model_path is None or not tokenizer_path.is_file():
            _error(f"--prompt needs {tokenizer_path if model_path is not None else 'a model directory with tokenizer.json'}; use --prompt-ids for models without a tokenizer")
        from tokenizers import Tokenizer

        tokenizer = Tokenizer.from_file(str(tokenizer_path))
        prompts.append(tokenizer.encode(prompt).ids)
    if prompt_ids is not None:
        prompts.append(_parse_ids(prompt_ids))
    if prompt_ids_file is not None:
        prompts += [_parse_ids(line) for line in prompt_ids_file.read_text().splitlines() if line.strip()]
    if not prompts:
        _error("give --prompt-ids, --prompt-ids-file or --prompt")
    engine_config = EngineConfig(dtype=dtype, page_size=page_size, max_tokens=max_cache_tokens, max_batch_tokens=max_batch_tokens, max_requests=max_requests)
    try:
        if preset is not None or random_weights is not None:
            model = LanguageModel.random(preset if preset is not None else model_path, random_weights or 0, std=std, engine_config=engine_config, spec=spec)
        else:
            model = LanguageModel.load(model_path, engine_config, spec=spec)
    except (FileNotFoundError, ValueError, RuntimeError) as error:
        _error(str(error))
    config = model.generation_config
    overrides = {"temperature": temperature, "top_k": top_k, "top_p": top_p, "min_p": min_p, "repetition_penalty": repetition_penalty}
    config = replace(config, **{key: value for key, value in overrides.items() if value is not None})
    results: dict[int, dict] = {}
    for sequence in model.generate_tokens_many(prompts, config, max_output_length=max_tokens, seed=seed, chunk_size=chunk_size):
        results[sequence.index] = {"index": sequence.index, "token_ids": sequence.token_ids, "finish_reason": sequence.finish_reason}
        if tokenizer is not None:
            results[sequence.index]["text"] = tokenizer.decode(sequence.token_ids)
    for index in sorted(results):
        print(json.dumps(results[index]))
    if stats:
        executor = model.engine.executor
        err_console.print(f"steps run: {executor.steps_run}, tokens run: {executor.tokens_run}, replayed from graphs: {executor.graph_replays}")


@app.command(help="Chat with a model (needs tokenizer.json in the model directory).")
def chat(
    model_path: Annotated[Path, Argument(help="Path to the model directory.", metavar="MODEL_PATH")],
    message: Annotated[Optional[str], Option(help="Message for non-interactive mode.", show_default="None, run interactively")] = None,
    max_tokens: Annotated[int, Option(help="Maximum number of tokens to generate per reply.")] = 8192,
    temperature: Annotated[Optional[float], Option(help="Sampling temperature. Use 0 for greedy decoding.", show_default="model default")] = None,
) -> None:
    from dataclasses import replace

    from .language_model import LanguageModel

    tokenizer_path = model_path / "tokenizer.json"
    if not tokenizer_path.is_file():
        _error(f"{tokenizer_path} does not exist; use `generate --prompt-ids` for models without a tokenizer")
    from tokenizers import Tokenizer

    tokenizer = Tokenizer.from_file(str(tokenizer_path))
    model = LanguageModel.load(model_path)
    config = model.generation_config
    if temperature is not None:
        config = replace(config, temperature=temperature)

    def reply(text: str, turn: int) -> None:
        prompt = tokenizer.encode(text).ids
        produced: list[int] = []
        shown = ""
        for token in model.stream_tokens(prompt, config, max_output_length=max_tokens, seed=turn + 1):
            produced.append(token)
            decoded = tokenizer.decode(produced)
            console.print(decoded[len(shown):], end="")
            shown = decoded
        console.print()

    if message is not None:
        reply(message, 0)
        return
    turn = 0
    while True:
        try:
            text = console.input("[cyan]user> [/cyan]")
        except (EOFError, KeyboardInterrupt):
            return
        console.print("[red]assistant> [/red]", end="")
        reply(text, turn)
        turn += 1


@app.command(help="Import a local Hugging Face model directory and write it in this engine's layout.")
def convert(
    model_repo: Annotated[str, Argument(help="A local model directory (there is no network), or a repo name from `list-models` whose files are at --source-dir.", metavar="MODEL_REPO")],
    dtype: Annotated[Optional[str], Option(help="Dtype to use for activations and non-quantized weights.", show_default="bfloat16")] = None,
    output_dir: Annotated[Optional[Path], Option(help="Directory to save the converted model to.", show_default="models/<model_name>")] = None,
    source_dir: Annotated[Optional[Path], Option(help="Where the repo's files are, if MODEL_REPO is a repo name.")] = None,
    overwrite: Annotated[bool, Option(help="Overwrite existing model files.")] = False,
) -> None:
    import torch

    from .config.registry import load_config
    from .weights.loader import load_weights
    from .weights.safetensors_io import write_safetensors

    source = Path(model_repo) if Path(model_repo).is_dir() else source_dir
    if source is None or not source.is_dir():
        known = ModelRegistry.build().repo_to_model
        hint = "" if model_repo not in known else " (a known repo; give its local files with --source-dir)"
        _error(f'Model "{model_repo}" not found as a directory{hint}.')
    name = Path(model_repo).name
    output_dir = output_dir or Path("models") / name
    if output_dir.exists() and any(output_dir.iterdir()):
        if not overwrite:
            _error(f"{output_dir} is not empty; pass --overwrite")
        shutil.rmtree(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    target = {"bfloat16": torch.bfloat16, "float32": torch.float32, None: torch.bfloat16}.get(dtype)
    if target is None:
        _error(f"unknown dtype {dtype!r}; known: bfloat16, float32")
    try:
        config = load_config(source)
        tensors = load_weights(source, config)
    except (FileNotFoundError, ValueError) as error:
        _error(str(error))
    from .parts import plan_tensor_decls

    shape_hook = getattr(config, "checkpoint_shape", lambda path, local, shape: shape)
    decls = plan_tensor_decls(config.to_plan())
    named = {}
    for (path, local), tensor in tensors.items():
        # only what the parts declare as matrices takes the target type; vectors (norm scales, taps, biases) and tables keep theirs
        keep = tensor.dtype == torch.int32 or decls[(path, local)].role != "matrix"
        named[config.checkpoint_names(path, local)[0]] = (tensor if keep else tensor.to(target)).reshape(shape_hook(path, local, tuple(tensor.shape)))
    write_safetensors(output_dir / "model.safetensors", named, metadata={"format": "pt"})
    shutil.copy(source / "config.json", output_dir / "config.json")
    for extra in ("generation_config.json", "tokenizer.json", "tokenizer_config.json", "chat_template.jinja"):
        if (source / extra).is_file():
            shutil.copy(source / extra, output_dir / extra)
    console.print(f"saved {len(named)} tensors to {output_dir}")


@app.command(name="random-weights", help="Write a model folder (config.json, model.safetensors) with random weights.")
def random_weights(
    config: Annotated[str, Argument(help=f"A config.json, or one of the presets {sorted(PRESETS)}.", metavar="CONFIG")],
    output_dir: Annotated[Path, Option(help="Directory to write the model folder to.")],
    seed: Annotated[int, Option(help="Seed of the weights.")] = 0,
    std: Annotated[float, Option(help="Standard deviation of the weights.")] = 0.02,
    dtype: Annotated[str, Option(help="Storage type of the matrices: bfloat16 or float32.")] = "bfloat16",
) -> None:
    from .weights.random_init import write_random_model

    raw = PRESETS[config] if config in PRESETS else json.loads(Path(config).read_text())
    try:
        folder = write_random_model(output_dir, raw, seed=seed, std=std, dtype=dtype)
    except ValueError as error:
        _error(str(error))
    console.print(f"wrote {folder}")


@app.command(help="Replay a trace of steps (JSON lines on standard input) and write logits; see bin/trace_run.")
def trace(
    model: Annotated[Path, Option(help="Folder with config.json and model.safetensors.")],
    out: Annotated[Path, Option(help="Folder that receives <step>.f32 files.")],
    max_tokens: Annotated[int, Option(help="Tokens the live requests hold at most.")],
    dtype: Annotated[str, Option(help="bfloat16 or float32.")] = "bfloat16",
    poison_freed: Annotated[bool, Option(help="Overwrite pages and state slots with NaN when they are given back (for tests).")] = False,
) -> None:
    from .engine.trace import run

    sys.exit(run(str(model), dtype, str(out), max_tokens, poison_freed))


def main() -> None:
    app()


if __name__ == "__main__":
    main()
