#!/usr/bin/env python3
"""Benchmark of the flagship serving step: decoding with the LFM2-1.2B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests at a context of 4,096 tokens, random bfloat16
weights (N(0, 0.02), seed 2), synthetic token ids.  One JSON line is printed:

* ``value``: decoded tokens a second, timed on the device with CUDA events around K steps;
* ``e2e``: the same through the Python entry point (scheduler, step function, sampler), with the
  step's description copied from pinned host memory and the sampled token ids read back every step;
* ``prefill``: one 2,048-token prompt in one step, with its fraction of the measured bf16 peak;
* ``roofline``: the decode step's bytes (every weight once + the live requests' cache) over its time,
  against the measured copy bandwidth;
* ``points``: decoding at batch 1 and 64.

Inputs are larger than L2 (2.3 GB of weights are read every step), so no L2 flush is needed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at batch 8, context 4096 (LFM2-1.2B shape)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as stream:
                raw = json.load(stream)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(raw.get(key), (int, float)) and raw[key] > 0:
                    peaks[key] = float(raw[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.process: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        assert self.process is not None and self.process.stdout is not None
        for line in self.process.stdout:
            fields = [field.strip() for field in line.split(",")]
            if len(fields) == 6:
                self.samples.append(fields)

    def stop(self) -> dict:
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        clocks = [int(s[0]) for s in self.samples if s[0].isdigit()]
        maxima = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for index, name in enumerate(names) if any(s[2 + index] == "Active" for s in self.samples)]
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": reasons, "samples": len(self.samples)}


def reference_arm() -> int:
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import lalamo  # noqa: F401
    except Exception as error:  # the reference needs jax and equinox, which cannot be installed offline
        print(json.dumps({"impl": "reference", "unavailable": f"import lalamo fails: {type(error).__name__}: {error}"[:300]}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "lalamo imports, but no JAX GPU backend is installed to run it on a B200"}))
    return 0


PRESET_SEEDS = {"lfm2-1.2b": 2, "lfm2-350m": 3, "lfm2-700m": 4}


def build_engine(max_tokens: int, max_requests: int, max_batch_tokens: int, seed: int | None = None, cuda_graphs: bool = True, preset: str = "lfm2-1.2b",
                 page_size: int = 16):
    import torch

    from lalamo_b200.config import config_from_dict
    from lalamo_b200.engine import Engine, EngineConfig
    from lalamo_b200.model_registry import PRESETS

    config = config_from_dict(PRESETS[preset])
    engine = Engine.random(config, seed=PRESET_SEEDS[preset] if seed is None else seed, std=0.02,
                           engine_config=EngineConfig(dtype="bfloat16", page_size=page_size, max_tokens=max_tokens, max_requests=max_requests,
                                                      max_batch_tokens=max_batch_tokens, cuda_graphs=cuda_graphs))
    torch.cuda.empty_cache()
    return engine, config


def fill_cache_randomly(engine, generator) -> None:
    """Synthetic cache contents: random keys, values and convolution states."""
    import torch

    for pages in list(engine.cache.k_pages.values()) + list(engine.cache.v_pages.values()):
        pages.copy_(torch.randn(pages.shape, device=pages.device, generator=generator, dtype=torch.float32).to(pages.dtype))
    for state in engine.cache.states.values():
        state.copy_((0.1 * torch.randn(state.shape, device=state.device, generator=generator, dtype=torch.float32)).to(state.dtype))


def prompt_flops(config, tokens: int, wanted_rows: int = 1) -> float:
    """Floating-point operations of reading a prompt of `tokens` tokens whole: every product of every
    layer, causal attention (a multiply-add per query, visible key and channel, for scores and for
    values), and the read-out of the wanted rows."""
    hidden, ffn, heads, groups, head_dim = config.hidden_size, config.ffn_dim, config.num_attention_heads, config.num_key_value_heads, config.head_dim
    attention_layers = sum(kind == "full_attention" for kind in config.layer_types)
    conv_layers = len(config.layer_types) - attention_layers
    per_token = conv_layers * 2 * (3 * hidden * hidden + hidden * hidden)
    per_token += attention_layers * 2 * ((heads + 2 * groups) * head_dim * hidden + heads * head_dim * hidden)
    per_token += len(config.layer_types) * 2 * 3 * hidden * ffn
    return per_token * tokens + attention_layers * 4 * heads * head_dim * tokens * (tokens + 1) / 2 + 2 * hidden * config.vocab_size * wanted_rows


def time_decode(engine, batch: int, context: int, steps: int, warmup: int) -> dict:
    """Device-timed decode steps of `batch` requests whose contexts end near `context` tokens: K steps
    between two synchronisations, an event after every step (their differences give the median)."""
    import torch

    from lalamo_b200 import ops
    from lalamo_b200.engine import StepEntry
    from lalamo_b200.sampling import GenerationConfig, SampleRow, Sampler

    start_length = context - steps - warmup
    names = [f"bench{index}" for index in range(batch)]
    for name in names:
        engine.admit(name)
        engine.cache.reserve(name, start_length)
        engine.cache.commit(name, start_length)
    sampler = Sampler(engine.cache, engine.vocab_size, engine.runtime.device)
    policy = GenerationConfig(temperature=0.0).default_policy()
    rows = [SampleRow(policy, (0, 0), 0) for _ in names]
    tokens = [1 + index for index in range(batch)]
    in_flight = None

    def one_step() -> None:
        # As the generation loop does while requests only decode: the step takes the ids of the step
        # before from the device, and that step's ids are awaited on the host after this one's launch.
        nonlocal tokens, in_flight
        if in_flight is None:
            entries = [StepEntry(name, [token], [0]) for name, token in zip(names, tokens)]
            logits = engine.step(entries)
        else:
            entries = [StepEntry(name, [0], [0], row) for row, name in enumerate(names)]
            logits = engine.step(entries, in_flight.device)
        launched = sampler.sample_async(logits, rows)
        if in_flight is not None:
            tokens = in_flight.wait()
        in_flight = launched

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    bytes_read = engine.model.weight_bytes() + sum(engine.cache.bytes_held(name) for name in names)
    ops.reset_launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for index in range(steps):
        one_step()
        marks[index + 1].record()
    torch.cuda.synchronize()
    tokens = in_flight.wait()
    launches = ops.launch_count()  # launches replayed from CUDA graphs are counted by the executor
    milliseconds = marks[0].elapsed_time(marks[-1]) / steps
    median = statistics.median(marks[index].elapsed_time(marks[index + 1]) for index in range(steps))
    for name in names:
        engine.release(name)
    return {"ms_per_step": milliseconds, "ms_median": median, "tokens_per_s": batch / (milliseconds / 1e3), "tokens_per_s_median": batch / (median / 1e3),
            "bytes_per_step": bytes_read, "launches": launches}


def time_prefill(engine, config, tokens: int, steps: int, warmup: int) -> dict:
    import torch

    from lalamo_b200.engine import StepEntry

    generator = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, engine.vocab_size, (tokens,), generator=generator).tolist()
    times = []
    for iteration in range(warmup + steps):
        engine.admit("prefill")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.step([StepEntry("prefill", prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.release("prefill")
        if iteration >= warmup:
            times.append(begin.elapsed_time(end))
    milliseconds = statistics.median(times)
    return {"ms": milliseconds, "tokens": tokens, "value": tokens / (milliseconds / 1e3), "flops": prompt_flops(config, tokens)}


def time_prompts(model, config, count: int, tokens: int, rounds: int = 2, max_batch_tokens: int | None = None) -> dict:
    """`count` prompts of `tokens` tokens read under the scheduler's token budget (each request generates one
    token, so it is finished when its prompt is read); device-timed from the first step to the last."""
    import torch

    from lalamo_b200.engine.generation import Generator
    from lalamo_b200.sampling import GenerationConfig

    random = torch.Generator().manual_seed(13)
    policy = GenerationConfig(temperature=0.0).default_policy()
    times = []
    for _ in range(rounds):
        generator = Generator(model.engine, seed=0, max_batch_tokens=max_batch_tokens)
        for index in range(count):
            generator.add(torch.randint(0, model.engine.vocab_size, (tokens,), generator=random).tolist(), policy, (), max_new_tokens=1, key_number=index)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        steps = 0
        while generator.has_work():
            generator.step()
            steps += 1
        end.record()
        torch.cuda.synchronize()
        generator.close()
        times.append(begin.elapsed_time(end))
    milliseconds = min(times)
    return {"ms": milliseconds, "value": count * tokens / (milliseconds / 1e3), "steps": steps, "flops": count * prompt_flops(config, tokens)}


def time_e2e(model, batch: int, context: int, steps: int, warmup: int) -> dict:
    """Decode steps through the Python entry point: host token ids in, host token ids out."""
    import torch

    from lalamo_b200.engine.generation import Generator
    from lalamo_b200.sampling import GenerationConfig

    generator = Generator(model.engine, seed=0)
    # Prompts are read in portions under the token budget, so requests start decoding a few steps apart;
    # the margin keeps the longest one inside the context, and nobody finishes inside the timed region.
    prompt_length = context - steps - warmup - 32
    random = torch.Generator().manual_seed(9)
    policy = GenerationConfig(temperature=0.0).default_policy()
    for index in range(batch):
        prompt = torch.randint(0, model.engine.vocab_size, (prompt_length,), generator=random).tolist()
        generator.add(prompt, policy, (), max_new_tokens=steps + warmup + 4096, key_number=index)
    while any(request.pending > 1 for request in list(generator.scheduler.waiting) + generator.scheduler.running) or generator.scheduler.waiting:
        generator.step()
    for _ in range(warmup):
        generator.step()
    torch.cuda.synchronize()
    h2d = d2h = 0
    laps = []
    started = time.perf_counter()
    for _ in range(steps):
        lap = time.perf_counter()
        replays = model.engine.executor.graph_replays
        generator.step()
        laps.append((time.perf_counter() - lap, model.engine.executor.graph_replays - replays))
        h2d += model.engine.executor.last_h2d_bytes
        d2h += generator.sampler.last_d2h_bytes
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    if os.environ.get("BENCH_VERBOSE"):
        print("e2e step times (ms, * = not a graph replay):", " ".join(f"{lap * 1e3:.2f}{'' if replayed else '*'}" for lap, replayed in laps), file=sys.stderr)
    generator.close()
    return {"value": batch * steps / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d // steps, "d2h_bytes_per_step": d2h // steps}


def shape_record(config, preset: str) -> dict:
    return {"model": f"{preset.upper()} shape", "layers": config.num_hidden_layers, "layers_of_config": 16, "hidden": config.hidden_size,
            "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim, "ffn": config.ffn_dim,
            "vocab": config.vocab_size, "conv_taps": config.conv_kernel_size,
            "attention_layers": sum(kind == "full_attention" for kind in config.layer_types)}


def run_mixed(arguments, peaks: dict, peak_source: str) -> int:
    """LFM2-350M shape: 64 requests with prompts of 128 to 2,048 random tokens generate 256 tokens each
    through `LanguageModel.generate_tokens_many` (admission, prompts in portions beside decoding, greedy
    sampling, host token ids in and out); wall clock, best of the rounds after the first."""
    import numpy as np
    import torch

    from lalamo_b200.language_model import LanguageModel
    from lalamo_b200.sampling import GenerationConfig

    requests, new_tokens = arguments.mixed_requests, arguments.mixed_new_tokens
    lengths = np.random.default_rng(3).integers(128, 2049, size=requests)
    pool = int(sum(-(-(int(n) + new_tokens) // 16) * 16 for n in lengths)) if arguments.pool_tokens == 0 else arguments.pool_tokens
    engine, config = build_engine(max_tokens=pool, max_requests=requests, max_batch_tokens=arguments.max_batch_tokens, preset="lfm2-350m")
    model = LanguageModel(engine, GenerationConfig(temperature=0.0))
    random = np.random.default_rng(4)
    clocks = ClockSampler()
    clocks.start()
    rounds = []
    for _ in range(3):   # the first round records the graphs of the steps' shapes
        prompts = [random.integers(0, engine.vocab_size, size=int(n)).tolist() for n in lengths]
        laps, occupancy, preemptions, host = [], [0.0], [0], [{}]
        last = [time.perf_counter()]

        def on_step(generator) -> None:
            now = time.perf_counter()
            laps.append(now - last[0])
            last[0] = now
            occupancy[0] = max(occupancy[0], 1.0 - engine.cache.free_pages() / engine.cache.num_pages)
            preemptions[0] = generator.scheduler.stats.preemptions
            host[0] = generator.host_seconds

        steps_before, replays_before = engine.executor.steps_run, engine.executor.graph_replays
        torch.cuda.synchronize()
        begin = time.perf_counter()
        last[0] = begin
        finished = list(model.generate_tokens_many(prompts, GenerationConfig(temperature=0.0), max_output_length=new_tokens, eos_token_ids=[], on_step=on_step))
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        produced = sum(len(sequence.token_ids) for sequence in finished)
        rounds.append({"seconds": seconds, "produced": produced, "laps": laps, "occupancy": occupancy[0], "preemptions": preemptions[0], "host": dict(host[0]),
                       "steps": engine.executor.steps_run - steps_before, "replays": engine.executor.graph_replays - replays_before})
    best = min(rounds[1:], key=lambda r: r["seconds"])
    prompt_tokens = int(lengths.sum())
    print(json.dumps({
        "metric": "tokens/s of 64 mixed requests through the scheduler (LFM2-350M shape)", "value": round((best["produced"] + prompt_tokens) / best["seconds"], 1),
        "unit": "tokens/s (prompt + generated)", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "impl": "ours",
        "data": "synthetic: random bf16 weights N(0,0.02) seed 3, prompt lengths default_rng(3).integers(128, 2049), random token ids",
        "generated_tokens_per_s": round(best["produced"] / best["seconds"], 1), "prompt_tokens_per_s": round(prompt_tokens / best["seconds"], 1),
        "seconds": round(best["seconds"], 4), "requests": requests, "prompt_tokens": prompt_tokens, "generated_tokens": best["produced"],
        "steps": best["steps"], "graph_replays": best["replays"], "ms_per_step_mean": round(1e3 * statistics.mean(best["laps"]), 3),
        "ms_per_step_median": round(1e3 * statistics.median(best["laps"]), 3), "peak_page_occupancy": round(best["occupancy"], 3),
        "preemptions": best["preemptions"], "host_ms_per_step": {name: round(1e3 * seconds / max(1, best["steps"]), 4) for name, seconds in best["host"].items()},
        "config": {**shape_record(config, "lfm2-350m"), "requests": requests, "new_tokens": new_tokens, "max_batch_tokens": arguments.max_batch_tokens,
                   "pool_tokens": pool, "page_size": 16, "peaks": peak_source},
        "clocks": clocks.stop(),
    }))
    return 0


def run_long(arguments, peaks: dict, peak_source: str) -> int:
    """LFM2-700M shape: prompts of 16,384 random tokens at batch 1 and 8 read through the scheduler under a
    token budget of 2,048 and of 8,192 tokens a step, pages of 16 keys, then 512 decode steps; device-timed."""
    import torch

    from lalamo_b200.engine.generation import Generator
    from lalamo_b200.language_model import LanguageModel
    from lalamo_b200.sampling import GenerationConfig

    prompt_tokens, decode_steps = arguments.long_prompt, arguments.long_decode
    engine, config = build_engine(max_tokens=8 * (prompt_tokens + decode_steps + 64), max_requests=8, max_batch_tokens=8192, preset="lfm2-700m", page_size=16)
    model = LanguageModel(engine, GenerationConfig(temperature=0.0))
    peak_flops = (peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]) * 1e12
    policy = GenerationConfig(temperature=0.0).default_policy()
    random = torch.Generator().manual_seed(21)
    clocks = ClockSampler()
    clocks.start()
    results = {}
    for batch in (1, 8):
        for budget in (2048, 8192):
            best = None
            for _ in range(3):  # the later rounds find their graphs recorded; the fastest round counts, per phase
                generator = Generator(engine, seed=0, max_batch_tokens=budget)
                requests = [generator.add(torch.randint(0, engine.vocab_size, (prompt_tokens,), generator=random).tolist(), policy, (),
                                          max_new_tokens=decode_steps + 1, key_number=index) for index in range(batch)]
                torch.cuda.synchronize()
                marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                marks[0].record()
                prefill_steps = 0
                while any(request.num_generated == 0 for request in requests):
                    generator.step()
                    prefill_steps += 1
                marks[1].record()
                bytes_read = engine.model.weight_bytes()
                decoded = 0
                while generator.has_work():
                    if decoded == decode_steps // 2:
                        bytes_read += sum(engine.cache.bytes_held(request.request_id) for request in generator.scheduler.running)
                    generator.step()
                    decoded += 1
                marks[2].record()
                torch.cuda.synchronize()
                generator.close()
                prefill_ms, decode_ms = marks[0].elapsed_time(marks[1]), marks[1].elapsed_time(marks[2])
                # the faster of the two rounds, for the prompts and for the decoding separately
                best = (prefill_ms, decode_ms, prefill_steps, decoded, bytes_read) if best is None else (
                    min(best[0], prefill_ms), min(best[1], decode_ms), prefill_steps, decoded, bytes_read)
            prefill_ms, decode_ms, prefill_steps, decoded, bytes_read = best
            flops = batch * prompt_flops(config, prompt_tokens)
            key = f"b{batch}_budget{budget}"
            results[f"prefill_{key}_tokens_per_s"] = round(batch * prompt_tokens / (prefill_ms / 1e3), 1)
            results[f"prefill_{key}_ms"] = round(prefill_ms, 2)
            results[f"prefill_{key}_frac"] = round(flops / (prefill_ms / 1e3) / peak_flops, 4)
            results[f"prefill_{key}_steps"] = prefill_steps
            if budget == 2048:
                step_ms = decode_ms / decoded
                results[f"decode_b{batch}_tokens_per_s"] = round(batch / (step_ms / 1e3), 1)
                results[f"decode_b{batch}_ms_per_step"] = round(step_ms, 4)
                results[f"decode_b{batch}_frac"] = round(bytes_read / (step_ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
                results[f"decode_b{batch}_gb_per_step"] = round(bytes_read / 1e9, 3)
    print(json.dumps({
        "metric": "prefill and decode tokens/s, 16,384-token prompts at batch 1 and 8 (LFM2-700M shape)",
        "value": results["prefill_b1_budget8192_tokens_per_s"], "unit": "tokens/s (prefill, batch 1, 8,192 tokens a step)", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "impl": "ours", "data": "synthetic: random bf16 weights N(0,0.02) seed 4, random token ids",
        "tflop_per_prompt": round(prompt_flops(config, prompt_tokens) / 1e12, 2), **results,
        "config": {**shape_record(config, "lfm2-700m"), "prompt_tokens": prompt_tokens, "decode_steps": decode_steps, "page_size": 16, "peaks": peak_source},
        "clocks": clocks.stop(),
    }))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", default="lfm2-1.2b-decode", choices=["lfm2-1.2b-decode", "lfm2-350m-mixed", "lfm2-700m-long"],
                        help="lfm2-1.2b-decode (default): the decode step and its points; lfm2-350m-mixed: 64 requests with prompts of 128 to 2,048 "
                             "tokens and 256 new tokens through the scheduler; lfm2-700m-long: 16,384-token prompts at batch 1 and 8, then 512 decode steps")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points and the prefill (for quick runs)")
    parser.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel instead of replaying CUDA graphs")
    parser.add_argument("--skip-e2e", action="store_true", help="leave out the end-to-end measurement (for profiling runs)")
    parser.add_argument("--prefill-only", type=int, default=0, metavar="TOKENS", help="time only a prefill of TOKENS tokens (for profiling runs)")
    parser.add_argument("--requests", default="", metavar="N,PROMPT,NEW",
                        help="instead of the decode step: N requests with prompts of PROMPT random tokens generate NEW tokens each through "
                             "LanguageModel.generate_tokens_many (admission, prompts in portions beside decoding, greedy sampling); wall-clock time")
    parser.add_argument("--mixed-requests", type=int, default=64)
    parser.add_argument("--mixed-new-tokens", type=int, default=256)
    parser.add_argument("--max-batch-tokens", type=int, default=2048, help="the scheduler's token budget of --config lfm2-350m-mixed")
    parser.add_argument("--pool-tokens", type=int, default=0, help="cache pool of --config lfm2-350m-mixed in tokens (0: room for every request)")
    parser.add_argument("--long-prompt", type=int, default=16384)
    parser.add_argument("--long-decode", type=int, default=512)
    arguments = parser.parse_args()
    if arguments.impl == "reference":
        return reference_arm()
    if arguments.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {arguments.gpus} is not supported")
        return 2
    warmup = max(arguments.warmup, 3)
    steps = max(arguments.steps, 1)

    import torch

    from lalamo_b200.language_model import LanguageModel
    from lalamo_b200.sampling import GenerationConfig

    peaks, peak_source = load_peaks()
    if arguments.config == "lfm2-350m-mixed":
        return run_mixed(arguments, peaks, peak_source)
    if arguments.config == "lfm2-700m-long":
        return run_long(arguments, peaks, peak_source)
    if arguments.requests:
        requests, prompt_length, new_tokens = (int(part) for part in arguments.requests.split(","))
        engine, config = build_engine(max_tokens=requests * (prompt_length + new_tokens + 64), max_requests=max(requests, 2), max_batch_tokens=2048)
        model = LanguageModel(engine, GenerationConfig(temperature=0.0))
        generator = torch.Generator().manual_seed(3)
        seconds = []
        for _ in range(3):   # the first round records the decode graphs
            prompts = [torch.randint(0, engine.vocab_size, (prompt_length,), generator=generator).tolist() for _ in range(requests)]
            torch.cuda.synchronize()
            begin = time.perf_counter()
            finished = list(model.generate_tokens_many(prompts, GenerationConfig(temperature=0.0), max_output_length=new_tokens))
            torch.cuda.synchronize()
            seconds.append(time.perf_counter() - begin)
            produced = sum(len(sequence.token_ids) for sequence in finished)
        best = min(seconds[1:])
        print(json.dumps({"requests": requests, "prompt_tokens": prompt_length, "new_tokens": produced // requests, "seconds": round(best, 4),
                          "generated_tokens_per_s": round(produced / best, 1), "prompt_tokens_per_s": round(requests * prompt_length / best, 1),
                          "steps": engine.executor.steps_run, "graph_replays": engine.executor.graph_replays}))
        return 0
    peak_flops = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
    if arguments.prefill_only:
        engine, config = build_engine(max_tokens=arguments.prefill_only + 64, max_requests=2, max_batch_tokens=arguments.prefill_only)
        measured = time_prefill(engine, config, arguments.prefill_only, steps=steps, warmup=warmup)
        print(json.dumps({"prefill_only": True, "tokens": measured["tokens"], "ms": round(measured["ms"], 3), "value": round(measured["value"], 1),
                          "frac": round(measured["flops"] / (measured["ms"] / 1e3) / (peak_flops * 1e12), 4), "peaks": peak_source}))
        return 0
    batch, context = arguments.batch, arguments.context
    largest = 64 if not arguments.skip_points else batch
    engine, config = build_engine(max_tokens=largest * (context + 64), max_requests=max(largest, batch), max_batch_tokens=2048,
                                  cuda_graphs=not arguments.no_graphs)
    fill_cache_randomly(engine, torch.Generator(device="cuda").manual_seed(3))

    def fraction(measured: dict) -> float:
        return round(measured["bytes_per_step"] / (measured["ms_median"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)

    clocks = ClockSampler()   # samples until everything below has been measured
    clocks.start()
    time.sleep(0.25)  # a first sample before the timed region starts
    decode = time_decode(engine, batch, context, steps, warmup)
    model = LanguageModel(engine, GenerationConfig())
    e2e = {"value": None, "unit": "tokens/s"} if arguments.skip_e2e else time_e2e(model, batch, context, steps, warmup)
    points, prefill = {}, None
    if not arguments.skip_points:
        point_steps = max(50, min(steps, 200))
        for name, size in (("decode_b1", 1), ("decode_b64", 64)):
            measured = time_decode(engine, size, context, point_steps, warmup)
            points[name] = round(measured["tokens_per_s_median"], 1)
            points[f"{name}_ms"] = round(measured["ms_median"], 4)
            points[f"{name}_gb"] = round(measured["bytes_per_step"] / 1e9, 3)
            points[f"{name}_frac"] = fraction(measured)
        points["decode_b8_ms_median"] = round(decode["ms_median"], 4)
        points["decode_b8_frac_median"] = fraction(decode)
        if engine.executor.use_graphs:
            engine.executor.use_graphs = False   # the same step launched kernel by kernel
            measured = time_decode(engine, batch, context, point_steps, warmup)
            engine.executor.use_graphs = True
            points["decode_b8_no_graphs"] = round(measured["tokens_per_s_median"], 1)
            points["decode_b8_no_graphs_ms"] = round(measured["ms_median"], 4)
        measured = time_prefill(engine, config, 2048, steps=5, warmup=3)
        prefill = {"value": round(measured["value"], 1), "tokens": measured["tokens"], "ms": round(measured["ms"], 3),
                   "frac": round(measured["flops"] / (measured["ms"] / 1e3) / (peak_flops * 1e12), 4)}
        for name, count in (("prefill_b8", 8), ("prefill_b64", 64)):   # prompts of 2,048 tokens under the budget of 2,048 tokens a step
            measured = time_prompts(model, config, count, 2048)
            points[name] = round(measured["value"], 1)
            points[f"{name}_ms"] = round(measured["ms"], 2)
            points[f"{name}_frac"] = round(measured["flops"] / (measured["ms"] / 1e3) / (peak_flops * 1e12), 4)
    clock_record = clocks.stop()
    achieved = decode["bytes_per_step"] / (decode["ms_per_step"] / 1e3) / 1e9
    record = {
        "metric": METRIC if (batch, context) == (8, 4096) else f"decode tok/s at batch {batch}, context {context} (LFM2-1.2B shape)",
        "value": round(decode["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(decode["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random bf16 weights N(0,0.02) seed 2, random token ids, random cache contents",
        "impl": "ours",
        "config": {
            "model": "LFM2-1.2B shape", "global_batch": batch, "seq_len": context, "parallelism": "none (1 GPU)",
            "layers": config.num_hidden_layers, "layers_of_config": 16, "hidden": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim, "ffn": config.ffn_dim, "vocab": config.vocab_size,
            "conv_taps": config.conv_kernel_size, "attention_layers": sum(kind == "full_attention" for kind in config.layer_types),
            "page_size": 16, "l2": "inputs larger than L2 (2.3 GB of weights read per step)", "peaks": peak_source,
            "graphs": "off" if arguments.no_graphs else "on",
        },
        "e2e": {key: (round(value, 1) if isinstance(value, float) else value) for key, value in e2e.items()},
        "gpu_launches": decode["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "clocks": clock_record,
    }
    if prefill is not None:
        record["prefill"] = prefill
    if points:
        record["points"] = points
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
