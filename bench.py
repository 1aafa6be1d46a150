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


def build_engine(max_tokens: int, max_requests: int, max_batch_tokens: int, seed: int = 2, cuda_graphs: bool = True):
    import torch

    from lalamo_b200.config import config_from_dict
    from lalamo_b200.engine import Engine, EngineConfig
    from lalamo_b200.model_registry import PRESETS
    from lalamo_b200.parts import plan_tensor_decls
    from lalamo_b200.weights import random_tensors

    config = config_from_dict(PRESETS["lfm2-1.2b"])
    plan = config.to_plan()
    named = random_tensors(config, seed=seed, std=0.02, dtype="bfloat16")
    tensors = {}
    for (path, local), decl in plan_tensor_decls(plan).items():
        tensors[(path, local)] = named[config.checkpoint_names(path, local)[0]].reshape(decl.shape)
    engine = Engine(plan, tensors, EngineConfig(dtype="bfloat16", page_size=16, max_tokens=max_tokens, max_requests=max_requests,
                                                max_batch_tokens=max_batch_tokens, cuda_graphs=cuda_graphs), config)
    del named, tensors
    torch.cuda.empty_cache()
    return engine, config


def fill_cache_randomly(engine, generator) -> None:
    """Synthetic cache contents: random keys, values and convolution states."""
    import torch

    for pages in list(engine.cache.k_pages.values()) + list(engine.cache.v_pages.values()):
        pages.copy_(torch.randn(pages.shape, device=pages.device, generator=generator, dtype=torch.float32).to(pages.dtype))
    for state in engine.cache.states.values():
        state.copy_((0.1 * torch.randn(state.shape, device=state.device, generator=generator, dtype=torch.float32)).to(state.dtype))


def time_decode(engine, batch: int, context: int, steps: int, warmup: int) -> dict:
    """Device-timed decode steps of `batch` requests whose contexts end near `context` tokens."""
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

    def one_step() -> None:
        nonlocal tokens
        logits = engine.step([StepEntry(name, [token], [0]) for name, token in zip(names, tokens)])
        tokens = sampler.sample(logits, rows)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    bytes_read = engine.model.weight_bytes() + sum(engine.cache.bytes_held(name) for name in names)
    ops.reset_launch_count()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    launches = ops.launch_count()  # launches replayed from CUDA graphs are counted by the executor
    milliseconds = begin.elapsed_time(end) / steps
    for name in names:
        engine.release(name)
    return {"ms_per_step": milliseconds, "tokens_per_s": batch / (milliseconds / 1e3), "bytes_per_step": bytes_read, "launches": launches}


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
    hidden, ffn, heads, groups, head_dim = config.hidden_size, config.ffn_dim, config.num_attention_heads, config.num_key_value_heads, config.head_dim
    per_token = 0
    attention_layers = sum(kind == "full_attention" for kind in config.layer_types)
    conv_layers = len(config.layer_types) - attention_layers
    per_token += conv_layers * 2 * (3 * hidden * hidden + hidden * hidden)
    per_token += attention_layers * 2 * ((heads + 2 * groups) * head_dim * hidden + heads * head_dim * hidden)
    per_token += len(config.layer_types) * 2 * 3 * hidden * ffn
    flops = per_token * tokens + attention_layers * 4 * heads * head_dim * tokens * (tokens + 1) / 2 + 2 * hidden * config.vocab_size
    return {"ms": milliseconds, "tokens": tokens, "value": tokens / (milliseconds / 1e3), "flops": flops}


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
    for request in list(generator.scheduler.running):
        generator.scheduler.abort(request)
    return {"value": batch * steps / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d // steps, "d2h_bytes_per_step": d2h // steps}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points and the prefill (for quick runs)")
    parser.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel instead of replaying CUDA graphs")
    parser.add_argument("--skip-e2e", action="store_true", help="leave out the end-to-end measurement (for profiling runs)")
    parser.add_argument("--prefill-only", type=int, default=0, metavar="TOKENS", help="time only a prefill of TOKENS tokens (for profiling runs)")
    parser.add_argument("--requests", default="", metavar="N,PROMPT,NEW",
                        help="instead of the decode step: N requests with prompts of PROMPT random tokens generate NEW tokens each through "
                             "LanguageModel.generate_tokens_many (admission, prompts in portions beside decoding, greedy sampling); wall-clock time")
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
    if arguments.prefill_only:
        engine, config = build_engine(max_tokens=arguments.prefill_only + 64, max_requests=2, max_batch_tokens=arguments.prefill_only)
        measured = time_prefill(engine, config, arguments.prefill_only, steps=steps, warmup=warmup)
        peak_flops = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        print(json.dumps({"prefill_only": True, "tokens": measured["tokens"], "ms": round(measured["ms"], 3), "value": round(measured["value"], 1),
                          "frac": round(measured["flops"] / (measured["ms"] / 1e3) / (peak_flops * 1e12), 4), "peaks": peak_source}))
        return 0
    batch, context = arguments.batch, arguments.context
    largest = 64 if not arguments.skip_points else batch
    engine, config = build_engine(max_tokens=largest * (context + 64), max_requests=max(largest, batch), max_batch_tokens=2048,
                                  cuda_graphs=not arguments.no_graphs)
    fill_cache_randomly(engine, torch.Generator(device="cuda").manual_seed(3))

    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.25)  # a first sample before the timed region starts
    decode = time_decode(engine, batch, context, steps, warmup)
    model = LanguageModel(engine, GenerationConfig())
    e2e = {"value": None, "unit": "tokens/s"} if arguments.skip_e2e else time_e2e(model, batch, context, steps, warmup)
    clock_record = clocks.stop()
    points, prefill = {}, None
    if not arguments.skip_points:
        point_steps = max(10, min(steps, 50))
        points["decode_b1"] = round(time_decode(engine, 1, context, point_steps, warmup)["tokens_per_s"], 1)
        points["decode_b64"] = round(time_decode(engine, 64, context, point_steps, warmup)["tokens_per_s"], 1)
        measured = time_prefill(engine, config, 2048, steps=5, warmup=3)
        peak_flops = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        prefill = {"value": round(measured["value"], 1), "tokens": measured["tokens"], "ms": round(measured["ms"], 3),
                   "frac": round(measured["flops"] / (measured["ms"] / 1e3) / (peak_flops * 1e12), 4)}
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
