"""Times single kernels in a loop with CUDA events, outside any profiler.

    python -m lalamo_b200.microbench linear --tokens 512 --rows 2048 --width 8192 --epilogue residual_add [--tile 64]
    python -m lalamo_b200.microbench prefill-attention --tokens 2048 [--kernel mma] [--last-tiles 1]
    python -m lalamo_b200.microbench decode-attention --batch 8 --context 4096
    python -m lalamo_b200.microbench step-kernels --tokens 2048 [--preset lfm2-1.2b] [--batch 8 --context 4096]

Each prints one JSON line.  Sizes default to the LFM2-1.2B shape (32 query heads over 8 K/V heads
of 64 channels, pages of 16 keys).  ``linear`` rotates over several weight matrices; with
``--copies`` large enough that they exceed the L2 cache the weights come from memory every time.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops


def _time(run, repeats: int, graph: bool = False) -> float:
    """Microseconds per call of ``run``; with ``graph`` the call is recorded in a CUDA graph first, so that
    kernels of a few microseconds are not timed by how fast the host can launch them."""
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    if graph:
        recorded = torch.cuda.CUDAGraph()
        with torch.cuda.graph(recorded):
            run()
        run = recorded.replay
        run()
        torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(repeats):
        run()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) * 1e3 / repeats


def linear(arguments: argparse.Namespace) -> dict:
    if arguments.tile:
        os.environ["LALAMO_B200_TCGEN05_TILE"] = str(arguments.tile)  # 64, 128, 256, or 512 for the pair of CTAs
    tokens, rows, width = arguments.tokens, arguments.rows, arguments.width
    weights = [torch.randn(rows, width, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(arguments.copies)]
    x = torch.randn(tokens, width, device="cuda", dtype=torch.bfloat16)
    residual = torch.zeros(tokens, rows, device="cuda")

    def run() -> None:
        for weight in weights:
            if arguments.library:
                torch.mm(x, weight.t())  # the library's product, for comparison (no epilogue)
            elif arguments.auto:
                # what the engine would call for this product (the weight-streaming kernel for few tokens)
                if arguments.epilogue == "residual_add":
                    ops.linear_accumulate(x, weight, residual)
                elif arguments.epilogue == "gated":
                    ops.gated_linear(x, weight, "silu")
                else:
                    ops.linear(x, weight)
            elif arguments.epilogue == "residual_add":
                ops.linear_tcgen05(x, weight, "residual_add", residual=residual, slices=arguments.slices)
            elif arguments.epilogue == "gated":
                ops.linear_tcgen05(x, weight, "gated", activation="silu")
            else:
                ops.linear_tcgen05(x, weight, arguments.epilogue, slices=arguments.slices)

    microseconds = _time(run, arguments.repeats, arguments.graph) / len(weights)
    return {"kernel": "library" if arguments.library else "linear_tcgen05", "tokens": tokens, "rows": rows, "width": width, "epilogue": arguments.epilogue, "tile": arguments.tile or "auto",
            "slices": arguments.slices or "auto", "us": round(microseconds, 2), "tflops": round(2 * tokens * rows * width / microseconds / 1e6, 1)}


def prefill_attention(arguments: argparse.Namespace) -> dict:
    tokens, heads, groups, head_dim, page = arguments.tokens, arguments.heads, arguments.groups, arguments.head_dim, 16
    pages = -(-tokens // page)
    keys = torch.randn(pages, page, groups, head_dim, device="cuda").to(torch.bfloat16)
    values = torch.randn(pages, groups, head_dim, page, device="cuda").to(torch.bfloat16)
    q = torch.randn(tokens, heads * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    table = torch.arange(pages, dtype=torch.int32, device="cuda").reshape(1, pages)
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    segments = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    records = [[first, min(32, tokens - first)] for first in range(0, tokens, 32)]
    if arguments.last_tiles:
        records = records[-arguments.last_tiles:]  # only the prompt's last tiles: the CTAs that walk the most keys
    tiles = torch.tensor(records, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run() -> None:
        ops.attention_prefill(q, keys, values, out, tiles=tiles, num_tiles=len(records), positions=positions, token_segment=segments, block_table=table,
                              num_heads=heads, num_groups=groups, head_dim=head_dim, scale=head_dim**-0.5, window=None, status=status, kernel=arguments.kernel,
                              split_tiles=arguments.split_tiles)

    microseconds = _time(run, arguments.repeats)
    flops = sum(4 * heads * head_dim * count * (first + (count + 1) / 2) for first, count in records)
    return {"kernel": f"attention_prefill[{arguments.kernel}]", "tokens": tokens, "tiles": len(records), "us": round(microseconds, 1),
            "tflops": round(flops / microseconds / 1e6, 1), "status": int(status.item())}


def decode_attention(arguments: argparse.Namespace) -> dict:
    batch, context, heads, groups, head_dim, page, layers = arguments.batch, arguments.context, arguments.heads, arguments.groups, arguments.head_dim, 16, 6
    per_request = -(-context // page)
    pages = batch * per_request
    keys = [torch.randn(pages, page, groups, head_dim, device="cuda").to(torch.bfloat16) for _ in range(layers)]
    values = [torch.randn(pages, groups, head_dim, page, device="cuda").to(torch.bfloat16) for _ in range(layers)]
    q = torch.randn(batch, heads * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    table = torch.arange(pages, dtype=torch.int32, device="cuda").reshape(batch, per_request)
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
    segments = torch.arange(batch, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    if arguments.ctas_per_sm:
        # plan the splits as if an SM held this many CTAs (default: what the runtime reports for the kernel)
        plan = ops.decode_attention_plan
        ops.decode_attention_plan = lambda *a, **k: plan(*a, **{**k, "resident_ctas": ops.sm_count() * arguments.ctas_per_sm})

    def layers_once() -> None:
        for layer in range(layers):
            ops.attention_decode(q, keys[layer], values[layer], out, positions=positions, token_segment=segments, block_table=table, num_heads=heads,
                                 num_groups=groups, head_dim=head_dim, scale=head_dim**-0.5, window=None, max_context=context, status=status)

    layers_once()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()  # as the engine runs it: the layers' caches one after the other, replayed
    with torch.cuda.graph(graph):
        layers_once()
    microseconds = _time(graph.replay, arguments.repeats) / layers
    bytes_read = batch * context * groups * head_dim * 2 * 2
    return {"kernel": "attention_decode + merge", "batch": batch, "context": context, "splits": ops.decode_attention_plan(batch, heads, groups, context, None, head_dim)[0],
            "us_per_layer": round(microseconds, 2), "tb_per_s": round(bytes_read / microseconds / 1e6, 2), "status": int(status.item())}


def step_kernels(arguments: argparse.Namespace) -> dict:
    """The kernels of one step with their durations while the step runs as it does in production (warm
    caches, launches overlapping, recorded graphs), as CUPTI reports them through ``torch.profiler``: a
    prompt of ``--tokens`` tokens in one step, or with ``--batch`` a decode step of that many requests at
    ``--context``."""
    import numpy as np
    from torch.profiler import ProfilerActivity, profile

    from .config import config_from_dict
    from .engine import Engine, EngineConfig, StepEntry
    from .model_registry import PRESETS

    decode = arguments.batch > 0
    tokens = arguments.tokens
    room = arguments.batch * (arguments.context + 64) if decode else tokens + 64
    engine = Engine.random(config_from_dict(PRESETS[arguments.preset]), seed=1, std=0.02,
                           engine_config=EngineConfig(dtype="bfloat16", page_size=16, max_tokens=room, max_requests=max(1, arguments.batch),
                                                      max_batch_tokens=max(tokens, 2048), cuda_graphs=True))
    random = np.random.default_rng(0)
    if decode:
        names = list(range(arguments.batch))
        for name in names:
            engine.admit(name)
            engine.cache.reserve(name, arguments.context - 8)
            engine.cache.commit(name, arguments.context - 8)

        def one() -> None:
            engine.step([StepEntry(name, [int(random.integers(0, engine.vocab_size))], [0]) for name in names])
            torch.cuda.synchronize()
    else:
        def one() -> None:
            engine.admit("prompt")
            engine.step([StepEntry("prompt", random.integers(0, engine.vocab_size, size=tokens).tolist(), [tokens - 1])])
            torch.cuda.synchronize()
            engine.release("prompt")

    for _ in range(3):
        one()
    with profile(activities=[ProfilerActivity.CUDA]) as session:
        one()
    rows = [(event.key, event.count, event.device_time_total) for event in session.key_averages() if event.device_time_total > 0]
    rows.sort(key=lambda row: -row[2])
    total = sum(row[2] for row in rows)
    return {"step": f"decode batch {arguments.batch} context {arguments.context}" if decode else f"prompt of {tokens} tokens", "preset": arguments.preset,
            "us_total": round(total, 1), "kernels": [{"name": name[:90], "launches": count, "us": round(time, 1), "us_each": round(time / count, 2)} for name, count, time in rows]}


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="python -m lalamo_b200.microbench", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    commands = parser.add_subparsers(dest="command", required=True)
    one = commands.add_parser("linear")
    one.add_argument("--tokens", type=int, default=2048)
    one.add_argument("--rows", type=int, default=2048)
    one.add_argument("--width", type=int, default=2048)
    one.add_argument("--epilogue", default="store", choices=["store", "store_float", "residual_add", "gated"])
    one.add_argument("--tile", type=int, default=0)
    one.add_argument("--slices", type=int, default=None)
    one.add_argument("--copies", type=int, default=6)
    one.add_argument("--repeats", type=int, default=5)
    one.add_argument("--graph", action="store_true", help="record the loop in a CUDA graph and time its replays")
    one.add_argument("--library", action="store_true", help="time torch.mm on the same shapes instead")
    one.add_argument("--auto", action="store_true", help="call the product the way the engine does (ops.linear, linear_accumulate, gated_linear)")
    one.set_defaults(function=linear)
    for name, function in (("prefill-attention", prefill_attention), ("decode-attention", decode_attention)):
        one = commands.add_parser(name)
        one.add_argument("--heads", type=int, default=32)
        one.add_argument("--groups", type=int, default=8)
        one.add_argument("--head-dim", type=int, default=64)
        one.add_argument("--repeats", type=int, default=10)
        one.set_defaults(function=function)
        if name == "prefill-attention":
            one.add_argument("--tokens", type=int, default=2048)
            one.add_argument("--kernel", default="tcgen05", choices=["tcgen05", "mma"])
            one.add_argument("--last-tiles", type=int, default=0)
            one.add_argument("--split-tiles", type=int, default=0, help="tiles that see at least this many tiles of 64 keys are shared by two CTAs")
        else:
            one.add_argument("--batch", type=int, default=8)
            one.add_argument("--context", type=int, default=4096)
            one.add_argument("--ctas-per-sm", type=int, default=0)
    one = commands.add_parser("step-kernels")
    one.add_argument("--tokens", type=int, default=2048)
    one.add_argument("--batch", type=int, default=0, help="a decode step of this many requests instead of a prompt")
    one.add_argument("--context", type=int, default=4096)
    one.add_argument("--preset", default="lfm2-1.2b")
    one.set_defaults(function=step_kernels)
    arguments = parser.parse_args(argv)
    if not torch.cuda.is_available():
        parser.error("a CUDA device is needed")
    print(json.dumps(arguments.function(arguments)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
