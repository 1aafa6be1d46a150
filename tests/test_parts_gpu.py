"""Each part alone against the plain implementation's function for it; a plan that runs a layer twice,
lets a layer read another layer's cache and gives one attention layer a window; and toy parts defined
here (a mixer with state of its own; a feed-forward with routing; a position encoding used by another toy
mixer) that are registered, built and stepped without touching the framework."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_lfm2 as plain

pytestmark = pytest.mark.gpu

LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double().cpu() - want).norm() / want.norm())


class Harness:
    """A runtime, a cache manager for the given mixers, and a batch builder: what a part needs to run."""

    def __init__(self, mixers, dtype: str, page_size: int = 8, num_pages: int = 64, num_slots: int = 4, cache_from=None):
        from lalamo_b200 import ops
        from lalamo_b200.cache import CacheManager
        from lalamo_b200.engine.executor import BatchBuilder
        from lalamo_b200.parts import Runtime

        ops.configure_matmul_precision()
        self.runtime = Runtime(device=torch.device("cuda:0"), dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
        self.mixers = mixers
        needs = [mixer.cache_need() for mixer in mixers]
        self.cache = CacheManager(needs, cache_from or [None] * len(needs), self.runtime, page_size=page_size, num_pages=num_pages, num_slots=num_slots)
        self.builder = BatchBuilder(self.cache, self.runtime.device, vocab_size=1 << 20, planners=mixers)

    def step(self, portions: dict[str, int]):
        """Advances each named request by the given number of tokens; returns (step inputs, views)."""
        from lalamo_b200.engine import StepEntry

        for name in portions:
            if name not in self.cache.requests:
                self.cache.admit(name)
        entries = [StepEntry(name, [0] * count) for name, count in portions.items()]
        built = self.builder.build(entries)
        step, tables = built.inputs, built.block_tables
        views = self.cache.views(tables, step.segment_slot)
        for name, count in portions.items():
            self.cache.commit(name, self.cache.length(name) + count)
        return step, views


def as_type(tensor: torch.Tensor, dtype: str) -> torch.Tensor:
    return tensor.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32)


def random(generator, *shape, scale=1.0):
    return torch.randn(*shape, generator=generator) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_part(dtype):
    from lalamo_b200.config import RMSNormSpec
    from lalamo_b200.parts import Runtime, build_part

    generator = torch.Generator().manual_seed(0)
    runtime = Runtime(device=torch.device("cuda:0"), dtype=as_type(torch.zeros(1), dtype).dtype)
    scale = 1 + random(generator, 200, scale=0.2)
    norm = build_part(RMSNormSpec(dim=200, eps=1e-3), {"scale": scale}, runtime)
    residual = random(generator, 11, 200, scale=2.0)
    delta = as_type(random(generator, 11, 200), dtype)
    on_device = residual.cuda()
    out = norm.residual_forward(on_device, delta.cuda())
    summed = residual.double() + delta.double()
    assert relative_error(out, plain.rms_norm(summed, scale.double(), 1e-3)) < LIMIT[dtype]
    assert relative_error(on_device, summed) < 1e-6  # the stream now holds the sum
    rows = torch.tensor([3, 9], dtype=torch.int32, device="cuda")
    picked = norm.forward(on_device, rows)
    assert relative_error(picked, plain.rms_norm(summed[[3, 9]], scale.double(), 1e-3)) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_mlp_part(dtype):
    from lalamo_b200.config import GatedMLPSpec
    from lalamo_b200.parts import Runtime, build_part

    generator = torch.Generator().manual_seed(1)
    runtime = Runtime(device=torch.device("cuda:0"), dtype=as_type(torch.zeros(1), dtype).dtype)
    weights = {name: as_type(random(generator, *shape, scale=0.1), dtype) for name, shape in
               (("gate_proj", (336, 80)), ("up_proj", (336, 80)), ("down_proj", (80, 336)))}
    part = build_part(GatedMLPSpec(model_dim=80, hidden_dim=336), weights, runtime)
    x = as_type(random(generator, 13, 80), dtype)
    oracle = {"f.w1.weight": weights["gate_proj"].double(), "f.w3.weight": weights["up_proj"].double(), "f.w2.weight": weights["down_proj"].double()}
    assert relative_error(part.forward(x.cuda(), None), plain.swiglu(x.double(), oracle, "f")) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,bias", [(3, False), (5, True)])
def test_short_conv_part(dtype, taps, bias):
    from lalamo_b200.config import ShortConvSpec
    from lalamo_b200.parts import Runtime, build_part

    generator = torch.Generator().manual_seed(taps)
    dim = 72
    weights = {"in_proj": as_type(random(generator, 3 * dim, dim, scale=0.2), dtype), "out_proj": as_type(random(generator, dim, dim, scale=0.2), dtype),
               "conv_weight": random(generator, dim, taps, scale=0.5)}
    if bias:
        weights["conv_bias"] = random(generator, dim, scale=0.5)
    runtime = Runtime(device=torch.device("cuda:0"), dtype=as_type(torch.zeros(1), dtype).dtype)
    part = build_part(ShortConvSpec(model_dim=dim, kernel_size=taps, has_bias=bias), weights, runtime)
    harness = Harness([part], dtype)
    harness.runtime = runtime
    oracle = {"c.in_proj.weight": weights["in_proj"].double(), "c.out_proj.weight": weights["out_proj"].double(), "c.conv.weight": weights["conv_weight"].double()}
    if bias:
        oracle["c.conv.bias"] = weights["conv_bias"].double()
    inputs = {"a": as_type(random(generator, 30, dim), dtype), "b": as_type(random(generator, 17, dim), dtype)}
    expected = {name: plain.short_conv_mixer(x.double(), oracle, "c", {"taps": taps, "conv_bias": bias}) for name, x in inputs.items()}
    done = {"a": 0, "b": 0}
    for portions in ({"a": 9, "b": 1}, {"b": 2}, {"a": 1, "b": 1}, {"b": 13, "a": 20}):
        step, views = harness.step(portions)
        x = torch.cat([inputs[name][done[name] : done[name] + count] for name, count in portions.items()])
        out = part.forward(x.cuda(), step, views[0])
        start = 0
        for name, count in portions.items():
            assert relative_error(out[start : start + count], expected[name][done[name] : done[name] + count]) < LIMIT[dtype], (portions, name)
            done[name] += count
            start += count


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,groups,head_dim,window,normed,rotary", [(4, 2, 16, None, True, True), (3, 1, 32, 13, True, True), (6, 6, 48, None, False, False)])
def test_attention_part(dtype, heads, groups, head_dim, window, normed, rotary):
    from lalamo_b200.config import AttentionSpec, RMSNormSpec, RopeSpec
    from lalamo_b200.parts import Runtime, build_part

    generator = torch.Generator().manual_seed(heads)
    dim = 88
    eps, theta = 1e-4, 5000.0
    weights = {
        "q_proj": as_type(random(generator, heads * head_dim, dim, scale=0.2), dtype), "k_proj": as_type(random(generator, groups * head_dim, dim, scale=0.2), dtype),
        "v_proj": as_type(random(generator, groups * head_dim, dim, scale=0.2), dtype), "out_proj": as_type(random(generator, dim, heads * head_dim, scale=0.2), dtype),
    }
    if normed:
        weights["q_norm"] = 1 + random(generator, head_dim, scale=0.2)
        weights["k_norm"] = 1 + random(generator, head_dim, scale=0.2)
    spec = AttentionSpec(model_dim=dim, num_heads=heads, num_groups=groups, head_dim=head_dim, qk_norm=RMSNormSpec(dim=head_dim, eps=eps) if normed else None,
                         position=RopeSpec(rotary_dim=head_dim, theta=theta) if rotary else None, window=window)
    runtime = Runtime(device=torch.device("cuda:0"), dtype=as_type(torch.zeros(1), dtype).dtype)
    part = build_part(spec, weights, runtime)
    harness = Harness([part], dtype)
    oracle = {f"a.{name}.weight": tensor.double() for name, tensor in weights.items() if name.endswith("proj")}
    oracle["a.q_layernorm.weight"] = weights["q_norm"].double() if normed else torch.ones(head_dim, dtype=torch.float64)
    oracle["a.k_layernorm.weight"] = weights["k_norm"].double() if normed else torch.ones(head_dim, dtype=torch.float64)
    cfg = {"heads": heads, "groups": groups, "head_dim": head_dim, "block_eps": eps, "theta": theta}
    inputs = {"a": as_type(random(generator, 41, dim), dtype), "b": as_type(random(generator, 20, dim), dtype)}

    def reference(x: torch.Tensor) -> torch.Tensor:
        if normed and rotary:
            return plain.attention_mixer(x.double(), oracle, "a", cfg, torch.arange(x.shape[0]), window)
        # no norm, no position encoding: plain causal attention written out here
        T = x.shape[0]
        q = (x.double() @ oracle["a.q_proj.weight"].T).reshape(T, heads, head_dim)
        k = (x.double() @ oracle["a.k_proj.weight"].T).reshape(T, groups, head_dim)
        v = (x.double() @ oracle["a.v_proj.weight"].T).reshape(T, groups, head_dim)
        out = torch.zeros(T, heads, head_dim, dtype=torch.float64)
        for h in range(heads):
            g = h // (heads // groups)
            scores = (q[:, h] @ k[:, g].T) / math.sqrt(head_dim)
            scores = scores.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            out[:, h] = torch.softmax(scores, -1) @ v[:, g]
        return out.reshape(T, -1) @ oracle["a.out_proj.weight"].T

    expected = {name: reference(x) for name, x in inputs.items()}
    done = {"a": 0, "b": 0}
    for portions in ({"a": 17}, {"b": 3, "a": 1}, {"a": 1, "b": 1}, {"a": 22, "b": 16}):
        step, views = harness.step(portions)
        x = torch.cat([inputs[name][done[name] : done[name] + count] for name, count in portions.items()])
        out = part.forward(x.cuda(), step, views[0])
        start = 0
        for name, count in portions.items():
            assert relative_error(out[start : start + count], expected[name][done[name] : done[name] + count]) < LIMIT[dtype], (portions, name)
            done[name] += count
            start += count
    if window is not None:  # pages the window has passed were given back
        assert any(page < 0 for page in harness.cache.requests["a"].blocks[0])
    assert int(runtime.status.item()) == 0


# ------------------------------------------------------------------------------------------------
# A toy mixer with state of its own, defined here: the running mean of its inputs over the request,
# times a learned per-channel gain.  Its state is (sum [dim], count [1]) in one slot tensor.
# ------------------------------------------------------------------------------------------------
def define_toy_mixer():
    from lalamo_b200.config.plan import MixerSpec
    from lalamo_b200.parts import Mixer, SlotStateNeed, TensorDecl, register_part

    @dataclass(frozen=True)
    class RunningMeanSpec(MixerSpec):
        kind: ClassVar[str] = "running_mean"
        model_dim: int = 0

    @register_part(RunningMeanSpec)
    class RunningMean(Mixer):
        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.gain = runtime.vector(tensors["gain"])

        @classmethod
        def tensor_decls(cls, spec):
            return {"gain": TensorDecl((spec.model_dim,), role="vector", init="ones")}

        def cache_need(self):
            return SlotStateNeed(shape=(self.spec.model_dim + 1,), dtype=torch.float32)

        def forward(self, x, step, cache):
            out = torch.empty_like(x)
            slots = cache.segment_slot.tolist()
            for slot, start, length in zip(slots, step.host_segment_start, step.host_segment_length):
                state = cache.state[slot]
                rows = x[start : start + length].float()
                sums = state[:-1] + torch.cumsum(rows, dim=0)
                counts = state[-1] + torch.arange(1, length + 1, device=x.device, dtype=torch.float32)
                out[start : start + length] = (sums / counts[:, None] * self.gain).to(x.dtype)
                state[:-1] = sums[-1]
                state[-1] = counts[-1]
            return out

    return RunningMeanSpec


def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped():
    from lalamo_b200.config import BlockSpec, GatedMLPSpec, ModelPlan, RMSNormSpec
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry
    from lalamo_b200.parts import plan_tensor_decls

    RunningMeanSpec = define_toy_mixer()
    dim, hidden, vocab = 48, 96, 211
    norm = RMSNormSpec(dim=dim, eps=1e-5)
    block = BlockSpec(norm, RunningMeanSpec(model_dim=dim), norm, GatedMLPSpec(model_dim=dim, hidden_dim=hidden))
    plan = ModelPlan(vocab_size=vocab, model_dim=dim, layers=(block, block), final_norm=norm)
    generator = torch.Generator().manual_seed(4)
    tensors = {}
    for key, decl in plan_tensor_decls(plan).items():
        values = torch.randn(decl.shape, generator=generator) * 0.3
        tensors[key] = values + 1 if decl.init == "ones" else values
    engine = Engine(plan, tensors, EngineConfig(dtype="float32", max_tokens=256, max_requests=3))
    assert [type(need).__name__ for need in engine.model.cache_needs()] == ["SlotStateNeed", "SlotStateNeed"]

    def oracle(tokens: list[int]) -> torch.Tensor:
        x = tensors[(("embedding",), "weight")][tokens].double()
        for index in range(2):
            get = lambda role, local: tensors[(("layers", index, role), local)].double()
            n1 = plain.rms_norm(x, get("pre_mixer_norm", "scale"), 1e-5)
            mixed = torch.cumsum(n1, 0) / torch.arange(1, len(tokens) + 1)[:, None] * get("mixer", "gain")
            h = x + mixed
            n2 = plain.rms_norm(h, get("pre_ffn_norm", "scale"), 1e-5)
            x = h + plain.swiglu(n2, {"f.w1.weight": get("ffn", "gate_proj"), "f.w3.weight": get("ffn", "up_proj"), "f.w2.weight": get("ffn", "down_proj")}, "f")
        return plain.rms_norm(x, tensors[(("final_norm",), "scale")].double(), 1e-5) @ tensors[(("embedding",), "weight")].double().T

    sequences = {name: np.random.default_rng(seed).integers(0, vocab, size=n).tolist() for name, seed, n in (("x", 1, 23), ("y", 2, 9))}
    expected = {name: oracle(tokens) for name, tokens in sequences.items()}
    done = {"x": 0, "y": 0}
    for name in sequences:
        engine.admit(name)
    for portions in ({"x": 5, "y": 1}, {"y": 2}, {"x": 1, "y": 1}, {"x": 17, "y": 5}):
        entries = [StepEntry(name, sequences[name][done[name] : done[name] + count], list(range(count))) for name, count in portions.items()]
        logits = engine.step(entries)
        start = 0
        for name, count in portions.items():
            assert relative_error(logits[start : start + count], expected[name][done[name] : done[name] + count]) < 2e-5
            done[name] += count
            start += count
    engine.release("x")
    engine.admit("z")  # takes over x's slot: the state must have been zeroed
    logits = engine.step([StepEntry("z", sequences["y"], list(range(9)))])
    assert relative_error(logits, expected["y"]) < 2e-5


# ------------------------------------------------------------------------------------------------
# Two more toy parts defined here: a feed-forward that routes every token to one of several experts
# (arg-max of a router product, router logits in 32-bit), and a position encoding of its own (a table
# of sines with a made-up period, added to the input) used by a toy mixer that shifts tokens by one.
# Neither is a model of anybody's; they show that the step function, the cache manager and the block do
# not care what a part does.
# ------------------------------------------------------------------------------------------------
def define_toy_routed_ffn_and_position_parts():
    from lalamo_b200.config.plan import FeedForwardSpec, MixerSpec, PositionSpec
    from lalamo_b200.parts import FeedForward, Mixer, PositionEncoding, SlotStateNeed, TensorDecl, build_part, register_part

    @dataclass(frozen=True)
    class RoutedSpec(FeedForwardSpec):
        kind: ClassVar[str] = "toy_routed"
        model_dim: int = 0
        hidden_dim: int = 0
        experts: int = 2

    @register_part(RoutedSpec)
    class Routed(FeedForward):
        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.router = runtime.vector(tensors["router"])   # kept in 32-bit: the router logits are computed in 32-bit
            self.up = runtime.matrix(tensors["up"])
            self.down = runtime.matrix(tensors["down"])

        @classmethod
        def tensor_decls(cls, spec):
            return {"router": TensorDecl((spec.experts, spec.model_dim), role="vector"),
                    "up": TensorDecl((spec.experts * spec.hidden_dim, spec.model_dim)),
                    "down": TensorDecl((spec.experts * spec.model_dim, spec.hidden_dim))}

        def forward(self, x, step=None):
            spec = self.spec
            choice = (x.float() @ self.router.T).argmax(-1)
            up = self.up.reshape(spec.experts, spec.hidden_dim, spec.model_dim)
            down = self.down.reshape(spec.experts, spec.model_dim, spec.hidden_dim)
            out = torch.zeros_like(x)
            for expert in range(spec.experts):
                rows = torch.nonzero(choice == expert).flatten()
                if rows.numel():
                    out[rows] = torch.relu(x[rows] @ up[expert].T) @ down[expert].T
            return out

    @dataclass(frozen=True)
    class SineTableSpec(PositionSpec):
        kind: ClassVar[str] = "toy_sine_table"
        dim: int = 0
        period: float = 7.0

    @register_part(SineTableSpec)
    class SineTable(PositionEncoding):
        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.phase = torch.arange(spec.dim, device=runtime.device, dtype=torch.float32) / spec.dim

        def encode(self, positions):
            return torch.sin((positions.float()[:, None] / self.spec.period + self.phase) * 2 * math.pi)

    @dataclass(frozen=True)
    class ShiftSpec(MixerSpec):
        kind: ClassVar[str] = "toy_shift"
        model_dim: int = 0
        position: PositionSpec | None = None

    @register_part(ShiftSpec)
    class Shift(Mixer):
        """out[t] = gain * (x[t - 1] + encoding(position[t - 1])), zero for a request's first token; its
        state is the previous token's row."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.gain = runtime.vector(tensors["gain"])
            self.position = build_part(spec.position, {}, runtime)

        @classmethod
        def tensor_decls(cls, spec):
            return {"gain": TensorDecl((spec.model_dim,), role="vector", init="ones")}

        def cache_need(self):
            return SlotStateNeed(shape=(self.spec.model_dim,), dtype=torch.float32)

        def forward(self, x, step, cache):
            carried = x.float() + self.position.encode(step.positions[: x.shape[0]])
            out = torch.empty_like(x)
            for slot, start, length in zip(cache.segment_slot.tolist(), step.host_segment_start, step.host_segment_length):
                rows = torch.cat([cache.state[slot][None], carried[start : start + length - 1]])
                out[start : start + length] = (rows * self.gain).to(x.dtype)
                cache.state[slot] = carried[start + length - 1]
            return out

    return RoutedSpec, SineTableSpec, ShiftSpec


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_run_through_the_engine():
    from lalamo_b200.config import BlockSpec, ModelPlan, RMSNormSpec
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry
    from lalamo_b200.parts import plan_tensor_decls

    RoutedSpec, SineTableSpec, ShiftSpec = define_toy_routed_ffn_and_position_parts()
    dim, hidden, experts, vocab = 40, 24, 3, 97
    norm = RMSNormSpec(dim=dim, eps=1e-5)
    block = BlockSpec(norm, ShiftSpec(model_dim=dim, position=SineTableSpec(dim=dim, period=5.5)), norm, RoutedSpec(model_dim=dim, hidden_dim=hidden, experts=experts))
    plan = ModelPlan(vocab_size=vocab, model_dim=dim, layers=(block, block), final_norm=norm)
    generator = torch.Generator().manual_seed(9)
    tensors = {}
    for key, decl in plan_tensor_decls(plan).items():
        values = torch.randn(decl.shape, generator=generator) * 0.4
        tensors[key] = values + 1 if decl.init == "ones" else values
    engine = Engine(plan, tensors, EngineConfig(dtype="float32", max_tokens=128, max_requests=2))

    def oracle(tokens: list[int]) -> torch.Tensor:
        x = tensors[(("embedding",), "weight")][tokens].double()
        places = torch.arange(len(tokens), dtype=torch.float64)
        encoding = torch.sin((places[:, None] / 5.5 + torch.arange(dim, dtype=torch.float64) / dim) * 2 * math.pi)
        for index in range(2):
            get = lambda role, local: tensors[(("layers", index, role), local)].double()
            n1 = plain.rms_norm(x, get("pre_mixer_norm", "scale"), 1e-5)
            carried = n1 + encoding
            h = x + torch.cat([torch.zeros(1, dim, dtype=torch.float64), carried[:-1]]) * get("mixer", "gain")
            n2 = plain.rms_norm(h, get("pre_ffn_norm", "scale"), 1e-5)
            choice = (n2 @ get("ffn", "router").T).argmax(-1)
            up, down = get("ffn", "up").reshape(experts, hidden, dim), get("ffn", "down").reshape(experts, dim, hidden)
            routed = torch.stack([torch.relu(n2[t] @ up[choice[t]].T) @ down[choice[t]].T for t in range(len(tokens))])
            x = h + routed
        return plain.rms_norm(x, tensors[(("final_norm",), "scale")].double(), 1e-5) @ tensors[(("embedding",), "weight")].double().T

    sequences = {name: np.random.default_rng(seed).integers(0, vocab, size=n).tolist() for name, seed, n in (("p", 5, 19), ("q", 6, 11))}
    expected = {name: oracle(tokens) for name, tokens in sequences.items()}
    done = {"p": 0, "q": 0}
    for name in sequences:
        engine.admit(name)
    for portions in ({"p": 4, "q": 1}, {"q": 3}, {"p": 1, "q": 2}, {"p": 14, "q": 5}):
        entries = [StepEntry(name, sequences[name][done[name] : done[name] + count], list(range(count))) for name, count in portions.items()]
        logits = engine.step(entries)
        start = 0
        for name, count in portions.items():
            assert relative_error(logits[start : start + count], expected[name][done[name] : done[name] + count]) < 2e-5
            done[name] += count
            start += count


# ------------------------------------------------------------------------------------------------
# Toy parts that need what the built-in ones do not: a mixer whose kernels want a work list of their
# own for every step, made on the host from the portions *and their contexts* (plan_step); an
# arrangement with its norms after the sub-blocks; a read-out that scales and caps its logits.  They
# run through the engine, its recorded decode steps and its steps recorded by shape, untouched.
# ------------------------------------------------------------------------------------------------
def define_toy_planned_mixer_post_norm_and_capped_head():
    from lalamo_b200 import ops
    from lalamo_b200.config.plan import FeedForwardSpec, HeadSpec, MixerSpec, NormSpec
    from lalamo_b200.parts import Block, Mixer, TensorDecl, register_arrangement, register_part
    from lalamo_b200.parts.embedding import LMHead

    @dataclass(frozen=True)
    class PositionGateSpec(MixerSpec):
        kind: ClassVar[str] = "toy_position_gate"
        model_dim: int = 0
        period: int = 3

    @register_part(PositionGateSpec)
    class PositionGate(Mixer):
        """out[t] = gain * x[t] where the token's absolute position is no multiple of ``period``, else 0.
        Which rows pass is decided on the host, step by step, and reaches the device as a list."""

        graph_safe = True
        plans_made = 0

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.gain = runtime.vector(tensors["gain"])

        @classmethod
        def tensor_decls(cls, spec):
            return {"gain": TensorDecl((spec.model_dim,), role="vector", init="ones")}

        def step_plan_key(self):
            return ("toy_position_gate", self.spec.period)

        def plan_step(self, segments):
            type(self).plans_made += 1
            keep = [int((context + offset) % self.spec.period != 0) for context, length in zip(segments.context, segments.length) for offset in range(length)]
            return {"keep": np.asarray(keep, dtype=np.int32)}

        def forward(self, x, step, cache):
            lists, host_lists = step.plan_of(self)
            assert host_lists["keep"].size == step.tokens
            return (x.float() * self.gain * lists["keep"][:, None].float()).to(x.dtype)

    @dataclass(frozen=True)
    class PostNormSpec:
        mixer: MixerSpec
        post_mixer_norm: NormSpec
        ffn: FeedForwardSpec
        post_ffn_norm: NormSpec
        arrangement: str = "toy_post_norm"

    @register_arrangement("toy_post_norm")
    class PostNorm(Block):
        """x = norm(x + mixer(x)); x = norm(x + ffn(x)): the norms rewrite the residual stream itself."""

        roles = ("mixer", "post_mixer_norm", "ffn", "post_ffn_norm")

        def forward(self, residual, pending, step, cache):
            if pending is not None:
                ops.residual_add(residual, pending)
            mixed = self.mixer.forward(residual.to(self.runtime.dtype), step, cache)
            residual.copy_(self.post_mixer_norm.forward(residual + mixed.float()))
            out = self.ffn.forward(residual.to(self.runtime.dtype), step)
            residual.copy_(self.post_ffn_norm.forward(residual + out.float()))
            return None

    @dataclass(frozen=True)
    class CappedHeadSpec(HeadSpec):
        kind: ClassVar[str] = "toy_capped_head"
        logit_scale: float = 1.0
        soft_cap: float = 30.0

    @register_part(CappedHeadSpec)
    class CappedHead(LMHead):
        def forward(self, x):
            return self.spec.soft_cap * torch.tanh(super().forward(x) * (self.spec.logit_scale / self.spec.soft_cap))

    return PositionGateSpec, PostNormSpec, CappedHeadSpec, PositionGate


def test_toy_parts_with_a_step_plan_a_post_norm_arrangement_and_a_capped_head_run_and_replay():
    from lalamo_b200.config import BlockSpec, GatedMLPSpec, ModelPlan, RMSNormSpec
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry
    from lalamo_b200.parts import plan_tensor_decls

    PositionGateSpec, PostNormSpec, CappedHeadSpec, PositionGate = define_toy_planned_mixer_post_norm_and_capped_head()
    dim, hidden, vocab, period = 32, 64, 131, 3
    norm = RMSNormSpec(dim=dim, eps=1e-5)
    gate, mlp = PositionGateSpec(model_dim=dim, period=period), GatedMLPSpec(model_dim=dim, hidden_dim=hidden)
    plan = ModelPlan(vocab_size=vocab, model_dim=dim, layers=(BlockSpec(norm, gate, norm, mlp), PostNormSpec(gate, norm, mlp, norm)), final_norm=norm,
                     tie_embeddings=False, head=CappedHeadSpec(vocab, dim, tied=False, logit_scale=3.0, soft_cap=4.0))
    generator = torch.Generator().manual_seed(12)
    tensors = {}
    for key, decl in plan_tensor_decls(plan).items():
        values = torch.randn(decl.shape, generator=generator) * 0.3
        tensors[key] = values + 1 if decl.init == "ones" else values
    assert (("lm_head",), "weight") in tensors and (("layers", 1, "post_ffn_norm"), "scale") in tensors
    engine = Engine(plan, tensors, EngineConfig(dtype="float32", max_tokens=256, max_requests=3, cuda_graphs=True))
    assert engine.executor.use_graphs and len(engine.executor.builder.planners) == 1  # both layers share one plan

    def oracle(tokens: list[int]) -> torch.Tensor:
        x = tensors[(("embedding",), "weight")][tokens].double()
        keep = torch.tensor([float(place % period != 0) for place in range(len(tokens))], dtype=torch.float64)[:, None]
        get = lambda index, role, local: tensors[(("layers", index, role), local)].double()
        mlp_of = lambda index, rows: plain.swiglu(rows, {"f.w1.weight": get(index, "ffn", "gate_proj"), "f.w3.weight": get(index, "ffn", "up_proj"),
                                                         "f.w2.weight": get(index, "ffn", "down_proj")}, "f")
        h = x + plain.rms_norm(x, get(0, "pre_mixer_norm", "scale"), 1e-5) * keep * get(0, "mixer", "gain")
        x = h + mlp_of(0, plain.rms_norm(h, get(0, "pre_ffn_norm", "scale"), 1e-5))
        x = plain.rms_norm(x + x * keep * get(1, "mixer", "gain"), get(1, "post_mixer_norm", "scale"), 1e-5)
        x = plain.rms_norm(x + mlp_of(1, x), get(1, "post_ffn_norm", "scale"), 1e-5)
        logits = plain.rms_norm(x, tensors[(("final_norm",), "scale")].double(), 1e-5) @ tensors[(("lm_head",), "weight")].double().T
        return 4.0 * torch.tanh(logits * 3.0 / 4.0)

    sequences = {name: np.random.default_rng(seed).integers(0, vocab, size=n).tolist() for name, seed, n in (("u", 21, 40), ("v", 22, 31))}
    expected = {name: oracle(tokens) for name, tokens in sequences.items()}
    done = {"u": 0, "v": 0}
    for name in sequences:
        engine.admit(name)
    # portions of one shape three times over (run, recorded, replayed), then a dozen decode steps of both requests
    # (recorded at the first, replayed afterwards) at contexts that differ between the two and move on every step
    schedule = [{"u": 7, "v": 2}, {"u": 4, "v": 1}, {"u": 4, "v": 1}, {"u": 4, "v": 1}] + [{"u": 1, "v": 1}] * 12
    for portions in schedule:
        entries = [StepEntry(name, sequences[name][done[name] : done[name] + count], [count - 1]) for name, count in portions.items()]
        logits = engine.step(entries)
        for row, (name, count) in enumerate(portions.items()):
            done[name] += count
            assert relative_error(logits[row : row + 1], expected[name][done[name] - 1 : done[name]]) < 2e-5, (portions, name)
    assert engine.executor.graph_replays == 1 + 11
    assert PositionGate.plans_made >= len(schedule)  # made again for every step, replayed ones included
    engine.executor.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_with_a_layer_twice_a_shared_cache_and_a_window(dtype):
    """Three layers (conv, windowed attention, full attention) scheduled as
    conv, windowed, full, conv again, full again reading the first full entry's cache."""
    from lalamo_b200.config import Lfm2Config, ModelPlan, ScheduleEntry
    from lalamo_b200.config.plan import AttentionSpec, BlockSpec
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry
    from lalamo_b200.parts import plan_tensor_decls
    from dataclasses import replace
    from tiny import TINY_B

    config = Lfm2Config.from_dict(dict(TINY_B, num_hidden_layers=3, full_attn_idxs=[1, 2]))
    base = config.to_plan()
    window = 21
    layers = (base.layers[0], replace(base.layers[1], mixer=replace(base.layers[1].mixer, window=window)), base.layers[2])
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0), ScheduleEntry(2, cache_from=2))
    plan = ModelPlan(base.vocab_size, base.model_dim, layers, base.final_norm, base.tie_embeddings, schedule=schedule)
    generator = torch.Generator().manual_seed(9)
    tensors, named = {}, {}
    for (path, local), decl in plan_tensor_decls(plan).items():
        values = torch.randn(decl.shape, generator=generator) * 0.08
        values = (values + 1 if decl.init == "ones" else values).to(torch.bfloat16 if decl.role == "matrix" else torch.float32)
        tensors[(path, local)] = values
        named[config.checkpoint_names(path, local)[0]] = values.double().reshape(config.checkpoint_shape(path, local, decl.shape))
    engine = Engine(plan, tensors, EngineConfig(dtype=dtype, page_size=8, max_tokens=512, max_requests=2))
    layout = engine.cache.layout
    assert layout.group_windows == [window, None] and layout.entry_owner == [0, 1, 2, 3, 2]
    assert len(engine.cache.states) == 2  # the conv layer runs twice and holds a state for each run

    cfg = {"hidden": 96, "heads": 3, "groups": 1, "head_dim": 32, "taps": 4, "conv_bias": True, "theta": 1e6, "block_eps": 1e-6, "eps": 3e-6}

    def oracle(tokens: list[int]) -> torch.Tensor:
        T = len(tokens)
        positions = torch.arange(T)
        x = named["model.embed_tokens.weight"][tokens]
        shared_kv = None
        for entry in schedule:
            root = f"model.layers.{entry.layer}"
            n1 = plain.rms_norm(x, named[f"{root}.operator_norm.weight"], cfg["block_eps"])
            if entry.layer == 0:
                mixed = plain.short_conv_mixer(n1, named, f"{root}.conv", cfg)
            elif entry.cache_from is None:
                mixed = plain.attention_mixer(n1, named, f"{root}.self_attn", cfg, positions, window if entry.layer == 1 else None)
                if entry.layer == 2:  # remember this run's keys and values for the run that shares them
                    k = (n1 @ named[f"{root}.self_attn.k_proj.weight"].T).reshape(T, 1, 32)
                    v = (n1 @ named[f"{root}.self_attn.v_proj.weight"].T).reshape(T, 1, 32)
                    shared_kv = (plain.rope(plain.rms_norm(k, named[f"{root}.self_attn.k_layernorm.weight"], cfg["block_eps"]), positions, cfg["theta"]), v)
            else:
                q = (n1 @ named[f"{root}.self_attn.q_proj.weight"].T).reshape(T, 3, 32)
                q = plain.rope(plain.rms_norm(q, named[f"{root}.self_attn.q_layernorm.weight"], cfg["block_eps"]), positions, cfg["theta"])
                k, v = shared_kv
                out = torch.zeros(T, 3, 32, dtype=torch.float64)
                for h in range(3):
                    scores = (q[:, h] @ k[:, 0].T) / math.sqrt(32)
                    scores = scores.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
                    out[:, h] = torch.softmax(scores, -1) @ v[:, 0]
                mixed = out.reshape(T, 96) @ named[f"{root}.self_attn.out_proj.weight"].T
            h = x + mixed
            n2 = plain.rms_norm(h, named[f"{root}.ffn_norm.weight"], cfg["block_eps"])
            x = h + plain.swiglu(n2, named, f"{root}.feed_forward")
        return plain.rms_norm(x, named["model.embedding_norm.weight"], cfg["eps"]) @ named["lm_head.weight"].T

    tokens = np.random.default_rng(3).integers(0, 1000, size=90).tolist()
    expected = oracle(tokens)
    engine.admit("r")
    start = 0
    limit = 2e-5 if dtype == "float32" else 1e-1
    for size in (30, 1, 1, 7, 2, 40, 9):
        logits = engine.step([StepEntry("r", tokens[start : start + size], list(range(size)))])
        error = (logits.double().cpu() - expected[start : start + size]).norm(dim=-1) / expected[start : start + size].norm(dim=-1)
        assert error.max() < limit, f"portion at {start}: first wrong row {int((error >= limit).nonzero()[0])}"
        start += size
    blocks = engine.cache.requests["r"].blocks
    assert sum(page < 0 for page in blocks[0]) == (90 - window + 1) // 8 and all(page >= 0 for page in blocks[1])
    engine.executor.check_status()


def test_rope_part_table():
    """The rotary part owns the inverse-frequency table theta ** (-2i / rotary_dim), in float32."""
    from lalamo_b200.config import RopeSpec
    from lalamo_b200.parts import Runtime, build_part

    runtime = Runtime(device=torch.device("cuda:0"), dtype=torch.bfloat16)
    part = build_part(RopeSpec(rotary_dim=48, theta=1e6), {}, runtime)
    expected = torch.tensor([1e6 ** (-2 * i / 48) for i in range(24)], dtype=torch.float64)
    assert part.inv_freq.dtype == torch.float32 and part.rotary_dim == 48
    torch.testing.assert_close(part.inv_freq.cpu().double(), expected, rtol=1e-6, atol=0)
    with pytest.raises(ValueError):
        build_part(RopeSpec(rotary_dim=7, theta=10.0), {}, runtime)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["conv", "full_attention"])
def test_block_alone(dtype, kind):
    """One block (norm, mixer, residual, norm, feed-forward, residual) against the plain block, in
    two portions; the block hands back its feed-forward output unadded or adds it itself."""
    from lalamo_b200.config import Lfm2Config
    from lalamo_b200 import ops
    from lalamo_b200.parts import Runtime, block_tensor_decls, build_block
    from tiny import TINY_B

    config = Lfm2Config.from_dict(dict(TINY_B, num_hidden_layers=1, full_attn_idxs=[0] if kind == "full_attention" else []))
    spec = config.to_plan().layers[0]
    generator = torch.Generator().manual_seed(5)
    tensors, named = {}, {}
    for (role, local), decl in block_tensor_decls(spec).items():
        values = torch.randn(decl.shape, generator=generator) * 0.1
        values = (values + 1 if decl.init == "ones" else values).to(torch.bfloat16 if decl.role == "matrix" else torch.float32)
        tensors[(role, local)] = values
        named[config.checkpoint_names(("layers", 0, role), local)[0]] = values.double().reshape(config.checkpoint_shape(("layers", 0, role), local, decl.shape))
    runtime = Runtime(device=torch.device("cuda:0"), dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    block = build_block(spec, tensors, runtime)
    harness = Harness([block.mixer], dtype)
    cfg = {"hidden": 96, "heads": 3, "groups": 1, "head_dim": 32, "taps": 4, "conv_bias": True, "theta": 1e6, "block_eps": 1e-6, "kinds": [kind]}
    x = torch.randn(29, 96, generator=generator)
    expected = plain.block(x.double(), named, 0, cfg, torch.arange(29))
    start = 0
    for count in (20, 9):
        step, views = harness.step({"r": count})
        residual = x[start : start + count].clone().cuda()
        pending = block.forward(residual, None, step, views[0])
        if isinstance(pending, ops.SlicedSum):
            pending = pending.sum()
        got = residual.double().cpu() + (pending.double().cpu() if pending is not None else 0.0)
        assert relative_error(got, expected[start : start + count]) < (2e-5 if dtype == "float32" else 2e-2)
        start += count
