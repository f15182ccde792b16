"""A mixer with state of its own, an architecture that uses it, and a schedule that runs a layer twice
and lets a layer read another's cache: all defined HERE, registered, built, loaded from a model folder
and stepped without a change to the framework's files."""

import json
import math
from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

import plain_impl
from helpers import random_ids

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------ the toy parts
@dataclass(frozen=True)
class DecayMixerSpec:
    hidden_size: int = 0
    decay: float = 0.9
    kind: str = field(init=False, default="toy_decay_state")


def make_toy():
    """Registration happens inside a function so that collecting this file without a GPU does nothing."""
    from libmir_b200 import register_architecture, register_part
    from libmir_b200.config.spec import (EmbeddingSpec, FixedState, HeadSpec, LayerSpec, ModelSpec, ParamSpec,
                                         RmsNormSpec, RotarySpec, ScheduleEntry, SoftmaxAttentionSpec, SwiGluSpec)
    from libmir_b200.parts import Mixer

    class DecayMixer(Mixer):
        """state <- decay * state + W x_t ; output_t = state.  The state [hidden] lives in the request's slot."""

        def parameters(self):
            return {"mix.weight": ParamSpec((self.spec.hidden_size, self.spec.hidden_size))}

        def bind(self, tensors):
            self.weight = tensors["mix.weight"]

        def cache_requirement(self):
            return FixedState((self.spec.hidden_size,), "float32")

        def forward(self, ctx, cache, x, residual):
            projected = x.float() @ self.weight.float().T
            for row in range(ctx.num_rows):
                begin, end = ctx.host_query_starts[row], ctx.host_query_starts[row + 1]
                state = cache.state[ctx.host_state_slots[row]]
                for token in range(begin, end):
                    state.mul_(self.spec.decay).add_(projected[token])
                    residual[token] += state

    register_part("toy_decay_state", DecayMixer)

    def build(config, catalog):
        hidden = config["hidden_size"]
        norm = lambda: RmsNormSpec(size=hidden, eps=config["eps"])
        ff = SwiGluSpec(hidden_size=hidden, intermediate_size=config["intermediate_size"])
        names = {"mixer_norm": "norm_a.", "mixer": "mixer.", "feed_forward_norm": "norm_b.", "feed_forward": "ff."}
        attention = SoftmaxAttentionSpec(hidden_size=hidden, heads=4, kv_heads=2, head_dim=16, scale=0.25,
                                         position=RotarySpec(head_dim=16, rotary_dim=16, theta=1000.0))
        layers = (
            LayerSpec("toy.layers.0.", DecayMixerSpec(hidden, config["decay"]), ff, norm(), norm(), names),
            LayerSpec("toy.layers.1.", attention, ff, norm(), norm(), names),
        )
        # layer 0 runs twice (two states), layer 1 runs twice and the second run reads the first one's cache
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))
        return ModelSpec("ToyStateForCausalLM", hidden, config["vocab_size"], config["max_positions"],
                         EmbeddingSpec("toy.embed.weight", config["vocab_size"], hidden), layers, schedule,
                         norm(), "toy.final_norm.", HeadSpec("toy.head.weight", config["vocab_size"], hidden, tied=True))

    register_architecture("ToyStateForCausalLM", build)


TOY_CONFIG = {"architectures": ["ToyStateForCausalLM"], "hidden_size": 40, "intermediate_size": 72, "vocab_size": 90,
              "max_positions": 200, "eps": 1e-5, "decay": 0.8}


# ------------------------------------------------------------------------------ its plain implementation
def plain_toy(weights, ids):
    w = {name: tensor.double() for name, tensor in weights.items()}
    seq, hidden = len(ids), 40
    x = w["toy.embed.weight"][torch.tensor(ids)]
    positions = torch.arange(seq)
    frequencies = plain_impl.rope_inverse_frequencies(16, 1000.0, None)

    def feed_forward(x, prefix):
        normed = plain_impl.rms_norm(x, w[prefix + "norm_b.weight"], 1e-5)
        return x + plain_impl.swiglu(normed, w, prefix + "ff.")

    def decay_layer(x):
        prefix = "toy.layers.0."
        projected = plain_impl.rms_norm(x, w[prefix + "norm_a.weight"], 1e-5) @ w[prefix + "mixer.mix.weight"].T
        state = torch.zeros(hidden, dtype=torch.float64)
        out = []
        for token in range(seq):
            state = 0.8 * state + projected[token]
            out.append(state)
        return feed_forward(x + torch.stack(out), prefix)

    def attention_layer(x, cached=None):
        prefix = "toy.layers.1."
        normed = plain_impl.rms_norm(x, w[prefix + "norm_a.weight"], 1e-5)
        q = plain_impl.linear(normed, w[prefix + "mixer.q_proj.weight"]).reshape(seq, 4, 16)
        q = plain_impl.rope(q, positions, frequencies)
        if cached is None:
            k = plain_impl.linear(normed, w[prefix + "mixer.k_proj.weight"]).reshape(seq, 2, 16)
            v = plain_impl.linear(normed, w[prefix + "mixer.v_proj.weight"]).reshape(seq, 2, 16)
            cached = (plain_impl.rope(k, positions, frequencies), v)
        mixed = plain_impl.attention_scores_softmax_values(q, cached[0], cached[1], 0.25, None)
        x = x + plain_impl.linear(mixed.reshape(seq, -1), w[prefix + "mixer.o_proj.weight"])
        return feed_forward(x, prefix), cached

    x = decay_layer(x)
    x, cached = attention_layer(x)
    x = decay_layer(x)
    x, _ = attention_layer(x, cached)
    return plain_impl.linear(plain_impl.rms_norm(x, w["toy.final_norm.weight"], 1e-5), w["toy.embed.weight"]).numpy()


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 4e-2)])
def test_toy_architecture_is_registered_built_loaded_and_stepped(tmp_path, dtype, tol):
    make_toy()
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    from libmir_b200.config.spec import FixedState, PagedKv
    from libmir_b200.weights import write_model_folder
    folder = write_model_folder(tmp_path, TOY_CONFIG, seed=3, dtype=dtype)
    _, weights = plain_impl.read_model(folder)
    for name in weights:                                   # make the toy's numbers large enough to matter
        if name.endswith("mix.weight"):
            weights[name] = weights[name] * 10
    from libmir_b200.weights import write_file
    write_file(folder / "model.safetensors", weights)
    _, weights = plain_impl.read_model(folder)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=8, block_count=40), dtype=dtype)).load(folder)
    plan = model.decoder.cache_plan()
    assert [type(p.requirement) for p in plan] == [FixedState, PagedKv, FixedState, PagedKv]
    assert [(p.source, p.writes) for p in plan] == [(0, True), (1, True), (2, True), (1, False)]
    assert sorted(model.storage.states) == [0, 2] and len(model.cache.groups[0].entries) == 1
    rng = np.random.default_rng(0)
    first, second = random_ids(rng, 90, 60), random_ids(rng, 90, 45)
    want_first, want_second = plain_toy(weights, first), plain_toy(weights, second)
    model.admit("a")
    model.admit("b")
    got_first, got_second = [], []
    cursor_a = cursor_b = 0
    for size_a, size_b in ((20, 7), (1, 1), (2, 30), (30, 1), (7, 6)):
        result = model.step([StepEntry("a", first[cursor_a:cursor_a + size_a], range(size_a)),
                             StepEntry("b", second[cursor_b:cursor_b + size_b], range(size_b))])
        logits = result.logits.cpu().numpy()
        got_first.append(logits[:size_a])
        got_second.append(logits[size_a:])
        cursor_a += size_a
        cursor_b += size_b
    for got, want in ((np.concatenate(got_first), want_first), (np.concatenate(got_second), want_second)):
        error = np.abs(got - want).max()
        assert error <= tol * max(1.0, np.abs(want).max()), f"max |diff| {error:.3e}"
    # the slot is zeroed when the next request takes it
    model.release("a")
    model.admit("c")
    result = model.step([StepEntry("c", second, range(45))])
    error = np.abs(result.logits.cpu().numpy() - want_second).max()
    assert error <= tol * max(1.0, np.abs(want_second).max()), f"reused slot: max |diff| {error:.3e}"


# ------------------------------------------------------------------------------ a routed feed-forward and another position encoding
@dataclass(frozen=True)
class WaveOffsetSpec:
    """Toy position encoding: q += a sin(p f_d), k += a cos(p f_d) with f_d = 1 / (d + 2)."""

    head_dim: int = 0
    amplitude: float = 0.5
    kind: str = field(init=False, default="toy_wave_offset")


@dataclass(frozen=True)
class RoutedSpec:
    """Toy routed feed-forward: the `top` experts with the largest router logits, weighted by the softmax over
    those logits; an expert is out(relu(in(x)))."""

    hidden_size: int = 0
    inner_size: int = 0
    experts: int = 0
    top: int = 1
    kind: str = field(init=False, default="toy_routed")


def make_routed_toy():
    from libmir_b200 import register_architecture, register_part
    from libmir_b200.config.spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, ParamSpec, RmsNormSpec,
                                         RotarySpec, ScheduleEntry, SoftmaxAttentionSpec, SwiGluSpec)
    from libmir_b200.parts import FeedForward, Position

    class WaveOffset(Position):
        graph_safe = True                                  # reads positions from the device only

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.frequency = 1.0 / (torch.arange(spec.head_dim, dtype=torch.float32, device=env.device) + 2.0)

        def apply(self, ctx, queries, keys):
            angle = ctx.positions[:queries.shape[0]].float()[:, None, None] * self.frequency
            queries.copy_(queries.float() + self.spec.amplitude * torch.sin(angle))
            keys.copy_(keys.float() + self.spec.amplitude * torch.cos(angle))

    class Routed(FeedForward):
        def parameters(self):
            s = self.spec
            return {"router.weight": ParamSpec((s.experts, s.hidden_size), store="float32"),
                    "experts.in": ParamSpec((s.experts, s.inner_size, s.hidden_size)),
                    "experts.out": ParamSpec((s.experts, s.hidden_size, s.inner_size))}

        def bind(self, tensors):
            self.router, self.w_in, self.w_out = (tensors[n] for n in ("router.weight", "experts.in", "experts.out"))

        def forward(self, ctx, x, residual):
            x = x.float()
            logits = x @ self.router.T                                    # 32-bit router
            chosen = logits.topk(self.spec.top, dim=-1)
            share = torch.softmax(chosen.values, dim=-1)
            for expert in range(self.spec.experts):
                tokens, place = (chosen.indices == expert).nonzero(as_tuple=True)
                if tokens.numel():
                    inner = torch.relu(x[tokens] @ self.w_in[expert].float().T)
                    residual.index_add_(0, tokens, (inner @ self.w_out[expert].float().T) * share[tokens, place, None])

    register_part("toy_wave_offset", WaveOffset)
    register_part("toy_routed", Routed)

    def build(config, catalog):
        hidden = config["hidden_size"]
        norm = lambda: RmsNormSpec(size=hidden, eps=config["eps"])
        names = {"mixer_norm": "norm_a.", "mixer": "mixer.", "feed_forward_norm": "norm_b.", "feed_forward": "ff."}
        def attention(position, qk_norm):
            return SoftmaxAttentionSpec(hidden_size=hidden, heads=3, kv_heads=1, head_dim=16, scale=0.25,
                                        qk_norm=qk_norm, qk_norm_eps=1e-5, position=position)
        routed = RoutedSpec(hidden, config["expert_size"], config["experts"], config["top"])
        dense = SwiGluSpec(hidden_size=hidden, intermediate_size=config["intermediate_size"])
        layers = (
            LayerSpec("toy.layers.0.", attention(WaveOffsetSpec(16, 0.5), True), routed, norm(), norm(), names),
            LayerSpec("toy.layers.1.", attention(RotarySpec(head_dim=16, rotary_dim=8, theta=100.0), False), dense,
                      norm(), norm(), names),
            LayerSpec("toy.layers.2.", attention(WaveOffsetSpec(16, 0.25), False), routed, norm(), norm(), names),
        )
        return ModelSpec("ToyRoutedForCausalLM", hidden, config["vocab_size"], config["max_positions"],
                         EmbeddingSpec("toy.embed.weight", config["vocab_size"], hidden), layers,
                         tuple(ScheduleEntry(i) for i in range(3)), norm(), "toy.final_norm.",
                         HeadSpec("toy.head.weight", config["vocab_size"], hidden, tied=False))

    register_architecture("ToyRoutedForCausalLM", build)


ROUTED_CONFIG = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "intermediate_size": 56,
                 "vocab_size": 77, "max_positions": 160, "eps": 1e-5, "experts": 4, "top": 2, "expert_size": 24}


def plain_routed_toy(weights, ids, wave_scale=1.0):
    """Returns the logits and the smallest gap between the last chosen and the first rejected router logit."""
    w = {name: tensor.double() for name, tensor in weights.items()}
    seq = len(ids)
    x = w["toy.embed.weight"][torch.tensor(ids)]
    positions = torch.arange(seq)
    smallest_gap = math.inf

    def attention(x, prefix, qk_norm, encode):
        normed = plain_impl.rms_norm(x, w[prefix + "norm_a.weight"], 1e-5)
        q = plain_impl.linear(normed, w[prefix + "mixer.q_proj.weight"]).reshape(seq, 3, 16)
        k = plain_impl.linear(normed, w[prefix + "mixer.k_proj.weight"]).reshape(seq, 1, 16)
        v = plain_impl.linear(normed, w[prefix + "mixer.v_proj.weight"]).reshape(seq, 1, 16)
        if qk_norm:
            q = plain_impl.rms_norm(q, w[prefix + "mixer.q_norm.weight"], 1e-5)
            k = plain_impl.rms_norm(k, w[prefix + "mixer.k_norm.weight"], 1e-5)
        q, k = encode(q, k)
        mixed = plain_impl.attention_scores_softmax_values(q, k, v, 0.25, None)
        return x + plain_impl.linear(mixed.reshape(seq, -1), w[prefix + "mixer.o_proj.weight"])

    def wave(amplitude):
        angle = positions.double()[:, None, None] / (torch.arange(16, dtype=torch.float64) + 2.0)
        amplitude = amplitude * wave_scale
        return lambda q, k: (q + amplitude * torch.sin(angle), k + amplitude * torch.cos(angle))

    def rotary(q, k):
        frequencies = plain_impl.rope_inverse_frequencies(8, 100.0, None)
        turn = lambda t: torch.cat([plain_impl.rope(t[..., :8], positions, frequencies), t[..., 8:]], dim=-1)
        return turn(q), turn(k)

    def routed(x, prefix):
        nonlocal smallest_gap
        normed = plain_impl.rms_norm(x, w[prefix + "norm_b.weight"], 1e-5)
        logits = normed @ w[prefix + "ff.router.weight"].T
        ordered = logits.sort(dim=-1, descending=True)
        smallest_gap = min(smallest_gap, float((ordered.values[:, 1] - ordered.values[:, 2]).min()))
        share = torch.softmax(ordered.values[:, :2], dim=-1)
        out = torch.zeros_like(x)
        for token in range(seq):
            for place in range(2):
                expert = int(ordered.indices[token, place])
                inner = torch.relu(w[prefix + "ff.experts.in"][expert] @ normed[token])
                out[token] += share[token, place] * (w[prefix + "ff.experts.out"][expert] @ inner)
        return x + out

    x = routed(attention(x, "toy.layers.0.", True, wave(0.5)), "toy.layers.0.")
    x = attention(x, "toy.layers.1.", False, rotary)
    x = x + plain_impl.swiglu(plain_impl.rms_norm(x, w["toy.layers.1.norm_b.weight"], 1e-5), w, "toy.layers.1.ff.")
    x = routed(attention(x, "toy.layers.2.", False, wave(0.25)), "toy.layers.2.")
    logits = plain_impl.linear(plain_impl.rms_norm(x, w["toy.final_norm.weight"], 1e-5), w["toy.head.weight"])
    return logits.numpy(), smallest_gap


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 4e-2)])
def test_toy_routed_feed_forward_and_other_position_encoding(tmp_path, dtype, tol):
    make_routed_toy()
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    from libmir_b200.weights import write_file, write_model_folder
    folder = write_model_folder(tmp_path, ROUTED_CONFIG, seed=12, dtype=dtype)
    _, weights = plain_impl.read_model(folder)
    for name in weights:                     # make the router decisive and the toy parts' numbers matter
        if name.endswith("router.weight"):
            weights[name] = weights[name] * 200
        elif "experts." in name or name.endswith(("q_proj.weight", "k_proj.weight")):
            weights[name] = weights[name] * 8
    write_file(folder / "model.safetensors", weights)
    _, weights = plain_impl.read_model(folder)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=8, block_count=24), dtype=dtype)).load(folder)
    rng = np.random.default_rng(5)
    ids = random_ids(rng, 77, 70)
    want, gap = plain_routed_toy(weights, ids)
    assert gap > 0.2, f"the router's choice is too close to call for a comparison across precisions (gap {gap:.3g})"
    model.admit("a")
    got, cursor = [], 0
    for size in (33, 2, 1, 1, 17, 1, 15):    # portions, then decoded tokens, across page edges
        result = model.step([StepEntry("a", ids[cursor:cursor + size], range(size))])
        got.append(result.logits.cpu().numpy())
        cursor += size
    got = np.concatenate(got)
    error = np.abs(got - want).max()
    assert error <= tol * max(1.0, np.abs(want).max()), f"max |diff| {error:.3e}"
    without_wave = plain_routed_toy(weights, ids, wave_scale=0.0)[0]
    assert np.abs(want - without_wave).max() > 10 * tol * np.abs(want).max(), "the toy position encoding must matter"


# ------------------------------------------------------------------------------ keys and values of different widths
@dataclass(frozen=True)
class NarrowKeySpec:
    """Toy mixer: one-head softmax attention whose keys are `key_dim` wide and whose values are `value_dim` wide
    (a compressed key beside a full value), both in pages of the cache."""

    hidden_size: int = 0
    key_dim: int = 8
    value_dim: int = 24
    kind: str = field(init=False, default="toy_narrow_key")


def make_narrow_key_toy():
    from libmir_b200 import register_architecture, register_part
    from libmir_b200.config.spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PagedKv, ParamSpec, RmsNormSpec,
                                         ScheduleEntry, SwiGluSpec)
    from libmir_b200.parts import Mixer

    class NarrowKeyAttention(Mixer):
        def parameters(self):
            s = self.spec
            return {"q.weight": ParamSpec((s.key_dim, s.hidden_size)), "k.weight": ParamSpec((s.key_dim, s.hidden_size)),
                    "v.weight": ParamSpec((s.value_dim, s.hidden_size)), "o.weight": ParamSpec((s.hidden_size, s.value_dim))}

        def bind(self, tensors):
            self.w = {name.split(".")[0]: tensor.float() for name, tensor in tensors.items()}

        def cache_requirement(self):
            return PagedKv(kv_heads=1, head_dim=self.spec.key_dim, value_head_dim=self.spec.value_dim)

        def forward(self, ctx, cache, x, residual):
            x = x.float()
            group = ctx.groups[cache.group]
            slots = group.slot_mapping[:x.shape[0]].long()
            cache.k_pages[slots, 0] = (x @ self.w["k"].T).to(cache.k_pages.dtype)
            cache.v_pages[slots, 0] = (x @ self.w["v"].T).to(cache.v_pages.dtype)
            queries = x @ self.w["q"].T
            table = group.block_table.cpu()
            page = cache.page_size
            for row in range(ctx.num_rows):
                begin, end = ctx.host_query_starts[row], ctx.host_query_starts[row + 1]
                length = ctx.host_start_positions[row] + (end - begin)
                rows = torch.cat([torch.arange(page) + int(table[row, block]) * page for block in range(-(-length // page))])
                rows = rows[:length].to(x.device)
                keys, values = cache.k_pages[rows, 0].float(), cache.v_pages[rows, 0].float()
                scores = queries[begin:end] @ keys.T
                positions = torch.arange(ctx.host_start_positions[row], length, device=x.device)
                scores = scores.masked_fill(torch.arange(length, device=x.device)[None, :] > positions[:, None], float("-inf"))
                residual[begin:end] += (torch.softmax(scores, dim=-1) @ values) @ self.w["o"].T

    register_part("toy_narrow_key", NarrowKeyAttention)

    def build(config, catalog):
        hidden = config["hidden_size"]
        norm = lambda: RmsNormSpec(size=hidden, eps=1e-5)
        names = {"mixer_norm": "norm_a.", "mixer": "mixer.", "feed_forward_norm": "norm_b.", "feed_forward": "ff."}
        layers = (LayerSpec("toy.layers.0.", NarrowKeySpec(hidden, config["key_dim"], config["value_dim"]),
                            SwiGluSpec(hidden_size=hidden, intermediate_size=config["intermediate_size"]), norm(), norm(),
                            names),)
        return ModelSpec("ToyNarrowKeyForCausalLM", hidden, config["vocab_size"], 128,
                         EmbeddingSpec("toy.embed.weight", config["vocab_size"], hidden), layers, (ScheduleEntry(0),),
                         norm(), "toy.final_norm.", HeadSpec("toy.head.weight", config["vocab_size"], hidden, tied=True))

    register_architecture("ToyNarrowKeyForCausalLM", build)


NARROW_CONFIG = {"architectures": ["ToyNarrowKeyForCausalLM"], "hidden_size": 32, "intermediate_size": 40,
                 "vocab_size": 50, "key_dim": 8, "value_dim": 24}


def plain_narrow_key_toy(weights, ids):
    w = {name: tensor.double() for name, tensor in weights.items()}
    x = w["toy.embed.weight"][torch.tensor(ids)]
    prefix = "toy.layers.0."
    normed = plain_impl.rms_norm(x, w[prefix + "norm_a.weight"], 1e-5)
    q, k, v = (normed @ w[prefix + f"mixer.{name}.weight"].T for name in "qkv")
    scores = (q @ k.T).masked_fill(torch.triu(torch.ones(len(ids), len(ids), dtype=torch.bool), 1), float("-inf"))
    x = x + (torch.softmax(scores, dim=-1) @ v) @ w[prefix + "mixer.o.weight"].T
    x = x + plain_impl.swiglu(plain_impl.rms_norm(x, w[prefix + "norm_b.weight"], 1e-5), w, prefix + "ff.")
    return plain_impl.linear(plain_impl.rms_norm(x, w["toy.final_norm.weight"], 1e-5), w["toy.embed.weight"]).numpy()


def test_toy_mixer_with_keys_and_values_of_different_widths(tmp_path):
    """The cache requirement names a key width and a value width; the storage gives the mixer pages of each width,
    and the cache manager, the step function and the scheduler's cuts need to know nothing about it."""
    make_narrow_key_toy()
    from libmir_b200 import CacheConfig, Library, RuntimeConfig, StepEntry
    from libmir_b200.weights import write_file, write_model_folder
    folder = write_model_folder(tmp_path, NARROW_CONFIG, seed=7, dtype="float32")
    _, weights = plain_impl.read_model(folder)
    for name in weights:
        if ".mixer." in name:
            weights[name] = weights[name] * 20
    write_file(folder / "model.safetensors", weights)
    _, weights = plain_impl.read_model(folder)
    model = Library(RuntimeConfig(kv_cache=CacheConfig(block_size=4, block_count=24), dtype="float32")).load(folder)
    assert model.storage.key_buffers[0].shape[-2:] == (1, 8) and model.storage.value_buffers[0].shape[-2:] == (1, 24)
    stats = model.cache_stats()["groups"][0]
    assert (stats["head_dim"], stats["value_head_dim"]) == (8, 24)
    ids = random_ids(np.random.default_rng(3), 50, 37)
    want = plain_narrow_key_toy(weights, ids)
    model.admit("a")
    got, cursor = [], 0
    for size in (9, 1, 2, 13, 1, 11):
        got.append(model.step([StepEntry("a", ids[cursor:cursor + size], range(size))]).logits.cpu().numpy())
        cursor += size
    error = np.abs(np.concatenate(got) - want).max()
    assert error <= 3e-5 * max(1.0, np.abs(want).max()), f"max |diff| {error:.3e}"
