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
