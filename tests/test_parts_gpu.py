"""Each part alone on the device against the plain function of the same part, at sizes of its own."""

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_impl

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2.5e-2}


def env(dtype):
    from libmir_b200.parts import BuildEnv
    return BuildEnv(dtype, torch.device("cuda"))


def harness(requirement, dtype, page_size=8, pages=32, vocab=100):
    """A step runner around one cache entry, so that a single mixer can be stepped."""
    from libmir_b200.cache import CacheManager, CacheStorage
    from libmir_b200.engine.step import StepRunner
    from libmir_b200.models.decoder import CacheEntryPlan
    plan = [CacheEntryPlan(0, requirement, 0, True)]
    manager = CacheManager(plan, page_size, pages, 4)
    storage = CacheStorage(manager, plan, dtype, torch.device("cuda"))
    model = SimpleNamespace(spec=SimpleNamespace(vocab_size=vocab, max_positions=4096), env=env(dtype))
    return StepRunner(model, manager, storage, torch.device("cuda")), manager


def bind_random(part, dtype, seed=0, std=0.3):
    torch.manual_seed(seed)
    host, tensors = {}, {}
    for name, spec in part.parameters().items():
        value = torch.randn(spec.shape) * std + (1.0 if spec.init == "ones" else 0.0)
        target = torch.float32 if spec.store == "float32" else dtype
        value = value.to(target)
        host[name] = value
        tensors[name] = value.cuda()
    part.bind(tensors)
    return host


def close(got, want, dtype, factor=1.0):
    want, got = want.double().cpu(), got.double().cpu()
    bound = TOL[dtype] * factor * max(1.0, float(want.abs().max()))
    error = float((got - want).abs().max())
    assert torch.isfinite(got).all() and error <= bound, f"max |diff| {error:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from libmir_b200.config.spec import RmsNormSpec
    from libmir_b200.engine.context import Arena
    from libmir_b200.parts import ScratchContext
    from libmir_b200.registry import build_part
    part = build_part(RmsNormSpec(size=136, eps=2e-4), env(dtype))
    weights = bind_random(part, dtype)
    x = torch.randn(5, 136) * 2
    ctx = ScratchContext(Arena(torch.device("cuda")).alloc, dtype)
    out = part.forward(ctx, x.cuda())
    assert out.dtype == dtype
    close(out, plain_impl.rms_norm(x.double(), weights["weight"], 2e-4), dtype)


def test_rotary_table_with_llama3_scaling():
    from libmir_b200.config import RopeScaling
    from libmir_b200.config.spec import RotarySpec
    from libmir_b200.registry import build_part
    scaling = RopeScaling(8.0, 1.0, 4.0, 64)
    part = build_part(RotarySpec(head_dim=64, rotary_dim=32, theta=5e5, scaling=scaling), env(torch.float32))
    expected = plain_impl.rope_inverse_frequencies(32, 5e5, {"factor": 8.0, "low_freq_factor": 1.0,
                                                             "high_freq_factor": 4.0,
                                                             "original_max_position_embeddings": 64})
    assert part.rotary_dim == 32 and torch.equal(part.table.cpu(), expected)
    plain = plain_impl.rope_inverse_frequencies(32, 5e5, None)
    assert (expected < plain).any() and (expected == plain).any()        # some slowed, the fastest kept


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from libmir_b200.config.spec import SwiGluSpec
    from libmir_b200.engine.context import Arena
    from libmir_b200.parts import ScratchContext
    from libmir_b200.registry import build_part
    part = build_part(SwiGluSpec(hidden_size=72, intermediate_size=200), env(dtype))
    weights = bind_random(part, dtype, std=0.15)
    x = torch.randn(9, 72).to(dtype)
    residual = torch.randn(9, 72)
    device_residual = residual.clone().cuda()
    ctx = ScratchContext(Arena(torch.device("cuda")).alloc, dtype)
    part.forward(ctx, x.cuda(), device_residual)
    expected = residual.double() + plain_impl.swiglu(x.double(), weights, "")
    close(device_residual, expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("options", [
    dict(heads=6, kv_heads=2, head_dim=32, qk_norm=True, qkv_bias=False, out_bias=False, window=None, rotary=32),
    dict(heads=4, kv_heads=4, head_dim=16, qk_norm=False, qkv_bias=True, out_bias=True, window=21, rotary=8),
    dict(heads=3, kv_heads=1, head_dim=80, qk_norm=True, qkv_bias=True, out_bias=False, window=None, rotary=0),
])
def test_attention_part_in_portions(dtype, options):
    """The mixer alone: one request fed in three portions, against plain attention of the whole sequence."""
    from libmir_b200.config.spec import RotarySpec, SoftmaxAttentionSpec
    from libmir_b200.engine.step import StepEntry
    from libmir_b200.registry import build_part
    hidden, o = 88, options
    position = RotarySpec(head_dim=o["head_dim"], rotary_dim=o["rotary"], theta=1e4) if o["rotary"] else None
    spec = SoftmaxAttentionSpec(hidden_size=hidden, heads=o["heads"], kv_heads=o["kv_heads"], head_dim=o["head_dim"],
                                scale=0.5 / math.sqrt(o["head_dim"]), qk_norm=o["qk_norm"], qk_norm_eps=1e-5,
                                qkv_bias=o["qkv_bias"], out_bias=o["out_bias"], window=o["window"], position=position)
    part = build_part(spec, env(dtype))
    weights = bind_random(part, dtype, std=0.2)
    runner, manager = harness(part.cache_requirement(), dtype)
    seq = 50
    x = torch.randn(seq, hidden).to(dtype)
    residual = torch.randn(seq, hidden)
    manager.admit("r")
    outputs = []
    cursor = 0
    for size in (23, 1, 26):
        entries, sequences = runner.reserve([StepEntry("r", [0] * size, [])])
        runner.arena.reset()
        ctx, _, _ = runner.build_context(entries, sequences)
        part_residual = residual[cursor:cursor + size].clone().cuda()
        part.forward(ctx, ctx.cache_view(0), x[cursor:cursor + size].cuda(), part_residual)
        runner.commit(entries, sequences)
        outputs.append(part_residual.cpu())
        cursor += size
    s = dict(heads=o["heads"], kv_heads=o["kv_heads"], head_dim=o["head_dim"], eps=1e-5, rotary_dim=o["rotary"],
             theta=1e4, scaling=None, scale=spec.scale)
    if not o["rotary"]:
        s["rotary_dim"] = 0
    expected = residual.double() + plain_impl.attention(x.double(), weights, "", s, torch.arange(seq), o["window"])
    close(torch.cat(outputs), expected, dtype, factor=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    from libmir_b200.config.spec import LayerSpec, RmsNormSpec, RotarySpec, SoftmaxAttentionSpec, SwiGluSpec
    from libmir_b200.engine.step import StepEntry
    from libmir_b200.parts import build_block
    hidden = 48
    names = {"mixer_norm": "n1.", "mixer": "att.", "feed_forward_norm": "n2.", "feed_forward": "ff."}
    layer = LayerSpec(prefix="", names=names,
                      mixer=SoftmaxAttentionSpec(hidden_size=hidden, heads=2, kv_heads=1, head_dim=24, scale=0.2,
                                                 position=RotarySpec(head_dim=24, rotary_dim=24, theta=100.0)),
                      feed_forward=SwiGluSpec(hidden_size=hidden, intermediate_size=100),
                      mixer_norm=RmsNormSpec(size=hidden, eps=1e-5), feed_forward_norm=RmsNormSpec(size=hidden, eps=1e-5))
    block = build_block(layer, env(dtype))
    weights = {}
    for slot, part in block.parts():
        for name, value in bind_random(part, dtype, seed=len(weights), std=0.2).items():
            weights["model.layers.0." + {"n1.": "input_layernorm.", "att.": "self_attn.",
                                         "n2.": "post_attention_layernorm.", "ff.": "mlp."}[names[slot]] + name] = value
    runner, manager = harness(block.cache_requirement(), dtype)
    x = torch.randn(19, hidden)
    manager.admit("r")
    entries, sequences = runner.reserve([StepEntry("r", [0] * 19, [])])
    runner.arena.reset()
    ctx, _, _ = runner.build_context(entries, sequences)
    residual = x.clone().cuda()
    block.forward(ctx, ctx.cache_view(0), residual)
    s = dict(heads=2, kv_heads=1, head_dim=24, eps=1e-5, rotary_dim=24, theta=100.0, scaling=None, scale=0.2,
             windows=[None])
    close(residual, plain_impl.block(x.double(), weights, 0, s, torch.arange(19)), dtype, factor=2)
