"""The description a model is built from: data only, no tensors and no kernels.

An architecture's builder (libmir_b200/models) turns its config.json into a ModelSpec:
a list of LayerSpec, each naming the kind and the numbers of its mixer, feed-forward,
norms and position encoding, and a schedule, the order in which the layers run.
Parts are looked up by `kind` in the part registry, so a layer may use any registered
mixer or feed-forward, and different layers may use different ones.

The seams follow libmir's semantic model: MixerSpec / FeedForwardSpec /
PositionEncodingSpec / NormalizationKind (models/src/semantic/attention.rs:5-9,111-124,
feed_forward.rs:5-30, model.rs:110-115).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Union

from ..errors import ConfigError


# --------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class TensorSource:
    """Another way a checkpoint may store a wanted tensor: as rows [rows[0], rows[1]) of the stored tensor
    `name` (a name local to the part, like the key of the ParamSpec that lists this source), which has
    `total_rows` rows in all.  libmir splits a fused `self_attn.qkv_proj.weight` / `query_key_value.weight`
    into query, key and value rows this way (models/src/weights/binding/shapes/transforms.rs:22-35)."""

    name: str
    rows: tuple
    total_rows: int


@dataclass(frozen=True)
class ParamSpec:
    """One tensor that a part wants from the checkpoint.

    `store` says how it is kept on the device: "compute" follows the engine's dtype
    (bfloat16 or float32), "float32" is kept in 32-bit whatever the engine's dtype
    (norm weights and biases: small, and exact for every stored dtype), "int32" is an
    integer table.  `init` is what the random-weights writer fills it with.
    """

    shape: tuple
    init: str = "normal"          # "normal" N(0, 0.02), "ones", "zeros"
    store: str = "compute"        # "compute" | "float32" | "int32"
    optional: bool = False        # absent from the checkpoint is fine (bias, q/k-norm discovery)
    sources: tuple = ()           # TensorSource: other stored tensors this one may be cut from
    # A 2-d tensor stored with its two dimensions swapped ([in, out] for [out, in]) is recognised by its shape
    # and transposed while loading (transforms.rs:52-58); a square tensor is always taken as stored.
    accept_transposed: bool = True


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKv:
    """Keys and values of every token in pages; with a window only the last `window` are kept.  Keys are
    `head_dim` wide; values too unless `value_head_dim` says otherwise (libmir's KvStorageSpec has both widths,
    cuda/src/backend/kv/storage/mod.rs:17-25)."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.value_head_dim is None else self.value_head_dim

    @property
    def elements_per_token(self) -> int:
        """Cached elements per token and schedule entry: keys and values of every kv head."""
        return self.kv_heads * (self.head_dim + self.value_dim)


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, kept in the request's state slot."""

    shape: tuple
    dtype: str = "float32"


CacheRequirement = Union[PagedKv, FixedState, None]


# --------------------------------------------------------------------------- parts
@dataclass(frozen=True)
class PartSpec:
    """Base of every part description; `kind` selects the implementation in the registry."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class RmsNormSpec(PartSpec):
    size: int = 0
    eps: float = 1e-5
    kind: str = field(init=False, default="rms_norm")


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Half-split rotary position encoding of the first `rotary_dim` dims of a head."""

    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Any = None           # config.RopeScaling or None
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class SoftmaxAttentionSpec(PartSpec):
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    qkv_bias: bool = False
    out_bias: bool = False
    window: Optional[int] = None
    position: Optional[PartSpec] = None
    kind: str = field(init=False, default="softmax_attention")


@dataclass(frozen=True)
class SwiGluSpec(PartSpec):
    hidden_size: int = 0
    intermediate_size: int = 0
    kind: str = field(init=False, default="swiglu")


# --------------------------------------------------------------------------- layers and model
@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement of a mixer and a feed-forward with their norms.

    `prefix` is the checkpoint prefix of the layer; `names` maps each slot of the
    arrangement to the sub-prefix of its tensors, so names are data of the architecture.
    """

    prefix: str
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: Optional[PartSpec]
    feed_forward_norm: Optional[PartSpec]
    names: Mapping[str, str]
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes ModelSpec.layers and may repeat.

    Every entry has a cache of its own unless `cache_of` names an earlier entry (by its
    index in the schedule) whose cache it reads without writing to it.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    name: str
    vocab_size: int
    hidden_size: int
    multiplier: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """Output projection; `tied_to` names the embedding tensor it shares, else `name` is its own."""

    name: str
    vocab_size: int
    hidden_size: int
    tied: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    final_norm_name: str
    head: HeadSpec
    strip_prefixes: tuple = ()      # checkpoint prefixes that may wrap every name

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule entry {index} names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ConfigError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                                      "which must be an earlier entry")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                                      "which has no cache of its own")
