"""Runtime options, as typed structures only: nothing is read from the process environment
(libmir's rule, AGENTS.md:107-110).  Names and defaults follow src/config.rs:11-46,
runtime/src/kv/cache/types.rs:57-66, runtime/src/scheduler.rs:80-91,159-172 and
cuda/src/backend/model/config.rs:3."""

from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import ConfigError

DTYPES = ("bfloat16", "float32")


@dataclass
class CacheConfig:
    block_size: int = 16          # tokens in one page
    block_count: int = 4096       # pages in every group's pool
    prefix_cache: bool = False    # full pages are remembered by their tokens and shared by requests that start alike

    def validate(self) -> None:
        if self.block_size <= 0 or self.block_count <= 0:
            raise ConfigError("block_size and block_count must be greater than zero")


@dataclass
class SchedulerConfig:
    max_batch_requests: int = 16      # live requests (and state slots)
    max_batch_tokens: int = 8192      # tokens in one step
    prefill_chunk_tokens: int = 2096  # the longest portion of one prompt in one step
    reserve_tokens: int = 0           # tokens of growth reserved at admission (0 = pages on demand)
    out_of_pages: str = "preempt"     # "preempt" (youngest is recomputed later) or "finish" (reason out_of_pages)

    def validate(self) -> None:
        if self.max_batch_requests <= 0 or self.max_batch_tokens <= 0 or self.prefill_chunk_tokens <= 0:
            raise ConfigError("max_batch_requests, max_batch_tokens and prefill_chunk_tokens must be greater than zero")
        if self.out_of_pages not in ("preempt", "finish"):
            raise ConfigError("out_of_pages must be 'preempt' or 'finish'")


@dataclass
class CudaConfig:
    device_ordinal: int = 0
    decode_graphs: bool = True        # capture decode-only steps of bucketed sizes as CUDA graphs


@dataclass
class RuntimeConfig:
    kv_cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    cuda: CudaConfig = field(default_factory=CudaConfig)
    dtype: str = "bfloat16"           # "bfloat16": the serving kernels; "float32": everything in true 32-bit
    strict_weights: bool = False      # a stored tensor that the model does not ask for is an error, not auxiliary

    def validate(self) -> None:
        if self.dtype not in DTYPES:
            raise ConfigError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        self.kv_cache.validate()
        self.scheduler.validate()
