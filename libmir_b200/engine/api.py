"""The programming interface: Library -> Model -> generate / Session, in libmir's manner.

libmir (README.md:42-106, src/model/library/mod.rs:45-146, src/generation/mod.rs:29-49,
src/session/mod.rs:16-181, examples/incremental.rs:16-38):
    Library::new(RuntimeConfig); library.load(path, overrides, progress) -> Model
    model.generate(request, progress, on_token) -> GenerationOutput{text, token_ids, finish_reason, metrics}
    model.session() -> Session; session.prefill(ids, SamplingLogits) ; session.decode(token, SamplingLogits)
    session.cache_stats(); model.unload()
Here requests are token ids in and token ids out (tokenizers and chat templates are not part of the
engine), `generate_batch` runs several requests through the scheduler at once, and `Model.step` is
the raw step function that the trace replay drives.
"""

from __future__ import annotations

import itertools
import json
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache import CacheManager, CacheStorage
from ..config.generation import DEFAULT_SEED, GenerationConfig, GenerationOverrides, GenerationSettings
from ..config.runtime import RuntimeConfig
from ..errors import ConfigError, KernelError, SchedulerError
from ..models.decoder import DecoderModel
from ..parts.base import BuildEnv
from ..registry import build_spec
from ..sampling.sampler import DeviceSampler, RequestSampler
from ..weights import bind_random, catalog_shapes, load_into
from .scheduler import Request, Scheduler
from .step import StepEntry, StepResult, StepRunner

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class SamplingLogits:
    """What a Session call returns: a sampled token, or the full logits of the last position
    (runtime/src/backend/traits.rs: SamplingLogits::{None, Sample, Full})."""

    TOKEN = "token"
    FULL = "logits"


@dataclass
class GenerationRequest:
    prompt_ids: Sequence[int]
    options: GenerationOverrides = field(default_factory=GenerationOverrides)
    seed: Optional[int] = None
    request_id: Optional[object] = None


@dataclass
class GenerationOutput:
    token_ids: List[int]
    finish_reason: str
    metrics: Dict[str, float] = field(default_factory=dict)
    request_id: Optional[object] = None


@dataclass
class PrefillOutput:
    next_token: Optional[int] = None
    logits: Optional[np.ndarray] = None      # float32 [vocab]
    cached_tokens: int = 0                   # tokens of the session in the cache after the call
    reused_tokens: int = 0                   # of these, found in the prefix cache instead of computed


DecodeOutput = PrefillOutput


def _require_gpu(ordinal: int) -> torch.device:
    if not torch.cuda.is_available():
        raise KernelError("libmir_b200 runs on an NVIDIA B200 (sm_100a) only: no CUDA device is visible, and "
                          "there is no CPU path")
    device = torch.device("cuda", ordinal)
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise KernelError(f"libmir_b200's kernels are compiled for sm_100a; device {ordinal} is sm_{major}{minor}")
    return device


class Library:
    """Entry point: holds the runtime configuration and loads models."""

    def __init__(self, config: Optional[RuntimeConfig] = None):
        self.config = config or RuntimeConfig()
        self.config.validate()
        self.models: List["Model"] = []

    def load(self, path, overrides: Optional[GenerationOverrides] = None,
             progress: Optional[Callable[[str], None]] = None) -> "Model":
        """Load a model folder (config.json + safetensors)."""
        folder = Path(path)
        config_path = folder / "config.json"
        if not config_path.is_file():
            raise ConfigError(f"missing file {config_path}")
        config_json = json.loads(config_path.read_text())
        device = _require_gpu(self.config.cuda.device_ordinal)
        spec = build_spec(config_json, catalog_shapes(folder))
        env = BuildEnv(_TORCH_DTYPES[self.config.dtype], device)
        if progress:
            progress(f"building {spec.architecture}")
        decoder = DecoderModel(spec, env)
        with torch.cuda.device(device):
            load_into(decoder, folder, strict=self.config.strict_weights)
        generation = GenerationConfig.from_folder(folder)
        model = Model(self, decoder, generation, overrides, config_json)
        self.models.append(model)
        return model

    def load_random(self, config_json: Mapping, seed: int = 0,
                    overrides: Optional[GenerationOverrides] = None) -> "Model":
        """Build the model that config_json describes with random weights made on the device."""
        device = _require_gpu(self.config.cuda.device_ordinal)
        spec = build_spec(config_json, None)
        decoder = DecoderModel(spec, BuildEnv(_TORCH_DTYPES[self.config.dtype], device))
        with torch.cuda.device(device):
            bind_random(decoder, seed)
        model = Model(self, decoder, GenerationConfig(), overrides, dict(config_json))
        self.models.append(model)
        return model


class Model:
    def __init__(self, library: Library, decoder: DecoderModel, generation: GenerationConfig,
                 overrides: Optional[GenerationOverrides], config_json: Mapping):
        self.library = library
        self.decoder = decoder
        self.spec = decoder.spec
        self.generation_config = generation
        self.default_overrides = overrides or GenerationOverrides()
        self.config_json = dict(config_json)
        runtime = library.config
        self.device = decoder.env.device
        plan = decoder.cache_plan()
        self.cache = CacheManager(plan, runtime.kv_cache.block_size, runtime.kv_cache.block_count,
                                  runtime.scheduler.max_batch_requests, prefix_cache=runtime.kv_cache.prefix_cache,
                                  model_key=f"{decoder.env.dtype}:{id(self)}")
        with torch.cuda.device(self.device):
            self.storage = CacheStorage(self.cache, plan, decoder.env.dtype, self.device)
            self.runner = StepRunner(decoder, self.cache, self.storage, self.device,
                                     decode_graphs=runtime.cuda.decode_graphs)
        self.sampler = self.runner.sampler
        self._ids = itertools.count()
        self._unloaded = False

    # -- the raw step (trace replay, tests) ------------------------------------------
    def admit(self, request_id, tokens: Optional[Sequence[int]] = None) -> int:
        """Make a request live.  With `tokens` (what it will be fed) and a prefix cache, the pages that hold its first
        tokens already are taken over; returns how many tokens that is: feed the request from there."""
        return self.cache.admit(request_id, tokens).length

    def release(self, request_id) -> None:
        self.cache.release(request_id)

    def step(self, entries: Sequence[StepEntry], samplers: Optional[Sequence[RequestSampler]] = None) -> StepResult:
        """Run one batch of (request, next tokens); every request must have been admitted.  With
        `samplers`, one per wanted row, the result also carries the sampled tokens."""
        with torch.cuda.device(self.device):
            return self.runner.step(entries, samplers)

    # -- profiling, in libmir's manner (src/engine/profile.rs:46-90, cuda/src/engine/mod.rs:75-103) -------------
    def set_profile_decode(self, enabled: bool) -> None:
        """While on, every decode step (one token per request) carries DecodeTimings (StepResult.timings, kept in
        runner.decode_timings; generate's metrics add them up), and an accelerator-profiler capture range is open."""
        if enabled:
            self.start_profiler_capture()
            self.runner.profile_decode = True
            return
        self.runner.profile_decode = False
        self.stop_profiler_capture()

    def start_profiler_capture(self) -> None:
        """Opens a capture range for an attached profiler (cudaProfilerStart) without changing what runs."""
        if not getattr(self, "_capturing", False):
            torch.cuda.profiler.start()
            self._capturing = True

    def stop_profiler_capture(self) -> None:
        if getattr(self, "_capturing", False):
            torch.cuda.profiler.stop()
            self._capturing = False

    def decode_many(self, entries: Sequence[StepEntry], samplers: Sequence[RequestSampler], steps: int):
        """Several greedy decode steps back to back on the device; see StepRunner.decode_many."""
        with torch.cuda.device(self.device):
            return self.runner.decode_many(entries, samplers, steps)

    # -- generation ----------------------------------------------------------------------
    def _settings(self, options: Optional[GenerationOverrides]) -> GenerationSettings:
        merged = GenerationOverrides(**{
            key: getattr(options, key) if options is not None and getattr(options, key) is not None
            else getattr(self.default_overrides, key)
            for key in GenerationOverrides.__dataclass_fields__})
        return self.generation_config.resolve(merged)

    def _run_and_sample(self, entries: Sequence[StepEntry], samplers: Sequence[RequestSampler]) -> List[int]:
        result = self.step(entries, samplers)
        return result.tokens.cpu().tolist() if result.tokens is not None else []

    def _scheduler(self) -> Scheduler:
        return Scheduler(self.cache, self.library.config.scheduler, self.spec.max_positions, self._run_and_sample,
                         portion_multiple=self.decoder.portion_multiple())

    def generate_batch(self, requests: Sequence[GenerationRequest],
                       on_token: Optional[Callable[[object, int], None]] = None) -> List[GenerationOutput]:
        """Run requests together through the scheduler; outputs come back in the order given."""
        self._check_loaded()
        scheduler = self._scheduler()
        started = time.perf_counter()
        first_timing = len(self.runner.decode_timings)
        records = []
        for request in requests:
            settings = self._settings(request.options)
            request_id = request.request_id if request.request_id is not None else f"g{next(self._ids)}"
            callback = (lambda token, rid=request_id: on_token(rid, token)) if on_token else None
            record = Request(request_id, [int(t) for t in request.prompt_ids], settings,
                             RequestSampler.from_settings(settings, request.seed), callback)
            scheduler.submit(record)
            records.append(record)
        try:
            with torch.cuda.device(self.device):
                scheduler.run()
        finally:
            scheduler.abandon()          # after a step that raised: nothing of this call stays live in the shared cache
        elapsed = time.perf_counter() - started
        generated = sum(len(r.output) for r in records)
        profile = {}
        if self.runner.profile_decode:
            timings = self.runner.decode_timings[first_timing:]
            profile = {"decode_steps_profiled": len(timings),
                       "decode_backend_seconds": sum(t.backend_execution for t in timings),
                       "decode_device_seconds": sum(t.device_execution for t in timings)}
        outputs = []
        for record in records:
            outputs.append(GenerationOutput(list(record.output), record.finish_reason or "unknown", {
                "seconds": elapsed, "steps": scheduler.steps, "prompt_tokens": len(record.prompt),
                "generated_tokens": len(record.output), "preemptions": record.preemptions,
                "cached_prompt_tokens": record.cached_tokens,
                "batch_tokens_per_second": generated / elapsed if elapsed > 0 else 0.0, **profile,
            }, record.request_id))
        return outputs

    def generate(self, request: GenerationRequest,
                 on_token: Optional[Callable[[int], None]] = None) -> GenerationOutput:
        callback = (lambda _rid, token: on_token(token)) if on_token else None
        return self.generate_batch([request], callback)[0]

    def session(self) -> "Session":
        self._check_loaded()
        return Session(self)

    def clear_prefix_cache(self) -> int:
        """Forget the cached prefixes of this model (libmir: Engine::clear_prefix_cache, src/engine/mod.rs:187-200)."""
        return self.cache.clear_prefix()

    def cache_stats(self) -> dict:
        return self.cache.stats()

    def unload(self) -> None:
        """Drop the weights and the cache (src/model/lifecycle.rs:38-49)."""
        self._unloaded = True
        for request_id in list(self.cache.live):
            self.cache.release(request_id)
        self.storage = None
        self.runner = None
        self.decoder = None
        if self in self.library.models:
            self.library.models.remove(self)
        torch.cuda.empty_cache()

    def _check_loaded(self) -> None:
        if self._unloaded:
            raise SchedulerError("the model was unloaded")


class Session:
    """One request's cache, driven by hand: prefill, then decode token by token."""

    def __init__(self, model: Model):
        self.model = model
        self.request_id = f"s{next(model._ids)}"
        model.admit(self.request_id)
        self.sampler = RequestSampler()
        self._open = True

    def _run(self, tokens: Sequence[int], want: str) -> PrefillOutput:
        if not self._open:
            raise SchedulerError("the session is closed")
        tokens = [int(t) for t in tokens]
        reused = 0
        cache = self.model.cache
        if cache.prefix is not None and cache.live[self.request_id].length == 0 and len(tokens) > 1:
            # a prompt into an empty session: take over the pages that hold its first tokens already
            self.model.release(self.request_id)
            reused = self.model.admit(self.request_id, tokens)
        entry = StepEntry(self.request_id, tokens[reused:], [len(tokens) - reused - 1])
        if want == SamplingLogits.FULL:
            result = self.model.step([entry])
            cached = cache.live[self.request_id].length
            return PrefillOutput(logits=result.logits[0].float().cpu().numpy(), cached_tokens=cached, reused_tokens=reused)
        self.sampler.observe(tokens)
        result = self.model.step([entry], [self.sampler])
        cached = cache.live[self.request_id].length
        return PrefillOutput(next_token=int(result.tokens.cpu()[0]), cached_tokens=cached, reused_tokens=reused)

    def prefill(self, prompt_ids: Sequence[int], sampling: str = SamplingLogits.TOKEN,
                settings: Optional[GenerationSettings] = None, seed: Optional[int] = None) -> PrefillOutput:
        if settings is not None:
            self.sampler = RequestSampler.from_settings(settings, seed)
        return self._run(prompt_ids, sampling)

    def decode(self, token: int, sampling: str = SamplingLogits.TOKEN) -> DecodeOutput:
        return self._run([token], sampling)

    def cache_stats(self) -> dict:
        stats = self.model.cache.stats()
        stats["cached_tokens"] = self.model.cache.live[self.request_id].length if self._open else 0
        return stats

    def close(self) -> None:
        if self._open:
            self.model.release(self.request_id)
            self._open = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
