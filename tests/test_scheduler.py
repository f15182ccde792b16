"""The scheduler's decisions with the real cache manager and a step function that runs nothing (no GPU)."""

import pytest
import torch

from libmir_b200 import KvCapacity, SchedulerError, build_spec
from libmir_b200.cache import CacheManager
from libmir_b200.config import GenerationSettings, SchedulerConfig
from libmir_b200.engine.scheduler import Request, Scheduler
from libmir_b200.engine.step import StepResult, StepRunner
from libmir_b200.models.decoder import DecoderModel
from libmir_b200.parts.base import BuildEnv
from libmir_b200.sampling import RequestSampler
from tiny_configs import TINY_A, TINY_C


class HostOnlyRunner(StepRunner):
    """The real reserve/commit on the host; the device part is replaced by a record of what ran."""

    def __init__(self, model, manager):
        super().__init__(model, manager, None, torch.device("cpu"))
        self.ran = []

    def execute(self, entries, sequences, samplers=None):
        self.ran.append([(e.request_id, seq.length, len(e.tokens), list(e.want)) for e, seq in zip(entries, sequences)])
        keys = [(e.request_id, w) for e in entries for w in e.want]
        return StepResult(None, keys, sum(len(e.tokens) for e in entries))


def build(config=TINY_A, pages=64, page_size=4, prefix_cache=False, **scheduler_options):
    model = DecoderModel(build_spec(config), BuildEnv(torch.float32, torch.device("meta")))
    options = SchedulerConfig(**scheduler_options)
    manager = CacheManager(model.cache_plan(), page_size, pages, options.max_batch_requests,
                           prefix_cache=prefix_cache, model_key="tiny")
    runner = HostOnlyRunner(model, manager)
    counter = {"n": 0}

    def sample(result, samplers):
        out = []
        for _ in samplers:
            counter["n"] += 1
            out.append(100 + counter["n"] % 50)
        return out

    def run_step(entries, samplers):
        runner.step(entries)
        return run_step.sample(None, samplers)

    run_step.sample = sample
    scheduler = Scheduler(manager, options, model.spec.max_positions, run_step)
    return scheduler, runner, manager


def request(name, prompt_len, max_tokens, stop=(), **kw):
    settings = GenerationSettings(max_tokens=max_tokens, stop_token_ids=tuple(stop), **kw)
    return Request(name, list(range(1, prompt_len + 1)), settings, RequestSampler())


def test_prompt_is_cut_into_portions_under_the_token_budget():
    scheduler, runner, manager = build(max_batch_tokens=16, prefill_chunk_tokens=10)
    scheduler.submit(request("a", 23, 2))
    scheduler.run()
    portions = [[(rid, start, count) for rid, start, count, _ in step] for step in runner.ran]
    assert portions == [[("a", 0, 10)], [("a", 10, 10)], [("a", 20, 3)], [("a", 23, 1)]]
    assert runner.ran[1][0][3] == [] and runner.ran[2][0][3] == [2]      # logits only where the prompt ends
    assert scheduler.finished[0].finish_reason == "length" and len(scheduler.finished[0].output) == 2
    assert manager.groups[0].pool.free == 64 and manager.free_slots == 16
    manager.check()


def test_decode_rows_come_first_and_prompts_get_the_rest():
    scheduler, runner, _ = build(max_batch_tokens=12, prefill_chunk_tokens=100)
    scheduler.submit(request("a", 5, 6))
    scheduler.step()                                  # a's whole prompt
    scheduler.submit(request("b", 30, 2))
    scheduler.step()
    assert runner.ran[1] == [("a", 5, 1, [0]), ("b", 0, 11, [])]        # budget 12 - 1 decode row
    scheduler.step()
    assert runner.ran[2] == [("a", 6, 1, [0]), ("b", 11, 11, [])]
    scheduler.step()
    assert runner.ran[3] == [("a", 7, 1, [0]), ("b", 22, 8, [7])]
    scheduler.step()
    assert [e[:3] for e in runner.ran[4]] == [("a", 8, 1), ("b", 30, 1)]


def test_completion_first_oldest_prompt_takes_the_budget():
    scheduler, runner, _ = build(max_batch_tokens=20, prefill_chunk_tokens=100)
    scheduler.submit(request("a", 30, 1))
    scheduler.submit(request("b", 8, 1))
    scheduler.step()
    assert runner.ran[0] == [("a", 0, 20, [])]
    scheduler.step()
    assert runner.ran[1] == [("a", 20, 10, [9]), ("b", 0, 8, [7])]


def test_stop_token_min_tokens_and_ignore_eos():
    scheduler, _, _ = build()
    scheduler.run_step.sample = lambda result, samplers: [7 for _ in samplers]
    scheduler.submit(request("stops", 3, 10, stop=[7]))
    scheduler.submit(request("min", 3, 10, stop=[7], min_tokens=4))
    scheduler.submit(request("ignores", 3, 5, stop=[7], ignore_eos=True))
    scheduler.run()
    by_name = {r.request_id: r for r in scheduler.finished}
    assert (by_name["stops"].finish_reason, len(by_name["stops"].output)) == ("stop", 1)
    assert (by_name["min"].finish_reason, len(by_name["min"].output)) == ("stop", 4)
    assert (by_name["ignores"].finish_reason, len(by_name["ignores"].output)) == ("length", 5)


def test_requests_beyond_the_slots_wait_their_turn_in_order():
    scheduler, runner, manager = build(max_batch_requests=2)
    for name in "abcd":
        scheduler.submit(request(name, 4, 2))
    scheduler.run()
    assert [r.request_id for r in scheduler.finished] == ["a", "b", "c", "d"]
    first_seen = {}
    for index, step in enumerate(runner.ran):
        assert len(step) <= 2
        for rid, *_ in step:
            first_seen.setdefault(rid, index)
    assert first_seen["a"] == first_seen["b"] < first_seen["c"] == first_seen["d"]
    manager.check()


def test_a_request_that_can_never_fit_is_refused_at_submission():
    scheduler, _, _ = build(pages=4, page_size=4)
    with pytest.raises(KvCapacity):
        scheduler.submit(request("big", 40, 1))
    with pytest.raises(SchedulerError, match="at least one prompt token"):
        scheduler.submit(request("empty", 0, 1))
    with pytest.raises(SchedulerError, match="max_position_embeddings"):
        scheduler.submit(request("long", 128, 1))


def test_waiting_request_is_admitted_only_when_its_prompt_fits():
    scheduler, runner, manager = build(pages=10, page_size=4)
    scheduler.submit(request("a", 30, 3))                 # 8 pages, 9 with its decoded tokens
    scheduler.submit(request("b", 12, 2))                 # 3 pages: does not fit beside a
    scheduler.run()
    first_b = next(i for i, step in enumerate(runner.ran) if any(e[0] == "b" for e in step))
    last_a = max(i for i, step in enumerate(runner.ran) if any(e[0] == "a" for e in step))
    assert first_b > last_a                               # b ran on a's pages after a had finished
    assert manager.groups[0].pool.reused > 0
    assert {r.request_id: r.finish_reason for r in scheduler.finished} == {"a": "length", "b": "length"}


def test_out_of_pages_preempts_the_youngest_and_recomputes_it():
    scheduler, runner, manager = build(pages=6, page_size=4, out_of_pages="preempt")
    scheduler.submit(request("old", 8, 12))               # grows to 20 tokens = 5 pages
    scheduler.submit(request("young", 7, 12))             # 2 pages at admission: both fit at first
    scheduler.run()
    by_name = {r.request_id: r for r in scheduler.finished}
    assert by_name["young"].preemptions >= 1 and by_name["old"].preemptions == 0
    assert len(by_name["old"].output) == 12 and len(by_name["young"].output) == 12
    assert by_name["old"].finish_reason == by_name["young"].finish_reason == "length"
    # after the preemption young was fed again from position 0, with the tokens it had produced
    restarts = [step for step in runner.ran for e in step if e[0] == "young" and e[1] == 0]
    assert len(restarts) >= 2
    assert manager.groups[0].pool.free == 6
    manager.check()


def test_out_of_pages_finish_policy_and_lonely_request():
    scheduler, _, manager = build(pages=6, page_size=4, out_of_pages="finish")
    scheduler.submit(request("old", 8, 12))
    scheduler.submit(request("young", 7, 12))
    scheduler.run()
    by_name = {r.request_id: r for r in scheduler.finished}
    assert by_name["young"].finish_reason == "out_of_pages" and by_name["old"].finish_reason == "length"
    scheduler, _, manager = build(pages=3, page_size=4)
    scheduler.submit(request("alone", 8, 30))             # can never hold 38 tokens in 12 slots
    scheduler.run()
    lonely = scheduler.finished[0]
    assert lonely.finish_reason == "out_of_pages" and 0 < len(lonely.output) < 30
    assert manager.groups[0].pool.free == 3
    manager.check()


def test_cancel_frees_everything():
    scheduler, _, manager = build()
    scheduler.submit(request("a", 6, 50))
    scheduler.submit(request("b", 6, 3))
    scheduler.step()
    scheduler.cancel("a")
    scheduler.run()
    assert {r.request_id: r.finish_reason for r in scheduler.finished} == {"a": "cancelled", "b": "length"}
    assert manager.groups[0].pool.free == 64 and manager.free_slots == 16


def test_windowed_model_runs_long_requests_in_few_pages():
    scheduler, runner, manager = build(TINY_C, pages=12, page_size=8, prefill_chunk_tokens=16)
    scheduler.submit(request("w", 60, 30))                # 90 tokens: 12 pages in the full group
    scheduler.run()
    assert scheduler.finished[0].finish_reason == "length"
    full, windowed = manager.groups
    assert full.pool.high_water == 12 and windowed.pool.high_water <= (40 + 16) // 8 + 2
    manager.check()


def test_deterministic_schedule():
    def schedule():
        scheduler, runner, _ = build(pages=12, page_size=4, max_batch_tokens=9, prefill_chunk_tokens=7)
        for name, n, m in (("a", 9, 5), ("b", 17, 4), ("c", 3, 8), ("d", 11, 2)):
            scheduler.submit(request(name, n, m))
        scheduler.run()
        return runner.ran
    assert schedule() == schedule()


def test_a_step_that_raises_leaves_nothing_live_once_the_caller_abandons():
    """What Model.generate_batch does around Scheduler.run: a failing step must not leave this call's requests as
    holders of pages and slots in the cache manager that later calls share."""
    scheduler, _, manager = build(max_batch_tokens=16)
    calls = {"n": 0}
    inner = scheduler.run_step

    def failing(entries, samplers):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("device failure")
        return inner(entries, samplers)

    scheduler.run_step = failing
    for name in "abc":
        scheduler.submit(request(name, 9, 6))
    with pytest.raises(RuntimeError, match="device failure"):
        try:
            scheduler.run()
        finally:
            scheduler.abandon()
    assert scheduler.idle and not manager.live
    assert manager.groups[0].pool.free == 64 and manager.free_slots == 16
    assert {r.finish_reason for r in scheduler.finished} == {"aborted"}
    manager.check()


def test_portions_keep_to_the_multiple_the_model_asks_for():
    """A model whose parts scan in chunks of 8 tokens: every portion but the one that ends a request's pending
    tokens is a multiple of 8, whatever the budget leaves."""
    scheduler, runner, manager = build(max_batch_tokens=21, prefill_chunk_tokens=100)
    scheduler.portion_multiple = 8
    scheduler.submit(request("a", 45, 3))
    scheduler.submit(request("b", 13, 2))
    scheduler.run()
    for step in runner.ran:
        for rid, start, count, want in step:
            total = 45 if rid == "a" else 13
            if start < total and start + count < total:
                assert count % 8 == 0 and start % 8 == 0, (rid, start, count)
    assert [e for e in runner.ran[0]] == [("a", 0, 16, [])]              # 21 cut down to 16
    assert runner.ran[1] == [("a", 16, 16, [])]
    assert runner.ran[2] == [("a", 32, 13, [12]), ("b", 0, 8, [])]       # the rest of a; b gets a multiple of what is left
    assert {r.request_id: len(r.output) for r in scheduler.finished} == {"a": 3, "b": 2}
    manager.check()
    with pytest.raises(SchedulerError, match="multiples of 64"):
        Scheduler(manager, SchedulerConfig(max_batch_tokens=40), 128, lambda e, s: [], portion_multiple=64)


def test_a_prompt_that_was_seen_before_is_fed_from_where_the_cached_pages_end():
    scheduler, runner, manager = build(prefix_cache=True, max_batch_tokens=16, prefill_chunk_tokens=10)
    scheduler.submit(request("a", 23, 3))
    scheduler.run()
    assert scheduler.finished[0].cached_tokens == 0
    runner.ran.clear()
    scheduler.submit(request("b", 23, 2))                  # the same 23 tokens: five full pages are there
    scheduler.submit(request("c", 9, 2))                   # its first two pages too
    scheduler.run()
    by_name = {r.request_id: r for r in scheduler.finished}
    assert by_name["b"].cached_tokens == 20 and by_name["c"].cached_tokens == 8
    first = {rid: (start, count) for rid, start, count, _ in runner.ran[0]}
    assert first == {"b": (20, 3), "c": (8, 1)}
    assert all(start >= 20 for step in runner.ran for rid, start, _, _ in step if rid == "b")
    assert len(by_name["b"].output) == 2 and len(by_name["c"].output) == 2
    pool = manager.groups[0].pool
    assert pool.available == 64 and pool.free == 64 - len(manager.prefix)
    manager.check()


def test_a_preempted_request_finds_its_own_pages_again_unless_they_were_needed():
    scheduler, runner, manager = build(pages=6, page_size=4, prefix_cache=True, out_of_pages="preempt")
    scheduler.submit(request("old", 8, 12))
    scheduler.submit(request("young", 7, 12))
    scheduler.run()
    by_name = {r.request_id: r for r in scheduler.finished}
    assert by_name["young"].preemptions >= 1
    assert len(by_name["old"].output) == 12 and len(by_name["young"].output) == 12
    assert manager.groups[0].pool.available == 6 and manager.prefix_evictions > 0
    manager.check()


@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("policy", ["preempt", "finish"])
def test_random_traffic_with_a_prefix_cache_feeds_every_token_once_in_order(seed, policy):
    """Requests that share prefixes, a pool too small for all of them, both policies for running out of pages: every
    request that finishes by length or stop has been fed, since its last (re)admission, exactly the tokens from where
    its cached pages end up to its last token, in order and without a gap; cached starts are whole pages; nothing is
    left held at the end."""
    import random
    rng = random.Random(seed)
    page = 4
    scheduler, runner, manager = build(pages=rng.choice([10, 14, 24]), page_size=page, prefix_cache=True,
                                       out_of_pages=policy, max_batch_tokens=rng.choice([8, 16, 64]),
                                       prefill_chunk_tokens=rng.choice([5, 8, 32]), max_batch_requests=4)
    stems = [[rng.randrange(5, 9) for _ in range(rng.randrange(4, 20))] for _ in range(3)]
    requests = []
    for index in range(10):
        stem = rng.choice(stems)
        prompt = stem[:rng.randrange(1, len(stem) + 1)] + [rng.randrange(5, 9) for _ in range(rng.randrange(0, 6))]
        settings = GenerationSettings(max_tokens=rng.randrange(1, 9))
        requests.append(Request(f"r{index}", prompt, settings, RequestSampler()))
    for item in requests[:5]:
        scheduler.submit(item)
    steps = 0
    while scheduler.waiting or scheduler.running:
        scheduler.step()
        steps += 1
        if steps == 3:
            for item in requests[5:]:
                scheduler.submit(item)
        assert steps < 2000
        manager.check()
    fed = {item.request_id: [] for item in requests}
    for step in runner.ran:
        names = [rid for rid, _, _, _ in step]
        assert len(names) == len(set(names))
        for rid, start, count, _ in step:
            fed[rid].append((start, count))
    for item in requests:
        assert item.state == "finished"
        portions = fed[item.request_id]
        if item.finish_reason in ("length", "stop"):
            total = len(item.prompt) + len(item.output)
            # walk back from the last portion to the start of the last (re)admission
            end = total - 1                                    # the last generated token is never fed
            cursor = len(portions) - 1
            while cursor >= 0 and portions[cursor][0] + portions[cursor][1] == end:
                end = portions[cursor][0]
                cursor -= 1
            assert end % page == 0 and end < len(item.prompt) + len(item.output), (item.request_id, portions)
            assert item.cached_tokens >= end or end == 0
        else:
            assert item.finish_reason == "out_of_pages"
    pool = manager.groups[0].pool
    assert pool.available == pool.count and manager.free_slots == 4 and not manager.live
