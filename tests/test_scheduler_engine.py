"""The scheduler's decisions and the engine loop's transactions, on the CPU with an executor
that returns scripted tokens."""

from __future__ import annotations

import pytest

import miniserve_b200  # noqa: F401
from miniserve_b200.cache import CacheManager
from miniserve_b200.engine.core import Engine, RequestRejected
from miniserve_b200.engine.scheduler import Scheduler
from miniserve_b200.engine.sequence import Sequence, Status
from miniserve_b200.parts import CacheGroup, PagedKVNeed
from miniserve_b200.sampling import SamplingParams

GROUP = CacheGroup(PagedKVNeed(2, 16, None), 2)


class ScriptedExecutor:
    """Next token = (sum of the request's tokens so far + draw index) % vocab: depends on the whole
    sequence, so any lost or repeated token changes everything after it."""

    def __init__(self, vocab=97):
        self.vocab, self.admitted, self.calls, self.fail_next = vocab, [], [], None
        self.history: dict[str, list[int]] = {}

    def admit(self, slot, params, seed):
        self.admitted.append((slot, params.temperature, seed))

    def execute(self, entries, reservation, samples):
        if self.fail_next is not None:
            error, self.fail_next = self.fail_next, None
            raise error
        self.calls.append([(e.request_id, len(e.tokens), tuple(e.want)) for e in entries])
        for entry, item in zip(entries, reservation.items):
            seen = self.history.setdefault(entry.request_id, [])
            assert item.start <= len(seen), "a gap in the positions that reached the executor"
            del seen[item.start:]
            seen.extend(entry.tokens)
        return [(sum(self.history[entries[s.entry].request_id]) + s.draw_index) % self.vocab for s in samples]


def expected_tokens(prompt, n, vocab=97, stop=()):
    tokens, out = list(prompt), []
    for draw in range(n):
        token = (sum(tokens) + draw) % vocab
        out.append(token)
        tokens.append(token)
        if token in stop:
            break
    return out


def make_engine(num_pages=16, page_size=4, max_seqs=4, budget=24, chunked=True, chunk=None, prefix=False, max_len=256):
    manager = CacheManager([GROUP], page_size, num_pages, max_seqs, enable_prefix_cache=prefix)
    scheduler = Scheduler(max_num_seqs=max_seqs, max_num_batched_tokens=budget, enable_chunked_prefill=chunked,
                          prefill_chunk_size=chunk)
    executor = ScriptedExecutor()
    return Engine(manager, scheduler, executor, vocab_size=97, max_model_len=max_len), executor


def run(engine):
    engine.run_until_done()
    results = dict(engine.finished)
    engine.manager.check_invariants()
    return results


def test_sampling_params_bounds():
    for bad in (dict(temperature=-0.1), dict(temperature=2.5), dict(temperature=float("nan")), dict(top_p=0.0),
                dict(top_p=1.5), dict(top_k=-1), dict(max_new_tokens=0), dict(stop_token_ids=[1]),
                dict(stop_token_ids=(1, 1)), dict(seed=-1), dict(seed=2 ** 63), dict(temperature=True)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams().temperature == 0.0 and SamplingParams().max_new_tokens == 4


def test_sequence_invariant_and_finish_rules():
    seq = Sequence("r", (1, 2, 3), SamplingParams(max_new_tokens=3, stop_token_ids=(9,)), 0, 0)
    seq.status = Status.RUNNING
    with pytest.raises(RuntimeError):
        seq.append_sampled(5)                       # nothing computed yet
    seq.advance(2)
    assert not seq.is_decoding and seq.remaining == 1
    seq.advance(3)
    seq.append_sampled(5)
    assert seq.is_decoding and seq.total == seq.computed + 1 and seq.token_slice(2, 4) == [3, 5]
    with pytest.raises(RuntimeError):
        seq.advance(5)
    seq.advance(4)
    seq.append_sampled(9)
    assert seq.done and seq.finish_reason == "stop" and seq.generated == [5, 9]


def test_plan_decodes_first_then_portions_within_the_budget():
    engine, executor = make_engine(num_pages=32, budget=24, chunk=12)
    prompts = {"r0": [1], "r1": list(range(7)), "r2": list(range(16)), "r3": list(range(33))}
    for rid, prompt in prompts.items():
        engine.submit(rid, prompt, SamplingParams(max_new_tokens=3))
    plan = engine.step()
    assert [(i.request_id, i.start, i.end) for i in plan.items] == [("r0", 0, 1), ("r1", 0, 7), ("r2", 0, 12), ("r3", 0, 4)]
    assert executor.calls[0] == [("r0", 1, (0,)), ("r1", 7, (6,)), ("r2", 12, ()), ("r3", 4, ())]
    plan = engine.step()
    assert [(i.request_id, i.start, i.end, i.is_decode) for i in plan.items] == [
        ("r0", 1, 2, True), ("r1", 7, 8, True), ("r2", 12, 16, False), ("r3", 4, 16, False)]
    results = run(engine)
    for rid, prompt in prompts.items():
        assert results[rid].token_ids == expected_tokens(prompt, 3) and results[rid].finish_reason == "length"
    assert engine.manager.capacity().free_pages == (32,) and engine.manager.capacity().free_slots == 4


def test_stop_token_ends_and_is_not_forwarded():
    engine, executor = make_engine()
    prompt = [3, 4]
    first = expected_tokens(prompt, 1)[0]
    engine.submit("r", prompt, SamplingParams(max_new_tokens=8, stop_token_ids=(first,)))
    results = run(engine)
    assert results["r"].token_ids == [first] and results["r"].finish_reason == "stop"
    assert sum(n for call in executor.calls for _, n, _ in call) == 2          # the stop token never ran


def test_unchunked_prompts_wait_for_budget_and_rejections():
    engine, _ = make_engine(budget=10, chunked=False)
    with pytest.raises(RequestRejected, match="CHUNKED_PREFILL_DISABLED"):
        engine.submit("big", list(range(11)), SamplingParams())
    engine.submit("a", list(range(8)), SamplingParams(max_new_tokens=2))
    engine.submit("b", list(range(8)), SamplingParams(max_new_tokens=2))
    plan = engine.step()
    assert [(i.request_id, i.end) for i in plan.items] == [("a", 8)]            # b does not fit the budget whole
    with pytest.raises(RequestRejected, match="duplicate"):
        engine.submit("a", [1], SamplingParams())
    with pytest.raises(RequestRejected, match="vocabulary"):
        engine.submit("c", [97], SamplingParams())
    with pytest.raises(RequestRejected, match="max_model_len"):
        engine.submit("c", [1] * 250, SamplingParams(max_new_tokens=10))
    small, _ = make_engine(num_pages=2)
    with pytest.raises(RequestRejected, match="CONTEXT_CAPACITY_EXCEEDED"):
        small.submit("c", [1] * 8, SamplingParams(max_new_tokens=1))
    results = run(engine)
    assert results["b"].token_ids == expected_tokens(list(range(8)), 2)


def test_more_requests_than_state_slots():
    engine, executor = make_engine(max_seqs=2, num_pages=64)
    prompts = {f"r{i}": [i + 1, i + 2, i + 3] for i in range(5)}
    for rid, prompt in prompts.items():
        engine.submit(rid, prompt, SamplingParams(max_new_tokens=4))
    plan = engine.step()
    assert len(plan.items) == 2
    results = run(engine)
    assert all(results[rid].token_ids == expected_tokens(p, 4) for rid, p in prompts.items())
    assert len({slot for slot, _, _ in executor.admitted}) == 2


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 4 tokens; two requests of 9 + 12 tokens each need 6 pages: they cannot both finish at once.
    engine, executor = make_engine(num_pages=6, page_size=4, budget=64)
    prompts = {"old": list(range(1, 10)), "young": list(range(11, 20))}
    engine.submit("old", prompts["old"], SamplingParams(max_new_tokens=12), arrival=0)
    engine.submit("young", prompts["young"], SamplingParams(max_new_tokens=12), arrival=1)
    results = run(engine)
    assert engine.stats.preemptions >= 1 and results["young"].preemptions >= 1 and results["old"].preemptions == 0
    for rid, prompt in prompts.items():
        assert results[rid].token_ids == expected_tokens(prompt, 12), rid
    assert engine.manager.capacity().free_pages == (6,)


def test_executor_failure_aborts_the_step():
    engine, executor = make_engine()
    engine.submit("a", [1, 2, 3], SamplingParams(max_new_tokens=2))
    engine.step()
    engine.submit("b", [4, 5], SamplingParams(max_new_tokens=2))
    free_before = engine.manager.capacity().free_pages
    executor.fail_next = RuntimeError("device fault")
    with pytest.raises(RuntimeError, match="device fault"):
        engine.step()
    assert engine.finished["a"].finish_reason.startswith("error") and engine.finished["b"].finish_reason.startswith("error")
    engine.manager.check_invariants()
    assert engine.manager.capacity().free_pages == (16,) and engine.manager.capacity().free_slots == 4
    assert free_before != (16,)
    engine.submit("c", [7, 8], SamplingParams(max_new_tokens=2))
    assert run(engine)["c"].token_ids == expected_tokens([7, 8], 2)


def test_prefix_hit_skips_shared_pages():
    engine, executor = make_engine(num_pages=32, page_size=4, budget=64, prefix=True)
    shared = list(range(20, 36))                                  # 4 full pages
    engine.submit("a", shared + [1, 2], SamplingParams(max_new_tokens=2))
    run(engine)
    engine.submit("b", shared + [3], SamplingParams(max_new_tokens=2))
    executor.history["b"] = list(shared)                          # what is in the shared pages already
    results = run(engine)
    assert engine.stats.prefix_hit_tokens == 16
    assert ("b", 1, (0,)) in executor.calls[-2]                   # only the token after the shared pages ran
    assert results["b"].token_ids == expected_tokens(shared + [3], 2)


def test_preemption_with_reusable_prefix_makes_progress():
    """A preempted request finds its own prompt pages cached on re-admission; the pages the
    scheduler counted as reclaimable are then held again.  The step must shrink, not repeat."""
    engine, executor = make_engine(num_pages=9, page_size=4, budget=64, prefix=True, max_seqs=3)
    prompts = {"r0": list(range(1, 6)), "r1": list(range(11, 20)), "r2": list(range(21, 34))}
    for index, (rid, prompt) in enumerate(prompts.items()):
        engine.submit(rid, prompt, SamplingParams(max_new_tokens=18), arrival=index)
    results = run(engine)
    assert engine.stats.preemptions >= 1
    for rid, prompt in prompts.items():
        assert results[rid].token_ids == expected_tokens(prompt, 18), rid


class DeferringExecutor(ScriptedExecutor):
    """The scripted executor with deferred reads: a deferred step's tokens are computed only when they are
    read, and a step fed back from the one before takes its input tokens from that step's results, as the
    device does; the token ids in its entries are placeholders."""

    def __init__(self, vocab=97):
        super().__init__(vocab)
        self.deferred_steps = self.fed_back_steps = 0
        self._last = None                      # the last deferred step's handle

    def can_defer(self, entries):
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def execute_deferred(self, entries, reservation, samples, feed_back=False):
        executor, previous = self, self._last
        self.deferred_steps += 1
        self.fed_back_steps += bool(feed_back)
        if feed_back:
            assert previous is not None and [e.request_id for e in entries] == previous.ids

        class Handle:
            ids = [e.request_id for e in entries]
            result = None

            def tokens(self):
                if self.result is None:
                    fed = previous.tokens() if feed_back else [e.tokens[0] for e in entries]
                    real = [type(e)(e.request_id, [t], e.want) for e, t in zip(entries, fed)]
                    self.result = ScriptedExecutor.execute(executor, real, reservation, samples)
                return self.result

        self._last = Handle()
        return self._last


@pytest.mark.parametrize("stop", [(), (5, 11, 23, 42, 77)])
def test_decoding_one_step_ahead_gives_the_same_tokens(stop):
    """With deferred reads the engine starts each decode step before it has read the tokens of the step
    before; results, finish reasons and the cache's books are as without."""
    prompts = {"a": [3, 1, 4, 1, 5], "b": [9, 2, 6], "c": list(range(20, 31)), "d": [7]}
    budgets = {"a": 12, "b": 3, "c": 9, "d": 17}
    outcomes = []
    for look_ahead in (False, True):
        manager = CacheManager([GROUP], 4, 32, 4, enable_prefix_cache=False)
        scheduler = Scheduler(max_num_seqs=4, max_num_batched_tokens=24)
        executor = DeferringExecutor()
        engine = Engine(manager, scheduler, executor, vocab_size=97, max_model_len=256, look_ahead=look_ahead)
        for rid, prompt in prompts.items():
            engine.submit(rid, prompt, SamplingParams(max_new_tokens=budgets[rid], stop_token_ids=stop))
        engine.run_until_done()
        outcomes.append({rid: (engine.finished[rid].token_ids, engine.finished[rid].finish_reason) for rid in prompts})
        for rid, prompt in prompts.items():
            assert outcomes[-1][rid][0] == expected_tokens(prompt, budgets[rid], stop=stop)
        manager.check_invariants()
        assert not manager.requests and manager.capacity().free_pages == (32,)
        assert (executor.fed_back_steps > 0) == look_ahead
    assert outcomes[0] == outcomes[1]


def test_look_ahead_yields_to_a_new_request():
    """A request that arrives while decoding runs ahead is planned in the next step: the pending tokens
    are read first and the step is an ordinary mixed one."""
    manager = CacheManager([GROUP], 4, 32, 4, enable_prefix_cache=False)
    executor = DeferringExecutor()
    engine = Engine(manager, Scheduler(max_num_seqs=4, max_num_batched_tokens=24), executor, vocab_size=97,
                    max_model_len=256, look_ahead=True)
    engine.submit("a", [1, 2, 3], SamplingParams(max_new_tokens=10))
    for _ in range(4):
        engine.step()
    fed_back = executor.fed_back_steps
    assert fed_back >= 2
    engine.submit("b", [4, 5, 6, 7, 8], SamplingParams(max_new_tokens=6))
    engine.step()
    assert executor.fed_back_steps == fed_back            # no look-ahead past a waiting request
    assert {item.request_id for item in engine.last_plan.items} == {"a", "b"}
    engine.run_until_done()
    assert engine.finished["a"].token_ids == expected_tokens([1, 2, 3], 10)
    assert engine.finished["b"].token_ids == expected_tokens([4, 5, 6, 7, 8], 6)


def test_failure_of_a_step_started_ahead():
    """The device refuses the step that was started ahead: the reservation is undone, the tokens of the
    step before are kept, the requests end as failed and give their pages back."""
    manager = CacheManager([GROUP], 4, 32, 4, enable_prefix_cache=False)
    executor = DeferringExecutor()
    engine = Engine(manager, Scheduler(max_num_seqs=4, max_num_batched_tokens=24), executor, vocab_size=97,
                    max_model_len=256, look_ahead=True)
    engine.submit("a", [1, 2, 3], SamplingParams(max_new_tokens=10))
    for _ in range(3):
        engine.step()
    produced = len(engine.sequences["a"].generated)
    original = executor.execute_deferred

    def refuse(*args, **kwargs):
        raise RuntimeError("device lost")

    executor.execute_deferred = refuse
    with pytest.raises(RuntimeError):
        engine.step()
    executor.execute_deferred = original
    result = engine.finished["a"]
    assert result.finish_reason == "error: RuntimeError"
    assert result.token_ids == expected_tokens([1, 2, 3], produced + 1)      # the pending token was still read
    manager.check_invariants()
    assert not manager.requests and manager.capacity().free_pages == (32,)


def test_pages_are_planned_per_cache_group():
    """A model with a group that keeps every key beside one with a window: the group with a window gives pages
    back as it goes, so the two have different numbers free, and the scheduler plans against each group's own
    count (the arithmetic is the cache's: ``CapacitySnapshot.pages_for`` / ``room``)."""
    from miniserve_b200.parts import StateNeed

    full, windowed = CacheGroup(PagedKVNeed(2, 16, None), 1), CacheGroup(PagedKVNeed(2, 16, 6), 1)
    manager = CacheManager([full, windowed], page_size=4, num_pages=8, max_seqs=3)
    scheduler = Scheduler(max_num_seqs=3, max_num_batched_tokens=64, enable_chunked_prefill=True)
    engine = Engine(manager, scheduler, ScriptedExecutor(), vocab_size=97, max_model_len=64)
    engine.submit("b", list(range(1, 18)), SamplingParams(max_new_tokens=2), arrival=1)   # 17 tokens: five pages
    manager.admit("hold")
    manager.commit(manager.prepare([("hold", 20)]))     # five pages in each group, of which
    capacity = manager.capacity()
    assert capacity.free_pages == (3, 6)                # the window has given three back already
    assert capacity.pages_for(0, 17) == (5, 5) and capacity.room(0, capacity.available()) == 12
    plan = scheduler.schedule(list(engine.sequences.values()), capacity)
    assert [(i.request_id, i.start, i.end) for i in plan.items] == [("b", 0, 12)]   # what the fuller group can hold
    manager.release("hold")
    manager.check_invariants()

    # a model whose only cache is per-request state has no pages to run out of
    state_only = CacheManager([CacheGroup(StateNeed((8,)), 2)], page_size=4, num_pages=1, max_seqs=2)
    snapshot = state_only.capacity()
    assert snapshot.pages_for(0, 1000) == () and snapshot.room(0, snapshot.available()) >= 1 << 60
    plan = Scheduler(max_num_seqs=2, max_num_batched_tokens=512).schedule(
        [Sequence("s", tuple(range(300)), SamplingParams(), 0, 0)], snapshot)
    assert [(i.start, i.end) for i in plan.items] == [(0, 300)]
