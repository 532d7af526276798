"""The generation loop's decisions, with a scripted backend (no GPU)."""
import pytest


class FakeBackend:
    """Draws the next token of a request from a script; records what the loop asked for."""

    def __init__(self, scripts, pages=1000):
        self.scripts = scripts          # request index -> list of tokens it will draw
        self.pages = pages
        self.free = list(range(7, -1, -1))
        self.held = set()
        self.steps = []                 # [(slot, tokens, want), ...] per step
        self.max_held = 0
        self.sample_calls = []

    def alloc_slot(self):
        s = self.free.pop()
        assert s not in self.held
        self.held.add(s)
        self.max_held = max(self.max_held, len(self.held))
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        self.held.remove(s)
        self.free.append(s)

    def free_pages(self):
        return self.pages

    def step(self, entries):
        assert len({e.slot for e in entries}) == len(entries)
        assert all(e.slot in self.held for e in entries)
        self.steps.append([(e.slot, list(e.tokens), tuple(e.want)) for e in entries])
        return sum(len(e.want) for e in entries)     # stands for the logits: one row per wanted place

    def sample(self, logits, params, seed, requests, steps, recent=None):
        assert logits == len(requests)
        self.sample_calls.append((list(requests), list(steps)))
        return [self.scripts[r][k] for r, k in zip(requests, steps)]


def _loop(pe, backend, **kw):
    args = dict(max_context=64, max_batch=3, eos_token_ids=(99,), bos_token_id=5)
    args.update(kw)
    return pe.engine.GenerationLoop(backend, **args)


def test_unequal_prompts_stop_tokens_and_early_leavers(pe):
    scripts = {0: [10, 11, 99], 1: [20, 21, 22, 23, 24], 2: [99]}
    be = FakeBackend(scripts)
    res = _loop(pe, be).generate([[1, 2, 3], [4], [6, 7]], pe.SamplingParams(max_tokens=4, temperature=0.0))
    assert [r.token_ids for r in res] == [[10, 11], [20, 21, 22, 23], []]
    assert [r.finish_reason for r in res] == ["stop", "length", "stop"]
    assert [r.prompt_tokens for r in res] == [3, 1, 2] and [r.completion_tokens for r in res] == [2, 4, 0]
    # one prefill step with all prompts, logits wanted at each prompt's last token
    assert [(t, w) for _, t, w in be.steps[0]] == [([1, 2, 3], (2,)), ([4], (0,)), ([6, 7], (1,))]
    # then one token each for the sequences still alive: request 2 left after its first draw
    assert [[t for _, t, _ in st] for st in be.steps[1:]] == [[[10], [20]], [[11], [21]], [[22]]]
    assert not be.held  # every slot came back
    # the token that ends a sequence by length is never fed back
    assert len(be.steps) == 4


def test_batches_follow_one_another_and_reuse_slots(pe):
    scripts = {i: [30 + i, 99] for i in range(7)}
    be = FakeBackend(scripts)
    res = _loop(pe, be).generate([[1]] * 7, pe.SamplingParams(max_tokens=5, temperature=0.0))
    assert [r.token_ids for r in res] == [[30 + i] for i in range(7)]
    assert be.max_held == 3                         # never more than max_batch live
    prefills = [st for st in be.steps if len(st[0][1]) == 1 and st[0][2] == (0,) and st[0][1] == [1]]
    assert len(prefills) == 3                       # 3 + 3 + 1 requests
    assert {s for st in be.steps for s, _, _ in st} == {0, 1, 2}   # the same slots again


def test_page_limit_splits_batches(pe):
    be = FakeBackend({i: [1] * 40 for i in range(4)}, pages=3)
    lp = _loop(pe, be, max_batch=8, max_context=200)
    params = pe.SamplingParams(max_tokens=30, temperature=0.0)
    prompts = [[1] * 40, [1] * 100, [1] * 10, [1] * 20]
    # pages if run to the limit: 69 -> 2, 129 -> 3, 39 -> 1, 49 -> 1
    assert lp.plan_batches(prompts, params, 3) == [[0], [1], [2, 3]]
    with pytest.raises(ValueError, match="cache pages"):
        lp.plan_batches([[1] * 150], params, 2)


def test_limits_follow_the_reference(pe):
    lp = _loop(pe, FakeBackend({}), max_context=10)
    assert lp.new_token_limit(3, 512) == 7
    assert lp.new_token_limit(10, 512) == 1          # max(1, ...)
    assert lp.new_token_limit(3, 2) == 2
    assert lp.normalise_prompt([]) == [5]            # bos stands in for an empty prompt
    with pytest.raises(ValueError, match="context"):
        lp.plan_batches([[1] * 11], pe.SamplingParams(), 100)


def test_request_stop_ids_and_random_keys(pe):
    be = FakeBackend({0: [10, 42, 11], 1: [42]})
    res = _loop(pe, be).generate([[1], [2]], pe.SamplingParams(max_tokens=8, temperature=0.8, stop_token_ids=[42], seed=3))
    assert [r.token_ids for r in res] == [[10], []]
    # random numbers are keyed by (request index, tokens drawn so far), not by the place in the batch
    assert be.sample_calls == [([0, 1], [0, 0]), ([0], [1])]


def test_stream_yields_every_token_once(pe):
    be = FakeBackend({0: [10, 11, 12], 1: [20, 99]})
    chunks = list(_loop(pe, be).stream([[1], [2]], pe.SamplingParams(max_tokens=3, temperature=0.0)))
    assert [(c.request, c.token_id, c.finish_reason) for c in chunks] == [
        (0, 10, None), (1, 20, None), (0, 11, None), (1, 99, "stop"), (0, 12, "length")]
    assert chunks[-1].stats.token_ids == [10, 11, 12]


def test_slots_come_back_when_a_step_fails(pe):
    class Failing(FakeBackend):
        def step(self, entries):
            if self.steps:
                raise RuntimeError("boom")
            return super().step(entries)

    be = Failing({0: [1, 2], 1: [3, 4]})
    with pytest.raises(RuntimeError):
        _loop(pe, be).generate([[1], [2]], pe.SamplingParams(max_tokens=3, temperature=0.0))
    assert not be.held


def test_sampling_params_validate(pe):
    for bad in (dict(max_tokens=0), dict(temperature=-1.0), dict(top_p=0.0), dict(top_k=-1), dict(min_p=2.0),
                dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            pe.SamplingParams(**bad).validate()
    d = pe.SamplingParams()
    assert (d.max_tokens, d.temperature, d.top_p, d.top_k, d.min_p, d.repetition_penalty) == (512, 0.7, 0.95, 40, 0.05, 1.0)


class AheadBackend(FakeBackend):
    """A backend that can launch decode steps without waiting (``launch_decode``).  It checks what the
    loop may and may not do: feed a step from the device only right after a launch for the same slots,
    and never give a slot back while a launched step that uses it has not been waited for."""

    def __init__(self, scripts, pages=1000):
        super().__init__(scripts, pages)
        self.launches = []          # (slots, tokens or None, requests, steps)
        self.in_flight = []         # handles not yet waited for
        self.last_slots = None

    class Handle:
        def __init__(self, be, slots, toks):
            self.be, self.slots, self.toks, self.done = be, list(slots), toks, False

        def result(self):
            assert self.be.in_flight and self.be.in_flight[0] is self, "steps are waited for in launch order"
            self.be.in_flight.pop(0)
            self.done = True
            return self.toks

    def free_slot(self, s):
        assert all(s not in h.slots for h in self.in_flight), "a slot was given back under a step in flight"
        super().free_slot(s)

    def launch_decode(self, slots, tokens, params, seed, requests, steps):
        assert all(s in self.held for s in slots)
        if tokens is None:
            assert self.last_slots == list(slots), "device tokens belong to the launch just before, same slots"
        self.launches.append((list(slots), None if tokens is None else list(tokens), list(requests), list(steps)))
        self.last_slots = list(slots)
        # a sequence that has ended may still be in a step launched ahead: its draw is never looked at
        toks = [self.scripts[r][k] if k < len(self.scripts[r]) else -1 for r, k in zip(requests, steps)]
        h = self.Handle(self, slots, toks)
        self.in_flight.append(h)
        return h


def test_one_step_ahead_gives_the_same_tokens(pe):
    scripts = {0: [10, 11, 99, 55, 56], 1: [20, 21, 22, 23, 24, 25], 2: [99], 3: [30, 31, 32, 99, 1, 2]}
    prompts = [[1, 2, 3], [4], [6, 7], [8]]
    params = pe.SamplingParams(max_tokens=5, temperature=0.0)
    plain_be, ahead_be = FakeBackend(scripts), AheadBackend(scripts)
    want = _loop(pe, plain_be, max_batch=4).generate(prompts, params)
    got = _loop(pe, ahead_be, max_batch=4).generate(prompts, params)
    assert [r.token_ids for r in got] == [r.token_ids for r in want] == [[10, 11], [20, 21, 22, 23, 24], [], [30, 31, 32]]
    assert [r.finish_reason for r in got] == ["stop", "length", "stop", "stop"]
    assert not ahead_be.held and not ahead_be.in_flight
    # steps fed from the device exist, and none was launched when a sequence was sure to end by length
    assert any(t is None for _, t, _, _ in ahead_be.launches)
    for slots, toks, reqs, steps in ahead_be.launches:
        if toks is None:
            assert all(k + 1 <= 5 - 1 for k in steps)
    # the tokens a launch is fed from the host are the sequences' last tokens
    first = ahead_be.launches[0]
    assert first[1] == [10, 20, 30] and first[2] == [0, 1, 3] and first[3] == [1, 1, 1]


def test_one_step_ahead_is_not_used_with_a_repetition_penalty(pe):
    be = AheadBackend({0: [10, 11, 12]})
    res = _loop(pe, be).generate([[1]], pe.SamplingParams(max_tokens=3, temperature=0.0, repetition_penalty=1.3))
    assert res[0].token_ids == [10, 11, 12] and not be.launches


def test_one_step_ahead_stream_order_and_stats(pe):
    be = AheadBackend({0: [10, 11, 12, 13], 1: [20, 99]})
    chunks = list(_loop(pe, be).stream([[1], [2]], pe.SamplingParams(max_tokens=4, temperature=0.0)))
    assert [(c.request, c.token_id, c.finish_reason) for c in chunks] == [
        (0, 10, None), (1, 20, None), (0, 11, None), (1, 99, "stop"), (0, 12, None), (0, 13, "length")]
    assert chunks[-1].stats.token_ids == [10, 11, 12, 13]


def test_prompts_beyond_the_step_limit_come_in_several_steps(pe):
    lp = _loop(pe, FakeBackend({}), max_step_tokens=5)
    assert lp.plan_prefill([2, 3]) == [[(0, 0, 2), (1, 0, 3)]]                       # fits: one step
    assert lp.plan_prefill([4, 3, 7]) == [[(0, 0, 4), (1, 0, 1)], [(1, 1, 3), (2, 0, 3)], [(2, 3, 7)]]
    assert _loop(pe, FakeBackend({})).plan_prefill([100, 200]) == [[(0, 0, 100), (1, 0, 200)]]   # no limit
    scripts = {0: [10, 11], 1: [20, 99], 2: [30, 31]}
    be = FakeBackend(scripts)
    prompts = [[1, 2, 3, 4], [5, 6, 7], [8, 9, 10, 11, 12, 13, 14]]
    res = _loop(pe, be, max_step_tokens=5).generate(prompts, pe.SamplingParams(max_tokens=2, temperature=0.0))
    assert [r.token_ids for r in res] == [[10, 11], [20], [30, 31]]
    # three steps bring the prompts; logits are wanted only where a prompt ends
    assert [[(t, w) for _, t, w in st] for st in be.steps[:3]] == [
        [([1, 2, 3, 4], (3,)), ([5], ())], [([6, 7], (1,)), ([8, 9, 10], ())], [([11, 12, 13, 14], (3,))]]
    # each sequence's first token is drawn when its prompt is through, keyed by its own request and step
    assert be.sample_calls[:3] == [([0], [0]), ([1], [0]), ([2], [0])]
    assert [[t for _, t, _ in st] for st in be.steps[3:]] == [[[10], [20], [30]]]
    assert not be.held
    # the same requests without a limit give the same tokens
    be2 = FakeBackend(scripts)
    res2 = _loop(pe, be2).generate(prompts, pe.SamplingParams(max_tokens=2, temperature=0.0))
    assert [r.token_ids for r in res2] == [r.token_ids for r in res]
