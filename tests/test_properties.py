"""Generated cases (hypothesis): the cache's books under any sequence of operations, the generation loop's
decisions for any mix of prompt lengths, limits and stop tokens, and (on the GPU) the logits of a prompt cut into
steps in any way."""
import random

import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st
from hypothesis.stateful import RuleBasedStateMachine, invariant, precondition, rule

import plain_qwen3 as plain
from conftest import TEST_CONFIGS, TOL


# ---- the cache: no page lost, held twice or freed twice, whatever is asked of it --------------------------------
def _make_cache():
    import importlib
    pe = importlib.import_module("pytorch-engine_b200")
    CR = pe.parts.CacheRequest
    reqs = {0: CR("kv", kv_heads=1, head_dim=8), 1: CR("kv", kv_heads=1, head_dim=8, window=100),
            2: CR("state", state_shapes=(("s", (2,), "float32"),))}
    return pe, pe.cache.PagedCache(reqs, max_tokens=64 * 24, max_slots=5, max_seq_len=640, dtype=torch.float32, device="cpu")


class CacheMachine(RuleBasedStateMachine):
    def __init__(self):
        super().__init__()
        self.pe, self.cache = _make_cache()
        self.lengths = {}

    @precondition(lambda self: len(self.lengths) < 5)
    @rule()
    def take_a_slot(self):
        s = self.cache.alloc_slot()
        assert s not in self.lengths                      # never handed out twice
        assert float(self.cache.view(2).state("s")[s].abs().sum()) == 0.0   # state starts at zero
        self.lengths[s] = 0
        self.cache.view(2).state("s")[s].fill_(1.0)

    @precondition(lambda self: len(self.lengths) == 5)
    @rule()
    def no_sixth_slot(self):
        with pytest.raises(self.pe.cache.CacheFull):
            self.cache.alloc_slot()

    @precondition(lambda self: self.lengths)
    @rule(pick=st.integers(0, 4), grow=st.sampled_from([1, 1, 2, 17, 64, 65, 200, 700]))
    def grow_a_sequence(self, pick, grow):
        s = sorted(self.lengths)[pick % len(self.lengths)]
        new = self.lengths[s] + grow
        free_before = self.cache.free_pages()
        try:
            self.cache.reserve(s, new)
        except self.pe.cache.CacheFull:
            assert self.cache.free_pages() == free_before     # a refusal changes nothing
            assert self.cache.length(s) == self.lengths[s]
            return
        assert new <= 640
        self.cache.commit(s, new)
        self.lengths[s] = new

    @precondition(lambda self: self.lengths)
    @rule(pick=st.integers(0, 4))
    def reserve_and_give_up(self, pick):
        s = sorted(self.lengths)[pick % len(self.lengths)]
        free_before = self.cache.free_pages()
        try:
            self.cache.reserve(s, self.lengths[s] + 130)
        except self.pe.cache.CacheFull:
            return
        self.cache.release_reserved(s)                    # a step that was prepared and not run
        assert self.cache.free_pages() == free_before

    @precondition(lambda self: self.lengths)
    @rule(pick=st.integers(0, 4))
    def give_a_slot_back(self, pick):
        s = sorted(self.lengths)[pick % len(self.lengths)]
        self.cache.free_slot(s)
        del self.lengths[s]
        with pytest.raises(self.pe.cache.CacheBookkeepingError):
            self.cache.free_slot(s)                       # not twice

    @rule()
    def forget_everything(self):
        self.cache.reset()
        self.lengths = {}
        assert self.cache.free_pages() == 24

    @invariant()
    def the_books_are_right(self):
        self.cache.check()
        assert self.cache.live_slots == sorted(self.lengths)
        for s, n in self.lengths.items():
            assert self.cache.length(s) == n
        # pages held by the full-length group: exactly what the lengths need
        held = sum(-(-n // 64) for n in self.lengths.values())
        assert self.cache.groups[0].pool.held_count == held
        # the windowed group never holds more than the window needs (plus the page being written)
        for s, n in self.lengths.items():
            live = [p for p in self.cache.groups[1].pages_of_slot[s] if p >= 0]
            assert len(live) <= -(-100 // 64) + 1


TestCacheMachine = CacheMachine.TestCase
TestCacheMachine.settings = settings(max_examples=40, stateful_step_count=40, deadline=None,
                                     suppress_health_check=[HealthCheck.too_slow])


# ---- the generation loop: any prompts, limits and stop tokens -------------------------------------------------
class ScriptedBackend:
    """A backend whose 'model' emits, for a sequence of length L, token (L * 7 + first prompt token) % 50: the loop's
    decisions can be checked without a device."""

    def __init__(self, slots):
        self.free = list(range(slots))
        self.length, self.first = {}, {}
        self.steps = []

    def alloc_slot(self):
        return self.free.pop()

    def free_slot(self, s):
        assert s in self.length or s in self.first or True
        self.length.pop(s, None)
        self.first.pop(s, None)
        self.free.append(s)

    def free_pages(self):
        return 1 << 20

    def step(self, entries):
        rows = []
        self.steps.append([len(e.tokens) for e in entries])
        for e in entries:
            if e.slot not in self.first:
                self.first[e.slot] = e.tokens[0]
                self.length[e.slot] = 0
            self.length[e.slot] += len(e.tokens)
            for _ in e.want:
                rows.append((self.length[e.slot] * 7 + self.first[e.slot]) % 50)
        return rows

    def sample(self, logits, params, seed, requests, steps, recent=None):
        return list(logits)


def _expected(prompt, max_tokens, max_context, stops):
    out, length = [], len(prompt)
    limit = max(1, min(max_tokens, max_context - len(prompt)))
    while len(out) < limit:
        tok = (length * 7 + prompt[0]) % 50
        if tok in stops:
            return out, "stop"
        out.append(tok)
        length += 1
    return out, "length"


@settings(max_examples=60, deadline=None)
@given(lens=st.lists(st.integers(1, 40), min_size=1, max_size=9), max_tokens=st.integers(1, 30),
       max_batch=st.integers(1, 4), stops=st.sets(st.integers(0, 49), max_size=4), seed=st.integers(0, 1000),
       step_limit=st.sampled_from([None, 7, 64]))
def test_generation_loop_decisions(lens, max_tokens, max_batch, stops, seed, step_limit):
    import importlib
    pe = importlib.import_module("pytorch-engine_b200")
    rng = random.Random(seed)
    prompts = [[rng.randrange(50) for _ in range(n)] for n in lens]
    backend = ScriptedBackend(slots=max_batch)
    loop = pe.engine.generate.GenerationLoop(backend, max_context=48, max_batch=max_batch, eos_token_ids=(),
                                             bos_token_id=0, max_step_tokens=step_limit)
    params = pe.SamplingParams.greedy_params(max_tokens=max_tokens, stop_token_ids=sorted(stops))
    results = loop.generate(prompts, params)
    assert len(results) == len(prompts)
    for prompt, res in zip(prompts, results):
        want, why = _expected(prompt, max_tokens, 48, stops)
        assert res.token_ids == want and res.finish_reason == why
        assert res.prompt_tokens == len(prompt) and res.completion_tokens == len(want)
    assert sorted(backend.free) == list(range(max_batch))      # every slot came back
    if step_limit:
        assert all(sum(s) <= max(step_limit, 1) or max(s) == 1 for s in backend.steps)


# ---- on the GPU: a prompt cut into steps in any way gives the logits of the whole prompt -----------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_any_cut_of_a_prompt_gives_the_same_logits(pe, model_folders, tmp_path, dtype):
    from test_model_gpu import Replay, _check, _ref, _tokens
    key = "E"
    cfg, w = plain.load_folder(model_folders[dtype][key])
    eng = pe.Engine(model_folders[dtype][key], dtype=dtype, max_cache_tokens=64 * 24, max_batch=4)
    refs = {}

    @settings(max_examples=12, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])
    @given(n=st.integers(2, 260), cuts=st.lists(st.integers(1, 140), min_size=1, max_size=12), other=st.integers(0, 2),
           seed=st.integers(0, 3))
    def run(n, cuts, other, seed):
        toks = _tokens(cfg["vocab_size"], n, 500 + seed)
        rp = Replay(pe, eng, tmp_path)
        # `other` more requests run beside it, one token per step, to change what else is in the batch
        others = {f"o{i}": _tokens(cfg["vocab_size"], 40, 900 + i) for i in range(other)}
        fed, step = 0, 0
        pieces = list(cuts)
        while fed < n:
            take = min(n - fed, pieces.pop(0) if pieces else 1)
            entries = [("r", toks[fed:fed + take], list(range(take)))]
            ends = ["r"] if fed + take == n else []
            for oid, ot in others.items():
                if step < len(ot):
                    entries.append((oid, [ot[step]], []))
                    if step == len(ot) - 1:
                        ends.append(oid)
            rp.run(entries, end=ends)
            fed += take
            step += 1
        for oid, ot in others.items():
            if step < len(ot):
                rp.run([], end=[oid])
        if (n, seed) not in refs:
            refs[n, seed] = _ref(cfg, w, toks, dtype)
        ref = refs[n, seed]
        _check(rp.got, {("r", i): ref[i] for i in range(n)}, dtype, f"{n} tokens cut {cuts[:6]}.. beside {other} others")
        assert not eng.cache.live_slots

    run()
    eng.cache.check()
