"""The engine against the plain implementation, in float32 and bfloat16: whole requests, the last
tokens one by one, unequal batches with slots used again, long decoding, the first tokens,
generation through the entry point, and the replay program itself."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
from conftest import ROOT, TEST_CONFIGS, TOL, rel_err

pytestmark = pytest.mark.gpu
KEYS = ["A", "B", "C", "D", "E"]
DTYPES = ["float32", "bfloat16"]


def _ref(cfg, w, toks, dtype):
    """The plain implementation's logits; for a bfloat16 run it stores its activations in bfloat16 at
    the places where the engine does (the attention of these test models is sharpened, which turns
    every rounding of a query or key into a visible change of the softmax weights)."""
    return plain.forward_logits(cfg, w, toks, store=torch.bfloat16 if dtype == "bfloat16" else None)


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class _Oracles:
    """(config, weights) of a test model; ``oracles[key]`` is the float32 variant, ``oracles[key, dtype]``
    the one whose attention is sharpened as that dtype's runs are."""

    def __init__(self, folders):
        self.folders = folders
        self.loaded = {}

    def __getitem__(self, item):
        key, dtype = item if isinstance(item, tuple) else (item, "float32")
        if (key, dtype) not in self.loaded:
            self.loaded[key, dtype] = plain.load_folder(self.folders[dtype][key])
        return self.loaded[key, dtype]


@pytest.fixture(scope="module")
def oracles(model_folders):
    return _Oracles(model_folders)


@pytest.fixture(scope="module")
def engines(pe, model_folders):
    made = {}

    def get(key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in made:
            args = dict(dtype=dtype, max_cache_tokens=64 * 40, max_batch=8)
            args.update(kw)
            made[ident] = pe.Engine(model_folders[dtype][key], **args)
        return made[ident]

    return get


class Replay:
    """Drives the engine's replayer in-process and collects logits per (request, position)."""

    def __init__(self, pe, engine, tmp_path):
        self.rep = pe.engine.replay.TraceReplayer(engine, str(tmp_path))
        self.step = 0
        self.fed = {}
        self.got = {}

    def run(self, entries, end=()):
        rec = {"step": self.step, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)}
        path = self.rep.run_step(rec)
        vocab = self.rep.engine.config.vocab_size
        n_want = sum(len(w) for _, _, w in entries)
        if n_want:
            arr = torch.frombuffer(bytearray(open(path, "rb").read()), dtype=torch.float32).view(n_want, vocab)
            r = 0
            for i, t, w in entries:
                base = self.fed.get(i, 0)
                for j in w:
                    self.got[(i, base + j)] = arr[r].clone()
                    r += 1
        else:
            assert path is None
        for i, t, _ in entries:
            self.fed[i] = self.fed.get(i, 0) + len(t)
        for i in end:
            self.fed.pop(i, None)
        self.step += 1


def _check(got, oracle_rows, dtype, what):
    worst = 0.0
    scale = max(float(r.abs().max()) for r in oracle_rows.values())
    for key, ref in oracle_rows.items():
        err = float((got[key].double() - ref.double()).abs().max()) / scale
        worst = max(worst, err)
    assert worst < TOL[dtype], f"{what}: worst error {worst:.3e} (limit {TOL[dtype]:.0e})"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_each_request_alone_and_whole(pe, engines, oracles, tmp_path, key, dtype):
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    for n, seed in [(150, 1), (1, 2), (65, 3), (333, 4)]:
        toks = _tokens(cfg["vocab_size"], n, seed)
        rp = Replay(pe, eng, tmp_path)
        rp.run([("r", toks, list(range(n)))], end=["r"])
        ref = _ref(cfg, w, toks, dtype)
        _check(rp.got, {("r", i): ref[i] for i in range(n)}, dtype, f"{key} whole, {n} tokens")
    assert not eng.cache.live_slots
    eng.cache.check()


@pytest.mark.parametrize("key", KEYS)
def test_bfloat16_against_the_float32_implementation(pe, tmp_path_factory, tmp_path, key):
    """The bfloat16 engine against the plain implementation in pure float32, on plain random weights
    (attention not sharpened): whole requests, then a few tokens one by one."""
    from conftest import make_model_folder
    folder = make_model_folder(pe, tmp_path_factory, key, sharpen=None)
    cfg, w = plain.load_folder(folder)
    eng = pe.Engine(folder, dtype="bfloat16", max_cache_tokens=64 * 12, max_batch=4)
    toks = _tokens(cfg["vocab_size"], 200, 21)
    rp = Replay(pe, eng, tmp_path)
    rp.run([("r", toks[:190], list(range(190)))])
    for i in range(190, 200):
        rp.run([("r", [toks[i]], [0])], end=["r"] if i == 199 else [])
    ref = plain.forward_logits(cfg, w, toks)
    _check(rp.got, {("r", i): ref[i] for i in range(200)}, "bfloat16", f"{key} bfloat16 against float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_last_32_tokens_one_by_one(pe, engines, oracles, tmp_path, key, dtype):
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    for n, seed in [(33, 5), (100, 6), (290, 7)]:
        toks = _tokens(cfg["vocab_size"], n, seed)
        rp = Replay(pe, eng, tmp_path)
        head = n - 32
        rp.run([("r", toks[:head], [head - 1])])
        for i in range(head, n):
            rp.run([("r", [toks[i]], [0])], end=["r"] if i == n - 1 else [])
        ref = _ref(cfg, w, toks, dtype)
        _check(rp.got, {("r", i): ref[i] for i in range(head - 1, n)}, dtype, f"{key} last 32 of {n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_unequal_batches_one_after_another(pe, engines, oracles, tmp_path, key, dtype):
    """Two batches; in each, prompts of unequal lengths go in together, every request is then fed
    its remaining tokens one per step, and the shorter requests end earlier.  The second batch gets
    the slots and pages that the first gave back."""
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    rp = Replay(pe, eng, tmp_path)
    want = {}
    plans = [
        [("a", 5, 9), ("b", 70, 3), ("c", 130, 40), ("d", 1, 20)],      # (id, prompt length, decoded tokens)
        [("e", 64, 12), ("f", 9, 30), ("g", 200, 1), ("h", 33, 33), ("i", 2, 5)],
    ]
    seed = 10
    slots_seen = []
    for plan in plans:
        seqs = {}
        for rid, p, dec in plan:
            seed += 1
            seqs[rid] = _tokens(cfg["vocab_size"], p + dec, seed)
        rp.run([(rid, seqs[rid][:p], [p - 1]) for rid, p, dec in plan])
        slots_seen.append(sorted(rp.rep.slots.values()))
        for k in range(max(dec for _, _, dec in plan)):
            live = [(rid, p, dec) for rid, p, dec in plan if k < dec]
            rp.run([(rid, [seqs[rid][p + k]], [0]) for rid, p, dec in live],
                   end=[rid for rid, p, dec in live if k == dec - 1])
        for rid, p, dec in plan:
            ref = _ref(cfg, w, seqs[rid], dtype)
            for i in range(p - 1, p + dec):
                want[(rid, i)] = ref[i]
        assert not eng.cache.live_slots
        eng.cache.check()
    assert set(slots_seen[0]) <= set(slots_seen[1])      # the second batch used the first one's slots again
    _check(rp.got, want, dtype, f"{key} unequal batches")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", ["A", "B"])
def test_long_decoding_and_first_tokens(pe, engines, oracles, tmp_path, key, dtype):
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    n = 600
    toks = _tokens(cfg["vocab_size"], n, 30)
    rp = Replay(pe, eng, tmp_path)
    rp.run([("r", toks[:1], [0])])                         # a sequence's very first token, alone
    for i in range(1, n):
        rp.run([("r", [toks[i]], [0])], end=["r"] if i == n - 1 else [])
    ref = _ref(cfg, w, toks, dtype)
    _check(rp.got, {("r", i): ref[i] for i in range(n)}, dtype, f"{key} {n} tokens one by one")
    _check({k: v for k, v in rp.got.items() if k[1] < 3}, {("r", i): ref[i] for i in range(3)}, dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", ["B", "D", "E"])
def test_random_cuts_into_steps(pe, engines, oracles, tmp_path, key, dtype):
    """Three requests run together; every step brings each of them a random number of its next tokens
    (one, a few, or many; a request that has none left sits the step out).  Whatever the cuts, the
    logits at every position are those of the whole sequence."""
    import random
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    for seed in range(3):
        rng = random.Random(100 + seed)
        seqs = {str(i): _tokens(cfg["vocab_size"], rng.choice([40, 97, 130, 201]), 200 + 10 * seed + i) for i in range(3)}
        fed = {i: 0 for i in seqs}
        rp = Replay(pe, eng, tmp_path)
        while any(fed[i] < len(seqs[i]) for i in seqs):
            entries, end = [], []
            for i, toks in seqs.items():
                left = len(toks) - fed[i]
                if left == 0:
                    continue
                n = min(left, rng.choice([1, 1, 2, 5, 17, 64, 65, 120]))
                entries.append((i, toks[fed[i]:fed[i] + n], list(range(n))))
                fed[i] += n
                if fed[i] == len(toks):
                    end.append(i)
            rp.run(entries, end=end)
        want = {}
        for i, toks in seqs.items():
            ref = _ref(cfg, w, toks, dtype)
            want.update({(i, j): ref[j] for j in range(len(toks))})
        _check(rp.got, want, dtype, f"{key} random cuts, seed {seed}")
    assert not eng.cache.live_slots
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_equals_eager_steps(pe, engines, oracles, tmp_path, dtype):
    cfg, w = oracles["B", dtype]
    toks = [_tokens(cfg["vocab_size"], 90, 40 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        eng = engines("B", dtype, enable_cuda_graph=graphs)
        rp = Replay(pe, eng, tmp_path)
        rp.run([(str(i), t[:50 + i], [49 + i]) for i, t in enumerate(toks)])
        for k in range(30):
            rp.run([(str(i), [t[50 + i + k]], [0]) for i, t in enumerate(toks)], end=[str(i) for i in range(3)] if k == 29 else [])
        outs.append(rp.got)
        assert bool(eng.runner._graphs) == graphs
    for k in outs[0]:
        assert torch.equal(outs[0][k], outs[1][k]), f"graph and eager steps differ at {k}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key", KEYS)
def test_greedy_generation_through_the_entry_point(pe, engines, oracles, key, dtype):
    cfg, w = oracles[key, dtype]
    eng = engines(key, dtype)
    prompts = [_tokens(cfg["vocab_size"], n, 50 + n) for n in (5, 9, 13, 70)]
    params = pe.SamplingParams(max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0)
    results = eng.generate(prompts, params)
    assert not eng.cache.live_slots
    for p, r in zip(prompts, results):
        assert r.prompt_tokens == len(p) and r.finish_reason in ("length", "stop")
        if r.finish_reason == "length":
            assert r.completion_tokens == 8
        # every chosen token is the plain implementation's argmax, or within rounding of it
        ref = _ref(cfg, w, p + r.token_ids, dtype)
        scale = float(ref.abs().max())
        for j, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + j]
            assert float(row.max() - row[tok]) <= 2 * TOL[dtype] * scale, f"token {j} of a {len(p)}-token prompt"
    if dtype == "float32":
        for p, r in zip(prompts[:2], results[:2]):
            stops = cfg.get("eos_token_id", [])
            stops = stops if isinstance(stops, list) else [stops]
            assert r.token_ids == plain.generate_greedy(cfg, w, p, 8, stop_ids=stops)
    single = eng.generate(prompts[1], params)
    assert single.token_ids == results[1].token_ids


def test_generate_and_step_share_an_engine(pe, engines, oracles):
    """generate() and step() on the same engine, in either order, inside or outside torch's no-grad
    contexts: the buffers one call makes are written by the other."""
    cfg, w = oracles["D", "bfloat16"]
    eng = engines("D", "bfloat16")
    prompt = _tokens(cfg["vocab_size"], 20, 63)
    first = eng.generate([prompt, prompt[:7]], pe.SamplingParams.greedy_params(max_tokens=5))
    s = eng.alloc_slot()
    lg = eng.step([pe.StepEntry(s, prompt, (19,))])
    lg2 = eng.step([pe.StepEntry(s, [first[0].token_ids[0]], (0,))])
    eng.free_slot(s)
    assert int(lg[0].argmax()) == first[0].token_ids[0] and int(lg2[0].argmax()) == first[0].token_ids[1]
    with torch.inference_mode():
        again = eng.generate([prompt, prompt[:7]], pe.SamplingParams.greedy_params(max_tokens=5))
    assert [r.token_ids for r in again] == [r.token_ids for r in first]


def test_streaming_leaves_the_callers_grad_mode_alone_and_frees_slots_when_abandoned(pe, engines, oracles):
    cfg, w = oracles["A"]
    eng = engines("A", "float32")
    prompts = [_tokens(cfg["vocab_size"], n, 90 + n) for n in (5, 9)]
    whole = eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=6))
    got = {0: [], 1: []}
    for chunk in eng.stream_tokens(prompts, pe.SamplingParams.greedy_params(max_tokens=6)):
        assert torch.is_grad_enabled()           # between two chunks the caller's code runs in the caller's mode
        got[chunk.request].append(chunk.token_id)
    assert [got[0], got[1]] == [r.token_ids for r in whole]
    stream = eng.stream_tokens(prompts, pe.SamplingParams.greedy_params(max_tokens=6))
    next(stream)
    stream.close()                               # given up in mid-batch: the slots and pages come back
    assert eng.cache.live_slots == []
    eng.cache.check()
    assert [r.token_ids for r in eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=6))] == \
        [r.token_ids for r in whole]


def test_prompts_fed_in_several_steps_give_the_same_tokens(pe, engines, oracles):
    """A step limit of 37 tokens cuts these prompts into pieces, one of them in the middle of a page."""
    cfg, w = oracles["B"]
    prompts = [_tokens(cfg["vocab_size"], n, 200 + n) for n in (70, 3, 130, 36)]
    params = pe.SamplingParams.greedy_params(max_tokens=6)
    whole = engines("B", "float32").generate(prompts, params)
    cut = engines("B", "float32", max_step_tokens=37)
    pieces = cut.generate(prompts, params)
    assert [r.token_ids for r in pieces] == [r.token_ids for r in whole]
    assert pieces[3].token_ids == plain.generate_greedy(cfg, w, prompts[3], 6)
    assert not cut.cache.live_slots
    cut.cache.check()


def test_stop_token_and_context_limit(pe, engines, oracles):
    cfg, w = oracles["A"]
    eng = engines("A", "float32")
    prompt = _tokens(cfg["vocab_size"], 6, 60)
    free = eng.generate(prompt, pe.SamplingParams.greedy_params(max_tokens=6))
    assert free.completion_tokens == 6
    stopped = eng.generate(prompt, pe.SamplingParams.greedy_params(max_tokens=6, stop_token_ids=[free.token_ids[3]]))
    first = free.token_ids.index(free.token_ids[3])
    assert stopped.token_ids == free.token_ids[:first] and stopped.finish_reason == "stop"
    small = engines("A", "float32", max_context_len=16, max_cache_tokens=64)
    r = small.generate(_tokens(cfg["vocab_size"], 12, 61), pe.SamplingParams.greedy_params(max_tokens=50))
    assert r.completion_tokens == 4 and r.finish_reason == "length"
    with pytest.raises(ValueError, match="context"):
        small.generate(_tokens(cfg["vocab_size"], 17, 62), pe.SamplingParams.greedy_params(max_tokens=1))


def test_seeded_sampling_does_not_depend_on_batching(pe, engines, oracles):
    cfg, w = oracles["B"]
    prompts = [_tokens(cfg["vocab_size"], n, 70 + n) for n in (1, 7, 31, 64)]
    params = pe.SamplingParams(max_tokens=16, temperature=0.8, seed=11)
    together = engines("B", "float32").generate(prompts, params)
    again = engines("B", "float32").generate(prompts, params)
    assert [r.token_ids for r in together] == [r.token_ids for r in again]
    one_by_one = engines("B", "float32", max_batch=1).generate(prompts, params)
    assert [r.token_ids for r in together] == [r.token_ids for r in one_by_one]
    other = engines("B", "float32").generate(prompts, pe.SamplingParams(max_tokens=16, temperature=0.8, seed=12))
    assert [r.token_ids for r in together] != [r.token_ids for r in other]
    # every drawn token is the plain restatement's draw (same filters, same generator, keyed by the request's
    # number in the call and by how many tokens it has drawn), from the plain implementation's own logits
    differed = 0
    for r, res in enumerate(together):
        assert res.completion_tokens == 16
        differed += plain.check_drawn_tokens(cfg, w, prompts[r], res.token_ids, seed=11, request=r, margin=1e-3,
                                             temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)
    assert differed <= 2          # near ties may fall the other way; they are rare


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_repetition_penalty_through_generation(pe, engines, oracles, temperature):
    """A repetition penalty of 1.6, greedy and sampled, for three prompts of unequal lengths in one batch: every
    token is the plain implementation's draw from its own logits with the penalty on the prompt and on what has
    been drawn so far; the penalised greedy run differs from the run without."""
    cfg, w = oracles["A"]
    prompts = [_tokens(cfg["vocab_size"], n, 90 + n) for n in (5, 23, 2)]
    kw = dict(max_tokens=12, temperature=temperature, top_k=0, top_p=1.0, min_p=0.0, seed=5)
    eng = engines("A", "float32")
    pen = eng.generate(prompts, pe.SamplingParams(repetition_penalty=1.6, **kw))
    differed = 0
    for r, res in enumerate(pen):
        assert res.completion_tokens == 12
        differed += plain.check_drawn_tokens(cfg, w, prompts[r], res.token_ids, seed=5, request=r, margin=1e-3,
                                             temperature=temperature, repetition_penalty=1.6)
    assert differed <= 1
    if temperature == 0.0:
        # (a sampled draw with the same random numbers and slightly shifted probabilities often stays the same)
        free = eng.generate(prompts, pe.SamplingParams(**kw))
        assert [r.token_ids for r in pen] != [r.token_ids for r in free]


def test_cache_too_small_is_an_error_not_a_wrong_result(pe, engines, oracles):
    cfg, w = oracles["A"]
    eng = engines("A", "float32", max_cache_tokens=128, max_context_len=128)
    s = eng.alloc_slot()
    with pytest.raises(pe.cache.CacheFull):
        eng.step([pe.StepEntry(s, _tokens(cfg["vocab_size"], 129, 80), (0,))])
    assert eng.cache.length(s) == 0
    eng.free_slot(s)
    with pytest.raises(pe.kernels.KernelError, match="token id"):
        s = eng.alloc_slot()
        try:
            eng.step([pe.StepEntry(s, [cfg["vocab_size"] + 3], (0,))])
        finally:
            eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(pe, model_folders, oracles, tmp_path, dtype):
    """The program itself, as a user runs it: steps on standard input, ``done`` lines, .f32 files."""
    cfg, w = oracles["B", dtype]
    a, b = _tokens(cfg["vocab_size"], 75, 90), _tokens(cfg["vocab_size"], 20, 91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:18], "want": [17]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[70]], "want": [0]}, {"id": "b", "tokens": [b[18]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[71]], "want": [0]}, {"id": "b", "tokens": [b[19]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[72]], "want": []}], "end": []},
             {"step": 7, "entries": [{"id": "a", "tokens": [a[73]], "want": [0]}, ], "end": ["a"]},
             {"step": 8, "entries": [{"id": "c", "tokens": b, "want": [19]}], "end": ["c"]}]
    out = tmp_path / "out"
    env = dict(os.environ)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders[dtype]["B"], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "192"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "7", "done", "8"]
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32", "7.f32", "8.f32"]
    V = cfg["vocab_size"]
    read = lambda s: torch.frombuffer(bytearray(open(out / f"{s}.f32", "rb").read()), dtype=torch.float32).view(-1, V)
    ra, rb = _ref(cfg, w, a, dtype), _ref(cfg, w, b, dtype)
    got = {("a", 0): read(0)[0], ("a", 69): read(0)[1], ("b", 17): read(0)[2], ("a", 70): read(1)[0],
           ("a", 71): read(2)[0], ("b", 19): read(2)[1], ("a", 73): read(7)[0], ("c", 19): read(8)[0]}
    assert read(0).shape == (3, V) and read(1).shape == (1, V)
    want = {k: (ra if k[0] == "a" else rb)[k[1]] for k in got}
    _check(got, want, dtype, "trace_run")


@pytest.mark.parametrize("hidden,inter,heads,kv,d,window", [(256, 384, 4, 2, 128, None), (200, 328, 6, 2, 64, 300),
                                                           (320, 640, 2, 1, 128, 700), (192, 256, 5, 1, 128, None)])
def test_a_prompt_of_more_than_a_thousand_tokens(pe, hidden, inter, heads, kv, d, window):
    """Prompts this long take the many-row kernels (the tcgen05 products where K is a multiple of 64,
    the tcgen05 attention at head size 128): a long and a short prompt in one step, then single tokens,
    at the first, a middle and the last position of the long prompt."""
    cfgd = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv, head_dim=d, intermediate_size=inter, vocab_size=515, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048)
    if window:
        cfgd.update(use_sliding_window=True, sliding_window=window, max_window_layers=1)
    cfg = pe.Qwen3Config.from_dict(cfgd)
    eng = pe.Engine.from_random(cfg, seed=5, dtype="bfloat16", max_context_len=2048, max_cache_tokens=4096, max_batch=2)
    w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 5, device="cuda:0").items()}
    lens = [1100, 70]
    seqs = [_tokens(515, L + 3, 40 + i) for i, L in enumerate(lens)]
    wants = [(0, 600, 1099), (69,)]
    slots = [eng.alloc_slot(), eng.alloc_slot()]
    lg = eng.step([pe.StepEntry(s, q[:L], wt) for s, q, L, wt in zip(slots, seqs, lens, wants)]).float().cpu()
    got = [[lg[0], lg[1], lg[2]], [lg[3]]]
    for t in range(3):
        lg = eng.step([pe.StepEntry(s, [q[L + t]], (0,)) for s, q, L in zip(slots, seqs, lens)]).float().cpu()
        got[0].append(lg[0]); got[1].append(lg[1])
    for s in slots:
        eng.free_slot(s)
    for i, (q, L) in enumerate(zip(seqs, lens)):
        ref = plain.forward_logits(cfg.to_dict(), w, q, store=torch.bfloat16)
        idx = list(wants[i]) + [L + t for t in range(3)]
        assert rel_err(torch.stack(got[i]), ref[idx]) < TOL["bfloat16"]
