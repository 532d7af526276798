"""Batches of 9 to 64 sequences against the plain implementation, and what a request's result may and may
not depend on: in float32 nothing but its own tokens (bit for bit, with the matrix product held fixed), in
bfloat16 the batch size within a stated bound."""
import math
import random

import pytest
import torch

import plain_qwen3 as plain
from conftest import TEST_CONFIGS, TOL, rel_err
from test_model_gpu import Replay, _check, _ref, _tokens, oracles  # noqa: F401  (oracles is a fixture)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def big_engines(pe, model_folders):
    made = {}

    def get(key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in made:
            args = dict(dtype=dtype, max_cache_tokens=64 * 384, max_batch=64)
            args.update(kw)
            made[ident] = pe.Engine(model_folders[dtype][key], **args)
        return made[ident]

    return get


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key,n_requests", [("B", 12), ("D", 33), ("E", 64), ("B", 64), ("D", 12), ("E", 33)])
def test_many_sequences_in_one_batch(pe, big_engines, oracles, tmp_path, key, n_requests, dtype):
    """``n_requests`` requests of unequal lengths (1 to 300 tokens) go in as one prefill step; then each gets one
    token per step and the shorter ones end earlier (the batch shrinks through every size down to one); a second
    batch of as many requests follows on the slots and pages the first gave back.  Every logit row against the
    plain implementation.  Decode steps of more than 8 sequences run other kernels than the small batches of the
    other tests: library products inside captured graphs, the fused gate|up product on tcgen05 at few rows,
    longer attention ranges, the sampler-free logits of up to 64 rows."""
    cfg, w = oracles[key, dtype]
    eng = big_engines(key, dtype)
    rp = Replay(pe, eng, tmp_path)
    rng = random.Random(1000 * n_requests + len(key))
    want = {}
    slots_seen = []
    for batch in range(2):
        plan = []
        for r in range(n_requests):
            p = rng.choice([1, 2, 7, 31, 63, 64, 65, 100, 128, 200, 300]) if r else 300
            dec = rng.randint(1, 14)
            plan.append((f"{batch}.{r}", p, dec))
        seqs = {rid: _tokens(cfg["vocab_size"], p + dec, rng.randrange(1 << 30)) for rid, p, dec in plan}
        rp.run([(rid, seqs[rid][:p], [p - 1]) for rid, p, dec in plan])
        slots_seen.append(sorted(rp.rep.slots.values()))
        sizes = set()
        for k in range(max(dec for _, _, dec in plan)):
            live = [(rid, p, dec) for rid, p, dec in plan if k < dec]
            sizes.add(len(live))
            rp.run([(rid, [seqs[rid][p + k]], [0]) for rid, p, dec in live],
                   end=[rid for rid, p, dec in live if k == dec - 1])
        assert max(sizes) == n_requests and min(sizes) <= 8        # large and small decode batches both ran
        for rid, p, dec in plan:
            ref = _ref(cfg, w, seqs[rid], dtype)
            for i in range(p - 1, p + dec):
                want[(rid, i)] = ref[i]
        assert not eng.cache.live_slots
        eng.cache.check()
    assert set(slots_seen[0]) == set(slots_seen[1])                 # the second batch ran on the first one's slots
    assert eng.runtime.status.tolist()[0] == 0
    _check(rp.got, want, dtype, f"{key}, {n_requests} requests in a batch")


# ---- what a request's result depends on ----------------------------------------------------------------------
@pytest.mark.parametrize("nh,nkv,d", [(8, 2, 64), (6, 2, 32), (5, 5, 48)])
def test_float32_decode_attention_is_bit_equal_in_any_batch(pe, nh, nkv, d):
    """The float32 decode attention cuts a sequence's keys into ranges by that sequence's length alone and adds
    in a fixed order: the same sequence gives the same bits alone, among 8 and among 64, wherever it stands in
    the batch and whatever the others hold."""
    from test_kernels_gpu import PagedSetup
    ops = pe.kernels.ops
    split = 512
    rng = random.Random(3)
    for own_len in (1, 700, 1300):
        outs = []
        for others in (0, 7, 63):
            lens = [rng.choice([1, 5, 64, 300, 513, 1100, 1500]) for _ in range(others)]
            where = rng.randrange(others + 1)
            lens.insert(where, own_len)
            ps = PagedSetup(lens, nkv, d, torch.float32, seed=others, key_scale=2.0)
            # the sequence under test has the same keys, values and query in every batch
            g = torch.Generator().manual_seed(99)
            k_own = torch.randn(own_len, nkv, d, generator=g) * 2.0
            v_own = torch.randn(own_len, nkv, d, generator=g)
            q_own = torch.randn(nh * d, generator=g)
            for lp in range((own_len + 63) // 64):
                page = int(ps.table[ps.slots[where], lp])
                n = min(64, own_len - lp * 64)
                ps.k_pages[page, :, :n] = k_own[lp * 64: lp * 64 + n].transpose(0, 1).to(DEV)
                ps.v_pages[page, :, :n] = v_own[lp * 64: lp * 64 + n].transpose(0, 1).to(DEV)
            B = len(lens)
            q = torch.randn(B, nh * d, generator=g)
            q[where] = q_own
            q = q.to(DEV)
            max_splits = -(-max(lens) // split)
            out = torch.zeros(B, nh * d, device=DEV)
            scratch = torch.zeros(ops.attention_generic_scratch_floats(B, nh, d, max_splits), device=DEV)
            status = torch.zeros(4, dtype=torch.int32, device=DEV)
            ops.attention_generic(True, q, out, B, 1, nh, nkv, d, 1 / math.sqrt(d), 0,
                                  torch.arange(B + 1, dtype=torch.int32, device=DEV),
                                  torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=DEV), ps.seq_slot, ps.table,
                                  ps.num_pages, ps.k_pages, ps.v_pages, scratch, split, max_splits, status)
            assert status.tolist()[0] == 0
            outs.append(out[where].cpu())
        want = plain.causal_gqa_attention(q_own.view(1, nh, d).expand(own_len, nh, d).contiguous(), k_own, v_own, d ** -0.5)[-1]
        assert rel_err(outs[0], want.reshape(-1)) < 5e-6
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), f"length {own_len}"


def _row_by_row(x, weight, out, out_dtype):
    """A matrix product whose every output row is computed by the same call whatever the number of rows: the
    library's matrix-vector product, one row at a time (true float32)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        y = torch.stack([torch.mv(weight, x[i]) for i in range(x.shape[0])])
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    if out_dtype is not None:
        y = y.to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


@pytest.mark.parametrize("key", ["B", "D"])
def test_float32_logits_do_not_depend_on_the_batch_bit_for_bit(pe, model_folders, oracles, tmp_path, key):
    """With the matrix product held fixed (the same routine for every row: the library picks other kernels, with
    other summation orders, for other numbers of rows, and that is its business), everything this package adds
    (norms, rotation, cache, attention over ranges, their merge) must give a request the same bits alone, with
    7 others and with 63 others, in prefill and in decode."""
    cfg, w = oracles[key, "float32"]
    eng = pe.Engine(model_folders["float32"][key], dtype="float32", max_cache_tokens=64 * 200, max_batch=64,
                    enable_cuda_graph=False)
    eng.runtime.gemm_backend = _row_by_row
    own = _tokens(cfg["vocab_size"], 150, 77)
    p, dec = 140, 10
    rows = []
    for others in (0, 7, 63):
        rp = Replay(pe, eng, tmp_path)
        rng = random.Random(others)
        ids = [f"o{i}" for i in range(others)]
        lens = {i: rng.choice([1, 9, 64, 65, 130]) for i in ids}
        seqs = {i: _tokens(cfg["vocab_size"], lens[i] + dec, rng.randrange(1 << 30)) for i in ids}
        where = rng.randrange(others + 1)
        order = ids[:where] + ["own"] + ids[where:]
        seqs["own"], lens["own"] = own, p
        rp.run([(i, seqs[i][:lens[i]], [lens[i] - 1]) for i in order])
        for k in range(dec):
            rp.run([(i, [seqs[i][lens[i] + k]], [0]) for i in order], end=order if k == dec - 1 else [])
        rows.append(torch.stack([rp.got[("own", j)] for j in range(p - 1, p + dec)]))
    ref = _ref(cfg, w, own, "float32")[p - 1:]
    assert rel_err(rows[0], ref) < TOL["float32"]
    assert torch.equal(rows[0], rows[1]), "alone and with 7 others"
    assert torch.equal(rows[0], rows[2]), "alone and with 63 others"


# How far a request's bfloat16 logits may move with the batch it runs in, relative to the largest logit.  The
# batch size picks the kernels (products of <= 8, 9..1,023 and more rows; how many ranges the decode attention
# cuts a sequence into), and each sums in another order, so single roundings to bfloat16 fall differently.  The
# bound is half the tolerance against the plain implementation.
BATCH_DRIFT_BF16 = 1e-2


@pytest.mark.parametrize("key", ["B", "D", "E"])
def test_bfloat16_logits_move_with_the_batch_by_less_than_the_stated_bound(pe, big_engines, oracles, tmp_path, key):
    cfg, w = oracles[key, "bfloat16"]
    eng = big_engines(key, "bfloat16")
    own = _tokens(cfg["vocab_size"], 150, 78)
    p, dec = 140, 10
    rows = []
    for others in (0, 7, 63):
        rp = Replay(pe, eng, tmp_path)
        rng = random.Random(others)
        ids = [f"o{i}" for i in range(others)]
        lens = {i: rng.choice([1, 9, 64, 65, 130]) for i in ids}
        seqs = {i: _tokens(cfg["vocab_size"], lens[i] + dec, rng.randrange(1 << 30)) for i in ids}
        where = rng.randrange(others + 1)
        order = ids[:where] + ["own"] + ids[where:]
        seqs["own"], lens["own"] = own, p
        rp.run([(i, seqs[i][:lens[i]], [lens[i] - 1]) for i in order])
        for k in range(dec):
            rp.run([(i, [seqs[i][lens[i] + k]], [0]) for i in order], end=order if k == dec - 1 else [])
        rows.append(torch.stack([rp.got[("own", j)] for j in range(p - 1, p + dec)]))
    scale = float(rows[0].abs().max())
    drift = max(float((rows[0] - r).abs().max()) / scale for r in rows[1:])
    assert drift < BATCH_DRIFT_BF16, f"{key}: logits moved by {drift:.2e} of the largest logit with the batch"
    ref = _ref(cfg, w, own, "bfloat16")[p - 1:]
    for r in rows:
        assert rel_err(r, ref) < TOL["bfloat16"]


def greedy_agreement(pe, eng, vocab, n_requests=64, new_tokens=24, seed=5):
    """Greedy generation of ``n_requests`` random prompts, each alone and all in one batch: (share of requests whose
    tokens are the same both ways, share of tokens equal up to each request's first difference)."""
    rng = random.Random(seed)
    prompts = [_tokens(vocab, rng.choice([3, 17, 64, 90, 150]), rng.randrange(1 << 30)) for _ in range(n_requests)]
    params = pe.SamplingParams.greedy_params(max_tokens=new_tokens)
    together = [r.token_ids for r in eng.generate(prompts, params)]
    alone = [eng.generate([p], params)[0].token_ids for p in prompts]
    same = sum(a == b for a, b in zip(alone, together))
    agree = 0
    for a, b in zip(alone, together):
        n = 0
        while n < min(len(a), len(b)) and a[n] == b[n]:
            n += 1
        agree += n
    return same / n_requests, agree / (n_requests * new_tokens)


def test_greedy_tokens_alone_and_in_a_batch_of_64(pe, big_engines, oracles, model_folders):
    """float32: the logits differ by 1e-6 of their scale at most between the two ways (the library's products pick
    other kernels for other numbers of rows), so the tokens are the same unless two top logits are that close: on
    these models all 64 requests came out identical, and at most a stray near tie may change that.  bfloat16: random
    weights give nearly tied logits, so a rounding that falls differently can change a token, and every later token
    with it; the figure is printed (run with -s) and must not collapse."""
    cfg, _ = oracles["D", "float32"]
    eng32 = pe.Engine(model_folders["float32"]["D"], dtype="float32", max_cache_tokens=64 * 256, max_batch=64)
    same32, agree32 = greedy_agreement(pe, eng32, cfg["vocab_size"])
    eng16 = big_engines("D", "bfloat16")
    same16, agree16 = greedy_agreement(pe, eng16, cfg["vocab_size"])
    print(f"\ngreedy, 64 requests x 24 tokens, alone vs in one batch: float32 {same32:.0%} of requests identical "
          f"({agree32:.1%} of tokens before a first difference); bfloat16 {same16:.0%} ({agree16:.1%})")
    assert same32 >= 0.95 and agree32 >= 0.97
    assert agree16 > 0.5
