"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""
import math
import random

import pytest
import torch

import plain_qwen3 as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
KTOL = {torch.float32: 2e-6, torch.bfloat16: 8e-3}   # one rounding of the output (2^-9 = 2e-3, a few ulps)


@pytest.fixture(scope="module")
def ops(pe):
    pe.kernels.library()
    return pe.kernels.ops


def _status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(515, 80, device=DEV).to(dtype)
    ids = torch.tensor([0, 514, 7, 7, 300], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 80, device=DEV)
    st = _status()
    ops.embed_gather(table, ids, out, st)
    assert torch.equal(out, table.float()[ids.long()])
    assert st.tolist()[0] == 0
    bad = torch.tensor([3, 515], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, 80, device=DEV)
    ops.embed_gather(table, bad, out2, st)
    assert st.tolist()[:3] == [1, 1, 515] and float(out2[1].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [80, 1000, 4096, 5120])
@pytest.mark.parametrize("n", [7, 100])    # a handful of rows get more threads a row than many rows do
def test_rmsnorm_with_residual(ops, dtype, dim, n):
    torch.manual_seed(1)
    res = torch.randn(n, dim, device=DEV) * 3
    delta = torch.randn(n, dim, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(dim, device=DEV)
    eps = 3e-6
    want_h = res + delta.float()
    want = plain.rms_norm(want_h.cpu(), w.cpu(), eps)
    # add + write back + norm
    r1, out = res.clone(), torch.empty(n, dim, device=DEV, dtype=dtype)
    ops.rmsnorm_residual(r1, delta, w, out, eps)
    assert torch.equal(r1, want_h)
    assert rel_err(out.float().cpu(), want) < KTOL[dtype]
    # no delta: the stream is left alone
    r2, out2 = res.clone(), torch.empty(n, dim, device=DEV, dtype=dtype)
    ops.rmsnorm_residual(r2, None, w, out2, eps)
    assert torch.equal(r2, res)
    assert rel_err(out2.float().cpu(), plain.rms_norm(res.cpu(), w.cpu(), eps)) < KTOL[dtype]
    # gathered rows: nothing written back
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    r3, out3 = res.clone(), torch.empty(3, dim, device=DEV, dtype=dtype)
    ops.rmsnorm_residual(r3, delta, w, out3, eps, rows)
    assert torch.equal(r3, res)
    assert rel_err(out3.float().cpu(), want[[5, 0, 5]]) < KTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_plain(ops, dtype):
    torch.manual_seed(2)
    x = torch.randn(6, 5, 48, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(48, device=DEV)
    out = torch.empty_like(x)
    ops.rmsnorm(x, w, out, 1e-5)
    assert rel_err(out.float().cpu(), plain.rms_norm(x.float().cpu(), w.cpu(), 1e-5)) < KTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,inter", [(1, 176), (9, 200), (33, 3072)])
def test_silu_mul(ops, dtype, n, inter):
    torch.manual_seed(3)
    gu = (torch.randn(n, 2 * inter, device=DEV) * 4).to(dtype)
    out = torch.empty(n, inter, device=DEV, dtype=dtype)
    ops.silu_mul(gu, out)
    g, u = gu.float().cpu()[:, :inter], gu.float().cpu()[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    assert rel_err(out.float().cpu(), want) < KTOL[dtype]


def test_batch_expand(ops):
    qstart = torch.tensor([0, 3, 4, 4, 9], dtype=torch.int32, device=DEV)      # the third sequence brings nothing
    past = torch.tensor([10, 0, 7, 100], dtype=torch.int32, device=DEV)
    seq = torch.full((9,), -1, dtype=torch.int32, device=DEV)
    pos = torch.full((9,), -1, dtype=torch.int32, device=DEV)
    ops.batch_expand(qstart, past, 4, seq, pos)
    assert seq.tolist() == [0, 0, 0, 1, 3, 3, 3, 3, 3]
    assert pos.tolist() == [10, 11, 12, 0, 100, 101, 102, 103, 104]


class PagedSetup:
    """A batch of sequences with keys and values scattered over shuffled pages of a pool."""

    def __init__(self, lens, nkv, d, dtype, seed=0, extra_pages=5, key_scale=1.0):
        g = torch.Generator().manual_seed(seed)
        self.lens, self.nkv, self.d, self.dtype = lens, nkv, d, dtype
        B = len(lens)
        pages_per = [(L + 63) // 64 for L in lens]
        self.num_pages = sum(pages_per) + extra_pages
        order = list(range(self.num_pages))
        random.Random(seed).shuffle(order)
        self.table_width = max(pages_per) + 2
        self.slots = list(range(B - 1, -1, -1))   # slot numbers differ from batch order
        table = torch.full((B + 1, self.table_width), -1, dtype=torch.int32)
        self.k = [(torch.randn(L, nkv, d, generator=g) * key_scale).to(dtype) for L in lens]
        self.v = [torch.randn(L, nkv, d, generator=g).to(dtype) for L in lens]
        kp = torch.randn(self.num_pages, nkv, 64, d, generator=g).to(dtype)   # junk where nothing was written
        vp = torch.randn(self.num_pages, nkv, 64, d, generator=g).to(dtype)
        it = iter(order)
        for b, L in enumerate(lens):
            for lp in range(pages_per[b]):
                page = next(it)
                table[self.slots[b], lp] = page
                n = min(64, L - lp * 64)
                kp[page, :, :n] = self.k[b][lp * 64: lp * 64 + n].transpose(0, 1)
                vp[page, :, :n] = self.v[b][lp * 64: lp * 64 + n].transpose(0, 1)
        self.k_pages, self.v_pages, self.table = kp.to(DEV), vp.to(DEV), table.to(DEV)
        self.seq_slot = torch.tensor(self.slots, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot", [(4, 2, 16, 16), (6, 2, 32, 32), (5, 5, 48, 48), (8, 1, 128, 64), (3, 3, 80, 80),
                                        (8, 2, 128, 128), (2, 1, 256, 256), (7, 3, 96, 96), (9, 3, 64, 64)])
@pytest.mark.parametrize("lens,q_lens", [([70, 3, 129], [6, 3, 65]), ([300, 3, 200], [230, 3, 136])])
def test_qk_norm_rope_append(ops, dtype, nh, nkv, d, rot, lens, q_lens):
    # lens: lengths after the step; q_lens: tokens this step brings (the second sequence starts here);
    # the longer step takes the 16-byte kernel where the sizes allow it
    torch.manual_seed(4)
    ps = PagedSetup(lens, nkv, d, dtype, seed=4)
    N = sum(q_lens)
    ld = (nh + 2 * nkv) * d + 16        # row stride larger than the row
    qkv = torch.randn(N, ld, device=DEV).to(dtype)
    before = qkv.clone()
    qw = 1 + 0.2 * torch.randn(d, device=DEV)
    kw = 1 + 0.2 * torch.randn(d, device=DEV)
    eps, theta, max_pos = 1e-5, 1e4, 512
    inv = plain.rope_inv_freq(rot, theta)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    cos, sin = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    token_seq = torch.tensor(sum(([b] * n for b, n in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
    pos_list = sum(([lens[b] - q_lens[b] + i for i in range(q_lens[b])] for b in range(3)), [])
    token_pos = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0, q_lens[0], q_lens[0] + q_lens[1], N], dtype=torch.int32, device=DEV)
    k_before, v_before = ps.k_pages.clone(), ps.v_pages.clone()
    st = _status()
    ops.qk_norm_rope_append(qkv[:, : ld], N, nh, nkv, d, qw, kw, eps, cos, sin, rot, token_seq, token_pos, ps.seq_slot,
                            qstart, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, True, st)
    assert st.tolist()[0] == 0
    x = before.float().cpu()
    q_in = x[:, : nh * d].view(N, nh, d)
    k_in = x[:, nh * d: (nh + nkv) * d].view(N, nkv, d)
    v_in = x[:, (nh + nkv) * d: (nh + 2 * nkv) * d].view(N, nkv, d)
    c, s = plain.rope_cos_sin(torch.tensor(pos_list), rot, theta)
    q_want = plain.rope_rotate_neox(plain.rms_norm(q_in, qw.cpu(), eps), c, s, rot)
    k_want = plain.rope_rotate_neox(plain.rms_norm(k_in, kw.cpu(), eps), c, s, rot)
    got = qkv.float().cpu()
    assert rel_err(got[:, : nh * d].view(N, nh, d), q_want) < KTOL[dtype]
    assert rel_err(got[:, nh * d: (nh + nkv) * d].view(N, nkv, d), k_want) < KTOL[dtype]
    assert torch.equal(got[:, (nh + nkv) * d:], x[:, (nh + nkv) * d:])     # v and the padding are untouched
    # the cache holds exactly the new rows, at their pages; every other row is as before
    touched = torch.zeros(ps.num_pages, 64, dtype=torch.bool)
    kp, vp = ps.k_pages.float().cpu(), ps.v_pages.float().cpu()
    for t, (b, p) in enumerate(zip(token_seq.tolist(), pos_list)):
        page = int(ps.table[ps.slots[b], p // 64])
        touched[page, p % 64] = True
        assert rel_err(kp[page, :, p % 64], k_want[t]) < KTOL[dtype]
        assert torch.equal(vp[page, :, p % 64], v_in[t])
    # the last token of each multi-token step clears the rest of its page (rows after it hold zeros);
    # every other row is as before
    cleared = torch.zeros(ps.num_pages, 64, dtype=torch.bool)
    for b in range(3):
        last = lens[b] - 1
        page = int(ps.table[ps.slots[b], last // 64])
        cleared[page, last % 64 + 1:] = True
    keep = ~touched & ~cleared
    assert torch.equal(ps.k_pages.cpu().transpose(1, 2)[keep], k_before.cpu().transpose(1, 2)[keep])
    assert torch.equal(ps.v_pages.cpu().transpose(1, 2)[keep], v_before.cpu().transpose(1, 2)[keep])
    assert float(ps.k_pages.float().cpu().transpose(1, 2)[cleared].abs().sum()) == 0.0
    assert float(ps.v_pages.float().cpu().transpose(1, 2)[cleared].abs().sum()) == 0.0
    # write_cache off: q and k are still rewritten, the cache is not
    k_now = ps.k_pages.clone()
    qkv2 = before.clone()
    ops.qk_norm_rope_append(qkv2, N, nh, nkv, d, qw, kw, eps, cos, sin, rot, token_seq, token_pos, ps.seq_slot,
                            qstart, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, False, st)
    assert torch.equal(qkv2, qkv) and torch.equal(ps.k_pages, k_now)


def _plain_attention(ps, q_list, pasts, nh, scale, window):
    outs = []
    for b, q in enumerate(q_list):
        T = pasts[b] + q.shape[0]
        outs.append(plain.causal_gqa_attention(q.float(), ps.k[b][:T].float(), ps.v[b][:T].float(), scale,
                                               window=window, q_start=pasts[b]))
    return torch.cat(outs, 0)


ATT_TOL = {torch.float32: 5e-6, torch.bfloat16: 8e-3}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 16), (6, 2, 32), (5, 5, 48), (8, 1, 128), (4, 1, 256), (2, 2, 80)])
@pytest.mark.parametrize("window", [0, 37])
def test_attention_prefill(ops, dtype, nh, nkv, d, window):
    torch.manual_seed(5)
    lens = [200, 1, 77, 64]
    pasts = [0, 0, 50, 0]                # the third sequence continues an earlier chunk
    q_lens = [L - p for L, p in zip(lens, pasts)]
    ps = PagedSetup(lens, nkv, d, dtype, seed=5, key_scale=2.0)
    N = sum(q_lens)
    ld = nh * d + 32
    q_all = torch.randn(N, ld, device=DEV).to(dtype)
    out = torch.zeros(N, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    st = _status()
    ops.attention_generic(False, q_all, out, len(lens), max(q_lens), nh, nkv, d, scale, window, qstart, past_t,
                          ps.seq_slot, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, None, 0, 0, st)
    assert st.tolist()[0] == 0
    qs, o = [], 0
    for n in q_lens:
        qs.append(q_all[o:o + n, : nh * d].cpu().view(n, nh, d)); o += n
    want = _plain_attention(ps, qs, pasts, nh, scale, window or None)
    assert rel_err(out.float().cpu().view(N, nh, d), want) < ATT_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 16), (6, 2, 32), (5, 5, 48), (32, 8, 128), (4, 1, 256), (16, 2, 64)])
@pytest.mark.parametrize("window", [0, 300])
def test_attention_decode(ops, dtype, nh, nkv, d, window):
    torch.manual_seed(6)
    lens = [1, 700, 256, 257, 33]        # one token, several ranges, a range's edge on both sides
    pasts = [L - 1 for L in lens]
    ps = PagedSetup(lens, nkv, d, dtype, seed=6, key_scale=2.0)
    B = len(lens)
    q_all = torch.randn(B, nh * d, device=DEV).to(dtype)
    out = torch.zeros(B, nh * d, device=DEV, dtype=dtype)
    qstart = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    split_keys, max_splits = 256, 4       # 4 ranges allowed although the longest needs 3
    scratch = torch.full((ops.attention_generic_scratch_floats(B, nh, d, max_splits),), float("nan"), device=DEV)
    st = _status()
    ops.attention_generic(True, q_all, out, B, 1, nh, nkv, d, scale, window, qstart, past_t, ps.seq_slot, ps.table,
                          ps.num_pages, ps.k_pages, ps.v_pages, scratch, split_keys, max_splits, st)
    assert st.tolist()[0] == 0
    qs = [q_all[b: b + 1].cpu().view(1, nh, d) for b in range(B)]
    want = _plain_attention(ps, qs, pasts, nh, scale, window or None)
    assert rel_err(out.float().cpu().view(B, nh, d), want) < ATT_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_attention_finds_a_far_key(ops, decode, dtype):
    """One key among hundreds matches the query; the output must be that key's value."""
    nh, nkv, d = 4, 2, 32
    L, far = 650, 13
    ps = PagedSetup([L], nkv, d, dtype, seed=7, key_scale=0.05)
    q = torch.zeros(1, nh * d)
    probe = torch.randn(d)
    probe = probe / probe.norm() * 12.0
    for h in range(nh):
        q[0, h * d:(h + 1) * d] = probe
    page = int(ps.table[ps.slots[0], far // 64])
    ps.k_pages[page, :, far % 64] = (probe.to(DEV) * 2.0).to(dtype)       # score 288*scale against ~0 elsewhere
    q_lens = [1]
    out = torch.zeros(1, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    past_t = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    scratch = torch.zeros(ops.attention_generic_scratch_floats(1, nh, d, 3), device=DEV)
    ops.attention_generic(decode, q.to(DEV, dtype), out, 1, 1, nh, nkv, d, 1 / math.sqrt(d), 0, qstart, past_t, ps.seq_slot,
                          ps.table, ps.num_pages, ps.k_pages, ps.v_pages, scratch if decode else None,
                          256 if decode else 0, 3 if decode else 0, _status())
    v_far = ps.v_pages[page, :, far % 64].float().cpu()       # [nkv, d]
    got = out.float().cpu().view(nh, d)
    for h in range(nh):
        assert torch.allclose(got[h], v_far[h // 2], atol=1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("kernel,decode", [("generic_f32", False), ("generic_f32", True), ("generic_bf16", False),
                                           ("generic_bf16", True), ("mma", False), ("mma", True), ("umma", False)])
def test_attention_at_the_windows_edge(ops, kernel, decode):
    """Two keys match the query strongly: the last one outside the window of the last query and the
    first one inside it.  With an edge off by one either way the output changes by tens."""
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    nh, nkv, d = (8, 2, 128) if kernel in ("mma", "umma") else (4, 2, 32)
    L, W = 200, 50
    outside, inside = L - 1 - W, L - W            # positions 149 and 150 for the query at 199
    ps = PagedSetup([L], nkv, d, dtype, seed=21, key_scale=0.05)
    probe = torch.randn(d)
    probe = probe / probe.norm() * 12.0
    for pos, value in ((outside, 50.0), (inside, -30.0)):
        page = int(ps.table[ps.slots[0], pos // 64])
        ps.k_pages[page, :, pos % 64] = (probe * 2.0).to(DEV, dtype)
        ps.v_pages[page, :, pos % 64] = value
        ps.k[0][pos] = (probe * 2.0).to(dtype)
        ps.v[0][pos] = value
    n_q = 1 if decode else L
    past = L - n_q
    q = probe.repeat(n_q, nh).contiguous()          # every query matches the two keys
    ld = nh * d + 2 * nkv * d
    q_all = torch.zeros(n_q, ld)
    q_all[:, : nh * d] = q
    q_all = q_all.to(DEV, dtype)
    out = torch.zeros(n_q, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0, n_q], dtype=torch.int32, device=DEV)
    past_t = torch.tensor([past], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    scratch = torch.zeros(ops.attention_generic_scratch_floats(1, nh, d, 4), device=DEV) if decode else None
    split = (64, 4) if decode else (0, 0)
    st = _status()
    if kernel == "umma":
        ops.attention_umma_prefill(q_all, out, 1, n_q, nh, nkv, d, scale, W, qstart, past_t, ps.seq_slot, ps.table,
                                   ps.num_pages, ps.k_pages, ps.v_pages, st)
    else:
        fn = ops.attention_mma if kernel == "mma" else ops.attention_generic
        fn(decode, q_all, out, 1, n_q, nh, nkv, d, scale, W, qstart, past_t, ps.seq_slot, ps.table, ps.num_pages,
           ps.k_pages, ps.v_pages, scratch, split[0], split[1], st)
    assert st.tolist()[0] == 0
    got = out.float().cpu().view(n_q, nh, d)
    want = plain.causal_gqa_attention(q.view(n_q, nh, d).float(), ps.k[0].float(), ps.v[0].float(), scale, window=W,
                                      q_start=past)
    tol = 1e-3 if dtype == torch.float32 else 0.3
    assert float((got - want).abs().max()) < tol
    # the last query sees the inside key only, the one before it both
    assert abs(float(got[-1].mean()) + 30.0) < 0.5
    if not decode:
        assert abs(float(got[-2].mean()) - 10.0) < 0.5


MMA_SHAPES = [(8, 2, 64), (32, 8, 128), (16, 1, 128), (3, 3, 64), (6, 2, 128), (10, 2, 64)]


@pytest.mark.parametrize("nh,nkv,d", MMA_SHAPES)
@pytest.mark.parametrize("window", [0, 37, 150])
def test_attention_mma_prefill(ops, nh, nkv, d, window):
    torch.manual_seed(15)
    dtype = torch.bfloat16
    assert ops.attention_mma_supported(dtype, d, nh, nkv)
    lens = [200, 1, 77, 64, 130]
    pasts = [0, 0, 50, 0, 127]            # the third and the last sequence continue earlier chunks
    q_lens = [L - p for L, p in zip(lens, pasts)]
    ps = PagedSetup(lens, nkv, d, dtype, seed=15, key_scale=2.0)
    N = sum(q_lens)
    ld = nh * d + 2 * nkv * d             # q rows inside a fused q|k|v buffer
    q_all = torch.randn(N, ld, device=DEV).to(dtype)
    out = torch.zeros(N, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    st = _status()
    ops.attention_mma(False, q_all, out, len(lens), max(q_lens), nh, nkv, d, scale, window, qstart, past_t,
                      ps.seq_slot, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, None, 0, 0, st)
    assert st.tolist()[0] == 0
    qs, o = [], 0
    for n in q_lens:
        qs.append(q_all[o:o + n, : nh * d].cpu().view(n, nh, d)); o += n
    want = _plain_attention(ps, qs, pasts, nh, scale, window or None)
    assert rel_err(out.float().cpu().view(N, nh, d), want) < ATT_TOL[dtype]


@pytest.mark.parametrize("nh,nkv", [(32, 8), (16, 1), (3, 3), (8, 4), (16, 2), (10, 2), (6, 2), (3, 1), (24, 1)])
@pytest.mark.parametrize("window", [0, 37, 150])
def test_attention_umma_prefill(ops, nh, nkv, window):
    """The tcgen05 prefill attention against the plain formula (head size 128; groups 4, 16, 1, 2, 8, and
    5, 3, 24, which do not divide a block's 128 rows)."""
    torch.manual_seed(25)
    d, dtype = 128, torch.bfloat16
    assert ops.attention_umma_supported(dtype, d, nh, nkv)
    lens = [300, 1, 77, 64, 130, 513]
    pasts = [0, 0, 50, 0, 127, 0]
    q_lens = [L - p for L, p in zip(lens, pasts)]
    ps = PagedSetup(lens, nkv, d, dtype, seed=25, key_scale=2.0)
    N = sum(q_lens)
    ld = nh * d + 2 * nkv * d
    q_all = torch.randn(N, ld, device=DEV).to(dtype)
    out = torch.zeros(N, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    st = _status()
    ops.attention_umma_prefill(q_all, out, len(lens), max(q_lens), nh, nkv, d, scale, window, qstart, past_t, ps.seq_slot,
                               ps.table, ps.num_pages, ps.k_pages, ps.v_pages, st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0, st.tolist()
    qs, o = [], 0
    for n in q_lens:
        qs.append(q_all[o:o + n, : nh * d].cpu().view(n, nh, d)); o += n
    want = _plain_attention(ps, qs, pasts, nh, scale, window or None)
    assert rel_err(out.float().cpu().view(N, nh, d), want) < ATT_TOL[dtype]


def test_attention_umma_prefill_blocks_of_two_pages_again_and_again(ops):
    """Blocks that see two or three pages only (a short window) end a few barrier phases after they
    start; a wait that names a phase by its parity must not pass because the barrier is two phases
    behind.  The same launch forty times must give the same, right result every time."""
    torch.manual_seed(27)
    nh, nkv, d, dtype, window = 8, 4, 128, torch.bfloat16, 37
    lens = [300, 77, 513, 130]
    ps = PagedSetup(lens, nkv, d, dtype, seed=27, key_scale=2.0)
    N = sum(lens)
    q_all = torch.randn(N, nh * d + 2 * nkv * d, device=DEV).to(dtype)
    qstart = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past_t = torch.zeros(len(lens), dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    st = _status()
    qs, o = [], 0
    for n in lens:
        qs.append(q_all[o:o + n, : nh * d].cpu().view(n, nh, d)); o += n
    want = _plain_attention(ps, qs, [0] * len(lens), nh, scale, window)
    outs = []
    for _ in range(40):
        out = torch.zeros(N, nh * d, device=DEV, dtype=dtype)
        ops.attention_umma_prefill(q_all, out, len(lens), max(lens), nh, nkv, d, scale, window, qstart, past_t, ps.seq_slot,
                                   ps.table, ps.num_pages, ps.k_pages, ps.v_pages, st)
        outs.append(out)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0
    for out in outs:
        assert torch.equal(out, outs[0])
    assert rel_err(outs[0].float().cpu().view(N, nh, d), want) < ATT_TOL[dtype]


def test_attention_umma_prefill_rescales_when_the_maximum_grows(ops):
    """Scores that grow by far more than 2^8 along the sequence: the reference of the exponentials
    must move and the accumulated output be rescaled."""
    nh, nkv, d, dtype = 4, 1, 128, torch.bfloat16
    L = 400
    ps = PagedSetup([L], nkv, d, dtype, seed=26, key_scale=0.1)
    probe = torch.randn(d)
    probe = probe / probe.norm()
    q_all = (probe * 6.0).repeat(L, nh).to(dtype).to(DEV)                 # every query points along `probe`
    for pos in range(L):                                                   # keys grow along `probe` with the position
        page = int(ps.table[ps.slots[0], pos // 64])
        ps.k_pages[page, 0, pos % 64] += (probe * (pos / 10.0)).to(dtype).to(DEV)
    ps.k[0] = torch.stack([ps.k_pages[int(ps.table[ps.slots[0], p // 64]), :, p % 64].cpu() for p in range(L)])
    out = torch.zeros(L, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    past_t = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    st = _status()
    ops.attention_umma_prefill(q_all, out, 1, L, nh, nkv, d, scale, 0, qstart, past_t, ps.seq_slot, ps.table,
                               ps.num_pages, ps.k_pages, ps.v_pages, st)
    assert st.tolist()[0] == 0
    want = _plain_attention(ps, [q_all.cpu().view(L, nh, d)], [0], nh, scale, None)
    assert rel_err(out.float().cpu().view(L, nh, d), want) < ATT_TOL[dtype]


@pytest.mark.parametrize("nh,nkv,d", MMA_SHAPES)
@pytest.mark.parametrize("window", [0, 300])
# split_keys 0: even shares of each length, of at least `least` keys (spare ranges of the grid do nothing)
@pytest.mark.parametrize("split_keys,max_splits,least", [(256, 5, 0), (0, 5, 0), (0, 1, 0), (0, 23, 0), (0, 23, 128), (0, 9, 512)])
def test_attention_mma_decode(ops, nh, nkv, d, window, split_keys, max_splits, least):
    torch.manual_seed(16)
    dtype = torch.bfloat16
    lens = [1, 700, 256, 257, 33, 64, 65, 513]
    pasts = [L - 1 for L in lens]
    ps = PagedSetup(lens, nkv, d, dtype, seed=16, key_scale=2.0)
    B = len(lens)
    ld = nh * d + 2 * nkv * d
    q_all = torch.randn(B, ld, device=DEV).to(dtype)
    out = torch.zeros(B, nh * d, device=DEV, dtype=dtype)
    qstart = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    past_t = torch.tensor(pasts, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)
    scratch = torch.full((ops.attention_generic_scratch_floats(B, nh, d, max_splits),), float("nan"), device=DEV)
    st = _status()
    ops.attention_mma(True, q_all, out, B, 1, nh, nkv, d, scale, window, qstart, past_t, ps.seq_slot, ps.table,
                      ps.num_pages, ps.k_pages, ps.v_pages, scratch, split_keys, max_splits, st, min_range_keys=least)
    assert st.tolist()[0] == 0
    qs = [q_all[b: b + 1, : nh * d].cpu().view(1, nh, d) for b in range(B)]
    want = _plain_attention(ps, qs, pasts, nh, scale, window or None)
    assert rel_err(out.float().cpu().view(B, nh, d), want) < ATT_TOL[dtype]


@pytest.mark.parametrize("decode", [False, True])
def test_attention_mma_finds_a_far_key_and_ignores_what_lies_beyond_the_length(ops, decode):
    nh, nkv, d = 8, 2, 128
    dtype = torch.bfloat16
    L, far = 650, 13
    ps = PagedSetup([L], nkv, d, dtype, seed=17, key_scale=0.05)
    probe = torch.randn(d)
    probe = probe / probe.norm() * 12.0
    q = probe.repeat(nh).view(1, nh * d)
    page = int(ps.table[ps.slots[0], far // 64])
    ps.k_pages[page, :, far % 64] = (probe * 2.0).to(DEV, dtype)
    # the row after the sequence's last key matches even better and must not be seen (the cache keeps
    # such rows finite, see the append kernel; a huge value shows any leak)
    last_page = int(ps.table[ps.slots[0], L // 64])
    ps.k_pages[last_page, :, L % 64] = (probe * 4.0).to(DEV, dtype)
    ps.v_pages[last_page, :, L % 64] = 1e30
    out = torch.zeros(1, nh * d, device=DEV, dtype=dtype)
    qstart = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    past_t = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    scratch = torch.zeros(ops.attention_generic_scratch_floats(1, nh, d, 3), device=DEV)
    ops.attention_mma(decode, q.to(DEV, dtype), out, 1, 1, nh, nkv, d, 1 / math.sqrt(d), 0, qstart, past_t, ps.seq_slot,
                      ps.table, ps.num_pages, ps.k_pages, ps.v_pages, scratch if decode else None,
                      256 if decode else 0, 3 if decode else 0, _status())
    v_far = ps.v_pages[page, :, far % 64].float().cpu()
    got = out.float().cpu().view(nh, d)
    for h in range(nh):
        assert torch.allclose(got[h], v_far[h // 4], atol=2e-2)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 64), (100, 80), (515, 200), (4096, 4096), (1000, 12288), (48, 8)])
def test_gemm_smallm(ops, M, N, K):
    torch.manual_seed(20)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.5).to(torch.bfloat16)
    want = x.float().cpu() @ w.float().cpu().T
    out32 = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_smallm(x, w, out32)
    assert rel_err(out32.cpu(), want) < 2e-5
    out16 = torch.zeros(M, N + 8, device=DEV, dtype=torch.bfloat16)[:, :N]      # a row stride larger than N
    ops.gemm_smallm(x, w, out16)
    assert rel_err(out16.float().cpu(), want) < KTOL[torch.bfloat16]
    # x as rows of a wider buffer
    wide = torch.randn(M, K + 24, device=DEV).to(torch.bfloat16)
    ops.gemm_smallm(wide[:, :K], w, out32)
    assert rel_err(out32.cpu(), wide[:, :K].float().cpu() @ w.float().cpu().T) < 2e-5


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(176, 80), (200, 96), (3072, 1024), (24, 4096)])
def test_gemm_smallm_with_the_gate_fused(ops, M, I, K):
    torch.manual_seed(21)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * (2.0 / K ** 0.5)).to(torch.bfloat16)
    gu = x.float().cpu() @ w.float().cpu().T
    g, u = gu[:, :I], gu[:, I:]
    want = g / (1 + torch.exp(-g)) * u
    out = torch.zeros(M, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_smallm(x, w, out, pair_offset=I)
    assert rel_err(out.float().cpu(), want) < KTOL[torch.bfloat16]
    out32 = torch.zeros(M, I, device=DEV)
    ops.gemm_smallm(x, w, out32, pair_offset=I)
    assert rel_err(out32.cpu(), want) < 2e-5


def test_gemm_smallm_refuses_what_it_does_not_take(pe, ops):
    x = torch.zeros(17, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(32, 64, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_smallm_supported(x, w)
    assert not ops.gemm_smallm_supported(x[:4, :60], w[:, :60].contiguous())
    with pytest.raises(pe.kernels.KernelError):
        ops.gemm_smallm(x, w, torch.zeros(17, 32, device=DEV))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 16, 8), (300, 515, 200), (2048, 1024, 512), (129, 257, 72),
                                   (640, 4096, 1024), (77, 1000, 4096)])
@pytest.mark.parametrize("kernel", ["gemm_umma", "gemm_umma2"])
def test_gemm_umma(ops, M, N, K, kernel):
    gemm = getattr(ops, kernel)    # one SM per 128 x 256 tile, or a pair of SMs per 256 x 256 tile
    if kernel == "gemm_umma2":
        K = -(-K // 64) * 64       # the pair kernel takes whole k blocks of 64
    torch.manual_seed(30)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.5).to(torch.bfloat16)
    want = x.float().cpu() @ w.float().cpu().T
    st = _status()
    out32 = torch.full((M, N), float("nan"), device=DEV)
    gemm(x, w, out32, st)
    assert st.tolist()[0] == 0
    assert rel_err(out32.cpu(), want) < 2e-5
    out16 = torch.zeros(M, N + 8, device=DEV, dtype=torch.bfloat16)[:, :N]
    gemm(x, w, out16, st)
    assert rel_err(out16.float().cpu(), want) < KTOL[torch.bfloat16]
    wide = torch.randn(M, K + 24, device=DEV).to(torch.bfloat16)
    gemm(wide[:, :K], w, out32, st)
    assert rel_err(out32.cpu(), wide[:, :K].float().cpu() @ w.float().cpu().T) < 2e-5
    assert st.tolist()[0] == 0


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (200, 384, 200), (1000, 1280, 1024), (5, 256, 4096)])
@pytest.mark.parametrize("kernel", ["gemm_umma", "gemm_umma2"])
def test_gemm_umma_with_the_gate_fused(ops, M, I, K, kernel):
    if kernel == "gemm_umma2":
        K = -(-K // 64) * 64
    torch.manual_seed(31)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * (2.0 / K ** 0.5)).to(torch.bfloat16)
    gu = x.float().cpu() @ w.float().cpu().T
    g, u = gu[:, :I], gu[:, I:]
    want = g / (1 + torch.exp(-g)) * u
    out = torch.zeros(M, I, device=DEV, dtype=torch.bfloat16)
    st = _status()
    getattr(ops, kernel)(x, w, out, st, pair_offset=I)
    assert st.tolist()[0] == 0
    assert rel_err(out.float().cpu(), want) < KTOL[torch.bfloat16]


@pytest.mark.parametrize("M,N,K,fused", [(2048, 4096, 12288, False), (1536, 6144, 4096, False), (1024, 4096, 4096, False),
                                         (2048, 12288, 4096, True)])
@pytest.mark.parametrize("kernel", ["gemm_umma", "gemm_umma2"])
def test_gemm_umma_at_the_layer_shapes_of_an_8b_model(ops, M, N, K, fused, kernel):
    """The products of a 2,048-token prompt at width 4,096 / 12,288 (K = 12,288 is 192 k blocks: the 3- and 4-stage
    rings turn over dozens of times).  Every output against the library's true float32 product on the device, and
    a sample of rows against a float64 product on the CPU."""
    torch.manual_seed(33)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    rows_w = 2 * N if fused else N
    w = (torch.randn(rows_w, K, device=DEV) * (2.0 / K ** 0.5)).to(torch.bfloat16)
    st = _status()
    out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16 if fused else torch.float32)
    getattr(ops, kernel)(x, w, out, st, **({"pair_offset": N} if fused else {}))
    assert st.tolist()[0] == 0

    def finish(prod):
        if not fused:
            return prod
        g, u = prod[:, :N], prod[:, N:]
        return g / (1 + torch.exp(-g)) * u

    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        want = finish(torch.mm(x.float(), w.float().t()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    tol = KTOL[torch.bfloat16] if fused else 2e-5
    assert rel_err(out.float().cpu(), want.cpu()) < tol
    pick = torch.randperm(M)[:48].sort().values
    exact = finish(x[pick].double().cpu() @ w.double().cpu().T)
    assert rel_err(out[pick].double().cpu(), exact) < tol


@pytest.mark.parametrize("nh,nkv,K,norm,rotate", [(8, 2, 256, True, True), (3, 1, 320, True, True), (6, 3, 192, False, True),
                                                  (4, 4, 128, True, False)])
def test_qkv_product_with_norm_rotation_and_append_in_its_epilogue(ops, nh, nkv, K, norm, rotate):
    """The q|k|v product with q/k-norm, rotation and cache append in its epilogue against the three kernels it
    stands for (product, then norm + rotation + append): three sequences, one of which starts in this step and one
    ends in the middle of a page; 3 and 5 heads' worth of columns do not fill the last 256-column tile.  Queries as
    the separate kernels leave them, the cache's pages bit for bit except the rounding of the norm's sum."""
    torch.manual_seed(41)
    d, dtype = 128, torch.bfloat16
    lens, q_lens = [300, 130, 200], [230, 130, 136]
    N = sum(q_lens)
    x = torch.randn(N, K, device=DEV).to(dtype)
    w = (torch.randn((nh + 2 * nkv) * d, K, device=DEV) * (1.5 / K ** 0.5)).to(dtype)
    qw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    kw = (1 + 0.2 * torch.randn(d, device=DEV)) if norm else None
    eps, theta, max_pos = 1e-5, 1e4, 512
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), plain.rope_inv_freq(d, theta))
    cos, sin = (torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)) if rotate else (None, None)
    token_seq = torch.tensor(sum(([b] * n for b, n in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
    pos_list = sum(([lens[b] - q_lens[b] + i for i in range(q_lens[b])] for b in range(3)), [])
    token_pos = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0, q_lens[0], q_lens[0] + q_lens[1], N], dtype=torch.int32, device=DEV)
    assert ops.gemm_umma2_qkv_rope_supported(x, w, nh, nkv, d, d if rotate else 0)
    results = []
    for fused in (False, True):
        ps = PagedSetup(lens, nkv, d, dtype, seed=41)
        ld = (nh + 2 * nkv) * d
        qkv = torch.zeros(N, ld, device=DEV, dtype=dtype)
        st = _status()
        if fused:
            ops.gemm_umma2_qkv_rope(x, w, qkv, nh, nkv, d, qw, kw, eps, cos, sin, d if rotate else 0, token_seq, token_pos,
                                    ps.seq_slot, qstart, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, True, st)
        else:
            ops.gemm_umma2(x, w, qkv, st)
            ops.qk_norm_rope_append(qkv, N, nh, nkv, d, qw, kw, eps, cos, sin, d if rotate else 0, token_seq, token_pos,
                                    ps.seq_slot, qstart, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, True, st)
        assert st.tolist()[0] == 0
        results.append((qkv[:, : nh * d].float().cpu(), ps.k_pages.float().cpu(), ps.v_pages.float().cpu()))
    (q0, k0, v0), (q1, k1, v1) = results
    assert rel_err(q1, q0) < 4e-3 and rel_err(k1, k0) < 4e-3         # one bfloat16 step where the norm's sum rounds differently
    assert (q1 != q0).float().mean() < 0.02 and (k1 != k0).float().mean() < 0.02
    assert torch.equal(v1, v0)                                        # values are copied: bit for bit, cleared rows included
    # and against the plain formulas
    prod = x.float().cpu() @ w.float().cpu().T
    prod = prod.to(dtype).float()
    q_in = prod[:, : nh * d].view(N, nh, d)
    want = plain.rms_norm(q_in, qw.cpu(), eps) if norm else q_in
    if rotate:
        c, s_ = plain.rope_cos_sin(torch.tensor(pos_list), d, theta)
        want = plain.rope_rotate_neox(want, c, s_, d)
    assert rel_err(q1.view(N, nh, d), want) < KTOL[dtype]
    # a layer that only reads a cache: nothing is appended
    ps = PagedSetup(lens, nkv, d, dtype, seed=41)
    k_before = ps.k_pages.clone()
    qkv = torch.zeros(N, (nh + 2 * nkv) * d, device=DEV, dtype=dtype)
    ops.gemm_umma2_qkv_rope(x, w, qkv, nh, nkv, d, qw, kw, eps, cos, sin, d if rotate else 0, token_seq, token_pos,
                            ps.seq_slot, qstart, ps.table, ps.num_pages, ps.k_pages, ps.v_pages, False, _status())
    assert torch.equal(ps.k_pages, k_before) and torch.equal(qkv[:, : nh * d].float().cpu(), q1)


def test_sampler_greedy_and_ties(ops):
    torch.manual_seed(8)
    logits = torch.randn(6, 1000, device=DEV)
    logits[2, 17] = logits[2, 900] = 50.0                     # a tie: the lower index wins
    logits[3, 999] = 60.0
    req = torch.arange(6, dtype=torch.int32, device=DEV)
    step = torch.zeros(6, dtype=torch.int32, device=DEV)
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample(logits, 0.0, 0, 1.0, 0.0, 1, req, step, out)
    want = logits.argmax(-1).tolist()
    want[2] = 17
    assert out.tolist() == want


@pytest.mark.parametrize("filters", [dict(), dict(top_k=5), dict(top_k=40, top_p=0.9, min_p=0.05), dict(top_p=0.6),
                                     dict(min_p=0.2), dict(top_k=1500)])
def test_sampler_matches_the_plain_draw(ops, filters):
    torch.manual_seed(9)
    V, rows = 2000, 24
    logits = torch.randn(rows, V, device=DEV) * 2.5
    req = torch.arange(rows, dtype=torch.int32, device=DEV) % 5
    step = torch.arange(rows, dtype=torch.int32, device=DEV) // 5
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    kw = dict(top_k=0, top_p=1.0, min_p=0.0)
    kw.update(filters)
    ops.sample(logits, 0.8, kw["top_k"], kw["top_p"], kw["min_p"], 1234, req, step, out)
    got = out.tolist()
    agree = 0
    for r in range(rows):
        want = plain.sample_token(logits[r].cpu(), seed=1234, request=int(req[r]), step=int(step[r]), temperature=0.8, **kw)
        _, probs = plain.filter_logits(logits[r].cpu(), temperature=0.8, **kw)
        assert probs[got[r]] > 0, "the kernel drew a token that the filters exclude"
        agree += got[r] == want
    assert agree >= rows - 1     # float32 vs float64 Gumbel arithmetic may flip one near-tie


@pytest.mark.parametrize("V", [4097, 10000, 151936])
def test_sampler_with_scratch_greedy(ops, V):
    """Rows cut into chunks by a first kernel: the same argmax, ties to the lower index, across chunk borders."""
    torch.manual_seed(11)
    rows = 5
    logits = torch.randn(rows, V, device=DEV)
    logits[1, 4095] = logits[1, 4096] = 40.0                  # a tie across the first chunk border
    logits[2, V - 1] = 41.0                                   # the last entry of the last (short) chunk
    logits[3, 0] = 42.0
    logits[4, 5000 % V] = float("nan")                        # NaN never wins
    req = torch.arange(rows, dtype=torch.int32, device=DEV)
    step = torch.zeros(rows, dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    need = ops.sample_scratch_bytes(rows, V, 0.0, 0)
    assert need > 0
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
    ops.sample(logits, 0.0, 0, 1.0, 0.0, 1, req, step, out, scratch=scratch)
    want = torch.nan_to_num(logits, nan=-float("inf")).argmax(-1).tolist()
    want[1] = 4095
    assert out.tolist() == want


@pytest.mark.parametrize("filters", [dict(top_k=5), dict(top_k=40, top_p=0.9, min_p=0.05), dict(top_k=40, top_p=0.95, min_p=0.05),
                                     dict(top_k=64, top_p=0.5), dict(top_k=1)])
def test_sampler_with_scratch_matches_the_plain_draw_and_the_single_kernel(ops, filters):
    torch.manual_seed(12)
    V, rows = 20011, 16
    logits = torch.randn(rows, V, device=DEV) * 2.5
    logits[3, 100:140] = 9.0                                  # forty ties at the top of one chunk
    logits[5, :] = 0.25                                       # every entry ties: the chunks overflow, the row is read whole
    req = torch.arange(rows, dtype=torch.int32, device=DEV) % 5
    step = torch.arange(rows, dtype=torch.int32, device=DEV) // 5
    kw = dict(top_k=0, top_p=1.0, min_p=0.0)
    kw.update(filters)
    need = ops.sample_scratch_bytes(rows, V, 0.8, kw["top_k"], kw["top_p"], kw["min_p"])
    assert need > 0
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    single = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, 0.8, kw["top_k"], kw["top_p"], kw["min_p"], 99, req, step, out, scratch=scratch)
    ops.sample(logits, 0.8, kw["top_k"], kw["top_p"], kw["min_p"], 99, req, step, single)
    got = out.tolist()
    assert sum(a != b for a, b in zip(got, single.tolist())) <= 1
    agree = 0
    for r in range(rows):
        want = plain.sample_token(logits[r].cpu(), seed=99, request=int(req[r]), step=int(step[r]), temperature=0.8, **kw)
        _, probs = plain.filter_logits(logits[r].cpu(), temperature=0.8, **kw)
        if r != 5:    # with every entry tied, which k of them a top-k keeps is not defined
            assert probs[got[r]] > 0, "the kernel drew a token that the filters exclude"
            agree += got[r] == want
    assert agree >= rows - 2
    assert ops.sample_scratch_bytes(rows, V, 0.8, 0, 0.9) == 0 and ops.sample_scratch_bytes(rows, 3000, 0.8, 40) == 0


def test_sampler_with_scratch_unfiltered_draw_is_the_single_kernels(ops):
    torch.manual_seed(13)
    rows, V = 12, 30000
    logits = torch.randn(rows, V, device=DEV) * 2
    req = torch.arange(rows, dtype=torch.int32, device=DEV)
    step = torch.full((rows,), 3, dtype=torch.int32, device=DEV)
    a, b = (torch.empty(rows, dtype=torch.int32, device=DEV) for _ in range(2))
    scratch = torch.empty(ops.sample_scratch_bytes(rows, V, 0.9, 0), dtype=torch.uint8, device=DEV)
    assert scratch.numel() > 0
    ops.sample(logits, 0.9, 0, 1.0, 0.0, 5, req, step, a, scratch=scratch)
    ops.sample(logits, 0.9, 0, 1.0, 0.0, 5, req, step, b)
    assert a.tolist() == b.tolist()


def test_sampler_is_keyed_by_request_and_step_not_by_row(ops):
    torch.manual_seed(10)
    row = torch.randn(1, 3000, device=DEV)
    logits = row.repeat(4, 1)
    req = torch.tensor([3, 3, 4, 3], dtype=torch.int32, device=DEV)
    step = torch.tensor([0, 1, 0, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample(logits, 1.0, 0, 1.0, 0.0, 77, req, step, out)
    a = out.tolist()
    assert a[0] == a[3] and len({a[0], a[1], a[2]}) >= 2
    ops.sample(logits, 1.0, 0, 1.0, 0.0, 78, req, step, out)
    assert out.tolist() != a


def test_repetition_penalty(ops):
    logits = torch.tensor([[2.0, -1.0, 0.5, 3.0], [1.0, 1.0, 1.0, 1.0]], device=DEV)
    recent = torch.tensor([[3, 1, 3, 0], [2, 0, 0, 0]], dtype=torch.int32, device=DEV)
    count = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    ops.repetition_penalty(logits, recent, count, 2.0)
    assert logits.tolist() == [[2.0, -2.0, 0.5, 1.5], [1.0, 1.0, 0.5, 1.0]]


def test_unsupported_sizes_are_refused(pe, ops):
    q = torch.zeros(1, 1024, device=DEV)
    with pytest.raises(pe.kernels.KernelError, match="size"):
        ops.attention_generic(False, q, q.clone(), 1, 1, 1, 1, 1024, 1.0, 0, torch.zeros(2, dtype=torch.int32, device=DEV),
                              torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                              torch.zeros(1, 1, dtype=torch.int32, device=DEV), 1, q, q, None, 0, 0, _status())
    with pytest.raises(pe.kernels.KernelError):
        ops.embed_gather(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4), torch.zeros(4, dtype=torch.int32))


def test_a_bounded_wait_gives_up_within_seconds(ops):
    """Every wait inside a kernel polls an mbarrier a limited number of times.  A poll that finds the phase incomplete
    takes microseconds (the hardware parks the thread for a while), so the limit in polls is a limit in time: the
    probe kernel polls a barrier on which nothing arrives, a counted number of times, and ends by itself."""
    poll = ops.wait_poll_seconds(DEV, polls=20000)
    assert 1e-7 < poll < 2e-5, f"one failing poll took {poll * 1e6:.2f} us"
    limit = ops.wait_limit_seconds(DEV)
    assert 0.5 < limit < 10.0, f"a wait that nothing ends would last {limit:.1f} s"
