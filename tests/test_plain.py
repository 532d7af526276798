"""The plain implementation checks itself: each part against a second, independent formulation."""
import math

import pytest
import torch

import plain_qwen3 as plain
from conftest import TEST_CONFIGS


def test_rms_norm():
    x = torch.randn(5, 12)
    w = torch.randn(12)
    got = plain.rms_norm(x, w, 1e-5)
    want = torch.stack([r / math.sqrt(float((r * r).sum()) / 12 + 1e-5) * w for r in x])
    assert torch.allclose(got, want, atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    d, theta = 8, 100.0
    q, k = torch.randn(1, 1, d), torch.randn(1, 1, d)
    def at(x, p):
        c, s = plain.rope_cos_sin(torch.tensor([p]), d, theta)
        return plain.rope_rotate_neox(x, c, s, d)[0, 0]
    assert torch.allclose(at(q, 7).norm(), q.norm(), atol=1e-5)
    # the score depends on the distance only
    a = at(q, 9) @ at(k, 4)
    b = at(q, 25) @ at(k, 20)
    assert abs(float(a - b)) < 1e-4
    assert torch.allclose(at(q, 0), q[0, 0])
    # partial rotation leaves the tail alone
    c, s = plain.rope_cos_sin(torch.tensor([3]), 4, theta)
    out = plain.rope_rotate_neox(q, c, s, 4)
    assert torch.equal(out[..., 4:], q[..., 4:])


def test_attention_masks():
    torch.manual_seed(0)
    S, nh, nkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(S, nh, d), torch.randn(S, nkv, d), torch.randn(S, nkv, d)
    out = plain.causal_gqa_attention(q, k, v, 0.3)
    # row 0 sees key 0 only
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    # changing a future key changes nothing before it
    k2, v2 = k.clone(), v.clone()
    k2[6:], v2[6:] = 5.0, -3.0
    out2 = plain.causal_gqa_attention(q, k2, v2, 0.3)
    assert torch.allclose(out[:6], out2[:6]) and not torch.allclose(out[6:], out2[6:])
    # a window of 1 sees the own position only
    w1 = plain.causal_gqa_attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0], atol=1e-6) and torch.allclose(w1[:, 3], v[:, 1], atol=1e-6)
    # a window as long as the sequence is no window
    assert torch.allclose(plain.causal_gqa_attention(q, k, v, 0.3, window=S), out)
    # second formulation: explicit loop
    h, i = 2, 5
    sc = torch.tensor([float(q[i, h] @ k[j, 1]) * 0.3 for j in range(i + 1)])
    p = torch.softmax(sc, 0)
    assert torch.allclose(out[i, h], (p[:, None] * v[: i + 1, 1]).sum(0), atol=1e-5)


def test_swiglu():
    x, g, u, dn = torch.randn(3, 6), torch.randn(10, 6), torch.randn(10, 6), torch.randn(6, 10)
    want = (torch.nn.functional.silu(x @ g.T) * (x @ u.T)) @ dn.T
    assert torch.allclose(plain.swiglu(x, g, u, dn), want, atol=1e-5)


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_whole_model_is_causal_and_uses_its_options(pe, tmp_path, key):
    cfg = pe.Qwen3Config.from_dict(TEST_CONFIGS[key])
    pe.write_random_model(str(tmp_path), cfg, 1)
    c, w = plain.load_folder(str(tmp_path))
    toks = torch.randint(0, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(0)).tolist()
    full = plain.forward_logits(c, w, toks)
    assert full.shape == (150, cfg.vocab_size)
    part = plain.forward_logits(c, w, toks[:60])
    assert torch.allclose(full[:60], part, atol=1e-5)     # causal
    if cfg.use_sliding_window:                                # the window really is in use
        c2 = dict(c, use_sliding_window=False)
        assert not torch.allclose(plain.forward_logits(c2, w, toks)[-1], full[-1], atol=1e-4)
    c3 = dict(c, rms_norm_eps=1e-2)
    assert not torch.allclose(plain.forward_logits(c3, w, toks[:20]), full[:20], atol=1e-5)


def test_filters_and_uniforms():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    _, p = plain.filter_logits(logits, temperature=1.0, top_k=2)
    assert p.nonzero().flatten().tolist() == [0, 4] and abs(float(p.sum()) - 1) < 1e-6
    _, p = plain.filter_logits(logits, temperature=1.0, min_p=0.3)
    assert p.nonzero().flatten().tolist() == [0, 4]          # e^-1 = .37 of the max stays, e^-2 = .14 goes
    _, p = plain.filter_logits(logits, temperature=1.0, top_p=0.5)
    assert p.nonzero().flatten().tolist() == [4]             # p(4) = .61 > .5: the next entry's preceding mass exceeds
    _, p = plain.filter_logits(logits, temperature=1.0, top_p=0.7)
    assert p.nonzero().flatten().tolist() == [0, 4]
    pen, _ = plain.filter_logits(logits, temperature=0.0, repetition_penalty=2.0, recent_tokens=[3, 4, 4])
    assert pen.tolist() == [2.0, 1.0, 0.5, -2.0, 1.5]
    us = [plain.uniform_for(1, 2, 3, i) for i in range(2000)]
    assert 0 < min(us) and max(us) < 1 and abs(sum(us) / 2000 - 0.5) < 0.03
    assert plain.uniform_for(1, 2, 3, 4) != plain.uniform_for(1, 2, 4, 4) != plain.uniform_for(1, 3, 3, 4)
    # the draw follows the filtered distribution
    counts = [0] * 5
    for step in range(3000):
        counts[plain.sample_token(logits, seed=9, request=0, step=step, temperature=1.0, top_k=3)] += 1
    _, p = plain.filter_logits(logits, temperature=1.0, top_k=3)
    for i in range(5):
        assert abs(counts[i] / 3000 - float(p[i])) < 0.03
