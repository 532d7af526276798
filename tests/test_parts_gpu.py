"""Each part alone against its plain formula, and toy architectures whose parts are defined here (a
mixer that keeps state of its own, a feed-forward with routing, another position encoding, another
block arrangement, another norm):
registered, built and stepped from the test, with no change to the package's files."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PTOL = {torch.float32: 1e-5, torch.bfloat16: 1.5e-2}


def _ctx(pe, rt, cache, slots, tokens_per_seq, want=()):
    """A step context for sequences that bring ``tokens_per_seq`` tokens each (all tokens zero)."""
    entries = [pe.StepEntry(s, [0] * n, ()) for s, n in zip(slots, tokens_per_seq)]
    pasts = [cache.length(s) for s in slots]
    for s, p, n in zip(slots, pasts, tokens_per_seq):
        cache.reserve(s, p + n)
    ints, n_tokens, n_want = pe.engine.StepContext.pack_meta(entries, pasts)
    pool = pe.engine.BufferPool(DEV)
    ctx = pe.engine.StepContext(rt, pool, n_tokens=n_tokens, n_seqs=len(slots), max_q=max(tokens_per_seq),
                                decode=all(n == 1 for n in tokens_per_seq),
                                max_kv_len=max(p + n for p, n in zip(pasts, tokens_per_seq)), n_want=0)
    ctx.meta.copy_(torch.tensor(ints, dtype=torch.int32))
    pe.kernels.ops.batch_expand(ctx.seq_qstart, ctx.seq_past, len(slots), ctx.token_seq, ctx.token_pos)
    return ctx, pasts


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(pe, dtype):
    rt = pe.parts.Runtime(DEV, dtype)
    w = (1 + 0.1 * torch.randn(200)).to(torch.bfloat16)
    norm = pe.parts.lookup("norm", "rmsnorm")({"dim": 200, "eps": 2e-5}, {"weight": w}, rt)
    assert norm.weight.dtype == torch.float32
    stream = torch.randn(9, 200, device=DEV)
    delta = torch.randn(9, 200, device=DEV).to(dtype)
    out = torch.empty(9, 200, device=DEV, dtype=dtype)
    before = stream.clone()
    norm.add_forward(stream, delta, out)
    assert torch.equal(stream, before + delta.float())
    assert rel_err(out.float().cpu(), plain.rms_norm(stream.cpu(), w.float(), 2e-5)) < PTOL[dtype]


def test_rope_part_tables(pe):
    rt = pe.parts.Runtime(DEV, torch.float32)
    rope = pe.parts.lookup("position", "rope")({"rotary_dim": 48, "theta": 5e5, "max_positions": 700}, {}, rt)
    cos, sin, rot = rope.tables()
    c, s = plain.rope_cos_sin(torch.arange(700), 48, 5e5)
    assert rot == 48 and cos.shape == (700, 24)
    assert float((cos.cpu() - c).abs().max()) < 1e-6 and float((sin.cpu() - s).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 50])
def test_attention_part_prefill_then_decode(pe, dtype, window):
    """The attention part alone over a small cache: two sequences, a prompt each, then single tokens."""
    torch.manual_seed(0)
    H, nh, nkv, d = 72, 6, 3, 24
    rt = pe.parts.Runtime(DEV, dtype)
    wts = {"q_proj": torch.randn(nh * d, H) * 0.2, "k_proj": torch.randn(nkv * d, H) * 0.2,
           "v_proj": torch.randn(nkv * d, H) * 0.2, "o_proj": torch.randn(H, nh * d) * 0.2,
           "q_norm": 3 + torch.randn(d) * 0.1, "k_norm": 1 + torch.randn(d) * 0.1}
    wts = {k: v.to(torch.bfloat16) for k, v in wts.items()}
    rope = pe.parts.lookup("position", "rope")({"rotary_dim": d, "theta": 1e4, "max_positions": 256}, {}, rt)
    params = {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "qk_norm": True, "eps": 1e-6,
              "scale": None, "window": window, "position": "rope"}
    cls = pe.parts.lookup("mixer", "attention")
    att = cls(params, wts, rt, positions={"rope": rope})
    cache = pe.cache.PagedCache({0: cls.cache_request(params)}, max_tokens=512, max_slots=4, max_seq_len=256,
                                dtype=dtype, device=DEV)
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    lens = [90, 7]
    xs = [torch.randn(L + 5, H).to(torch.bfloat16) for L in lens]       # inputs: prompt plus five more tokens
    got = [[], []]
    ctx, pasts = _ctx(pe, rt, cache, slots, lens)
    x = torch.cat([xs[0][:90], xs[1][:7]]).to(DEV, dtype)
    y = att.forward(x, ctx, cache.view(0)).float().cpu()
    got[0].append(y[:90]); got[1].append(y[90:])
    for s, L in zip(slots, lens):
        cache.commit(s, L)
    for k in range(5):
        ctx, pasts = _ctx(pe, rt, cache, slots, [1, 1])
        x = torch.stack([xs[0][90 + k], xs[1][7 + k]]).to(DEV, dtype)
        y = att.forward(x, ctx, cache.view(0)).float().cpu()
        got[0].append(y[0:1]); got[1].append(y[1:2])
        for s in slots:
            cache.commit(s, cache.length(s) + 1)
    assert rt.status.tolist()[0] == 0
    w = {f"p.self_attn.{k}.weight": v for k, v in wts.items()}
    for b in range(2):
        want = plain.attention_layer(xs[b].float(), w, "p", n_heads=nh, n_kv_heads=nkv, head_dim=d, eps=1e-6,
                                     theta=1e4, window=window)
        assert rel_err(torch.cat(got[b]), want) < PTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_embedding_and_head_parts(pe, dtype):
    torch.manual_seed(1)
    rt = pe.parts.Runtime(DEV, dtype)
    H, I, V = 80, 176, 515
    wts = {"gate_proj": torch.randn(I, H) * 0.2, "up_proj": torch.randn(I, H) * 0.2, "down_proj": torch.randn(H, I) * 0.2}
    wts = {k: v.to(torch.bfloat16) for k, v in wts.items()}
    ffn = pe.parts.lookup("feed_forward", "swiglu")({"hidden": H, "intermediate": I}, wts, rt)
    x = torch.randn(11, H).to(torch.bfloat16)

    class Ctx:
        pool = pe.engine.BufferPool(DEV)
        def buffer(self, name, shape, dt):
            return self.pool.get(name, shape, dt)

    y = ffn.forward(x.to(DEV, dtype), Ctx()).float().cpu()
    want = plain.swiglu(x.float(), wts["gate_proj"], wts["up_proj"], wts["down_proj"])
    assert rel_err(y, want) < PTOL[dtype]
    table = (torch.randn(V, H) * 0.5).to(torch.bfloat16)
    emb = pe.parts.lookup("embedding", "token_embedding")({"vocab": V, "hidden": H}, {"weight": table}, rt)
    head = pe.parts.lookup("head", "linear_head")({"vocab": V, "hidden": H}, {"weight": table}, rt)
    assert head.weight.data_ptr() == emb.weight.data_ptr()        # a tied head shares the table
    ids = torch.tensor([0, 514, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, H, device=DEV)
    emb.forward(ids, out)
    assert torch.equal(out.cpu(), table.float()[[0, 514, 3]])
    logits = head.forward(x[:4].to(DEV, dtype))
    assert logits.dtype == torch.float32
    assert rel_err(logits.cpu(), x[:4].float() @ table.float().T) < PTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement_alone(pe, dtype):
    """The pre-norm arrangement around real parts: one block of test configuration B, a whole prompt,
    against the plain block.  The block hands its last delta on instead of adding it."""
    from conftest import TEST_CONFIGS
    cfg = pe.Qwen3Config.from_dict(dict(TEST_CONFIGS["B"], use_sliding_window=False))
    plan = pe.config.architecture(cfg.architecture).plan(cfg)
    w = pe.weights.random_weights(plan, 5, device="cpu")
    rt = pe.parts.Runtime(DEV, dtype)
    spec = plan.blocks[1]
    lookup = pe.parts.lookup
    pick = lambda part: {k: w[v] for k, v in part.weights.items()}
    rope = lookup("position", "rope")(plan.positions["rope"].params, {}, rt)
    parts = {}
    for name, (role, part) in spec.parts.items():
        extra = {"positions": {"rope": rope}} if role == "mixer" else {}
        parts[name] = lookup(role, part.kind)(part.params, pick(part), rt, **extra)
    block = lookup("arrangement", spec.arrangement)(spec, parts, rt)
    cache = pe.cache.PagedCache({1: lookup("mixer", "attention").cache_request(spec.part("mixer").params)}, max_tokens=256,
                                max_slots=2, max_seq_len=256, dtype=dtype, device=DEV)
    slot = cache.alloc_slot()
    S = 70
    ctx, _ = _ctx(pe, rt, cache, [slot], [S])
    x = torch.randn(S, cfg.hidden_size)
    prev = (torch.randn(S, cfg.hidden_size) * 0.1).to(torch.bfloat16)             # the delta of a block before
    stream = x.to(DEV).clone()
    pending = block.forward(stream, prev.to(DEV, dtype), ctx, cache.view(1))
    got = (stream + pending.float()).cpu()
    want = plain.decoder_block(x + prev.float(), {k: v.float() for k, v in w.items()}, 1, cfg.to_dict(), None,
                               torch.bfloat16 if dtype == torch.bfloat16 else None)
    assert rt.status.tolist()[0] == 0
    assert rel_err(got, want) < PTOL[dtype]


# ---- a toy architecture with a mixer that keeps fixed-size state -------------------------------------
@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int
    vocab_size: int
    layers: int
    decay: float
    max_position_embeddings: int = 256
    architecture: str = "ToyRunningMeanLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden_size"], d["vocab_size"], d["layers"], d["decay"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "layers": self.layers, "decay": self.decay}

    max_positions = property(lambda self: self.max_position_embeddings)
    stop_token_ids = ()
    bos_token = 0


class DecayingSumMixer:
    """state <- decay * state + W x_t ; output_t = state (per sequence, in token order).  The state
    is fixed-size per sequence and lives in the cache's state group."""

    @classmethod
    def weight_decls(cls, params):
        from importlib import import_module
        WeightDecl = import_module("pytorch-engine_b200").parts.WeightDecl
        return {"proj": WeightDecl((params["hidden"], params["hidden"]))}

    @classmethod
    def cache_request(cls, params):
        from importlib import import_module
        CR = import_module("pytorch-engine_b200").parts.CacheRequest
        return CR("state", state_shapes=(("acc", (params["hidden"],), "float32"),))

    def __init__(self, params, weights, runtime):
        self.rt, self.decay = runtime, float(params["decay"])
        self.proj = runtime.adopt(weights["proj"])

    def forward(self, x, ctx, view):
        z = self.rt.linear(x, self.proj).float()
        state = view.state("acc")
        out = torch.empty_like(z)
        qs = ctx.seq_qstart.tolist()
        for b, slot in enumerate(ctx.seq_slot.tolist()):
            acc = state[slot]
            for t in range(qs[b], qs[b + 1]):
                acc = self.decay * acc + z[t]
                out[t] = acc
            state[slot] = acc
        return out.to(x.dtype)


def test_toy_mixer_with_state_of_its_own(pe):
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep

    def plan(cfg):
        h = cfg.hidden_size
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": 1e-6}, {"weight": n})
        blocks = tuple(B.standard("pre_norm", norm(f"l{i}.n1"), P("decaying_sum", {"hidden": h, "decay": cfg.decay}, {"proj": f"l{i}.proj"}),
                         norm(f"l{i}.n2"), P("swiglu", {"hidden": h, "intermediate": 2 * h},
                                             {"gate_proj": f"l{i}.g", "up_proj": f"l{i}.u", "down_proj": f"l{i}.d"}),
                         name=f"toy {i}") for i in range(cfg.layers))
        return pe.parts.ModelPlan(hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                                  embedding=P("token_embedding", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "emb"}),
                                  blocks=blocks, order=tuple(R(i) for i in range(cfg.layers)), final_norm=norm("fn"),
                                  head=P("linear_head", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "emb"}))

    pe.parts.register("mixer", "decaying_sum", DecayingSumMixer, replace=True)
    pe.register_architecture("ToyRunningMeanLM", ToyConfig, plan, replace=True)
    try:
        cfg = ToyConfig(hidden_size=48, vocab_size=97, layers=2, decay=0.75)
        eng = pe.Engine.from_random(cfg, seed=4, dtype="float32", max_cache_tokens=256, max_batch=4)
        assert [g.request.kind for g in eng.cache.groups] == ["state"]
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 4, device=DEV).items()}

        def plain_toy(tokens):
            x = w["emb"][tokens]
            for i in range(2):
                n = plain.rms_norm(x, w[f"l{i}.n1"], 1e-6)
                z = n @ w[f"l{i}.proj"].T
                acc, rows = torch.zeros(48), []
                for t in range(len(tokens)):
                    acc = 0.75 * acc + z[t]
                    rows.append(acc)
                x = x + torch.stack(rows)
                x = x + plain.swiglu(plain.rms_norm(x, w[f"l{i}.n2"], 1e-6), w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
            return plain.rms_norm(x, w["fn"], 1e-6) @ w["emb"].T

        seqs = [[5, 9, 2, 77, 31, 8, 8, 40], [96, 0, 3, 3, 14]]
        for rnd in range(2):                                        # second round: the slots' state must start at zero
            slots = [eng.alloc_slot(), eng.alloc_slot()]
            got = [[], []]
            lg = eng.step([pe.StepEntry(slots[0], seqs[0][:5], (0, 4)), pe.StepEntry(slots[1], seqs[1][:2], (1,))])
            got[0] += [lg[0].cpu(), lg[1].cpu()]; got[1].append(lg[2].cpu())
            for k in range(3):
                lg = eng.step([pe.StepEntry(slots[0], [seqs[0][5 + k]], (0,)), pe.StepEntry(slots[1], [seqs[1][2 + k]], (0,))])
                got[0].append(lg[0].cpu()); got[1].append(lg[1].cpu())
            for s in slots:
                eng.free_slot(s)
            ref0, ref1 = plain_toy(seqs[0]), plain_toy(seqs[1])
            assert rel_err(torch.stack(got[0]), ref0[[0, 4, 5, 6, 7]]) < 1e-5
            assert rel_err(torch.stack(got[1]), ref1[[1, 2, 3, 4]]) < 1e-5
        res = eng.generate([seqs[0][:3]], pe.SamplingParams.greedy_params(max_tokens=4))
        assert res[0].completion_tokens == 4
    finally:
        pe.parts.unregister("mixer", "decaying_sum")
        pe.config.unregister_architecture("ToyRunningMeanLM")


def test_order_is_data_a_block_twice_and_a_shared_cache(pe):
    """The plan's order may name a block twice (with a cache entry of its own for the second run) and
    let a block read another block's keys and values without writing."""
    from conftest import TEST_CONFIGS
    cfg = pe.Qwen3Config.from_dict(dict(TEST_CONFIGS["A"], tie_word_embeddings=True))
    base = pe.config.architecture("Qwen3ForCausalLM").plan(cfg)
    R = pe.parts.RunStep
    import dataclasses
    plan = dataclasses.replace(base, order=(R(0), R(1), R(0, cache=2), R(1, cache=1, writes_cache=False)))

    def planner(_cfg):
        return plan

    @dataclass(frozen=True)
    class LoopCfg(pe.Qwen3Config):
        pass

    pe.register_architecture("LoopedQwen3", pe.Qwen3Config, planner, replace=True)
    try:
        cfg2 = dataclasses.replace(cfg, architecture="LoopedQwen3")
        eng = pe.Engine.from_random(cfg2, seed=9, dtype="float32", max_cache_tokens=256, max_batch=2)
        assert sorted(eng.model.cache_requests()) == [0, 1, 2]
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(plan, 9, device=DEV).items()}
        toks = [3, 200, 17, 17, 42, 9, 250, 1, 77]
        c = cfg.to_dict()

        def plain_looped(tokens):
            x = w["model.embed_tokens.weight"][tokens]
            S = len(tokens)
            kv1 = {}

            def block(x, layer, reuse=None):
                p = f"model.layers.{layer}"
                n = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], c["rms_norm_eps"])
                f = lambda nm: w[f"{p}.self_attn.{nm}.weight"]
                q = plain.rms_norm((n @ f("q_proj").T).view(S, 4, 16), f("q_norm"), c["rms_norm_eps"])
                cos, sin = plain.rope_cos_sin(torch.arange(S), 16, c["rope_theta"])
                q = plain.rope_rotate_neox(q, cos, sin, 16)
                if reuse is None:
                    k = plain.rms_norm((n @ f("k_proj").T).view(S, 2, 16), f("k_norm"), c["rms_norm_eps"])
                    k = plain.rope_rotate_neox(k, cos, sin, 16)
                    v = (n @ f("v_proj").T).view(S, 2, 16)
                    kv1[layer] = (k, v)
                else:
                    k, v = reuse
                a = plain.causal_gqa_attention(q, k, v, 0.25).reshape(S, 64) @ f("o_proj").T
                h = x + a
                n2 = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], c["rms_norm_eps"])
                return h + plain.swiglu(n2, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"])

            x = block(x, 0)
            x = block(x, 1)
            first_kv1 = kv1[1]
            x = block(x, 0)
            x = block(x, 1, reuse=first_kv1)
            return plain.rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T

        s = eng.alloc_slot()
        lg = [eng.step([pe.StepEntry(s, toks[:6], (0, 5))]).cpu()]
        for t in toks[6:]:
            lg.append(eng.step([pe.StepEntry(s, [t], (0,))]).cpu())
        eng.free_slot(s)
        ref = plain_looped(toks)
        assert rel_err(torch.cat(lg), ref[[0, 5, 6, 7, 8]]) < 1e-5
    finally:
        pe.config.unregister_architecture("LoopedQwen3")


# ---- a toy feed-forward with routing and a toy position encoding ---------------------------------------
@dataclass(frozen=True)
class ToyMixConfig:
    hidden_size: int = 40
    vocab_size: int = 83
    heads: int = 5
    kv_heads: int = 1
    head_dim: int = 16
    experts: int = 3
    expert_size: int = 24
    slow_factor: float = 4.0
    max_position_embeddings: int = 128
    architecture: str = "ToyRoutedLM"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: v for k, v in d.items() if k != "architectures"})

    def to_dict(self):
        out = {k: getattr(self, k) for k in self.__dataclass_fields__ if k != "architecture"}
        out["architectures"] = [self.architecture]
        return out

    max_positions = property(lambda self: self.max_position_embeddings)
    stop_token_ids = ()
    bos_token = 0


class TopOneExperts:
    """Every token goes to the expert with the largest router logit; its SwiGLU output is scaled by
    that expert's softmax probability.  Router logits and probabilities in float32."""

    graph_safe = False   # the routing is read on the host

    @classmethod
    def weight_decls(cls, params):
        from importlib import import_module
        WeightDecl = import_module("pytorch-engine_b200").parts.WeightDecl
        h, e, i = params["hidden"], params["experts"], params["expert_size"]
        decls = {"router": WeightDecl((e, h))}
        for x in range(e):
            decls.update({f"gate{x}": WeightDecl((i, h)), f"up{x}": WeightDecl((i, h)), f"down{x}": WeightDecl((h, i))})
        return decls

    def __init__(self, params, weights, runtime):
        self.rt, self.n = runtime, int(params["experts"])
        self.router = runtime.adopt(weights["router"], torch.float32)
        self.w = [{k: runtime.adopt(weights[f"{k}{x}"]) for k in ("gate", "up", "down")} for x in range(self.n)]

    def forward(self, x, ctx):
        prob = torch.softmax(x.float() @ self.router.T, -1)
        top_p, top_e = prob.max(-1)
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in range(self.n):
            rows = (top_e == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows].contiguous()
            g, u = self.rt.linear(xe, self.w[e]["gate"]).float(), self.rt.linear(xe, self.w[e]["up"]).float()
            act = (g / (1 + torch.exp(-g)) * u).to(x.dtype)
            out[rows] = self.rt.linear(act, self.w[e]["down"]).float() * top_p[rows, None]
        return out.to(x.dtype)


class SlowRotaryPosition:
    """Rotary tables whose angles advance ``factor`` times slower (position / factor)."""

    graph_safe = True
    fusable_rotary = True

    @classmethod
    def weight_decls(cls, params):
        return {}

    def __init__(self, params, weights, runtime):
        self.rotary_dim = int(params["rotary_dim"])
        inv = plain.rope_inv_freq(self.rotary_dim, float(params["theta"]))
        pos = torch.arange(int(params["max_positions"]), dtype=torch.float32) / float(params["factor"])
        ang = torch.outer(pos, inv)
        self.cos, self.sin = torch.cos(ang).to(runtime.device), torch.sin(ang).to(runtime.device)

    def tables(self):
        return self.cos, self.sin, self.rotary_dim


def test_toy_routed_feed_forward_and_another_position_encoding(pe):
    """Parts defined here are registered, chosen layer by layer next to the package's own, built and
    stepped: layer 0 has the slow rotary encoding and routed experts, layer 1 the usual ones."""
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep
    eps, theta = 1e-5, 500.0

    def plan(cfg):
        h, d = cfg.hidden_size, cfg.head_dim
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": eps}, {"weight": n})
        att = lambda i, position: P("attention", {"hidden": h, "n_heads": cfg.heads, "n_kv_heads": cfg.kv_heads, "head_dim": d,
                                                  "qk_norm": False, "eps": eps, "scale": None, "window": None,
                                                  "position": position},
                                    {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        routed = P("top_one_experts", {"hidden": h, "experts": cfg.experts, "expert_size": cfg.expert_size},
                   {"router": "l0.router", **{f"{k}{x}": f"l0.{k}{x}" for x in range(cfg.experts) for k in ("gate", "up", "down")}})
        dense = P("swiglu", {"hidden": h, "intermediate": 2 * h}, {"gate_proj": "l1.g", "up_proj": "l1.u", "down_proj": "l1.d"})
        blocks = (B.standard("pre_norm", norm("l0.n1"), att(0, "slow"), norm("l0.n2"), routed, name="routed"),
                  B.standard("pre_norm", norm("l1.n1"), att(1, "rope"), norm("l1.n2"), dense, name="dense"))
        return pe.parts.ModelPlan(
            hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
            embedding=P("token_embedding", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "emb"}),
            blocks=blocks, order=(R(0), R(1)), final_norm=norm("fn"),
            head=P("linear_head", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "head"}),
            positions={"rope": P("rope", {"rotary_dim": d, "theta": theta, "max_positions": cfg.max_position_embeddings}),
                       "slow": P("slow_rope", {"rotary_dim": d, "theta": theta, "factor": cfg.slow_factor,
                                               "max_positions": cfg.max_position_embeddings})})

    pe.parts.register("feed_forward", "top_one_experts", TopOneExperts, replace=True)
    pe.parts.register("position", "slow_rope", SlowRotaryPosition, replace=True)
    pe.register_architecture("ToyRoutedLM", ToyMixConfig, plan, replace=True)
    try:
        cfg = ToyMixConfig()
        eng = pe.Engine.from_random(cfg, seed=11, dtype="float32", max_cache_tokens=256, max_batch=2)
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 11, device=DEV).items()}
        nH, nKV, d, h = cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.hidden_size

        def attention(x, i, factor):
            S = x.shape[0]
            pos = torch.arange(S, dtype=torch.float32) / factor
            ang = torch.outer(pos, plain.rope_inv_freq(d, theta))
            cos, sin = torch.cos(ang), torch.sin(ang)
            q = plain.rope_rotate_neox((x @ w[f"l{i}.q_proj"].T).view(S, nH, d), cos, sin, d)
            k = plain.rope_rotate_neox((x @ w[f"l{i}.k_proj"].T).view(S, nKV, d), cos, sin, d)
            v = (x @ w[f"l{i}.v_proj"].T).view(S, nKV, d)
            return plain.causal_gqa_attention(q, k, v, d ** -0.5).reshape(S, nH * d) @ w[f"l{i}.o_proj"].T

        def plain_toy(tokens):
            x = w["emb"][tokens]
            x = x + attention(plain.rms_norm(x, w["l0.n1"], eps), 0, cfg.slow_factor)
            n = plain.rms_norm(x, w["l0.n2"], eps)
            prob = torch.softmax(n @ w["l0.router"].T, -1)
            rows, chosen = [], []
            for t in range(len(tokens)):
                e = int(prob[t].argmax())
                chosen.append(e)
                rows.append(prob[t, e] * plain.swiglu(n[t:t + 1], w[f"l0.gate{e}"], w[f"l0.up{e}"], w[f"l0.down{e}"])[0])
            x = x + torch.stack(rows)
            x = x + attention(plain.rms_norm(x, w["l1.n1"], eps), 1, 1.0)
            x = x + plain.swiglu(plain.rms_norm(x, w["l1.n2"], eps), w["l1.g"], w["l1.u"], w["l1.d"])
            return plain.rms_norm(x, w["fn"], eps) @ w["head"].T, chosen

        seqs = [[5, 9, 2, 77, 31, 8, 8, 40, 3, 61], [82, 0, 3, 3, 14, 7]]
        refs = [plain_toy(s) for s in seqs]
        assert len({e for _, ch in refs for e in ch}) > 1          # more than one expert is in use
        slots = [eng.alloc_slot(), eng.alloc_slot()]
        got = [[], []]
        lg = eng.step([pe.StepEntry(slots[0], seqs[0][:6], (0, 5)), pe.StepEntry(slots[1], seqs[1][:2], (1,))])
        got[0] += [lg[0].cpu(), lg[1].cpu()]; got[1].append(lg[2].cpu())
        for k in range(4):
            lg = eng.step([pe.StepEntry(slots[0], [seqs[0][6 + k]], (0,)), pe.StepEntry(slots[1], [seqs[1][2 + k]], (0,))])
            got[0].append(lg[0].cpu()); got[1].append(lg[1].cpu())
        for s in slots:
            eng.free_slot(s)
        assert rel_err(torch.stack(got[0]), refs[0][0][[0, 5, 6, 7, 8, 9]]) < 1e-5
        assert rel_err(torch.stack(got[1]), refs[1][0][[1, 2, 3, 4, 5]]) < 1e-5
    finally:
        pe.parts.unregister("feed_forward", "top_one_experts")
        pe.parts.unregister("position", "slow_rope")
        pe.config.unregister_architecture("ToyRoutedLM")


# ---- a toy block arrangement ------------------------------------------------------------------------------
class ParallelBlock:
    """``out = x + mixer(norm(x)) + ffn(norm(x))``: mixer and feed-forward read the same normed input
    (the second norm of the block's description is built but not used)."""

    graph_safe = True

    def __init__(self, spec, parts, runtime):
        self.rt, self.norm, self.mixer, self.ffn = runtime, parts["mixer_norm"], parts["mixer"], parts["ffn"]

    def forward(self, stream, pending, ctx, view, writes_cache=True):
        normed = ctx.buffer("parallel.normed", tuple(stream.shape), self.rt.dtype)
        self.norm.add_forward(stream, pending, normed)            # adds the block before's delta, then norms
        mixed = self.mixer.forward(normed, ctx, view)
        return (mixed.float() + self.ffn.forward(normed, ctx).float()).to(self.rt.dtype)


def test_toy_block_arrangement(pe):
    """An arrangement defined here is registered and chosen for one block of a model whose other block
    keeps the package's pre-norm arrangement."""
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep
    eps, theta = 1e-6, 10000.0
    cfg = ToyMixConfig(hidden_size=48, vocab_size=101, heads=3, kv_heads=3, head_dim=16, architecture="ToyParallelLM")

    def plan(c):
        h, d = c.hidden_size, c.head_dim
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": eps}, {"weight": n})
        att = lambda i: P("attention", {"hidden": h, "n_heads": c.heads, "n_kv_heads": c.kv_heads, "head_dim": d,
                                        "qk_norm": False, "eps": eps, "scale": None, "window": None, "position": "rope"},
                          {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        ffn = lambda i: P("swiglu", {"hidden": h, "intermediate": 2 * h}, {"gate_proj": f"l{i}.g", "up_proj": f"l{i}.u", "down_proj": f"l{i}.d"})
        blocks = (B.standard("parallel", norm("l0.n1"), att(0), norm("l0.n2"), ffn(0), name="parallel"),
                  B.standard("pre_norm", norm("l1.n1"), att(1), norm("l1.n2"), ffn(1), name="sequential"))
        return pe.parts.ModelPlan(
            hidden_size=h, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
            embedding=P("token_embedding", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            blocks=blocks, order=(R(0), R(1)), final_norm=norm("fn"),
            head=P("linear_head", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            positions={"rope": P("rope", {"rotary_dim": d, "theta": theta, "max_positions": c.max_position_embeddings})})

    pe.parts.register("arrangement", "parallel", ParallelBlock, replace=True)
    pe.register_architecture("ToyParallelLM", ToyMixConfig, plan, replace=True)
    try:
        eng = pe.Engine.from_random(cfg, seed=12, dtype="float32", max_cache_tokens=256, max_batch=2)
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 12, device=DEV).items()}
        nH, d = cfg.heads, cfg.head_dim

        def attention(x, i):
            S = x.shape[0]
            cos, sin = plain.rope_cos_sin(torch.arange(S), d, theta)
            q = plain.rope_rotate_neox((x @ w[f"l{i}.q_proj"].T).view(S, nH, d), cos, sin, d)
            k = plain.rope_rotate_neox((x @ w[f"l{i}.k_proj"].T).view(S, nH, d), cos, sin, d)
            v = (x @ w[f"l{i}.v_proj"].T).view(S, nH, d)
            return plain.causal_gqa_attention(q, k, v, d ** -0.5).reshape(S, nH * d) @ w[f"l{i}.o_proj"].T

        def plain_toy(tokens):
            x = w["emb"][tokens]
            n = plain.rms_norm(x, w["l0.n1"], eps)
            x = x + attention(n, 0) + plain.swiglu(n, w["l0.g"], w["l0.u"], w["l0.d"])
            x = x + attention(plain.rms_norm(x, w["l1.n1"], eps), 1)
            x = x + plain.swiglu(plain.rms_norm(x, w["l1.n2"], eps), w["l1.g"], w["l1.u"], w["l1.d"])
            return plain.rms_norm(x, w["fn"], eps) @ w["emb"].T

        toks = [5, 9, 2, 77, 31, 8, 8, 40, 3, 61, 100]
        s = eng.alloc_slot()
        lg = [eng.step([pe.StepEntry(s, toks[:7], (0, 6))]).cpu()]
        for t in toks[7:]:
            lg.append(eng.step([pe.StepEntry(s, [t], (0,))]).cpu())
        eng.free_slot(s)
        assert rel_err(torch.cat(lg), plain_toy(toks)[[0, 6, 7, 8, 9, 10]]) < 1e-5
    finally:
        pe.parts.unregister("arrangement", "parallel")
        pe.config.unregister_architecture("ToyParallelLM")


# ---- a toy norm ----------------------------------------------------------------------------------------------
class CenteredNorm:
    """LayerNorm without bias: ``(x - mean) / sqrt(var + eps) * weight``, statistics in float32."""

    graph_safe = True

    @classmethod
    def weight_decls(cls, params):
        from importlib import import_module
        WeightDecl = import_module("pytorch-engine_b200").parts.WeightDecl
        return {"weight": WeightDecl((int(params["dim"]),), "norm")}

    def __init__(self, params, weights, runtime):
        self.eps = float(params["eps"])
        self.weight = runtime.adopt(weights["weight"], torch.float32)

    def _norm(self, x):
        x = x.float()
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight

    def add_forward(self, residual, delta, out, rows=None):
        if delta is not None:
            residual.add_(delta.float())          # the stream takes the pending delta, as the package's norm does
        src = residual if rows is None else residual[rows.long()]
        out.copy_(self._norm(src).to(out.dtype))
        return out

    def forward(self, x, out=None):
        y = self._norm(x).to(x.dtype)
        return y if out is None else out.copy_(y)


def test_toy_norm(pe):
    """A norm defined here takes the place of every norm of a small model (final norm included)."""
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep
    eps, theta = 1e-5, 10000.0
    cfg = ToyMixConfig(hidden_size=40, vocab_size=89, heads=2, kv_heads=1, head_dim=16, architecture="ToyCenteredLM")

    def plan(c):
        h, d = c.hidden_size, c.head_dim
        norm = lambda n: P("centered", {"dim": h, "eps": eps}, {"weight": n})
        att = P("attention", {"hidden": h, "n_heads": c.heads, "n_kv_heads": c.kv_heads, "head_dim": d, "qk_norm": False,
                              "eps": eps, "scale": None, "window": None, "position": "rope"},
                {k: f"l0.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        ffn = P("swiglu", {"hidden": h, "intermediate": 64}, {"gate_proj": "l0.g", "up_proj": "l0.u", "down_proj": "l0.d"})
        return pe.parts.ModelPlan(
            hidden_size=h, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
            embedding=P("token_embedding", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            blocks=(B.standard("pre_norm", norm("l0.n1"), att, norm("l0.n2"), ffn, name="only"),), order=(R(0),),
            final_norm=norm("fn"), head=P("linear_head", {"vocab": c.vocab_size, "hidden": h}, {"weight": "head"}),
            positions={"rope": P("rope", {"rotary_dim": d, "theta": theta, "max_positions": c.max_position_embeddings})})

    pe.parts.register("norm", "centered", CenteredNorm, replace=True)
    pe.register_architecture("ToyCenteredLM", ToyMixConfig, plan, replace=True)
    try:
        eng = pe.Engine.from_random(cfg, seed=13, dtype="float32", max_cache_tokens=128, max_batch=2)
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 13, device=DEV).items()}
        nH, nKV, d = cfg.heads, cfg.kv_heads, cfg.head_dim

        def cnorm(x, weight):
            x = x - x.mean(-1, keepdim=True)
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight

        def plain_toy(tokens):
            x = w["emb"][tokens]
            S = len(tokens)
            n = cnorm(x, w["l0.n1"])
            cos, sin = plain.rope_cos_sin(torch.arange(S), d, theta)
            q = plain.rope_rotate_neox((n @ w["l0.q_proj"].T).view(S, nH, d), cos, sin, d)
            k = plain.rope_rotate_neox((n @ w["l0.k_proj"].T).view(S, nKV, d), cos, sin, d)
            v = (n @ w["l0.v_proj"].T).view(S, nKV, d)
            x = x + plain.causal_gqa_attention(q, k, v, d ** -0.5).reshape(S, nH * d) @ w["l0.o_proj"].T
            x = x + plain.swiglu(cnorm(x, w["l0.n2"]), w["l0.g"], w["l0.u"], w["l0.d"])
            return cnorm(x, w["fn"]) @ w["head"].T

        seqs = [[5, 9, 2, 77, 31, 8, 8, 40], [88, 0, 3]]
        slots = [eng.alloc_slot(), eng.alloc_slot()]
        lg = eng.step([pe.StepEntry(slots[0], seqs[0][:6], (2, 5)), pe.StepEntry(slots[1], seqs[1][:2], (1,))]).cpu()
        got0, got1 = [lg[0], lg[1]], [lg[2]]
        lg = eng.step([pe.StepEntry(slots[0], [seqs[0][6]], (0,)), pe.StepEntry(slots[1], [seqs[1][2]], (0,))]).cpu()
        got0.append(lg[0]); got1.append(lg[1])
        lg = eng.step([pe.StepEntry(slots[0], [seqs[0][7]], (0,))]).cpu()
        got0.append(lg[0])
        for s in slots:
            eng.free_slot(s)
        assert rel_err(torch.stack(got0), plain_toy(seqs[0])[[2, 5, 6, 7]]) < 1e-5
        assert rel_err(torch.stack(got1), plain_toy(seqs[1])[[1, 2]]) < 1e-5
    finally:
        pe.parts.unregister("norm", "centered")
        pe.config.unregister_architecture("ToyCenteredLM")


# ---- a position encoding without rotary tables, and a block with four norms ----------------------------------
class LearnedAbsolutePosition:
    """A learned vector per position, added to every query and key head (nothing rotates).  It has no
    ``tables()``: attention calls ``apply`` between its q/k-norm and the append to the cache."""

    graph_safe = True   # apply() only launches

    @classmethod
    def weight_decls(cls, params):
        from importlib import import_module
        WeightDecl = import_module("pytorch-engine_b200").parts.WeightDecl
        return {"table": WeightDecl((int(params["max_positions"]), int(params["head_dim"])))}

    def __init__(self, params, weights, runtime):
        self.table = runtime.adopt(weights["table"])

    def apply(self, q, k, positions):
        add = self.table.index_select(0, positions.long())[:, None, :]
        q.add_(add)
        k.add_(add)


class SandwichBlock:
    """``h = x + post1(mixer(pre1(x)))``; ``out = h + post2(ffn(pre2(h)))``: four norms, the outputs of mixer and
    feed-forward normalised before they join the stream (the shape of pygguf_engine/model.py:1035-1041)."""

    graph_safe = True

    def __init__(self, spec, parts, runtime):
        self.rt, self.p = runtime, parts

    def forward(self, stream, pending, ctx, view, writes_cache=True):
        normed = ctx.buffer("sandwich.normed", tuple(stream.shape), self.rt.dtype)
        self.p["pre_mixer"].add_forward(stream, pending, normed)
        mixed = self.p["post_mixer"].forward(self.p["mixer"].forward(normed, ctx, view))
        self.p["pre_ffn"].add_forward(stream, mixed, normed)
        return self.p["post_ffn"].forward(self.p["ffn"].forward(normed, ctx))


def test_toy_learned_positions_and_a_block_with_four_norms(pe):
    """Registered from here, with no change to the package: a position encoding that is no rotary table, used by
    the package's own attention (with q/k-norm, so the order norm -> position -> append shows), and an
    arrangement whose block carries six parts, four of them norms."""
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep
    eps, theta = 1e-5, 10000.0
    cfg = ToyMixConfig(hidden_size=48, vocab_size=97, heads=4, kv_heads=2, head_dim=16, architecture="ToySandwichLM")

    def plan(c):
        h, d = c.hidden_size, c.head_dim
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": eps}, {"weight": n})
        att = lambda i, position: P(
            "attention", {"hidden": h, "n_heads": c.heads, "n_kv_heads": c.kv_heads, "head_dim": d, "qk_norm": True,
                          "eps": eps, "scale": None, "window": None, "position": position},
            {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})
        ffn = lambda i: P("swiglu", {"hidden": h, "intermediate": 2 * h},
                          {"gate_proj": f"l{i}.g", "up_proj": f"l{i}.u", "down_proj": f"l{i}.d"})
        sandwich = B("sandwich", {"pre_mixer": ("norm", norm("l0.n1")), "mixer": ("mixer", att(0, "learned")),
                                  "post_mixer": ("norm", norm("l0.n1b")), "pre_ffn": ("norm", norm("l0.n2")),
                                  "ffn": ("feed_forward", ffn(0)), "post_ffn": ("norm", norm("l0.n2b"))}, name="sandwich")
        usual = B.standard("pre_norm", norm("l1.n1"), att(1, "rope"), norm("l1.n2"), ffn(1), name="usual")
        return pe.parts.ModelPlan(
            hidden_size=h, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
            embedding=P("token_embedding", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            blocks=(sandwich, usual), order=(R(0), R(1)), final_norm=norm("fn"),
            head=P("linear_head", {"vocab": c.vocab_size, "hidden": h}, {"weight": "head"}),
            positions={"rope": P("rope", {"rotary_dim": d, "theta": theta, "max_positions": c.max_position_embeddings}),
                       "learned": P("learned_abs", {"head_dim": d, "max_positions": c.max_position_embeddings},
                                    {"table": "pos.table"})})

    pe.parts.register("position", "learned_abs", LearnedAbsolutePosition, replace=True)
    pe.parts.register("arrangement", "sandwich", SandwichBlock, replace=True)
    pe.register_architecture("ToySandwichLM", ToyMixConfig, plan, replace=True)
    try:
        eng = pe.Engine.from_random(cfg, seed=21, dtype="float32", max_cache_tokens=256, max_batch=2)
        assert eng.runner.cuda_graphs                       # every part said graph_safe: decode replays graphs
        labels = [label for label, _, _ in eng.plan.part_specs()]
        assert "sandwich post_mixer" in labels and "sandwich post_ffn" in labels
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 21, device=DEV).items()}
        w["pos.table"] = w["pos.table"] * 25.0             # make the position term matter next to unit-norm heads
        eng = pe.Engine(None, config=cfg, weights={k: v.to(DEV) for k, v in w.items()}, dtype="float32",
                        max_cache_tokens=256, max_batch=2)
        nH, nKV, d = cfg.heads, cfg.kv_heads, cfg.head_dim

        def attention(n, i, position):
            S = n.shape[0]
            q = plain.rms_norm((n @ w[f"l{i}.q_proj"].T).view(S, nH, d), w[f"l{i}.q_norm"], eps)
            k = plain.rms_norm((n @ w[f"l{i}.k_proj"].T).view(S, nKV, d), w[f"l{i}.k_norm"], eps)
            if position == "learned":
                q, k = q + w["pos.table"][:S, None, :], k + w["pos.table"][:S, None, :]
            else:
                cos, sin = plain.rope_cos_sin(torch.arange(S), d, theta)
                q, k = plain.rope_rotate_neox(q, cos, sin, d), plain.rope_rotate_neox(k, cos, sin, d)
            v = (n @ w[f"l{i}.v_proj"].T).view(S, nKV, d)
            return plain.causal_gqa_attention(q, k, v, d ** -0.5).reshape(S, nH * d) @ w[f"l{i}.o_proj"].T

        def plain_toy(tokens, learned=True):
            x = w["emb"][tokens]
            mixed = attention(plain.rms_norm(x, w["l0.n1"], eps), 0, "learned" if learned else "none")
            x = x + plain.rms_norm(mixed, w["l0.n1b"], eps)
            f = plain.swiglu(plain.rms_norm(x, w["l0.n2"], eps), w["l0.g"], w["l0.u"], w["l0.d"])
            x = x + plain.rms_norm(f, w["l0.n2b"], eps)
            x = x + attention(plain.rms_norm(x, w["l1.n1"], eps), 1, "rope")
            x = x + plain.swiglu(plain.rms_norm(x, w["l1.n2"], eps), w["l1.g"], w["l1.u"], w["l1.d"])
            return plain.rms_norm(x, w["fn"], eps) @ w["head"].T

        seqs = [[5, 9, 2, 77, 31, 8, 8, 40, 3, 61], [82, 0, 3, 3, 14, 7]]
        refs = [plain_toy(s) for s in seqs]
        # the learned positions change the result by far more than the tolerance: the check below sees them
        assert rel_err(plain_toy(seqs[0], learned=False), refs[0]) > 1e-2
        for rnd in range(2):
            slots = [eng.alloc_slot(), eng.alloc_slot()]
            got = [[], []]
            lg = eng.step([pe.StepEntry(slots[0], seqs[0][:6], (0, 5)), pe.StepEntry(slots[1], seqs[1][:2], (1,))])
            got[0] += [lg[0].cpu(), lg[1].cpu()]; got[1].append(lg[2].cpu())
            for k in range(4):
                lg = eng.step([pe.StepEntry(slots[0], [seqs[0][6 + k]], (0,)), pe.StepEntry(slots[1], [seqs[1][2 + k]], (0,))])
                got[0].append(lg[0].cpu()); got[1].append(lg[1].cpu())
            for s in slots:
                eng.free_slot(s)
            assert rel_err(torch.stack(got[0]), refs[0][[0, 5, 6, 7, 8, 9]]) < 1e-5
            assert rel_err(torch.stack(got[1]), refs[1][[1, 2, 3, 4, 5]]) < 1e-5
    finally:
        pe.parts.unregister("position", "learned_abs")
        pe.parts.unregister("arrangement", "sandwich")
        pe.config.unregister_architecture("ToySandwichLM")


# ---- a state mixer whose decode step only launches: CUDA graphs must fold each token in once ----------------
class LaunchOnlySumMixer(DecayingSumMixer):
    """``DecayingSumMixer`` whose one-token step reads nothing on the host, so that decode steps of a model
    made of it are replayed from CUDA graphs (prompts still go token by token on the host)."""

    graph_safe = True

    def forward(self, x, ctx, view):
        if not ctx.decode:
            return super().forward(x, ctx, view)
        z = self.rt.linear(x, self.proj).float()
        state = view.state("acc")
        slots = ctx.seq_slot.long()
        new = self.decay * state.index_select(0, slots) + z
        state.index_copy_(0, slots, new)
        return new.to(x.dtype)


def test_state_mixer_under_cuda_graphs_sees_every_token_once(pe):
    """The first decode step of each batch size is the one that captures a graph; a mixer with state of fixed
    size would show a token folded in twice there.  Graph replay and eager steps must agree, step by step,
    as the batch shrinks 3 -> 2 -> 1 (three captures)."""
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep

    def plan(cfg):
        h = cfg.hidden_size
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": 1e-6}, {"weight": n})
        blocks = tuple(B.standard("pre_norm", norm(f"l{i}.n1"), P("launch_only_sum", {"hidden": h, "decay": cfg.decay}, {"proj": f"l{i}.proj"}),
                                  norm(f"l{i}.n2"), P("swiglu", {"hidden": h, "intermediate": 2 * h},
                                                      {"gate_proj": f"l{i}.g", "up_proj": f"l{i}.u", "down_proj": f"l{i}.d"}),
                                  name=f"toy {i}") for i in range(cfg.layers))
        return pe.parts.ModelPlan(hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                                  embedding=P("token_embedding", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "emb"}),
                                  blocks=blocks, order=tuple(R(i) for i in range(cfg.layers)), final_norm=norm("fn"),
                                  head=P("linear_head", {"vocab": cfg.vocab_size, "hidden": h}, {"weight": "emb"}))

    pe.parts.register("mixer", "launch_only_sum", LaunchOnlySumMixer, replace=True)
    pe.register_architecture("ToyRunningMeanLM", ToyConfig, plan, replace=True)
    try:
        cfg = ToyConfig(hidden_size=48, vocab_size=97, layers=2, decay=0.75)
        seqs = [[5, 9, 2, 77, 31, 8, 8, 40, 1], [96, 0, 3, 3, 14, 9], [7, 7, 50, 2]]
        runs = {}
        for graphs in (True, False):
            eng = pe.Engine.from_random(cfg, seed=4, dtype="float32", max_cache_tokens=256, max_batch=4,
                                        enable_cuda_graph=graphs)
            assert eng.runner.cuda_graphs == graphs
            slots = [eng.alloc_slot() for _ in seqs]
            out = [eng.step([pe.StepEntry(s, q[:2], (1,)) for s, q in zip(slots, seqs)]).cpu().clone()]
            for k in range(2, 9):
                live = [(s, q) for s, q in zip(slots, seqs) if k < len(q)]
                out.append(eng.step([pe.StepEntry(s, [q[k]], (0,)) for s, q in live]).cpu().clone())
            runs[graphs] = out
            if graphs:
                assert sorted(eng.runner._graphs) == [1, 2, 3]
        for a, b in zip(runs[True], runs[False]):
            assert a.shape == b.shape and rel_err(a, b) < 1e-6
    finally:
        pe.parts.unregister("mixer", "launch_only_sum")
        pe.config.unregister_architecture("ToyRunningMeanLM")


# ---- a block with two mixers: each gets a cache entry of its own ------------------------------------------------
class TwoMixerBlock:
    """``out = x + local(norm(x)) + global(norm(x))`` and no feed-forward: two attention mixers (a windowed and a
    full one) read the same normed input; the block's cache view is a dict by mixer name."""

    graph_safe = True

    def __init__(self, spec, parts, runtime):
        self.rt, self.p = runtime, parts

    def forward(self, stream, pending, ctx, view, writes_cache=True):
        normed = ctx.buffer("two.normed", tuple(stream.shape), self.rt.dtype)
        self.p["norm"].add_forward(stream, pending, normed)
        # a part's delta lies in a step buffer that the next call of a part of the same class uses again: the two
        # mixers are both attention, so the first one's output is copied before the second runs
        a = self.p["local"].forward(normed, ctx, view["local"]).to(torch.float32, copy=True)
        b = self.p["global"].forward(normed, ctx, view["global"]).float()
        return (a + b).to(self.rt.dtype)


def test_toy_block_with_two_mixers_and_no_feed_forward(pe):
    P, B, R = pe.parts.PartSpec, pe.parts.BlockSpec, pe.parts.RunStep
    eps, theta, window = 1e-6, 10000.0, 9
    cfg = ToyMixConfig(hidden_size=48, vocab_size=101, heads=3, kv_heads=1, head_dim=16, architecture="ToyTwoMixerLM")

    def plan(c):
        h, d = c.hidden_size, c.head_dim
        norm = lambda n: P("rmsnorm", {"dim": h, "eps": eps}, {"weight": n})
        att = lambda tag, win: P("attention", {"hidden": h, "n_heads": c.heads, "n_kv_heads": c.kv_heads, "head_dim": d,
                                               "qk_norm": False, "eps": eps, "scale": None, "window": win, "position": "rope"},
                                 {k: f"l0.{tag}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        two = B("two_mixers", {"norm": ("norm", norm("l0.n")), "local": ("mixer", att("local", window)),
                               "global": ("mixer", att("global", None))}, name="two")
        usual = B.standard("pre_norm", norm("l1.n1"), att("usual", None), norm("l1.n2"),
                           P("swiglu", {"hidden": h, "intermediate": 2 * h}, {"gate_proj": "l1.g", "up_proj": "l1.u", "down_proj": "l1.d"}),
                           name="usual")
        return pe.parts.ModelPlan(
            hidden_size=h, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
            embedding=P("token_embedding", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            blocks=(two, usual), order=(R(0), R(1)), final_norm=norm("fn"),
            head=P("linear_head", {"vocab": c.vocab_size, "hidden": h}, {"weight": "emb"}),
            positions={"rope": P("rope", {"rotary_dim": d, "theta": theta, "max_positions": c.max_position_embeddings})})

    pe.parts.register("arrangement", "two_mixers", TwoMixerBlock, replace=True)
    pe.register_architecture("ToyTwoMixerLM", ToyMixConfig, plan, replace=True)
    try:
        eng = pe.Engine.from_random(cfg, seed=31, dtype="float32", max_cache_tokens=256, max_batch=2)
        # three cache entries in two groups: the windowed mixer's, and the two full ones (block 0's and block 1's)
        kinds = sorted((g.request.window or 0, [str(e) for e in g.entries]) for g in eng.cache.groups)
        assert kinds == [(0, ["(0, 'global')", "1"]), (window, ["(0, 'local')"])]
        w = {k: v.float().cpu() for k, v in pe.weights.random_weights(eng.plan, 31, device=DEV).items()}
        nH, nKV, d = cfg.heads, cfg.kv_heads, cfg.head_dim

        def attention(n, tag, win):
            S = n.shape[0]
            cos, sin = plain.rope_cos_sin(torch.arange(S), d, theta)
            q = plain.rope_rotate_neox((n @ w[f"{tag}.q_proj"].T).view(S, nH, d), cos, sin, d)
            k = plain.rope_rotate_neox((n @ w[f"{tag}.k_proj"].T).view(S, nKV, d), cos, sin, d)
            v = (n @ w[f"{tag}.v_proj"].T).view(S, nKV, d)
            return plain.causal_gqa_attention(q, k, v, d ** -0.5, window=win).reshape(S, nH * d) @ w[f"{tag}.o_proj"].T

        def plain_toy(tokens):
            x = w["emb"][tokens]
            n = plain.rms_norm(x, w["l0.n"], eps)
            x = x + attention(n, "l0.local", window) + attention(n, "l0.global", None)
            x = x + attention(plain.rms_norm(x, w["l1.n1"], eps), "l0.usual", None)
            x = x + plain.swiglu(plain.rms_norm(x, w["l1.n2"], eps), w["l1.g"], w["l1.u"], w["l1.d"])
            return plain.rms_norm(x, w["fn"], eps) @ w["emb"].T

        seqs = [list(range(5, 45)), [88, 0, 3, 7, 7, 21]]
        refs = [plain_toy(s) for s in seqs]
        for rnd in range(2):
            slots = [eng.alloc_slot(), eng.alloc_slot()]
            got = [[], []]
            lg = eng.step([pe.StepEntry(slots[0], seqs[0][:30], (0, 29)), pe.StepEntry(slots[1], seqs[1][:2], (1,))])
            got[0] += [lg[0].cpu(), lg[1].cpu()]; got[1].append(lg[2].cpu())
            for k in range(4):
                lg = eng.step([pe.StepEntry(slots[0], [seqs[0][30 + k]], (0,)), pe.StepEntry(slots[1], [seqs[1][2 + k]], (0,))])
                got[0].append(lg[0].cpu()); got[1].append(lg[1].cpu())
            for s in slots:
                eng.free_slot(s)
            e0 = [rel_err(g, r) for g, r in zip(got[0], refs[0][[0, 29, 30, 31, 32, 33]])]
            e1 = [rel_err(g, r) for g, r in zip(got[1], refs[1][[1, 2, 3, 4, 5]])]
            assert max(e0) < 1e-5 and max(e1) < 1e-5, (rnd, e0, e1)
        eng.cache.check()
    finally:
        pe.parts.unregister("arrangement", "two_mixers")
        pe.config.unregister_architecture("ToyTwoMixerLM")
