"""Each part alone against its plain formula, and a model put together in the test from a toy
mixer with state of its own, without a change to the framework's files."""

import math
from dataclasses import dataclass

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu
TOL = {torch.float32: dict(rtol=2e-5, atol=2e-6), torch.bfloat16: dict(rtol=3e-2, atol=2e-2)}


def rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def ctx(dtype):
    from scratch_llm_b200.parts import BuildContext
    return BuildContext(dtype=dtype, device=torch.device("cuda"))


@pytest.fixture(scope="module", autouse=True)
def compiled():
    from scratch_llm_b200.kernels import ops
    ops.prepare([16, 48], verbose=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from scratch_llm_b200.parts import NORMS, make
    from scratch_llm_b200.config.spec import PartSpec
    norm = make(NORMS, "norm", PartSpec("rmsnorm", {"size": 100, "eps": 1e-3}))
    assert set(norm.param_specs()) == {"weight"}
    w = rand(100, seed=1) + 1
    norm.load({"weight": w}, ctx(dtype))
    resid, delta = rand(6, 100, seed=2), rand(6, 100, seed=3).to(dtype)
    r = resid.cuda()
    out = norm.forward(r, delta.cuda())
    assert out.dtype == dtype
    torch.testing.assert_close(out.cpu().float(), P.rmsnorm(resid + delta.float(), w, 1e-3), **TOL[dtype])
    torch.testing.assert_close(r.cpu(), resid + delta.float(), rtol=0, atol=0)


def test_rotary_part_tables():
    from scratch_llm_b200.parts.position import Rotary
    rot = Rotary(head_dim=48, theta=50000.0, max_position=500, interleaved=True)
    rot.load({}, ctx(torch.float32))
    cos, sin = P.rope_tables(48, 500, 50000.0)
    assert torch.equal(rot.cos.cpu(), cos) and torch.equal(rot.sin.cpu(), sin)
    assert rot.cos.dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from scratch_llm_b200.parts.feed_forward import SwiGLU
    ff = SwiGLU(hidden_size=72, intermediate_size=200)
    t = {"gate_proj.weight": rand(200, 72, seed=1, scale=0.1), "up_proj.weight": rand(200, 72, seed=2, scale=0.1),
         "down_proj.weight": rand(72, 200, seed=3, scale=0.1)}
    assert {k: v.shape for k, v in ff.param_specs().items()} == {k: tuple(v.shape) for k, v in t.items()}
    ff.load(t, ctx(dtype))
    x = rand(11, 72, seed=4).to(dtype)
    tw = {k: v.to(dtype).float() for k, v in t.items()}
    want = P.swiglu(x.float(), tw["gate_proj.weight"], tw["up_proj.weight"], tw["down_proj.weight"])
    torch.testing.assert_close(ff.forward(x.cuda()).cpu().float(), want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_in_portions(dtype, window):
    """The attention mixer alone, fed a sequence in three steps through a cache of its own."""
    from scratch_llm_b200.cache import CacheManager
    from scratch_llm_b200.engine.batch import BatchStager, RowInput, build_batch
    from scratch_llm_b200.parts import CacheView
    from scratch_llm_b200.parts.attention import GQAttention
    from scratch_llm_b200.parts.position import Rotary
    d, H, G, hd, S = 80, 6, 2, 16, 45
    att = GQAttention(d, H, G, hd, scale=0.2, window=window)
    # weights sized so that q, k, v and the output are of order 1, as in a trained model: the
    # bfloat16 tolerance is absolute
    t = {"q_proj.weight": rand(H * hd, d, seed=1, scale=0.1), "k_proj.weight": rand(G * hd, d, seed=2, scale=0.1),
         "v_proj.weight": rand(G * hd, d, seed=3, scale=0.1), "o_proj.weight": rand(d, H * hd, seed=4, scale=0.1)}
    att.load(t, ctx(dtype))
    rot = Rotary(hd, 1000.0, 64)
    rot.load({}, ctx(dtype))
    cache = CacheManager([att.kv_spec()], [None], page_size=4, n_pages=16, max_requests=2,
                         dtype=dtype, device="cuda")
    stager = BatchStager(torch.device("cuda"))
    x = rand(S, d, seed=5).to(dtype)
    cache.admit("r")
    outs = []
    for a, b in ((0, 20), (20, 22), (22, 45)):
        assert cache.reserve("r", b - a)
        batch = build_batch(cache, stager, [RowInput("r", [0] * (b - a))], 10, 64)
        pages, g = cache.entry_pages(0)
        view = CacheView(pages=pages, block_table=batch.block_tables[g], page_size=4)
        outs.append(att.forward(x[a:b].cuda(), batch, view, True, rot).cpu().float())
        cache.commit("r", b - a)
    got = torch.cat(outs)
    tw = {f"p.{k}": v.to(dtype).float() for k, v in t.items()}
    cfgd = dict(num_attention_heads=H, num_key_value_heads=G, head_dim=hd, hidden_size=d,
                sliding_window=window)
    cos, sin = P.rope_tables(hd, 64, 1000.0)
    # the plain layer divides by sqrt(hd); this part was given scale 0.2 = 0.8 / sqrt(16)
    want, _ = P.attention_layer(x.float(), torch.arange(S), {**tw, "p.q_proj.weight": tw["p.q_proj.weight"] * 0.8},
                                "p", cfgd, cos, sin)
    torch.testing.assert_close(got, want, **TOL[dtype])
    if window is not None:
        assert any(p < 0 for p in cache.table_of("r", 0))  # pages behind the window went back


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_part(dtype):
    """The pre-norm arrangement alone: x + Mixer(Norm(x)), then x + FeedForward(Norm(x)), with
    the last delta handed on as pending."""
    from scratch_llm_b200.cache import CacheManager
    from scratch_llm_b200.engine.batch import BatchStager, RowInput, build_batch
    from scratch_llm_b200.parts import BLOCKS, CacheView
    from scratch_llm_b200.parts.attention import GQAttention
    from scratch_llm_b200.parts.feed_forward import SwiGLU
    from scratch_llm_b200.parts.norm import RMSNorm
    from scratch_llm_b200.parts.position import Rotary
    d, H, G, hd, F, S, eps = 96, 4, 2, 16, 136, 21, 1e-4
    w = {"input_layernorm.weight": rand(d, seed=1) * 0.1 + 1,
         "post_attention_layernorm.weight": rand(d, seed=2) * 0.1 + 1,
         "self_attn.q_proj.weight": rand(H * hd, d, seed=3, scale=0.1),
         "self_attn.k_proj.weight": rand(G * hd, d, seed=4, scale=0.1),
         "self_attn.v_proj.weight": rand(G * hd, d, seed=5, scale=0.1),
         "self_attn.o_proj.weight": rand(d, H * hd, seed=6, scale=0.1),
         "mlp.gate_proj.weight": rand(F, d, seed=7, scale=0.1),
         "mlp.up_proj.weight": rand(F, d, seed=8, scale=0.1),
         "mlp.down_proj.weight": rand(d, F, seed=9, scale=0.1)}
    c = ctx(dtype)
    att = GQAttention(d, H, G, hd, scale=1 / math.sqrt(hd))
    att.load({k.split(".", 1)[1]: v for k, v in w.items() if k.startswith("self_attn")}, c)
    ff = SwiGLU(d, F)
    ff.load({k.split(".", 1)[1]: v for k, v in w.items() if k.startswith("mlp")}, c)
    n1, n2 = RMSNorm(d, eps), RMSNorm(d, eps)
    n1.load({"weight": w["input_layernorm.weight"]}, c)
    n2.load({"weight": w["post_attention_layernorm.weight"]}, c)
    rot = Rotary(hd, 10000.0, 64)
    rot.load({}, c)
    block = BLOCKS["pre_norm"](att, ff, n1, n2, rot)
    cache = CacheManager([att.kv_spec()], [None], 8, 8, 1, dtype=dtype, device="cuda")
    cache.admit("r")
    cache.reserve("r", S)
    batch = build_batch(cache, BatchStager(torch.device("cuda")), [RowInput("r", [0] * S)], 4, 64)
    pages, g = cache.entry_pages(0)
    x, pending_in = rand(S, d, seed=10), rand(S, d, seed=11, scale=0.3).to(dtype)
    resid = x.cuda()
    pending = block.forward(resid, pending_in.cuda(), batch,
                            CacheView(pages=pages, block_table=batch.block_tables[g], page_size=8), True)
    tw = {f"model.layers.0.{k}": v.to(dtype).float() for k, v in w.items()}
    cfgd = dict(num_attention_heads=H, num_key_value_heads=G, head_dim=hd, hidden_size=d, rms_norm_eps=eps)
    cos, sin = P.rope_tables(hd, 64, 10000.0)
    want, _ = P.block(x + pending_in.float(), torch.arange(S), tw, 0, cfgd, cos, sin)
    got = resid.cpu() + pending.cpu().float()     # the stream plus the delta still pending
    torch.testing.assert_close(got, want, **TOL[dtype])


# ----------------------------------------------------------------- a toy mixer with state

def make_toy():
    """A mixer whose output at token t is W applied to the running mean of the inputs up to t.
    Its state per request is (sum of inputs, count): fixed size, carried from step to step in
    the cache manager's state slots."""
    from scratch_llm_b200.config import LlamaConfig, register_architecture, ARCHITECTURES
    from scratch_llm_b200.config.spec import ModelSpec, PartSpec, Run, standard_layer as LayerSpec
    from scratch_llm_b200.parts import MIXERS, Mixer, StateSpec, register_mixer
    from scratch_llm_b200.weights import ParamSpec

    if "running_mean" not in MIXERS:
        @register_mixer("running_mean")
        class RunningMean(Mixer):
            def __init__(self, hidden_size):
                self.d = hidden_size

            def state_spec(self):
                return StateSpec((self.d + 1,), torch.float32)

            def param_specs(self):
                return {"mix.weight": ParamSpec((self.d, self.d))}

            def load(self, tensors, ctx):
                self.w = tensors["mix.weight"].to(ctx.device, torch.float32)
                self.dtype = ctx.dtype

            def forward(self, x, batch, cache, write, position):
                out = torch.empty_like(x)
                t = 0
                for n, slot in zip(batch.host_row_new, batch.row_slot.tolist()):
                    st = cache.state[slot]
                    sums = st[:self.d] + torch.cumsum(x[t:t + n].float(), 0)
                    counts = st[self.d] + torch.arange(1, n + 1, device=x.device)
                    out[t:t + n] = ((sums / counts[:, None]) @ self.w.T).to(x.dtype)
                    st[:self.d] = sums[-1]
                    st[self.d] = counts[-1]
                    t += n
                return out

    if "ToyStateForCausalLM" not in ARCHITECTURES:
        @dataclass(frozen=True)
        class ToyConfig:
            width: int
            n_vocab: int
            inner: int
            architecture = "ToyStateForCausalLM"

            @classmethod
            def from_dict(cls, raw):
                return cls(raw["width"], raw["n_vocab"], raw["inner"])

            def to_dict(self):
                return {"architectures": [self.architecture], "width": self.width,
                        "n_vocab": self.n_vocab, "inner": self.inner}

            def model_spec(self):
                d = self.width
                norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
                ff = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": self.inner})
                att = PartSpec("gqa_attention", {"hidden_size": d, "n_heads": 2, "n_kv_heads": 1,
                                                 "head_dim": 16, "scale": 0.25, "window": None})
                rot = PartSpec("rotary", {"head_dim": 16, "theta": 100.0, "max_position": 128})
                names = {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "n1",
                         "feed_forward_norm": "n2"}
                layers = (
                    LayerSpec("l0", "pre_norm", att, ff, norm, norm, rot, names),
                    LayerSpec("l1", "pre_norm", PartSpec("running_mean", {"hidden_size": d}), ff,
                              norm, norm, PartSpec("none"), names))
                # layer 0 runs twice: once with a cache of its own, once more reading it
                order = (Run(0, 0), Run(1, 1), Run(0, 0, write=False))
                return ModelSpec(d, self.n_vocab, 128, layers, order, norm, "emb.weight", "out_norm",
                                 "head.weight", tie_embeddings=True)

        register_architecture("ToyStateForCausalLM", ToyConfig)
    return ARCHITECTURES["ToyStateForCausalLM"].config_cls


def toy_plain(cfg, w, ids):
    d = cfg.width
    x = w["emb.weight"][torch.tensor(ids)]
    pos = torch.arange(len(ids))
    cos, sin = P.rope_tables(16, 128, 100.0)
    acfg = dict(num_attention_heads=2, num_key_value_heads=1, head_dim=16, hidden_size=d)

    def ffn(x, p):
        h = P.rmsnorm(x, w[f"{p}.n2.weight"], 1e-5)
        return x + P.swiglu(h, w[f"{p}.ff.gate_proj.weight"], w[f"{p}.ff.up_proj.weight"],
                            w[f"{p}.ff.down_proj.weight"])

    def attn(x, kv):
        a, kv = P.attention_layer(P.rmsnorm(x, w["l0.n1.weight"], 1e-5), pos, w, "l0.mixer", acfg,
                                  cos, sin, kv)
        return ffn(x + a, "l0"), kv
    x, kv = attn(x, None)
    h = P.rmsnorm(x, w["l1.n1.weight"], 1e-5)
    mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1)[:, None]
    x = ffn(x + mean @ w["l1.mixer.mix.weight"].T, "l1")
    x, _ = attn(x, kv)
    return P.rmsnorm(x, w["out_norm.weight"], 1e-5) @ w["emb.weight"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    import trace_util as T
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.weights import write_random_model
    Toy = make_toy()
    cfg = Toy(width=48, n_vocab=90, inner=100)
    d = write_random_model(cfg, tmp_path / "toy", seed=4, std=0.1, dtype="float32")
    _, w = P.read_model_dir(d)
    # the attention scale of the toy is 0.25 = 1/sqrt(16), the plain layer's own
    model = load_model(d, "float32", verbose=False)
    kv, st = model.cache_specs()
    assert kv[0] is not None and kv[1] is None and st[1] is not None and st[0] is None
    reqs = T.make_requests(90, [37, 5, 64, 20, 9], seed=2)
    want = {rid: toy_plain(cfg, w, toks) for rid, toks in reqs.items()}
    for way in (T.whole, T.changing_portions, T.mixed):
        steps = way(reqs)
        runner = ModelRunner(model, 8, -(-T.peak_tokens(steps) // 8), 4)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        for (rid, pos), row in got.items():
            torch.testing.assert_close(row, want[rid][pos], rtol=1e-4, atol=1e-5,
                                       msg=lambda m: f"{way.__name__} {rid} {pos}: {m}")


# ------------------------------- a toy feed-forward with routing, a toy position encoding

def make_toy_routed():
    """Two more parts defined here, outside the framework's files: a feed-forward that routes
    every token to the one of three small experts whose router logit (32-bit) is largest and
    weighs its output with the softmax probability of that logit; and a position encoding that
    is not rotary: it adds alpha * sin(position * 2^-j) to component j of every query and key
    head.  A model with one layer of each beside a standard layer."""
    from scratch_llm_b200.config import register_architecture, ARCHITECTURES
    from scratch_llm_b200.config.spec import ModelSpec, PartSpec, sequential_order, standard_layer as LayerSpec
    from scratch_llm_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward,
                                        PositionEncoding, register_feed_forward,
                                        register_position_encoding)
    from scratch_llm_b200.weights import ParamSpec

    if "top1_experts" not in FEED_FORWARDS:
        @register_feed_forward("top1_experts")
        class Top1Experts(FeedForward):
            def __init__(self, hidden_size, inner, n_experts):
                self.d, self.f, self.e = hidden_size, inner, n_experts

            def param_specs(self):
                return {"router.weight": ParamSpec((self.e, self.d)),
                        "w_in": ParamSpec((self.e * self.f, self.d)),
                        "w_out": ParamSpec((self.e * self.d, self.f))}

            def load(self, tensors, ctx):
                put = lambda t: t.to(ctx.device, torch.float32)  # noqa: E731
                self.router = put(tensors["router.weight"])
                self.w_in = put(tensors["w_in"]).view(self.e, self.f, self.d)
                self.w_out = put(tensors["w_out"]).view(self.e, self.d, self.f)

            def forward(self, x):
                xf = x.float()
                probs = torch.softmax(xf @ self.router.T, -1)      # router logits in 32-bit
                p, idx = probs.max(-1)
                h = torch.relu(torch.bmm(self.w_in[idx], xf[:, :, None]))
                return (torch.bmm(self.w_out[idx], h)[:, :, 0] * p[:, None]).to(x.dtype)

    if "added_sinusoid" not in POSITION_ENCODINGS:
        @register_position_encoding("added_sinusoid")
        class AddedSinusoid(PositionEncoding):
            def __init__(self, head_dim, alpha):
                self.hd, self.alpha = head_dim, float(alpha)

            def load(self, tensors, ctx):
                self.freq = (2.0 ** -torch.arange(self.hd, dtype=torch.float32)).to(ctx.device)

            def apply(self, q, k, positions):
                add = self.alpha * torch.sin(positions.float()[:, None] * self.freq)   # [n, hd]
                q += add[:, None, :].to(q.dtype)
                k += add[:, None, :].to(k.dtype)

    if "ToyRoutedForCausalLM" not in ARCHITECTURES:
        @dataclass(frozen=True)
        class ToyRoutedConfig:
            width: int
            n_vocab: int
            architecture = "ToyRoutedForCausalLM"

            @classmethod
            def from_dict(cls, raw):
                return cls(raw["width"], raw["n_vocab"])

            def to_dict(self):
                return {"architectures": [self.architecture], "width": self.width,
                        "n_vocab": self.n_vocab}

            def model_spec(self):
                d = self.width
                norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
                att = PartSpec("gqa_attention", {"hidden_size": d, "n_heads": 3, "n_kv_heads": 3,
                                                 "head_dim": 16, "scale": 0.25, "window": None})
                names = {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "n1",
                         "feed_forward_norm": "n2"}
                layers = (
                    LayerSpec("l0", "pre_norm", att,
                              PartSpec("top1_experts", {"hidden_size": d, "inner": 24, "n_experts": 3}),
                              norm, norm, PartSpec("added_sinusoid", {"head_dim": 16, "alpha": 0.5}),
                              names),
                    LayerSpec("l1", "pre_norm", att,
                              PartSpec("swiglu", {"hidden_size": d, "intermediate_size": 40}),
                              norm, norm,
                              PartSpec("rotary", {"head_dim": 16, "theta": 100.0, "max_position": 128}),
                              names))
                return ModelSpec(d, self.n_vocab, 128, layers, sequential_order(2), norm,
                                 "emb.weight", "out_norm", "head.weight", tie_embeddings=True)

        register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    return ARCHITECTURES["ToyRoutedForCausalLM"].config_cls


def toy_routed_plain(cfg, w, ids):
    d, hd, H = cfg.width, 16, 3
    x = w["emb.weight"][torch.tensor(ids)]
    s = len(ids)
    pos = torch.arange(s)
    heads = lambda t: t.view(s, H, hd).transpose(0, 1)  # noqa: E731
    # layer 0: attention with the added sinusoid, then the routed experts
    h = P.rmsnorm(x, w["l0.n1.weight"], 1e-5)
    add = 0.5 * torch.sin(pos.float()[:, None] * 2.0 ** -torch.arange(hd, dtype=torch.float32))
    q = heads(h @ w["l0.mixer.q_proj.weight"].T) + add
    k = heads(h @ w["l0.mixer.k_proj.weight"].T) + add
    v = heads(h @ w["l0.mixer.v_proj.weight"].T)
    a = P.attention(q, k, v, pos, pos, 0.25).transpose(0, 1).reshape(s, H * hd)
    x = x + a @ w["l0.mixer.o_proj.weight"].T
    h = P.rmsnorm(x, w["l0.n2.weight"], 1e-5)
    probs = torch.softmax(h @ w["l0.ff.router.weight"].T, -1)
    w_in, w_out = w["l0.ff.w_in"].view(3, 24, d), w["l0.ff.w_out"].view(3, d, 24)
    out = torch.zeros_like(x)
    for t in range(s):
        e = int(probs[t].argmax())
        out[t] = (w_out[e] @ torch.relu(w_in[e] @ h[t])) * probs[t, e]
    x = x + out
    # layer 1: the standard layer
    cos, sin = P.rope_tables(hd, 128, 100.0)
    acfg = dict(num_attention_heads=H, num_key_value_heads=H, head_dim=hd, hidden_size=d)
    a, _ = P.attention_layer(P.rmsnorm(x, w["l1.n1.weight"], 1e-5), pos, w, "l1.mixer", acfg, cos, sin)
    x = x + a
    h = P.rmsnorm(x, w["l1.n2.weight"], 1e-5)
    x = x + P.swiglu(h, w["l1.ff.gate_proj.weight"], w["l1.ff.up_proj.weight"],
                     w["l1.ff.down_proj.weight"])
    return P.rmsnorm(x, w["out_norm.weight"], 1e-5) @ w["emb.weight"].T


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """A feed-forward with routing and a position encoding that is not rotary are registered
    from here, built by the framework from a configuration and stepped (whole prompts, portions
    of changing size, mixed batches with reused pages, and captured decode steps) without a
    change to the framework's files."""
    import trace_util as T
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.weights import write_random_model
    Toy = make_toy_routed()
    cfg = Toy(width=36, n_vocab=70)
    d = write_random_model(cfg, tmp_path / "toy_routed", seed=6, std=0.15, dtype="float32")
    _, w = P.read_model_dir(d)
    model = load_model(d, "float32", verbose=False)
    reqs = T.make_requests(70, [37, 5, 64, 20, 9], seed=3)
    want = {rid: toy_routed_plain(cfg, w, toks) for rid, toks in reqs.items()}
    # the router's choices are not all the same: the test would else say little
    h = torch.randn(50, 36)
    assert len(set((h @ w["l0.ff.router.weight"].T).argmax(-1).tolist())) > 1
    for way in (T.whole, T.tail_one_by_one, T.changing_portions, T.mixed):
        steps = way(reqs)
        runner = ModelRunner(model, 8, -(-T.peak_tokens(steps) // 8), 4)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        for (rid, pos), row in got.items():
            torch.testing.assert_close(row, want[rid][pos], rtol=1e-4, atol=2e-5,
                                       msg=lambda m: f"{way.__name__} {rid} {pos}: {m}")


# --------------------------------------- a toy norm and a toy arrangement of a layer's parts

def make_toy_parallel():
    """Two more parts defined here: a norm that centres before it scales (mean and variance in
    32-bit, no bias), and a block that gives ONE normed copy of the stream to mixer and
    feed-forward side by side, x + Mixer(Norm(x)) + FeedForward(Norm(x)).  A model with such
    a layer before a standard one, and the toy norm before the output matrix."""
    from scratch_llm_b200.config import register_architecture, ARCHITECTURES
    from scratch_llm_b200.config.spec import ModelSpec, PartSpec, sequential_order, standard_layer as LayerSpec
    from scratch_llm_b200.config.spec import LayerSpec as RolesLayerSpec
    from scratch_llm_b200.parts import BLOCKS, NORMS, Block, Norm, register_block, register_norm
    from scratch_llm_b200.weights import ParamSpec

    if "centred_norm" not in NORMS:
        @register_norm("centred_norm")
        class CentredNorm(Norm):
            def __init__(self, size, eps):
                self.size, self.eps = size, float(eps)

            def param_specs(self):
                return {"weight": ParamSpec((self.size,), "gain")}

            def load(self, tensors, ctx):
                self.weight = tensors["weight"].to(ctx.device, torch.float32)
                self.dtype = ctx.dtype

            def forward(self, resid, delta, out_rows=None):
                if out_rows is None:
                    if delta is not None:
                        resid += delta.float()      # the norm owns the add into the stream
                    x = resid
                else:                               # the gathered final norm: stream untouched
                    x = resid[out_rows.long()]
                    if delta is not None:
                        x = x + delta[out_rows.long()].float()
                mu = x.mean(-1, keepdim=True)
                var = ((x - mu) ** 2).mean(-1, keepdim=True)
                return ((x - mu) * torch.rsqrt(var + self.eps) * self.weight).to(self.dtype)

    if "parallel" not in BLOCKS:
        @register_block("parallel")
        class ParallelBlock(Block):
            # other roles than the standard arrangement's: ONE norm feeds both branches
            ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm",
                     "position": "position"}
            pad_safe = True

            def __init__(self, mixer, feed_forward, norm, position):
                self.mixer, self.feed_forward = mixer, feed_forward
                self.norm, self.position = norm, position

            def forward(self, resid, pending, batch, cache, write):
                h = self.norm.forward(resid, pending)
                return self.mixer.forward(h, batch, cache, write, self.position) + \
                    self.feed_forward.forward(h)

    if "ToyParallelForCausalLM" not in ARCHITECTURES:
        @dataclass(frozen=True)
        class ToyParallelConfig:
            width: int
            n_vocab: int
            architecture = "ToyParallelForCausalLM"

            @classmethod
            def from_dict(cls, raw):
                return cls(raw["width"], raw["n_vocab"])

            def to_dict(self):
                return {"architectures": [self.architecture], "width": self.width,
                        "n_vocab": self.n_vocab}

            def model_spec(self):
                d = self.width
                rms = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
                centred = PartSpec("centred_norm", {"size": d, "eps": 1e-4})
                att = PartSpec("gqa_attention", {"hidden_size": d, "n_heads": 4, "n_kv_heads": 2,
                                                 "head_dim": 16, "scale": 0.25, "window": None})
                ff = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": 56})
                rope = PartSpec("rotary", {"head_dim": 16, "theta": 1000.0, "max_position": 128})
                names = {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "n1",
                         "feed_forward_norm": "n2"}
                layers = (RolesLayerSpec("l0", "parallel",
                                         {"mixer": att, "feed_forward": ff, "norm": centred,
                                          "position": rope},
                                         {"feed_forward": "ff", "norm": "n1"}),
                          LayerSpec("l1", "pre_norm", att, ff, rms, rms, rope, names))
                return ModelSpec(d, self.n_vocab, 128, layers, sequential_order(2), centred,
                                 "emb.weight", "out_norm", "head.weight", tie_embeddings=False)

        register_architecture("ToyParallelForCausalLM", ToyParallelConfig)
    return ARCHITECTURES["ToyParallelForCausalLM"].config_cls


def toy_parallel_plain(cfg, w, ids):
    d, hd, H, G = cfg.width, 16, 4, 2
    x = w["emb.weight"][torch.tensor(ids)]
    pos = torch.arange(len(ids))
    cos, sin = P.rope_tables(hd, 128, 1000.0)
    acfg = dict(num_attention_heads=H, num_key_value_heads=G, head_dim=hd, hidden_size=d)

    def centred(x, weight, eps=1e-4):
        mu = x.mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(((x - mu) ** 2).mean(-1, keepdim=True) + eps) * weight

    h = centred(x, w["l0.n1.weight"])
    a, _ = P.attention_layer(h, pos, w, "l0.mixer", acfg, cos, sin)
    x = x + a + P.swiglu(h, w["l0.ff.gate_proj.weight"], w["l0.ff.up_proj.weight"],
                         w["l0.ff.down_proj.weight"])
    a, _ = P.attention_layer(P.rmsnorm(x, w["l1.n1.weight"], 1e-5), pos, w, "l1.mixer", acfg, cos, sin)
    x = x + a
    x = x + P.swiglu(P.rmsnorm(x, w["l1.n2.weight"], 1e-5), w["l1.ff.gate_proj.weight"],
                     w["l1.ff.up_proj.weight"], w["l1.ff.down_proj.weight"])
    return centred(x, w["out_norm.weight"]) @ w["head.weight"].T


@pytest.mark.parametrize("dtype, tol", [("float32", dict(rtol=1e-4, atol=2e-5)),
                                        ("bfloat16", dict(rtol=3e-2, atol=3e-2))])
def test_toy_norm_and_another_arrangement_of_a_layer(dtype, tol, tmp_path):
    """A norm and a block arrangement are registered from here, built by the framework from a
    configuration and stepped in every way of cutting (with captured decode steps and, the
    parts being the framework's own attention and feed-forward, padded small steps) without a
    change to the framework's files."""
    import trace_util as T
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.weights import write_random_model
    Toy = make_toy_parallel()
    cfg = Toy(width=40, n_vocab=90)
    d = write_random_model(cfg, tmp_path / "toy_parallel", seed=9, std=0.15, dtype="float32")
    _, w = P.read_model_dir(d)
    if dtype == "bfloat16":
        w = {k: (v if k.endswith(("n1.weight", "n2.weight", "out_norm.weight"))
                 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    model = load_model(d, dtype, verbose=False)
    reqs = T.make_requests(90, [33, 6, 64, 21, 10], seed=5)
    want = {rid: toy_parallel_plain(cfg, w, toks) for rid, toks in reqs.items()}
    for way in (T.whole, T.tail_one_by_one, T.changing_portions, T.mixed):
        steps = way(reqs)
        runner = ModelRunner(model, 8, -(-T.peak_tokens(steps) // 8), 4)
        runner.capture_padded_after = 2
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        for (rid, pos), row in got.items():
            torch.testing.assert_close(row, want[rid][pos], **tol,
                                       msg=lambda m: f"{way.__name__} {rid} {pos}: {m}")


# ------------------------------ layers with different needs of the cache: a window and all keys

def make_toy_windowed():
    """An architecture of the framework's own parts whose first and third layer attend to the
    last 12 keys only while the second attends to all of them: two groups of cache entries with
    pages of their own, and pages of the windowed group go back while a request is live."""
    from scratch_llm_b200.config import register_architecture, ARCHITECTURES
    from scratch_llm_b200.config.spec import ModelSpec, PartSpec, sequential_order, standard_layer as LayerSpec

    if "ToyWindowedForCausalLM" not in ARCHITECTURES:
        @dataclass(frozen=True)
        class ToyWindowedConfig:
            width: int
            n_vocab: int
            window: int
            architecture = "ToyWindowedForCausalLM"

            @classmethod
            def from_dict(cls, raw):
                return cls(raw["width"], raw["n_vocab"], raw["window"])

            def to_dict(self):
                return {"architectures": [self.architecture], "width": self.width,
                        "n_vocab": self.n_vocab, "window": self.window}

            def model_spec(self):
                d = self.width
                norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
                att = lambda window: PartSpec("gqa_attention", {  # noqa: E731
                    "hidden_size": d, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "scale": 0.25,
                    "window": window})
                ff = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": 72})
                rope = PartSpec("rotary", {"head_dim": 16, "theta": 1000.0, "max_position": 256})
                names = {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "n1",
                         "feed_forward_norm": "n2"}
                layers = tuple(LayerSpec(f"l{i}", "pre_norm", att(w), ff, norm, norm, rope, names)
                               for i, w in enumerate((self.window, None, self.window)))
                return ModelSpec(d, self.n_vocab, 256, layers, sequential_order(3), norm,
                                 "emb.weight", "out_norm", "head.weight", tie_embeddings=True)

        register_architecture("ToyWindowedForCausalLM", ToyWindowedConfig)
    return ARCHITECTURES["ToyWindowedForCausalLM"].config_cls


def toy_windowed_plain(cfg, w, ids):
    d, hd = cfg.width, 16
    x = w["emb.weight"][torch.tensor(ids)]
    pos = torch.arange(len(ids))
    cos, sin = P.rope_tables(hd, 256, 1000.0)
    for i, window in enumerate((cfg.window, None, cfg.window)):
        acfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=hd, hidden_size=d,
                    sliding_window=window)
        a, _ = P.attention_layer(P.rmsnorm(x, w[f"l{i}.n1.weight"], 1e-5), pos, w, f"l{i}.mixer",
                                 acfg, cos, sin)
        x = x + a
        x = x + P.swiglu(P.rmsnorm(x, w[f"l{i}.n2.weight"], 1e-5), w[f"l{i}.ff.gate_proj.weight"],
                         w[f"l{i}.ff.up_proj.weight"], w[f"l{i}.ff.down_proj.weight"])
    return P.rmsnorm(x, w["out_norm.weight"], 1e-5) @ w["emb.weight"].T


@pytest.mark.parametrize("dtype, tol", [("float32", dict(rtol=1e-4, atol=2e-5)),
                                        ("bfloat16", dict(rtol=3e-2, atol=3e-2))])
def test_windowed_and_full_layers_share_a_model(dtype, tol, tmp_path):
    """Two groups of cache entries in one model (a window of 12 keys; all keys): every way of
    cutting gives the plain logits, the windowed group needs far fewer pages than the other,
    and its pages go back while requests are live."""
    import trace_util as T
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.weights import write_random_model
    Toy = make_toy_windowed()
    cfg = Toy(width=48, n_vocab=80, window=12)
    d = write_random_model(cfg, tmp_path / "toy_windowed", seed=12, std=0.08, dtype="float32")
    _, w = P.read_model_dir(d)
    if dtype == "bfloat16":
        w = {k: (v if k.endswith(("n1.weight", "n2.weight", "out_norm.weight"))
                 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    model = load_model(d, dtype, verbose=False)
    kv, _ = model.cache_specs()
    assert [s.window for s in kv] == [12, None, 12]
    reqs = T.make_requests(80, [40, 7, 100, 13, 64, 90], seed=8)
    want = {rid: toy_windowed_plain(cfg, w, toks) for rid, toks in reqs.items()}
    # the window's edge matters: with a window one key wider the logits move by far more
    # than the 32-bit tolerance (the 32-bit run is the one that would show such a fault)
    wider = toy_windowed_plain(Toy(width=48, n_vocab=80, window=13), w, reqs[list(reqs)[2]])
    assert float((wider - want[list(reqs)[2]]).abs().max()) > 20 * 2e-5
    for way in (T.whole, T.tail_one_by_one, T.changing_portions, T.mixed):
        steps = way(reqs)
        runner = ModelRunner(model, 8, -(-T.peak_tokens(steps) // 8), 4)
        runner.capture_padded_after = 2
        assert len(runner.cache.groups) == 2
        low = [g.pool.n_pages for g in runner.cache.groups]

        def watch():
            for i, g in enumerate(runner.cache.groups):
                low[i] = min(low[i], g.pool.n_free)

        with torch.no_grad():
            got = T.run_in_process(runner, steps, after_step=watch)
        used = [g.pool.n_pages - a for g, a in zip(runner.cache.groups, low)]
        windowed = [i for i, g in enumerate(runner.cache.groups) if g.spec.window][0]
        assert used[windowed] < used[1 - windowed]       # pages behind the window went back
        for (rid, pos), row in got.items():
            torch.testing.assert_close(row, want[rid][pos], **tol,
                                       msg=lambda m: f"{way.__name__} {rid} {pos}: {m}")
        assert not runner.cache.requests and all(
            g.pool.n_free == g.pool.n_pages for g in runner.cache.groups)


# --------------------------- the constants around the layers: embedding multiplier, logit cap

def make_toy_scaled():
    """An architecture of the framework's own parts that multiplies its embedded tokens, scales
    its logits and squashes them: the three constants a :class:`ModelSpec` has beside its
    layers."""
    from scratch_llm_b200.config import register_architecture, ARCHITECTURES
    from scratch_llm_b200.config.spec import ModelSpec, PartSpec, sequential_order, standard_layer

    if "ToyScaledForCausalLM" not in ARCHITECTURES:
        @dataclass(frozen=True)
        class ToyScaledConfig:
            width: int
            n_vocab: int
            multiplier: float
            logit_scale: float
            cap: float
            architecture = "ToyScaledForCausalLM"

            @classmethod
            def from_dict(cls, raw):
                return cls(raw["width"], raw["n_vocab"], raw["multiplier"], raw["logit_scale"],
                           raw["cap"])

            def to_dict(self):
                return {"architectures": [self.architecture], "width": self.width,
                        "n_vocab": self.n_vocab, "multiplier": self.multiplier,
                        "logit_scale": self.logit_scale, "cap": self.cap}

            def model_spec(self):
                d = self.width
                norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
                att = PartSpec("gqa_attention", {"hidden_size": d, "n_heads": 4, "n_kv_heads": 2,
                                                 "head_dim": 16, "scale": 0.25, "window": None})
                ff = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": 72})
                rope = PartSpec("rotary", {"head_dim": 16, "theta": 1000.0, "max_position": 256})
                names = {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "n1",
                         "feed_forward_norm": "n2"}
                layers = tuple(standard_layer(f"l{i}", "pre_norm", att, ff, norm, norm, rope, names)
                               for i in range(2))
                return ModelSpec(d, self.n_vocab, 256, layers, sequential_order(2), norm,
                                 "emb.weight", "out_norm", "head.weight", tie_embeddings=False,
                                 embedding_multiplier=self.multiplier,
                                 logit_scale=self.logit_scale, logit_softcap=self.cap)

        register_architecture("ToyScaledForCausalLM", ToyScaledConfig)
    return ARCHITECTURES["ToyScaledForCausalLM"].config_cls


def toy_scaled_plain(cfg, w, ids):
    d, hd = cfg.width, 16
    x = w["emb.weight"][torch.tensor(ids)] * cfg.multiplier
    pos = torch.arange(len(ids))
    cos, sin = P.rope_tables(hd, 256, 1000.0)
    for i in range(2):
        acfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=hd, hidden_size=d,
                    sliding_window=None)
        a, _ = P.attention_layer(P.rmsnorm(x, w[f"l{i}.n1.weight"], 1e-5), pos, w, f"l{i}.mixer",
                                 acfg, cos, sin)
        x = x + a
        x = x + P.swiglu(P.rmsnorm(x, w[f"l{i}.n2.weight"], 1e-5), w[f"l{i}.ff.gate_proj.weight"],
                         w[f"l{i}.ff.up_proj.weight"], w[f"l{i}.ff.down_proj.weight"])
    logits = P.rmsnorm(x, w["out_norm.weight"], 1e-5) @ w["head.weight"].T * cfg.logit_scale
    return cfg.cap * torch.tanh(logits / cfg.cap) if cfg.cap > 0 else logits


@pytest.mark.parametrize("cap", [0.0, 1.5])
@pytest.mark.parametrize("dtype, tol", [("float32", dict(rtol=1e-4, atol=2e-5)),
                                        ("bfloat16", dict(rtol=3e-2, atol=3e-2))])
def test_embedding_multiplier_and_logit_cap(dtype, tol, cap, tmp_path):
    """The constants a model has around its layers are the spec's, not the engine's: embedded
    tokens times a multiplier, logits times a scale and squashed by a tanh (or not)."""
    import trace_util as T
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.weights import write_random_model
    Toy = make_toy_scaled()
    cfg = Toy(width=48, n_vocab=80, multiplier=48 ** 0.5, logit_scale=3.0, cap=cap)
    d = write_random_model(cfg, tmp_path / "toy_scaled", seed=21, std=0.08, dtype="float32")
    _, w = P.read_model_dir(d)
    if dtype == "bfloat16":
        w = {k: (v if k.endswith(("n1.weight", "n2.weight", "out_norm.weight"))
                 else v.to(torch.bfloat16).float()) for k, v in w.items()}
    model = load_model(d, dtype, verbose=False)
    reqs = T.make_requests(80, [40, 7, 70], seed=9)
    want = {rid: toy_scaled_plain(cfg, w, toks) for rid, toks in reqs.items()}
    # each constant matters: without it the logits move by far more than the tolerance
    some = list(reqs)[0]
    for other in (Toy(48, 80, 1.0, 3.0, cap), Toy(48, 80, 48 ** 0.5, 1.0, cap),
                  Toy(48, 80, 48 ** 0.5, 3.0, 0.0 if cap else 1.5)):
        assert float((toy_scaled_plain(other, w, reqs[some]) - want[some]).abs().max()) > 0.1
    for way in (T.whole, T.tail_one_by_one, T.mixed):
        steps = way(reqs)
        runner = ModelRunner(model, 8, -(-T.peak_tokens(steps) // 8), 4)
        runner.capture_padded_after = 2
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        for (rid, pos), row in got.items():
            torch.testing.assert_close(row, want[rid][pos], **tol,
                                       msg=lambda m: f"{way.__name__} {rid} {pos}: {m}")
