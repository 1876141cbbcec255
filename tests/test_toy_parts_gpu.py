"""Generality of the parts: a toy architecture defined HERE -- a mixer with per-request state of its own, a
feed-forward with routing, attention without a position encoding and attention with a position encoding of the
test's own (half of each head rotated, frequencies in arithmetic steps), a norm of the test's own (mean removed
first, no weights), a schedule that runs a layer twice and lets a layer read another layer's cache -- is
registered, built from a folder, and stepped through the engine without any change to the framework's files.  It is compared with a plain computation written here.
It is a test fixture, not a model of anything.
"""
import numpy as np
import pytest
import torch

import traces
from plain_llama import attention, matvec_rows, read_folder, rmsnorm, rope_apply, swiglu

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyForCausalLM"], "vocab": 97, "width": 48, "heads": 4, "kv_heads": 2, "head_dim": 16,
       "inner": 72, "eps": 1e-5, "experts": 3, "state": 24, "rotary_dim": 8, "rotary_step": 3.0, "max_positions": 512}


def toy_inv_freq(rotary_dim, step):
    return (1.0 / (1.0 + np.float32(step) * np.arange(rotary_dim // 2, dtype=np.float32))).astype(np.float32)


def centred(x, eps):
    c = x.astype(np.float64) - x.astype(np.float64).mean(axis=-1, keepdims=True)
    return (c / np.sqrt((c * c).mean(axis=-1, keepdims=True) + np.float64(np.float32(eps)))).astype(np.float32)


def _define():
    """Parts and architecture of the toy model (defined inside a function so that importing this file on a
    machine without a GPU does nothing)."""
    from xyntetik_runner_b200.config.registry import register_architecture
    from xyntetik_runner_b200.engine.model import ModelPlan, ScheduleEntry
    from xyntetik_runner_b200.parts import (Embedding, FeedForward, GQAAttention, Head, Mixer, NoPosition, Norm,
                                            PositionEncoding, PreNormBlock, RMSNorm, Rotary, StateNeed, SwiGLU, make,
                                            register_feed_forward, register_mixer, register_norm, register_position)
    from xyntetik_runner_b200.weights.loader import TensorSpec

    class RunningSumMixer(Mixer):
        """out_t = W_out . (sum over i <= t of W_in . h_i): the sum is a state of fixed size per request."""

        def __init__(self, width, state, prefix):
            self.width, self.state, self.prefix = width, state, prefix

        def tensors(self):
            return {self.prefix + "in.weight": TensorSpec((self.state, self.width)),
                    self.prefix + "out.weight": TensorSpec((self.width, self.state))}

        def bind(self, tensors, rt):
            self.w_in = tensors[self.prefix + "in.weight"].float()
            self.w_out = tensors[self.prefix + "out.weight"].float()

        def state_need(self):
            return StateNeed((self.state,), torch.float32)

        def forward(self, ctx, h, x, lay):
            ctx.materialize(x)
            u = h.float() @ self.w_in.T
            for s in range(ctx.n_seg):
                a, n = int(ctx.host["seg_start"][s]), int(ctx.host["seg_len"][s])
                slot = int(ctx.host["seg_slot"][s])
                run = torch.cumsum(u[a:a + n], dim=0) + lay.state[slot]
                lay.state[slot] = run[-1]
                x[a:a + n] += run @ self.w_out.T

    class RoutedFF(FeedForward):
        """Each token goes to the one expert its router logit (float32) favours; experts are small SwiGLUs."""

        def __init__(self, width, inner, experts, prefix):
            self.width, self.inner, self.experts, self.prefix = width, inner, experts, prefix

        def tensors(self):
            t = {self.prefix + "router.weight": TensorSpec((self.experts, self.width))}
            for e in range(self.experts):
                t[f"{self.prefix}experts.{e}.gate_up.weight"] = TensorSpec((2 * self.inner, self.width))
                t[f"{self.prefix}experts.{e}.down.weight"] = TensorSpec((self.width, self.inner))
            return t

        def bind(self, tensors, rt):
            self.router = tensors[self.prefix + "router.weight"].float()
            self.gu = [tensors[f"{self.prefix}experts.{e}.gate_up.weight"].float() for e in range(self.experts)]
            self.dn = [tensors[f"{self.prefix}experts.{e}.down.weight"].float() for e in range(self.experts)]

        def forward(self, ctx, h, x):
            ctx.materialize(x)
            hf = h.float()
            choice = (hf @ self.router.T).argmax(dim=1)
            for e in range(self.experts):
                idx = (choice == e).nonzero().flatten()
                if idx.numel() == 0:
                    continue
                gu = hf[idx] @ self.gu[e].T
                g, u = gu[:, :self.inner], gu[:, self.inner:]
                x[idx] += (g / (1 + torch.exp(-g)) * u) @ self.dn[e].T

    class StepRotary(PositionEncoding):
        """A rotary encoding with laws of its own: only the first `rotary_dim` values of a head are rotated, and
        pair j turns at 1 / (1 + step * j) radians a position."""

        def __init__(self, rotary_dim, step):
            self.rotary_dim = rotary_dim
            self.inv_freq_host = toy_inv_freq(rotary_dim, step)
            self.inv_freq = None

        def prepare(self, rt):
            self.inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(rt.device)

        def rotary(self):
            return Rotary(self.rotary_dim, self.inv_freq)

    class CentredNorm(Norm):
        """out = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps): no weights, float32."""

        def __init__(self, width, eps):
            self.width, self.eps = width, float(eps)

        def tensors(self):
            return {}

        def bind(self, tensors, rt):
            pass

        def forward(self, ctx, x, out, rows=None):
            ctx.materialize(x)
            src = x if rows is None else x[rows.long()]
            c = src - src.mean(dim=1, keepdim=True)
            out[:src.shape[0]] = (c * torch.rsqrt((c * c).mean(dim=1, keepdim=True) + self.eps)).to(out.dtype)

    register_mixer("toy_running_sum", RunningSumMixer, replace=True)
    register_feed_forward("toy_routed", RoutedFF, replace=True)
    register_position("toy_step_rotary", StepRotary, replace=True)
    register_norm("toy_centred", CentredNorm, replace=True)

    class ToyConfig:
        def __init__(self, d):
            self.__dict__.update(d)
            self.architecture = d["architectures"][0]
            self.torch_dtype = d.get("torch_dtype", "float32")

    def build(c):
        emb = Embedding(c.vocab, c.width, "emb.weight")
        norm = lambda name: RMSNorm(c.width, c.eps, name)
        att0 = GQAAttention(c.width, c.heads, c.kv_heads, c.head_dim, NoPosition(), "l0.att.")
        att2 = GQAAttention(c.width, c.heads, c.kv_heads, c.head_dim,
                            make("position", "toy_step_rotary", rotary_dim=c.rotary_dim, step=c.rotary_step), "l2.att.", window=40)
        blocks = [
            PreNormBlock(norm("l0.n1"), att0, norm("l0.n2"), RoutedFF(c.width, c.inner, c.experts, "l0.ff.")),
            PreNormBlock(norm("l1.n1"), RunningSumMixer(c.width, c.state, "l1.mix."), make("norm", "toy_centred", width=c.width, eps=c.eps),
                         SwiGLU(c.width, c.inner, "l1.ff.")),
            PreNormBlock(norm("l2.n1"), att2, norm("l2.n2"), SwiGLU(c.width, c.inner, "l2.ff.")),
        ]
        schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0), ScheduleEntry(2, cache_from=2)]
        return ModelPlan(emb, blocks, schedule, norm("final.weight"), Head(c.vocab, c.width, tied_to=emb), c.width,
                         c.vocab, c.max_positions)

    register_architecture("ToyForCausalLM", ToyConfig, build, replace=True)
    return ToyConfig, build


def plain_toy(folder, ids):
    """The same model computed plainly: whole sequence, no cache, float64 sums."""
    cfg, w = read_folder(folder)
    T = len(ids)
    H, K, hd, d, F = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["width"], cfg["inner"]
    pos = np.arange(T)
    inv = toy_inv_freq(cfg["rotary_dim"], cfg["rotary_step"])        # rope_apply rotates the first 2 * len(inv) values of a head
    x = w["emb.weight"][np.asarray(ids)].astype(np.float32)

    def att(prefix, h, rope, window, kv_from=None):
        q = matvec_rows(h, w[prefix + "q_proj.weight"]).reshape(T, H, hd)
        src = h if kv_from is None else kv_from
        k = matvec_rows(src, w[prefix + "k_proj.weight"]).reshape(T, K, hd)
        v = matvec_rows(src, w[prefix + "v_proj.weight"]).reshape(T, K, hd)
        if rope:
            q, k = rope_apply(q, pos, inv), rope_apply(k, pos, inv)
        o = attention(q, k, v, 1.0 / np.sqrt(hd), window).reshape(T, H * hd)
        return matvec_rows(o, w[prefix + "o_proj.weight"])

    def routed(h):
        out = np.zeros((T, d), dtype=np.float64)
        choice = (h.astype(np.float64) @ w["l0.ff.router.weight"].astype(np.float64).T).argmax(axis=1)
        for t in range(T):
            e = int(choice[t])
            gu = matvec_rows(h[t:t + 1], w[f"l0.ff.experts.{e}.gate_up.weight"])
            out[t] = matvec_rows(swiglu(gu[:, :F], gu[:, F:]), w[f"l0.ff.experts.{e}.down.weight"])[0]
        return out.astype(np.float32)

    def ffn(prefix, h):
        return matvec_rows(swiglu(matvec_rows(h, w[prefix + "gate_proj.weight"]), matvec_rows(h, w[prefix + "up_proj.weight"])),
                           w[prefix + "down_proj.weight"])

    def block0(x):
        x = x + att("l0.att.", rmsnorm(x, w["l0.n1"], cfg["eps"]), False, None)
        return x + routed(rmsnorm(x, w["l0.n2"], cfg["eps"]))

    x = block0(x)
    h = rmsnorm(x, w["l1.n1"], cfg["eps"])
    run = np.cumsum(h.astype(np.float64) @ w["l1.mix.in.weight"].astype(np.float64).T, axis=0)
    x = x + (run @ w["l1.mix.out.weight"].astype(np.float64).T).astype(np.float32)
    x = x + ffn("l1.ff.", centred(x, cfg["eps"]))
    h2 = rmsnorm(x, w["l2.n1"], cfg["eps"])                     # the keys of schedule entry 2 come from here
    x = x + att("l2.att.", h2, True, 40)
    x = x + ffn("l2.ff.", rmsnorm(x, w["l2.n2"], cfg["eps"]))
    x = block0(x)                                               # layer 0 again (a cache entry of its own)
    h4 = rmsnorm(x, w["l2.n1"], cfg["eps"])
    x = x + att("l2.att.", h4, True, 40, kv_from=h2)            # layer 2 again, reading entry 2's keys and values
    x = x + ffn("l2.ff.", rmsnorm(x, w["l2.n2"], cfg["eps"]))
    return matvec_rows(rmsnorm(x, w["final.weight"], cfg["eps"]), w["emb.weight"])


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from xyntetik_runner_b200.weights.loader import write_model_folder
    ToyConfig, build = _define()
    path = str(tmp_path_factory.mktemp("toy"))
    specs = build(ToyConfig(TOY)).tensor_specs()
    write_model_folder(path, TOY, specs, seed=5, dtype=torch.float32, std=0.15, norm_jitter=0.1)
    return path


def test_toy_architecture_is_registered_built_and_stepped(toy_folder):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    reqs = {f"r{i}": traces.random_tokens(i, n, TOY["vocab"]) for i, n in enumerate((7, 45, 90, 31))}
    ref = {rid: plain_toy(toy_folder, t) for rid, t in reqs.items()}
    for cut in (traces.whole, traces.portions, lambda r: traces.mixed(r, seed=2, max_live=3)):
        steps = cut(reqs)
        eng = Engine(toy_folder, EngineParams(dtype="float32", max_tokens=traces.pool_tokens(steps, 8) + 64, page_size=8,
                                              max_requests=3))
        # two cache groups (all keys for layer 0's two entries, a window of 40 for layer 2) and one state array
        assert sorted(g.spec.window or 0 for g in eng.model.groups) == [0, 40]
        assert [g.n_layers for g in eng.model.groups] == [2, 1]
        assert [lay.writes_cache for lay in eng.model.layers] == [True, False, True, True, False]
        assert sum(lay.state is not None for lay in eng.model.layers) == 1
        got = traces.collect(steps, replay(eng, steps), TOY["vocab"])
        for rid in reqs:
            traces.assert_close(got[rid], ref[rid], "float32", f"toy/{rid}")
        eng.cache.audit()


def test_state_slot_is_zeroed_when_it_is_given_to_a_new_request(toy_folder):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams, StepEntry
    eng = Engine(toy_folder, EngineParams(dtype="float32", max_tokens=256, page_size=8, max_requests=1))
    a, b = traces.random_tokens(1, 20, TOY["vocab"]), traces.random_tokens(2, 20, TOY["vocab"])
    eng.step([StepEntry("a", a, [19])])
    eng.end("a")
    got = eng.step([StepEntry("b", b, list(range(20)))]).cpu().numpy()      # same slot, state from "a" must be gone
    eng.end("b")
    traces.assert_close(got, plain_toy(toy_folder, b), "float32", "slot reuse")


def test_unknown_part_kinds_are_refused():
    from xyntetik_runner_b200.parts import kinds, make
    _define()
    assert "toy_running_sum" in kinds("mixer") and "gqa_attention" in kinds("mixer") and "swiglu" in kinds("feed_forward")
    assert "toy_step_rotary" in kinds("position") and "rope" in kinds("position") and "toy_centred" in kinds("norm")
    with pytest.raises(ValueError, match="unknown mixer kind"):
        make("mixer", "nope")
    m = make("norm", "rmsnorm", width=8, eps=1e-5, name="n")
    assert m.width == 8


# ---------------------------------------------------------------------------------------------
# A second toy, for the parts that the first one does not reach: a block that runs mixer and feed-forward side by
# side from ONE norm (so a product whose sum is still pending on the residual stream meets other products cut along
# K), the built-in attention with an adjacent-pair rotation whose cosines and sines are scaled, an ungated GELU
# feed-forward and a gated GELU one -- all through ``Linear`` in bfloat16 at widths where the tensor-core product
# is cut along K and its sum deferred.  Block and architecture are defined here; nothing in the package changes.
# ---------------------------------------------------------------------------------------------
TOY2 = {"architectures": ["Toy2ForCausalLM"], "vocab": 131, "width": 1024, "heads": 16, "kv_heads": 4, "head_dim": 64,
        "inner": 1536, "eps": 1e-5, "theta": 777.0, "mscale": 0.9, "max_positions": 512, "torch_dtype": "bfloat16"}


def gelu_tanh(g):
    g = g.astype(np.float64)
    return (0.5 * g * (1.0 + np.tanh(0.7978845608 * (g + 0.044715 * g ** 3)))).astype(np.float32)


def _define2():
    from xyntetik_runner_b200.config.registry import register_architecture
    from xyntetik_runner_b200.engine.model import ModelPlan, ScheduleEntry
    from xyntetik_runner_b200.parts import (Block, Embedding, GQAAttention, Head, PreNormBlock, RMSNorm, make, register_block)

    class ParallelBlock(Block):
        """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, both parts read it, both add into the stream."""

        def __init__(self, norm, mixer, feed_forward):
            self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward

        graph_safe = True

        def parts(self):
            return (self.norm, self.mixer, self.feed_forward)

        def tensors(self):
            out = {}
            for p in self.parts():
                out.update(p.tensors())
            return out

        def bind(self, tensors, rt):
            for p in self.parts():
                p.bind(tensors, rt)

        def weight_bytes(self):
            return sum(p.weight_bytes() for p in self.parts())

        def forward(self, ctx, x, lay):
            h = ctx.buf("parallel_normed", (x.shape[0], x.shape[1]), ctx.act_dtype)
            self.norm.forward(ctx, x, h)
            self.mixer.forward(ctx, h, x, lay)          # leaves its last product's sum pending on x ...
            self.feed_forward.forward(ctx, h, x)        # ... while these products run, cut along K themselves

    register_block("toy_parallel", ParallelBlock, replace=True)

    class Toy2Config:
        def __init__(self, d):
            self.__dict__.update(d)
            self.architecture = d["architectures"][0]

    def build(c):
        emb = Embedding(c.vocab, c.width, "emb.weight")
        norm = lambda name: RMSNorm(c.width, c.eps, name)
        rope = lambda: make("position", "rope", head_dim=c.head_dim, theta=c.theta, pairing="adjacent", mscale=c.mscale)
        att = lambda p: GQAAttention(c.width, c.heads, c.kv_heads, c.head_dim, rope(), p)
        blocks = [
            make("block", "toy_parallel", norm=norm("l0.n"), mixer=att("l0.att."),
                 feed_forward=make("feed_forward", "mlp", width=c.width, inner=c.inner, prefix="l0.ff.", activation="gelu_tanh")),
            PreNormBlock(norm("l1.n1"), att("l1.att."), norm("l1.n2"),
                         make("feed_forward", "gated", width=c.width, inner=c.inner, prefix="l1.ff.", activation="gelu_tanh")),
        ]
        return ModelPlan(emb, blocks, [ScheduleEntry(0), ScheduleEntry(1)], norm("final.weight"),
                         Head(c.vocab, c.width, name="head.weight"), c.width, c.vocab, c.max_positions)

    register_architecture("Toy2ForCausalLM", Toy2Config, build, replace=True)
    return Toy2Config, build


def plain_toy2(folder, ids):
    from plain_llama import rope_inv_freq
    cfg, w = read_folder(folder)
    T = len(ids)
    H, K, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    pos = np.arange(T)
    inv = rope_inv_freq(cfg["theta"], hd)
    x = w["emb.weight"][np.asarray(ids)].astype(np.float32)

    def att(prefix, h):
        q = matvec_rows(h, w[prefix + "q_proj.weight"]).reshape(T, H, hd)
        k = matvec_rows(h, w[prefix + "k_proj.weight"]).reshape(T, K, hd)
        v = matvec_rows(h, w[prefix + "v_proj.weight"]).reshape(T, K, hd)
        q, k = rope_apply(q, pos, inv, True, cfg["mscale"]), rope_apply(k, pos, inv, True, cfg["mscale"])
        return matvec_rows(attention(q, k, v, 1.0 / np.sqrt(hd)).reshape(T, H * hd), w[prefix + "o_proj.weight"])

    h = rmsnorm(x, w["l0.n"], cfg["eps"])
    x = x + att("l0.att.", h) + matvec_rows(gelu_tanh(matvec_rows(h, w["l0.ff.up_proj.weight"])), w["l0.ff.down_proj.weight"])
    x = x + att("l1.att.", rmsnorm(x, w["l1.n1"], cfg["eps"]))
    h = rmsnorm(x, w["l1.n2"], cfg["eps"])
    gated = gelu_tanh(matvec_rows(h, w["l1.ff.gate_proj.weight"])) * matvec_rows(h, w["l1.ff.up_proj.weight"])
    x = x + matvec_rows(gated.astype(np.float32), w["l1.ff.down_proj.weight"])
    return matvec_rows(rmsnorm(x, w["final.weight"], cfg["eps"]), w["head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parallel_block_adjacent_rotation_and_gelu_feed_forwards(tmp_path, dtype):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    from xyntetik_runner_b200.parts import linear
    from xyntetik_runner_b200.weights.loader import write_model_folder
    Toy2Config, build = _define2()
    folder = str(tmp_path / "toy2")
    write_model_folder(folder, TOY2, build(Toy2Config(TOY2)).tensor_specs(), seed=6, dtype=torch.bfloat16, std=0.03,
                       norm_jitter=0.1, gen_device="cuda:0")
    reqs = {f"r{i}": traces.random_tokens(10 + i, n, TOY2["vocab"]) for i, n in enumerate((5, 40, 70))}
    ref = {rid: plain_toy2(folder, t) for rid, t in reqs.items()}
    before = dict(linear.counters)
    for cut in (traces.whole, lambda r: traces.tail_decoded(r, 12), lambda r: traces.mixed(r, seed=3, max_live=3)):
        steps = cut(reqs)
        eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=traces.pool_tokens(steps, 16) + 64, page_size=16, max_requests=3))
        got = traces.collect(steps, replay(eng, steps), TOY2["vocab"])
        for rid in reqs:
            traces.assert_close(got[rid], ref[rid], dtype, f"toy2/{dtype}/{rid}")
        eng.cache.audit()
        eng.check_status()
    if dtype == "bfloat16":
        # the serving path ran, and products were cut along K with their sums deferred (the parallel block then holds
        # one pending on the stream while the feed-forward's products run)
        assert linear.counters["tcgen05"] > before["tcgen05"] and linear.counters["deferred"] > before["deferred"] + 10
        from xyntetik_runner_b200 import kernels
        assert kernels.workspace(eng.device).live <= 1


def test_a_position_encoding_that_is_no_rotation_is_refused_by_name():
    from xyntetik_runner_b200.parts import GQAAttention, PositionEncoding, Runtime

    class ScoreBias(PositionEncoding):
        """(a bias on the scores by distance: not something the built-in mixer can apply)"""

    m = GQAAttention(64, 4, 2, 16, ScoreBias(), "a.")
    tensors = {f"a.{n}_proj.weight": torch.zeros(s, dtype=torch.float32, device="cuda") for n, s in
               (("q", (64, 64)), ("k", (32, 64)), ("v", (32, 64)), ("o", (64, 64)))}
    with pytest.raises(ValueError, match="ScoreBias"):
        m.bind(tensors, Runtime(torch.device("cuda:0"), torch.float32, 16, 64, 2))
