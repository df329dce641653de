"""Each part alone against the plain functions, the layer schedule as data, and a toy mixer with
per-request state that is registered, built and stepped without touching the framework's files."""
from dataclasses import dataclass
from typing import ClassVar, List

import numpy as np
import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.double().flatten().cpu(), b.double().flatten().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


class Bench:
    """A cache manager, storage and step contexts for one part under test."""

    def __init__(self, needs, dtype, capacity=512, page=16):
        from ember_b200.cache.manager import CacheManager
        from ember_b200.cache.storage import CacheStorage
        from ember_b200.engine.batch import Workspace
        from ember_b200.parts import Runtime
        self.dev = torch.device("cuda:0")
        self.rt = Runtime(device=self.dev, dtype=dtype, page_tokens=page)
        self.cache = CacheManager(needs, page, capacity, 8)
        self.storage = CacheStorage(self.cache, self.dev, dtype)
        self.ws = Workspace(self.dev)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.dev)

    def ctx(self, runs, tile_sizes=()):
        """runs: list of (request, n_new_tokens)."""
        from ember_b200.engine.batch import StepContext, StepEntry, build_batch
        entries = []
        for rid, n in runs:
            if not self.cache.has(rid):
                rc = self.cache.admit(rid)
                self.storage.reset_slot(rc.slot)
            assert self.cache.ensure(rid, self.cache.get(rid).tokens + n)
            entries.append(StepEntry(rid, [0] * n, ()))
        batch = build_batch(entries, self.cache, 10)
        c = StepContext(batch, self.ws, self.dev, 256, err=self.err, tile_sizes=tile_sizes)
        for s, (rid, n) in enumerate(runs):
            self.cache.advance(rid, int(batch.context_len[s]))
        return c


def store_of(tensors):
    from ember_b200.weights import WeightStore
    return WeightStore.from_tensors(tensors)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from ember_b200.config import RMSNormSpec
    from ember_b200.parts import build_part
    b = Bench({}, dtype)
    for size, eps in ((96, 1e-5), (200, 1e-6)):
        w = (1 + 0.1 * torch.randn(size)).bfloat16()
        part = build_part("norm", RMSNormSpec(size=size, eps=eps), "n.")
        part.load(store_of({"n.weight": w}), b.rt)
        x = torch.randn(7, size, device=b.dev) * 2
        out = torch.empty(7, size, device=b.dev, dtype=dtype)
        part.forward(b.ctx([("r", 7)]), x, out, 7)
        want = plain.rmsnorm(x.cpu().double(), w.double(), eps)
        assert rel(out.float(), want) < (4e-3 if dtype == torch.bfloat16 else 1e-6)
        b.cache.release("r")


def test_rotary_part_table():
    from ember_b200.config import RotarySpec
    from ember_b200.parts import build_part
    from ember_b200.parts import Runtime
    rt = Runtime(device=torch.device("cuda:0"), dtype=torch.float32)
    for D, theta in ((16, 1e4), (32, 1e6), (128, 1e6)):
        part = build_part("position", RotarySpec(head_dim=D, rotary_dim=D, theta=theta))
        table, rotary = part.rotary_table(rt)
        assert rotary == D and torch.equal(table.cpu(), plain.rope_inv_freq(D, theta))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,inter", [(64, 192), (96, 200)])
def test_gated_mlp_part(dtype, hidden, inter):
    from ember_b200.config import GatedMLPSpec
    from ember_b200.parts import build_part
    b = Bench({}, dtype)
    g = (torch.randn(inter, hidden) * 0.1).bfloat16()
    u = (torch.randn(inter, hidden) * 0.1).bfloat16()
    d = (torch.randn(hidden, inter) * 0.1).bfloat16()
    part = build_part("feed_forward", GatedMLPSpec(hidden_size=hidden, intermediate_size=inter), "m.")
    part.load(store_of({"m.gate_proj.weight": g, "m.up_proj.weight": u, "m.down_proj.weight": d}), b.rt)
    x = torch.randn(256, hidden, device=b.dev).to(dtype)
    res0 = torch.randn(256, hidden, device=b.dev)
    res = res0.clone()
    part.forward(b.ctx([("r", 9)]), x, res)
    want = res0[:9].cpu().double() + plain.swiglu(x[:9].cpu().double(), g.double(), u.double(), d.double())
    assert rel(res[:9], want) < (6e-3 if dtype == torch.bfloat16 else 2e-6)
    assert torch.equal(res[9:], res0[9:])                      # rows beyond the step are untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,D,hidden,window,theta,eps", [(4, 2, 16, 64, 0, 1e4, 1e-6), (6, 1, 32, 96, 0, 1e6, 1e-5),
                                                                (4, 4, 64, 128, 23, 1e4, 1e-6), (8, 4, 128, 256, 0, 1e6, 1e-6)])
def test_attention_part_in_portions(dtype, heads, kv, D, hidden, window, theta, eps):
    """The attention mixer alone: a 90-token sequence fed as 40 + 3 + 1 + 46 next to another request."""
    from ember_b200.config import AttentionSpec, RotarySpec
    from ember_b200.parts import build_part
    spec = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=D, qk_norm=True, qk_norm_eps=eps,
                         window=window, position=RotarySpec(head_dim=D, rotary_dim=D, theta=theta))
    part = build_part("mixer", spec, "a.")
    torch.manual_seed(heads * D)
    w = {"a.q_proj.weight": torch.randn(heads * D, hidden) * 0.08, "a.k_proj.weight": torch.randn(kv * D, hidden) * 0.08,
         "a.v_proj.weight": torch.randn(kv * D, hidden) * 0.08, "a.o_proj.weight": torch.randn(hidden, heads * D) * 0.08,
         "a.q_norm.weight": 1 + 0.1 * torch.randn(D), "a.k_norm.weight": 1 + 0.1 * torch.randn(D)}
    w = {k: v.bfloat16() for k, v in w.items()}
    b = Bench({0: part.cache_need()}, dtype, capacity=512)
    part.load(store_of(w), b.rt)
    T = 90
    x_all = torch.randn(T, hidden).bfloat16()
    other = torch.randn(30, hidden).bfloat16()
    cfg = {"heads": heads, "kv_heads": kv, "head_dim": D, "eps": eps, "bias": False}
    want = plain.attention_block(x_all.double(), {k: v.double() for k, v in w.items()}, "a.", cfg, torch.arange(T),
                                 plain.rope_inv_freq(D, theta), window=window)
    got = torch.zeros(T, hidden)
    at, oat = 0, 0
    for n, m in ((40, 7), (3, 1), (1, 1), (46, 21)):           # the other request takes portions and single tokens too
        ctx = b.ctx([("x", n), ("o", m)], tile_sizes=part.tile_requests())
        x = torch.zeros(256, hidden, device=b.dev, dtype=dtype)
        x[:n] = x_all[at:at + n].to(dtype)
        x[n:n + m] = other[oat:oat + m].to(dtype)
        res = torch.zeros(256, hidden, device=b.dev)
        part.forward(ctx, x, res, b.storage.layer(0))
        got[at:at + n] = res[:n].cpu()
        at, oat = at + n, oat + m
    assert int(b.err.item()) == 0
    assert rel(got, want) < (1.5e-2 if dtype == torch.bfloat16 else 3e-6)
    if window:                                                  # the window's pages were given back on the way
        assert sum(p >= 0 for p in b.cache.get("x").tables[0]) <= (window + 15) // 16 + 1


def test_schedule_as_data_layer_twice_reading_another_cache(tiny_model_dirs):
    """Run order [0, 1, 0 again reading layer 1's cache]: whole and in portions agree."""
    from dataclasses import replace
    from ember_b200 import StepEntry
    from ember_b200.config import ScheduleEntry, load_config
    from ember_b200.engine.runner import ModelRunner
    from ember_b200.weights import WeightStore
    spec = load_config(tiny_model_dirs["a"]).to_model_spec()
    spec = replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=1)))
    toks = np.random.default_rng(1).integers(0, 512, size=50).tolist()

    def run(portions):
        r = ModelRunner(spec, WeightStore.from_dir(tiny_model_dirs["a"]), dtype="float32", capacity_tokens=128,
                        max_batch_tokens=128, max_requests=2)
        assert sorted(r.cache.layer_group) == [0, 1]            # layers 0 and 1 own caches; the third run borrows
        r.admit("s")
        out, at = [], 0
        for n in portions:
            r.reserve("s", n)
            out.append(r.step([StepEntry("s", toks[at:at + n], tuple(range(n)))]).cpu().clone())
            at += n
        return torch.cat(out)

    whole, cut = run([50]), run([17, 2, 30, 1])
    assert rel(cut, whole) < 2e-5
    base = ModelRunner(load_config(tiny_model_dirs["a"]).to_model_spec(), WeightStore.from_dir(tiny_model_dirs["a"]),
                       dtype="float32", capacity_tokens=128, max_batch_tokens=128, max_requests=2)
    base.admit("s"), base.reserve("s", 50)
    plain_two = base.step([StepEntry("s", toks, tuple(range(50)))]).cpu()
    assert rel(whole, plain_two) > 1e-3                         # the extra run really ran


# ------------------------------------------------------------------ a toy mixer with state of its own
@dataclass(frozen=True)
class RunningMeanSpec:
    """out_t = W . mean(x_0..x_t): needs the sum of everything before the step, per request."""
    kind: ClassVar[str] = "toy_running_mean"
    hidden_size: int = 0


def make_running_mean():
    from ember_b200.parts import CacheNeed, Mixer, WeightDecl

    class RunningMean(Mixer):
        def weight_decls(self) -> List:
            h = self.spec.hidden_size
            return [WeightDecl(self.prefix + "mix.weight", (h, h))]

        def load(self, store, rt):
            h = self.spec.hidden_size
            self.w = store.take(self.prefix + "mix.weight", (h, h)).to(rt.device, torch.float32)

        def cache_need(self):
            return CacheNeed(kind="state", state_shape=(self.spec.hidden_size,), state_dtype="float32")

        def forward(self, ctx, x, residual, cache, owns_cache=True):
            qs = ctx.query_start_host
            for s in range(ctx.S):                              # a test part may use torch; the product path does not
                a, b = int(qs[s]), int(qs[s + 1])
                slot = int(ctx.state_slots_host[s])
                cs = cache.state[slot] + torch.cumsum(x[a:b].float(), dim=0)
                cache.state[slot] = cs[-1]
                mean = cs / (ctx.positions[a:b].float() + 1)[:, None]
                residual[a:b] += mean @ self.w.t()

    return RunningMean


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from ember_b200 import StepEntry
    from ember_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec,
                                   default_schedule)
    from ember_b200.engine.runner import ModelRunner
    from ember_b200.parts import register_part
    from ember_b200.weights import WeightStore, random_tensors
    register_part("mixer", "toy_running_mean", make_running_mean())
    H, V = 48, 300
    norm = RMSNormSpec(size=H, eps=1e-6)
    attn = AttentionSpec(hidden_size=H, num_heads=3, num_kv_heads=1, head_dim=16, qk_norm=True, window=20,
                         position=RotarySpec(head_dim=16, rotary_dim=16, theta=1e4))
    mlp = GatedMLPSpec(hidden_size=H, intermediate_size=80)

    def layer(i, mixer):
        p = f"toy.layers.{i}."
        return LayerSpec.prenorm(mixer=mixer, feed_forward=mlp, mixer_norm=norm, feed_forward_norm=norm, mixer_prefix=p + "mixer.",
                         feed_forward_prefix=p + "mlp.", mixer_norm_prefix=p + "norm_a.", feed_forward_norm_prefix=p + "norm_b.")

    spec = ModelSpec(architecture="ToyForCausalLM", vocab_size=V, hidden_size=H,
                     layers=(layer(0, RunningMeanSpec(hidden_size=H)), layer(1, attn), layer(2, RunningMeanSpec(hidden_size=H))),
                     schedule=default_schedule(3), final_norm=norm, final_norm_prefix="toy.norm.",
                     embedding_name="toy.embed.weight", head_name="toy.head.weight", tie_embeddings=True, max_positions=512)
    weights = dict(random_tensors(spec, seed=4, dtype=torch.float32))
    assert "toy.layers.2.mixer.mix.weight" in weights           # the toy part's tensor was declared and made

    def runner():
        r = ModelRunner(spec, WeightStore.from_tensors(weights), dtype="float32", capacity_tokens=256,
                        max_batch_tokens=128, max_requests=4)
        kinds = [(g.need.kind, g.layers) for g in r.cache.groups]
        assert kinds == [("state", [0, 2]), ("window", [1])]    # groups by need: state slots and window pages
        return r

    rng = np.random.default_rng(7)
    a, b = rng.integers(0, V, size=70).tolist(), rng.integers(0, V, size=33).tolist()
    r = runner()
    r.admit("a"), r.reserve("a", 70)
    whole = r.step([StepEntry("a", a, tuple(range(70)))]).cpu().clone()
    r.release("a")
    # in portions, next to another request, in a slot that was used before (and is zeroed at admission)
    r.admit("b"), r.admit("a")
    got, at, bt = [], 0, 0
    for n, m in ((9, 5), (1, 1), (30, 20), (2, 1), (28, 6)):
        r.reserve("a", n), r.reserve("b", m)
        lg = r.step([StepEntry("b", b[bt:bt + m], ()), StepEntry("a", a[at:at + n], tuple(range(n)))])
        got.append(lg.cpu().clone())
        at, bt = at + n, bt + m
    assert rel(torch.cat(got), whole) < 2e-5
    assert r.cache.check() == ""
    assert not torch.isnan(whole).any() and whole.abs().max() > 0


# ------------------------------------- a toy feed-forward with routing and a toy position encoding
@dataclass(frozen=True)
class RoutedSpec:
    """Two experts, each y = W2 . relu(W1 . x); a token goes to the expert with the larger fp32 router logit."""
    kind: ClassVar[str] = "toy_top1_of_2"
    hidden_size: int = 0
    expert_size: int = 0


@dataclass(frozen=True)
class LearnedPositionSpec:
    """h_t += table[position of t]: acts on the embedded tokens, not inside a mixer."""
    kind: ClassVar[str] = "toy_learned_positions"
    hidden_size: int = 0
    max_positions: int = 0


def make_toy_feed_forward_and_positions():
    from ember_b200.parts import FeedForward, PositionEncoding, WeightDecl

    class Routed(FeedForward):
        used = set()                                            # which experts any step chose (looked at by the test)

        def weight_decls(self):
            h, e, p = self.spec.hidden_size, self.spec.expert_size, self.prefix
            d = [WeightDecl(p + "router.weight", (2, h))]
            for i in range(2):
                d += [WeightDecl(p + f"experts.{i}.w1", (e, h)), WeightDecl(p + f"experts.{i}.w2", (h, e))]
            return d

        def load(self, store, rt):
            h, e, p = self.spec.hidden_size, self.spec.expert_size, self.prefix
            self.router = store.take(p + "router.weight", (2, h)).to(rt.device, torch.float32)
            self.w1 = [store.take(p + f"experts.{i}.w1", (e, h)).to(rt.device, torch.float32) for i in range(2)]
            self.w2 = [store.take(p + f"experts.{i}.w2", (h, e)).to(rt.device, torch.float32) for i in range(2)]

        def forward(self, ctx, x, residual):
            xs = x[:ctx.T].float()
            choice = (xs @ self.router.t()).argmax(dim=-1)      # router logits in fp32
            for i in range(2):
                rows = torch.nonzero(choice == i).flatten()
                if rows.numel():
                    Routed.used.add(i)
                    residual[rows] += torch.relu(xs[rows] @ self.w1[i].t()) @ self.w2[i].t()

    class LearnedPositions(PositionEncoding):
        def weight_decls(self):
            return [WeightDecl(self.prefix + "weight", (self.spec.max_positions, self.spec.hidden_size))]

        def load(self, store, rt):
            self.table = store.take(self.prefix + "weight", (self.spec.max_positions, self.spec.hidden_size)).to(
                rt.device, torch.float32)

        def on_embedding(self, ctx, h):
            h[:ctx.T] += self.table[ctx.positions.long()]

    return Routed, LearnedPositions


def test_toy_routed_feed_forward_and_learned_positions():
    """A feed-forward with routing and a position encoding on the embedding, both defined here, registered and
    run through the engine's model, step function and cache: portions and mixed batches equal the whole, and
    the whole equals a plain computation of the same model."""
    from ember_b200 import StepEntry
    from ember_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NoPositionSpec, RMSNormSpec,
                                   default_schedule)
    from ember_b200.engine.runner import ModelRunner
    from ember_b200.parts import register_part
    from ember_b200.weights import WeightStore, random_tensors
    Routed, LearnedPositions = make_toy_feed_forward_and_positions()
    register_part("feed_forward", "toy_top1_of_2", Routed)
    register_part("position", "toy_learned_positions", LearnedPositions)
    H, V, P = 64, 200, 160
    norm = RMSNormSpec(size=H, eps=1e-5)
    attn = AttentionSpec(hidden_size=H, num_heads=2, num_kv_heads=2, head_dim=32, qk_norm=False, position=NoPositionSpec())
    routed, dense = RoutedSpec(hidden_size=H, expert_size=40), GatedMLPSpec(hidden_size=H, intermediate_size=96)

    def layer(i, ff):
        p = f"toy.layers.{i}."
        return LayerSpec.prenorm(mixer=attn, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm, mixer_prefix=p + "attn.",
                         feed_forward_prefix=p + "ff.", mixer_norm_prefix=p + "norm_a.", feed_forward_norm_prefix=p + "norm_b.")

    spec = ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=V, hidden_size=H,
                     layers=(layer(0, routed), layer(1, dense), layer(2, routed)),   # feed-forwards differ by layer
                     schedule=default_schedule(3), final_norm=norm, final_norm_prefix="toy.norm.",
                     embedding_name="toy.embed.weight", head_name="toy.head.weight", tie_embeddings=True, max_positions=P,
                     embedding_position=LearnedPositionSpec(hidden_size=H, max_positions=P),
                     embedding_position_prefix="toy.positions.", init_std=0.2)
    weights = dict(random_tensors(spec, seed=9, dtype=torch.float32))
    assert {"toy.positions.weight", "toy.layers.0.ff.router.weight", "toy.layers.2.ff.experts.1.w2",
            "toy.layers.1.ff.gate_proj.weight"} <= set(weights)

    rng = np.random.default_rng(17)
    a, b = rng.integers(0, V, size=75).tolist(), rng.integers(0, V, size=31).tolist()
    r = ModelRunner(spec, WeightStore.from_tensors(weights), dtype="float32", capacity_tokens=256, max_batch_tokens=128,
                    max_requests=4)
    r.admit("a"), r.reserve("a", 75)
    whole = r.step([StepEntry("a", a, tuple(range(75)))]).cpu().clone()
    r.release("a")
    assert Routed.used == {0, 1}                                # both experts were chosen by some token
    r.admit("b"), r.admit("a")
    got, at, bt = [], 0, 0
    for n, m in ((11, 4), (1, 1), (40, 20), (2, 1), (21, 5)):
        r.reserve("a", n), r.reserve("b", m)
        got.append(r.step([StepEntry("b", b[bt:bt + m], ()), StepEntry("a", a[at:at + n], tuple(range(n)))]).cpu().clone())
        at, bt = at + n, bt + m
    assert rel(torch.cat(got), whole) < 2e-5

    # the same model, plainly: no rotation (the positions come from the table), full causal attention
    w = {k: v.double() for k, v in weights.items()}
    h = w["toy.embed.weight"][a] + w["toy.positions.weight"][:75]
    for i, ff in enumerate((routed, dense, routed)):
        p = f"toy.layers.{i}."
        x = plain.rmsnorm(h, w[p + "norm_a.weight"], 1e-5)
        q = (x @ w[p + "attn.q_proj.weight"].t()).view(75, 2, 32)
        k = (x @ w[p + "attn.k_proj.weight"].t()).view(75, 2, 32)
        v = (x @ w[p + "attn.v_proj.weight"].t()).view(75, 2, 32)
        s = torch.einsum("thd,uhd->htu", q, k) / 32 ** 0.5
        s = s.masked_fill(torch.triu(torch.ones(75, 75, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("htu,uhd->thd", torch.softmax(s, dim=-1), v).reshape(75, 64)
        h = h + o @ w[p + "attn.o_proj.weight"].t()
        x = plain.rmsnorm(h, w[p + "norm_b.weight"], 1e-5)
        if ff is dense:
            h = h + plain.swiglu(x, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
        else:
            choice = (x.float() @ w[p + "ff.router.weight"].float().t()).argmax(dim=-1)
            y = torch.zeros_like(h)
            for e in range(2):
                rows = choice == e
                y[rows] = torch.relu(x[rows] @ w[p + f"ff.experts.{e}.w1"].t()) @ w[p + f"ff.experts.{e}.w2"].t()
            h = h + y
    want = plain.rmsnorm(h, w["toy.norm.weight"], 1e-5) @ w["toy.embed.weight"].t()
    assert rel(whole, want) < 1e-4


# ------------------------------------------------- toy arrangements: four norms; two mixers in one layer
def make_toy_arrangements():
    from ember_b200.parts.block import Arrangement

    class Sandwich(Arrangement):
        """h += post_a(mixer(pre_a(h))); h += post_b(ffn(pre_b(h))): four norms a layer.  Mixers and feed-forwards
        add into the buffer they are given, so the block hands them a zeroed one and norms it before adding."""
        ROLES = {"pre_mixer_norm": "norm", "mixer": "mixer", "post_mixer_norm": "norm",
                 "pre_feed_forward_norm": "norm", "feed_forward": "feed_forward", "post_feed_forward_norm": "norm"}

        def forward(self, ctx, h, caches, owns_cache=True):
            p, T = self.parts, ctx.T
            x = ctx.buf("sandwich.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
            branch = ctx.buf("sandwich.branch", (ctx.max_tokens, h.shape[-1]), torch.float32)
            normed = ctx.buf("sandwich.branch_normed", (ctx.max_tokens, h.shape[-1]), torch.float32)
            for pre, inner, post in (("pre_mixer_norm", "mixer", "post_mixer_norm"),
                                     ("pre_feed_forward_norm", "feed_forward", "post_feed_forward_norm")):
                p[pre].forward(ctx, h, x, T)
                branch.zero_()
                if inner == "mixer":
                    p[inner].forward(ctx, x, branch, caches[""], owns_cache)
                else:
                    p[inner].forward(ctx, x, branch)
                p[post].forward(ctx, branch, normed, T)
                h[:T] += normed[:T]

    class TwoMixers(Arrangement):
        """h += attention(norm_a(h)); h += memory(norm_m(h)); h += ffn(norm_f(h)): two mixers with caches of
        different kinds (pages and a state slot) in one layer."""
        ROLES = {"attention_norm": "norm", "attention": "mixer", "memory_norm": "norm", "memory": "mixer",
                 "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

        def forward(self, ctx, h, caches, owns_cache=True):
            p, T = self.parts, ctx.T
            x = ctx.buf("two.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
            p["attention_norm"].forward(ctx, h, x, T)
            p["attention"].forward(ctx, x, h, caches["attention"], owns_cache)
            p["memory_norm"].forward(ctx, h, x, T)
            p["memory"].forward(ctx, x, h, caches["memory"], owns_cache)
            p["feed_forward_norm"].forward(ctx, h, x, T)
            p["feed_forward"].forward(ctx, x, h)

    return Sandwich, TwoMixers


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_arrangements_four_norms_and_two_mixers(dtype):
    """Arrangements defined here, registered without touching the framework's files: a layer with four norms, a
    layer with two mixers (attention with pages beside a running mean with a state slot) and a plain pre-norm
    layer in one model, which also scales its embedded tokens and its logits.  Whole equals portions beside
    another request; the scales do what their definitions say."""
    from dataclasses import replace
    from ember_b200 import StepEntry
    from ember_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, default_schedule
    from ember_b200.engine.runner import ModelRunner
    from ember_b200.parts import register_part
    from ember_b200.weights import WeightStore, random_tensors
    Sandwich, TwoMixers = make_toy_arrangements()
    register_part("arrangement", "toy_sandwich", Sandwich)
    register_part("arrangement", "toy_two_mixers", TwoMixers)
    register_part("mixer", "toy_running_mean", make_running_mean())
    H, V = 64, 211
    norm = RMSNormSpec(size=H, eps=1e-5)
    attn = AttentionSpec(hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16, qk_norm=True,
                         position=RotarySpec(head_dim=16, rotary_dim=16, theta=1e4))
    mlp = GatedMLPSpec(hidden_size=H, intermediate_size=72)
    mean = RunningMeanSpec(hidden_size=H)
    sandwich = LayerSpec("toy_sandwich", (("pre_mixer_norm", norm, "t.0.n1."), ("mixer", attn, "t.0.attn."),
                                          ("post_mixer_norm", norm, "t.0.n2."), ("pre_feed_forward_norm", norm, "t.0.n3."),
                                          ("feed_forward", mlp, "t.0.mlp."), ("post_feed_forward_norm", norm, "t.0.n4.")))
    two = LayerSpec("toy_two_mixers", (("attention_norm", norm, "t.1.na."), ("attention", attn, "t.1.attn."),
                                       ("memory_norm", norm, "t.1.nm."), ("memory", mean, "t.1.mem."),
                                       ("feed_forward_norm", norm, "t.1.nf."), ("feed_forward", mlp, "t.1.mlp.")))
    pre = LayerSpec.prenorm(mixer=attn, feed_forward=mlp, mixer_norm=norm, feed_forward_norm=norm, mixer_prefix="t.2.attn.",
                            feed_forward_prefix="t.2.mlp.", mixer_norm_prefix="t.2.na.", feed_forward_norm_prefix="t.2.nf.")
    spec = ModelSpec(architecture="ToyArrangedForCausalLM", vocab_size=V, hidden_size=H, layers=(sandwich, two, pre),
                     schedule=default_schedule(3), final_norm=norm, final_norm_prefix="t.norm.", embedding_name="t.embed.weight",
                     head_name="t.head.weight", tie_embeddings=False, head_optional=False, max_positions=256,
                     embedding_multiplier=3.0, logit_scale=0.5, init_std=0.1)
    weights = dict(random_tensors(spec, seed=3, dtype=torch.float32))
    assert {"t.0.n4.weight", "t.1.mem.mix.weight", "t.1.attn.q_proj.weight", "t.2.na.weight"} <= set(weights)

    def runner(sp, w):
        return ModelRunner(sp, WeightStore.from_tensors(w), dtype=dtype, capacity_tokens=256, max_batch_tokens=128,
                           max_requests=4)

    r = runner(spec, weights)
    # the three attention mixers share one group of pages, the running mean has its slot: ids name (layer, sub-id)
    assert [(g.need.kind, g.layers) for g in r.cache.groups] == [("full", [0, (1, "attention"), 2]), ("state", [(1, "memory")])]
    rng = np.random.default_rng(5)
    a, b = rng.integers(0, V, size=66).tolist(), rng.integers(0, V, size=29).tolist()
    r.admit("a"), r.reserve("a", 66)
    whole = r.step([StepEntry("a", a, tuple(range(66)))]).float().cpu().clone()
    r.release("a")
    r.admit("b"), r.admit("a")
    got, at, bt = [], 0, 0
    for n, m in ((10, 6), (1, 1), (33, 12), (2, 1), (20, 9)):
        r.reserve("a", n), r.reserve("b", m)
        got.append(r.step([StepEntry("b", b[bt:bt + m], ()), StepEntry("a", a[at:at + n], tuple(range(n)))]).float().cpu().clone())
        at, bt = at + n, bt + m
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    assert rel(torch.cat(got), whole) < tol
    assert r.cache.check() == "" and not torch.isnan(whole).any() and whole.abs().max() > 0
    r.check_device()
    if dtype == "float32":
        # logit_scale: the logits halve; embedding_multiplier: the same as a table three times as large
        one = runner(replace(spec, logit_scale=1.0), weights)
        one.admit("a"), one.reserve("a", 66)
        assert rel(0.5 * one.step([StepEntry("a", a, tuple(range(66)))]).float().cpu(), whole) < 1e-6
        w3 = dict(weights)
        w3["t.embed.weight"] = weights["t.embed.weight"] * 3.0
        tab = runner(replace(spec, embedding_multiplier=1.0), w3)
        tab.admit("a"), tab.reserve("a", 66)
        assert rel(tab.step([StepEntry("a", a, tuple(range(66)))]).float().cpu(), whole) < 1e-6


def test_attention_refuses_a_group_the_kernels_do_not_take():
    """More query heads per key head than the general kernel's tile holds: refused when the part is built, with
    the limit the library itself reports."""
    from ember_b200 import ops
    from ember_b200.config import AttentionSpec, ConfigError
    from ember_b200.parts import build_part
    assert ops.attention_tile_queries(ops.ATTENTION_MAX_GROUP) >= 1
    with pytest.raises(ops.KernelError):
        ops.attention_tile_queries(ops.ATTENTION_MAX_GROUP + 1)
    build_part("mixer", AttentionSpec(hidden_size=64, num_heads=32, num_kv_heads=1, head_dim=16))
    with pytest.raises(ConfigError, match="at most 32"):
        build_part("mixer", AttentionSpec(hidden_size=64, num_heads=66, num_kv_heads=2, head_dim=16))
