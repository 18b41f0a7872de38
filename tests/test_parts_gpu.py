"""Each part alone against the plain implementation's function for it, and models put together from
parts in ways GPT-2 does not use: grouped key/value heads, a window, a layer that runs twice, a
layer that reads another layer's cache, and a toy mixer with state of its own that is defined and
registered here, without a change to the library's files."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2
from conftest import TOL, random_ids, rel_error, run_batch
from ember_cpp_b200.cache import SequenceCache
from ember_cpp_b200.engine import Engine, Runtime, StepContext, StepPlan, build_step
from ember_cpp_b200.engine.engine import AppHandle
from ember_cpp_b200.parts import (Application, Block, DecoderModel, FeedForward, LayerSpec, Mixer, ModelSpec, PartSpec, Position,
                                  StateNeed, build_block,
                                  build_part, register_part)
from ember_cpp_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
PART_TOL = {"float32": 2e-5, "bfloat16": 3e-2}      # absolute, on outputs of order one


@pytest.fixture(scope="module")
def ops():
    from ember_cpp_b200.csrc.ops import CudaOps
    return CudaOps()


def f64(t):
    return t.detach().double().cpu().numpy()


def loaded(role, spec, runtime, seed=0, std=None):
    part = build_part(role, spec)
    tensors = random_tensors(part.weight_specs(), seed, torch.bfloat16)
    if std is not None:
        tensors = {k: (v.float() * std / 0.02).to(torch.bfloat16) if v.ndim == 2 else v for k, v in tensors.items()}
    part.load(tensors.__getitem__, runtime)
    return part, {k: f64(v) for k, v in tensors.items()}


def context(ops, runtime, part_or_model_needs, seq_lengths, position=None):
    """A cache, a step of whole prompts of the given lengths, and the context parts run in."""
    cache = SequenceCache(part_or_model_needs, [None] * len(part_or_model_needs), 1024, None, runtime.dtype, "cuda")
    slots = [cache.open() for _ in seq_lengths]
    cache.reserve(list(zip(slots, seq_lengths)))
    host = build_step([(s, [0] * n, []) for s, n in zip(slots, seq_lengths)], cache.lengths,
                      [g.table for g in cache.groups], cache.max_blocks)
    plan = StepPlan(host, torch.from_numpy(host.packed).cuda())
    apps = [AppHandle(i, i, cache.views[i], cache.writes[i], cache.states[i]) for i in range(len(part_or_model_needs))]
    return StepContext(ops, runtime.dtype, plan, apps, position or build_part("position", PartSpec("none")))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layernorm_part(ops, dtype):
    rt = Runtime(dtype, "cuda", ops)
    part, w = loaded("norm", PartSpec("layernorm", "ln.", {"width": 96, "eps": 1e-6}), rt)
    x = torch.randn(13, 96, generator=torch.Generator().manual_seed(1)).cuda() * 2 + 0.3
    got = part.forward(StepContext(ops, rt.dtype, None, [], None), x, rt.dtype)
    want = plain_gpt2.layer_norm(f64(x), w["ln.weight"], w["ln.bias"], 1e-6)
    assert got.dtype == rt.dtype and np.abs(f64(got) - want).max() < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("activation", ["gelu_tanh", "gelu_erf"])
def test_feed_forward_part(ops, dtype, activation):
    rt = Runtime(dtype, "cuda", ops)
    spec = PartSpec("dense", "mlp.", {"width": 96, "inner": 320, "activation": activation, "stored": "in_out"})
    part, w = loaded("ffn", spec, rt, std=0.1)
    g = torch.Generator().manual_seed(2)
    h, res = torch.randn(9, 96, generator=g).to(rt.dtype).cuda(), torch.randn(9, 96, generator=g).cuda()
    got = part.forward(StepContext(ops, rt.dtype, None, [], None), h, res.clone())
    want = f64(res) + plain_gpt2.mlp(f64(h), w["mlp.c_fc.weight"].T, w["mlp.c_fc.bias"], w["mlp.c_proj.weight"].T,
                                     w["mlp.c_proj.bias"], activation[5:])
    assert got.dtype == torch.float32 and np.abs(f64(got) - want).max() < PART_TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, hd, window, stored", [(3, 3, 32, 0, "in_out"), (6, 2, 16, 0, "out_in"),
                                                                 (4, 1, 48, 20, "in_out")])
def test_attention_part(ops, dtype, heads, kv_heads, hd, window, stored):
    rt = Runtime(dtype, "cuda", ops)
    width, scale = 72, 0.5 / math.sqrt(hd)
    spec = PartSpec("causal_attention", "attn.", {"width": width, "n_heads": heads, "kv_heads": kv_heads, "head_dim": hd,
                                                  "scale": scale, "window": window, "stored": stored})
    part, w = loaded("mixer", spec, rt, std=0.1)
    lengths = [37, 1, 70]
    ctx = context(ops, rt, [(part.cache_need(), None)], lengths)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(sum(lengths), width, generator=g).to(rt.dtype).cuda()
    res = torch.randn(sum(lengths), width, generator=g).cuda()
    got = f64(part.forward(ctx, h, res.clone(), ctx.apps[0]))
    t = (lambda a: a.T) if stored == "in_out" else (lambda a: a)
    at = 0
    for n in lengths:
        hh = f64(h[at:at + n])
        qkv = plain_gpt2.linear(hh, t(w["attn.c_attn.weight"]), w["attn.c_attn.bias"])
        q, k, v = plain_gpt2.split_qkv(qkv, heads, kv_heads, hd)
        a = plain_gpt2.attention(q, k, v, heads, kv_heads, hd, scale, window)
        want = f64(res[at:at + n]) + plain_gpt2.linear(a, t(w["attn.c_proj.weight"]), w["attn.c_proj.bias"])
        assert np.abs(got[at:at + n] - want).max() < PART_TOL[dtype]
        at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_part_and_embedding(ops, dtype):
    rt = Runtime(dtype, "cuda", ops)
    pos, w = loaded("position", PartSpec("learned_absolute", "wpe.", {"width": 40, "n_positions": 50}), rt)
    assert pos.max_positions() == 50 and build_part("position", PartSpec("none")).embedding_table() is None
    table = torch.randn(30, 40, generator=torch.Generator().manual_seed(4)).to(rt.dtype).cuda()
    tokens = torch.tensor([29, 0, 7], dtype=torch.int32).cuda()
    positions = torch.tensor([49, 0, 3], dtype=torch.int32).cuda()
    got = f64(ops.embed(tokens, positions, table, pos.embedding_table()))
    ids = tokens.tolist()
    for r, (i, p) in enumerate(zip(ids, positions.tolist())):
        want = plain_gpt2.position_embedding(plain_gpt2.token_embedding(f64(table), [i]), w["wpe.weight"], p)
        assert np.abs(got[r] - want[0]).max() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_arrangement(ops, dtype, tiny_folders, plains):
    """One pre-norm block of tiny B (its second layer, so that the per-layer scale shows)."""
    plain = plains["tiny_b"]
    rt = Runtime(dtype, "cuda", ops)
    from ember_cpp_b200.config import get_architecture, load_config
    spec = get_architecture("GPT2LMHeadModel").build_spec(load_config(tiny_folders["tiny_b"]))
    layer = spec.layers[1]
    block = build_block(layer.block, build_part("norm", layer.norm1), build_part("mixer", layer.mixer),
                        build_part("norm", layer.norm2), build_part("ffn", layer.ffn))
    from ember_cpp_b200.weights import read_folder
    stored = read_folder(tiny_folders["tiny_b"])
    for p in block.parts():
        p.load(stored.__getitem__, rt)
    lengths = [20, 64]
    ctx = context(ops, rt, [(block.mixer.cache_need(), None)], lengths)
    x = torch.randn(sum(lengths), 96, generator=torch.Generator().manual_seed(5)).cuda()
    got = f64(block.forward(ctx, x.clone(), ctx.apps[0]))
    assert np.abs(got[:20] - plain_gpt2.block(plain, 1, f64(x[:20]))).max() < PART_TOL[dtype]
    assert np.abs(got[20:] - plain_gpt2.block(plain, 1, f64(x[20:]))).max() < PART_TOL[dtype]


# ------------------------------------------------------------------------------ models GPT-2 is not
class ToyDecay(Mixer):
    """A mixer with state of its own and no cache: s <- decay * s + h W^T per token, output s.
    Its loop runs on the host, so an engine that holds it does not replay graphs."""
    graph_safe = False

    def __init__(self, prefix, width, decay):
        super().__init__(prefix)
        self.width, self.decay = width, decay

    def weight_specs(self):
        from ember_cpp_b200.parts import WeightSpec
        return [WeightSpec(self.prefix + "mix.weight", (self.width, self.width), std=0.05)]

    def load(self, get, runtime):
        self.w = runtime.matrix(get(self.prefix + "mix.weight"))

    def state_need(self):
        return StateNeed((self.width,), init=0.25)

    def forward(self, ctx, h, residual, app):
        u = ctx.ops.linear(h, self.w, None, out_dtype=ctx.dtype).float()
        plan = ctx.plan
        slots, cu = plan.seq_slot.tolist(), plan.cu_new.tolist()
        out = torch.empty_like(u)
        for i, slot in enumerate(slots):
            if slot < 0:
                continue
            s = app.state[slot]
            for t in range(cu[i], cu[i + 1]):
                s = self.decay * s + u[t]
                out[t] = s
            app.state[slot] = s
        return residual + out


class ToyRouted(FeedForward):
    """A feed-forward with routing: router logits in float32, the best expert of each token,
    weighted by its softmax probability; each expert a small GELU MLP.  Every expert runs on every
    token and the unchosen ones are zeroed (a toy: it shows the interface, not a fast kernel), so
    nothing goes to the host and the step still replays as a graph."""

    def __init__(self, prefix, width, inner, experts):
        super().__init__(prefix)
        self.width, self.inner, self.experts = width, inner, experts

    def weight_specs(self):
        from ember_cpp_b200.parts import WeightSpec
        specs = [WeightSpec(self.prefix + "router.weight", (self.experts, self.width), std=0.5)]
        for e in range(self.experts):
            specs += [WeightSpec(f"{self.prefix}e{e}.up.weight", (self.inner, self.width), std=0.08),
                      WeightSpec(f"{self.prefix}e{e}.down.weight", (self.width, self.inner), std=0.08)]
        return specs

    def load(self, get, runtime):
        self.router = get(self.prefix + "router.weight").to(runtime.device, torch.float32)
        self.up = [runtime.matrix(get(f"{self.prefix}e{e}.up.weight")) for e in range(self.experts)]
        self.down = [runtime.matrix(get(f"{self.prefix}e{e}.down.weight")) for e in range(self.experts)]

    def forward(self, ctx, h, residual):
        logits = h.float() @ self.router.t()                       # router logits in 32-bit
        prob = torch.softmax(logits, dim=-1)
        best = logits.argmax(dim=-1)
        out = residual
        for e in range(self.experts):
            u = ctx.ops.linear(h, self.up[e], None, act="gelu_tanh", out_dtype=ctx.dtype)
            y = ctx.ops.linear(u, self.down[e], None, out_dtype=torch.float32)
            gate = torch.where(best == e, prob[:, e], torch.zeros_like(prob[:, e]))
            out = out + gate[:, None] * y
        return out


class ToyRotary(Position):
    """Another position encoding: nothing is added to the embedding; the attention mixer's q and k
    are rotated in place, pair (2i, 2i+1) of every head by position * base^(-2i/head size), the
    angles in float32."""

    def __init__(self, prefix, base):
        super().__init__(prefix)
        self.base = base

    def apply_qk(self, ctx, qkv, n_heads, kv_heads, head_dim):
        pos = ctx.plan.positions[:qkv.shape[0]].float()
        inv = self.base ** (-torch.arange(0, head_dim, 2, device=qkv.device, dtype=torch.float32) / head_dim)
        ang = pos[:, None] * inv[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        rot = qkv[:, :(n_heads + kv_heads) * head_dim].view(qkv.shape[0], n_heads + kv_heads, head_dim // 2, 2).float()
        a, b = rot[..., 0], rot[..., 1]
        turned = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).to(qkv.dtype)
        qkv[:, :(n_heads + kv_heads) * head_dim] = turned.view(qkv.shape[0], -1)


def toy_spec(width, vocab, n_pos, mixers, schedule, eps=1e-5, rotary=None, experts=0):
    """mixers: per layer ("attn", heads, kv_heads, hd, window) or ("decay", decay)."""
    layers = []
    for i, m in enumerate(mixers):
        p = f"layers.{i}."
        if m[0] == "attn":
            _, heads, kv, hd, window = m
            mixer = PartSpec("causal_attention", p + "attn.", {"width": width, "n_heads": heads, "kv_heads": kv,
                                                               "head_dim": hd, "scale": 1 / math.sqrt(hd), "window": window,
                                                               "qkv": "qkv", "out": "o", "stored": "out_in",
                                                               "init_std": 0.08, "out_init_std": 0.08})
        else:
            mixer = PartSpec("toy_decay", p + "decay.", {"width": width, "decay": m[1]})
        if experts and i % 2 == 1:                 # every other layer routes: different feed-forwards in one model
            ffn = PartSpec("toy_routed", p + "moe.", {"width": width, "inner": width + 8, "experts": experts})
        else:
            ffn = PartSpec("dense", p + "ffn.", {"width": width, "inner": 2 * width + 8, "activation": "gelu_tanh",
                                                 "up": "up", "down": "down", "stored": "out_in", "init_std": 0.08,
                                                 "down_init_std": 0.08})
        layers.append(LayerSpec("pre_norm", PartSpec("layernorm", p + "n1.", {"width": width, "eps": eps}), mixer,
                                PartSpec("layernorm", p + "n2.", {"width": width, "eps": eps}), ffn))
    position = (PartSpec("toy_rotary", "", {"base": rotary}) if rotary
                else PartSpec("learned_absolute", "pos.", {"width": width, "n_positions": n_pos}))
    return ModelSpec(width=width, vocab_size=vocab, token_table="embed.weight",
                     position=position,
                     layers=tuple(layers), schedule=tuple(Application(*a) for a in schedule),
                     final_norm=PartSpec("layernorm", "norm.", {"width": width, "eps": eps}), head="head.weight",
                     table_init_std=0.3)


def plain_rotate(x, heads, hd, base):
    """Rows of [T, heads * hd]: pair (2i, 2i+1) of every head turned by position * base^(-2i/hd)."""
    T = x.shape[0]
    ang = np.arange(T)[:, None] * base ** (-np.arange(0, hd, 2) / hd)[None, :]
    v = x.reshape(T, heads, hd // 2, 2)
    a, b = v[..., 0], v[..., 1]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    return np.stack((a * c - b * s, a * s + b * c), axis=-1).reshape(T, heads * hd)


def toy_plain(spec, mixers, w, ids):
    """The toy model on a whole sequence, from the plain implementation's functions."""
    rotary = spec.position.params.get("base") if spec.position.kind == "toy_rotary" else None
    x = plain_gpt2.token_embedding(w["embed.weight"], ids)
    if rotary is None:
        x = plain_gpt2.position_embedding(x, w["pos.weight"])
    kv = {}
    for a, app in enumerate(spec.schedule):
        i, m, p = app.layer, mixers[app.layer], f"layers.{app.layer}."
        eps = spec.layers[i].norm1.params["eps"]
        h = plain_gpt2.layer_norm(x, w[p + "n1.weight"], w[p + "n1.bias"], eps)
        if m[0] == "attn":
            _, heads, kvh, hd, window = m
            qkv = plain_gpt2.linear(h, w[p + "attn.qkv.weight"], w[p + "attn.qkv.bias"])
            q, k, v = plain_gpt2.split_qkv(qkv, heads, kvh, hd)
            if rotary is not None:
                q, k = plain_rotate(q, heads, hd, rotary), plain_rotate(k, kvh, hd, rotary)
            kv[a] = (k, v)
            if app.cache_of is not None:
                k, v = kv[app.cache_of]
            att = plain_gpt2.attention(q, k, v, heads, kvh, hd, 1 / math.sqrt(hd), window)
            x = x + plain_gpt2.linear(att, w[p + "attn.o.weight"], w[p + "attn.o.bias"])
        else:
            u = h @ w[p + "decay.mix.weight"].T
            s = np.full(x.shape[1], 0.25)
            out = np.zeros_like(u)
            for t in range(len(ids)):
                s = m[1] * s + u[t]
                out[t] = s
            x = x + out
        h = plain_gpt2.layer_norm(x, w[p + "n2.weight"], w[p + "n2.bias"], eps)
        if spec.layers[i].ffn.kind == "toy_routed":
            logits = h @ w[p + "moe.router.weight"].T
            prob = np.exp(logits - logits.max(-1, keepdims=True))
            prob /= prob.sum(-1, keepdims=True)
            best = logits.argmax(-1)
            for t in range(len(ids)):
                e = int(best[t])
                u = plain_gpt2.gelu(h[t:t + 1] @ w[f"{p}moe.e{e}.up.weight"].T, "tanh")
                x[t] = x[t] + prob[t, e] * (u @ w[f"{p}moe.e{e}.down.weight"].T)[0]
            continue
        x = x + plain_gpt2.mlp(h, w[p + "ffn.up.weight"], w[p + "ffn.up.bias"], w[p + "ffn.down.weight"],
                               w[p + "ffn.down.bias"], "tanh")
    h = plain_gpt2.layer_norm(x, w["norm.weight"], w["norm.bias"], spec.final_norm.params["eps"])
    return h @ w["head.weight"].T


TOYS = {
    # grouped heads; a window layer beside full ones (two cache groups); layer 0 runs twice
    "groups_window_twice": (dict(width=80, vocab=300, n_pos=200),
                            [("attn", 10, 2, 16, 0), ("attn", 5, 5, 16, 24), ("attn", 4, 1, 32, 0)],
                            [(0,), (1,), (0,), (2,)]),
    # the last entry runs layer 1 again and reads the cache that entry 1 wrote
    "shared_cache": (dict(width=64, vocab=200, n_pos=160), [("attn", 4, 4, 16, 0), ("attn", 2, 2, 32, 0)],
                     [(0,), (1,), (0,), (1, 1)]),
    # a mixer with state of its own between attention layers, and run twice
    "state_of_its_own": (dict(width=48, vocab=150, n_pos=160), [("attn", 3, 3, 16, 0), ("decay", 0.8), ("attn", 3, 1, 16, 10)],
                         [(0,), (1,), (2,), (1,)]),
    # another position encoding (q and k rotated, no table: the context is bounded by the cache alone) and
    # a feed-forward with routing in every other layer
    "rotary_routed": (dict(width=64, vocab=180, n_pos=160, rotary=100.0, experts=3),
                      [("attn", 4, 2, 16, 0), ("attn", 2, 2, 32, 40), ("attn", 4, 4, 16, 0)], [(0,), (1,), (2,)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("toy", list(TOYS))
def test_toy_models_step_like_whole_sequences(ops, dtype, toy):
    register_part("mixer", "toy_decay", ToyDecay)            # parts of the test's own
    register_part("ffn", "toy_routed", ToyRouted)
    register_part("position", "toy_rotary", ToyRotary)
    sizes, mixers, schedule = TOYS[toy]
    spec = toy_spec(sizes["width"], sizes["vocab"], sizes["n_pos"], mixers, schedule, rotary=sizes.get("rotary"),
                    experts=sizes.get("experts", 0))
    tensors = random_tensors(DecoderModel(spec).weight_specs(), 3, torch.bfloat16)
    w = {k: f64(v) for k, v in tensors.items()}
    eng = Engine.from_spec(spec, tensors, dtype=dtype, max_tokens=1024, ops=ops)
    assert eng.cuda_graphs == (toy != "state_of_its_own")
    if toy == "groups_window_twice":
        assert len(eng.cache.groups) == 3 and sorted(len(g.apps) for g in eng.cache.groups) == [1, 1, 2]
    if toy == "shared_cache":
        assert eng.cache.views[3] is eng.cache.views[1] and not eng.apps[3].writes_cache
    if toy == "state_of_its_own":
        assert eng.apps[1].state is not None and eng.apps[3].state is not None
        assert eng.apps[1].state.data_ptr() != eng.apps[3].state.data_ptr()
    if toy == "rotary_routed":
        assert eng.model.max_positions() is None and len(eng.cache.groups) == 3
        assert [type(b.ffn).__name__ for b in eng.model.blocks] == ["DenseFeedForward", "ToyRouted", "DenseFeedForward"]
    tol = 1e-5 if dtype == "float32" else 2e-2
    seqs = [random_ids(i, sizes["vocab"], n) for i, n in enumerate((150, 33, 70))]
    if toy == "rotary_routed":
        # The best expert of a token is a discontinuous function of the activations: where two router logits
        # nearly tie, bfloat16 may choose the other expert and no tolerance covers that.  These sequences
        # were picked (from the plain implementation) so that every token's best two router logits are at
        # least 6 % of the logits' spread apart.
        seqs = [random_ids(seed, sizes["vocab"], n) for seed, n in ((271, 150), (26, 33), (110, 70))]
    for batch in ((40, 1, 70), (100, 20, 5)):                 # the second batch reuses slots and state rows
        rows, _ = run_batch(eng, seqs, batch)
        for ids, got in zip(seqs, rows):
            assert rel_error(got, toy_plain(spec, mixers, w, ids)) < tol
        eng.cache.check()
        assert eng.cache.slots.held == 0
        assert all(g.pages.free == g.pages.size for g in eng.cache.groups)


# ------------------------------------------------------------------------------ other arrangements, model-level options
class ToySandwich(Block):
    """Norms before and after the mixer and the feed-forward: x + post1(mixer(norm1(x))), then the same
    around the feed-forward.  The spec names the two further norms in `more_norms`."""

    def __init__(self, norm1, mixer, norm2, ffn, post1, post2):
        super().__init__(norm1, mixer, norm2, ffn, post1=post1, post2=post2)

    def forward(self, ctx, x, app):
        zero = torch.zeros_like(x)
        a = self.mixer.forward(ctx, self.norm1.forward(ctx, x, ctx.dtype), zero, app)
        x = x + self.more_norms["post1"].forward(ctx, a, torch.float32)
        f = self.ffn.forward(ctx, self.norm2.forward(ctx, x, ctx.dtype), torch.zeros_like(x))
        return x + self.more_norms["post2"].forward(ctx, f, torch.float32)


class ToyParallel(Block):
    """One norm shared by the mixer and the feed-forward, both branches added to the stream at once."""

    def __init__(self, norm1, mixer, norm2, ffn):
        assert norm2 is None
        super().__init__(norm1, mixer, None, ffn)

    def forward(self, ctx, x, app):
        h = self.norm1.forward(ctx, x, ctx.dtype)
        a = self.mixer.forward(ctx, h, torch.zeros_like(x), app)
        f = self.ffn.forward(ctx, h, torch.zeros_like(x))
        return x + a + f


class ToyCounter(Mixer):
    """A mixer with two state tensors of different types: a float32 running sum `s` <- decay * s + h W^T
    and an int32 count of the sequence's tokens; its output is s + 0.01 * count."""
    graph_safe = False

    def __init__(self, prefix, width, decay):
        super().__init__(prefix)
        self.width, self.decay = width, decay

    def weight_specs(self):
        from ember_cpp_b200.parts import WeightSpec
        return [WeightSpec(self.prefix + "mix.weight", (self.width, self.width), std=0.05)]

    def load(self, get, runtime):
        self.w = runtime.matrix(get(self.prefix + "mix.weight"))

    def state_need(self):
        return {"s": StateNeed((self.width,), init=0.5), "count": StateNeed((1,), init=0, dtype="int32")}

    def forward(self, ctx, h, residual, app):
        u = ctx.ops.linear(h, self.w, None, out_dtype=ctx.dtype).float()
        slots, cu = ctx.plan.seq_slot.tolist(), ctx.plan.cu_new.tolist()
        out = torch.empty_like(u)
        for i, slot in enumerate(slots):
            if slot < 0:
                continue
            s, n = app.state["s"][slot], int(app.state["count"][slot])
            for t in range(cu[i], cu[i + 1]):
                s, n = self.decay * s + u[t], n + 1
                out[t] = s + 0.01 * n
            app.state["s"][slot] = s
            app.state["count"][slot] = n
        return residual + out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_arrangements_states_and_model_options(ops, dtype):
    """What a model needs beyond GPT-2's shape is data of the spec and parts registered from outside: a layer with
    four norms (before and after each branch), a layer with one shared norm and parallel branches, a mixer that
    keeps two state tensors of different types, a factor on the embedded rows, a bias on the logits and a cap on
    them.  Stepped in unequal batches one after another, like whole sequences in the plain restatement below."""
    register_part("block", "toy_sandwich", ToySandwich)
    register_part("block", "toy_parallel", ToyParallel)
    register_part("mixer", "toy_counter", ToyCounter)
    width, vocab, eps, cap = 64, 210, 1e-5, 5.0
    ln = lambda prefix: PartSpec("layernorm", prefix, {"width": width, "eps": eps})  # noqa: E731
    dense = lambda prefix: PartSpec("dense", prefix, {"width": width, "inner": 136, "activation": "gelu_tanh", "up": "up",  # noqa: E731
                                                      "down": "down", "stored": "out_in", "init_std": 0.08, "down_init_std": 0.08})
    attn = PartSpec("causal_attention", "l0.attn.", {"width": width, "n_heads": 4, "kv_heads": 2, "head_dim": 16, "scale": 0.25,
                                                     "qkv": "qkv", "out": "o", "stored": "out_in", "init_std": 0.08,
                                                     "out_init_std": 0.08})
    layers = (LayerSpec("toy_sandwich", ln("l0.n1."), attn, ln("l0.n2."), dense("l0.ffn."),
                        more_norms=(("post1", ln("l0.p1.")), ("post2", ln("l0.p2.")))),
              LayerSpec("toy_parallel", ln("l1.n1."), PartSpec("toy_counter", "l1.cnt.", {"width": width, "decay": 0.7}), None,
                        dense("l1.ffn.")))
    spec = ModelSpec(width=width, vocab_size=vocab, token_table="embed.weight",
                     position=PartSpec("learned_absolute", "pos.", {"width": width, "n_positions": 160}),
                     layers=layers, schedule=(Application(0), Application(1)), final_norm=ln("norm."), head="head.weight",
                     table_init_std=0.3, embedding_scale=math.sqrt(width), head_bias="head.bias", logit_cap=cap)
    tensors = random_tensors(DecoderModel(spec).weight_specs(), 9, torch.bfloat16)
    w = {k: f64(v) for k, v in tensors.items()}
    eng = Engine.from_spec(spec, tensors, dtype=dtype, max_tokens=1024, ops=ops)
    assert isinstance(eng.apps[1].state, dict) and eng.apps[1].state["count"].dtype == torch.int32
    assert len(eng.model.blocks[0].parts()) == 6 and len(eng.model.blocks[1].parts()) == 3

    def plain(ids):
        P = plain_gpt2
        norm = lambda x, p: P.layer_norm(x, w[p + "weight"], w[p + "bias"], eps)  # noqa: E731
        mlp = lambda h, p: P.mlp(h, w[p + "up.weight"], w[p + "up.bias"], w[p + "down.weight"], w[p + "down.bias"], "tanh")  # noqa: E731
        x = P.position_embedding(P.token_embedding(w["embed.weight"], ids), w["pos.weight"]) * math.sqrt(width)
        # (the factor applies to the embedded rows as a whole, positions included: it follows the embedding kernel)
        q, k, v = P.split_qkv(P.linear(norm(x, "l0.n1."), w["l0.attn.qkv.weight"], w["l0.attn.qkv.bias"]), 4, 2, 16)
        a = P.linear(P.attention(q, k, v, 4, 2, 16, 0.25), w["l0.attn.o.weight"], w["l0.attn.o.bias"])
        x = x + norm(a, "l0.p1.")
        x = x + norm(mlp(norm(x, "l0.n2."), "l0.ffn."), "l0.p2.")
        h = norm(x, "l1.n1.")
        u = h @ w["l1.cnt.mix.weight"].T
        s, out = np.full(width, 0.5), np.zeros_like(u)
        for t in range(len(ids)):
            s = 0.7 * s + u[t]
            out[t] = s + 0.01 * (t + 1)
        x = x + out + mlp(h, "l1.ffn.")
        logits = norm(x, "norm.") @ w["head.weight"].T + w["head.bias"]
        return cap * np.tanh(logits / cap)

    seqs = [random_ids(40 + i, vocab, n) for i, n in enumerate((150, 33, 70))]
    tol = 1e-5 if dtype == "float32" else 2e-2
    for batch in ((40, 1, 70), (100, 20, 5)):
        rows, _ = run_batch(eng, seqs, batch)
        for ids, got in zip(seqs, rows):
            assert np.abs(got).max() <= cap
            assert rel_error(got, plain(ids)) < tol
        eng.cache.check()
        assert eng.cache.slots.held == 0
    with pytest.raises(ValueError, match="exactly two norms"):       # GPT-2's arrangement says what it needs
        DecoderModel(ModelSpec(width=width, vocab_size=vocab, token_table="embed.weight", position=spec.position,
                               layers=(LayerSpec("pre_norm", ln("a."), attn, None, dense("b.")),), schedule=(Application(0),),
                               final_norm=ln("norm."), head=None))
