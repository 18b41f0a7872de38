"""Each kernel alone against a plain float32/float64 restatement of the same operation in torch, at
sizes that the engine's own models do not use (widths and vocabularies that are no power of two,
head sizes from 16 to 256, grouped key/value heads, windows, pages in scrambled order)."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2
from ember_cpp_b200.cache import PAGE, SequenceCache
from ember_cpp_b200.engine import StepPlan, build_step
from ember_cpp_b200.parts import CacheNeed

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Caches start full of NaN (ember.cpp's kernel tests do the same to catch reads of rows that no query may
# see, tools/window_attention_cuda_test.cu:57-86): a page that is new to a sequence holds what its last owner
# left, and only the rows past the step's end in such a page are cleared, as the engine clears them.
NAN = float("nan")
# against a float64 evaluation of the same inputs: float32 kernels differ by accumulation order
# only; bfloat16 outputs carry one rounding to 8 bits of mantissa (2^-9 relative) on top
ATOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def ops():
    from ember_cpp_b200.csrc.ops import CudaOps
    return CudaOps()


def gen(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


# ------------------------------------------------------------------------------ rows
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [48, 1600, 100])
def test_embed(ops, dtype, d):
    table, pos = gen((301, d), 0, DT[dtype]), gen((77, d), 1, DT[dtype])
    tokens = torch.tensor([300, 0, 17, 17, 255], dtype=torch.int32).cuda()
    positions = torch.tensor([76, 0, 5, 6, 7], dtype=torch.int32).cuda()
    x = ops.embed(tokens, positions, table, pos)
    assert x.dtype == torch.float32
    assert torch.equal(x, table[tokens.long()].float() + pos[positions.long()].float())
    assert torch.equal(ops.embed(tokens, positions, table, None), table[tokens.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [48, 1600, 100])
def test_embed_takes_tokens_that_a_sampler_left_on_the_device(ops, dtype, d):
    """With rows of sampled ids given, token t is ids[src[t]] where src[t] >= 0 and tokens[t] elsewhere (also where
    the row does not exist); an id outside the table reads row 0, never beyond the table."""
    table, pos = gen((301, d), 8, DT[dtype]), gen((77, d), 9, DT[dtype])
    tokens = torch.tensor([300, 0, 17, 17, 255], dtype=torch.int32).cuda()
    positions = torch.tensor([76, 0, 5, 6, 7], dtype=torch.int32).cuda()
    src = torch.tensor([2, -1, 0, 9, 3], dtype=torch.int32).cuda()
    ids = torch.tensor([40, 41, 42, 1000], dtype=torch.int32).cuda()
    x = ops.embed(tokens, positions, table, pos, token_src=src, ids=ids)
    taken = torch.tensor([42, 0, 40, 17, 0]).cuda()
    assert torch.equal(x, table[taken].float() + pos[positions.long()].float())
    assert tokens.tolist() == [300, 0, 17, 17, 255]                      # the step's own description is left as it is
    with pytest.raises(Exception, match="both"):
        ops.embed(tokens, positions, table, pos, token_src=src)


@pytest.mark.parametrize("out", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, d, eps", [(1, 64, 1e-5), (7, 1600, 1e-6), (130, 100, 1e-3), (3, 24, 1e-5)])
def test_layernorm(ops, out, rows, d, eps):
    x = gen((rows, d), 2) * 3 + 0.7
    w, b = gen((d,), 3) + 1, gen((d,), 4)
    got = ops.layernorm(x, w, b, eps, DT[out]).double()
    want = torch.nn.functional.layer_norm(x.double(), (d,), w.double(), b.double(), eps)
    tol = 2e-6 if out == "float32" else 2 ** -8
    assert ((got - want).abs() / (want.abs() + 1)).max().item() < tol


def test_layernorm_statistics_are_per_row(ops):
    """A row's result does not depend on its neighbours or on the number of rows."""
    x = gen((9, 200), 5)
    w, b = gen((200,), 6), gen((200,), 7)
    whole = ops.layernorm(x, w, b, 1e-5, torch.float32)
    for r in (0, 4, 8):
        assert torch.equal(ops.layernorm(x[r:r + 1].contiguous(), w, b, 1e-5, torch.float32)[0], whole[r])


def test_take_tokens(ops):
    tokens = torch.tensor([5, 6, 7, 8, 9], dtype=torch.int32).cuda()
    src = torch.tensor([2, -1, 0, 9, -1], dtype=torch.int32).cuda()      # row 9 does not exist: left alone
    ids = torch.tensor([40, 41, 42, 1000], dtype=torch.int32).cuda()
    ops.take_tokens(tokens, src, ids, 100)
    assert tokens.tolist() == [42, 6, 40, 8, 9]
    ops.take_tokens(tokens, torch.tensor([3, -1, -1, -1, -1], dtype=torch.int32).cuda(), ids, 100)
    assert tokens.tolist()[0] == 0                                       # an id outside the vocabulary never reaches the table


def test_gather_rows(ops):
    x = gen((11, 72), 8)
    rows = torch.tensor([10, 0, 3, 3], dtype=torch.int32).cuda()
    assert torch.equal(ops.gather_rows(x, rows, 4), x[rows.long()])
    assert torch.equal(ops.gather_rows(x, rows, 2), x[rows[:2].long()])


# ------------------------------------------------------------------------------ products
def linear_ref(a, w, bias, act, residual):
    y = a.double() @ w.double().t()
    if bias is not None:
        y = y + bias.double()
    if act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "gelu_erf":
        y = torch.nn.functional.gelu(y)
    if residual is not None:
        y = y + residual.double()
    return y


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M, N, K", [(1, 40, 24), (5, 4800, 1600), (130, 1000, 96), (64, 200, 320), (3, 50257, 64)])
@pytest.mark.parametrize("act, with_bias, with_res", [(None, True, False), ("gelu_tanh", True, False),
                                                      ("gelu_erf", True, False), (None, True, True), (None, False, False)])
def test_linear(ops, dtype, M, N, K, act, with_bias, with_res):
    a, w = gen((M, K), 9, DT[dtype]), gen((N, K), 10, DT[dtype], 0.1)
    bias = gen((N,), 11) if with_bias else None
    res = gen((M, N), 12) if with_res else None
    want = linear_ref(a, w, bias, act, res)
    got = ops.linear(a, w, bias, act=act, residual=None if res is None else res.clone(),
                     out_dtype=torch.float32 if with_res else DT[dtype])
    assert got.dtype == (torch.float32 if with_res else DT[dtype])
    scale = want.abs().max().item() + 1e-6
    tol = 1e-5 if dtype == "float32" else (2e-3 if with_res else 2 ** -7)
    assert (got.double() - want).abs().max().item() / scale < tol


@pytest.mark.parametrize("M, N, K", [(1, 1600, 1600), (8, 100, 40), (9, 50, 72), (16, 4800, 1600), (3, 17, 104),
                                     (16, 1600, 6400), (2, 50257, 96)])
@pytest.mark.parametrize("act, with_bias, with_res, out", [(None, True, False, "bfloat16"), ("gelu_tanh", True, False, "bfloat16"),
                                                           ("gelu_erf", False, False, "bfloat16"), (None, True, True, "float32"),
                                                           (None, False, False, "float32")])
def test_linear_few_rows_streams_the_weights(ops, M, N, K, act, with_bias, with_res, out):
    """Up to 16 rows take the weight-streaming kernel (tensor cores with the operands swapped):
    every tile shape, tails in N and K, both batch tiles."""
    a, w = gen((M, K), 30, torch.bfloat16), gen((N, K), 31, torch.bfloat16, 0.1)
    bias = gen((N,), 32) if with_bias else None
    res = gen((M, N), 33) if with_res else None
    want = linear_ref(a, w, bias, act, res)
    got = ops.linear(a, w, bias, act=act, residual=None if res is None else res.clone(), out_dtype=DT[out])
    assert got.dtype == DT[out]
    scale = want.abs().max().item() + 1e-6
    assert (got.double() - want).abs().max().item() / scale < (2e-4 if out == "float32" else 2 ** -7)


STREAM_SHAPES = [(4800, 1600), (1600, 1600), (6400, 1600), (1600, 6400), (50257, 1600), (200, 328), (130, 72), (77, 64)]


@pytest.mark.parametrize("N, K", STREAM_SHAPES)
@pytest.mark.parametrize("M", [17, 32, 33, 48, 64])
def test_linear_17_to_64_rows_streams_the_weights(ops, M, N, K):
    """17 to 64 rows take the tcgen05 weight-streaming kernel (operands swapped, K split over a
    cluster): GPT-2 XL's four products and its head (an output width that is no multiple of 8), and
    small shapes with tails in N (no multiple of 128) and K (no multiple of 64), with each epilogue."""
    a, w = gen((M, K), 40, torch.bfloat16), gen((N, K), 41, torch.bfloat16, 0.1)
    bias, res = gen((N,), 42), gen((M, N), 43)
    launches = ops.launches
    for act, with_bias, with_res, out in [(None, True, False, "bfloat16"), ("gelu_tanh", True, False, "bfloat16"),
                                          ("gelu_erf", False, False, "bfloat16"), (None, True, True, "float32"),
                                          (None, False, False, "float32")]:
        want = linear_ref(a, w, bias if with_bias else None, act, res if with_res else None)
        got = ops.linear(a, w, bias if with_bias else None, act=act, residual=res.clone() if with_res else None,
                         out_dtype=DT[out])
        assert got.dtype == DT[out]
        scale = want.abs().max().item() + 1e-6
        assert (got.double() - want).abs().max().item() / scale < (2e-4 if out == "float32" else 2 ** -7), (act, out)
    assert ops.launches == launches + 5          # one launch each: no separate activation or sum
    ops.check()


@pytest.mark.parametrize("M", [1, 16, 23, 64])
@pytest.mark.parametrize("N, K", [(1600, 1600), (300, 6400), (129, 200)])
def test_linear_stream_every_split_and_ring(ops, M, N, K):
    """Every number of blocks to a tile (1 to 8) and rings shorter than a block's share of K give the
    same sums up to float32 rounding, and each of them twice the same bits (no atomics, no timing)."""
    a, w = gen((M, K), 44, torch.bfloat16), gen((N, K), 45, torch.bfloat16, 0.1)
    bias, res = gen((N,), 46), gen((M, N), 47)
    want = linear_ref(a, w, bias, None, res)
    scale = want.abs().max().item()
    for k_split in range(1, 9):
        for stages in (0, 2, 3):
            first = res.clone()
            ops.linear_stream(a, w, bias, None, first, first, k_split, stages)
            again = res.clone()
            ops.linear_stream(a, w, bias, None, again, again, k_split, stages)
            assert torch.equal(first, again), (k_split, stages)
            assert (first.double() - want).abs().max().item() / scale < 2e-4, (k_split, stages)
    ops.check()


@pytest.mark.parametrize("M, N, K, tile_n", [(128, 64, 64, 0), (200, 1600, 1600, 0), (129, 1001, 72, 0), (65, 48, 4104, 16),
                                             (300, 500, 200, 48), (1000, 777, 136, 256), (2048, 4800, 1600, 0),
                                             (257, 6400, 320, 208)])
@pytest.mark.parametrize("act, with_bias, with_res, out", [(None, True, False, "bfloat16"), ("gelu_tanh", True, False, "bfloat16"),
                                                           ("gelu_erf", False, False, "bfloat16"), (None, True, True, "float32"),
                                                           (None, False, False, "float32")])
def test_linear_on_the_tcgen05_kernel(ops, M, N, K, tile_n, act, with_bias, with_res, out):
    """The TMA-fed tcgen05 product with its epilogue: tiles cut off in M, N and K, every tile
    width class (the narrowest, one that is no power of two, the widest), more tiles than SMs so
    that blocks walk several tiles and both accumulators, and a width that is no multiple of 8."""
    a, w = gen((M, K), 50, torch.bfloat16), gen((N, K), 51, torch.bfloat16, 0.1)
    bias = gen((N,), 52) if with_bias else None
    res = gen((M, N), 53) if with_res else None
    want = linear_ref(a, w, bias, act, res)
    got = res.clone() if with_res else torch.full((M, N), float("nan"), dtype=DT[out], device="cuda")
    ops.linear_tc(a, w, bias, act, got if with_res else None, got, tile_n=tile_n)
    torch.cuda.synchronize()
    ops.check()
    scale = want.abs().max().item() + 1e-6
    assert (got.double() - want).abs().max().item() / scale < (2e-4 if out == "float32" else 2 ** -7)


def test_linear_routes_large_products_to_the_tcgen05_kernel_when_asked(ops, monkeypatch):
    a, w = gen((130, 64), 54, torch.bfloat16), gen((96, 64), 55, torch.bfloat16, 0.1)
    seen = []
    monkeypatch.setattr(ops, "linear_tc", lambda *args, **kw: seen.append(1) or args[5])
    ops.linear(a, w, None)
    assert seen == []
    monkeypatch.setattr(ops, "gemm", "tc")
    ops.linear(a, w, None)
    assert seen == [1]


@pytest.mark.parametrize("M, N, K", [(8, 6400, 1600), (3, 100, 72), (16, 48, 4104)])
def test_linear_few_rows_warms_what_it_is_told_to(M, N, K):
    """A tensor announced with `warm` is asked into L2 by the next small product: the product is the
    same bit for bit, the tensor is not changed, and the announcement is used once."""
    from ember_cpp_b200.csrc.ops import CudaOps
    ops = CudaOps()
    ops.warm_ahead = True
    a, w, bias = gen((M, K), 41, torch.bfloat16), gen((N, K), 42, torch.bfloat16, 0.1), gen((N,), 43)
    for numel in (16, 8 * 1024 * 1024 + 24, 1600 * 6400):
        other = torch.full((numel,), 7.0, dtype=torch.bfloat16, device="cuda")
        plain = ops.linear(a, w, bias, act="gelu_tanh", out_dtype=torch.bfloat16)
        ops.warm(other)
        warmed = ops.linear(a, w, bias, act="gelu_tanh", out_dtype=torch.bfloat16)
        assert ops._warm is None
        torch.cuda.synchronize()
        assert torch.equal(plain, warmed) and bool((other == 7.0).all())
    ops.check()


def test_timeline_of_a_step_from_an_instrumented_build(tmp_path):
    """A library built with EMBER_TIMELINE=1 notes when the blocks of the decode kernels start, pass
    their wait and end; the ordinary build refuses to give a timeline."""
    import subprocess
    import sys
    with pytest.raises(Exception, match="EMBER_TIMELINE"):
        from ember_cpp_b200.csrc.ops import CudaOps
        CudaOps().timeline()
    code = """
import torch
from ember_cpp_b200.csrc.ops import CudaOps
ops = CudaOps()
x = torch.randn(8, 320, device="cuda")
w, b = torch.ones(320, device="cuda"), torch.zeros(320, device="cuda")
ops.timeline()
h = ops.layernorm(x, w, b, 1e-5, torch.bfloat16)
y = ops.linear(h, torch.randn(96, 320, device="cuda").bfloat16(), None)
marks = ops.timeline()
names = {(k, m) for _, k, m, _, _, _ in marks}
assert {("layernorm", 0), ("layernorm", 1), ("layernorm", 2), ("linear_decode", 0), ("linear_decode", 1),
        ("linear_decode", 2)} <= names, names
assert sum(1 for _, k, m, _, _, _ in marks if k == "linear_decode" and m == 0) == 6   # 96 / 16 tiles
assert all(0 <= sm < torch.cuda.get_device_properties(0).multi_processor_count for *_, sm in marks)
assert all(a[0] <= b[0] for a, b in zip(marks, marks[1:]))
assert ops.timeline() == []
print("ok")
"""
    import os
    env = dict(os.environ, EMBER_TIMELINE="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def test_linear_float32_rows_do_not_depend_on_the_batch(ops):
    """The 32-bit product adds each output element in one fixed order: a row computed alone is
    bit-identical to the same row of a large batch."""
    a, w, bias = gen((150, 200), 13), gen((333, 200), 14, scale=0.1), gen((333,), 15)
    whole = ops.linear(a, w, bias, act="gelu_tanh", out_dtype=torch.float32)
    for r in (0, 63, 64, 149):
        assert torch.equal(ops.linear(a[r:r + 1].contiguous(), w, bias, act="gelu_tanh", out_dtype=torch.float32)[0],
                           whole[r])


def test_linear_refuses_mismatches(ops):
    from ember_cpp_b200.csrc.ops import KernelError
    a, w = gen((4, 32), 0), gen((8, 16), 1)
    with pytest.raises(KernelError, match="width"):
        ops.linear(a, w, None)
    with pytest.raises(KernelError, match="float32"):
        ops.linear(a, gen((8, 32), 1, torch.bfloat16), None)
    with pytest.raises(KernelError, match="activation"):
        ops.linear(a, gen((8, 32), 1), None, act="relu")


# ------------------------------------------------------------------------------ cache and attention
def make_step(seqs, heads, kv_heads, hd, dtype, window=0, scramble=True, seed=0, poison=None):
    """seqs: (already cached, new) positions per sequence.  Returns plan, cache view, qkv and the
    dense K/V per sequence that the cache holds after the store."""
    need = CacheNeed("window" if window else "full", kv_heads, hd, window)
    total = sum(-(-(a + b) // PAGE) for a, b in seqs) + 3
    cache = SequenceCache([(need, None)], [None], total * PAGE, None, DT[dtype], "cuda")
    if scramble:                       # take the pages in a scrambled order
        order = np.random.default_rng(seed).permutation(cache.n_pages)[::1].tolist()
        cache.groups[0].pages._free = order
    view = cache.views[0]
    if poison is not None:
        view.k.fill_(poison)
        view.v.fill_(poison)
    width = (heads + 2 * kv_heads) * hd
    slots = [cache.open() for _ in seqs]
    dense = []
    g = torch.Generator().manual_seed(seed)
    # fill what is already cached by storing it through a first step
    return cache, view, slots, width, g


def attention_ref(q, k, v, heads, kv_heads, hd, scale, window, start):
    """q: [n, heads*hd] at positions start.., k/v: [start+n, kv*hd].  float64."""
    n = q.shape[0]
    out = torch.zeros(n, heads * hd, dtype=torch.float64)
    q, k, v = q.double().cpu(), k.double().cpu(), v.double().cpu()
    rep = heads // kv_heads
    for t in range(n):
        p = start + t
        lo = max(0, p - window + 1) if window else 0
        for h in range(heads):
            g = h // rep
            s = (k[lo:p + 1, g * hd:(g + 1) * hd] @ q[t, h * hd:(h + 1) * hd]) * scale
            out[t, h * hd:(h + 1) * hd] = torch.softmax(s, 0) @ v[lo:p + 1, g * hd:(g + 1) * hd]
    return out


def run_attention(ops, seqs, heads, kv_heads, hd, dtype, window=0, seed=0, poison=None, qkv_fn=None, ahead=False,
                  store_apart=False):
    """Stores `cached` positions per sequence in one step, then runs the step of `new` positions;
    returns (got, want) for the second step's tokens.  ahead: the view names the storage of a layer
    that attends next (which a kernel may warm but must not change)."""
    cache, view, slots, width, g = make_step(seqs, heads, kv_heads, hd, dtype, window, True, seed, poison)
    if ahead:
        view.following = (torch.full_like(view.k, 3.0), torch.full_like(view.v, 5.0))
    scale = 0.37 / math.sqrt(hd)
    tables = [cache.groups[0].table]
    data = [torch.randn(a + b, width, generator=g) for a, b in seqs]
    if qkv_fn is not None:
        data = qkv_fn(data)
    data = [d.to(DT[dtype]) for d in data]

    def step(entries, rows):
        tails = cache.reserve([(s, n) for s, n in entries])
        host = build_step([(s, [0] * n, []) for s, n in entries], cache.lengths, tables, cache.max_blocks, tails=tails)
        plan = StepPlan(host, torch.from_numpy(host.packed).cuda())
        if plan.has_tails:   # as the engine does: the rows past the step's end in pages new to their sequences
            ops.clear_tails(cache.groups[0], plan.tails[0])
        qkv = torch.cat(rows).cuda().contiguous()
        if store_apart:      # as a layer does that reads a cache which another layer has stored into in this step
            ops.kv_store(qkv, view, plan, heads, kv_heads, hd)
            out = ops.attention(qkv, view, plan, heads, kv_heads, hd, scale, window, DT[dtype], store=False)
        else:
            out = ops.attention(qkv, view, plan, heads, kv_heads, hd, scale, window, DT[dtype], store=True)
        cache.commit([(s, n) for s, n in entries])
        return out

    first = [(s, a) for s, (a, b) in zip(slots, seqs) if a > 0]
    if first:
        step(first, [d[:a] for d, (a, b) in zip(data, seqs) if a > 0])
    got = step([(s, b) for s, (a, b) in zip(slots, seqs)], [d[a:] for d, (a, b) in zip(data, seqs)])
    if ahead:
        torch.cuda.synchronize()
        assert bool((view.following[0] == 3.0).all()) and bool((view.following[1] == 5.0).all())
    want = []
    qw, kw = heads * hd, kv_heads * hd
    for d, (a, b) in zip(data, seqs):
        d = d.float()
        want.append(attention_ref(d[a:, :qw], d[:, qw:qw + kw], d[:, qw + kw:], heads, kv_heads, hd, scale, window, a))
    return got.double().cpu(), torch.cat(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, hd", [(4, 4, 16), (25, 25, 64), (6, 2, 32), (3, 1, 80), (2, 2, 128),
                                                 (5, 5, 256), (8, 4, 48)])
def test_attention_prompts_of_unequal_length(ops, dtype, heads, kv_heads, hd):
    got, want = run_attention(ops, [(0, 70), (0, 1), (0, 129), (0, 64)], heads, kv_heads, hd, dtype, seed=hd, poison=NAN)
    assert (got - want).abs().max().item() < ATOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, kv_heads, hd", [(4, 4, 16), (25, 25, 64), (6, 2, 32), (3, 1, 80), (4, 2, 128)])
def test_attention_one_token_each_over_the_cache(ops, dtype, heads, kv_heads, hd):
    seqs = [(199, 1), (63, 1), (64, 1), (0, 1), (300, 1), (127, 1), (128, 1)]
    got, want = run_attention(ops, seqs, heads, kv_heads, hd, dtype, seed=hd + 1, poison=NAN)
    assert (got - want).abs().max().item() < ATOL[dtype]


@pytest.mark.parametrize("heads, kv_heads, hd, window", [(25, 25, 64, 0), (16, 2, 64, 0), (4, 2, 128, 0), (8, 8, 64, 150),
                                                        (18, 2, 64, 0), (3, 3, 128, 0), (2, 2, 128, 200)])
def test_attention_one_token_each_on_the_tensor_cores(heads, kv_heads, hd, window):
    """The decode attention that runs its products on the tensor cores against the reference and against
    the kernel it replaces, with so many sequences that a block keeps a whole context (its warps refill
    their stages page after page) and with few (the context is cut into chunks that are merged).  Nine
    query heads to a key/value head are more than it takes as rows: the other kernel runs."""
    from ember_cpp_b200.csrc.ops import CudaOps
    tensor, other = CudaOps(), CudaOps()
    tensor.decode_mma, other.decode_mma = True, False
    many = [(n, 1) for n in (700, 1, 0, 63, 64, 65, 127, 128, 129, 300, 511, 512, 640)] * (5 if kv_heads > 2 else 40)
    for seqs in (many, [(700, 1), (64, 1), (0, 1), (129, 1)]):
        got, want = run_attention(tensor, seqs, heads, kv_heads, hd, "bfloat16", window=window, seed=7, poison=NAN)
        old, _ = run_attention(other, seqs, heads, kv_heads, hd, "bfloat16", window=window, seed=7, poison=NAN)
        assert (got - want).abs().max().item() < ATOL["bfloat16"]
        assert (old - want).abs().max().item() < ATOL["bfloat16"]
        tensor.check()
    if heads // kv_heads > 8:
        assert torch.equal(got, old)
    # the token's own key already in the cache (stored by a launch of its own): the same output
    apart, _ = run_attention(tensor, seqs, heads, kv_heads, hd, "bfloat16", window=window, seed=7, poison=NAN, store_apart=True)
    assert (apart - want).abs().max().item() < ATOL["bfloat16"]


@pytest.mark.parametrize("heads, kv_heads, hd, window", [(25, 25, 64, 0), (6, 2, 32, 0), (3, 1, 80, 100)])
def test_attention_one_token_each_warms_the_next_layers_rows(heads, kv_heads, hd, window):
    """Asked to, the decode attention asks the same rows of the next layer's pages into L2: the same
    output bit for bit, and that storage is not changed."""
    from ember_cpp_b200.csrc.ops import CudaOps
    seqs = [(199, 1), (63, 1), (64, 1), (0, 1), (300, 1), (127, 1), (128, 1)]
    plain, warming = CudaOps(), CudaOps()
    plain.cache_ahead, warming.cache_ahead = False, True
    got, want = run_attention(warming, seqs, heads, kv_heads, hd, "bfloat16", window=window, seed=hd + 1, poison=NAN,
                              ahead=True)
    same, _ = run_attention(plain, seqs, heads, kv_heads, hd, "bfloat16", window=window, seed=hd + 1, poison=NAN)
    assert (got - want).abs().max().item() < ATOL["bfloat16"]
    assert torch.equal(got, same)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_tokens_added_to_a_cache(ops, dtype):
    """More than one new token on top of cached ones: the general case of the step function."""
    got, want = run_attention(ops, [(50, 30), (64, 64), (1, 5), (100, 130)], 6, 3, 32, dtype, seed=3, poison=NAN)
    assert (got - want).abs().max().item() < ATOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 7, 64, 100])
def test_attention_window(ops, dtype, window):
    got, want = run_attention(ops, [(0, 150), (130, 1), (90, 20)], 4, 2, 32, dtype, window=window, seed=window)
    assert (got - want).abs().max().item() < ATOL[dtype]


@pytest.mark.parametrize("heads, kv_heads", [(25, 25), (8, 2), (3, 1)])
@pytest.mark.parametrize("window", [0, 1, 70, 200])
def test_attention_on_the_tcgen05_kernel(ops, heads, kv_heads, window):
    """Head size 64 in bfloat16 takes the TMA/tcgen05 prefill kernel: prompts that end inside a
    128-row tile, on its edge and past it, tokens added on top of cached ones (tiles that start in
    the middle of a page), grouped heads, windows that cut pages, scrambled page order, and the
    mma.sync kernel as its twin."""
    from ember_cpp_b200.csrc.ops import CudaOps
    seqs = [(0, 300), (0, 128), (0, 1), (70, 129), (64, 64), (200, 57), (0, 127)]
    assert ops.attention_tc
    launches = ops.launches
    got, want = run_attention(ops, seqs, heads, kv_heads, 64, "bfloat16", window=window, seed=7 + window, poison=NAN)
    torch.cuda.synchronize()
    ops.check()
    assert (got - want).abs().max().item() < ATOL["bfloat16"]
    twin = CudaOps()
    twin.attention_tc = False
    other, _ = run_attention(twin, seqs, heads, kv_heads, 64, "bfloat16", window=window, seed=7 + window, poison=NAN)
    assert (got - other).abs().max().item() < ATOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """One early key is made to stand out (its score far above the rest): every later query must
    return that key's value.  A kernel that skips, misplaces or double-counts a tile shows here."""
    heads, hd, far = 2, 64, 37

    def shape(data):
        for d in data:
            n = d.shape[0]
            d[:, :2 * heads * hd] *= 0.05                     # q and k small ...
            d[far, heads * hd:2 * heads * hd] = 4.0           # ... but key `far` large in every head
            d[far + 1:, :heads * hd] = 4.0                    # and the later queries aligned with it
            d[:, 2 * heads * hd:] = torch.arange(n)[:, None].float() / 8   # value row j = j / 8
        return data

    got, want = run_attention(ops, [(0, 700), (650, 1)], heads, heads, hd, dtype, seed=5, qkv_fn=shape)
    later = torch.cat([got[far + 1:700], got[700:]])
    assert (later - far / 8).abs().max().item() < (1e-4 if dtype == "float32" else 5e-2)
    assert (got - want).abs().max().item() < (1e-4 if dtype == "float32" else 5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(ops, dtype):
    """The key just outside the window stands out and must be ignored; in a second run the key
    just inside does and must be found."""
    heads, hd, window, p = 2, 32, 40, 199
    for offset, seen in ((window, False), (window - 1, True)):
        j = p - offset

        def shape(data):
            d = data[0]
            d[:, :2 * heads * hd] *= 0.05
            d[j, heads * hd:2 * heads * hd] = 4.0
            d[p, :heads * hd] = 4.0
            d[:, 2 * heads * hd:] = 0.0
            d[j, 2 * heads * hd:] = 100.0
            return data

        got, want = run_attention(ops, [(p, 1)], heads, heads, hd, dtype, window=window, seed=6, qkv_fn=shape)
        assert (got - want).abs().max().item() < 1e-1
        assert (got.min().item() > 99.0) if seen else (got.abs().max().item() < 1e-3)


def test_attention_refuses_sizes_it_cannot_run(ops):
    from ember_cpp_b200.csrc.ops import KernelError
    for heads, kv, hd in [(4, 3, 32), (2, 2, 512)]:
        with pytest.raises((KernelError, ValueError)):
            run_attention(ops, [(0, 4)], heads, kv, hd, "float32")
    with pytest.raises(KernelError, match="head size"):        # one token each in bfloat16: the decode kernels want 16s
        run_attention(ops, [(3, 1)], 2, 2, 24, "bfloat16")


@pytest.mark.parametrize("hd", [12, 24, 1, 250])
def test_attention_in_32_bit_takes_every_head_size(ops, hd):
    """The plain kernels of the 32-bit path (scalar copies where a head's row is no multiple of 16 bytes):
    prompts, tokens on top of a cache, one token each, NaN in every row that no query may see."""
    got, want = run_attention(ops, [(0, 70), (65, 3), (130, 1), (0, 1)], 3, 3, hd, "float32", seed=hd, poison=NAN)
    assert (got - want).abs().max().item() < ATOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_kv_store_writes_only_its_rows(ops, dtype):
    heads, kv_heads, hd = 3, 3, 16
    cache, view, slots, width, g = make_step([(0, 70)], heads, kv_heads, hd, dtype, poison=7.0)
    cache.reserve([(slots[0], 70)])
    host = build_step([(slots[0], [0] * 70, [])], cache.lengths, [cache.groups[0].table], cache.max_blocks)
    plan = StepPlan(host, torch.from_numpy(host.packed).cuda())
    qkv = torch.randn(70, width, generator=g).to(DT[dtype]).cuda()
    ops.kv_store(qkv, view, plan, heads, kv_heads, hd)
    pages = cache.groups[0].held[slots[0]]
    k = torch.cat([view.k[p] for p in pages], dim=1)          # [kv_heads, 128, hd]
    assert torch.equal(k[:, :70].transpose(0, 1).reshape(70, -1), qkv[:, heads * hd:(heads + kv_heads) * hd])
    assert (k[:, 70:] == 7.0).all()
    untouched = [p for p in range(cache.n_pages) if p not in pages]
    assert (view.k[untouched] == 7.0).all() and (view.v[untouched] == 7.0).all()


def rounded(v: float) -> float:
    """The value as the cache holds it in bfloat16."""
    return float(torch.tensor(v).bfloat16())


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("mma", [True, False])
def test_decode_attention_finds_one_far_key(hd, mma):
    """One-token steps (the decode kernels, on the tensor cores and on the CUDA cores) with one key in
    page 0 that stands out among 700 and more: every sequence must return that key's value.  Few
    sequences cut the context into chunks that are merged (in a cluster, and through scratch and a
    ticket where heads are grouped); many sequences let one block walk all pages.  Random inputs
    would hide a skipped, misplaced or double-counted page: the softmax over hundreds of keys is
    nearly flat, and one key moves the output by less than the tolerance."""
    from ember_cpp_b200.csrc.ops import CudaOps
    ops = CudaOps()
    ops.decode_mma = mma
    far = 37

    def shape(heads, kv_heads):
        def fn(data):
            qw, kw = heads * hd, kv_heads * hd
            for d in data:
                n = d.shape[0]
                d[:, :qw + kw] *= 0.05
                d[far, qw:qw + kw] = 4.0                      # the key that stands out, in every head
                d[far + 1:, :qw] = 4.0                        # the later queries aligned with it
                d[:, qw + kw:] = torch.arange(n)[:, None].float() / 8
            return data
        return fn

    for heads, kv_heads in ((2, 2), (8, 2)):
        few = [(700, 1), (895, 1), (64, 1), (far + 1, 1)]
        many = [(700 + 3 * i, 1) for i in range(90)]
        for seqs in (few, many):
            for apart in (False, True):
                got, want = run_attention(ops, seqs, heads, kv_heads, hd, "bfloat16", seed=5, qkv_fn=shape(heads, kv_heads),
                                          poison=NAN, store_apart=apart)
                ops.check()
                assert (got - rounded(far / 8)).abs().max().item() < 5e-2, (heads, kv_heads, len(seqs), apart)
                assert (got - want).abs().max().item() < 5e-2


@pytest.mark.parametrize("far", [5, 2111, 4031])
def test_attention_finds_one_key_among_thousands(ops, far):
    """Contexts of more than 4,000 positions (65 pages; a configuration may ask for them): a prompt through
    the tcgen05 kernel and one-token steps through the tensor-core decode kernel (few sequences: chunks merged
    in a cluster; many: longer walks), with one key that stands out in the first page, in the middle or in the
    last full page.  Every later query must return that key's value and nothing of the other rows, whose
    values differ from page to page."""
    heads, hd = 2, 64

    def shape(data):
        qw = heads * hd
        for d in data:
            n = d.shape[0]
            d[:, :2 * qw] *= 0.05
            if far < n:
                d[far, qw:2 * qw] = 4.0                          # the key that stands out, in every head
                d[far + 1:, :qw] = 4.0                           # the later queries aligned with it
            d[:, 2 * qw:] = ((torch.arange(n) // 7) % 16)[:, None].float() / 8
            if far < n:
                d[far, 2 * qw:] = 7.0
        return data

    got, want = run_attention(ops, [(0, 4100)], heads, heads, hd, "bfloat16", seed=7, qkv_fn=shape, poison=NAN)
    ops.check()
    assert (got[far + 1:] - 7.0).abs().max().item() < 5e-2
    assert (got - want).abs().max().item() < 5e-2
    few = [(4100, 1), (far + 1, 1), (4159, 1)]
    many = [(far + 1 + 5 * i, 1) for i in range(40)]
    for seqs in (few, many):
        got, want = run_attention(ops, seqs, heads, heads, hd, "bfloat16", seed=8, qkv_fn=shape, poison=NAN)
        ops.check()
        assert (got - 7.0).abs().max().item() < 5e-2, len(seqs)
        assert (got - want).abs().max().item() < 5e-2


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("mma", [True, False])
@pytest.mark.parametrize("p", [63, 64, 65, 191, 192, 511, 700])
def test_decode_attention_window_edge_and_own_key(hd, mma, p):
    """A window of 150 on one-token steps at positions around page and chunk edges: a key that stands
    out just outside the window (position p - 150) must be ignored, the same key just inside it
    (p - 149) must be found, and a token whose own key stands out must return its own value,
    whether its key is stored by the attention's launch or by a launch of its own."""
    from ember_cpp_b200.csrc.ops import CudaOps
    ops = CudaOps()
    ops.decode_mma = mma
    heads, window = 4, 150

    def shape(at):
        def fn(data):
            qw = heads * hd
            for d in data:
                n = d.shape[0]
                d[:, :2 * qw] *= 0.05
                if 0 <= at < n:
                    d[at, qw:2 * qw] = 4.0
                d[n - 1, :qw] = 4.0                            # the last token's query looks for it
                d[:, 2 * qw:] = torch.arange(n)[:, None].float() / 8
            return data
        return fn

    seqs = [(p, 1)] * 3
    for apart in (False, True):
        if p - window + 1 >= 0:
            inside = p - window + 1
            got, want = run_attention(ops, seqs, heads, heads, hd, "bfloat16", window=window, seed=6, qkv_fn=shape(inside),
                                      poison=NAN, store_apart=apart)
            assert (got - rounded(inside / 8)).abs().max().item() < 5e-2, ("inside", apart)
        if p - window >= 0:
            outside = p - window
            got, want = run_attention(ops, seqs, heads, heads, hd, "bfloat16", window=window, seed=6, qkv_fn=shape(outside),
                                      poison=NAN, store_apart=apart)
            # (the mean of about 150 values around p / 8, rounded to bfloat16's 8 bits)
            assert (got - want).abs().max().item() < 2 ** -7 * want.abs().max().item() + 2e-2, ("outside", apart)
            assert (got - outside / 8).abs().min().item() > 1.0          # nowhere near the ignored key's value
        got, want = run_attention(ops, seqs, heads, heads, hd, "bfloat16", window=window, seed=6, qkv_fn=shape(p),
                                  poison=NAN, store_apart=apart)
        assert (got - rounded(p / 8)).abs().max().item() < 5e-2, ("own", apart)
    ops.check()


# ------------------------------------------------------------------------------ bounded waits
def test_a_wait_that_runs_out_is_reported_and_harms_nothing(ops):
    """The kernels' waits on mbarriers give up after a time limit and say so in a status word instead of
    hanging.  A kernel whose only wait nothing ever ends (wait_probe.cu, the same tc::mbar_wait with a limit
    of a millisecond) returns; `check()` raises and names it, once; the launches after it work."""
    import time
    from ember_cpp_b200.csrc.ops import KernelError
    torch.cuda.synchronize()
    ops.check()
    t0 = time.perf_counter()
    ops.wait_probe(1_000_000)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0                 # it gave up after its millisecond, not after the kernels' two seconds
    with pytest.raises(KernelError, match="wait_probe"):
        ops.check()
    ops.check()                                           # the word is cleared by reading it
    a, w = gen((40, 256), 70, torch.bfloat16), gen((300, 256), 71, torch.bfloat16, 0.1)
    got = ops.linear(a, w, None, out_dtype=torch.float32)  # a tcgen05 kernel right after: the context is fine
    torch.cuda.synchronize()
    ops.check()
    want = a.double() @ w.double().t()
    assert (got.double() - want).abs().max().item() / want.abs().max().item() < 2e-4
    with pytest.raises(KernelError, match="limit"):
        ops.wait_probe(10)


# ------------------------------------------------------------------------------ sampling
@pytest.mark.parametrize("V", [512, 1000, 50257])
def test_sample_equals_plain(ops, V):
    rows = 6
    logits = gen((rows, V), 20, scale=2.0)
    streams = torch.arange(rows, dtype=torch.int32).cuda() + 3
    counters = torch.arange(rows, dtype=torch.int32).cuda() * 5
    host = logits.cpu().numpy()
    assert ops.sample(logits, 0.0, 0, 1.0, 1, streams, counters).tolist() == [int(r.argmax()) for r in host]
    for T, k, p in [(0.8, 0, 1.0), (0.1, 40, 0.9), (1.0, 40, 0.9), (0.7, 5, 1.0), (1.3, 0, 0.5), (2.0, 1, 1.0),
                    (1.0, 0, 0.0), (1.0, V + 5, 0.999)]:
        got = ops.sample(logits, T, k, p, 11, streams, counters).tolist()
        want = [plain_gpt2.sample(host[r], T, k, p, plain_gpt2.uniform01(11, 3 + r, 5 * r)) for r in range(rows)]
        assert got == want, (T, k, p)


def test_sample_small_top_k_takes_the_short_list_or_falls_back(ops):
    """A small top_k is finished on a short candidate list; rows whose candidates do not fit the
    list (thousands of equal logits at the edge of top_k) take the general selection.  Both give
    the plain implementation's token, for every top_p, a top_k of 1, 512 (the last short one) and
    513, and a top_p of 0 (the best candidate alone)."""
    V, rows = 50257, 5
    logits = gen((rows, V), 21, scale=3.0)
    logits[1, 1000:9000] = 9.0           # 8,000 equal maxima: the list cannot hold the bucket
    logits[2, 0:V - 1:2] = logits[2, 1:V:2]   # pairs of equal logits
    logits[3, 7] = 40.0                  # one token holds all the mass
    logits[4] = logits[4].round()        # many ties on every level
    streams = torch.arange(rows, dtype=torch.int32).cuda()
    counters = torch.arange(rows, dtype=torch.int32).cuda() + 2
    host = logits.cpu().numpy()
    for T, k, p in [(1.0, 40, 0.9), (0.1, 40, 0.9), (1.0, 1, 1.0), (1.0, 512, 0.95), (1.0, 513, 0.95), (0.7, 40, 0.0),
                    (2.0, 100, 1.0), (1.0, 40, 0.3)]:
        for seed in (1, 2):
            got = ops.sample(logits, T, k, p, seed, streams, counters).tolist()
            want = [plain_gpt2.sample(host[r], T, k, p, plain_gpt2.uniform01(seed, r, r + 2)) for r in range(rows)]
            assert got == want, (T, k, p, seed)


def test_sample_first_maximum_and_ties(ops):
    logits = torch.zeros(3, 300).cuda()
    logits[0, [17, 250]] = 5.0           # the first of two maxima
    logits[1, :] = float("-inf")
    logits[1, 299] = -3.0
    logits[2, 5] = float("nan")          # a NaN never wins
    logits[2, 9] = 1.0
    z = torch.zeros(3, dtype=torch.int32).cuda()
    assert ops.sample(logits, 0.0, 0, 1.0, 0, z, z).tolist() == [17, 299, 9]
    # ties at the edge of top_k: the larger indices are kept (pairs ordered by (p, index) descending)
    flat = torch.zeros(1, 10).cuda()
    seen = {ops.sample(flat, 1.0, 3, 1.0, s, z[:1], z[:1]).item() for s in range(64)}
    assert seen == {7, 8, 9}


def test_sample_distribution(ops):
    probs = torch.tensor([0.05, 0.4, 0.05, 0.3, 0.2])
    n = 4000
    logits = probs.log().repeat(n, 1).cuda()
    streams = torch.zeros(n, dtype=torch.int32).cuda()
    counters = torch.arange(n, dtype=torch.int32).cuda()
    got = torch.bincount(ops.sample(logits, 1.0, 0, 1.0, 5, streams, counters).long().cpu(), minlength=5) / n
    assert (got - probs).abs().max().item() < 0.03
    top2 = torch.bincount(ops.sample(logits, 1.0, 2, 1.0, 5, streams, counters).long().cpu(), minlength=5) / n
    assert top2[[0, 2, 4]].sum() == 0 and abs(top2[1].item() - 4 / 7) < 0.03
