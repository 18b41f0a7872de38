"""The engine on the GPU against the plain implementation: each request alone and whole, long
decoding, the first tokens of a sequence, batches that follow one another in the same slots, and
generation through the Python entry point and the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import ember_cpp_b200 as E
import plain_gpt2
from conftest import ROOT, TOL, random_ids, rel_error, run_batch
from ember_cpp_b200.engine import Engine

pytestmark = pytest.mark.gpu
NAMES = ["tiny_a", "tiny_b"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def engines(tiny_folders):
    return {(n, d): Engine.from_folder(tiny_folders[n], dtype=d, max_tokens=2048) for n in NAMES for d in DTYPES}


def test_the_kernels_are_the_librarys_own(engines):
    eng = engines[("tiny_a", "bfloat16")]
    assert eng.ops.name == "cuda-sm100a" and os.path.isfile(eng.ops.lib._path)
    with open("/proc/self/maps") as f:
        assert "libember_kernels.so" in f.read()


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_each_request_alone_and_whole(engines, plains, name, dtype):
    eng, plain = engines[(name, dtype)], plains[name]
    for i, n in enumerate((1, 2, 31, 64, 65, plain.n_positions)):
        ids = random_ids(100 + i, plain.vocab, n)
        rows, _ = run_batch(eng, [ids], (n,))
        ref = plain.logits(ids)
        assert rel_error(rows[0], ref) < TOL[dtype]
        if dtype == "float32":
            assert (rows[0].argmax(-1) == ref.argmax(-1)).all()


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(engines, plains, name, dtype):
    """From a one-token prompt to the last position, one token at a time: every row, the first
    ones (positions 0, 1, 2) and the ones at page edges (63, 64) included."""
    eng, plain = engines[(name, dtype)], plains[name]
    ids = random_ids(7, plain.vocab, plain.n_positions)
    rows, _ = run_batch(eng, [ids], (1,))
    ref = plain.logits(ids)
    per_row = [rel_error(rows[0][t], ref[t]) for t in range(len(ids))]
    assert max(per_row) < TOL[dtype], int(np.argmax(per_row))
    if dtype == "float32":
        whole, _ = run_batch(eng, [ids], (len(ids),))
        assert np.array_equal(whole[0], rows[0])


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_lengths_one_after_another(engines, plains, name, dtype):
    eng, plain = engines[(name, dtype)], plains[name]
    P = plain.n_positions
    plans = [((P, 30, 1, 70, 64), (P // 2, 9, 1, 33, 63)),        # the shorter ones end earlier
             ((65, P - 1, 17), (64, 1, 17)),                      # the slots of the first batch, other lengths
             ((12, 12, 12, 12, 12, 12, 12), (3, 3, 3, 3, 3, 3, 3))]
    used = []
    for b, (lengths, prompts) in enumerate(plans):
        seqs = [random_ids(200 + 10 * b + i, plain.vocab, n) for i, n in enumerate(lengths)]
        rows, slots = run_batch(eng, seqs, prompts)
        used.append(set(slots))
        for ids, got in zip(seqs, rows):
            assert rel_error(got, plain.logits(ids)) < TOL[dtype]
        eng.cache.check()
        assert eng.cache.slots.held == 0 and eng.cache.groups[0].pages.held == 0
    assert used[1] <= used[0]                  # slots are used again


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_no_result(engines, plains, dtype):
    """Three sequences decode in a graph padded to four; the same sequences alone give the same
    rows (bit for bit in 32-bit)."""
    eng, plain = engines[("tiny_b", dtype)], plains["tiny_b"]
    seqs = [random_ids(300 + i, plain.vocab, 40) for i in range(3)]
    together, _ = run_batch(eng, seqs, (20, 20, 20))
    for ids, got in zip(seqs, together):
        alone, _ = run_batch(eng, [ids], (20,))
        if dtype == "float32":
            assert np.array_equal(alone[0], got)
        else:
            assert rel_error(alone[0], got) < TOL[dtype]


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_that_left_nan_behind_does_not_reach_the_next(tiny_folders, plains, name, dtype):
    """Pages are not cleared when they change hands.  After a batch has ended, every page of the cache
    is filled with NaN (what a request whose activations overflowed leaves behind); the next batch
    takes the same pages and must equal the plain implementation, prompts that end inside a page,
    on a page's edge and one token at a time across page edges included."""
    plain = plains[name]
    P = plain.n_positions
    eng = Engine.from_folder(tiny_folders[name], dtype=dtype, max_tokens=4 * 128, max_slots=4)
    lengths, prompts = (P, 70, 65, 3), (P - 40, 64, 1, 2)
    first = [random_ids(700 + i, plain.vocab, n) for i, n in enumerate(lengths)]
    run_batch(eng, first, prompts)
    for group in eng.cache.groups:
        for t in list(group.k) + list(group.v):
            t.fill_(float("nan"))
    for b in range(2):                                             # twice: graphs captured, then replayed
        seqs = [random_ids(710 + 10 * b + i, plain.vocab, n) for i, n in enumerate(lengths)]
        rows, _ = run_batch(eng, seqs, prompts)
        for ids, got in zip(seqs, rows):
            assert np.isfinite(got).all()
            assert rel_error(got, plain.logits(ids)) < TOL[dtype]
        for group in eng.cache.groups:
            for t in list(group.k) + list(group.v):
                t.fill_(float("nan"))


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_20_40_and_64_sequences(tiny_folders, plains, name, dtype):
    """Decoding with more sequences than one weight-streaming tile of 16: 20, 40 and 64 sequences of
    unequal lengths whose shorter ones leave on the way (so the step passes through every bucket of
    batch sizes from 64 down, padded to 32 and 64 in between), one batch after another in the same
    slots.  Every row against the plain implementation; in 32-bit a sequence's rows are the same
    bits as when it runs alone."""
    plain = plains[name]
    P = plain.n_positions
    eng = Engine.from_folder(tiny_folders[name], dtype=dtype, max_tokens=64 * 128, max_slots=64)
    rng = np.random.default_rng(11)
    first_slots = None
    for b, count in enumerate((64, 20, 40)):
        lengths = [int(n) for n in rng.integers(2, P + 1, count)]
        lengths[0], lengths[-1] = P, 2                               # one to the last position, one that leaves at once
        prompts = [int(rng.integers(1, n)) for n in lengths]
        seqs = [random_ids(600 + 100 * b + i, plain.vocab, n) for i, n in enumerate(lengths)]
        rows, slots = run_batch(eng, seqs, prompts)
        eng.ops.check()
        worst = max(rel_error(got, plain.logits(ids)) for ids, got in zip(seqs, rows))
        assert worst < TOL[dtype], (count, worst)
        if dtype == "float32":
            for i in (0, count // 2, count - 1):
                alone, _ = run_batch(eng, [seqs[i]], (prompts[i],))
                assert np.array_equal(alone[0], rows[i]), (count, i)
        eng.cache.check()
        assert eng.cache.slots.held == 0 and eng.cache.groups[0].pages.held == 0
        first_slots = first_slots or set(slots)
        assert set(slots) <= first_slots                              # the slots of the first batch, used again
    assert {b for b, _ in eng._graphs} >= {64, 32, 16, 8, 4, 2, 1}    # every bucket of batch sizes was replayed


@pytest.mark.parametrize("name", NAMES)
def test_prompts_through_the_tcgen05_products(tiny_folders, plains, name):
    """Whole prompts with the library's own tcgen05 matrix products in place of cuBLASLt: batches of
    more than 64 tokens (one tile of 128 rows cut off, and two blocks sharing a 256-row tile), both
    GELU forms, the residual sums and the float32 head."""
    plain = plains[name]
    eng = Engine.from_folder(tiny_folders[name], dtype="bfloat16", max_tokens=1024)
    eng.ops.gemm = "tc"
    P = plain.n_positions
    seqs = [random_ids(460 + i, plain.vocab, n) for i, n in enumerate((P, P - 7, 70))]
    rows, _ = run_batch(eng, seqs, (P, P - 7, 66))
    eng.ops.check()
    for ids, got in zip(seqs, rows):
        assert rel_error(got, plain.logits(ids)) < TOL["bfloat16"]
    alone, _ = run_batch(eng, [seqs[0]], (P,))
    eng.ops.check()
    assert rel_error(alone[0], plain.logits(seqs[0])) < TOL["bfloat16"]


@pytest.mark.parametrize("gemm", ["lt", "tc"])
def test_wide_model_bfloat16_against_float32(gemm):
    """GPT-2 XL's layer sizes (width 1600, 25 heads of 64, inner 6400, vocabulary 50,257; two
    layers): the bfloat16 path (tcgen05 prefill attention, cuBLASLt or the tcgen05 products, the
    weight-streaming decode products, split decode attention in a replayed graph) against the
    32-bit path on the same weights: two prompts of unequal length over several pages, then
    decode steps, every wanted row within the bfloat16 tolerance and the same best token where the
    32-bit logits decide clearly."""
    from ember_cpp_b200.config import get_architecture
    from ember_cpp_b200.parts import DecoderModel
    from ember_cpp_b200.weights import random_tensors
    cfg = E.GPT2Config.from_dict(dict(vocab_size=50257, n_positions=1024, n_embd=1600, n_layer=2, n_head=25,
                                      n_inner=6400, activation_function="gelu_new", layer_norm_epsilon=1e-5))
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = random_tensors(DecoderModel(spec).weight_specs(), 5, torch.bfloat16, "cuda")
    engines = {d: Engine.from_spec(spec, tensors, dtype=d, max_tokens=2048) for d in DTYPES}
    engines["bfloat16"].ops.gemm = gemm
    seqs = [random_ids(900 + i, 50257, n) for i, n in enumerate((710, 135))]
    rows = {}
    for d, eng in engines.items():
        slots = [eng.open() for _ in seqs]
        out = [eng.step([(s, q[:-6], [len(q) - 9, len(q) - 7]) for s, q in zip(slots, seqs)]).float().cpu().numpy()]
        for k in range(6, 0, -1):
            out.append(eng.step([(s, [q[-k]], [0]) for s, q in zip(slots, seqs)]).float().cpu().numpy())
        rows[d] = np.concatenate(out)
        eng.ops.check()
        for s in slots:
            eng.close(s)
    ref, got = rows["float32"], rows["bfloat16"]
    assert ref.shape == got.shape == (4 + 12, 50257)
    assert rel_error(got, ref) < TOL["bfloat16"]
    assert check_top1(got, ref) > 0


def check_top1(got, ref) -> int:
    """The rows whose 32-bit logits decide clearly (a margin between the best two of more than twice the
    bfloat16 tolerance, relative to the row's range) must have the same best token; returns how many rows
    that was, so that a caller can insist the check ran at all."""
    top2 = np.sort(ref, axis=-1)[:, -2:]
    sure = (top2[:, 1] - top2[:, 0]) / (ref.max(-1) - ref.min(-1)) > 2 * TOL["bfloat16"]
    assert (got.argmax(-1)[sure] == ref.argmax(-1)[sure]).all()
    return int(sure.sum())


def shape_engines(n_embd, n_head, n_inner, n_layer, max_tokens, seed, n_positions=1024):
    """The two compute types over one set of random weights of the given layer sizes (vocabulary 50,257)."""
    from ember_cpp_b200.config import get_architecture
    from ember_cpp_b200.parts import DecoderModel
    from ember_cpp_b200.weights import random_tensors
    cfg = E.GPT2Config.from_dict(dict(vocab_size=50257, n_positions=n_positions, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                                      n_inner=n_inner, activation_function="gelu_new", layer_norm_epsilon=1e-5))
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = random_tensors(DecoderModel(spec).weight_specs(), seed, torch.bfloat16, "cuda")
    return {d: Engine.from_spec(spec, tensors, dtype=d, max_tokens=max_tokens) for d in DTYPES}


def test_a_context_of_four_thousand_positions():
    """A configuration with 4,096 positions (four heads of 64, two layers): prompts of 4,020 and 700 tokens in
    one step (63 pages for the longer one), then 24 one-token steps across a page's edge in the largest
    buckets of lengths, bfloat16 against the 32-bit path on the same weights."""
    engines = shape_engines(256, 4, 1024, 2, 2 * 4096, seed=41, n_positions=4096)
    seqs = [random_ids(4100 + i, 50257, n + 24) for i, n in enumerate((4020, 700))]
    rows = {}
    for d, eng in engines.items():
        slots = [eng.open() for _ in seqs]
        out = [eng.step([(s, q[:-24], [len(q) - 25]) for s, q in zip(slots, seqs)]).float().cpu().numpy()]
        for k in range(24, 0, -1):
            out.append(eng.step([(s, [q[-k]], [0]) for s, q in zip(slots, seqs)]).float().cpu().numpy())
        rows[d] = np.concatenate(out)
        eng.ops.check()
        assert eng.length(slots[0]) == 4044
        for s in slots:
            eng.close(s)
    assert rows["float32"].shape == (2 + 48, 50257)
    assert rel_error(rows["bfloat16"], rows["float32"]) < TOL["bfloat16"]
    assert check_top1(rows["bfloat16"], rows["float32"]) > 0


def test_large_shape_ragged_prompts_then_256_steps():
    """GPT-2 large's layer sizes (width 1,280, 20 heads, inner 5,120; two layers of its 36): a batch of 16
    ragged prompts with lengths uniform in [1, 512], then 256 decode steps, bfloat16 against the 32-bit
    path on the same weights: the prompts' last rows and every 16th step's rows."""
    rng = np.random.default_rng(36)
    lengths = [int(n) for n in rng.integers(1, 513, 16)]
    lengths[0], lengths[1] = 1, 512
    seqs = [random_ids(3600 + i, 50257, n + 256) for i, n in enumerate(lengths)]
    engines = shape_engines(1280, 20, 5120, 2, 16 * 768, seed=36)
    rows = {}
    for d, eng in engines.items():
        slots = [eng.open() for _ in seqs]
        out = [eng.step([(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lengths)]).float().cpu().numpy()]
        for k in range(256):
            want = [0] if k % 16 == 15 else []
            got = eng.step([(s, [q[n + k]], want) for s, q, n in zip(slots, seqs, lengths)])
            if want:
                out.append(got.float().cpu().numpy())
        eng.ops.check()
        for s in slots:
            eng.close(s)
        rows[d] = np.concatenate(out)
    assert rows["float32"].shape == (16 * 17, 50257)
    assert rel_error(rows["bfloat16"], rows["float32"]) < TOL["bfloat16"]
    assert check_top1(rows["bfloat16"], rows["float32"]) > 0


def test_medium_shape_64_ragged_prompts_decoded_to_the_full_context():
    """GPT-2 medium's layer sizes (width 1,024, 16 heads, inner 4,096; two layers of its 24): 64 ragged
    prompts with lengths uniform in [8, 960], each decoded to the full context of 1,024 (the shorter the
    prompt the longer it decodes; sequences leave as they reach the end, so the batch shrinks through
    every bucket).  bfloat16 against the 32-bit path at every 64th step; and whole prompts against token
    by token: four of the sequences fed whole in one step give, in 32-bit, the same bits as their rows
    from the batch, and in bfloat16 rows within the tolerance."""
    rng = np.random.default_rng(24)
    lengths = [int(n) for n in rng.integers(8, 961, 64)]
    lengths[0], lengths[1] = 8, 960
    seqs = [random_ids(2400 + i, 50257, 1024) for i in range(64)]
    engines = shape_engines(1024, 16, 4096, 2, 64 * 1024 + 4 * 1024, seed=24)
    rows, last = {}, {}
    for d, eng in engines.items():
        slots = [eng.open() for _ in seqs]
        fed = list(lengths)
        out = [eng.step([(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lengths)]).float().cpu().numpy()]
        live = list(range(64))
        step = 0
        final = {}
        while live:
            ending = [i for i in live if fed[i] + 1 == 1024]
            want_all = step % 64 == 63
            got = eng.step([(slots[i], [seqs[i][fed[i]]], [0] if (want_all or i in ending) else []) for i in live])
            if got is not None:
                got = got.float().cpu().numpy()
                r = 0
                for i in live:
                    if want_all or i in ending:
                        if want_all:
                            out.append(got[r:r + 1])
                        if i in ending:
                            final[i] = got[r]
                        r += 1
            for i in live:
                fed[i] += 1
            for i in ending:
                eng.close(slots[i])
            live = [i for i in live if i not in ending]
            step += 1
        eng.ops.check()
        eng.cache.check()
        assert eng.cache.slots.held == 0
        rows[d], last[d] = np.concatenate(out), final
        assert {b for b, _ in eng._graphs} >= {64, 32, 16, 8, 4, 2, 1}
    assert rel_error(rows["bfloat16"], rows["float32"]) < TOL["bfloat16"]
    assert check_top1(rows["bfloat16"], rows["float32"]) > 0
    for i in (0, 1, 17, 40):                       # whole in one step against token by token in the batch
        for d, eng in engines.items():
            slot = eng.open()
            whole = eng.step([(slot, seqs[i], [1023])]).float().cpu().numpy()[0]
            eng.close(slot)
            if d == "float32":
                assert np.array_equal(whole, last[d][i]), i
            else:
                assert rel_error(whole, last["float32"][i]) < TOL["bfloat16"], i


def test_a_head_size_that_is_no_multiple_of_16_runs_in_32_bit(tmp_path):
    """Width 36 with 3 heads of 12, inner 100, a vocabulary of 77: the true 32-bit path takes every size
    the configuration allows; the bfloat16 kernels refuse this model when it is loaded, naming the keys."""
    cfg = E.GPT2Config.from_dict(dict(vocab_size=77, n_positions=80, n_embd=36, n_layer=2, n_head=3, n_inner=100,
                                      activation_function="gelu", layer_norm_epsilon=1e-6, tie_word_embeddings=False))
    folder = str(tmp_path / "odd")
    E.write_random_model(folder, cfg, seed=8)
    plain = plain_gpt2.PlainGPT2(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    seqs = [random_ids(800 + i, 77, n) for i, n in enumerate((80, 66, 5))]
    rows, _ = run_batch(eng, seqs, (40, 65, 1))
    for ids, got in zip(seqs, rows):
        ref = plain.logits(ids)
        assert rel_error(got, ref) < TOL["float32"] and (got.argmax(-1) == ref.argmax(-1)).all()
    with pytest.raises(E.ConfigError, match="n_embd / n_head"):
        Engine.from_folder(folder, dtype="bfloat16", max_tokens=256)


def test_two_processes_give_the_same_bits_when_deterministic(tiny_folders, tmp_path):
    """With the `deterministic` option (EMBER_DETERMINISTIC=1) no algorithm is chosen by a timing: two
    processes give bit-equal bfloat16 logits for prompts that take the library products (more than 64
    rows) and for the decode steps after them."""
    script = ("import sys, numpy as np; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
              "from conftest import random_ids, run_batch\n"
              "from ember_cpp_b200.engine import Engine\n"
              "eng = Engine.from_folder(sys.argv[1], dtype='bfloat16', max_tokens=1024)\n"
              "assert eng.ops.options.deterministic and not eng.ops.lt_tune\n"
              "seqs = [random_ids(50 + i, 1000, n) for i, n in enumerate((96, 90, 70))]\n"
              "rows, _ = run_batch(eng, seqs, (90, 80, 66))\n"
              "np.save(sys.argv[2], np.concatenate(rows))\n") % (ROOT, os.path.join(ROOT, "tests"))
    outs = []
    for k in range(2):
        out = str(tmp_path / f"run{k}.npy")
        env = dict(os.environ, EMBER_DETERMINISTIC="1")
        r = subprocess.run([sys.executable, "-c", script, tiny_folders["tiny_b"], out], env=env, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        outs.append(np.load(out))
    assert np.array_equal(outs[0], outs[1])


def test_per_launch_timing_and_ranges(tiny_folders, plains):
    """With the op_timing option every launch of a prompt step and of decode steps is timed by name (the
    step then runs launch by launch, no graph), with NVTX ranges around launches and steps; the logits are
    the same as without."""
    plain = plains["tiny_b"]
    seqs = [random_ids(480 + i, plain.vocab, n) for i, n in enumerate((70, 9))]
    timed = Engine.from_folder(tiny_folders["tiny_b"], dtype="bfloat16", max_tokens=512,
                               options=E.RuntimeOptions.from_env().replace(op_timing=True, nvtx=True))
    assert not timed.cuda_graphs
    rows, _ = run_batch(timed, seqs, (60, 5))
    times = timed.ops.op_times()
    assert {"ember_embed", "ember_layernorm", "ember_attention_prefill", "ember_linear_decode", "ember_kv_store"} <= set(times)
    assert all(n > 0 and ms > 0 for n, ms in times.values())
    assert times["ember_layernorm"][0] == (2 * 3 + 1) * 11          # 3 layers and the final norm, 1 prompt step and 10 decode steps
    assert timed.ops.op_times() == {}                                # read and reset
    usual = run_batch(Engine.from_folder(tiny_folders["tiny_b"], dtype="bfloat16", max_tokens=512), seqs, (60, 5))[0]
    for a, b in zip(rows, usual):
        assert rel_error(a, b) < 1e-6


def test_graph_replay_equals_launch_by_launch(tiny_folders, plains):
    plain = plains["tiny_a"]
    seqs = [random_ids(400 + i, plain.vocab, 50) for i in range(3)]
    out = []
    for graphs in (True, False):
        eng = Engine.from_folder(tiny_folders["tiny_a"], dtype="float32", max_tokens=512, cuda_graphs=graphs)
        out.append(run_batch(eng, seqs, (10, 1, 30))[0])
    for a, b in zip(*out):
        assert np.array_equal(a, b)
    # graphs captured ahead of time over padding, for every bucket of lengths: the same rows, and no capture later
    for dtype in DTYPES:
        eng = Engine.from_folder(tiny_folders["tiny_a"], dtype=dtype, max_tokens=512)
        made = eng.capture_decode(3)
        assert made == len(eng._graphs) > 0 and all(batch == 4 for batch, _ in eng._graphs)
        kept = dict(eng._graphs)
        ahead = run_batch(eng, seqs, (10, 1, 30))[0]            # the batch shrinks to 2 and 1: those buckets are made then
        assert all(eng._graphs[key] is graph for key, graph in kept.items())
        late = run_batch(Engine.from_folder(tiny_folders["tiny_a"], dtype=dtype, max_tokens=512), seqs, (10, 1, 30))[0]
        for a, b in zip(ahead, late):
            assert np.array_equal(a, b)
        eng.ops.check()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(tiny_folders, plains, name):
    plain = plains[name]
    prompts = [random_ids(500 + i, plain.vocab, n) for i, n in enumerate((5, 17, 32, 1, plain.n_positions - 4))]
    session = E.Session(tiny_folders[name], max_batch_size=3, dtype="float32", max_tokens=1024)
    got = session.generate_detailed(prompts, steps=16, temperature=0.0)
    for p, g in zip(prompts, got):
        want, why = plain_gpt2.generate(plain, p, 16)
        assert g.tokens == want and g.finish_reason == why
    assert got[-1].finish_reason == "context"
    # bfloat16: the same ids wherever the 32-bit logits decide clearly
    s16 = E.Session(tiny_folders[name], max_batch_size=3, dtype="bfloat16", max_tokens=1024)
    for p, g in zip(prompts, s16.generate_detailed(prompts, steps=16, temperature=0.0)):
        ids = list(p)
        for tok in g.tokens:
            row = plain.logits(ids)[-1]
            best = np.sort(row)[-2:]
            if best[1] - best[0] > 4 * TOL["bfloat16"] * (row.max() - row.min()):
                assert tok == int(row.argmax())
            if len(ids) < plain.n_positions:
                ids.append(tok)
    assert session.engine.cache.slots.held == 0 and s16.engine.cache.slots.held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_running_a_step_ahead_changes_no_token_on_the_gpu(tiny_folders, plains, dtype):
    """The generation loop queues a step with the ids of the step before still on the device
    (`take_tokens`, then the replayed graph).  Against the loop that reads every id first: the
    same tokens and reasons, with stop ids, unequal counts and batches one after another."""
    plain = plains["tiny_a"]
    prompts = [random_ids(800 + i, plain.vocab, n) for i, n in enumerate((4, 33, 64, 1, 90, 7, plain.n_positions - 1))]
    out = []
    for ahead in (True, False):
        session = E.Session(tiny_folders["tiny_a"], max_batch_size=3, dtype=dtype, max_tokens=1024, seed=3)
        session.generator.run_ahead = ahead
        free = session.generate_detailed(prompts, steps=9, temperature=0.9, top_k=30, top_p=0.95, stop_token_ids=[])
        stops = [free[1].tokens[3], free[4].tokens[0]]
        session.set_seed(3)
        got = session.generate_detailed(prompts, steps=9, temperature=0.9, top_k=30, top_p=0.95, stop_token_ids=stops)
        out.append([(g.tokens, g.finish_reason) for g in free + got])
        assert got[1].finish_reason == "stop" and got[4].finish_reason == "stop" and got[6].finish_reason == "context"
        session.engine.ops.check()
        session.engine.cache.check()
        assert session.engine.cache.slots.held == 0
    assert out[0] == out[1]


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_replayed_step_takes_its_tokens_from_sampled_ids_wherever_they_lie(engines, dtype):
    """A one-token step whose tokens are ids on the device: given in the tensor that `sample_target` handed out
    (the captured step's embedding reads them there) or in any other tensor (copied there first), with rows in
    any order, the logits are those of the same tokens given by the host."""
    eng = engines[("tiny_a", dtype)]
    V = eng.vocab_size
    a, b, c = random_ids(900, V, 9), random_ids(901, V, 70), random_ids(902, V, 3)
    want = None
    for way in ("host", "ring", "elsewhere", "ring again"):
        slots = [eng.open() for _ in range(3)]
        eng.step([(s, p[:-1], []) for s, p in zip(slots, (a, b, c))])
        last = [a[-1], b[-1], c[-1]]
        if way == "host":
            out = eng.step([(s, [t], [0]) for s, t in zip(slots, last)])
        else:
            given = torch.tensor([7, last[2], last[0], 5, last[1]], dtype=torch.int32).cuda()   # rows 2, 4, 1 are wanted
            if way == "elsewhere":
                ids = given
            else:
                ids = eng.sample_target(5)
                ids.copy_(given)
            out = eng.step([(s, [0], [0]) for s in slots], device_tokens=(ids, [2, 4, 1]))
        out = out.clone()
        for s in slots:
            eng.close(s)
        if want is None:
            want = out
        else:
            assert torch.equal(out, want), way
    s0 = eng.open()
    with pytest.raises(E.StepError, match="taken from the device"):
        eng.step([(s0, [1], [])], device_tokens=(torch.zeros(2, dtype=torch.int32).cuda(), [2]))
    with pytest.raises(E.StepError, match="taken from the device"):
        eng.step([(s0, [1], [])], device_tokens=(torch.zeros(2, dtype=torch.int64).cuda(), [0]))
    assert eng.length(s0) == 0
    eng.close(s0)
    eng.ops.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_step_of_a_known_shape_replays_a_graph_and_changes_nothing(tiny_folders, dtype):
    """A step of prompts whose shape has come before is captured and replayed; the logits are, bit for bit, those
    of the same step launched from the host, for other tokens, other slots and other wanted rows of the same
    count; only the last few shapes are kept."""
    plain_way = Engine.from_folder(tiny_folders["tiny_b"], dtype=dtype, max_tokens=2048,
                                   options=E.RuntimeOptions(prompt_graphs=0))
    eng = Engine.from_folder(tiny_folders["tiny_b"], dtype=dtype, max_tokens=2048, options=E.RuntimeOptions(prompt_graphs=2))
    V = eng.vocab_size

    def both(lengths, wants, seed, hold=0):
        got = []
        for e in (plain_way, eng):
            held = [e.open() for _ in range(hold)]            # other slots, other pages
            slots = [e.open() for _ in lengths]
            out = e.step([(s, random_ids(seed + i, V, n), w) for i, (s, n, w) in enumerate(zip(slots, lengths, wants))])
            got.append(None if out is None else out.clone())
            for s in slots + held:
                e.close(s)
        assert (got[0] is None and got[1] is None) or torch.equal(got[0], got[1])

    both([70, 9, 33], [[69], [0, 8], [32]], 1000)
    assert len(eng._prompt_graphs) == 0                       # a new shape: launched from the host
    both([70, 9, 33], [[69], [0, 8], [32]], 1010)
    assert len(eng._prompt_graphs) == 1                       # the second time: captured
    both([70, 9, 33], [[1], [2, 3], [4]], 1020, hold=2)
    both([9, 70, 33], [[8], [0, 69], [32]], 1030)             # same counts, same longest: the same shape
    assert len(eng._prompt_graphs) == 1
    for lengths in ([5, 5], [64], [5, 5], [64], [3], [3]):
        both(lengths, [[n - 1] for n in lengths], 1040)
    assert len(eng._prompt_graphs) == 2                       # three shapes were captured in all, two are kept
    both([12], [[]], 1050)
    both([12], [[]], 1051)                                    # nothing wanted: no logits either way
    eng.ops.check()
    assert eng.cache.slots.held == 0 and plain_way.cache.slots.held == 0


def test_temperature_generation_equals_plain(tiny_folders, plains):
    plain = plains["tiny_b"]
    prompts = [random_ids(600 + i, plain.vocab, n) for i, n in enumerate((1, 9, 40, 63))]
    session = E.Session(tiny_folders["tiny_b"], max_batch_size=4, dtype="float32", max_tokens=1024, seed=7)
    got = session.generate_detailed(prompts, steps=24, temperature=0.8, top_k=0, top_p=1.0, stop_token_ids=[])
    for i, (p, g) in enumerate(zip(prompts, got)):
        want, why = plain_gpt2.generate(plain, p, 24, 0.8, 0, 1.0, seed=7, stream=i)
        assert g.tokens == want and g.finish_reason == why


def test_command_line(tiny_folders, plains, tmp_path):
    plain = plains["tiny_a"]
    prompt = random_ids(700, plain.vocab, 6)
    cli = [sys.executable, os.path.join(ROOT, "bin", "ember")]
    r = subprocess.run(cli + [tiny_folders["tiny_a"], "-", "1", "prompt", " ".join(map(str, prompt)), "-mt", "5", "-t", "0",
                              "--dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == plain_gpt2.generate(plain, prompt, 5)[0]
    r = subprocess.run(cli + [tiny_folders["tiny_a"], "-", "1", "batch", "--batch-prompts", "1 2 3", "4 5", "-mt", "3",
                              "--temperature", "0", "--dtype", "float32", "-mbs", "2"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr
    assert "--- Prompt 2 ---" in r.stdout
    want = " ".join(map(str, plain_gpt2.generate(plain, [4, 5], 3)[0]))
    assert f"Output: {want}" in r.stdout
    # the random-weights mode writes a folder that loads
    cfg = tmp_path / "cfg.json"
    cfg.write_text('{"architectures": ["GPT2LMHeadModel"], "vocab_size": 50, "n_positions": 16, "n_embd": 32, '
                   '"n_layer": 1, "n_head": 2}')
    out = tmp_path / "model"
    r = subprocess.run(cli + [str(out), "-", "1", "random-weights", "--config", str(cfg), "--seed", "3"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and (out / "model.safetensors").is_file() and (out / "config.json").is_file()
    r = subprocess.run(cli + [str(out), "-", "1", "prompt", "1 2", "-mt", "2"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and len(r.stdout.split()) == 2
    r = subprocess.run(cli + [str(out), "-", "1", "prompt", "1 99"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "vocabulary" in r.stderr


def test_missing_extension_is_an_error(monkeypatch):
    """No silent fallback: without a compiler and a built library there is no engine."""
    from ember_cpp_b200.csrc import build
    monkeypatch.setattr(build, "find_nvcc", lambda: (_ for _ in ()).throw(build.BuildError("nvcc was not found")))
    monkeypatch.setattr(build, "_digest", lambda: "0" * 16)      # makes the built library look stale
    with pytest.raises(build.BuildError, match="nvcc"):
        from ember_cpp_b200.csrc.ops import CudaOps
        CudaOps()
