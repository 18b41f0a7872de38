"""Trace replay through bin/trace_run, as a user runs it: the same requests whole, with their last
32 tokens one by one, and in batches of unequal lengths whose shorter requests end earlier, one
batch after another so that slots and pages are used again; in 32-bit and in bfloat16; every row
compared with the plain implementation, and the 32-bit rows of the three ways with each other."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TOL, random_ids, rel_error

pytestmark = pytest.mark.gpu
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Replay:
    """Drives one trace_run process: a step goes in only after the last one was answered."""

    def __init__(self, folder, dtype, out, max_tokens):
        self.out = str(out)
        self.proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", self.out,
                                      "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                     text=True, bufsize=1)
        self.n = 0

    def step(self, entries, end=()):
        """entries: (id, tokens, want).  Returns float32 [wanted, vocab] or None."""
        rec = {"step": self.n, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.n}", f"trace_run answered {line!r} (exit {self.proc.poll()})"
        path = os.path.join(self.out, f"{self.n}.f32")
        self.n += 1
        if not any(w for _, _, w in entries):
            assert not os.path.exists(path)
            return None
        return np.fromfile(path, dtype="<f4")

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


def whole(rp, seqs, vocab):
    out = []
    for i, ids in enumerate(seqs):
        out.append(rp.step([(f"w{i}", ids, list(range(len(ids))))], end=[f"w{i}"]).reshape(len(ids), vocab))
    return out


def last_32_one_by_one(rp, seqs, vocab):
    out = []
    for i, ids in enumerate(seqs):
        head = max(1, len(ids) - 32)
        rows = [rp.step([(f"t{i}", ids[:head], list(range(head)))]).reshape(head, vocab)]
        for t in range(head, len(ids)):
            rows.append(rp.step([(f"t{i}", [ids[t]], [0])], end=[f"t{i}"] if t == len(ids) - 1 else []).reshape(1, vocab))
        if head == len(ids):
            rp.step([], end=[f"t{i}"])
        out.append(np.concatenate(rows))
    return out


def in_batches(rp, seqs, vocab, batches, prompt_of):
    """batches: lists of request numbers; prompt_of: request -> tokens fed in its first step."""
    out = {}
    for batch in batches:
        fed = {i: prompt_of[i] for i in batch}
        ends = [f"b{i}" for i in batch if fed[i] == len(seqs[i])]
        flat = rp.step([(f"b{i}", seqs[i][:fed[i]], list(range(fed[i]))) for i in batch], end=ends)
        flat = flat.reshape(-1, vocab)
        at = 0
        for i in batch:
            out[i] = [flat[at:at + fed[i]]]
            at += fed[i]
        live = [i for i in batch if fed[i] < len(seqs[i])]
        while live:
            ends = [f"b{i}" for i in live if fed[i] + 1 == len(seqs[i])]
            flat = rp.step([(f"b{i}", [seqs[i][fed[i]]], [0]) for i in live], end=ends).reshape(-1, vocab)
            for r, i in enumerate(live):
                out[i].append(flat[r:r + 1])
                fed[i] += 1
            live = [i for i in live if fed[i] < len(seqs[i])]
    return [np.concatenate(out[i]) for i in range(len(seqs))]


LENGTHS = {"tiny_a": (128, 77, 40, 33, 5, 64, 65, 1), "tiny_b": (96, 63, 40, 33, 9, 1, 64, 65)}
BATCHES = [[0, 1, 2], [3, 4, 5, 6, 7]]


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways(tiny_folders, plains, tmp_path, name, dtype):
    plain = plains[name]
    V = plain.vocab
    seqs = [random_ids(40 + i, V, n) for i, n in enumerate(LENGTHS[name])]
    refs = [plain.logits(ids) for ids in seqs]
    prompt_of = {i: max(1, len(s) // 2) for i, s in enumerate(seqs)}
    prompt_of[2] = len(seqs[2])               # one request is over with its prompt
    # the most that live requests hold: a batch's requests, each rounded up to 64
    need = max(sum(-(-len(seqs[i]) // 64) * 64 for i in b) for b in BATCHES)
    rp = Replay(tiny_folders[name], dtype, tmp_path, need)
    ways = {"whole": whole(rp, seqs, V), "last 32 one by one": last_32_one_by_one(rp, seqs, V),
            "batches": in_batches(rp, seqs, V, BATCHES, prompt_of)}
    rp.close()
    for way, rows in ways.items():
        for i, (got, ref) in enumerate(zip(rows, refs)):
            assert got.shape == ref.shape, (way, i)
            assert rel_error(got, ref) < TOL[dtype], (way, i, rel_error(got, ref))
            if dtype == "float32":
                assert (got.argmax(-1) == ref.argmax(-1)).all(), (way, i)
    if dtype == "float32":
        # the 32-bit kernels add in an order that depends on positions alone: the cut changes no bit
        for i in range(len(seqs)):
            assert np.array_equal(ways["whole"][i], ways["last 32 one by one"][i]), i
            assert np.array_equal(ways["whole"][i], ways["batches"][i]), i
    else:
        for i in range(len(seqs)):
            for way in ("last 32 one by one", "batches"):
                assert rel_error(ways[way][i], ways["whole"][i]) < TOL[dtype], (way, i)


def test_replay_refuses_more_than_the_cache_holds(tiny_folders, tmp_path):
    rp = Replay(tiny_folders["tiny_a"], "float32", tmp_path, 64)
    rp.step([("a", [1] * 60, [59])])
    rp.proc.stdin.write(json.dumps({"step": 1, "entries": [{"id": "b", "tokens": [1], "want": [0]}], "end": []}) + "\n")
    rp.proc.stdin.flush()
    rp.proc.stdin.close()
    assert rp.proc.wait(timeout=60) != 0          # the second request needs a page that is not there


def test_replay_writes_nothing_where_nothing_is_wanted(tiny_folders, plains, tmp_path):
    plain = plains["tiny_b"]
    ids = random_ids(77, plain.vocab, 20)
    rp = Replay(tiny_folders["tiny_b"], "float32", tmp_path, 128)
    assert rp.step([("x", ids[:10], [])]) is None
    assert rp.step([("x", [ids[10]], []), ("y", [ids[0]], [])]) is None
    got = rp.step([("x", [ids[11]], [0]), ("y", [ids[1]], [])], end=["y"]).reshape(1, -1)
    rp.close()
    assert rel_error(got, plain.logits(ids[:12])[11:]) < TOL["float32"]


# ------------------------------------------------------------------------------ GPT-2 XL's layer sizes
XL_LAYERS = dict(vocab_size=50257, n_positions=1024, n_embd=1600, n_layer=2, n_head=25, n_inner=6400,
                 activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
XL_LENGTHS = (700, 520, 130, 64)          # two of them hold more than 8 pages: the decode attention is cut into chunks
XL_BATCHES = [[0, 2], [1, 3]]


@pytest.fixture(scope="module")
def xl_folder(tmp_path_factory):
    """A model folder with the layer sizes of GPT-2 XL (width 1,600, 25 heads of 64, inner 6,400, vocabulary
    50,257) and two layers, random weights."""
    import ember_cpp_b200 as E
    folder = str(tmp_path_factory.mktemp("xl_layers"))
    E.write_random_model(folder, E.GPT2Config.from_dict(XL_LAYERS), seed=2)
    return folder


def kept(n):
    """The positions of a request of n tokens whose rows are compared: the first ones, page edges, one in 61, the last 40."""
    return sorted({p for p in (0, 1, 2, 63, 64, 65, 127, 128) if p < n} | set(range(0, n, 61)) | set(range(max(0, n - 40), n)))


def replay_kept(rp, seqs, vocab, way):
    """Feeds the requests in one of the three ways and returns, per request, {position: row} for kept(n)."""
    out = [dict() for _ in seqs]

    def feed(entries, end=()):
        """entries: (request, first position, count); wants the kept positions among them."""
        wants = [[p - a for p in kept(len(seqs[i])) if a <= p < a + n] for i, a, n in entries]
        flat = rp.step([(f"{way}{i}", seqs[i][a:a + n], w) for (i, a, n), w in zip(entries, wants)], end=[f"{way}{i}" for i in end])
        if flat is None:
            return
        flat = flat.reshape(-1, vocab)
        at = 0
        for (i, a, n), w in zip(entries, wants):
            for r in w:
                out[i][a + r] = flat[at]
                at += 1

    if way == "w":
        for i, ids in enumerate(seqs):
            feed([(i, 0, len(ids))], end=[i])
    elif way == "t":
        for i, ids in enumerate(seqs):
            head = max(1, len(ids) - 32)
            feed([(i, 0, head)], end=[i] if head == len(ids) else [])
            for t in range(head, len(ids)):
                feed([(i, t, 1)], end=[i] if t == len(ids) - 1 else [])
    else:
        for batch in XL_BATCHES:
            fed = {i: max(1, len(seqs[i]) // 2) for i in batch}
            feed([(i, 0, fed[i]) for i in batch])
            live = list(batch)
            while live:
                feed([(i, fed[i], 1) for i in live], end=[i for i in live if fed[i] + 1 == len(seqs[i])])
                for i in live:
                    fed[i] += 1
                live = [i for i in live if fed[i] < len(seqs[i])]
    return out


def test_replay_three_ways_at_gpt2_xl_layer_sizes(xl_folder, tmp_path):
    """The benchmark's layer sizes through bin/trace_run in all three cuts: the tensor-core decode attention with
    its chunk merges, the tcgen05 prefill attention, the weight-streaming products at their real shapes, several
    buckets of lengths.  32-bit: the three cuts give the same bits, and rows within 1e-5 of the plain implementation
    with its top-1.  bfloat16: every cut within 8e-3 of the 32-bit rows, and the same top-1 wherever the 32-bit
    row's margin is wider than that."""
    import plain_gpt2
    plain = plain_gpt2.PlainGPT2(xl_folder)
    V = plain.vocab
    seqs = [random_ids(900 + i, V, n) for i, n in enumerate(XL_LENGTHS)]
    need = max(sum(-(-len(seqs[i]) // 64) * 64 for i in b) for b in XL_BATCHES)
    rows = {}
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        rp = Replay(xl_folder, dtype, out, need)
        rows[dtype] = {way: replay_kept(rp, seqs, V, way) for way in ("w", "t", "b")}
        rp.close()
    exact = rows["float32"]
    for i, ids in enumerate(seqs):
        ref = plain.logits(ids)
        assert sorted(exact["w"][i]) == kept(len(ids))
        for way in ("w", "t", "b"):
            assert sorted(exact[way][i]) == kept(len(ids)), (way, i)
            for p in kept(len(ids)):
                assert np.array_equal(exact[way][i][p], exact["w"][i][p]), (way, i, p)      # the cut changes no bit
        got = np.stack([exact["w"][i][p] for p in kept(len(ids))])
        want = ref[kept(len(ids))]
        assert rel_error(got, want) < TOL["float32"], (i, rel_error(got, want))
        assert (got.argmax(-1) == want.argmax(-1)).all(), i
    wide = 0
    for way in ("w", "t", "b"):
        for i, ids in enumerate(seqs):
            got = np.stack([rows["bfloat16"][way][i][p] for p in kept(len(ids))])
            want = np.stack([exact["w"][i][p] for p in kept(len(ids))])
            assert rel_error(got, want) < TOL["bfloat16"], (way, i, rel_error(got, want))
            top2 = np.sort(want, axis=-1)[:, -2:]
            margin = (top2[:, 1] - top2[:, 0]) / (want.max(-1) - want.min(-1))
            sure = margin > 2 * TOL["bfloat16"]
            wide += int(sure.sum())
            assert (got.argmax(-1)[sure] == want.argmax(-1)[sure]).all(), (way, i)
    assert wide > 0            # some rows did have a margin wider than the tolerance: the top-1 check ran
