"""The generation loop's decisions, the step description and the host side of the engine, run on
the CPU stand-in for the kernels (tests/cpu_ops.py) against the plain implementation (no GPU)."""
import numpy as np
import pytest

import ember_cpp_b200 as E
from ember_cpp_b200.engine import Engine, StepError, build_step
from ember_cpp_b200.engine.generate import GenerationError, finish_reason, plan_batches

import plain_gpt2
from conftest import random_ids, rel_error, run_batch
from cpu_ops import CpuOps


# ------------------------------------------------------------------------------ decisions
def test_finish_reason_order():
    assert finish_reason(7, 1, 10, {7}, 1, 11) == "stop"            # stop id wins over the count
    assert finish_reason(5, 3, 10, {7}, 3, 11) == "length"
    assert finish_reason(5, 2, 11, {7}, 3, 11) == "context"         # 11 positions cached of 11: no room to feed it
    assert finish_reason(5, 2, 10, {7}, 3, 11) is None
    assert finish_reason(5, 2, 10_000, {7}, 3, None) is None        # no position table: only the cache bounds it


def test_plan_batches():
    assert plan_batches([5, 5, 5, 5, 5], 10, 2, 10_000, 128) == [[0, 1], [2, 3], [4]]
    # pages: each request can come to hold ceil((60 + 9) / 64) = 2 pages; 5 pages in the cache
    assert plan_batches([60, 60, 60], 10, 8, 5 * 64, 128) == [[0, 1], [2]]
    # bounded by the context: 100 + 99 > 128 -> 128 positions = 2 pages
    assert plan_batches([100, 100], 100, 8, 4 * 64, 128) == [[0, 1]]
    assert plan_batches([5, 5, 5], 10, 8, 10_000, 128, max_slots=2) == [[0, 1], [2]]
    with pytest.raises(GenerationError, match="empty"):
        plan_batches([3, 0], 4, 2, 1000, 128)
    with pytest.raises(GenerationError, match="exceeds"):
        plan_batches([129], 4, 2, 1000, 128)
    with pytest.raises(GenerationError, match="cache has"):
        plan_batches([100], 100, 2, 64, 128)


def test_step_description_layout():
    lengths = {3: 0, 5: 70}
    tables = [lambda slots, w: np.arange(len(slots) * w, dtype=np.int32).reshape(len(slots), w)]
    h = build_step([(3, [9, 8, 7], [0, 2]), (5, [4], [0])], lengths, tables, max_blocks=2)
    lay, b = h.layout, h.packed
    assert (h.T, h.n, h.n_want, h.max_new, h.max_end, h.all_from_zero, h.all_single) == (4, 2, 3, 3, 71, False, False)
    assert b[lay.tokens:lay.tokens + 4].tolist() == [9, 8, 7, 4]
    assert b[lay.positions:lay.positions + 4].tolist() == [0, 1, 2, 70]
    assert b[lay.token_seq:lay.token_seq + 4].tolist() == [0, 0, 0, 1]
    assert b[lay.seq_slot:lay.seq_slot + 2].tolist() == [3, 5]
    assert b[lay.cu_new:lay.cu_new + 3].tolist() == [0, 3, 4]
    assert b[lay.want_rows:lay.want_rows + 3].tolist() == [0, 2, 3]
    assert b[lay.pages[0]:lay.pages[0] + 4].tolist() == [0, 1, 2, 3]
    assert all(off % 4 == 0 for off in (lay.tokens, lay.positions, lay.seq_slot, lay.want_rows, lay.pages[0]))
    assert b[lay.token_src:lay.token_src + 4].tolist() == [-1, -1, -1, -1]      # every token is the host's own
    # a padded one-token batch: dummy sequences of slot -1, every row wanted
    h = build_step([(5, [4], [])], lengths, tables, 2, pad_to=4, want_all=True)
    assert (h.T, h.n, h.n_want, h.all_single) == (4, 4, 4, True)
    assert h.packed[h.layout.seq_slot:h.layout.seq_slot + 4].tolist() == [5, -1, -1, -1]
    assert h.max_end == 71
    with pytest.raises(ValueError, match="wanted place"):
        build_step([(3, [1], [1])], lengths, tables, 2)
    # tokens that an earlier step's sampler left on the device: the row of each, padding has none
    h = build_step([(5, [0], []), (3, [0], [])], lengths, tables, 2, pad_to=4, want_all=True, token_rows=[2, 0])
    assert h.packed[h.layout.token_src:h.layout.token_src + 4].tolist() == [2, 0, -1, -1]
    with pytest.raises(ValueError, match="one token an entry"):
        build_step([(3, [1, 2], [])], lengths, tables, 2, token_rows=[0])


# ------------------------------------------------------------------------------ engine on the stand-in
@pytest.fixture(scope="module")
def cpu_engine(tiny_folders):
    return {name: Engine.from_folder(folder, dtype="float32", max_tokens=1024, device="cpu", ops=CpuOps())
            for name, folder in tiny_folders.items()}


def test_step_refusals_change_nothing(cpu_engine):
    eng = cpu_engine["tiny_a"]
    s = eng.open()
    for bad, word in [([(s, [], [])], "no tokens"), ([(s, [512], [0])], "vocabulary"), ([(s, [-1], [0])], "vocabulary"),
                      ([(s, [1, 2], [2])], "wanted place"), ([(s, [1] * 129, [])], "positions"),
                      ([(99, [1], [0])], "not open"), ([], "without sequences")]:
        with pytest.raises(StepError, match=word):
            eng.step(bad)
        assert eng.length(s) == 0
    eng.close(s)
    eng.cache.check()
    assert eng.cache.groups[0].pages.free == eng.cache.groups[0].pages.size


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_steps_equal_whole_sequences(cpu_engine, plains, name):
    """Prompts of unequal length in one step, then one token each (padded like a replayed
    graph), the shorter sequences leaving first, and a second batch in the slots of the first."""
    eng, plain = cpu_engine[name], plains[name]
    eng.cuda_graphs = True        # on the stand-in: the padded path without a capture
    try:
        first = [random_ids(i, plain.vocab, n) for i, n in enumerate((70, 30, 1))]
        rows, slots1 = run_batch(eng, first, (40, 9, 1))
        for ids, got in zip(first, rows):
            assert rel_error(got, plain.logits(ids)) < 1e-5
        second = [random_ids(5 + i, plain.vocab, n) for i, n in enumerate((45, 66))]
        rows, slots2 = run_batch(eng, second, (20, 65))
        for ids, got in zip(second, rows):
            assert rel_error(got, plain.logits(ids)) < 1e-5
        assert set(slots2) <= set(slots1)          # slots are used again
        eng.cache.check()
        assert eng.cache.slots.held == 0
    finally:
        eng.cuda_graphs = False


def test_one_token_steps_are_kept_per_bucket_of_batch_and_length(cpu_engine, plains):
    """The replayed one-token step is kept per bucket of batch sizes (powers of two) and of lengths
    (4, 6, 8, 12, 16, ... pages, at most what the cache gives a sequence); `capture_decode` makes a
    batch size's steps ahead of time, and a step then finds its bucket made."""
    eng, plain = cpu_engine["tiny_a"], plains["tiny_a"]
    top = eng.cache.max_blocks
    assert [eng._length_bucket(p) for p in (1, 4, 5, 6, 7, 9, 13, 17, 1000)] == [min(b, top) for b in (4, 4, 6, 6, 8, 12, 16, 24, 10 ** 9)]
    eng.cuda_graphs = True
    try:
        eng._graphs.clear()
        made = eng.capture_decode(3)
        lengths = sorted({eng._length_bucket(p) for p in range(1, top + 1)})
        assert made == len(lengths) and sorted(eng._graphs) == [(4, n) for n in lengths]
        assert eng.capture_decode(4) == 0                      # the same bucket: nothing new
        ids = [random_ids(40 + i, plain.vocab, 20) for i in range(3)]
        rows, _ = run_batch(eng, ids, (12, 12, 12))            # prompts, then eight one-token steps of three sequences
        for seq, got in zip(ids, rows):
            assert rel_error(got, plain.logits(seq)) < 1e-5
        assert sorted(eng._graphs) == [(4, n) for n in lengths]   # the steps found their bucket made
        eng.cache.check()
        assert eng.cache.slots.held == 0
    finally:
        eng.cuda_graphs = False
        eng._graphs.clear()


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_generate_equals_plain(tiny_folders, plains, name):
    plain = plains[name]
    stop = 7
    session = E.Session(tiny_folders[name], max_batch_size=2, dtype="float32", ops=CpuOps(), device="cpu", max_tokens=256)
    lens = (5, 17, 32, plain.n_positions - 3)
    prompts = [random_ids(10 + i, plain.vocab, n) for i, n in enumerate(lens)]
    seen = []
    session.set_token_callback(lambda i, tok: seen.append((i, tok)))
    got = session.generate_detailed(prompts, steps=6, temperature=0.9, top_k=50, top_p=0.95, stop_token_ids=[stop])
    for i, (p, g) in enumerate(zip(prompts, got)):
        want, why = plain_gpt2.generate(plain, p, 6, 0.9, 50, 0.95, seed=0, stream=i, stop_ids=(stop,))
        assert g.tokens == want and g.finish_reason == why
        assert [t for j, t in seen if j == i] == want
    assert got[3].finish_reason == "context" and len(got[3].tokens) == 4
    assert session.generator.stats["batches"] == 2
    session.engine.cache.check()
    assert session.engine.cache.slots.held == 0
    # greedy, and a second call continues the numbering of requests
    got = session.generate_batch(prompts[:2], steps=4, temperature=0.0)
    assert got == [plain_gpt2.generate(plain, p, 4)[0] for p in prompts[:2]]


def test_stop_token_ends_a_sequence_early(tiny_folders, plains):
    plain = plains["tiny_a"]
    session = E.Session(tiny_folders["tiny_a"], max_batch_size=3, dtype="float32", ops=CpuOps(), device="cpu",
                        max_tokens=512)
    prompts = [random_ids(20 + i, plain.vocab, 6 + i) for i in range(3)]
    free = session.generate_detailed(prompts, steps=8, temperature=1.0, top_k=0, top_p=1.0, stop_token_ids=[])
    stop = free[1].tokens[2]              # make the second request stop at its third token
    session.set_seed(0)                   # the same seed and the requests numbered from 0 again
    again = session.generate_detailed(prompts, steps=8, temperature=1.0, top_k=0, top_p=1.0, stop_token_ids=[stop])
    assert again[1].finish_reason == "stop" and again[1].tokens[-1] == stop and len(again[1].tokens) <= 3
    for g, f in zip(again, free):
        n = len(g.tokens)
        assert g.tokens == f.tokens[:n]   # what the others generate does not depend on who left
    assert session.engine.cache.slots.held == 0


def test_running_a_step_ahead_changes_no_token(tiny_folders, plains):
    """The loop queues step t+1 with the ids of step t still on the device and reads them
    afterwards.  Against the loop that reads every id before it goes on: the same tokens, reasons
    and callback order, with stop ids (whose sequences are stepped once for nothing), counts that
    run out at different steps and a prompt that ends at the context's end; no slot is left."""
    plain = plains["tiny_b"]
    prompts = [random_ids(30 + i, plain.vocab, n) for i, n in enumerate((3, 20, plain.n_positions - 2, 8, 1))]
    out = []
    for ahead in (True, False):
        session = E.Session(tiny_folders["tiny_b"], max_batch_size=4, dtype="float32", ops=CpuOps(), device="cpu",
                            max_tokens=512)
        session.generator.run_ahead = ahead
        free = session.generate_detailed(prompts, steps=7, temperature=1.0, top_k=0, top_p=1.0, stop_token_ids=[])
        stops = [free[0].tokens[1], free[3].tokens[4]]
        session.set_seed(0)
        seen = []
        session.set_token_callback(lambda i, tok: seen.append((i, tok)))
        got = session.generate_detailed(prompts, steps=7, temperature=1.0, top_k=0, top_p=1.0, stop_token_ids=stops)
        out.append(([(g.tokens, g.finish_reason) for g in free], [(g.tokens, g.finish_reason) for g in got], seen))
        assert got[0].finish_reason == "stop" and got[2].finish_reason == "context" and len(got[2].tokens) == 3
        session.engine.cache.check()
        assert session.engine.cache.slots.held == 0
    assert out[0] == out[1]
    for i, p in enumerate(prompts):
        want, why = plain_gpt2.generate(plain, p, 7, 1.0, 0, 1.0, seed=0, stream=i, stop_ids=tuple(stops))
        assert out[0][1][i] == (want, why)


def test_tokens_taken_from_the_device_equal_tokens_from_the_host(cpu_engine, plains):
    eng, plain = cpu_engine["tiny_a"], plains["tiny_a"]
    a, b = random_ids(40, plain.vocab, 9), random_ids(41, plain.vocab, 4)
    import torch
    rows = []
    for device in (False, True):
        s0, s1 = eng.open(), eng.open()
        eng.step([(s0, a[:-1], []), (s1, b[:-1], [])])
        ids = torch.tensor([7, b[-1], 3, a[-1]], dtype=torch.int32)       # as a sampler would have left them
        if device:
            out = eng.step([(s0, [0], [0]), (s1, [0], [0])], device_tokens=(ids, [3, 1]))
        else:
            out = eng.step([(s0, [a[-1]], [0]), (s1, [b[-1]], [0])])
        rows.append(out.clone())
        eng.close(s0)
        eng.close(s1)
    assert torch.equal(rows[0], rows[1])
    s0 = eng.open()
    with pytest.raises(StepError, match="taken from the device"):
        eng.step([(s0, [1, 2], [])], device_tokens=(torch.zeros(2, dtype=torch.int32), [0]))
    with pytest.raises(StepError, match="taken from the device"):
        eng.step([(s0, [1], [])], device_tokens=(torch.zeros(2, dtype=torch.int32), [2]))
    assert eng.length(s0) == 0
    eng.close(s0)


def test_session_refuses_what_is_not_built(tiny_folders):
    with pytest.raises(ValueError, match="n_gpu_layers"):
        E.Session(tiny_folders["tiny_a"], n_gpu_layers=0, ops=CpuOps(), device="cpu")
    with pytest.raises(ValueError, match="use_kv_quant"):
        E.Session(tiny_folders["tiny_a"], use_kv_quant=True, ops=CpuOps(), device="cpu")
