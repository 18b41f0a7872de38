"""How the decode attention's launch is cut (`csrc/ops.py: decode_chunks`): a rule of the host, checked without a GPU."""
import pytest

from ember_cpp_b200.csrc.ops import decode_chunks

SMS, SLOTS = 148, 6 * 148


@pytest.mark.parametrize("four_warps", [False, True])
@pytest.mark.parametrize("pairs", [1, 25, 200, 400, 1600, 5000])
def test_every_page_is_in_exactly_one_chunk_and_chunks_fit_a_cluster_or_the_scratch(pairs, four_warps):
    for blocks in range(1, 130):
        n = decode_chunks(blocks, pairs, SMS, SLOTS, four_warps)
        per_chunk = -(-blocks // n)              # what the kernel is given: pages a chunk ...
        launched = -(-blocks // per_chunk)       # ... from which it takes its number of chunks
        assert 1 <= launched <= n <= blocks
        assert launched * per_chunk >= blocks > (launched - 1) * per_chunk   # every page in a chunk, no chunk empty
        if n > 1:
            assert per_chunk >= 2                                     # a block's fixed costs are shared by 128 keys and more
        assert n * pairs <= max(SLOTS, pairs)                         # the launch is resident at once, or is not cut at all


def test_the_cuts_of_the_benchmarks_shapes():
    """GPT-2 XL's 25 heads: (batch, pages) -> chunks, with the tensor-core kernel's blocks of four warps."""
    pages = (1, 2, 3, 4, 6, 8, 12, 16)
    assert [decode_chunks(p, 25, SMS, SLOTS, True) for p in pages] == [1, 1, 1, 1, 2, 2, 3, 4]        # batch 1
    assert [decode_chunks(p, 200, SMS, SLOTS, True) for p in pages] == [1, 1, 1, 1, 2, 2, 2, 2]       # batch 8
    assert [decode_chunks(p, 1600, SMS, SLOTS, True) for p in pages] == [1] * 8                       # batch 64: never cut
    assert [decode_chunks(p, 200, SMS, SLOTS, False) for p in pages] == [1, 1, 2, 2, 3, 4, 4, 4]      # two-warp blocks only


def test_four_warp_blocks_are_all_resident_at_three_an_sm():
    for pairs in (25, 100, 200, 400):
        for blocks in range(3, 65):
            n = decode_chunks(blocks, pairs, SMS, SLOTS, True)
            per_chunk = -(-blocks // n)
            if n * pairs <= 3 * SMS and per_chunk >= 3:   # what the launch code takes four warps for
                assert per_chunk <= 8 or n == decode_chunks(blocks, pairs, SMS, SLOTS, False)
