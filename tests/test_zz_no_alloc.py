"""The decode attention entry point that allocates nothing (`ember_attention_decode_static`).

Some programs that embed these kernels cannot allocate device memory while they run: they handed the
whole GPU to a pool of their own, or they run under a budget that was checked once, or they call
from a place where `cudaMalloc`'s device synchronisation is not acceptable.  For them the library
carries the split decode attention's scratch inside itself, as fixed `__device__` arrays.  This test
calls that entry point the way such a program would, through its exported C symbol and with nothing
but raw pointers, and checks it against the ordinary entry point (which gets its scratch from the
caller) on two calls in a row: the second call finds the first one's leftovers in the scratch.

The file is named so that pytest collects it last.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from ember_cpp_b200.cache import PAGE, SequenceCache
from ember_cpp_b200.engine import StepPlan, build_step
from ember_cpp_b200.parts import CacheNeed

pytestmark = pytest.mark.gpu

I, F, P = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def load_symbol():
    from ember_cpp_b200.csrc import build
    lib = ctypes.CDLL(build.library_path())
    fn = lib.ember_attention_decode_static
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P]
    fn.restype = I
    lib.ember_last_error.restype = ctypes.c_char_p
    return lib, fn


def make_case(heads, kv_heads, hd, lengths, seed):
    """A cache that holds `lengths[i]` positions of sequence i, and a step of one new token each."""
    need = CacheNeed("full", kv_heads, hd)
    pages = sum(-(-(n + 1) // PAGE) for n in lengths) + 2
    cache = SequenceCache([(need, None)], [None], pages * PAGE, None, torch.bfloat16, "cuda")
    view = cache.views[0]
    g = torch.Generator().manual_seed(seed)
    view.k.copy_(torch.randn(view.k.shape, generator=g).to(torch.bfloat16))   # every page holds keys and values
    view.v.copy_(torch.randn(view.v.shape, generator=g).to(torch.bfloat16))
    slots = [cache.open() for _ in lengths]
    cache.reserve(list(zip(slots, lengths)))
    cache.commit(list(zip(slots, lengths)))
    cache.reserve([(s, 1) for s in slots])
    host = build_step([(s, [0], []) for s in slots], cache.lengths, [cache.groups[0].table], cache.max_blocks)
    plan = StepPlan(host, torch.from_numpy(host.packed).cuda())
    qkv = torch.randn(len(lengths), (heads + 2 * kv_heads) * hd, generator=g).to(torch.bfloat16).cuda()
    return cache, view, plan, qkv


def test_static_scratch_equals_callers_scratch_twice_in_a_row():
    from ember_cpp_b200.csrc.ops import CudaOps
    ops = CudaOps()
    ops.decode_mma = False         # the kernel that the static entry point runs, so that the results are equal bit for bit
    lib, static = load_symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # the second call has other sizes, so it reads scratch that the first call wrote differently
    for call, (heads, kv_heads, hd, lengths) in enumerate([(6, 2, 64, (300, 63, 64, 1, 129)), (4, 4, 32, (700, 5))]):
        cache, view, plan, qkv = make_case(heads, kv_heads, hd, lengths, seed=call)
        scale = 1.0 / math.sqrt(hd)
        k_before, v_before = view.k.clone(), view.v.clone()
        want = ops.attention(qkv, view, plan, heads, kv_heads, hd, scale, 0, torch.bfloat16, store=True)
        k_after, v_after = view.k.clone(), view.v.clone()
        view.k.copy_(k_before)
        view.v.copy_(v_before)
        got = torch.empty_like(want)
        blocks = min(plan.max_blocks, -(-plan.max_end // PAGE))
        rc = static(qkv.data_ptr(), view.k.data_ptr(), view.v.data_ptr(), got.data_ptr(), plan.positions.data_ptr(),
                    plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), plan.pages[0].data_ptr(), plan.max_blocks, blocks,
                    plan.T, heads, kv_heads, hd, scale, 0, min(2, blocks), 1, stream)
        assert rc == 0, lib.ember_last_error().decode()
        torch.cuda.synchronize()
        # the tolerance of the kernel tests for bfloat16 outputs; the two entry points run the same kernel
        assert (got.float() - want.float()).abs().max().item() < 2e-2
        assert torch.equal(got, want)
        assert torch.equal(view.k, k_after) and torch.equal(view.v, v_after)     # it stored the new keys and values too


def test_static_scratch_refuses_what_does_not_fit():
    lib, static = load_symbol()
    cache, view, plan, qkv = make_case(2, 2, 16, (10,), seed=3)
    out = torch.empty(1, 32, dtype=torch.bfloat16, device="cuda")
    args = [qkv.data_ptr(), view.k.data_ptr(), view.v.data_ptr(), out.data_ptr(), plan.positions.data_ptr(),
            plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), plan.pages[0].data_ptr(), plan.max_blocks, 1]
    tail = [2, 16, 0.25, 0, 1, 0, torch.cuda.current_stream().cuda_stream]
    assert static(*args, 20000, 2, *tail) != 0 and b"scratch" in lib.ember_last_error()       # too many (token, head) pairs
    assert static(*args[:-1], 4000, 4, 4, 2, 256, 0.25, 0, 1, 0, tail[-1]) != 0               # too many partial results
    assert b"floats of scratch" in lib.ember_last_error()
