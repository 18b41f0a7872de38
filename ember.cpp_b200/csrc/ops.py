"""The kernels as the parts call them.

`CudaOps` is the only implementation the library ships: it loads the shared library that
build.py makes from this folder's CUDA sources and calls its C entry points on torch's current
stream with raw device pointers.  There is no CPU path and no fallback to library model code; a
missing compiler, a failed build or a missing GPU is an error at construction.

Which kernel runs is decided here from the element types and the shape of the step:
float32 operands take the float32 kernels (FFMA product in a fixed order, plain attention),
bfloat16 operands take the tensor-core kernels.
"""
from __future__ import annotations

import ctypes

import torch

from . import build

_F32, _BF16 = 0, 1
_ACT = {None: 0, "gelu_tanh": 1, "gelu_erf": 2}
_LT_WORKSPACE = 32 << 20

_c_int, _c_float, _c_void, _c_size, _c_u64 = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64

_SIGNATURES = {
    "ember_embed": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ember_layernorm": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_gather_rows": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ember_take_tokens": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ember_act_inplace": [_c_void, _c_size, _c_int, _c_int, _c_void],
    "ember_scale_cap_inplace": [_c_void, _c_size, _c_float, _c_float, _c_void],
    "ember_gemm_f32": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_linear_bf16": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_void, _c_size, _c_void, _c_void],
    "ember_linear_tc": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_linear_stream": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_void, _c_size, _c_void],
    "ember_linear_decode": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void,
                            _c_size, _c_void],
    "ember_clear_tails": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ember_kv_store": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_void],
    "ember_attention_plain": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int,
                              _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void],
    "ember_attention_decode": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void],
    "ember_attention_decode_ahead": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                     _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                                     _c_int, _c_void, _c_void, _c_void],
    "ember_attention_decode_mma": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void,
                                   _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                   _c_int, _c_int, _c_void, _c_void, _c_void],
    "ember_attention_prefill": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_attention_prefill_tc": [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ember_sample": [_c_void, _c_void, _c_int, _c_int, _c_float, _c_int, _c_float, _c_u64, _c_void, _c_void, _c_u64, _c_void],
}


class KernelError(RuntimeError):
    pass


SMALL_M = 16          # rows up to which the mma.sync weight-streaming product (linear_decode.cu) is used
STREAM_M = 64         # rows up to which the tcgen05 weight-streaming product (linear_stream.cu) is used above that
TC_MIN_M = 64         # rows above which the tcgen05 product is used (its tiles have 128 rows)


def _current_stream() -> int:
    """The handle of torch's current stream on the current device.  Asked for at every launch, so by the shortest
    way torch has (a launch costs the host a few microseconds in all, and a prompt's step is some 500 launches)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is None:
        return torch.cuda.current_stream().cuda_stream
    return raw(torch.cuda.current_device())


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {dtype} is neither float32 nor bfloat16")


def load_library() -> ctypes.CDLL:
    """Builds the library if needed and loads it; every failure is an error that says why."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible: this library runs models on a GPU only")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
    path = build.library_path()
    lib = ctypes.CDLL(path)
    lib.ember_last_error.restype = ctypes.c_char_p
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = _c_int
    lib.ember_umma_issue_probe.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void]
    lib.ember_umma_issue_probe.restype = _c_int
    lib.ember_wait_probe.argtypes = [_c_u64, _c_void]
    lib.ember_wait_probe.restype = _c_int
    lib.ember_set_option.argtypes = [_c_int, _c_int]
    lib.ember_set_option.restype = _c_int
    lib.ember_attention_decode_partials.argtypes = [_c_int] * 5
    lib.ember_attention_decode_partials.restype = _c_size
    for name in ("ember_tc_status", "ember_linear_decode_status", "ember_attention_decode_status",
                 "ember_attention_decode_mma_status"):
        getattr(lib, name).argtypes = []
        getattr(lib, name).restype = _c_int
    lib._path = path
    return lib


def decode_chunks(blocks: int, pairs: int, sms: int, slots: int, four_warps: bool) -> int:
    """Into how many chunks the decode attention cuts a context of `blocks` pages, each chunk a block of the
    launch, for `pairs` (token, head) pairs on a chip of `sms` SMs that holds `slots` two-warp blocks at once.

    The context is cut so that the launch fills the chip once: as many chunks as resident blocks per pair
    allow, at least two pages each (a block's fixed costs are then shared by 128 keys).  Pairs that fill the
    chip by themselves are not cut: their blocks write the output directly, with no partial results to
    merge.  (A block that waits for an SM starts its copies late: a step of 12 layers at batch 8 and a
    context of 900 to 1,024 0.557 against 0.593 ms.)

    four_warps (head size 64 on the tensor cores): while chunks of up to four pages (else of up to eight)
    are few enough for three blocks of four warps an SM to hold them all, the chunks are that long and a block
    has four warps, a page each at a time: fewer blocks to merge (none up to four pages), and four pages of a
    chunk on their way from the block's start.  (GPT-2 XL at batch 8: the first steps 1.312 -> 1.260 ms, the
    sweep to 1,024 tokens 1.433 -> 1.414.)"""
    n_chunks = max(1, min(slots // max(pairs, 1), -(-blocks // 2)))
    if four_warps and blocks > 2:
        for longest in (4, 8):
            n = -(-blocks // longest)
            if n <= 8 and n * pairs <= 3 * sms:
                return n
    return n_chunks


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, options=None):
        """`options`: a RuntimeOptions; None takes the defaults with the EMBER_* variables laid on top."""
        from ..options import RuntimeOptions
        self.options = options = options if options is not None else RuntimeOptions.from_env()
        self.lib = load_library()
        self._workspace = None
        self._partials = None          # scratch of the decode attention: partial results ...
        self._counters = None          # ... and its per-(token, head) counters, zero between calls
        self._retired = []             # outgrown scratch stays alive: captured graphs may still name it
        self.launches = 0
        self.sms = torch.cuda.get_device_properties(0).multi_processor_count
        self.decode_slots = 6 * self.sms   # blocks of the decode attention that are resident at once
        # What the switches are and why their defaults are what they are (all measured on GPT-2 XL's shapes):
        # cache_ahead: a decode attention asks the next layer's rows of the cache into L2.  Off: with the kernel
        #   that loads keys into registers the step's time did not change (0.5822 against 0.5820 ms of 12 layers);
        #   with the tensor-core kernel it grew (0.538 against 0.516 ms): a layer's rows and weights together do
        #   not stay in L2 that long, and the rows are then fetched twice.
        self.cache_ahead = options.cache_ahead
        # decode_mma: decode attention on the tensor cores where that kernel has an instantiation (head size 64
        #   or 128, up to 8 query heads to a key/value head); off takes the other kernel.
        self.decode_mma = options.decode_mma
        self._warm = None              # tensor announced by `warm` for the next product
        self._coming = []              # weight matrices announced by `announce_weights`, in the order their products run
        # warm: the second product of a feed-forward has its weights landed about a microsecond earlier with it
        #   (its blocks cannot be resident beside the first product's); a step of 12 layers 0.519 against 0.521 ms.
        self.warm_ahead = options.warm
        # gemm: products of more than STREAM_M rows go to cuBLASLt ("lt"), as ember.cpp's own go to cuBLAS, or
        #   ("tc"), above TC_MIN_M rows, to this library's tcgen05 kernel.  On GPT-2 XL's four products the
        #   library is ahead at 2,048 rows; at 16,384 rows the tcgen05 kernel reaches 95 % of it on the QKV product.
        self.gemm = options.gemm
        # lt_tune: the first product of a shape times the library's candidate algorithms; `deterministic` turns
        #   it off, so that the choice does not depend on a timing
        self.lt_tune = options.lt_tune
        self._lt_tuned = set()
        # linear_stream: products of SMALL_M + 1 to STREAM_M rows stream the weights through this library's tcgen05
        #   kernel with the operands swapped (linear_stream.cu); off sends them to cuBLASLt.
        self.linear_stream_on = options.linear_stream
        # attention: prefill attention with head size 64 on the tcgen05 kernel, or ("mma") on the mma.sync kernel
        #   (which takes every other head size anyway)
        self.attention_tc = options.attention == "tc"
        # op_timing, nvtx: per-launch CUDA events and NVTX ranges (see options.py); both off by default
        self.op_timing, self.nvtx = options.op_timing, options.nvtx
        self._timed = []
        # the three switches that the kernels' launch code reads (process-wide)
        for which, value in ((0, options.pdl), (1, options.decode_bulk), (2, options.decode_cluster)):
            self.lib.ember_set_option(which, 1 if value else 0)

    # ------------------------------------------------------------------ helpers
    def _call(self, name: str, *args, allow=()) -> int:
        timed = self.op_timing and not torch.cuda.is_current_stream_capturing()
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if timed:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
        rc = getattr(self.lib, name)(*args, _current_stream())
        if timed:
            end.record()
            self._timed.append((name, begin, end))
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        if rc in allow:
            return rc
        self.launches += 1
        if rc != 0:
            raise KernelError(self.lib.ember_last_error().decode())
        return 0

    def op_times(self, reset: bool = True) -> dict:
        """With the `op_timing` option: {entry point: (launches, milliseconds)} since the last call, from CUDA
        events around every launch (an event between two launches keeps them from overlapping, so the sum is
        more than a step takes: read the shares).  Synchronizes with the device."""
        torch.cuda.synchronize()
        out: dict = {}
        for name, begin, end in self._timed:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + begin.elapsed_time(end))
        if reset:
            self._timed = []
        return out

    def _decode_scratch(self, n_partials: int, n_counters: int):
        if self._partials is None or self._partials.numel() < n_partials:
            self._retired.append(self._partials)
            self._partials = torch.empty(max(n_partials, 1 << 20), dtype=torch.float32, device="cuda")
        if self._counters is None or self._counters.numel() < n_counters:
            self._retired.append(self._counters)
            self._counters = torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device="cuda")
        return self._partials, self._counters

    @staticmethod
    def _ptr(t):
        return None if t is None else t.data_ptr()

    @staticmethod
    def _dense(t: torch.Tensor, what: str) -> torch.Tensor:
        if not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what} must be a contiguous CUDA tensor")
        return t

    def _lt_workspace(self) -> torch.Tensor:
        if self._workspace is None:
            self._workspace = torch.empty(_LT_WORKSPACE, dtype=torch.uint8, device="cuda")
        return self._workspace

    @staticmethod
    def _bias_bf16(bias: torch.Tensor) -> torch.Tensor:
        """The bfloat16 copy of a bias that cuBLASLt's epilogue reads.  It is kept on the bias tensor itself
        (made once, dies with it): a cache keyed by address would hand a freed model's copy to a new model
        whose bias landed on the same address."""
        copy = getattr(bias, "_ember_bf16", None)
        if copy is None or copy.shape != bias.shape or copy.device != bias.device:
            copy = bias.to(torch.bfloat16)
            bias._ember_bf16 = copy
        return copy

    # ------------------------------------------------------------------ rows
    def embed(self, tokens, positions, table, pos_table, token_src=None, ids=None):
        """Rows of the token table (plus rows of the position table) in float32.  With `token_src` and `ids`
        (int32, on the device) token t is ids[token_src[t]] where token_src[t] >= 0: an id that an earlier
        step's sampler left there."""
        T, d = tokens.shape[0], table.shape[1]
        if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != d):
            raise KernelError("embed: the position table must have the token table's type and width")
        if (token_src is None) != (ids is None):
            raise KernelError("embed: tokens from the device need both their rows and the ids")
        if ids is not None and (ids.dtype != torch.int32 or not ids.is_cuda or not ids.is_contiguous()):
            raise KernelError("embed: sampled ids are a contiguous int32 CUDA tensor")
        x = torch.empty((T, d), dtype=torch.float32, device=table.device)
        self._call("ember_embed", tokens.data_ptr(), positions.data_ptr(), self._dense(table, "token table").data_ptr(),
                   self._ptr(pos_table), x.data_ptr(), T, d, _code(table.dtype), self._ptr(token_src), self._ptr(ids),
                   0 if ids is None else ids.numel(), table.shape[0])
        return x

    def warm(self, tensor) -> None:
        """Announces constants that a kernel soon after the next product reads (the weights of the product
        after it).  A hint: a small product's kernel asks them into L2 while it waits for its own input."""
        fits = tensor is not None and tensor.numel() * tensor.element_size() <= self.AHEAD_BYTES
        self._warm = tensor if self.warm_ahead and fits else None

    def announce_weights(self, weights) -> None:
        """Announces the weight matrices of the products to come, in the order they run (a block announces
        its own and the first of what follows it).  A hint: a product of 17 to 64 rows asks the matrix after
        its own into L2, so that the next product's ring refills from there and not from DRAM."""
        self._coming = [w for w in weights if w is not None]

    def _after(self, w):
        """The announced matrix that follows `w`, if it is worth asking into L2 (it fits there with room to spare)."""
        if not self.warm_ahead:
            return None
        for i, c in enumerate(self._coming[:-1]):
            if c.data_ptr() == w.data_ptr():
                nxt = self._coming[i + 1]
                return nxt if nxt.numel() * nxt.element_size() <= self.AHEAD_BYTES else None
        return None

    def layernorm(self, x, w, b, eps, out_dtype):
        """Layer norm of float32 rows."""
        rows, d = x.shape
        if x.dtype != torch.float32 or w.dtype != torch.float32 or b.dtype != torch.float32:
            raise KernelError("layernorm: input, gain and bias are float32")
        if w.shape[0] != d or b.shape[0] != d:
            raise KernelError(f"layernorm: width {d} with gain {tuple(w.shape)} and bias {tuple(b.shape)}")
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        self._call("ember_layernorm", self._dense(x, "layernorm input").data_ptr(), w.data_ptr(), b.data_ptr(),
                   out.data_ptr(), rows, d, float(eps), _code(out_dtype))
        return out

    AHEAD_BYTES = 48 << 20   # rows of one layer's cache that are worth asking into L2 a layer early

    TIMELINE_KERNELS = {1: "embed", 2: "layernorm", 3: "linear_decode", 4: "attention_decode", 5: "sample", 6: "linear_stream"}
    TIMELINE_FILES = ("elementwise", "linear_decode", "linear_stream", "attention_decode", "attention_decode_mma", "sampling")

    def timeline(self):
        """What the kernels of a library built with EMBER_TIMELINE=1 noted since the last call: a list of
        (nanoseconds, kernel name, mark, block, blocks of the launch, SM) sorted by time; mark 0 = the block
        started, 1 = its wait for the kernel in front returned, 2 = it ended (3: it ended after merging
        the partial results of a decode attention), 4 to 7 = places in between that the kernel's source
        names.  Synchronizes with the device."""
        import struct
        if not hasattr(self.lib, "ember_timeline_read_elementwise"):
            raise KernelError("this library was built without EMBER_TIMELINE=1")
        cap, out = 1 << 18, []
        buf = ctypes.create_string_buffer(cap * 24)
        for name in self.TIMELINE_FILES:
            fn = getattr(self.lib, f"ember_timeline_read_{name}")
            fn.argtypes, fn.restype = [_c_void, ctypes.c_uint], _c_int
            n = fn(ctypes.cast(buf, ctypes.c_void_p), cap)
            if n < 0:
                raise KernelError(f"timeline: reading the log of {name}.cu failed")
            for i in range(n):
                t, what, block, grid, sm = struct.unpack_from("<QIIII", buf, i * 24)
                if t:
                    out.append((t, self.TIMELINE_KERNELS.get(what >> 8, str(what >> 8)), what & 255, block, grid, sm))
        out.sort()
        return out

    def scale_cap(self, x, scale: float = 1.0, cap: float | None = None):
        """x <- scale * x, then (with a cap) cap * tanh(x / cap), in place on float32 values: a factor on
        the embedded rows, a cap on the logits."""
        if x.dtype != torch.float32:
            raise KernelError("scale_cap: float32 values (the residual stream, the logits)")
        self._call("ember_scale_cap_inplace", self._dense(x, "values").data_ptr(), x.numel(), float(scale),
                   0.0 if cap is None else float(cap))
        return x

    def take_tokens(self, tokens, token_src, ids, vocab_size: int) -> None:
        """tokens[i] = ids[token_src[i]] where token_src[i] >= 0: a step's tokens taken from an earlier
        step's sampled ids on the device."""
        if ids.dtype != torch.int32 or not ids.is_cuda or not ids.is_contiguous():
            raise KernelError("take_tokens: sampled ids are a contiguous int32 CUDA tensor")
        self._call("ember_take_tokens", tokens.data_ptr(), token_src.data_ptr(), ids.data_ptr(), tokens.shape[0],
                   ids.numel(), int(vocab_size))

    def gather_rows(self, x, rows, n_rows):
        out = torch.empty((n_rows, x.shape[1]), dtype=torch.float32, device=x.device)
        self._call("ember_gather_rows", self._dense(x, "rows").data_ptr(), rows.data_ptr(), out.data_ptr(), n_rows,
                   x.shape[1])
        return out

    # ------------------------------------------------------------------ products
    def linear(self, a, w, bias, act=None, residual=None, out_dtype=None):
        """y = a w^T (+ bias) (activation) (+ residual).  `w` is [out, in].  With a residual the
        sum is made in float32 into the residual's buffer, which is returned."""
        if act not in _ACT:
            raise KernelError(f"linear: activation {act!r}")
        warm, self._warm = self._warm, None
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: input width {K} does not match the weight's {tuple(w.shape)}")
        if a.dtype != w.dtype:
            raise KernelError(f"linear: input is {a.dtype}, weight is {w.dtype}")
        if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != N):
            raise KernelError("linear: the bias is float32 of the output's width")
        if residual is not None and (residual.dtype != torch.float32 or tuple(residual.shape) != (M, N)):
            raise KernelError("linear: the residual is float32 of the output's shape")
        self._dense(a, "linear input")
        self._dense(w, "linear weight")
        if w.dtype == torch.float32:
            out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=a.device)
            self._call("ember_gemm_f32", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual),
                       out.data_ptr(), M, N, K, _ACT[act])
            return out if out_dtype in (None, torch.float32) or residual is not None else out.to(out_dtype)
        target = torch.float32 if residual is not None else (out_dtype or torch.bfloat16)
        out = residual if residual is not None else torch.empty((M, N), dtype=target, device=a.device)
        # A matrix that fills L2 by itself (a vocabulary head) streams faster through the tcgen05 kernel from 9
        # rows on (GPT-2 XL's head at 16 rows: 34.7 against 48.0 microseconds; at 8 rows 32.9 against 27.4).
        big = w.numel() * 2 > (64 << 20) and M > 8 and self.linear_stream_on
        if M <= SMALL_M and K % 8 == 0 and K <= 16384 and not big:
            # (Only a matrix that a part announced with `warm` is asked into L2 here.  Every product asking for the
            # next announced matrix paid at 8 rows once, 1.556 -> 1.512 ms a step of GPT-2 XL, and costs since the
            # launches spread over the chip: 1.307 against 1.280 ms.)
            self._call("ember_linear_decode", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                       M, N, K, _ACT[act], _code(target), None if warm is None else warm.data_ptr(),
                       0 if warm is None else warm.numel() * warm.element_size() // 16 * 16)
            return out
        if self.linear_stream_on and M <= STREAM_M and K % 8 == 0:
            return self.linear_stream(a, w, bias, act, residual, out, warm=warm if warm is not None else self._after(w))
        # an output width that is no multiple of 8 (a vocabulary of 50,257) leaves the library only unaligned,
        # slow kernels (167 against 50 microseconds for the head at 64 rows): those products take the tcgen05 kernel
        if K % 8 == 0 and ((self.gemm == "tc" and M > TC_MIN_M) or N % 8 != 0):
            return self.linear_tc(a, w, bias, act, residual, out)
        fused = _ACT[act] if act != "gelu_erf" else 0
        ws = self._lt_workspace()
        # the first product of a shape times the library's candidates into a scratch output (outside any capture)
        shape = (M, N, K, fused, bias is not None, residual is not None, target)
        scratch = None
        # (large products only, and a bounded number of shapes: timing costs a few milliseconds a shape)
        if (self.lt_tune and M >= 64 and shape not in self._lt_tuned and len(self._lt_tuned) < 512
                and not torch.cuda.is_current_stream_capturing()):
            self._lt_tuned.add(shape)
            scratch = torch.empty_like(out)
        self._call("ember_linear_bf16", a.data_ptr(), w.data_ptr(), self._ptr(bias),
                   None if bias is None else self._bias_bf16(bias).data_ptr(), self._ptr(residual), out.data_ptr(),
                   M, N, K, fused, _code(target), ws.data_ptr(), ws.numel(), self._ptr(scratch))
        if act == "gelu_erf":
            self._call("ember_act_inplace", out.data_ptr(), out.numel(), _ACT[act], _code(target))
        return out

    def linear_tc(self, a, w, bias, act, residual, out, tile_n: int = 0):
        """The tcgen05 product with its epilogue (bias, activation, float32 residual sum) into `out`."""
        M, K = a.shape
        self._call("ember_linear_tc", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                   M, w.shape[0], K, _ACT[act], _code(out.dtype), tile_n)
        return out

    def linear_stream(self, a, w, bias, act, residual, out, k_split: int = 0, stages: int = 0, warm=None):
        """The tcgen05 weight-streaming product for up to 64 rows with its epilogue into `out`; `k_split` and
        `stages` 0 let the kernel choose how many blocks share a tile and how deep its ring is; `warm`: a tensor
        that the launch asks into L2 (the next product's weights)."""
        M, K = a.shape
        self._call("ember_linear_stream", a.data_ptr(), w.data_ptr(), self._ptr(bias), self._ptr(residual), out.data_ptr(),
                   M, w.shape[0], K, _ACT[act], _code(out.dtype), int(k_split), int(stages),
                   None if warm is None else warm.data_ptr(), 0 if warm is None else warm.numel() * warm.element_size() // 16 * 16)
        return out

    def umma_issue_probe(self, m: int, n: int, iters: int = 512, elected: bool = True, commit_every: int = 0, wait_too: bool = False):
        """(cycles to issue, cycles until complete) per `tcgen05.mma` of M = m, N = n, K = 16, issued from a single
        thread's branch or by a converged warp with elect.sync (umma_probe.cu).  A measurement for the notes."""
        out = torch.zeros(3, dtype=torch.int64, device="cuda")
        self._call("ember_umma_issue_probe", int(m), int(n), int(iters), 1 if elected else 0, int(commit_every), 1 if wait_too else 0, out.data_ptr())
        issue, done, ended = out.tolist()
        if not ended:
            raise KernelError("umma_issue_probe: the products did not complete within the wait's limit")
        return issue / iters, done / iters

    def wait_probe(self, limit_ns: int = 1_000_000) -> None:
        """Launches the kernel whose only wait nothing ends (wait_probe.cu): it gives up after `limit_ns`
        and leaves code 31 in the status word, which the next `check()` raises for.  For tests of the
        kernels' bounded waits; nothing faults or hangs."""
        self._call("ember_wait_probe", int(limit_ns))

    def check(self) -> None:
        """Raises if a kernel with bounded waits gave up since the last call.  The caller has
        synchronized with the device (it has just read a step's results)."""
        if self.lib.ember_linear_decode_status():
            raise KernelError("linear_decode: a block gave up waiting for its weight copies; the results of that launch are not valid")
        if self.lib.ember_attention_decode_status() or self.lib.ember_attention_decode_mma_status():
            raise KernelError("attention_decode: a block gave up waiting for its copies of keys and values; the results of that launch are not valid")
        code = self.lib.ember_tc_status()
        if code:
            kernel = "linear_tc" if code < 10 else ("attention_prefill_tc" if code < 20 else
                                                    ("linear_stream" if code < 30 else "wait_probe"))
            role = {31: "the probe's wait, as it is meant to",1: "the TMA producer", 2: "the product issuer", 3: "the epilogue", 4: "copies in flight",
                    11: "the TMA loader", 12: "the product issuer", 13: "the softmax warps",
                    21: "the TMA producer", 22: "the product issuer", 23: "the epilogue", 24: "copies in flight"}.get(code, code)
            raise KernelError(f"{kernel}: a wait ran out ({role}); the results of that launch are not valid")

    # ------------------------------------------------------------------ cache and attention
    def clear_tails(self, group, tails) -> None:
        """Zeroes, in every key and value tensor of a cache group, the rows from `row` on of each page
        named in tails [n, 2] = (page, row) (page < 0: nothing)."""
        table = getattr(group, "_tensor_table", None)
        if table is None:      # the addresses of the group's tensors, once
            tensors = list(group.k) + list(group.v)
            table = group._tensor_table = torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=tensors[0].device)
        need = group.need
        self._call("ember_clear_tails", table.data_ptr(), table.numel(), tails.data_ptr(), tails.shape[0], need.kv_heads,
                   need.head_dim, group.k[0].element_size())

    def kv_store(self, qkv, cache, plan, n_heads, kv_heads, head_dim):
        if qkv.dtype != cache.k.dtype:
            raise KernelError(f"kv_store: activations are {qkv.dtype}, the cache is {cache.k.dtype}")
        self._call("ember_kv_store", self._dense(qkv, "qkv").data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                   plan.positions.data_ptr(), plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(),
                   plan.pages[cache.group_index].data_ptr(), plan.max_blocks, plan.T, n_heads, kv_heads, head_dim,
                   _code(qkv.dtype))

    def attention(self, qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store=False):
        """Causal attention of the step's tokens over the cache.  With `store` their own keys and
        values are written into the cache first (in the same launch where a kernel can).
        float32: the plain kernel, whose sums depend on positions alone.  bfloat16: one token per
        sequence takes the split decode kernel; anything else the tensor-core prefill kernel, or
        the plain kernel for head sizes that one has no instantiation for."""
        if qkv.dtype != cache.k.dtype or out_dtype != qkv.dtype:
            raise KernelError("attention: activations, cache and output have one element type")
        self._dense(qkv, "qkv")
        out = torch.empty((plan.T, n_heads * head_dim), dtype=out_dtype, device=qkv.device)
        pages = plan.pages[cache.group_index]
        if qkv.dtype == torch.bfloat16 and plan.all_single:
            if plan.T != plan.n:      # the decode kernels take token t for sequence t of the step
                raise KernelError("attention: a step of one token each has as many tokens as sequences")
            blocks = min(plan.max_blocks, max(1, -(-plan.max_end // 64)))
            mma = self.decode_mma and head_dim in (64, 128) and n_heads // kv_heads <= 8
            pairs = plan.T * (kv_heads if mma else n_heads)   # the tensor-core kernel takes a group of heads a block
            n_chunks = decode_chunks(blocks, pairs, self.sms, self.decode_slots, mma and head_dim == 64)
            per_chunk = -(-blocks // n_chunks)
            n_partials = self.lib.ember_attention_decode_partials(plan.T, n_heads, head_dim, blocks, per_chunk)
            partials, counters = self._decode_scratch(n_partials, plan.T * n_heads)
            # The layer that attends next from the same group of the cache reads the same rows of its own
            # pages: while they all fit in L2 beside a layer's weights, this launch asks them there.
            ahead = getattr(cache, "following", None) if self.cache_ahead else None
            rows_bytes = plan.T * blocks * 64 * kv_heads * head_dim * 2 * 2
            ahead_k, ahead_v = (ahead[0].data_ptr(), ahead[1].data_ptr()) if ahead and rows_bytes <= self.AHEAD_BYTES else (0, 0)
            if self.decode_mma:
                rc = self._call("ember_attention_decode_mma", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                out.data_ptr(), partials.data_ptr(), counters.data_ptr(), plan.positions.data_ptr(),
                                plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks,
                                blocks, cache.k.shape[0], plan.T, n_heads, kv_heads, head_dim, float(scale), int(window),
                                per_chunk, 1 if store else 0, ahead_k, ahead_v, allow=(2,))
                if rc == 0:
                    return out
            self._call("ember_attention_decode_ahead", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                       out.data_ptr(), partials.data_ptr(), counters.data_ptr(), plan.positions.data_ptr(),
                       plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(), pages.data_ptr(), plan.max_blocks, blocks,
                       plan.T, n_heads, kv_heads, head_dim, float(scale), int(window), per_chunk, 1 if store else 0,
                       ahead_k, ahead_v)
            return out
        if store:
            self.kv_store(qkv, cache, plan, n_heads, kv_heads, head_dim)
        if qkv.dtype == torch.bfloat16 and scale > 0 and self.attention_tc:
            rc = self._call("ember_attention_prefill_tc", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.seq_new.data_ptr(),
                            plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n, plan.max_new, plan.T,
                            cache.k.shape[0], n_heads, kv_heads, head_dim, float(scale), int(window), allow=(2,))
            if rc == 0:
                return out
        if qkv.dtype == torch.bfloat16 and scale > 0:
            rc = self._call("ember_attention_prefill", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                            out.data_ptr(), plan.seq_slot.data_ptr(), plan.seq_start.data_ptr(), plan.seq_new.data_ptr(),
                            plan.cu_new.data_ptr(), pages.data_ptr(), plan.max_blocks, plan.n, plan.max_new, n_heads,
                            kv_heads, head_dim, float(scale), int(window), allow=(2,))
            if rc == 0:
                return out
        self._call("ember_attention_plain", qkv.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                   out.data_ptr(), plan.positions.data_ptr(), plan.token_seq.data_ptr(), plan.seq_slot.data_ptr(),
                   pages.data_ptr(), plan.max_blocks, plan.T, n_heads, kv_heads, head_dim,
                   float(scale), int(window), _code(qkv.dtype))
        return out

    # ------------------------------------------------------------------ sampling
    sample_takes_base = True

    def sample(self, logits, temperature, top_k, top_p, seed, streams, counters, counter_base: int = 0, out=None):
        """One token per row of float32 logits.  `streams` and `counters` (int32, one per row) key
        the uniform number of each row's draw; `counter_base` is added to every row's counter.  `out`:
        where the ids go (int32, one per row; default: a new tensor)."""
        rows, V = logits.shape
        if logits.dtype != torch.float32:
            raise KernelError("sample: logits are float32")
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        elif out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous() or out.device != logits.device:
            raise KernelError("sample: the ids go into a contiguous int32 tensor with one entry per row, on the logits' device")
        self._call("ember_sample", self._dense(logits, "logits").data_ptr(), out.data_ptr(), rows, V, float(temperature),
                   int(top_k), float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, streams.data_ptr(), counters.data_ptr(),
                   int(counter_base))
        return out
