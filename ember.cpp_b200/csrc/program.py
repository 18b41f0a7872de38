"""A decode step as one launch: recording a step's operations and running them with the
persistent kernel of decode_program.cu.

`RecordingOps` has the methods that parts call on the kernels (embed, layernorm, linear, attention,
gather_rows) but launches nothing: it allocates each result and writes down what was asked for.
Running a model's forward once against it yields the step's program, an array of `EmberOp` in
device memory, in the way a CUDA graph capture yields a graph.  Only parts that do all their device
work through these methods can be recorded (`Part.ops_only`); everything else keeps to launches.
"""
from __future__ import annotations

import ctypes

import torch

from .ops import _ACT, KernelError, LazyNorm, _code

OP_EMBED, OP_LAYERNORM, OP_LINEAR, OP_ATTENTION = 0, 1, 2, 3
MAX_ROWS = 8
MAX_K = 6656           # 13 slices of 32 values for each of the kernel's 16 warps
NORM_WIDTH = 2048      # the widest row the kernel norms inside a product

_i, _f, _p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class EmberOp(ctypes.Structure):
    _fields_ = [("type", _i), ("M", _i), ("N", _i), ("K", _i),
                ("act", _i), ("out_f32", _i), ("n_heads", _i), ("kv_heads", _i),
                ("hd", _i), ("window", _i), ("store", _i), ("max_blocks", _i),
                ("table_dtype", _i), ("reserved", _i), ("eps", _f), ("scale", _f),
                ("a", _p), ("w", _p), ("w2", _p), ("bias", _p), ("residual", _p), ("out", _p), ("kc", _p), ("vc", _p),
                ("positions", _p), ("seq_slot", _p), ("pages", _p), ("reserved_ptr", _p)]


class NotRecordable(Exception):
    """The step asked for something the persistent kernel does not do."""


class RecordedNorm:
    """A layer norm whose only reader is the product that follows: it runs in that product's prologue."""

    def __init__(self, ops, x, w, b, eps, out_dtype):
        self.ops, self.x, self.w, self.b, self.eps, self.dtype = ops, x, w, b, float(eps), out_dtype
        self.shape = x.shape

    def materialize(self):
        return self.ops.layernorm(self.x, self.w, self.b, self.eps, self.dtype)


class RecordingOps:
    name = "recording"

    def __init__(self):
        self.program: list[EmberOp] = []
        self.keep: list[torch.Tensor] = []       # everything a recorded pointer refers to
        self.launches = 0

    def _new(self, shape, dtype, device):
        t = torch.empty(shape, dtype=dtype, device=device)
        self.keep.append(t)
        return t

    def _add(self, **fields) -> None:
        op = EmberOp()
        for k, v in fields.items():
            if isinstance(v, torch.Tensor):
                self.keep.append(v)
                v = v.data_ptr()
            setattr(op, k, v)
        self.program.append(op)

    # ------------------------------------------------------------------ the methods parts call
    def embed(self, tokens, positions, table, pos_table):
        T, d = tokens.shape[0], table.shape[1]
        x = self._new((T, d), torch.float32, table.device)
        self._add(type=OP_EMBED, M=T, K=d, N=table.shape[0], reserved=0 if pos_table is None else pos_table.shape[0],
                  table_dtype=_code(table.dtype), a=tokens, positions=positions, w=table,
                  w2=pos_table if pos_table is not None else None, out=x)
        return x

    def layernorm(self, x, w, b, eps, out_dtype, lazy=False):
        rows, d = x.shape
        if x.dtype != torch.float32:
            raise NotRecordable("layer norm of a non-float32 stream")
        if (lazy and out_dtype == torch.bfloat16 and d % 8 == 0 and d <= NORM_WIDTH and rows <= MAX_ROWS
                and w.dtype == torch.float32 and b.dtype == torch.float32):
            return RecordedNorm(self, x, w, b, eps, out_dtype)
        out = self._new((rows, d), out_dtype, x.device)
        self._add(type=OP_LAYERNORM, M=rows, K=d, eps=float(eps), out_f32=int(out_dtype == torch.float32), a=x, w=w, w2=b,
                  out=out)
        return out

    def linear(self, a, w, bias, act=None, residual=None, out_dtype=None):
        if isinstance(a, LazyNorm):
            a = a.materialize()
        if act not in _ACT:
            raise KernelError(f"linear: activation {act!r}")
        norm = None
        if isinstance(a, RecordedNorm):
            if w.dtype == torch.bfloat16:
                norm, a = a, a.x
            else:
                a = a.materialize()
        M, K = a.shape
        N = w.shape[0]
        if (w.dtype != torch.bfloat16 or (norm is None and a.dtype != torch.bfloat16) or w.shape[1] != K or K % 8
                or M > MAX_ROWS or K > MAX_K or N >= 1 << 22):
            raise NotRecordable("a linear layer that is not a few bfloat16 rows with K a multiple of 8 up to 6,656")
        target = torch.float32 if residual is not None else (out_dtype or torch.bfloat16)
        out = residual if residual is not None else self._new((M, N), target, a.device)
        fused = {} if norm is None else dict(reserved=1, w2=norm.w, reserved_ptr=norm.b, eps=norm.eps)
        self._add(type=OP_LINEAR, M=M, N=N, K=K, act=_ACT[act], out_f32=int(target == torch.float32), a=a, w=w,
                  bias=bias if bias is not None else None, residual=residual if residual is not None else None, out=out,
                  **fused)
        return out

    def attention(self, qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store=False):
        if not plan.all_single or qkv.dtype != torch.bfloat16 or cache.k.dtype != torch.bfloat16:
            raise NotRecordable("attention that is not one bfloat16 token per sequence")
        if n_heads % kv_heads or head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"attention: {n_heads} heads, {kv_heads} key/value heads, head size {head_dim}")
        out = self._new((plan.T, n_heads * head_dim), out_dtype, qkv.device)
        self._add(type=OP_ATTENTION, M=plan.T, n_heads=n_heads, kv_heads=kv_heads, hd=head_dim, window=int(window),
                  store=int(bool(store)), max_blocks=plan.max_blocks, reserved=cache.k.shape[0], scale=float(scale), a=qkv, kc=cache.k, vc=cache.v,
                  out=out, positions=plan.positions, seq_slot=plan.seq_slot, pages=plan.pages[cache.group_index])
        return out

    def kv_store(self, *args, **kwargs):
        raise NotRecordable("a separate cache store")

    def gather_rows(self, x, rows, n_rows):
        raise NotRecordable("a row gather")


class DecodeProgram:
    """A recorded step on the device, and its launcher."""

    def __init__(self, lib, recording: RecordingOps, rows: int, device):
        if ctypes.sizeof(EmberOp) != lib.ember_decode_program_op_size():
            raise KernelError("the program's operation record differs between Python and the kernels")
        self.lib, self.rows, self.keep = lib, rows, recording.keep
        self.n_ops = len(recording.program)
        raw = b"".join(bytes(op) for op in recording.program)
        self.ops = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.state = torch.zeros(max(2, lib.ember_decode_program_state_size() // 4), dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        self.trace = None         # set to a pinned int32 tensor (one entry per SM) to see how far each block got

    def run(self) -> None:
        rc = self.lib.ember_decode_program_run(self.ops.data_ptr(), self.n_ops, self.rows, self.state.data_ptr(),
                                               self.error.data_ptr(), None if self.trace is None else self.trace.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise KernelError(self.lib.ember_last_error().decode())

    def check(self) -> None:
        """Reads the kernel's error flag (waits for the device)."""
        code = int(self.error.item())
        if code != 0:
            self.state.zero_()
            self.error.zero_()
            what = {1: "a block gave up waiting at a grid barrier",
                    2: "a token id, position or page number of the step's description was out of range",
                    3: "a block gave up waiting for a weight copy"}.get(code, f"error {code}")
            raise KernelError(f"decode_program: {what}; the step's results are not valid")
