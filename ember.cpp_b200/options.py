"""Every switch of the runtime in one typed place.

ember.cpp reads its switches from environment variables, each once, and documents them in one
table (docs/USAGE.md:242-271); `EMBER_DETERMINISTIC` pins the algorithms its libraries may
otherwise choose between (determinism.h:17-35).  Here the switches are the fields of
`RuntimeOptions`.  An engine, a session and the kernels take one; the environment variables of the
same meaning are overrides that `RuntimeOptions.from_env()` applies on top of the defaults (or of
options given in code), so a measurement can flip a switch without touching the program.

  field            variable               meaning
  dtype            EMBER_DTYPE            compute type: bfloat16 (the fast kernels) or float32 (everything in true 32-bit)
  max_tokens       EMBER_MAX_TOKENS       positions the cache holds over all live sequences, each rounded up to 64
  max_slots        EMBER_MAX_SLOTS        most live sequences (default: as many as the cache has pages)
  cuda_graphs      EMBER_CUDA_GRAPHS      one-token steps replay a captured graph (0: launch by launch)
  prompt_graphs    EMBER_PROMPT_GRAPHS    steps that bring prompts replay a captured graph from the second time their shape
                                          comes; this many shapes are kept (0: never)
  deterministic    EMBER_DETERMINISTIC    no choice is made by timing: the library products take the heuristic's first
                                          algorithm, so two processes give the same bits (it implies lt_tune = False)
  gemm             EMBER_GEMM             products of more than 64 rows: "lt" cuBLASLt (as ember.cpp's go to cuBLAS), "tc" this
                                          library's tcgen05 kernel
  lt_tune          EMBER_LT_TUNE          time cuBLASLt's candidate algorithms once per shape and keep the fastest
  linear_stream    EMBER_LINEAR_STREAM    products of 17 to 64 rows on the tcgen05 weight-streaming kernel (0: cuBLASLt)
  attention        EMBER_ATTENTION        bfloat16 prefill attention at head size 64: "tc" tcgen05, "mma" the mma.sync kernel
  decode_mma       EMBER_DECODE_MMA       bfloat16 decode attention on the tensor cores where it has an instantiation
  decode_cluster   EMBER_DECODE_CLUSTER   its chunks merge in a thread-block cluster (0: through scratch and a ticket)
  decode_bulk      EMBER_DECODE_BULK      the CUDA-core decode attention brings pages in by bulk copies (0: by loads)
  pdl              EMBER_PDL              programmatic dependent launch between the kernels of a step
  cache_ahead      EMBER_CACHE_AHEAD      a decode attention asks the next layer's rows of the cache into L2
  warm             EMBER_WARM             a product asks into L2 the weights that a part announced for the product after it
                                          (a feed-forward its second matrix; the tcgen05 streaming product the next matrix)
  op_timing        EMBER_OP_TIMING        every launch is bracketed by CUDA events; `CudaOps.op_times()` gives the time per
                                          kernel entry point (ember.cpp: EMBER_OP_TIMING=1, model.h:465-467).  Steps then run
                                          launch by launch (no graph) and without overlap between kernels: read the shares
  nvtx             EMBER_NVTX             every launch is an NVTX range named after its entry point, and every step a range
                                          around them (ember.cpp names its prefill range for nsys, api.cpp:32, 1043-1045)

The kernel switches are measurement switches: the defaults are what measured fastest, and every
combination computes the same function.  The three that the launch code of the kernels reads
(pdl, decode_cluster, decode_bulk) are process-wide: the options of the `CudaOps` made last win.
"""
from __future__ import annotations

import dataclasses
import os


class OptionError(ValueError):
    pass


def _flag(text: str, name: str) -> bool:
    if text.strip().lower() in ("1", "true", "yes", "on"):
        return True
    if text.strip().lower() in ("0", "false", "no", "off"):
        return False
    raise OptionError(f"{name}={text!r}: expected 0 or 1")


@dataclasses.dataclass(frozen=True)
class RuntimeOptions:
    dtype: str = "bfloat16"
    max_tokens: int = 4096
    max_slots: int | None = None
    cuda_graphs: bool = True
    prompt_graphs: int = 4
    deterministic: bool = False
    gemm: str = "lt"
    lt_tune: bool = True
    linear_stream: bool = True
    attention: str = "tc"
    decode_mma: bool = True
    decode_cluster: bool = True
    decode_bulk: bool = True
    pdl: bool = True
    cache_ahead: bool = False
    warm: bool = True
    op_timing: bool = False
    nvtx: bool = False

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "bf16", "float32", "fp32"):
            raise OptionError(f"dtype = {self.dtype!r}: 'bfloat16' or 'float32'")
        if self.gemm not in ("lt", "tc"):
            raise OptionError(f"gemm = {self.gemm!r}: 'tc' (this library's tcgen05 kernel) or 'lt' (cuBLASLt)")
        if self.attention not in ("tc", "mma"):
            raise OptionError(f"attention = {self.attention!r}: 'tc' (tcgen05) or 'mma' (mma.sync)")
        if self.max_tokens <= 0 or (self.max_slots is not None and self.max_slots <= 0):
            raise OptionError(f"max_tokens = {self.max_tokens}, max_slots = {self.max_slots}: both positive")
        if self.prompt_graphs < 0:
            raise OptionError(f"prompt_graphs = {self.prompt_graphs}: a number of shapes, or 0 for never")
        if self.deterministic and self.lt_tune:
            object.__setattr__(self, "lt_tune", False)      # a choice by timing is not reproducible

    @staticmethod
    def variable(field: str) -> str:
        return "EMBER_" + field.upper()

    @classmethod
    def from_env(cls, base: "RuntimeOptions | None" = None, environ=None) -> "RuntimeOptions":
        """`base` (default: the defaults) with every EMBER_* variable that is set laid on top."""
        environ = os.environ if environ is None else environ
        values = dataclasses.asdict(base) if base is not None else {}
        for f in dataclasses.fields(cls):
            name = cls.variable(f.name)
            text = environ.get(name)
            if text is None:
                continue
            if f.type in ("bool", bool):
                values[f.name] = _flag(text, name)
            elif f.name in ("max_tokens", "max_slots", "prompt_graphs"):
                try:
                    values[f.name] = int(text)
                except ValueError:
                    raise OptionError(f"{name}={text!r}: expected a whole number") from None
            else:
                values[f.name] = text
        if values.get("deterministic"):
            values["lt_tune"] = False
        return cls(**values)

    def replace(self, **changes) -> "RuntimeOptions":
        return dataclasses.replace(self, **{k: v for k, v in changes.items() if v is not None})
