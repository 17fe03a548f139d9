"""What every part shares: the runtime (compute type, device, scratch buffers,
the kernels' status word), the residual stream, and the part registries.

A part is built from the ``params`` of its :class:`PartSpec` and knows nothing
about the model it sits in.  Interfaces (duck-typed):

* every part: ``tensor_needs() -> {key: TensorNeed}`` and
  ``bind({key: tensor})`` (tensors arrive as stored; the part moves them to the
  device in the type it computes with);
* norm: ``__call__(stream, rows=None) -> h`` (normalised rows in the compute
  type; folds the stream's pending partial sums in);
* mixer: ``cache_need() -> None | CacheNeed | {name: CacheNeed}`` (several needs:
  keys and values and a state, say) and ``forward(h, batch, stream, view,
  shared=False)``, which must add its output to ``stream`` (``stream.add_linear``
  or ``stream.add_tensor``).  ``view`` is one ``CacheView`` for a single need, a
  dict of them by need name for several, None for none.  ``forward`` returns
  None, or a function that writes the cache and that the model calls once every
  run entry that reads this entry's cache has run;
* feed-forward: ``forward(h, batch, stream)``, likewise;
* position encoding: owned by the mixer that uses it (see ``position.py``);
* block: ``parts()``, ``mixers() -> {name: mixer}`` and
  ``forward(stream, batch, views, shared)`` with ``views[name]`` the view of the
  mixer of that name;
* optional, for roofline figures: ``flops(q_lens, past)`` on any part and
  ``cache_read_bytes(contexts, element_size)`` on a mixer; and
  ``prefers_longest_first`` on a mixer that wants a batch's rows in that order.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch

from ..csrc import ops

# ---------------------------------------------------------------- registries
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITIONS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}
EMBEDDINGS: Dict[str, Callable] = {}
HEADS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], what: str):
    def deco(kind: str):
        def inner(cls):
            table[kind] = cls
            return cls
        return inner
    return deco


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_block = _register(BLOCKS, "block")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def make_part(table: Dict[str, Callable], spec, rt: "Runtime"):
    if spec.kind not in table:
        raise KeyError(f"no part of kind {spec.kind!r} is registered (known: {sorted(table)})")
    return table[spec.kind](spec.params, rt)


# ------------------------------------------------------------------- runtime
class Runtime:
    """Compute type, device, the status word that kernels raise errors in, and
    named scratch buffers that keep their address from step to step (a captured
    CUDA graph relies on that)."""

    def __init__(self, dtype: torch.dtype, device="cuda:0", gemm: str = "auto",
                 attention: str = "auto", float32_matrices: str = "keep"):
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise ValueError(f"compute type must be float32, bfloat16 or float16, not {dtype}")
        if float32_matrices not in ("keep", "round"):
            raise ValueError("float32_matrices is 'keep' or 'round'")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("this library runs on a CUDA device (sm_100a) only; "
                               "there is no CPU path")
        ops.lib()   # builds/loads the kernels now: a missing library fails here, loudly
        self.gemm = gemm                      # "auto" | "simt" (debugging aid: no tensor cores)
        self.attention = attention            # "auto" | "mma" (no tcgen05 prefill attention) | "simt"
        # small decode batches: the attention kernel does the rotary kernel's work (False: never)
        self.decode_rope_in_attention = True
        # the tensor-core decode attention's plan, for measurements: warps per block (4 or 2) and
        # 64-key chunks per block; None: the part decides
        self.decode_attention_warps = None
        self.decode_attention_chunks = None
        # a matrix stored in 32 bits under 16-bit compute: "keep" it (it is then multiplied by
        # the FMA kernel, without tensor cores) or "round" it to the compute type
        self.float32_matrices = float32_matrices
        self.kept_float32 = 0
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._buffers: Dict[str, torch.Tensor] = {}
        self._shared = []
        self.frozen = False                   # set while a graph is captured or replayed
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.buffer_generation = 0

    @classmethod
    def shapes_only(cls, dtype: torch.dtype = torch.bfloat16) -> "Runtime":
        """A runtime without a device: parts can be built and asked for the
        tensors they need (random-weights mode, checks), but not run."""
        rt = cls.__new__(cls)
        rt.dtype, rt.device, rt.gemm, rt.attention = dtype, torch.device("cpu"), "auto", "auto"
        rt.float32_matrices, rt.kept_float32 = "keep", 0
        rt.status, rt._buffers, rt._shared = None, {}, []
        rt.frozen, rt.sm_count, rt.buffer_generation = True, 148, 0
        rt.decode_rope_in_attention = True
        rt.decode_attention_warps = rt.decode_attention_chunks = None
        return rt

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = f"{name}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"scratch buffer {name!r} would grow while a graph holds it")
            grow = max(n, 0 if buf is None else int(buf.numel() * 1.5))
            buf = torch.empty(max(grow, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.buffer_generation += 1       # captured graphs that used the old one are stale
        return buf[:n].view(*shape)

    def zeros(self, name: str, n: int, dtype: torch.dtype = torch.int32) -> torch.Tensor:
        """A named buffer that starts at zero and that kernels leave at zero
        (tile and chunk counters)."""
        key = f"zero:{name}:{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"counter buffer {name!r} would grow while a graph holds it")
            buf = torch.zeros(max(n, 1024 if buf is None else 2 * buf.numel()), dtype=dtype,
                              device=self.device)
            self._buffers[key] = buf
            self.buffer_generation += 1
        return buf

    def matrix(self, t: torch.Tensor, share: bool = False) -> torch.Tensor:
        """A weight matrix in the type it is multiplied in: the compute type (a 16-bit
        matrix stored in the other 16-bit type is rounded to it; 32-bit compute widens
        16-bit storage exactly), except that a matrix stored in 32 bits stays 32-bit unless
        ``float32_matrices="round"``.  ``share``: parts that are bound to the same stored
        tensor (a tied head) get one copy."""
        keep32 = t.dtype == torch.float32 and self.float32_matrices == "keep"
        dt = torch.float32 if (self.dtype == torch.float32 or keep32) else self.dtype
        if keep32 and self.dtype != torch.float32:
            self.kept_float32 += 1
        if share:
            for src, dev in self._shared:
                if src is t:
                    return dev
        dev = t.to(device=self.device, dtype=dt).contiguous()
        if share:
            self._shared.append((t, dev))
        return dev

    def end_binding(self) -> None:
        self._shared.clear()
        if self.kept_float32:
            import warnings
            warnings.warn(f"{self.kept_float32} weight matrices are stored in float32 and stay so: "
                          f"their products run on the FMA kernel, not on tensor cores "
                          f"(float32_matrices='round' converts them to {self.dtype})", stacklevel=3)
            self.kept_float32 = 0

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            what = []
            if code & ops.ERR_TOKEN_RANGE:
                what.append("a token id outside the vocabulary")
            if code & ops.ERR_WAIT_TIMEOUT:
                what.append("a bounded barrier wait ran out inside a kernel")
            if code & ops.ERR_SLOT_RANGE:
                what.append("a slot index outside the cache")
            if code & ops.ERR_CONTEXT_RANGE:
                what.append("a sequence longer than the bound its attention launch was sized for")
            raise ops.KernelError("kernel status: " + "; ".join(what or [f"code {code}"]))


# ----------------------------------------------------------- residual stream
class ResidualStream:
    """The 32-bit residual sum x [N, D].  A projection may leave its result as
    split-K partial sums (``pending``); the next norm folds them into x while
    it reads x anyway."""

    def __init__(self, rt: Runtime, x: torch.Tensor):
        self.rt = rt
        self.x = x
        self.pending: Optional[torch.Tensor] = None    # float32 [S, N, D]
        self.n_pending = 0

    def add_linear(self, a: torch.Tensor, w: torch.Tensor) -> None:
        """x += a @ w.T"""
        from .linear import matmul_into_stream
        matmul_into_stream(self.rt, a, w, self)

    def resolve(self) -> torch.Tensor:
        if self.n_pending:
            self.x += self.pending[:self.n_pending].sum(0)
            self.pending, self.n_pending = None, 0
        return self.x

    def add_tensor(self, y: torch.Tensor) -> None:
        self.resolve()
        self.x += y.to(torch.float32)
