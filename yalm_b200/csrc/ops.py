"""Thin typed wrappers around the kernel library's C interface.

Arguments are CUDA tensors (their ``data_ptr`` is handed over) and plain
numbers; every call runs on torch's current stream, so the calls can be
captured into a CUDA graph.  A non-zero return code raises ``KernelError``:
there is no fallback to another implementation.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

F32, BF16, F16 = 0, 1, 2
HALF_TYPES = (torch.bfloat16, torch.float16)

ERR_TOKEN_RANGE, ERR_WAIT_TIMEOUT, ERR_SLOT_RANGE, ERR_CONTEXT_RANGE = 1, 2, 4, 8

_REFUSALS = {
    -2: "a size that this kernel does not take",
    -3: "an unsupported combination of types or modes",
    -4: "a launch grid beyond the device limits",
    -5: "a bad split count",
    -6: "a pointer that is not 16-byte aligned",
    -10: "cuTensorMapEncodeTiled was not found in the driver",
    -11: "cuTensorMapEncodeTiled refused the tensor",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float16:
        return F16
    raise KernelError(f"the kernels take float32, bfloat16 and float16 tensors, not {dt}")


_c = ctypes
_vp, _i, _ll, _f, _ull = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float, _c.c_ulonglong
_SIGNATURES = {
    "yalm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "yalm_rmsnorm": [_vp, _vp, _i, _ll, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "yalm_copy_async": [_vp, _vp, _ll, _i, _vp],
    "yalm_wait_probe": [_ull, _vp, _vp],
    "yalm_stream_wait": [_vp],
    "yalm_silu_mul": [_vp, _i, _ll, _vp, _i, _i, _i, _i, _vp],
    "yalm_rope_store": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                        _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_advance": [_vp, _vp, _vp, _i, _vp],
    "yalm_cache_write": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                       _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                              _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_prefill_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                   _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_prefill_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_attention_prefill_tc_cache": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                        _i, _vp, _i, _i, _vp, _vp],
    "yalm_attention_decode_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                  _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_decode_mma_fused": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i,
                                        _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "yalm_sample": [_vp, _i, _i, _f, _ull, _vp, _vp, _vp, _vp, _vp, _vp],
    "yalm_gemm_tc": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_gemm_tc_available": [],
    "yalm_gemm_2sm": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_gemm_2sm_token_tile": [_i, _i, _i],
    "yalm_gemm_2sm_rope": [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "yalm_rope_table": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load()
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _c.c_int
        l.yalm_uniform01.argtypes = [_ull, _c.c_uint, _c.c_uint]
        l.yalm_uniform01.restype = _c.c_float
        _lib = l
    return _lib


def loaded_library_path() -> str:
    lib()
    return build.library_path()


LAUNCHES = 0     # kernels launched through this module (a graph replay adds its captured count)


def _check(rc: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += kernels
        return
    if rc < 0:
        raise KernelError(f"{what}: refused, {_REFUSALS.get(rc, f'code {rc}')}")
    raise KernelError(f"{what}: CUDA error {rc} at launch "
                      f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the direct query is ten times cheaper than building
    a Stream object for every launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


KV_PAGE = 64     # positions per page of a paged cache


def _pages(pages, cache: torch.Tensor, G: int, hd: int):
    """(page_table pointer, pages per slot, pages) of a cache argument.  ``pages`` None: the
    cache is contiguous per sequence, [slots, G, capacity, hd].  Else ``pages`` is the int32
    table [slots, pages_per_slot] and the cache is [G, pages, 64, hd]."""
    if pages is None:
        return None, 0, 0
    _need(pages.dtype == torch.int32 and pages.dim() == 2 and pages.is_contiguous(),
          "page table: int32 [slots, pages_per_slot]")
    _need(cache.dim() == 4 and cache.shape[0] == G and tuple(cache.shape[2:]) == (KV_PAGE, hd),
          f"a paged cache is [{G}, pages, {KV_PAGE}, {hd}]")
    return pages.data_ptr(), pages.shape[1], cache.shape[1]


# --------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    n, dim = x.shape
    _need(tokens.dtype == torch.int32 and tokens.numel() >= n, "embed: tokens must be int32 [n]")
    _need(table.shape[1] == dim and x.dtype == torch.float32 and x.is_contiguous()
          and table.is_contiguous(), "embed: shapes")
    _check(lib().yalm_embed(_p(tokens), _p(table), dtype_code(table.dtype), _p(x), n, dim,
                            table.shape[0], _p(status), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            partials: Optional[torch.Tensor] = None, n_partials: int = 0,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = norm(x[rows[r]] + sum of partials) * weight; with partials and no
    ``rows`` the sum is written back to x.  partials: float32 [n_partials, N, dim]."""
    dim = x.shape[1]
    n_rows = out.shape[0]
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == dim
          and out.shape[1] == dim and x.is_contiguous() and out.is_contiguous(), "rmsnorm: shapes")
    stride = 0
    if n_partials:
        _need(partials is not None and partials.dtype == torch.float32
              and partials.shape[-1] == dim and partials.shape[-2] == x.shape[0],
              "rmsnorm: partials must be float32 [s, N, dim]")
        stride = x.shape[0] * dim
    if rows is None:
        _need(n_rows == x.shape[0], "rmsnorm: out rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "rmsnorm: rows int32")
    _check(lib().yalm_rmsnorm(_p(x), _p(partials) if n_partials else None, n_partials, stride,
                              _p(rows), _p(weight), _p(out), dtype_code(out.dtype), n_rows, dim,
                              float(eps), _stream()), "rmsnorm")


def copy_async(dst_ptr: int, src_ptr: int, n_bytes: int, to_device: bool) -> None:
    """A small copy between pinned host memory and the device on the current stream."""
    _check(lib().yalm_copy_async(dst_ptr, src_ptr, n_bytes, 1 if to_device else 0, _stream()),
           "copy_async", kernels=0)


def wait_probe(limit_ns: int, status: torch.Tensor) -> None:
    """Launches a kernel whose bounded barrier wait runs out after ``limit_ns`` and raises
    ERR_WAIT_TIMEOUT in ``status`` (the path a stuck copy or product would take)."""
    _check(lib().yalm_wait_probe(int(limit_ns), _p(status), _stream()), "wait_probe")


def stream_wait() -> None:
    _check(lib().yalm_stream_wait(_stream()), "stream_wait", kernels=0)


def silu_mul(gu: torch.Tensor, out: torch.Tensor, n_partials: int = 1, paired: bool = False) -> None:
    """gu: float32 [(n_partials,) rows, 2F]; out: [rows, F].  Columns of gu are
    (gate | up) or, with ``paired``, 16 gate columns then the 16 up columns of the
    same features, and so on."""
    rows, F = out.shape
    _need(gu.dtype == torch.float32 and gu.shape[-1] == 2 * F and gu.shape[-2] == rows
          and gu.is_contiguous() and out.is_contiguous(), "silu_mul: shapes")
    _check(lib().yalm_silu_mul(_p(gu), n_partials, rows * 2 * F, _p(out), dtype_code(out.dtype),
                               rows, F, 1 if paired else 0, _stream()), "silu_mul")


def rope_store(qkv: torch.Tensor, n_partials: int, inv_freq: torch.Tensor, batch,
               q_out: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, slot_pos: torch.Tensor, H: int, G: int, hd: int,
               capacity: int, write_cache: bool = True, pages=None) -> None:
    n = q_out.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(qkv.dtype == torch.float32 and qkv.shape[-1] == (H + 2 * G) * hd
          and qkv.shape[-2] == n and qkv.is_contiguous(), "rope_store: qkv float32 [(s,) N, (H+2G)hd]")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2, "rope_store: inv_freq")
    _need(q_out.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype, "rope_store: dtypes")
    _need(q_out.is_contiguous() and kv_step.is_contiguous() and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "rope_store: contiguity")
    _check(lib().yalm_rope_store(_p(qkv), n_partials, n * (H + 2 * G) * hd, _p(inv_freq),
                                 _p(batch.token_seq), _p(batch.q_start), _p(batch.seq_slot),
                                 _p(slot_pos), _p(q_out), _p(kv_step), _p(k_cache), _p(v_cache),
                                 dtype_code(q_out.dtype), n, H, G, hd, capacity,
                                 1 if write_cache else 0, pt, pps, npg, _stream()), "rope_store")


def cache_write(kv_step: torch.Tensor, batch, k_cache: torch.Tensor, v_cache: torch.Tensor,
                slot_pos: torch.Tensor, G: int, hd: int, capacity: int, pages=None) -> None:
    """This step's keys and values (kv_step [N, 2, G, hd]) into the ring rows of the
    positions the ring keeps; positions are those before the step's advance."""
    n = kv_step.shape[0]
    _need(kv_step.dtype == k_cache.dtype == v_cache.dtype and kv_step.is_contiguous()
          and k_cache.is_contiguous() and v_cache.is_contiguous()
          and kv_step.numel() == n * 2 * G * hd, "cache_write: kv_step [N, 2, G, hd] and the cache")
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _check(lib().yalm_cache_write(_p(kv_step), _p(batch.token_seq), _p(batch.q_start),
                                  _p(batch.seq_slot), _p(slot_pos), _p(k_cache), _p(v_cache),
                                  dtype_code(kv_step.dtype), n, G, hd, capacity, pt, pps, npg, _stream()),
           "cache_write")


def advance(batch, slot_pos: torch.Tensor) -> None:
    _check(lib().yalm_advance(_p(batch.q_start), _p(batch.seq_slot), _p(slot_pos), batch.n_seqs,
                              _stream()), "advance")


def attention(q: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              batch, slot_pos: torch.Tensor, out: torch.Tensor, H: int, G: int, hd: int,
              capacity: int, window: Optional[int], nsplit: int = 1,
              part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
              pages=None) -> None:
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == out.dtype,
          "attention: dtypes")
    _need(hd % 8 == 0 and 0 < hd <= 256,
          f"attention: head size {hd} is not supported (multiples of 8 up to 256)")
    if nsplit > 1:
        _need(part_o is not None and part_ml is not None
              and part_o.numel() >= n * H * nsplit * hd and part_ml.numel() >= n * H * nsplit * 2
              and part_o.dtype == torch.float32 and part_ml.dtype == torch.float32,
              "attention: split scratch")
    _check(lib().yalm_attention(_p(q), _p(kv_step), _p(k_cache), _p(v_cache), _p(batch.token_seq),
                                _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos), _p(out),
                                _p(part_o), _p(part_ml), dtype_code(q.dtype), n, H, G, hd,
                                capacity, int(window or 0), nsplit, pt, pps, npg, _stream()), "attention",
           kernels=2 if nsplit > 1 else 1)


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     seq_slot: torch.Tensor, slot_pos: torch.Tensor, out: torch.Tensor,
                     part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                     status: torch.Tensor, H: int, G: int, hd: int, capacity: int,
                     window: Optional[int], chunk: int, max_context: int, pages=None) -> None:
    """One query per sequence over the cache (the query's own row included)."""
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype, "attention_decode: dtypes")
    visible = min(max_context, window) if window else max_context
    max_chunks = -(-visible // chunk)
    hc = -(-(H // G) // 4)
    _need(part_o.numel() >= n * H * max_chunks * hd and part_ml.numel() >= n * H * max_chunks * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode: workspace")
    _check(lib().yalm_attention_decode(_p(q), _p(k_cache), _p(v_cache), _p(seq_slot), _p(slot_pos),
                                       _p(out), _p(part_o), _p(part_ml), _p(counters), _p(status),
                                       dtype_code(q.dtype), n, H, G, hd, capacity,
                                       int(window or 0), chunk, max_context, pt, pps, npg, _stream()),
           "attention_decode")


def mma_attention_usable(dtype: torch.dtype, hd: int) -> bool:
    """The tensor-core attention kernels take bfloat16 or float16 and head sizes in steps of
    16 up to 128."""
    return dtype in HALF_TYPES and hd % 16 == 0 and 0 < hd <= 128


def attention_prefill_mma(q: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                          v_cache: torch.Tensor, batch, slot_pos: torch.Tensor, out: torch.Tensor,
                          H: int, G: int, hd: int, capacity: int, window: Optional[int],
                          pages=None) -> None:
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == out.dtype
          and q.dtype in HALF_TYPES, "attention_prefill_mma: one 16-bit type throughout")
    _check(lib().yalm_attention_prefill_mma(_p(q), _p(kv_step), _p(k_cache), _p(v_cache),
                                            _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos),
                                            _p(out), dtype_code(q.dtype), batch.n_seqs,
                                            max(batch.q_lens), H, G, hd,
                                            capacity, int(window or 0), pt, pps, npg, _stream()),
           "attention_prefill_mma")


def tc_attention_usable(dtype: torch.dtype, hd: int, past, q_lens=None, capacity=None) -> bool:
    """The tcgen05 prefill attention takes bfloat16 or float16 and head size 64 or 128;
    sequences that start at their first token (every key is one of this step's), or, read
    from the cache, sequences that go on without wrapping around their ring in this step."""
    if dtype not in HALF_TYPES or hd not in (64, 128):
        return False
    if all(p == 0 for p in past):
        return True
    return (q_lens is not None and capacity is not None
            and all(p + n <= capacity for p, n in zip(past, q_lens)))


def attention_prefill_tc(q: torch.Tensor, kv_step: torch.Tensor, batch, out: torch.Tensor,
                         H: int, G: int, hd: int, window: Optional[int],
                         status: torch.Tensor) -> None:
    _need(q.dtype == kv_step.dtype == out.dtype and q.dtype in HALF_TYPES and q.is_contiguous()
          and kv_step.is_contiguous() and out.is_contiguous(),
          "attention_prefill_tc: one 16-bit type throughout")
    _check(lib().yalm_attention_prefill_tc(_p(q), _p(kv_step), _p(batch.q_start), _p(out),
                                           dtype_code(q.dtype), q.shape[0], batch.n_seqs, max(batch.q_lens), H, G, hd,
                                           int(window or 0), _p(status), _stream()),
           "attention_prefill_tc")


def attention_prefill_tc_cache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch,
                               slot_pos: torch.Tensor, out: torch.Tensor, H: int, G: int, hd: int,
                               capacity: int, window: Optional[int], status: torch.Tensor,
                               pages=None) -> None:
    """attention_prefill_tc with every key (this step's too) read from the cache, which the
    step wrote before this call; for sequences that go on and do not wrap in this step."""
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and q.dtype in HALF_TYPES
          and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
          and out.is_contiguous(), "attention_prefill_tc_cache: one 16-bit type throughout")
    n_slots = slot_pos.numel() if pt is not None else k_cache.shape[0]
    if pt is None:
        _need(tuple(k_cache.shape[1:]) == (G, capacity, hd),
              f"attention_prefill_tc_cache: a cache of one block per sequence is [slots, {G}, {capacity}, {hd}]")
    _check(lib().yalm_attention_prefill_tc_cache(_p(q), _p(k_cache), _p(v_cache), _p(batch.q_start),
                                                 _p(batch.seq_slot), _p(slot_pos), _p(out),
                                                 dtype_code(q.dtype), q.shape[0], batch.n_seqs,
                                                 max(batch.q_lens), n_slots, H, G, hd, capacity,
                                                 int(window or 0), pt, pps, npg, _p(status), _stream()),
           "attention_prefill_tc_cache")


def decode_mma_parts(max_context: int, window: Optional[int], chunks_per_block: int) -> int:
    """Blocks (partial results) per query of attention_decode_mma."""
    visible = min(max_context, window) if window else max_context
    return -(-(-(-visible // 64)) // chunks_per_block)


def attention_decode_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         seq_slot: torch.Tensor, slot_pos: torch.Tensor, out: torch.Tensor,
                         part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                         status: torch.Tensor, H: int, G: int, hd: int, capacity: int,
                         window: Optional[int], max_context: int, chunks_per_block: int,
                         pages=None, warps: int = 4) -> None:
    """``warps``: 4 (one block to an SM) or 2 (two blocks of two warps to an SM)."""
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and q.dtype in HALF_TYPES,
          "attention_decode_mma: one 16-bit type throughout")
    parts = decode_mma_parts(max_context, window, chunks_per_block)
    hc = -(-(H // G) // 16)
    _need(part_o.numel() >= n * H * parts * hd and part_ml.numel() >= n * H * parts * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode_mma: workspace")
    _check(lib().yalm_attention_decode_mma(_p(q), _p(k_cache), _p(v_cache), _p(seq_slot),
                                           _p(slot_pos), _p(out), _p(part_o), _p(part_ml),
                                           _p(counters), _p(status), dtype_code(q.dtype), n, H, G,
                                           hd, capacity, int(window or 0), max_context,
                                           chunks_per_block, warps, pt, pps, npg,
                                           _stream()),
           "attention_decode_mma")


def attention_decode_mma_fused(qkv: torch.Tensor, n_partials: int, cos_sin: torch.Tensor,
                               k_cache: torch.Tensor, v_cache: torch.Tensor, seq_slot: torch.Tensor,
                               slot_pos: torch.Tensor, out: torch.Tensor, part_o: torch.Tensor,
                               part_ml: torch.Tensor, counters: torch.Tensor, status: torch.Tensor,
                               H: int, G: int, hd: int, capacity: int, window: Optional[int],
                               max_context: int, chunks_per_block: int, pages=None) -> None:
    """attention_decode_mma with the rotary kernel's work inside: ``qkv`` is this step's q/k/v
    product as float32 slices [n_partials, n, (H + 2 G) hd] (or [n, ...] for one), ``cos_sin`` the
    step's table of ``rope_table`` [n, hd / 2, 2]; q is rotated in the kernel and the new k and v
    rows are written into the cache by it."""
    n = out.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    row = (H + 2 * G) * hd
    _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.numel() == n_partials * n * row,
          "attention_decode_mma_fused: qkv is float32 [n_partials, n, (H + 2 G) hd]")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
          and tuple(cos_sin.shape) == (n, hd // 2, 2), "attention_decode_mma_fused: cos_sin [n, hd/2, 2]")
    _need(k_cache.dtype == v_cache.dtype == out.dtype and out.dtype in HALF_TYPES,
          "attention_decode_mma_fused: one 16-bit type throughout")
    parts = decode_mma_parts(max_context, window, chunks_per_block)
    hc = -(-(H // G) // 16)
    _need(part_o.numel() >= n * H * parts * hd and part_ml.numel() >= n * H * parts * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode_mma_fused: workspace")
    _check(lib().yalm_attention_decode_mma_fused(_p(qkv), n_partials, n * row, _p(cos_sin), _p(k_cache),
                                                 _p(v_cache), _p(seq_slot), _p(slot_pos), _p(out),
                                                 _p(part_o), _p(part_ml), _p(counters), _p(status),
                                                 dtype_code(out.dtype), n, H, G, hd, capacity,
                                                 int(window or 0), max_context, chunks_per_block, pt, pps,
                                                 npg, _stream()),
           "attention_decode_mma_fused")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(out.shape) == (M, N) and a.is_contiguous()
          and w.is_contiguous() and out.is_contiguous(), "gemm_simt: shapes")
    _need(not accumulate or out.dtype == torch.float32, "gemm_simt: accumulate needs float32 out")
    _check(lib().yalm_gemm_simt(_p(a), dtype_code(a.dtype), _p(w), dtype_code(w.dtype), _p(out),
                                dtype_code(out.dtype), M, N, K, 1 if accumulate else 0, _stream()),
           "gemm_simt")


GEMM_STORE, GEMM_ADD, GEMM_SILU_MUL, GEMM_SPLIT, GEMM_SILU_PAIRED = 0, 1, 2, 3, 4


def gemm_tc_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == w.dtype and a.dtype in HALF_TYPES and a.shape[1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, status: torch.Tensor,
            splits: int = 1) -> None:
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K
          and a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm_tc: operands")
    if mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED):
        _need(tuple(out.shape) == (M, N // 2), "gemm_tc: silu-mul out is [M, N/2]")
    elif mode == GEMM_SPLIT:
        _need(out.dtype == torch.float32 and out.numel() >= splits * M * N, "gemm_tc: split scratch")
    else:
        _need(tuple(out.shape) == (M, N), "gemm_tc: out is [M, N]")
    _check(lib().yalm_gemm_tc(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                              N, K, mode, splits, _p(status), _stream()), "gemm_tc")


def gemm_2sm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int,
             status: torch.Tensor, splits: int = 1) -> None:
    """Two-SM tcgen05 product (pairs of blocks on one 256-feature tile) with a fused epilogue;
    with GEMM_SPLIT, ``splits`` slices of K as 32-bit partial sums in out [splits, M, N]."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K
          and a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm_2sm: operands")
    if mode == GEMM_SPLIT:
        _need(out.dtype == torch.float32 and tuple(out.shape) == (splits, M, N),
              "gemm_2sm: split-K partials are float32 [splits, M, N]")
    else:
        _need(tuple(out.shape) == ((M, N // 2) if mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED) else (M, N)),
              "gemm_2sm: out shape")
    _check(lib().yalm_gemm_2sm(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                               N, K, mode, splits, _p(status), _stream()), "gemm_2sm")


def gemm_2sm_token_tile(M: int, N: int, splits: int = 1) -> int:
    """The token tile (256 or 240) that gemm_2sm takes for these sizes."""
    return lib().yalm_gemm_2sm_token_tile(M, N, splits)


class _RopeArgs(ctypes.Structure):
    _fields_ = [("cos_sin", _vp), ("token_seq", _vp), ("q_start", _vp), ("seq_slot", _vp),
                ("slot_pos", _vp), ("q_out", _vp), ("kv_step", _vp), ("k_cache", _vp),
                ("v_cache", _vp), ("page_table", _vp), ("pages_per_slot", _i), ("n_pages", _i),
                ("H", _i), ("G", _i), ("hd", _i), ("capacity", _i), ("write_cache", _i)]


def gemm_2sm_rope_usable(a: torch.Tensor, w: torch.Tensor, hd: int) -> bool:
    """The q/k/v product with the rotary epilogue takes what the tcgen05 product takes and
    head sizes that divide 128 (a block's 128 rows then hold whole heads)."""
    return gemm_tc_usable(a, w) and hd % 2 == 0 and 128 % hd == 0


def rope_table(inv_freq: torch.Tensor, batch, slot_pos: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = (cos, sin) of position(t) * inv_freq[i] for the batch's tokens."""
    n, half = batch.n_tokens, inv_freq.numel()
    _need(inv_freq.dtype == torch.float32 and out.dtype == torch.float32 and out.is_contiguous()
          and tuple(out.shape) == (n, half, 2), "rope_table: out is float32 [tokens, hd/2, 2]")
    _check(lib().yalm_rope_table(_p(inv_freq), _p(batch.token_seq), _p(batch.q_start),
                                 _p(batch.seq_slot), _p(slot_pos), _p(out), n, half, _stream()),
           "rope_table")


def gemm_2sm_rope(a: torch.Tensor, w: torch.Tensor, cos_sin: torch.Tensor, batch,
                  q_out: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, slot_pos: torch.Tensor, H: int, G: int, hd: int,
                  capacity: int, status: torch.Tensor, write_cache: bool = True, pages=None) -> None:
    """rope_store(a @ w.T) in one launch: the two-SM product of many tokens whose epilogue
    rotates q and k and writes q_out, kv_step and the cache rows (no 32-bit q/k/v in between).
    ``cos_sin`` is the table of ``rope_table`` for this batch."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K and a.is_contiguous()
          and w.is_contiguous() and N == (H + 2 * G) * hd, "gemm_2sm_rope: operands")
    _need(q_out.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == a.dtype
          and q_out.is_contiguous() and kv_step.is_contiguous() and k_cache.is_contiguous()
          and v_cache.is_contiguous() and q_out.numel() == M * H * hd
          and kv_step.numel() == M * 2 * G * hd and cos_sin.dtype == torch.float32
          and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (M, hd // 2, 2),
          "gemm_2sm_rope: buffers")
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    r = _RopeArgs()
    r.cos_sin, r.token_seq, r.q_start = _p(cos_sin), _p(batch.token_seq), _p(batch.q_start)
    r.seq_slot, r.slot_pos = _p(batch.seq_slot), _p(slot_pos)
    r.q_out, r.kv_step, r.k_cache, r.v_cache = _p(q_out), _p(kv_step), _p(k_cache), _p(v_cache)
    r.page_table, r.pages_per_slot, r.n_pages = pt, pps, npg
    r.H, r.G, r.hd, r.capacity, r.write_cache = H, G, hd, capacity, 1 if write_cache else 0
    _check(lib().yalm_gemm_2sm_rope(_p(a), _p(w), dtype_code(a.dtype), M, N, K, ctypes.byref(r),
                                    _p(status), _stream()), "gemm_2sm_rope")


def sample(logits: torch.Tensor, temperature: float, seed: int, row_key: torch.Tensor,
           seq_slot: torch.Tensor, slot_pos: torch.Tensor, out_tokens: torch.Tensor,
           params: Optional[torch.Tensor] = None) -> None:
    """``params``: int64 [2] on the device holding (seed, temperature bits), which then
    replace the two arguments (see ``sampling_params``)."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and out_tokens.dtype == torch.int32
          and row_key.dtype == torch.int32, "sample: types")
    _need(params is None or (params.dtype == torch.int64 and params.numel() >= 2),
          "sample: params is int64 [2]")
    _check(lib().yalm_sample(_p(logits), rows, vocab, float(temperature), int(seed) & (2 ** 64 - 1),
                             _p(params), _p(row_key), _p(seq_slot), _p(slot_pos), _p(out_tokens),
                             _stream()), "sample")


def sampling_params(temperature: float, seed: int):
    """The two 64-bit words ``sample`` reads from ``params`` (as signed Python ints)."""
    import struct
    if temperature < 0:
        raise KernelError("sample: the temperature must not be negative")
    s = int(seed) & (2 ** 64 - 1)
    s = s - 2 ** 64 if s >= 2 ** 63 else s
    return s, struct.unpack("<I", struct.pack("<f", float(temperature)))[0]


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch on (default) or off for all later launches."""
    l = lib()
    l.yalm_set_pdl.argtypes = [_i]
    l.yalm_set_pdl.restype = _c.c_int
    l.yalm_set_pdl(1 if on else 0)


def uniform01(seed: int, key: int, counter: int) -> float:
    return float(lib().yalm_uniform01(int(seed) & (2 ** 64 - 1), int(key) & 0xffffffff,
                                      int(counter) & 0xffffffff))
