"""Matrix products of the parts: which kernel, which epilogue, how many K
slices.

16-bit operands (bfloat16 or float16) go to the tcgen05 kernel.  When the token count is small the
grid of 128-row weight tiles is too small to pull from HBM with every SM, so K
is split and each slice writes a 32-bit partial product; the consumer (norm,
rotary or SiLU kernel) sums the slices while it reads them.  With many tokens
the epilogue is fused instead (store, residual add, SiLU*up).  32-bit operands,
mixed operands (a matrix stored in 32 bits under 16-bit compute) and shapes
TMA cannot address go to the FMA kernel.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..csrc import ops


# Up to this many tokens a product runs on the single-SM kernel (split over K where its tiles
# are few); above it on the two-SM kernel, which splits over K too where its tiles leave pairs
# idle (measured at 7B sizes, ms per 8 layers, single-SM against two-SM: 129 tokens 1.70 / 1.45,
# 256 tokens 2.02 / 1.63).
MANY_TOKENS = 128


def _token_tile(M: int) -> int:
    for bt in (16, 32, 64, 128):
        if M <= bt:
            return bt
    return 256


def _valid_splits(nkb: int, s: int) -> bool:
    per = -(-nkb // s)
    return s <= nkb and (s - 1) * per < nkb            # no empty slice


def plan_splits(M: int, N: int, K: int, sm_count: int = 148) -> int:
    """Number of K slices for a small-M product.

    With few tokens the 32-bit partial sums cost next to nothing, and what counts is how
    much of the product is already on the chip when its activations arrive: every block
    asks for its first stages of weights while the previous kernel still runs, two blocks
    fit an SM, and a short K slice leaves little to fetch after the hand-over.  So the
    slices fill the 2 x SMs block slots (measured on 7B shapes at batch 8: 6 slices
    instead of 3 for q/k/v, 9 instead of 5 for the down projection: 2.5-3 us per layer).
    That holds up to 64 tokens even where the partial sums (written once, read once, 4
    bytes each) come to a third of the weights' bytes (batch 32: 159 -> 149 us per layer,
    batch 64: 194 -> 180); only when they would exceed the weights does the count trade
    idle SMs against that traffic instead."""
    bt = _token_tile(M)
    tiles = -(-N // 128) * -(-M // bt)
    nkb = -(-K // 64)
    weight_bytes = 2.0 * N * K
    s = min(2 * sm_count // max(1, tiles), nkb // 4)
    while s > 1 and not _valid_splits(nkb, s):
        s -= 1
    if s > 1 and 2.0 * s * M * N * 4.0 <= weight_bytes:
        return s
    best, best_cost = 1, None
    for s in (1, 2, 3, 4, 5, 6, 8, 10, 12, 16):
        if not _valid_splits(nkb, s):
            continue
        busy = min(1.0, tiles * s / float(sm_count))
        cost = weight_bytes / busy + 2.0 * s * M * N * 4.0
        if best_cost is None or cost < best_cost * 0.97:
            best, best_cost = s, cost
    return best


def _use_tc(rt, a: torch.Tensor, w: torch.Tensor) -> bool:
    return rt.gemm != "simt" and ops.gemm_tc_usable(a, w)


def plan_splits_many(M: int, N: int, K: int, sm_count: int = 148) -> int:
    """Number of K slices for a product of many tokens on the two-SM kernel.

    That kernel gives every pair of SMs whole 256-feature x 256- (or 240-)token tiles; a few
    hundred tokens make fewer tiles than there are pairs (512 tokens x 4,096 features: 32 or
    48 tiles on 74 pairs).  Slices of K then fill the idle pairs; their 32-bit partial sums are
    added by the consumer, as in decode.  Cost of a plan: waves of work items over the pairs
    x (the tile's tokens / slices + a work item's fixed cost of about 24 tokens' worth);
    a split must win by 20 % and its partial sums, written and read once, may come to at
    most twice the weights' bytes.  (Measured at 7B sizes, 512 tokens: down projection 88
    -> 50 us, o-proj 38 -> 25 us.)"""
    pairs = max(1, sm_count // 2)
    nkb = -(-K // 64)
    feats = -(-N // 256)

    def cost(S):
        return min(-(-feats * -(-M // bt) * S // pairs) * (bt / S + 24.0) for bt in (256, 240))

    best, best_cost = 1, cost(1)
    for S in (2, 3, 4, 6, 8):
        if not _valid_splits(nkb, S) or nkb // S < 16:
            continue
        if 2.0 * S * M * N * 4.0 > 2.0 * (2.0 * N * K):
            continue
        c = cost(S)
        if c < 0.8 * cost(1) and c < best_cost:
            best, best_cost = S, c
    return best


def _small(rt, M: int, N: int) -> bool:
    return -(-N // 128) * -(-M // _token_tile(M)) < rt.sm_count and M <= MANY_TOKENS


def matmul_partials(rt, a: torch.Tensor, w: torch.Tensor, name: str) -> Tuple[torch.Tensor, int]:
    """a @ w.T as S 32-bit slices [S, M, N] whose sum is the product."""
    M, K = a.shape
    N = w.shape[0]
    if _use_tc(rt, a, w) and M > MANY_TOKENS:
        buf = rt.buffer(name, (1, M, N), torch.float32)
        _many_tokens(rt, a, w, buf[0], ops.GEMM_STORE)
        return buf, 1
    if _use_tc(rt, a, w):
        S = plan_splits(M, N, K, rt.sm_count) if _small(rt, M, N) else 1
        buf = rt.buffer(name, (S, M, N), torch.float32)
        ops.gemm_tc(a, w, buf, ops.GEMM_SPLIT, rt.status, splits=S)
        return buf, S
    buf = rt.buffer(name, (1, M, N), torch.float32)
    ops.gemm_simt(a, w, buf[0])
    return buf, 1


def _many_tokens(rt, a, w, out, mode) -> None:
    """Many tokens: the two-SM kernel (pairs of blocks share a 256-feature tile, so each
    byte from L2 feeds 1.5 times the arithmetic; measured 1.03-1.31 PFLOP/s at 2,048
    tokens against 0.66-1.05 for the single-SM kernels), epilogue fused."""
    ops.gemm_2sm(a, w, out, mode, rt.status)


def matmul_store(rt, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T (out float32 or the compute type)."""
    if _use_tc(rt, a, w) and a.shape[0] > MANY_TOKENS:
        _many_tokens(rt, a, w, out, ops.GEMM_STORE)
    elif _use_tc(rt, a, w):
        ops.gemm_tc(a, w, out, ops.GEMM_STORE, rt.status)
    else:
        ops.gemm_simt(a, w, out)


def matmul_into_stream(rt, a: torch.Tensor, w: torch.Tensor, stream) -> None:
    """stream.x += a @ w.T, directly or as pending partial sums."""
    M, K = a.shape
    N = w.shape[0]
    if stream.n_pending:
        stream.resolve()
    if _use_tc(rt, a, w):
        if _small(rt, M, N):
            S = plan_splits(M, N, K, rt.sm_count)
            buf = rt.buffer("stream_partials", (S, M, N), torch.float32)
            ops.gemm_tc(a, w, buf, ops.GEMM_SPLIT, rt.status, splits=S)
            stream.pending, stream.n_pending = buf, S
        elif M > MANY_TOKENS:
            S = plan_splits_many(M, N, K, rt.sm_count)
            if S > 1:
                buf = rt.buffer("stream_partials", (S, M, N), torch.float32)
                ops.gemm_2sm(a, w, buf, ops.GEMM_SPLIT, rt.status, splits=S)
                stream.pending, stream.n_pending = buf, S
            else:
                _many_tokens(rt, a, w, stream.x, ops.GEMM_ADD)
        else:
            ops.gemm_tc(a, w, stream.x, ops.GEMM_ADD, rt.status)
    else:
        ops.gemm_simt(a, w, stream.x, accumulate=True)


def matmul_silu_mul(rt, a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor,
                    paired: bool = False) -> None:
    """out = silu(a @ Wg.T) * (a @ Wu.T).  w_gate_up is [Wg; Wu], or with ``paired``
    16 rows of Wg, the 16 rows of Wu for the same features, and so on: a 128-row
    tile of the product then holds gate and up of 64 features, and the epilogue
    pairs them inside a warp."""
    M, K = a.shape
    N2 = w_gate_up.shape[0]
    if _use_tc(rt, a, w_gate_up):
        if paired:
            if M > MANY_TOKENS:
                ops.gemm_2sm(a, w_gate_up, out, ops.GEMM_SILU_PAIRED, rt.status)
                return
            # nearly as many tiles as SMs: one fused launch beats two slices of K plus a
            # SiLU kernel (Llama-3.2-1B sizes, 128 tiles: 3-5 % of a decode step at batch 1 to 64)
            tiles = -(-N2 // 128) * -(-M // _token_tile(M))
            if (not _small(rt, M, N2) or plan_splits(M, N2, K, rt.sm_count) == 1
                    or 5 * tiles >= 4 * rt.sm_count):
                ops.gemm_tc(a, w_gate_up, out, ops.GEMM_SILU_PAIRED, rt.status)
                return
        elif not _small(rt, M, N2 // 2):
            if M > MANY_TOKENS:
                _many_tokens(rt, a, w_gate_up, out, ops.GEMM_SILU_MUL)
            else:
                ops.gemm_tc(a, w_gate_up, out, ops.GEMM_SILU_MUL, rt.status)
            return
    buf, S = matmul_partials(rt, a, w_gate_up, "gate_up")
    ops.silu_mul(buf, out, n_partials=S, paired=paired)
