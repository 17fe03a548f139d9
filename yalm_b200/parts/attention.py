"""Grouped-query causal attention with an optional sliding window.

q = Wq h, k = Wk h, v = Wv h (one product over the stacked matrix); position
encoding on q and k; k, v into the cache; softmax((q.k)/sqrt(hd)) v over the
visible keys with head h reading kv head h // (H/G); x += Wo o.  The formulas
are the reference's (infer.cpp:278-338, infer.cu:730-920); the window
(keys p-W+1..p) is the checkpoint's ``sliding_window``, which the reference
does not read.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import POSITIONS, make_part, register_mixer
from . import decode_plan, linear
from .linear import matmul_partials


@register_mixer("gqa_attention")
class GQAAttention:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.G = int(params["num_kv_heads"])
        self.hd = int(params["head_dim"])
        self.window: Optional[int] = params.get("window")
        if self.H % self.G:
            raise ValueError(f"{self.H} heads do not divide into {self.G} kv heads")
        if self.hd % 8 or not 0 < self.hd <= 256:
            raise ValueError(f"head size {self.hd} is not supported by the attention kernel "
                             f"(multiples of 8 up to 256)")
        self.position = make_part(POSITIONS, params["position"], rt)
        self.w_qkv = None
        self.w_o = None

    def tensor_needs(self):
        return {"q": TensorNeed((self.H * self.hd, self.D)),
                "k": TensorNeed((self.G * self.hd, self.D)),
                "v": TensorNeed((self.G * self.hd, self.D)),
                "o": TensorNeed((self.D, self.H * self.hd))}

    def bind(self, tensors) -> None:
        parts = [tensors["q"], tensors["k"], tensors["v"]]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.w_qkv = self.rt.matrix(torch.cat(parts, 0))
        self.w_o = self.rt.matrix(tensors["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed("kv", kv_heads=self.G, head_dim=self.hd, window=self.window)

    def decode_chunk(self, batch) -> int:
        """Keys per block of the decode kernel: 64 KiB of keys and values, so
        that three blocks share an SM and hide each other's copy latency."""
        esz = 4 if self.rt.dtype == torch.float32 else 2
        chunk = (64 * 1024) // (2 * self.hd * esz)
        return max(8, min(128, chunk))

    def planned_chunks(self, batch):
        """64-key chunks of every sequence as the decode kernel's plan counts them: at the
        lengths the sequences will have when the longest reaches the step's context bound.
        A captured decode step keeps its plan until then, and a plan made for today's lengths
        goes wrong on the way: sequences of equal length that outgrow their block's run by one
        chunk all split in two, the grid doubles and every query is merged (measured at 7B
        sizes, 16 sequences of 700 keys: 3.46 against 3.10 ms per step)."""
        slack = max(0, max(1, batch.ctx_bound) - (max(batch.past) + 1))
        return [-(-(min(p + 1 + slack, self.window) if self.window else p + 1 + slack) // 64)
                for p in batch.past]

    def decode_chunks_per_block(self, batch, visible: int) -> int:
        """How many 64-key chunks one block of the tensor-core decode kernel walks
        through: the fewest with which all blocks are resident at once (one per
        SM; its four warps take the chunks' halves in turn), but no fewer than
        leave a sequence about six parts, and a whole sequence of up to eight
        chunks (lengths as they are when the longest reaches the step's bound).
        A few sequences then get several blocks each and a merge; with many
        sequences a block takes its whole sequence and nothing is merged.
        (Merging costs about 2 us and 0.3 to 0.4 us per part, a further unit of 32
        keys per warp about 1 us: one or two sequences of 1,000 to 4,000 keys in
        16 parts each, as the first rule alone has it, take 2.5 to 4 % longer per
        step at 7B sizes than in 6; a sequence of 300 keys in 5 parts 1.5 to 2 %
        longer than in one.)"""
        groups = self.G * -(-(self.H // self.G) // 16)
        chunks = self.planned_chunks(batch)
        resident = self.rt.sm_count
        most = max(1, -(-visible // 64))
        if self.rt.decode_attention_chunks:
            return min(most, int(self.rt.decode_attention_chunks))
        cpc = max(1, min(most, -(-groups * sum(chunks) // resident)))
        while cpc < most and groups * sum(-(-c // cpc) for c in chunks) > resident:
            cpc += 1
        longest = max(chunks)
        return max(cpc, most if longest <= 8 else min(most, -(-most // 6)))

    def decode_warps(self, batch, visible: int, cpc: int) -> int:
        """Warps per block of the tensor-core decode kernel: four, unless the blocks take
        whole sequences, outnumber the SMs' block slots, and the estimate of
        ``decode_plan`` says that two blocks of two warps per SM get through the grid
        sooner (few long blocks of equal length; many waves)."""
        if self.rt.decode_attention_warps:
            return int(self.rt.decode_attention_warps)
        if cpc < max(1, -(-visible // 64)):
            return 4
        chunks = tuple(self.planned_chunks(batch))
        groups = self.G * -(-(self.H // self.G) // 16)
        return decode_plan.decode_warps(decode_plan.rounded(chunks), groups, self.hd,
                                        self.rt.sm_count)

    # The decode kernel's grid takes sequences in row order, and long blocks that start
    # last leave the SMs idle at the end: the generation loop orders a batch by this.
    prefers_longest_first = True

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        """Bytes of keys and values one decode step reads for sequences of these lengths."""
        seen = sum(min(c, self.window) if self.window else c for c in contexts)
        return seen * 2 * self.G * self.hd * element_size

    def flops(self, q_lens, past) -> float:
        """Multiply-adds times two of a step: the four projections and, for each query,
        scores and value mix over the keys it sees."""
        n = sum(q_lens)
        linear = 2.0 * n * ((self.H + 2 * self.G) * self.hd * self.D + self.D * self.H * self.hd)
        pairs = 0
        for q, p in zip(q_lens, past):
            for pos in range(p, p + q):
                pairs += min(pos + 1, self.window) if self.window else pos + 1
        return linear + 4.0 * self.H * self.hd * pairs

    def forward(self, h, batch, stream, view, shared: bool = False):
        rt, H, G, hd = self.rt, self.H, self.G, self.hd
        n = batch.n_tokens
        q = rt.buffer("q_rot", (n, H * hd), rt.dtype)
        # many tokens: the q/k/v product rotates and stores in its own epilogue
        table = getattr(self.position, "step_table", None)
        fused = (not shared and n > linear.MANY_TOKENS and table is not None and rt.gemm != "simt"
                 and ops.gemm_2sm_rope_usable(h, self.w_qkv, hd))
        if not fused:
            qkv, S = matmul_partials(rt, h, self.w_qkv, "qkv")
        tensor_cores = ops.mma_attention_usable(rt.dtype, hd) and rt.attention != "simt"
        # one token per sequence on the tensor-core kernel, a small batch: that kernel sums the
        # product's slices, rotates and writes the cache row itself (no rotary kernel, one
        # hand-over less: 2-3 % of a step at batch 1, 0.5 % at 8 to 16; from 32 sequences on the
        # rotary kernel's many small blocks are the faster way, by 1-2 %)
        in_attention = (batch.is_decode and n <= 16 and tensor_cores and not shared and not fused
                        and table is not None and getattr(view, "kv_step", None) is None
                        and getattr(rt, "decode_rope_in_attention", True))
        # a layer whose cache another run entry reads keeps its step keys apart
        kv_step = view.kv_step if getattr(view, "kv_step", None) is not None else \
            rt.buffer("kv_step", (n, 2, G, hd), rt.dtype)
        # Several tokens on top of a ring that is already full: their rows would
        # replace keys that the first of them still has to see, so the ring is
        # written after the attention instead of before it -- and after every later
        # run entry that reads this cache: then the write is handed back to the model.
        late_write = (not shared) and any(
            p > 0 and ql > 1 and p + ql > view.capacity for p, ql in zip(batch.past, batch.q_lens))
        if fused:
            ops.gemm_2sm_rope(h, self.w_qkv, table(batch, view.slot_pos), batch, q, kv_step, view.k,
                              view.v, view.slot_pos,
                              H, G, hd, view.capacity, rt.status, write_cache=not late_write,
                              pages=view.pages)
        elif in_attention:
            pass
        elif shared:
            # this run reads the owner's keys and values: rotate q only
            scratch = rt.buffer("kv_step_unused", (n, 2, G, hd), rt.dtype)
            self.position.rotate_and_store(qkv, S, batch, view, q, scratch, H, G,
                                           write_cache=False)
        else:
            self.position.rotate_and_store(qkv, S, batch, view, q, kv_step, H, G,
                                           write_cache=not late_write)
        o = rt.buffer("attn_out", (n, H * hd), rt.dtype)
        if batch.is_decode:
            # one query per sequence, every key already in the cache
            bound = max(1, batch.ctx_bound)
            visible = min(bound, self.window) if self.window else bound
            if tensor_cores:
                cpc = self.decode_chunks_per_block(batch, visible)
                warps = 4 if in_attention else self.decode_warps(batch, visible, cpc)
                parts = ops.decode_mma_parts(bound, self.window, cpc)
            else:
                chunk = self.decode_chunk(batch)
                parts = -(-visible // chunk)
            part_o = rt.buffer("attn_part_o", (n, H, parts, hd), torch.float32)
            part_ml = rt.buffer("attn_part_ml", (n, H, parts, 2), torch.float32)
            counters = rt.zeros("attn_counters", n * G * -(-(H // G) // 4))
            if in_attention:
                ops.attention_decode_mma_fused(qkv, S, table(batch, view.slot_pos), view.k, view.v,
                                               batch.seq_slot, view.slot_pos, o, part_o, part_ml,
                                               counters, rt.status, H, G, hd, view.capacity,
                                               self.window, bound, cpc, pages=view.pages)
            elif tensor_cores:
                ops.attention_decode_mma(q, view.k, view.v, batch.seq_slot, view.slot_pos, o,
                                         part_o, part_ml, counters, rt.status, H, G, hd,
                                         view.capacity, self.window, bound, cpc, pages=view.pages,
                                         warps=warps)
            else:
                ops.attention_decode(q, view.k, view.v, batch.seq_slot, view.slot_pos, o, part_o,
                                     part_ml, counters, rt.status, H, G, hd, view.capacity,
                                     self.window, chunk, bound, pages=view.pages)
        elif rt.attention in ("auto", "tcgen05") and ops.tc_attention_usable(
                rt.dtype, hd, batch.past, batch.q_lens, view.capacity):
            # S, P and O in tensor memory, two query tiles per block in ping-pong (41 us
            # against 357 us for the mma.sync kernel per layer at 2,048 tokens of 32 heads
            # of 128).  Whole prompts read this step's own keys; prompts that go on (and do
            # not wrap around their ring in this step) read every key from the cache, which
            # holds this step's rows by now.
            if all(p == 0 for p in batch.past):
                ops.attention_prefill_tc(q, kv_step, batch, o, H, G, hd, self.window, rt.status)
            else:
                ops.attention_prefill_tc_cache(q, view.k, view.v, batch, view.slot_pos, o, H, G, hd,
                                               view.capacity, self.window, rt.status, pages=view.pages)
        elif tensor_cores:
            ops.attention_prefill_mma(q, kv_step, view.k, view.v, batch, view.slot_pos, o, H, G,
                                      hd, view.capacity, self.window, pages=view.pages)
        else:
            ops.attention(q, kv_step, view.k, view.v, batch, view.slot_pos, o, H, G, hd,
                          view.capacity, self.window, 1, None, None, pages=view.pages)
        stream.add_linear(o, self.w_o)
        if late_write:
            def write_ring():
                ops.cache_write(kv_step, batch, view.k, view.v, view.slot_pos, G, hd, view.capacity,
                                pages=view.pages)
            if getattr(view, "kv_step", None) is not None:
                return write_ring                  # other run entries still read the old rows
            write_ring()
        return None
