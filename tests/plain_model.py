"""A plain, slow implementation of the Llama / Mistral dense decoder for tests.

Whole sequences, no cache, one function per part, 32-bit floats on the CPU.
It is written from the reference's formulas (each function cites the
reference's file:line) and shares no code with the library under test: it
reads the raw ``config.json`` dictionary and tensors by their checkpoint names.

Two things the reference does not have are written from their public
definitions: the llama3 frequency rule (``rope_scaling``) and the sliding
window (a query at position p sees keys max(0, p-W+1)..p).  The reference
rotates interleaved pairs of a weight matrix whose rows its packer permuted
(convert.py:145-158); on the unpermuted checkpoint that equals rotating the
pairs (i, i + head_dim/2), which is what ``plain_rope`` does.
``tests/golden/`` holds logits of the reference's own CPU code that pin this.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def plain_embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x = float(E[token, :]) -- infer.cpp:454-475."""
    return table.float()[torch.tensor(list(tokens), dtype=torch.long)]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """o_i = x_i * w_i / sqrt(mean(x^2) + eps) -- infer.cpp:136-146."""
    ms = (x.float() ** 2).sum(-1, keepdim=True) / x.shape[-1]
    return x.float() * (1.0 / torch.sqrt(ms + eps)) * weight.float()


def plain_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """freq_j = theta^(-j/head_dim) for even j -- infer.cpp:202-207.  With
    ``scaling`` of type llama3 each frequency is rescaled by its wavelength:
    long waves are divided by ``factor``, short ones kept, and the band between
    is blended linearly in (original_len / wavelength)."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (j / head_dim))
    kind = None if scaling is None else scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv.float()
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = []
    for f in inv.tolist():
        wavelen = 2.0 * math.pi / f
        if wavelen > orig / low:
            out.append(f / factor)
        elif wavelen < orig / high:
            out.append(f)
        else:
            s = (orig / wavelen - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return torch.tensor(out, dtype=torch.float64).float()


def plain_rope(v: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """v: [T, heads, head_dim].  (a, b) <- (a cos - b sin, a sin + b cos) with
    angle = pos * freq in 32-bit -- infer.cpp:202-215; the pair is
    (i, i + head_dim/2) on unpermuted weights (see the module header)."""
    half = v.shape[-1] // 2
    ang = positions.float()[:, None] * inv_freq.float()[None, :]       # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half].float(), v[..., half:].float()
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    window: Optional[int]) -> torch.Tensor:
    """q: [T, H, hd], k, v: [T, G, hd] of one whole sequence.  Head h uses kv
    head h // (H/G); scores (q.k)/sqrt(hd) over the visible keys, softmax with
    the maximum subtracted, weighted sum of values -- infer.cpp:218-250,
    172-187, 321-330.  Causality is "keys 0..p" (kv_len = pos + 1,
    infer.cpp:488); the window keeps keys p-W+1..p."""
    T, H, hd = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, hd, dtype=torch.float32)
    for h in range(H):
        g = h // rep
        for p in range(T):
            lo = 0 if window is None else max(0, p - window + 1)
            s = (k[lo:p + 1, g].float() @ q[p, h].float()) / math.sqrt(hd)
            e = torch.exp(s - s.max())
            a = e / e.sum()
            out[p, h] = a @ v[lo:p + 1, g].float()
    return out


def plain_swiglu(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                 down: torch.Tensor) -> torch.Tensor:
    """W2 (silu(W1 x) * (W3 x)), silu(z) = z / (1 + exp(-z)) --
    infer.cpp:193-195, 356-385."""
    g = x @ gate.float().T
    u = x @ up.float().T
    return ((g / (1.0 + torch.exp(-g))) * u) @ down.float().T


def plain_block(x: torch.Tensor, cfg: dict, w: Dict[str, torch.Tensor], layer: int,
                positions: torch.Tensor) -> torch.Tensor:
    """x + attn(norm(x)) then x + ffn(norm(x)) -- infer.cpp:257-386."""
    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg["rms_norm_eps"]
    p = f"model.layers.{layer}"
    T = x.shape[0]
    h = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps)
    q = (h @ w[f"{p}.self_attn.q_proj.weight"].float().T).view(T, H, hd)
    k = (h @ w[f"{p}.self_attn.k_proj.weight"].float().T).view(T, G, hd)
    v = (h @ w[f"{p}.self_attn.v_proj.weight"].float().T).view(T, G, hd)
    inv = plain_inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    q = plain_rope(q, positions, inv)
    k = plain_rope(k, positions, inv)
    a = plain_attention(q, k, v, cfg.get("sliding_window")).reshape(T, H * hd)
    x = x + a @ w[f"{p}.self_attn.o_proj.weight"].float().T
    h = plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
    return x + plain_swiglu(h, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                            w[f"{p}.mlp.down_proj.weight"])


def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                  run_order: Optional[List[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence -- infer.cpp:477-521.  The head
    is the embedding when ``tie_word_embeddings`` is set (model.cpp:389-398)."""
    T = len(tokens)
    positions = torch.arange(T)
    x = plain_embedding(w["model.embed_tokens.weight"], tokens)
    order = run_order if run_order is not None else list(range(cfg["num_hidden_layers"]))
    for layer in order:
        x = plain_block(x, cfg, w, layer, positions)
    x = plain_rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = (w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False)
            else w["lm_head.weight"])
    return x @ head.float().T


# ---- sampling ------------------------------------------------------------

def plain_argmax(logits: torch.Tensor) -> int:
    """First maximal index -- sampler.cpp:27-38."""
    best, arg = -float("inf"), 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, arg = v, i
    return arg


def plain_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """p_i = exp((l_i - max)/T) / sum -- sampler.cpp:44-57 (in 64-bit here)."""
    l = logits.double()
    e = torch.exp((l - l.max()) / temperature)
    return e / e.sum()


def plain_sample(logits: torch.Tensor, temperature: float, r: float) -> int:
    """First i whose cumulative probability reaches r; the last index if none
    does -- sampler.cpp:58-64.  ``r`` stands for rand()/RAND_MAX."""
    if temperature == 0.0:
        return plain_argmax(logits)
    c = torch.cumsum(plain_probs(logits, temperature), 0)
    idx = int(torch.searchsorted(c, torch.tensor(r, dtype=torch.float64)).item())
    return min(idx, logits.numel() - 1)


def plain_generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int],
                          n_new: int, stop: Sequence[int] = ()) -> List[int]:
    """sample -> append -> stop check -> forward -- main.cpp:119-129 (the stop
    token is part of the output)."""
    toks = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        t = plain_argmax(plain_forward(cfg, w, toks)[-1])
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out


def plain_perplexity(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]):
    """exp(-mean log p(next)) and its error estimate -- main.cpp:201-218."""
    logits = plain_forward(cfg, w, tokens)
    lp = torch.log_softmax(logits.double(), -1)
    n = len(tokens) - 1
    vals = torch.stack([lp[i, tokens[i + 1]] for i in range(n)])
    s, ss = vals.sum().item(), (vals ** 2).sum().item()
    ppl = math.exp(-s / n)
    return ppl, ppl * math.sqrt(max(0.0, (ss - s * s / n) / n / n))
