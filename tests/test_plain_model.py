"""Self-checks of the plain implementation (no GPU)."""
import math

import torch

from helpers import TINY_A, TINY_B, make_weights, random_tokens
from plain_model import (plain_argmax, plain_attention, plain_forward, plain_generate_greedy,
                         plain_inv_freq, plain_perplexity, plain_rmsnorm, plain_rope,
                         plain_sample, plain_swiglu)


def test_window_at_least_the_length_is_no_window():
    q, k, v = torch.randn(12, 4, 16), torch.randn(12, 2, 16), torch.randn(12, 2, 16)
    assert torch.allclose(plain_attention(q, k, v, None), plain_attention(q, k, v, 12))
    w3 = plain_attention(q, k, v, 3)
    assert torch.allclose(w3[:3], plain_attention(q, k, v, None)[:3])
    assert not torch.allclose(w3[5:], plain_attention(q, k, v, None)[5:])
    # a window of 1 returns each position's own value
    assert torch.allclose(plain_attention(q, k, v, 1), v.repeat_interleave(2, 1), atol=1e-6)


def test_grouping_maps_head_h_to_kv_head_h_over_ratio():
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    full = plain_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), None)
    assert torch.allclose(plain_attention(q, k, v, None), full, atol=1e-6)


def test_attention_saturates_on_a_planted_key():
    T, hd = 9, 16
    k = torch.zeros(T, 1, hd)
    v = torch.zeros(T, 1, hd)
    for t in range(T):
        k[t, 0, t] = 1.0
        v[t, 0, t] = 1.0
    q = torch.zeros(T, 2, hd)
    for t in range(T):
        q[t, 0, max(0, t - 2)] = 1e4
        q[t, 1, t] = 1e4
    out = plain_attention(q, k, v, None)
    for t in range(T):
        assert out[t, 0].argmax().item() == max(0, t - 2) and abs(out[t, 0].sum().item() - 1) < 1e-5
        assert out[t, 1].argmax().item() == t


def test_llama3_frequencies():
    sc = TINY_B["rope_scaling"]
    base = plain_inv_freq(32, 500000.0, None)
    got = plain_inv_freq(32, 500000.0, sc)
    assert got[0] == base[0]                                   # shortest wave: kept
    assert abs(got[-1].item() - base[-1].item() / 4.0) < 1e-12  # longest wave: divided
    mid = [i for i in range(16) if 64 / 4 <= 2 * math.pi / base[i].item() <= 64 / 1]
    assert mid, "the test needs a frequency inside the blended band"
    for i in mid:
        assert base[i] / 4.0 <= got[i] <= base[i]
    assert torch.equal(plain_inv_freq(16, 1e4, {"rope_type": "default"}), plain_inv_freq(16, 1e4, None))


def test_rope_rotates_pairs_half_a_head_apart_and_keeps_norms():
    v = torch.randn(6, 3, 16)
    inv = plain_inv_freq(16, 1e4, None)
    r = plain_rope(v, torch.arange(6), inv)
    assert torch.allclose(r[0], v[0])                          # position 0: identity
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1), atol=1e-5)
    a = 3 * inv[2].item()
    assert abs(r[3, 1, 2].item() - (v[3, 1, 2] * math.cos(a) - v[3, 1, 10] * math.sin(a)).item()) < 1e-5
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    s1 = (plain_rope(q, torch.tensor([7]), inv) * plain_rope(k, torch.tensor([4]), inv)).sum()
    s2 = (plain_rope(q, torch.tensor([23]), inv) * plain_rope(k, torch.tensor([20]), inv)).sum()
    assert abs(s1.item() - s2.item()) < 1e-4


def test_rmsnorm_and_swiglu_formulas():
    x = torch.randn(3, 10)
    w = torch.randn(10)
    ref = torch.stack([xi * wi for xi, wi in zip(x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3), [w] * 3)])
    assert torch.allclose(plain_rmsnorm(x, w, 1e-3), ref, atol=1e-6)
    g, u, d = torch.randn(7, 10), torch.randn(7, 10), torch.randn(10, 7)
    ref = (torch.nn.functional.silu(x @ g.T) * (x @ u.T)) @ d.T
    assert torch.allclose(plain_swiglu(x, g, u, d), ref, atol=1e-5)


def test_tied_head_is_the_embedding_and_prefixes_agree():
    w = make_weights(TINY_B, 1)
    assert "lm_head.weight" not in w
    t = random_tokens(40, TINY_B["vocab_size"], 3)
    full = plain_forward(TINY_B, w, t)
    assert full.shape == (40, 384)
    assert torch.allclose(plain_forward(TINY_B, w, t[:17]), full[:17], atol=1e-5)   # causal


def test_sampling_rules():
    l = torch.tensor([0.5, 3.0, 3.0, -1.0])
    assert plain_argmax(l) == 1                                # first maximal index
    assert plain_sample(l, 0.0, 0.7) == 1
    p = torch.softmax(l.double(), 0)
    assert plain_sample(l, 1.0, 0.0) == 0
    assert plain_sample(l, 1.0, float(p[0]) + 1e-9) == 1
    assert plain_sample(l, 1.0, 1.0) == 3
    assert plain_sample(l, 0.1, 0.999) in (1, 2)


def test_greedy_generation_and_perplexity():
    w = make_weights(TINY_A, 0)
    out = plain_generate_greedy(TINY_A, w, [1, 5, 9], 4)
    assert len(out) == 4
    first = plain_argmax(plain_forward(TINY_A, w, [1, 5, 9])[-1])
    assert out[0] == first
    assert plain_generate_greedy(TINY_A, w, [1, 5, 9], 4, stop=[first]) == [first]
    ppl, err = plain_perplexity(TINY_A, w, random_tokens(20, 256, 1))
    assert 100 < ppl < 600 and err > 0
