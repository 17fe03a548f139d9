"""Randomly drawn configurations of the architecture through the engine, in 32-bit and in
bfloat16, against the plain model: head sizes in steps of 8 from 16 to 256, any number of
heads and groups, widths and vocabularies that are no power of two, with and without a
window, llama3 frequency scaling and tied embeddings; prompts whole or cut into two steps
(the second step's keys then come from the cache), then six tokens one by one."""
import random

import pytest
import torch

from helpers import TOL, make_weights, random_tokens
from plain_model import plain_forward

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    hd = rng.choice([16, 24, 32, 40, 48, 64, 72, 80, 96, 112, 128, 144, 256])
    G = rng.choice([1, 2, 3, 4])
    H = G * rng.choice([1, 2, 3, 4, 5, 8, 9, 12])
    cfg = {"architectures": [rng.choice(["LlamaForCausalLM", "MistralForCausalLM"])],
           "hidden_size": rng.choice([64, 72, 96, 100, 128, 136, 200, 256]),
           "intermediate_size": rng.choice([96, 104, 128, 150, 160, 256, 272, 344]),
           "num_hidden_layers": rng.choice([1, 2]), "num_attention_heads": H, "num_key_value_heads": G,
           "head_dim": hd, "vocab_size": rng.choice([97, 256, 500, 1001]),
           "max_position_embeddings": 512, "rms_norm_eps": rng.choice([1e-5, 1e-6]),
           "rope_theta": rng.choice([10000.0, 500000.0]),
           "tie_word_embeddings": rng.choice([False, True])}
    window = rng.choice([None, None, 37, 64, 100])
    if window:
        cfg["sliding_window"] = window
    if rng.random() < 0.3:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                               "high_freq_factor": 4.0, "original_max_position_embeddings": 128}
    lens = [rng.randint(1, 330) for _ in range(rng.choice([1, 2, 3]))]
    return cfg, lens, rng.random() < 0.5


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16, 17, 18])
def test_a_random_configuration_matches_the_plain_model(seed):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, lens, cut = draw(seed)
    w = make_weights(cfg, 100 + seed)
    toks = [random_tokens(n + 6, cfg["vocab_size"], 7 * seed + i) for i, n in enumerate(lens)]
    refs = [plain_forward(cfg, w, t) for t in toks]
    for dtype in ("float32", "bfloat16", "float16"):
        lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(lens), max_context=512)
        s = lm.acquire(len(lens))
        worst = 0.0

        def see(logits, i, pos):
            nonlocal worst
            worst = max(worst, float((logits - refs[i][pos]).abs().max() / refs[i].abs().max()))

        if cut:
            first = [max(1, n // 2) for n in lens]
            lg = lm.step([t[:c] for t, c in zip(toks, first)], s, [[c - 1] for c in first]).cpu()
            for i, c in enumerate(first):
                see(lg[i], i, c - 1)
            rest = [i for i, (c, n) in enumerate(zip(first, lens)) if n > c]
            if rest:
                lg = lm.step([toks[i][first[i]:lens[i]] for i in rest], [s[i] for i in rest],
                             [[lens[i] - first[i] - 1] for i in rest]).cpu()
                for k, i in enumerate(rest):
                    see(lg[k], i, lens[i] - 1)
        else:
            lg = lm.step([t[:n] for t, n in zip(toks, lens)], s, [[0, n - 1] for n in lens]).cpu()
            for i, n in enumerate(lens):
                see(lg[2 * i], i, 0)
                see(lg[2 * i + 1], i, n - 1)
        for k in range(6):
            lg = lm.step([[t[n + k]] for t, n in zip(toks, lens)], s, [[0]] * len(lens)).cpu()
            for i, n in enumerate(lens):
                see(lg[i], i, n + k)
        lm.rt.check_status()
        assert worst <= TOL[dtype], (dtype, cfg, lens, cut, worst)
