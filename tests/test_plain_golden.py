"""The plain implementation against logits of the reference's own CPU code
(made once by tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import torch

from plain_model import plain_forward
from yalm_b200.weights import read_file

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_reference_cpu_logits():
    with open(os.path.join(GOLDEN, "tiny_model", "config.json")) as f:
        cfg = json.load(f)
    w = read_file(os.path.join(GOLDEN, "tiny_model", "model.safetensors"))
    with open(os.path.join(GOLDEN, "tokens.json")) as f:
        tokens = json.load(f)
    ref = torch.from_numpy(np.fromfile(os.path.join(GOLDEN, "reference_logits.f32"),
                                       dtype=np.float32).reshape(len(tokens), cfg["vocab_size"]))
    got = plain_forward(cfg, w, tokens)
    # the reference stores keys and values as 16-bit floats and is built with
    # -ffast-math: agreement is to its cache's rounding, not to 32-bit rounding
    err = (got - ref).abs().max().item()
    assert err < 2e-3 * ref.abs().max().item(), err
    assert (got.argmax(-1) == ref.argmax(-1)).all()
