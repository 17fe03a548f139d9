"""Shared pieces of the tests: two tiny configurations of the architecture that
differ in every size and option, random model folders in temporary places, and
the tolerances (fixed here, once)."""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

# layers 2/3, width 64/96, heads 4/3, kv heads 2/1, head size 16/32, FFN 192/256,
# vocab 256/384, theta 1e4/5e5, scaling none/llama3, window none/32, eps 1e-5/1e-6,
# untied/tied, context 128/96
TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "sliding_window": None,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["MistralForCausalLM"],
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 384, "max_position_embeddings": 96, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "sliding_window": 32, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 1, "eos_token_id": [2, 3],
}
# a third shape with sizes that are no power of two anywhere (width 88, 5 heads of 24? no:
# head sizes go in steps of 16) -- heads 6 over 2 kv heads, head size 48, FFN 200, vocab 300
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 88, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "vocab_size": 300, "max_position_embeddings": 160, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "sliding_window": 40,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}

# sizes that no kernel likes: width 100 and FFN 150 (rows that are no multiple of 16 bytes, so
# the TMA-fed matrix product must hand over to the FMA one), 5 heads of 16 that do not add up
# to the width, vocabulary 301
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 100, "intermediate_size": 150, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 16,
    "vocab_size": 301, "max_position_embeddings": 70, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "sliding_window": None,
    "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}

# head size 64: the sizes at which the tcgen05 attention and the tensor-core decode run
TINY_E = {
    "architectures": ["MistralForCausalLM"],
    "hidden_size": 128, "intermediate_size": 320, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "vocab_size": 512, "max_position_embeddings": 400, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "sliding_window": 150,
    "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}

CONFIGS = {"tiny_a": (TINY_A, 0), "tiny_b": (TINY_B, 1), "tiny_c": (TINY_C, 2), "tiny_d": (TINY_D, 3),
           "tiny_e": (TINY_E, 4)}

# Tolerances on logits, relative to the largest reference logit in magnitude.
# float32: FMA chains in another order than the CPU's.  bfloat16: activations are
# rounded to 8 bits of mantissa between kernels (2^-9 each, a few dozen roundings
# deep), weights are identical on both sides.  float16: the same roundings with 11 bits
# of mantissa, so an eighth of bfloat16's bound.
TOL = {"float32": 1e-5, "bfloat16": 2e-2, "float16": 2.5e-3}
DTYPES = ["float32", "bfloat16", "float16"]


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, std: float = 0.05,
                 jitter: float = 0.1) -> Dict[str, torch.Tensor]:
    """Random weights by checkpoint name, written here independently of the
    library's own random-weights mode."""
    g = torch.Generator().manual_seed(seed)
    D, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or D // H
    mat = lambda *s: (std * torch.randn(*s, generator=g)).to(dtype)
    vec = lambda *s: (1.0 + jitter * torch.randn(*s, generator=g)).to(torch.float32)
    w = {"model.embed_tokens.weight": mat(V, D), "model.norm.weight": vec(D)}
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(V, D)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = vec(D)
        w[f"{p}.post_attention_layernorm.weight"] = vec(D)
        w[f"{p}.self_attn.q_proj.weight"] = mat(H * hd, D)
        w[f"{p}.self_attn.k_proj.weight"] = mat(G * hd, D)
        w[f"{p}.self_attn.v_proj.weight"] = mat(G * hd, D)
        w[f"{p}.self_attn.o_proj.weight"] = mat(D, H * hd)
        w[f"{p}.mlp.gate_proj.weight"] = mat(F, D)
        w[f"{p}.mlp.up_proj.weight"] = mat(F, D)
        w[f"{p}.mlp.down_proj.weight"] = mat(D, F)
    return w


def write_model(folder: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    from yalm_b200.weights import write_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), weights)
    return folder


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    return float((got.float().cpu() - ref.float().cpu()).abs().max() / ref.float().abs().max())
