"""Random-weights mode: a model from a configuration and a seed, either as
tensors in memory or as a model folder (config.json + model.safetensors).

Tensors are drawn one by one in the sorted order of their names from one
generator, so a (config, seed) pair names one model.  Matrices and embeddings
are N(0, std); norm weights are 1 + N(0, norm_jitter).  Values are drawn in
32-bit and rounded once to the storage type.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from . import safetensors_io as st
from .loader import TensorNeed


def random_tensors(needs: Dict[str, TensorNeed], seed: int, dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_jitter: float = 0.02,
                   device: str | torch.device = "cpu",
                   norm_dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(needs):
        need = needs[name]
        if need.init == "ones":
            t = torch.ones(need.shape, dtype=torch.float32, device=device)
            if norm_jitter:
                t += norm_jitter * torch.randn(need.shape, generator=gen, dtype=torch.float32,
                                               device=device)
            out[name] = t.to(norm_dtype)
        elif need.init == "normal":
            t = torch.empty(need.shape, dtype=dtype, device=device)
            # rows in chunks: a 32-bit staging copy of a large matrix is not needed
            flat = t.view(-1)
            chunk = 1 << 26
            for b in range(0, flat.numel(), chunk):
                e = min(flat.numel(), b + chunk)
                flat[b:e] = (std * torch.randn(e - b, generator=gen, dtype=torch.float32,
                                               device=device)).to(dtype)
            out[name] = t
        else:
            raise ValueError(f"tensor {name!r}: unknown init {need.init!r}")
    return out


def write_model_dir(out_dir: str, config, needs: Dict[str, TensorNeed], seed: int,
                    dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                    norm_jitter: float = 0.02) -> None:
    """``config`` is a typed configuration with ``to_dict()``."""
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(needs, seed, dtype=dtype, std=std, norm_jitter=norm_jitter)
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    st.write_file(os.path.join(out_dir, "model.safetensors"), tensors,
                  metadata={"format": "pt", "seed": str(seed)})
