"""Weights by tensor name.

``load_checkpoint`` reads every ``*.safetensors`` file of a model folder and
normalises storage types: bfloat16 and 32-bit floats stay as stored, integer
tables become int32.  float16 also stays as stored: a part that binds it keeps
it under float16 compute, rounds it to bfloat16 under bfloat16 compute, and widens
it exactly under 32-bit compute (a true 32-bit path must not round its inputs).  ``check_tensors``
compares what a model declares with what a checkpoint holds and reports every
problem in ONE error: missing tensors, unexpected tensors and wrong shapes
(the reference stops at the first missing or mis-shaped tensor,
model.cpp:98-126).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from . import safetensors_io as st


class WeightsError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class TensorNeed:
    """What a part declares about one of its tensors.  ``init`` is used by the
    random-weights mode: 'normal' (N(0, std)) or 'ones' (1 + N(0, jitter))."""
    shape: Tuple[int, ...]
    init: str = "normal"


def _normalise(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    return t


def load_checkpoint(model_dir: str) -> Dict[str, torch.Tensor]:
    files = list(st.list_files(model_dir))
    if not files:
        raise WeightsError(f"no .safetensors file in {model_dir}")
    out: Dict[str, torch.Tensor] = {}
    for path in files:
        for name, t in st.read_file(path).items():
            if name in out:
                raise WeightsError(f"tensor {name!r} appears in more than one file of {model_dir}")
            out[name] = _normalise(t)
    return out


def check_tensors(needs: Dict[str, TensorNeed], found: Dict[str, torch.Tensor],
                  optional_unexpected: Tuple[str, ...] = ()) -> None:
    missing = sorted(n for n in needs if n not in found)
    unexpected = sorted(n for n in found if n not in needs and n not in optional_unexpected)
    wrong = sorted(
        (n, tuple(needs[n].shape), tuple(found[n].shape))
        for n in needs if n in found and tuple(found[n].shape) != tuple(needs[n].shape))
    if not (missing or unexpected or wrong):
        return
    lines = ["the checkpoint does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n}: expected {list(e)}, found {list(g)}" for n, e, g in wrong))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)
