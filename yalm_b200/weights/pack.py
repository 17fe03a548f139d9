"""One-file model: every tensor of a model folder plus its configuration in one
safetensors file, the configuration as a JSON string in the file's metadata.

The reference ships models this way (convert.py:58-81 puts every configuration value
into the metadata of its packed file, codec.cpp:97-156 maps the file); here the file
is an ordinary safetensors file that other readers open too, the tensors keep their
checkpoint names and stored types, and nothing is permuted.

    python -m yalm_b200.weights.pack MODEL_DIR OUT.safetensors
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Dict, Tuple

import torch

from . import safetensors_io as st
from .loader import WeightsError, _normalise

CONFIG_KEY = "yalm_b200.config"


def pack_model_dir(model_dir: str, out_path: str) -> None:
    with open(os.path.join(model_dir, "config.json"), "r") as f:
        config = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    for path in st.list_files(model_dir):
        for name, t in st.read_file(path).items():
            if name in tensors:
                raise WeightsError(f"tensor {name!r} appears in more than one file of {model_dir}")
            tensors[name] = t
    if not tensors:
        raise WeightsError(f"no .safetensors file in {model_dir}")
    st.write_file(out_path, tensors, {CONFIG_KEY: json.dumps(config), "format": "yalm_b200 packed model"})


def load_packed(path: str) -> Tuple[Dict[str, Any], Dict[str, torch.Tensor]]:
    """(configuration as a dict, tensors by name) of a packed file."""
    meta = st.read_metadata(path)
    if CONFIG_KEY not in meta:
        raise WeightsError(f"{path} carries no configuration in its metadata (key {CONFIG_KEY!r}): "
                           f"pack a model folder with python -m yalm_b200.weights.pack")
    return json.loads(meta[CONFIG_KEY]), {k: _normalise(v) for k, v in st.read_file(path).items()}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    pack_model_dir(argv[0], argv[1])
    print(f"packed {argv[0]} into {argv[1]} ({os.path.getsize(argv[1])} bytes)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
