#!/usr/bin/env python3
"""Makes the golden logits of tests/golden/: the reference's own CPU code
(its packer convert.py and its C++ engine, compiled here without changes) run
on a tiny random Llama-shaped model, token by token.

    python tests/golden/make_golden.py --reference /path/to/yalm

Written files (all small, committed):
    tiny_model/config.json, tiny_model/model.safetensors   the model (32-bit)
    tokens.json                                            the token ids fed
    reference_logits.f32                                   [n_tokens, vocab] float32

The reference engine keeps its key/value cache in 16-bit floats and is built
with -ffast-math, so its logits agree with a plain 32-bit model to about 1e-4,
not to rounding.  What the reference cannot anchor (rope_scaling, the sliding
window, batches) rests on the formulas cited in tests/plain_model.py.
"""
import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from yalm_b200.weights import write_file  # noqa: E402  (container writer only)

CONFIG = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 2,
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
    "vocab_size": 64, "max_position_embeddings": 64, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "float32",
}

HARNESS = r"""
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "model.h"
#include "codec.h"
int main(int argc, char** argv) {
  // argv: model.yalm out.f32 tok0 tok1 ...
  YALMData data;
  data.from_file(argv[1]);
  Model model(data, 0);
  InferenceState state(model.config);
  FILE* f = fopen(argv[2], "wb");
  for (int i = 3; i < argc; i++) {
    model.forward(state, atoi(argv[i]), i - 3);
    fwrite(state.logits(), sizeof(float), model.config->vocab_size, f);
  }
  fclose(f);
  return 0;
}
"""


def make_weights(seed: int):
    g = torch.Generator().manual_seed(seed)
    c = CONFIG
    D, F, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    H, G, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    n = lambda *s: 0.2 * torch.randn(*s, generator=g)
    o = lambda *s: 1.0 + 0.1 * torch.randn(*s, generator=g)
    w = {"model.embed_tokens.weight": n(V, D), "lm_head.weight": n(V, D),
         "model.norm.weight": o(D)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = o(D)
        w[f"{p}.post_attention_layernorm.weight"] = o(D)
        w[f"{p}.self_attn.q_proj.weight"] = n(H * hd, D)
        w[f"{p}.self_attn.k_proj.weight"] = n(G * hd, D)
        w[f"{p}.self_attn.v_proj.weight"] = n(G * hd, D)
        w[f"{p}.self_attn.o_proj.weight"] = n(D, H * hd)
        w[f"{p}.mlp.gate_proj.weight"] = n(F, D)
        w[f"{p}.mlp.up_proj.weight"] = n(F, D)
        w[f"{p}.mlp.down_proj.weight"] = n(D, F)
    return w


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of andrewkchan/yalm")
    ap.add_argument("--cxx", default="/usr/bin/g++")
    args = ap.parse_args()

    model_dir = os.path.join(HERE, "tiny_model")
    os.makedirs(model_dir, exist_ok=True)
    weights = make_weights(1234)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(CONFIG, f, indent=1)
    write_file(os.path.join(model_dir, "model.safetensors"), weights)
    tokens = torch.randint(0, CONFIG["vocab_size"], (24,),
                           generator=torch.Generator().manual_seed(7)).tolist()
    with open(os.path.join(HERE, "tokens.json"), "w") as f:
        json.dump(tokens, f)

    work = tempfile.mkdtemp(prefix="yalm_golden_")
    try:
        ref = os.path.join(work, "ref")
        shutil.copytree(args.reference, ref)
        hf = os.path.join(work, "hf")
        shutil.copytree(model_dir, hf)
        vocab = {f"<t{i}>": i for i in range(CONFIG["vocab_size"])}
        with open(os.path.join(hf, "tokenizer.json"), "w") as f:
            json.dump({"model": {"vocab": vocab, "byte_fallback": True}, "added_tokens": []}, f)
        yalm = os.path.join(work, "tiny.yalm")
        subprocess.check_call([sys.executable, os.path.join(ref, "convert.py"),
                               "--dtype", "fp32", yalm, hf])
        with open(os.path.join(ref, "src", "dump_logits.cpp"), "w") as f:
            f.write(HARNESS)
        cflags = ["-O3", "-ffast-math", "-std=c++20", "-fopenmp", "-mf16c", "-mavx2", "-mfma",
                  "-Ivendor", "-iquote", "src", "-I/usr/local/cuda/include"]
        objs = []
        for src in ["src/codec.cpp", "src/model.cpp", "src/infer.cpp", "src/sampler.cpp",
                    "src/time.cpp", "src/debug.cpp", "src/tokenizer.cpp", "vendor/format.cc",
                    "src/dump_logits.cpp"]:
            obj = os.path.join(work, os.path.basename(src) + ".o")
            subprocess.check_call([args.cxx, src, *cflags, "-c", "-o", obj], cwd=ref)
            objs.append(obj)
        cu = os.path.join(work, "infer.cu.o")
        subprocess.check_call(["nvcc", "src/infer.cu", "-O2", "-Ivendor", "-arch=sm_90",
                               "-allow-unsupported-compiler", "-ccbin", args.cxx,
                               "-c", "-o", cu], cwd=ref)
        exe = os.path.join(work, "dump_logits")
        subprocess.check_call([args.cxx, *objs, cu, "-lm", "-fopenmp",
                               "-L/usr/local/cuda/lib64", "-lcudart", "-o", exe])
        out = os.path.join(work, "logits.f32")
        subprocess.check_call([exe, yalm, out, *map(str, tokens)])
        logits = np.fromfile(out, dtype=np.float32).reshape(len(tokens), CONFIG["vocab_size"])
        logits.tofile(os.path.join(HERE, "reference_logits.f32"))
        print("wrote", logits.shape, "abs max", float(np.abs(logits).max()))
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    main()
