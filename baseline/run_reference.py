"""The reference arm of bench.py: andrewkchan/yalm itself, unmodified, on the same
layer sizes.

yalm is a Makefile project (no setup.py or pyproject.toml, so pip has nothing to
install): a copy of its tree under ``baseline/_ref`` is built with its own Makefile
(``make CUARCH=sm_100 build/main``; its kernels are plain CUDA and compile for
sm_100 as they are).  A random float16 model folder of the benchmark's sizes is
written with torch and the ``safetensors`` package, packed by the reference's own
``convert.py --dtype fp16``, and served by its own ``build/main <ckpt> -m completion
-t 0 -n N -f prompt``.  Nothing of yalm_b200 is imported or loaded on this path.

What is measured: yalm serves one sequence at a time (``Model::forward(state, token,
pos)``, src/model.h:260), so a workload of several requests runs one after another
and its decode rate is its batch-1 rate.  ``build/main`` prints every token as it is
sampled (src/main.cpp:119-129); this script timestamps the tokens as they arrive on
the pipe, skips the first W (warm-up) and times exactly K decode steps, host to host.
The program's own totals ("Generation stats", src/main.cpp:131-147) are reported
beside that figure.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
REF_SOURCE = "/root/reference"


class Unavailable(Exception):
    pass


def _say(msg: str) -> None:
    print(f"[reference] {msg}", file=sys.stderr, flush=True)


def ensure_built() -> str:
    """baseline/_ref/build/main, built with the reference's own Makefile if absent."""
    exe = os.path.join(REF, "build", "main")
    if os.path.isfile(exe):
        return exe
    if not os.path.isfile(os.path.join(REF, "Makefile")):
        if not os.path.isfile(os.path.join(REF_SOURCE, "Makefile")):
            raise Unavailable("no copy of the reference under baseline/_ref and none to copy")
        shutil.copytree(REF_SOURCE, REF, dirs_exist_ok=True)
        for dirpath, _, files in os.walk(REF):
            os.chmod(dirpath, 0o755)
            for f in files:
                os.chmod(os.path.join(dirpath, f), 0o644)
    cxx = "/usr/bin/g++" if os.path.isfile("/usr/bin/g++") else "g++"
    _say("building baseline/_ref with its Makefile (CUARCH=sm_100)")
    r = subprocess.run(["make", f"CXX={cxx}", "CUARCH=sm_100", "build/main"], cwd=REF,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0 or not os.path.isfile(exe):
        raise Unavailable("make CUARCH=sm_100 build/main failed: " + r.stdout.strip()[-300:])
    return exe


def _work_dir(need_bytes: int) -> str:
    """A temporary folder on the file system with the most room."""
    best, best_free = None, -1
    for d in (tempfile.gettempdir(), "/dev/shm", os.path.join(ROOT, "baseline")):
        try:
            free = shutil.disk_usage(d).free
        except OSError:
            continue
        if free > best_free:
            best, best_free = d, free
    if best is None or best_free < need_bytes:
        raise Unavailable(f"{need_bytes / 1e9:.0f} GB of scratch space are needed for the float16 "
                          f"model and its packed form; {max(best_free, 0) / 1e9:.0f} GB are free")
    return tempfile.mkdtemp(prefix="yalm_ref_", dir=best)


def write_random_model(folder: str, cfg: dict, seed: int) -> None:
    """config.json, tokenizer.json (token i is the text "<ti>") and one float16
    safetensors file per layer: N(0, 0.02) matrices, norms at 1."""
    import torch
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    V = cfg["vocab_size"]
    with open(os.path.join(folder, "tokenizer.json"), "w") as f:
        json.dump({"model": {"vocab": {f"<t{i}>": i for i in range(V)}, "byte_fallback": True},
                   "added_tokens": []}, f)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(seed)
    D, F = cfg["hidden_size"], cfg["intermediate_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    mat = lambda *s: (0.02 * torch.randn(*s, generator=g, device=dev)).to(torch.float16).cpu()
    one = lambda n: torch.ones(n, dtype=torch.float32)
    top = {"model.embed_tokens.weight": mat(V, D), "model.norm.weight": one(D)}
    if not cfg.get("tie_word_embeddings", False):
        top["lm_head.weight"] = mat(V, D)
    save_file(top, os.path.join(folder, "model-top.safetensors"))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        save_file({f"{p}.input_layernorm.weight": one(D),
                   f"{p}.post_attention_layernorm.weight": one(D),
                   f"{p}.self_attn.q_proj.weight": mat(H * hd, D),
                   f"{p}.self_attn.k_proj.weight": mat(G * hd, D),
                   f"{p}.self_attn.v_proj.weight": mat(G * hd, D),
                   f"{p}.self_attn.o_proj.weight": mat(D, H * hd),
                   f"{p}.mlp.gate_proj.weight": mat(F, D),
                   f"{p}.mlp.up_proj.weight": mat(F, D),
                   f"{p}.mlp.down_proj.weight": mat(D, F)},
                  os.path.join(folder, f"model-{i:03d}.safetensors"))


def run(cfg: dict, context: int, prompt_len: int, steps: int, warmup: int, sampler=None,
        seed: int = 0) -> dict:
    """Packs a random model of ``cfg`` and times ``steps`` decode steps of the reference
    after ``warmup`` untimed ones, on a prompt of ``prompt_len`` tokens."""
    import torch
    if not torch.cuda.is_available():
        raise Unavailable("no CUDA device here: the reference's build/main -d cuda cannot run")
    exe = ensure_built()
    D, F, V, L = (cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"],
                  cfg["num_hidden_layers"])
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    params = L * ((H + 2 * G) * hd * D + D * H * hd + 3 * F * D) + \
        (1 if cfg.get("tie_word_embeddings") else 2) * V * D
    work = _work_dir(2 * 2 * params + (1 << 30))
    try:
        t0 = time.time()
        hf = os.path.join(work, "hf")
        write_random_model(hf, cfg, seed)
        _say(f"wrote the float16 model folder ({2 * params / 1e9:.1f} GB) in {time.time() - t0:.0f} s")
        t0 = time.time()
        ckpt = os.path.join(work, "model.yalm")
        r = subprocess.run([sys.executable, os.path.join(REF, "convert.py"), "--dtype", "fp16", ckpt, hf],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise Unavailable("the reference's convert.py failed: " + r.stdout.strip()[-300:])
        shutil.rmtree(hf, ignore_errors=True)
        _say(f"packed it with the reference's convert.py in {time.time() - t0:.0f} s")
        g = torch.Generator().manual_seed(seed + 1)
        prompt = torch.randint(3, V, (prompt_len - 1,), generator=g).tolist()   # BOS is added by yalm
        with open(os.path.join(work, "prompt.txt"), "w") as f:
            f.write("".join(f"<t{t}>" for t in prompt))
        n_new = warmup + steps + 1
        cmd = [exe, ckpt, "-m", "completion", "-T", str(context), "-t", "0", "-n", str(n_new),
               "-f", os.path.join(work, "prompt.txt")]
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
        t0 = time.time()
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, bufsize=0)
        # Tokens arrive as "<t123>" pieces, flushed one by one after the line that lists the
        # prompt's encoding and the "Encoding stats" line; stamp each as it arrives.
        stamps, text, body_at, sampling = [], b"", -1, False
        tok = re.compile(rb"<t\d+>")
        while True:
            chunk = proc.stdout.read(65536)
            if not chunk:
                break
            now = time.perf_counter()
            text += chunk
            if body_at < 0:
                i = text.find(b"Encoding stats")
                j = text.find(b"\n\n", i) if i >= 0 else -1
                if j < 0:
                    continue
                body_at = j + 2
            end = text.find(b"Generation stats", body_at)
            n = len(tok.findall(text[body_at:end if end >= 0 else len(text)]))
            if n > warmup and sampler is not None and not sampling:
                sampler.start()
                sampling = True
            stamps.extend([now] * (n - len(stamps)))
        rc = proc.wait()
        clocks = sampler.stop() if sampling else None
        out = text.decode("utf-8", "replace")
        if rc != 0:
            raise Unavailable(f"the reference's build/main exited with {rc}: " + out.strip()[-300:])
        _say(f"build/main ran in {time.time() - t0:.0f} s")
        tail = out[out.find("Generation stats"):] if "Generation stats" in out else ""
        stats = {}
        for key, pat in (("tokens", r"(\d+) tokens"), ("throughput", r"throughput: ([0-9.eE+-]+)tok/s"),
                         ("hydrate", r"hydrate: ([0-9.eE+-]+)s"), ("bandwidth", r"bandwidth: ([0-9.eE+-]+)GB/s"),
                         ("total", r"total: ([0-9.eE+-]+)s")):
            m = re.search(pat, tail)
            if m:
                stats[key] = float(m.group(1))
        if len(stamps) < warmup + steps + 1:
            raise Unavailable(f"the reference stopped after {len(stamps)} of {n_new} tokens "
                              f"(a stop token was sampled)")
        # token i is printed after forward i-1 and sampling i: stamps[W] .. stamps[W+K] span K steps
        dt = stamps[warmup + steps] - stamps[warmup]
        res = {"tok_s": steps / dt, "ms_per_step": dt / steps * 1e3, "clocks": clocks,
               "reported": stats, "prompt_len": prompt_len}
        if stats.get("total") and stats.get("hydrate") is not None and stats.get("tokens"):
            gen = stats["tokens"] - prompt_len
            res["reported_decode_tok_s"] = gen / max(stats["total"] - stats["hydrate"], 1e-9)
        return res
    finally:
        shutil.rmtree(work, ignore_errors=True)
