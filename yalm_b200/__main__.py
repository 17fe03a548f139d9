"""Command line in the manner of the reference's ``main`` (main.cpp:17-40,
334-470): a checkpoint, then one-letter options that each take a value.

    python -m yalm_b200 <model_dir | packed.safetensors> [options]

    -h            this help
    -d cuda       device (only cuda: there is no CPU path)
    -m MODE       completion | passkey | perplexity (any prefix; default completion)
    -T N          context length (0 = the model's): the cache keeps the last N positions
                  of each sequence as a ring (a window of N where config.json sets none or
                  a longer one) and generation goes on past N, as the reference's -T does,
                  without its two sink tokens
    -i TEXT       prompt          -f FILE   prompt file   (exactly one of -i, -f, --tokens)
    -n N          completion: tokens to generate (default 256, 0 = up to the context, -1 = no limit
                  but the context); passkey: number of filler lines (default 250)
    -t T          temperature (default 1.0; 0 = greedy)
    -l N          passkey: line at which the key is put (-1 = random)
  and beyond the reference:
    --tokens 1,2,3        prompt as token ids (works without tokenizer.json); several
                          prompts separated by ';' run as a batch
    --batch-file FILE     one prompt per line (token ids separated by commas or blanks, or
                          text if the model folder has a tokenizer.json): they run as a batch
    --max-context N       the most positions a sequence may take (default: the model's)
    --dtype bfloat16|float16|float32      --seed N      --max-batch N
    --random-weights CONFIG.json  write <model_dir> (config.json, model.safetensors) from a
                                  configuration and --seed first, if it does not exist
"""
from __future__ import annotations

import json
import os
import random
import sys
import time


def usage(code: int = 1):
    sys.stderr.write(__doc__)
    sys.exit(code)


MODES = ("completion", "passkey", "perplexity")
FILLER = " The river runs north. The hills are low. The road is dry. On we walk. Back we come."


def parse(argv):
    if len(argv) < 1 or argv[0] in ("-h", "--help"):
        usage(0 if argv else 1)
    o = {"model": argv[0], "device": "cuda", "mode": "completion", "context": 0, "prompt": None,
         "file": None, "n": None, "temperature": 1.0, "line": -1, "tokens": None,
         "dtype": "bfloat16", "seed": None, "max_batch": 8, "random_weights": None,
         "batch_file": None, "max_context": 0}
    i = 1
    short = {"-d": "device", "-m": "mode", "-T": "context", "-i": "prompt", "-f": "file", "-n": "n",
             "-t": "temperature", "-l": "line"}
    long = {"--tokens": "tokens", "--dtype": "dtype", "--seed": "seed", "--max-batch": "max_batch",
            "--random-weights": "random_weights", "--max-new-tokens": "n",
            "--batch-file": "batch_file", "--max-context": "max_context"}
    while i < len(argv):
        flag = argv[i]
        if flag == "-h":
            usage(0)
        key = short.get(flag) or long.get(flag)
        if key is None or i + 1 >= len(argv):          # every option takes a value
            usage()
        val = argv[i + 1]
        if key in ("context", "n", "line", "seed", "max_batch", "max_context"):
            val = int(val)
        elif key == "temperature":
            val = float(val)
        o[key] = val
        i += 2
    match = [m for m in MODES if m.startswith(o["mode"])]
    if not match:
        usage()
    o["mode"] = match[0]
    if not "cuda".startswith(o["device"]):
        sys.stderr.write("only -d cuda is supported: this library has no CPU path\n")
        sys.exit(1)
    return o


def main(argv=None) -> int:
    o = parse(list(sys.argv[1:] if argv is None else argv))
    if o["random_weights"] and not os.path.isfile(os.path.join(o["model"], "config.json")):
        from .engine.lm import LM
        with open(o["random_weights"]) as f:
            LM.write_random_model(o["model"], json.load(f), seed=o["seed"] or 0, dtype=o["dtype"])
        print(f"wrote a random model to {o['model']}")
    from .engine.lm import LM
    from .tokenizer import Tokenizer
    lm = LM.from_pretrained(o["model"], dtype=o["dtype"], max_context=o["max_context"] or None,
                            window_override=o["context"] or None, max_batch=o["max_batch"])
    spec = lm.spec
    # a packed one-file model keeps its tokenizer.json beside it
    tok_dir = os.path.dirname(os.path.abspath(o["model"])) if os.path.isfile(o["model"]) else o["model"]
    tok = Tokenizer.from_dir(tok_dir, spec.vocab_size, spec.bos_token_id, spec.stop_token_ids)
    seed = o["seed"] if o["seed"] is not None else int(time.time() * 1000)     # as the reference seeds
    print(f"model: {spec.architecture}, {len(spec.layers)} layers, context {lm.context}, "
          f"{lm.model.weight_bytes() / 1e9:.2f} GB weights, {lm.engine.cache.bytes() / 1e9:.2f} GB cache")

    def ids_or_text(line):
        parts = line.replace(",", " ").split()
        if parts and all(p.lstrip("-").isdigit() for p in parts):
            return [int(p) for p in parts]
        if tok is None:
            sys.stderr.write("no tokenizer.json in the model folder: give prompts as token ids\n")
            sys.exit(1)
        return tok.encode(line, bos=True)

    def prompts_from_options():
        given = [x is not None for x in (o["prompt"], o["file"], o["tokens"], o["batch_file"])]
        if sum(given) != 1:
            usage()
        if o["batch_file"] is not None:
            with open(o["batch_file"]) as f:
                return [ids_or_text(l.rstrip("\n")) for l in f if l.strip()]
        if o["tokens"] is not None:
            return [[int(t) for t in part.replace(",", " ").split()] for part in o["tokens"].split(";")]
        text = o["prompt"] if o["prompt"] is not None else open(o["file"]).read()
        if tok is None:
            sys.stderr.write("no tokenizer.json in the model folder: give the prompt with --tokens\n")
            sys.exit(1)
        return [tok.encode(text, bos=True)]

    if o["mode"] == "completion":
        prompts = prompts_from_options()
        n = 256 if o["n"] is None else o["n"]
        if n == 0:
            n = o["context"] or lm.context              # "-n 0": as many steps as the context (-T) is long
        stop = tok.stop_ids if tok is not None else list(spec.stop_token_ids)
        last = {}

        def show(i, t):
            if len(prompts) == 1 and tok is not None:
                sys.stdout.write(tok.decode_one(last.get(i, prompts[i][-1]), t).decode("utf-8", "replace"))
                sys.stdout.flush()
            last[i] = t
        t0 = time.time()
        out = lm.generate(prompts, max_new_tokens=n, temperature=o["temperature"], seed=seed,
                          stop_ids=stop, on_token=show)
        dt = time.time() - t0
        print()
        if len(prompts) > 1 or tok is None:
            for p, c in zip(prompts, out):
                print(f"tokens: {' '.join(map(str, c.tokens))}   ({c.finish_reason})")
        st = lm.last_stats
        total = st["prompt_tokens"] + st["new_tokens"]
        print(f"Generation stats:\n  {total} tokens\n  throughput: {total / dt:.5g}tok/s\n"
              f"  latency: {dt / max(total, 1):.5g}s/tok\n  hydrate: {st['prefill_seconds']:.5g}s\n"
              f"  decode: {st['new_tokens'] / max(st['decode_seconds'], 1e-9):.5g}tok/s\n"
              f"  total: {dt:.5g}s")
    elif o["mode"] == "perplexity":
        (tokens,) = prompts_from_options()[:1]
        t0 = time.time()
        ppl, err = lm.perplexity(tokens)
        dt = time.time() - t0
        n = len(tokens) - 1
        print(f"Stats:\n  {n} tokens\n  perplexity: {ppl:.5g} ± {err:.5g}\n"
              f"  throughput: {n / dt:.5g}tok/s\n  total: {dt:.5g}s")
    else:
        if tok is None:
            sys.stderr.write("passkey mode needs tokenizer.json (and trained weights to succeed)\n")
            return 1
        n_junk = 250 if o["n"] is None else o["n"]
        if o["line"] != -1 and not 0 <= o["line"] < n_junk:
            sys.stderr.write(f"Error: passkey position must be between 0 and {n_junk - 1}\n")
            return 1
        rng = random.Random(seed)
        key = rng.randrange(50000) + 1
        line = rng.randrange(n_junk) if o["line"] == -1 else o["line"]
        text = ("Somewhere in the dull text below one important fact is hidden. "
                "Find it and keep it in mind; you will be asked about it.")
        for i in range(n_junk):
            if i == line:
                text += f" The secret number is {key}. Keep it in mind. {key} is the secret number."
            text += FILLER
        text += " What is the secret number? The secret number is"
        prompt = tok.encode(text, bos=True)
        print(f"Passkey test:\n  prompt: {len(prompt)} tokens\n  passkey: {key}\n  line: {line} of {n_junk}")
        out = lm.generate([prompt], max_new_tokens=16, temperature=0.0, stop_ids=tok.stop_ids)
        print(" What is the secret number? The secret number is" + tok.decode(out[0].tokens, prev=prompt[-1]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
