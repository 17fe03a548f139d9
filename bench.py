#!/usr/bin/env python3
"""Benchmark of the serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: Mistral-7B-v0.2 layer sizes with random bfloat16 weights (--dtype
float16 for the baseline's own 16-bit type: the same kernels, the same decode rate,
and a prefill some 8 % slower, because float16 products draw more power and the part
settles at a lower clock under its cap), a batch of 8 sequences with prompt lengths
drawn uniformly from [64, 2048] inside a context of 4096.  A "step" is one decode
step of the batch.  One JSON line:

  value        decoded tokens per second: K steps timed on the device (CUDA events)
               after W untimed ones that follow the prefill directly
  e2e          the same through LM.generate: every step the host's tokens go down
               from pinned memory and the sampled tokens come back
  prefill      one prompt of 2,048 tokens: tokens/s, ms, fraction of the 16-bit peak
  roofline     bytes the decode step must read (weights once + live cache) / time
  points       decode tokens/s at batch 1, 8 and 64 in the steady state (after 40
               untimed steps: the first steps after a prefill run with the SM clock
               still held down by the power cap), the first 32 steps after a batch
               of 2,048-token prompts, and the two other workloads
               (Llama-3.2-1B sizes at batch 64, Mistral-7B-v0.1 sizes at batch 8
               decoding past its window of 4096)
  clocks       SM clocks and throttle reasons sampled during the timed region
  gpu_launches kernels of this library launched inside the timed region

Inputs are far larger than L2 (a decode step streams all weights), so no L2
flush is needed between timed iterations.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MISTRAL_7B = {
    "architectures": ["MistralForCausalLM"],
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 32000, "max_position_embeddings": 32768, "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0, "sliding_window": None, "tie_word_embeddings": False,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
CONTEXT = 4096
LLAMA32_1B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "sliding_window": None, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 128000, "eos_token_id": 128001,
}
MISTRAL_7B_V01 = dict(MISTRAL_7B, rope_theta=10000.0, sliding_window=4096)
# name -> (config.json keys, context, default batch, prompt lengths lo..hi)
WORKLOADS = {
    "mistral-7b-v0.2": (MISTRAL_7B, 4096, 8, 64, 2048),
    "llama-3.2-1b": (LLAMA32_1B, 8192, 64, 16, 1024),
    "mistral-7b-v0.1": (MISTRAL_7B_V01, 8192, 8, 6000, 6000),     # decodes past the 4096 window
}
STEADY = 40          # untimed steps before a steady-state point is timed
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _find_number(d, key):
    """The first numeric value stored under `key` anywhere in a nested JSON value."""
    if isinstance(d, dict):
        v = d.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            return float(v)
        for x in d.values():
            r = _find_number(x, key)
            if r is not None:
                return r
    elif isinstance(d, list):
        for x in d:
            r = _find_number(x, key)
            if r is not None:
                return r
    return None


def peaks():
    """Measured peaks if the driver left them beside this file, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            hbm, burst = _find_number(d, "hbm_gbs"), _find_number(d, "bf16_tflops")
            if hbm and burst:
                out = {"hbm_gbs": hbm, "bf16_tflops": burst, "source": "measured"}
                sustained = _find_number(d, "bf16_tflops_sustained")
                if sustained:
                    out["bf16_tflops_sustained"] = sustained
                return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: NVML from a thread of this
    process every 10 ms (a timed region of 64 decode steps lasts 0.2 s), or `nvidia-smi -lms`
    where the NVML binding is missing.  Only reads; nothing is set."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.thread = None
        self.lines = []
        self.samples = []          # (sm MHz, reasons bit mask)
        self.max_mhz = None
        self.running = False

    def _nvml(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            first = visible.split(",")[0].strip() if visible else "0"
            h = (pynvml.nvmlDeviceGetHandleByUUID(first) if first.startswith("GPU-")
                 else pynvml.nvmlDeviceGetHandleByIndex(int(first) if first.isdigit() else 0))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            return pynvml, h
        except Exception:
            return None, None

    def start(self):
        nv, h = self._nvml()
        if nv is not None:
            self.running = True

            def loop():
                while self.running:
                    try:
                        self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                             int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                                             if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                             else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
                    except Exception:
                        pass
                    time.sleep(0.01)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.thread is not None:
            self.running = False
            self.thread.join(timeout=2)
            mhz = sorted(m for m, _ in self.samples)
            # NVML's reason bits: 0x8 hw slowdown, 0x40 hw thermal, 0x20 sw thermal, 0x4 sw power cap
            bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                    "sw_power_cap": 0x4}
            reasons = sorted(n for n, b in bits.items() if any(r & b for _, r in self.samples))
            return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                    "reasons": reasons, "samples": len(mhz), "source": "nvml, every 10 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        for l in self.lines:
            p = [x.strip() for x in l.split(",")]
            if len(p) < 6:
                continue
            try:
                mhz.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for n, v in zip(self.NAMES, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz), "source": "nvidia-smi -lms 100"}


def prompt_lengths(n, lo, hi, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def random_prompts(lengths, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def decode_bytes(lm, contexts):
    """Bytes one decode step has to read: every weight once (the embedding
    table only one row per sequence) plus the keys and values of the live
    sequences.  The model's parts do the counting."""
    return lm.model.step_bytes(contexts)


def prefill_flops(lm, T):
    return lm.model.step_flops([T], [0], n_want=1)


def prefill_batch(lm, prompts, group=8):
    """Prefills all prompts (in groups, to bound scratch memory) and leaves them
    ready to decode; returns slots and the first sampled tokens."""
    import torch
    slots = lm.acquire(len(prompts))
    first = []
    for i in range(0, len(prompts), group):
        ps, ss = prompts[i:i + group], slots[i:i + group]
        logits = lm.step(ps, ss, [[len(p) - 1] for p in ps])
        first += logits.argmax(-1).tolist()
    torch.cuda.synchronize()
    return slots, first


def time_decode(lm, batch, steps, warmup, seed, sampler=None, lo=64, hi=2048):
    """Device-timed decode steps of a batch with prompt lengths U[lo, hi]; `warmup`
    untimed steps come first, directly after the prefill."""
    import torch
    from yalm_b200.csrc import ops
    lens = sorted(prompt_lengths(batch, lo, hi, seed), reverse=True)   # rows longest first, as LM.generate orders them
    prompts = random_prompts(lens, lm.config.vocab_size, seed + 1)
    slots, first = prefill_batch(lm, prompts)
    eng = lm.engine
    eng.set_decode_batch(first, slots, list(range(batch)))
    for _ in range(warmup):
        eng.decode_step(batch, 0.0, 0)
    torch.cuda.synchronize()
    ctx0 = [eng.cache.host_pos[s] for s in slots]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.start()
    l0 = ops.LAUNCHES
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        eng.decode_step(batch, 0.0, 0)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    clocks = sampler.stop() if sampler else None
    launches = ops.LAUNCHES - l0
    ctx_mid = [c + steps // 2 for c in ctx0]
    lm.rt.check_status()
    lm.release(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "contexts": ctx_mid, "clocks": clocks, "prompt_lens": lens}


def time_e2e(lm, batch, steps, warmup, seed, lo=64, hi=2048):
    """The same steps through the public entry point: host tokens in, host tokens out.
    One generate() call decodes warmup + steps tokens per sequence; the last `steps`
    decode steps are the timed ones (each timed host to host around its pinned H2D
    copy, the graph replay and the D2H read)."""
    lens = prompt_lengths(batch, lo, hi, seed)
    prompts = random_prompts(lens, lm.config.vocab_size, seed + 1)
    lm.generate(prompts, max_new_tokens=4, temperature=0.0, ignore_eos=True)     # graphs, buffers
    lm.generate(prompts, max_new_tokens=warmup + steps + 1, temperature=0.0, ignore_eos=True)
    st = lm.last_stats
    timed = st["step_seconds"][-steps:]
    n = len(timed)
    all_n = st["decode_steps"]
    return {"value": batch * n / sum(timed), "unit": "tokens/s",
            "h2d_bytes_per_step": st["h2d_bytes"] / all_n, "d2h_bytes_per_step": st["d2h_bytes"] / all_n,
            "steps": n, "warmup_steps": all_n - n}


def time_prefill(lm, T, reps, pk):
    import torch
    prompt = random_prompts([T], lm.config.vocab_size, 99)[0]
    times = []
    for i in range(reps + 2):
        s = lm.acquire(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        lm.step([prompt], s, [[T - 1]])
        b.record()
        torch.cuda.synchronize()
        lm.release(s)
        if i >= 2:
            times.append(a.elapsed_time(b))
    ms = sorted(times)[len(times) // 2]
    fl = prefill_flops(lm, T)
    out = {"value": T / (ms / 1e3), "tokens": T, "ms": ms,
           "frac": fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "of": pk["source"]}
    if "bf16_tflops_sustained" in pk:       # the step is short; the burst figure is the denominator
        out["frac_of_sustained"] = fl / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)
    return out


def reference_arm(args):
    """The unmodified reference on the same layer sizes (see baseline/run_reference.py).
    It serves one sequence at a time, so the batch's requests run one after another and
    its decode rate is its batch-1 rate; the prompt has the batch's mean length."""
    if args.gpus != 1:
        print(f"bench.py: the reference runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import run_reference
    base_cfg, context, default_batch, lo, hi = WORKLOADS[args.workload]
    if args.prompt_lengths:
        lo, hi = args.prompt_lengths
    batch = args.batch or default_batch
    layers = args.layers or base_cfg["num_hidden_layers"]
    cfg = dict(base_cfg, num_hidden_layers=layers)
    cfg = {k: v for k, v in cfg.items() if v is not None}
    lens = prompt_lengths(batch, lo, hi, 1)                   # the lengths the other arm draws
    prompt_len = int(round(sum(lens) / len(lens)))
    W = max(3, args.warmup)
    try:
        r = run_reference.run(cfg, context, prompt_len, args.steps, W, sampler=ClockSampler())
    except run_reference.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e).replace("\n", " ")[:400]}))
        return 0
    out = {
        "metric": f"decode tokens/s at batch {batch} ({args.workload} shapes, context {context})",
        "value": r["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": W,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {
            "model": f"{args.workload}-shapes-random", "layers": layers,
            "layers_of_config": base_cfg["num_hidden_layers"], "hidden": base_cfg["hidden_size"],
            "ffn": base_cfg["intermediate_size"], "heads": base_cfg["num_attention_heads"],
            "kv_heads": base_cfg["num_key_value_heads"], "head_dim": base_cfg["head_dim"],
            "vocab": base_cfg["vocab_size"],
            "global_batch": f"{batch} requests served one after another (the reference takes one "
                            f"sequence per forward)",
            "seq_len": context, "prompt_len": r["prompt_len"], "parallelism": "single-gpu",
            "timing": "host clock between tokens arriving on the program's output",
            "weights": "random N(0,0.02) float16, norms 1, packed by the reference's convert.py",
            "reported_decode_tok_s": r.get("reported_decode_tok_s"),
            "reported_throughput": r["reported"].get("throughput"),
            "reported_bandwidth_gbs": r["reported"].get("bandwidth"),
        },
        # the program is end to end by construction: the token id goes down as a kernel
        # argument and the logits come back through mapped host memory every step
        "e2e": {"value": r["tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4,
                "d2h_bytes_per_step": 4 * base_cfg["vocab_size"], "steps": args.steps},
        "clocks": r["clocks"],
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mistral-7b-v0.2", choices=sorted(WORKLOADS),
                    help="layer sizes, context and prompt lengths (default: the headline one)")
    ap.add_argument("--dtype", default="bfloat16", choices=["float16", "bfloat16"],
                    help="the 16-bit type of weights, activations and cache (the reference arm "
                         "runs the baseline's float16: the same width)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1/64 and prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (profiling)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="only the 2,048-token prefill, once (profiling); prints its record alone")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="with --prefill-only: the prompt's length (the context grows to hold it)")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch decode kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--max-tokens", type=int, default=None,
                    help="a cache pool of this many tokens in pages of 64 behind a page table, "
                         "instead of one block of the context length per sequence")
    ap.add_argument("--prompt-lengths", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="prompt lengths are drawn from U[LO, HI] instead of the workload's range")
    ap.add_argument("--decode-chunks", type=int, default=None,
                    help="64-key chunks per block of the tensor-core decode attention (default: "
                         "the attention part decides by the batch)")
    ap.add_argument("--decode-warps", type=int, default=None, choices=[2, 4],
                    help="warps per block of the tensor-core decode attention (default: the "
                         "attention part decides by the batch)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    import torch
    from yalm_b200 import LM
    pk = peaks()
    base_cfg, context, default_batch, lo, hi = WORKLOADS[args.workload]
    args.batch = args.batch or default_batch
    args.layers = args.layers or base_cfg["num_hidden_layers"]
    headline = args.workload == "mistral-7b-v0.2"
    cfg = dict(base_cfg, num_hidden_layers=args.layers)
    points_wanted = headline and not (args.no_points or args.prefill_only)

    def build(config, ctx, max_batch):
        t0 = time.time()
        lm = LM.from_random(config, seed=0, dtype=args.dtype, std=0.02, norm_jitter=0.0,
                            max_context=ctx, max_batch=max_batch, max_tokens=args.max_tokens)
        torch.cuda.synchronize()
        print(f"[bench] model ready in {time.time() - t0:.0f} s "
              f"({lm.model.weight_bytes() / 1e9:.1f} GB weights, {lm.engine.cache.bytes() / 1e9:.1f} GB cache)",
              file=sys.stderr, flush=True)
        if args.no_graphs:
            lm.engine.use_graphs = False
        lm.rt.decode_attention_warps = args.decode_warps
        lm.rt.decode_attention_chunks = args.decode_chunks
        return lm

    if args.prefill_only:
        context = max(context, args.prefill_tokens)
        cfg = dict(cfg, max_position_embeddings=max(cfg.get("max_position_embeddings", 0), context))
    lm = build(cfg, context, max(64, args.batch) if points_wanted else (1 if args.prefill_only else args.batch))
    if args.prefill_only:
        print(json.dumps({"prefill": time_prefill(lm, args.prefill_tokens, 1, pk), "layers": args.layers}))
        return 0
    W = max(3, args.warmup)
    main_run = time_decode(lm, args.batch, args.steps, W, seed=1, sampler=ClockSampler(), lo=lo, hi=hi)
    by = decode_bytes(lm, main_run["contexts"])
    achieved = by / (main_run["ms_per_step"] / 1e3) / 1e9
    e2e = None if args.no_e2e else time_e2e(lm, args.batch, args.steps, W, seed=1, lo=lo, hi=hi)
    out = {
        "metric": f"decode tokens/s at batch {args.batch} ({args.workload} shapes, context {context})",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": W, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": {"float16": "fp16", "bfloat16": "bf16"}[args.dtype], "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{args.workload}-shapes-random", "layers": args.layers,
            "layers_of_config": base_cfg["num_hidden_layers"], "hidden": base_cfg["hidden_size"],
            "ffn": base_cfg["intermediate_size"], "heads": base_cfg["num_attention_heads"],
            "kv_heads": base_cfg["num_key_value_heads"], "head_dim": base_cfg["head_dim"],
            "vocab": base_cfg["vocab_size"], "global_batch": args.batch, "seq_len": context,
            "window": base_cfg.get("sliding_window"), "prompt_lens": f"uniform[{lo},{hi}]",
            "mean_context": sum(main_run["contexts"]) / len(main_run["contexts"]),
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights streamed each step)",
            "peaks": pk["source"], "weights": "random N(0,0.02), norms 1",
        },
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": by,
                     "of": pk["source"]},
    }
    if points_wanted:
        out["prefill"] = time_prefill(lm, 2048, 5, pk)
        pts = {"steady_warmup_steps": STEADY}

        def point(name, model, b, steps, warmup, seed, lo_, hi_):
            r = time_decode(model, b, steps, warmup, seed=seed, lo=lo_, hi=hi_)
            pts[name] = r["tok_s"]
            pts[name + "_ms"] = r["ms_per_step"]
            pts[name + "_hbm_frac"] = (decode_bytes(model, r["contexts"]) / (r["ms_per_step"] / 1e3)
                                       / 1e9 / pk["hbm_gbs"])

        half = max(16, args.steps // 2)
        point("decode_b1", lm, 1, half, STEADY, 11, lo, hi)
        point("decode_b8", lm, 8, half, STEADY, 1, lo, hi)
        point("decode_b64", lm, 64, half, STEADY, 74, lo, hi)
        # what a short generate() call sees: the 32 steps right after a batch of long prompts
        # (run once before, untimed, so that this shape's graph exists as it would in a server)
        time_decode(lm, 8, 32, 0, seed=5, lo=2048, hi=2048)
        point("decode_b8_first32_after_2048_token_prompts", lm, 8, 32, 0, 5, 2048, 2048)
        # the reference's one published figure: 63.8 tokens/s at batch 1 on an RTX 4090
        # (its README; other hardware, so no vs_baseline for the headline metric)
        pts["decode_b1_vs_published_63.8"] = pts["decode_b1"] / 63.8
        del lm
        torch.cuda.empty_cache()
        for name, key in (("llama-3.2-1b", "llama_3.2_1b_b64"), ("mistral-7b-v0.1", "mistral_7b_v0.1_b8")):
            c2, ctx2, b2, lo2, hi2 = WORKLOADS[name]
            other = build(dict(c2), ctx2, b2)
            point(key, other, b2, half, STEADY, 21, lo2, hi2)
            del other
            torch.cuda.empty_cache()
        out["points"] = pts
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
