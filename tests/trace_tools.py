"""Builders of replay traces (the JSON steps bin/trace_run reads) with, for each
step, which (request, position) each written logits row belongs to."""
from __future__ import annotations

import json
import os
import subprocess
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}
        self._n = 0
        self.max_tokens = 0

    def add(self, entries: List[dict], end: Sequence[str], rows: List[Tuple[str, int]]):
        self.steps.append({"step": self._n, "entries": entries, "end": list(end)})
        if rows:
            self.rows[self._n] = rows
        self._n += 1

    def need(self, lengths: Sequence[int]):
        self.max_tokens = max(self.max_tokens, sum((n + 63) // 64 * 64 for n in lengths))


def add_whole(tr: Trace, reqs: Dict[str, List[int]], tag="w"):
    """Each request alone and whole, logits at every position."""
    for rid, toks in reqs.items():
        name = f"{tag}-{rid}"
        tr.need([len(toks)])
        tr.add([{"id": name, "tokens": toks, "want": list(range(len(toks)))}], [name],
               [(rid, p) for p in range(len(toks))])


def add_tail(tr: Trace, reqs: Dict[str, List[int]], tail=32, tag="t"):
    """The prefix whole, then the last ``tail`` tokens one by one."""
    for rid, toks in reqs.items():
        name = f"{tag}-{rid}"
        cut = max(1, len(toks) - tail)
        tr.need([len(toks)])
        tr.add([{"id": name, "tokens": toks[:cut], "want": [cut - 1]}], [], [(rid, cut - 1)])
        for p in range(cut, len(toks)):
            tr.add([{"id": name, "tokens": [toks[p]], "want": [0]}],
                   [name] if p == len(toks) - 1 else [], [(rid, p)])
        if cut == len(toks):
            tr.add([], [name], [])


def add_batches(tr: Trace, reqs: Dict[str, List[int]], batches: List[List[str]],
                prompt_lens: Dict[str, int], tag="b"):
    """Batches of unequal prompts prefilled together, then decoded by feeding the
    trace's own next tokens; shorter requests end earlier; batch after batch."""
    for bi, ids in enumerate(batches):
        name = {rid: f"{tag}{bi}-{rid}" for rid in ids}
        tr.need([len(reqs[rid]) for rid in ids])
        entries, rows = [], []
        for rid in ids:
            n = prompt_lens[rid]
            entries.append({"id": name[rid], "tokens": reqs[rid][:n], "want": list(range(n))})
            rows += [(rid, p) for p in range(n)]
        at = {rid: prompt_lens[rid] for rid in ids}
        live = list(ids)
        done_now = [name[r] for r in live if at[r] == len(reqs[r])]
        live = [r for r in live if at[r] < len(reqs[r])]
        tr.add(entries, done_now, rows)
        while live:
            entries = [{"id": name[r], "tokens": [reqs[r][at[r]]], "want": [0]} for r in live]
            rows = [(r, at[r]) for r in live]
            for r in live:
                at[r] += 1
            done_now = [name[r] for r in live if at[r] == len(reqs[r])]
            live = [r for r in live if at[r] < len(reqs[r])]
            tr.add(entries, done_now, rows)


def run_trace_run(model_dir: str, dtype: str, tr: Trace, out_dir: str, timeout=600,
                  env=None) -> Dict[int, torch.Tensor]:
    """Runs bin/trace_run as a user would and reads the files it wrote."""
    text = "".join(json.dumps(s) + "\n" for s in tr.steps)
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(tr.max_tokens)]
    r = subprocess.run(cmd, input=text, text=True, capture_output=True, timeout=timeout, env=env)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in tr.steps], "a 'done <step>' line per step, in order"
    out = {}
    for step in tr.rows:
        path = os.path.join(out_dir, f"{step}.f32")
        assert os.path.isfile(path), f"no logits file for step {step}"
        out[step] = torch.from_numpy(np.fromfile(path, dtype="<f4").copy())
    extra = [f for f in os.listdir(out_dir) if f.endswith(".f32") and int(f[:-4]) not in tr.rows]
    assert not extra, f"files for steps in which nothing was wanted: {extra}"
    return out


def run_in_process(lm, tr: Trace) -> Dict[int, torch.Tensor]:
    """The same steps through the Python entry point's step function."""
    live, out = {}, {}
    for s in tr.steps:
        fresh = [e["id"] for e in s["entries"] if e["id"] not in live]
        if fresh:
            for rid, slot in zip(fresh, lm.acquire(len(fresh))):
                live[rid] = slot
        if s["entries"]:
            lg = lm.step([e["tokens"] for e in s["entries"]], [live[e["id"]] for e in s["entries"]],
                         [e["want"] for e in s["entries"]])
            if lg is not None:
                out[s["step"]] = lg.float().cpu().reshape(-1)
        ended = [r for r in s["end"] if r in live]
        if ended:
            lm.release([live.pop(r) for r in ended])
    assert not live, "every request of a trace ends"
    return out


def compare(tr: Trace, got: Dict[int, torch.Tensor], refs: Dict[str, torch.Tensor], vocab: int,
            tol: float) -> float:
    """Largest error over all rows relative to the request's largest logit; on a
    failure names the first wrong (step, request, position)."""
    worst = 0.0
    for step in sorted(tr.rows):
        rows = tr.rows[step]
        g = got[step].reshape(-1, vocab)
        assert g.shape[0] == len(rows), f"step {step}: {g.shape[0]} rows written, {len(rows)} wanted"
        for i, (rid, pos) in enumerate(rows):
            ref = refs[rid][pos]
            err = float((g[i] - ref).abs().max() / refs[rid].abs().max())
            worst = max(worst, err)
            assert err <= tol, (f"first wrong row: step {step}, request {rid}, position {pos} "
                                f"(row {i} of {len(rows)}): error {err:.3e} > {tol:.1e}")
    return worst


def forced_decode(lm, reqs, prompts, refs, tol, order=None):
    """Prefill of all prompts in one step, then decode steps through the device-side
    path with the trace's own next tokens forced; a request leaves the batch when its
    tokens run out.  Returns every logits row it compared, in order."""
    eng = lm.engine
    ids = list(order or reqs)
    slots = dict(zip(ids, lm.acquire(len(ids))))
    scale = {r: float(refs[r].abs().max()) for r in ids}
    seen = []

    def check(rid, pos, row):
        err = float((row - refs[rid][pos]).abs().max()) / scale[rid]
        assert err <= tol, f"request {rid}, position {pos}: error {err:.3e} > {tol:.1e}"
        seen.append(row)

    lg = lm.step([reqs[r][:prompts[r]] for r in ids], [slots[r] for r in ids],
                 [[prompts[r] - 1] for r in ids]).float().cpu()
    for i, r in enumerate(ids):
        check(r, prompts[r] - 1, lg[i])
    at = dict(prompts)
    live = [r for r in ids if at[r] < len(reqs[r])]
    current = None
    while live:
        if live != current:
            eng.set_decode_batch([reqs[r][at[r]] for r in live], [slots[r] for r in live],
                                 list(range(len(live))))
            current = list(live)
        else:
            eng.set_decode_tokens([reqs[r][at[r]] for r in live])
        eng.decode_step(len(live), 0.0, 0)
        lg = eng.decode_logits(len(live)).float().cpu()
        # the sampler runs inside the same step: greedy picks the row's maximum
        assert eng.read_decode_tokens(len(live)) == lg.argmax(-1).tolist()
        for i, r in enumerate(live):
            check(r, at[r], lg[i])
            at[r] += 1
        live = [r for r in live if at[r] < len(reqs[r])]
    lm.release(list(slots.values()))
    lm.rt.check_status()
    return torch.stack(seen)
