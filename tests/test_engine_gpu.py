"""The engine against the plain implementation on a GPU: every request alone
and whole; with the last 32 tokens one by one; in batches of unequal lengths
whose shorter requests end earlier, batch after batch so that slots are used
again; in 32-bit, bfloat16 and float16; through bin/trace_run and through the Python
entry point."""
import os

import pytest
import torch

from helpers import CONFIGS, DTYPES, TOL, make_weights, random_tokens, write_model
from plain_model import plain_forward, plain_generate_greedy, plain_perplexity
from trace_tools import (Trace, add_batches, add_tail, add_whole, compare, forced_decode, run_in_process,
                         run_trace_run)

pytestmark = pytest.mark.gpu

# request lengths and prompt lengths per configuration (contexts 128 / 96 / 160)
REQUESTS = {
    "tiny_a": {"lens": {"r0": 21, "r1": 33, "r2": 47, "r3": 100, "r4": 128, "r5": 2},
               "prompts": {"r0": 5, "r1": 17, "r2": 31, "r3": 64, "r4": 96, "r5": 1},
               "batches": [["r0", "r1", "r2"], ["r3", "r5", "r4"], ["r2", "r0"]]},
    "tiny_b": {"lens": {"r0": 21, "r1": 29, "r2": 60, "r3": 90, "r4": 96, "r5": 34},
               "prompts": {"r0": 1, "r1": 9, "r2": 40, "r3": 70, "r4": 33, "r5": 32},
               "batches": [["r0", "r1", "r2", "r3"], ["r4", "r5"], ["r3", "r0", "r1"]]},
    "tiny_c": {"lens": {"r0": 7, "r1": 45, "r2": 81, "r3": 160},
               "prompts": {"r0": 3, "r1": 41, "r2": 39, "r3": 100},
               "batches": [["r0", "r1", "r2"], ["r3", "r0"]]},
    "tiny_e": {"lens": {"r0": 40, "r1": 400, "r2": 170, "r3": 129},
               "prompts": {"r0": 8, "r1": 360, "r2": 160, "r3": 128},
               "batches": [["r0", "r1", "r2"], ["r3", "r0"]]},
    "tiny_d": {"lens": {"r0": 9, "r1": 70, "r2": 38},
               "prompts": {"r0": 2, "r1": 50, "r2": 37},
               "batches": [["r0", "r1", "r2"], ["r2", "r0"]]},
}


def _setup(name):
    cfg, seed = CONFIGS[name]
    w = make_weights(cfg, seed)
    reqs = {rid: random_tokens(n, cfg["vocab_size"], 100 + i)
            for i, (rid, n) in enumerate(REQUESTS[name]["lens"].items())}
    refs = {rid: plain_forward(cfg, w, t) for rid, t in reqs.items()}
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, reqs, tail=32)
    add_batches(tr, reqs, REQUESTS[name]["batches"], REQUESTS[name]["prompts"])
    return cfg, w, reqs, refs, tr


_cache = {}


def setup(name):
    if name not in _cache:
        _cache[name] = _setup(name)
    return _cache[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_trace_run_matches_plain_model(name, dtype, tmp_path):
    cfg, w, reqs, refs, tr = setup(name)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    got = run_trace_run(model_dir, dtype, tr, str(tmp_path / "out"))
    compare(tr, got, refs, cfg["vocab_size"], TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
def test_step_function_matches_plain_model(name, dtype):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, w, reqs, refs, tr = setup(name)
    # the cache is sized by the tokens held, so its rows live in pages wherever that is
    # less than slots x context (the same sizing as bin/trace_run's)
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=max(1, tr.max_tokens // 64),
            max_tokens=tr.max_tokens)
    got = run_in_process(lm, tr)
    compare(tr, got, refs, cfg["vocab_size"], TOL[dtype])
    assert lm.engine.cache.slots.free_count == lm.max_batch
    assert all(f == g["pool"].n_slots for f, g in zip(lm.engine.cache.free_pages(),
                                                      [g for g in lm.engine.cache.groups if "pool" in g]))


def test_the_two_ways_of_cutting_agree_beyond_the_plain_models_tolerance():
    """32-bit logits at a position are the same to rounding whether the position
    was part of a whole prompt, decoded alone, or decoded inside a batch."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, w, reqs, refs, tr = setup("tiny_b")
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=max(1, tr.max_tokens // 64))
    got = run_in_process(lm, tr)
    seen = {}
    for step, rows in tr.rows.items():
        g = got[step].reshape(-1, cfg["vocab_size"])
        for i, key in enumerate(rows):
            if key in seen:
                assert float((g[i] - seen[key]).abs().max()) <= 2e-5 * float(refs[key[0]].abs().max())
            else:
                seen[key] = g[i]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_the_window(dtype):
    """300 tokens decoded one by one through a ring of 32 rows."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg = dict(CONFIGS["tiny_b"][0], max_position_embeddings=512)
    w = make_weights(cfg, 7)
    toks = random_tokens(330, cfg["vocab_size"], 5)
    ref = plain_forward(cfg, w, toks)
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=1)
    s = lm.acquire(1)
    lg = lm.step([toks[:30]], s, [[29]])
    worst = float((lg[0].cpu() - ref[29]).abs().max() / ref.abs().max())
    for p in range(30, 330):
        lg = lm.step([[toks[p]]], s, [[0]])
        worst = max(worst, float((lg[0].cpu() - ref[p]).abs().max() / ref.abs().max()))
    lm.release(s)
    assert worst <= TOL[dtype], worst


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype):
    """A prompt of one token, then positions 1, 2, 3 alone; and steps that want nothing."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    toks = random_tokens(6, cfg["vocab_size"], 9)
    ref = plain_forward(cfg, w, toks)
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=2)
    s = lm.acquire(1)
    assert lm.step([[toks[0]]], s, [[]]) is None               # nothing wanted: no logits
    for p in range(1, 6):
        lg = lm.step([[toks[p]]], s, [[0]])
        assert float((lg[0].cpu() - ref[p]).abs().max() / ref.abs().max()) <= TOL[dtype], p
    lm.release(s)


def test_greedy_generation_through_the_entry_point():
    """Unequal prompts, a stop token, more requests than slots; 32-bit tokens
    equal the plain model's, step for step."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    for name in ("tiny_a", "tiny_b"):
        cfg, seed = CONFIGS[name]
        w = make_weights(cfg, seed)
        prompts = [random_tokens(n, cfg["vocab_size"], 40 + n) for n in (5, 17, 31, 2, 9)]
        lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2)
        free = plain_generate_greedy(cfg, w, prompts[0], 12)
        stop = [free[5]]
        want = [plain_generate_greedy(cfg, w, p, 12, stop=stop) for p in prompts]
        got = lm.generate(prompts, max_new_tokens=12, temperature=0.0, stop_ids=stop)
        assert [c.tokens for c in got] == want
        assert got[0].finish_reason == "stop" and got[0].tokens[-1] == stop[0]
        assert all(c.finish_reason in ("stop", "length") for c in got)
        assert lm.engine.cache.slots.free_count == 2
        # the same through replayed graphs a second time, and without graphs
        again = lm.generate(prompts, max_new_tokens=12, temperature=0.0, stop_ids=stop)
        assert [c.tokens for c in again] == want
        lm.engine.use_graphs = False
        assert [c.tokens for c in lm.generate(prompts, 12, 0.0, stop_ids=stop)] == want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_e"])
def test_decode_fast_path_logits_across_graph_keys(name, dtype, monkeypatch):
    """The path generation runs (device token buffer, captured graphs, sampler in the
    graph) with the trace's own tokens forced: its logits against the plain model at
    every step.  Context buckets of 32 positions and a capture on the second step make
    the sequences cross many graph keys, replay graphs planned for a shorter context,
    and shrink the batch when a request ends; the same schedule without graphs must
    give the same bits."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    from yalm_b200.engine.step import Engine
    monkeypatch.setattr(Engine, "CTX_BUCKET", 32)
    monkeypatch.setattr(Engine, "GRAPH_AFTER", 2)
    cfg, w, reqs, refs, _ = setup(name)
    prompts = dict(REQUESTS[name]["prompts"])
    ids = REQUESTS[name]["batches"][0]
    sub = {r: reqs[r] for r in ids}
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(ids))
    fast = forced_decode(lm, sub, prompts, refs, TOL[dtype])
    assert len(lm.engine._graphs) >= (2 if name == "tiny_e" else 1)    # tiny_e crosses a bucket
    lm.engine.use_graphs = False
    assert torch.equal(fast, forced_decode(lm, sub, prompts, refs, TOL[dtype]))
    assert lm.engine.cache.slots.free_count == lm.max_batch


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_e"])
def test_decode_with_two_warp_attention_blocks(name, dtype):
    """The decode attention's second block shape (two warps; the engine takes it by itself only
    for grids of several waves) forced on the trace's batch, with the rotary kernel apart:
    logits against the plain model at every step, with and without graphs."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, w, reqs, refs, _ = setup(name)
    prompts = dict(REQUESTS[name]["prompts"])
    ids = REQUESTS[name]["batches"][0]
    sub = {r: reqs[r] for r in ids}
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(ids))
    lm.rt.decode_attention_warps = 2
    lm.rt.decode_rope_in_attention = False
    fast = forced_decode(lm, sub, prompts, refs, TOL[dtype])
    lm.engine.use_graphs = False
    assert torch.equal(fast, forced_decode(lm, sub, prompts, refs, TOL[dtype]))
    lm.rt.decode_attention_warps = 4
    four = forced_decode(lm, sub, prompts, refs, TOL[dtype])
    assert (fast - four).abs().max().item() <= TOL[dtype] * max(1.0, four.abs().max().item())


def test_temperature_sampling_is_per_request_and_reproducible():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    prompts = [random_tokens(n, cfg["vocab_size"], 80 + n) for n in (6, 11, 3)]
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=4)
    a = lm.generate(prompts, max_new_tokens=8, temperature=1.0, seed=3, ignore_eos=True)
    b = lm.generate(prompts, max_new_tokens=8, temperature=1.0, seed=3, ignore_eos=True)
    c = lm.generate(prompts, max_new_tokens=8, temperature=1.0, seed=4, ignore_eos=True)
    assert [x.tokens for x in a] == [x.tokens for x in b]
    assert [x.tokens for x in a] != [x.tokens for x in c]
    # request 0 alone draws the same tokens as request 0 inside the batch
    alone = lm.generate(prompts[:1], max_new_tokens=8, temperature=1.0, seed=3, ignore_eos=True)
    assert alone[0].tokens == a[0].tokens


def test_perplexity_matches_plain_model():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_b"]
    w = make_weights(cfg, seed)
    toks = random_tokens(60, cfg["vocab_size"], 2)
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=1)
    ppl, err = lm.perplexity(toks)
    rp, re = plain_perplexity(cfg, w, toks)
    assert abs(ppl - rp) / rp < 1e-4 and abs(err - re) / re < 1e-3


def test_slots_do_not_leak_into_each_other():
    """Two sequences decoded in turn in neighbouring slots, then a third that
    takes over a used slot: each equals its own whole-prompt logits."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    V = cfg["vocab_size"]
    ta, tb, tc = (random_tokens(n, V, 200 + n) for n in (40, 23, 31))
    ra, rb, rc = (plain_forward(cfg, w, t) for t in (ta, tb, tc))
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2)
    sa, sb = lm.acquire(2)
    lm.step([ta[:10]], [sa], [[]])
    lm.step([tb[:20]], [sb], [[]])
    lm.step([ta[10:11]], [sa], [[]])
    # b alone, then a alone, with lengths 20 vs 11: a row of b must not show up in a
    lg = lm.step([tb[20:23]], [sb], [[2]])
    assert float((lg[0].cpu() - rb[22]).abs().max() / rb.abs().max()) <= TOL["float32"]
    lm.release([sb])
    (sc,) = lm.acquire(1)
    assert sc == sb                                           # the slot is used again
    lg = lm.step([tc, ta[11:40]], [sc, sa], [[30], [28]])
    assert float((lg[0].cpu() - rc[30]).abs().max() / rc.abs().max()) <= TOL["float32"]
    assert float((lg[1].cpu() - ra[39]).abs().max() / ra.abs().max()) <= TOL["float32"]


def test_step_refuses_bad_requests():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    from yalm_b200.engine.step import StepError
    cfg, seed = CONFIGS["tiny_a"]
    lm = LM(config_from_dict(cfg), make_weights(cfg, seed), dtype="float32", max_batch=2)
    (s,) = lm.acquire(1)
    with pytest.raises(StepError, match="vocabulary"):
        lm.step([[1, 999]], [s], [[]])
    with pytest.raises(StepError, match="context"):
        lm.step([[1] * 129], [s], [[]])
    with pytest.raises(StepError, match="not held"):
        lm.step([[1]], [1 - s], [[]])
    with pytest.raises(StepError, match="twice"):
        lm.step([[1], [2]], [s, s], [[], []])
    with pytest.raises(IndexError):
        lm.step([[1, 2]], [s], [[2]])
    lm.step([[1, 2]], [s], [[1]])                               # still usable afterwards


def test_a_cache_beyond_the_device_memory_is_refused_before_it_is_allocated():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    from yalm_b200.engine.step import CacheMemoryError
    cfg, seed = CONFIGS["tiny_a"]
    with pytest.raises(CacheMemoryError, match="GiB are free"):
        LM(config_from_dict(cfg), make_weights(cfg, seed), dtype="float32", max_batch=10 ** 8)


def test_command_line_completion_and_perplexity(tmp_path):
    """python -m yalm_b200 with token-id prompts on a random model folder that
    the random-weights mode wrote."""
    import json
    import subprocess
    import sys
    from trace_tools import ROOT
    cfg, _ = CONFIGS["tiny_a"]
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))
    model = str(tmp_path / "model")
    base = [sys.executable, "-m", "yalm_b200", model, "--dtype", "float32"]
    r = subprocess.run(base + ["--random-weights", str(tmp_path / "cfg.json"), "--seed", "3",
                               "--tokens", "5,6,7;9,10", "-n", "5", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert os.path.isfile(os.path.join(model, "model.safetensors"))
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens:")]
    assert len(lines) == 2 and "throughput" in r.stdout
    from yalm_b200.weights import load_checkpoint
    w = load_checkpoint(model)
    want = plain_generate_greedy(cfg, w, [5, 6, 7], 5, stop=[2])
    assert [int(t) for t in lines[0].split("(")[0].split()[1:]] == want
    r = subprocess.run(base + ["-m", "perp", "--tokens", ",".join(map(str, range(3, 40)))],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    ppl = float(r.stdout.split("perplexity:")[1].split()[0])
    assert abs(ppl - plain_perplexity(cfg, w, list(range(3, 40)))[0]) / ppl < 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_cut_into_steps_on_a_full_ring(dtype):
    """Several tokens at once on top of a ring that already wrapped (not a
    schedule of the generation loop, but the step function takes it): the ring
    rows are written after the attention has read the keys they replace."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_b"]                               # window 32, context 96
    w = make_weights(cfg, seed)
    toks = random_tokens(96, cfg["vocab_size"], 11)
    ref = plain_forward(cfg, w, toks)
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=1)
    s = lm.acquire(1)
    got = [lm.step([toks[a:b]], s, [list(range(b - a))]).cpu()
           for a, b in ((0, 50), (50, 51), (51, 80), (80, 96))]
    err = float((torch.cat(got) - ref).abs().max() / ref.abs().max())
    assert err <= TOL[dtype], err


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("attention", ["auto", "mma"])
def test_both_tensor_core_prefill_attentions_inside_the_engine(attention, dtype):
    """Whole prompts go through the TMEM attention kernel by default; attention="mma" keeps
    them on the mma.sync kernel, which otherwise only sees prompts cut into steps."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_e"]
    w = make_weights(cfg, seed)
    toks = [random_tokens(n, cfg["vocab_size"], 300 + n) for n in (390, 7, 129)]
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=3, attention=attention)
    s = lm.acquire(3)
    lg = lm.step(toks, s, [[len(t) - 1] for t in toks]).cpu()
    for i, t in enumerate(toks):
        ref = plain_forward(cfg, w, t)
        assert float((lg[i] - ref[-1]).abs().max() / ref.abs().max()) <= TOL[dtype]


def test_a_model_stored_in_float16(tmp_path):
    """float16 storage: the 32-bit path widens the stored values exactly (its logits match
    the plain model on those values to 32-bit rounding); the float16 path keeps them as
    stored; the bfloat16 path rounds them to bfloat16 and stays inside its tolerance.
    Norm weights stay in 32 bits as stored."""
    from yalm_b200 import LM
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    stored = {k: (v if v.dtype == torch.float32 else (v.float() * 1.001).to(torch.float16))
              for k, v in w.items()}                            # values that bfloat16 cannot hold
    assert any(v.dtype == torch.float16 and not torch.equal(v.float(), v.to(torch.bfloat16).float())
               for v in stored.values())
    write_model(str(tmp_path / "m"), cfg, stored)
    toks = random_tokens(40, cfg["vocab_size"], 77)
    ref = plain_forward(cfg, {k: v.float() for k, v in stored.items()}, toks)
    for dtype in DTYPES:
        lm = LM.from_pretrained(str(tmp_path / "m"), dtype=dtype, max_batch=1)
        if dtype == "float16":
            assert torch.equal(lm.model.head.weight.cpu(), stored["lm_head.weight"])
        s = lm.acquire(1)
        lg = lm.step([toks], s, [list(range(40))]).cpu()
        assert float((lg - ref).abs().max() / ref.abs().max()) <= TOL[dtype], dtype


def test_a_packed_one_file_model(tmp_path):
    """A folder packed into one file (configuration in the metadata) loads to the same model."""
    from yalm_b200 import LM
    from yalm_b200.weights import pack_model_dir
    cfg, seed = CONFIGS["tiny_b"]
    w = make_weights(cfg, seed)
    write_model(str(tmp_path / "m"), cfg, w)
    pack_model_dir(str(tmp_path / "m"), str(tmp_path / "one.safetensors"))
    toks = random_tokens(30, cfg["vocab_size"], 5)
    got = []
    for path in (str(tmp_path / "m"), str(tmp_path / "one.safetensors")):
        lm = LM.from_pretrained(path, dtype="float32", max_batch=1)
        s = lm.acquire(1)
        got.append(lm.step([toks], s, [list(range(30))]).cpu())
    assert torch.equal(got[0], got[1])
    ref = plain_forward(cfg, w, toks)
    assert float((got[1] - ref).abs().max() / ref.abs().max()) <= TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_window_imposed_on_a_model_that_has_none(dtype):
    """window_override=24 on tiny-A (no window in its config.json): generation goes on
    past 24 positions in a ring of 24 rows, and the logits are those of the plain model
    with sliding_window = 24."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    toks = random_tokens(100, cfg["vocab_size"], 31)
    ref = plain_forward(dict(cfg, sliding_window=24), w, toks)
    assert float((ref - plain_forward(cfg, w, toks)).abs().max()) > 1e-3     # the window matters
    lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=2, window_override=24)
    assert lm.engine.cache.groups[0]["capacity"] == 24 and lm.context == 128
    s = lm.acquire(1)
    lg = lm.step([toks[:40]], s, [list(range(40))]).cpu()      # a prompt longer than the ring
    worst = float((lg - ref[:40]).abs().max())
    for p in range(40, 100):
        worst = max(worst, float((lm.step([[toks[p]]], s, [[0]])[0].cpu() - ref[p]).abs().max()))
    assert worst / float(ref.abs().max()) <= TOL[dtype]


def test_context_option_of_the_command_line_is_a_window_and_batch_file(tmp_path):
    """-T 24 on the command line: 60 greedy tokens past a ring of 24 rows equal the plain
    model's with sliding_window = 24; --batch-file gives several prompts."""
    import subprocess
    import sys
    from trace_tools import ROOT
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    model = write_model(str(tmp_path / "m"), cfg, w)
    prompts = [random_tokens(9, cfg["vocab_size"], 50), random_tokens(30, cfg["vocab_size"], 51)]
    (tmp_path / "batch.txt").write_text("\n".join(",".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, "-m", "yalm_b200", model, "--dtype", "float32", "-T", "24",
                        "--batch-file", str(tmp_path / "batch.txt"), "-n", "60", "-t", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens:")]
    assert len(lines) == 2
    windowed = dict(cfg, sliding_window=24)
    for line, p in zip(lines, prompts):
        got = [int(t) for t in line.split("(")[0].split()[1:]]
        assert got == plain_generate_greedy(windowed, w, p, 60, stop=[2])


def test_perplexity_of_a_text_longer_than_the_context():
    """The text is cut into sequences of `context` tokens that overlap by one token, and
    each runs in portions: every token but the first is predicted once."""
    import math
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]                               # context 128
    w = make_weights(cfg, seed)
    toks = random_tokens(300, cfg["vocab_size"], 8)
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=1)
    ppl, err = lm.perplexity(toks, chunk=50)
    vals = []
    for a in (0, 127, 254):
        seg = toks[a:a + 128]
        lp = torch.log_softmax(plain_forward(cfg, w, seg).double(), -1)
        vals += [lp[i, seg[i + 1]].item() for i in range(len(seg) - 1)]
    assert len(vals) == 299
    want = math.exp(-sum(vals) / len(vals))
    assert abs(ppl - want) / want < 1e-4 and err > 0
    assert lm.engine.cache.slots.free_count == 1


def test_trace_run_takes_random_weights_of_a_configuration(tmp_path):
    """--model random:<config.json>:<seed> is the model that LM.from_random draws."""
    import json
    from yalm_b200 import LM
    cfg, _ = CONFIGS["tiny_c"]
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))
    toks = random_tokens(45, cfg["vocab_size"], 3)
    tr = Trace()
    add_whole(tr, {"r": toks})
    got = run_trace_run(f"random:{tmp_path / 'cfg.json'}:5", "float32", tr, str(tmp_path / "out"))
    lm = LM.from_random(cfg, seed=5, dtype="float32", max_batch=1)
    s = lm.acquire(1)
    want = lm.step([toks], s, [list(range(45))]).cpu()
    assert torch.equal(got[0].reshape(45, -1), want)


def test_seeds_and_temperatures_share_the_captured_decode_steps():
    """Seed and temperature are read from device memory, so a new seed costs no new
    graph; the number of kept graphs is bounded."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    prompts = [random_tokens(n, cfg["vocab_size"], 80 + n) for n in (6, 11)]
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2)
    outs = {}
    for sd in range(6):
        outs[sd] = [c.tokens for c in lm.generate(prompts, 10, temperature=0.8 + 0.1 * sd, seed=sd,
                                                  ignore_eos=True)]
    assert len(lm.engine._graphs) == 1
    lm.engine.use_graphs = False
    for sd in (0, 5):
        again = [c.tokens for c in lm.generate(prompts, 10, temperature=0.8 + 0.1 * sd, seed=sd,
                                               ignore_eos=True)]
        assert again == outs[sd]
    assert lm.engine.MAX_GRAPHS >= 1


def test_pages_are_taken_as_sequences_grow_and_a_full_pool_refuses():
    """max_tokens = 256 gives four pages of 64 positions to four slots of 128: what fits
    is decided by the tokens held (each count rounded up to 64), not by slots x context;
    pages come back when a sequence ends and serve the next one."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    from yalm_b200.engine.step import StepError
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    V = cfg["vocab_size"]
    ta, tb, tc = (random_tokens(n, V, 300 + n) for n in (128, 60, 70))
    ra, rb, rc = (plain_forward(cfg, w, t) for t in (ta, tb, tc))
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=4, max_tokens=256)
    cache = lm.engine.cache
    assert cache.free_pages() == [4]
    sa, sb, sc = lm.acquire(3)
    lg = lm.step([ta[:100], tb[:60]], [sa, sb], [[99], [59]]).cpu()      # 2 + 1 pages
    assert cache.free_pages() == [1]
    assert float((lg[0] - ra[99]).abs().max() / ra.abs().max()) <= TOL["float32"]
    with pytest.raises(StepError, match="more pages"):
        lm.step([tc], [sc], [[69]])                                      # would need 2
    assert cache.free_pages() == [1] and cache.host_pos[sc] == 0         # nothing happened
    lm.release([sb])                                                     # b's page comes back
    assert cache.free_pages() == [2]
    lg = lm.step([tc, ta[100:128]], [sc, sa], [[69], [27]]).cpu()        # c takes both; a stays in its two
    assert cache.free_pages() == [0]
    assert float((lg[0] - rc[69]).abs().max() / rc.abs().max()) <= TOL["float32"]
    assert float((lg[1] - ra[127]).abs().max() / ra.abs().max()) <= TOL["float32"]
    lm.release([sa, sc])
    assert cache.free_pages() == [4]


def test_every_page_of_every_layer_counts():
    """Spoiling one page of one layer's keys moves the next token's logits: the compared
    logits depend on each page that the table names."""
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, seed = CONFIGS["tiny_a"]
    w = make_weights(cfg, seed)
    toks = random_tokens(101, cfg["vocab_size"], 17)
    ref = plain_forward(cfg, w, toks)
    for layer in range(cfg["num_hidden_layers"]):
        for which in (0, 1):
            lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2, max_tokens=192)
            lm.acquire(1)                                                # the request sits in the second slot
            (s,) = lm.acquire(1)
            lm.step([toks[:100]], [s], [[]])
            g = lm.engine.cache.groups[0]
            page = g["held"][s][which]
            g["k"][layer, :, page] += 0.5
            lg = lm.step([toks[100:]], [s], [[0]])[0].cpu()
            assert float((lg - ref[100]).abs().max() / ref.abs().max()) > 100 * TOL["float32"], (layer, which)
