"""Logits at real layer sizes, on the paths that serving runs.

The tiny configurations never reach the sizes at which the fast paths differ from
the simple ones: several K slices per product, the paired SiLU epilogue over
28,672 rows, the two-SM product over hundreds of tiles, the tensor-memory
attention over 32 heads, decode attention split into parts that a last block
merges, and kernels that overlap through programmatic dependent launch.  Here the
layers have the sizes of Mistral-7B (hidden 4096, FFN 14336, 32/8 heads of 128,
vocabulary 32000) and of Llama-3.2-1B (hidden 2048, FFN 8192, 32/8 heads of 64,
tied head of 128,256 rows, llama3 frequency scaling), with 2 layers instead of
their 32 and 16, and the plain implementation on the CPU is the reference.

Schedules: each request whole; the last 32 tokens one by one through the step
function; and a batch of unequal prompts decoded through ``Engine.decode_step``
(CUDA graphs and dependent launches on, the trace's own tokens forced after each
step, ``decode_logits`` read after each step) whose shorter requests end earlier.
The decode schedule also runs with dependent launch and graphs switched off and
must give the same bits: the kernels read positions and old cache rows before
their dependency wait, and a stale read would show here.
"""
import pytest
import torch

from helpers import DTYPES, TOL, make_weights, random_tokens
from plain_model import plain_forward
from trace_tools import Trace, add_tail, add_whole, compare, forced_decode, run_in_process

pytestmark = pytest.mark.gpu

MISTRAL_7B_2L = {
    "architectures": ["MistralForCausalLM"],
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 32000, "max_position_embeddings": 32768, "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0, "sliding_window": None, "tie_word_embeddings": False,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
LLAMA32_1B_2L = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "sliding_window": None, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 128000, "eos_token_id": 128001,
}
# request -> (prompt length, whole length): unequal prompts, unequal numbers of decode steps
CASES = {
    "mistral_7b": (MISTRAL_7B_2L, 11, {"r0": (150, 195), "r1": (260, 320), "r2": (330, 400)}),
    "llama_1b": (LLAMA32_1B_2L, 12, {"r0": (70, 118), "r1": (301, 345), "r2": (16, 80)}),
}
CONTEXT = 512

_cache = {}


def setup(name):
    if name not in _cache:
        cfg, seed, lens = CASES[name]
        w = make_weights(cfg, seed, std=0.02, jitter=0.1)
        reqs = {rid: random_tokens(n, cfg["vocab_size"], 500 + i)
                for i, (rid, (_, n)) in enumerate(lens.items())}
        refs = {rid: plain_forward(cfg, w, t) for rid, t in reqs.items()}
        _cache[name] = (cfg, w, reqs, refs, {rid: p for rid, (p, _) in lens.items()})
    return _cache[name]


def make_lm(cfg, w, dtype, max_batch, max_tokens=None):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    return LM(config_from_dict(cfg), dict(w), dtype=dtype, max_context=CONTEXT, max_batch=max_batch,
              max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mistral_7b", "llama_1b"])
def test_whole_and_last_32_one_by_one(name, dtype):
    cfg, w, reqs, refs, _ = setup(name)
    tr = Trace()
    add_whole(tr, reqs)
    add_tail(tr, reqs, tail=32)
    lm = make_lm(cfg, w, dtype, 1, max_tokens=448)           # seven pages of 64: a paged cache
    assert lm.engine.cache.free_pages() == [7]
    got = run_in_process(lm, tr)
    compare(tr, got, refs, cfg["vocab_size"], TOL[dtype])
    assert int(lm.rt.status.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mistral_7b", "llama_1b"])
def test_decode_path_with_graphs_and_dependent_launch(name, dtype):
    from yalm_b200.csrc import ops
    cfg, w, reqs, refs, prompts = setup(name)
    lm = make_lm(cfg, w, dtype, 3)
    fast = forced_decode(lm, reqs, prompts, refs, TOL[dtype])
    assert any(g is not None for g in lm.engine._graphs.values()), "no decode graph was captured"
    # the same steps, every kernel after the previous one has ended, launched one by one
    lm.engine.use_graphs = False
    ops.set_pdl(False)
    try:
        plain = forced_decode(lm, reqs, prompts, refs, TOL[dtype])
    finally:
        ops.set_pdl(True)
    assert torch.equal(fast, plain), "overlapping kernels changed a result"
    # longest row first, as the generation loop orders a batch
    lm.engine.use_graphs = True
    forced_decode(lm, reqs, prompts, refs, TOL[dtype],
                  order=sorted(reqs, key=lambda r: -prompts[r]))


@pytest.mark.parametrize("max_tokens", [None, 1024])
@pytest.mark.parametrize("dtype", [d for d in DTYPES if d != "float32"])
@pytest.mark.parametrize("name", ["mistral_7b", "llama_1b"])
def test_prompts_cut_into_two_steps(name, dtype, max_tokens):
    """A batch of three prompts whose second parts go on top of the cache in one step of many
    tokens each (what perplexity over a long text and a cut prefill do): the tensor-memory
    attention then reads every key from the cache (one block per sequence, or pages).  Cuts
    inside a tile, past one, and past a block of two tiles."""
    cfg, w, reqs, refs, _ = setup(name)
    lm = make_lm(cfg, w, dtype, 3, max_tokens=max_tokens)
    ids = list(reqs)
    cuts = {r: c if c < len(reqs[r]) - 1 else len(reqs[r]) // 2 for r, c in zip(ids, (100, 257, 130))}
    slots = lm.acquire(3)
    try:
        first = lm.step([reqs[r][:cuts[r]] for r in ids], slots, [list(range(cuts[r])) for r in ids])
        second = lm.step([reqs[r][cuts[r]:] for r in ids], slots,
                         [list(range(len(reqs[r]) - cuts[r])) for r in ids])
    finally:
        lm.release(slots)
    a = b = 0
    for r in ids:
        n, c = len(reqs[r]), cuts[r]
        scale = refs[r].abs().max()
        got = torch.cat([first[a:a + c], second[b:b + n - c]]).cpu()
        a, b = a + c, b + n - c
        err = ((got - refs[r]).abs().max() / scale).item()
        assert err <= TOL[dtype], (r, err)
    assert int(lm.rt.status.item()) == 0
