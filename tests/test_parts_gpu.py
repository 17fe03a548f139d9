"""Each part alone against its plain function, and a toy mixer with state of
its own that is registered, built and stepped without touching the library."""
import dataclasses

import pytest
import torch

from helpers import TINY_A, TINY_C, make_weights, random_tokens
from plain_model import (plain_attention, plain_block, plain_embedding, plain_forward,
                         plain_inv_freq, plain_rmsnorm, plain_rope, plain_swiglu)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# bounds of the 16-bit checks are stated for bfloat16; float16 keeps three more bits
SCALE = {torch.bfloat16: 1.0, torch.float16: 0.125}


def _rt(dtype):
    from yalm_b200.parts import Runtime
    return Runtime(dtype, DEV)


def _prefill_batch(n):
    from yalm_b200.engine.batch import build_batch
    return build_batch([[0] * n], [0], [0], [[]], DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_norm_part(dtype):
    from yalm_b200.parts import NORMS, ResidualStream
    rt = _rt(dtype)
    norm = NORMS["rmsnorm"]({"size": 200, "eps": 1e-4}, rt)
    assert norm.tensor_needs()["weight"].shape == (200,)
    w = torch.randn(200)
    norm.bind({"weight": w})
    x = torch.randn(9, 200, device=DEV)
    h = norm(ResidualStream(rt, x.clone()))
    ref = plain_rmsnorm(x.cpu(), w, 1e-4)
    tol = 2e-6 if dtype == torch.float32 else 2 ** -8 * SCALE[dtype]
    assert h.dtype == dtype and (h.float().cpu() - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_feed_forward_part(dtype):
    from yalm_b200.parts import FEED_FORWARDS, ResidualStream
    rt = _rt(dtype)
    ffn = FEED_FORWARDS["swiglu"]({"hidden_size": 88, "intermediate_size": 200}, rt)
    w = {k: (0.1 * torch.randn(s)).to(torch.bfloat16)
         for k, s in (("gate", (200, 88)), ("up", (200, 88)), ("down", (88, 200)))}
    ffn.bind(w)
    for n in (3, 150):                                          # few tokens (split K) and many
        h = torch.randn(n, 88).to(dtype)
        stream = ResidualStream(rt, torch.ones(n, 88, device=DEV))
        ffn.forward(h.to(DEV), _prefill_batch(n), stream)
        got = stream.resolve().cpu()
        ref = 1.0 + plain_swiglu(h.float(), w["gate"], w["up"], w["down"])
        tol = 1e-5 if dtype == torch.float32 else 1e-2 * SCALE[dtype]
        assert (got - ref).abs().max() <= tol * ref.abs().max(), n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_with_its_position_encoding(dtype, window):
    from yalm_b200.cache import Cache
    from yalm_b200.config import PartSpec
    from yalm_b200.parts import MIXERS, ResidualStream
    rt = _rt(dtype)
    D, H, G, hd, T = 88, 6, 2, 48, 70
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
               "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    mixer = MIXERS["gqa_attention"]({
        "hidden_size": D, "num_heads": H, "num_kv_heads": G, "head_dim": hd, "window": window,
        "position": PartSpec("rope", {"head_dim": hd, "theta": 5000.0, "scaling": scaling})}, rt)
    w = {k: (0.1 * torch.randn(s)).to(torch.bfloat16)
         for k, s in (("q", (H * hd, D)), ("k", (G * hd, D)), ("v", (G * hd, D)), ("o", (D, H * hd)))}
    mixer.bind(w)
    need = mixer.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("kv", G, hd, window)
    cache = Cache({0: need}, n_slots=1, context=96, dtype=dtype, device=DEV)
    cache.acquire(1)
    cache.ensure([0], [T])
    cache.sync_tables()
    h = torch.randn(T, D).to(dtype)
    stream = ResidualStream(rt, torch.zeros(T, D, device=DEV))
    mixer.forward(h.to(DEV), _prefill_batch(T), stream, cache.view(0))
    got = stream.resolve().cpu()
    hf = h.float()
    inv = plain_inv_freq(hd, 5000.0, scaling)
    pos = torch.arange(T)
    q = plain_rope((hf @ w["q"].float().T).view(T, H, hd), pos, inv)
    k = plain_rope((hf @ w["k"].float().T).view(T, G, hd), pos, inv)
    v = (hf @ w["v"].float().T).view(T, G, hd)
    ref = plain_attention(q, k, v, window).reshape(T, H * hd) @ w["o"].float().T
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2 * SCALE[dtype]
    assert (got - ref).abs().max() <= tol * ref.abs().max()
    # the ring holds the last `capacity` rotated keys at row pos % capacity
    cap = cache.view(0).capacity
    p = T - 1
    assert (cache.rows(0, 0)[0][1, p % cap].float().cpu() - k[p, 1]).abs().max() <= (
        1e-5 if dtype == torch.float32 else 2e-2 * SCALE[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_block_embedding_and_head(dtype):
    from yalm_b200.cache import Cache
    from yalm_b200.config import config_from_dict
    from yalm_b200.parts import BLOCKS, EMBEDDINGS, HEADS, ResidualStream
    rt = _rt(dtype)
    cfg = TINY_C
    spec = config_from_dict(cfg).to_spec()
    w = make_weights(cfg, 3)
    toks = random_tokens(50, cfg["vocab_size"], 1)
    emb = EMBEDDINGS["embedding"](spec.embedding.params, rt)
    emb.bind({"weight": w["model.embed_tokens.weight"]})
    from yalm_b200.engine.batch import build_batch
    batch = build_batch([toks], [0], [0], [[]], DEV)
    x = emb.forward(batch)
    assert torch.equal(x.cpu(), plain_embedding(w["model.embed_tokens.weight"], toks))
    block = BLOCKS["prenorm"](spec.layers[1], rt)
    for part, pspec in block.parts():
        part.bind({k: w[pspec.tensors[k]] for k in part.tensor_needs()})
    cache = Cache({0: block.mixer.cache_need()}, 1, 160, dtype, DEV)
    cache.acquire(1)
    cache.ensure([0], [50])
    cache.sync_tables()
    stream = ResidualStream(rt, x)
    block.forward(stream, batch, {"mixer": cache.view(0)})
    ref = plain_block(plain_embedding(w["model.embed_tokens.weight"], toks), cfg, w, 1,
                      torch.arange(50))
    tol = 1e-5 if dtype == torch.float32 else 1e-2 * SCALE[dtype]
    got = stream.resolve().cpu()
    assert (got - ref).abs().max() <= tol * ref.abs().max()
    head = HEADS["linear_head"](spec.head.params, rt)
    head.bind({"weight": w["lm_head.weight"]})
    hh = torch.randn(5, cfg["hidden_size"]).to(dtype)
    out = head.forward(hh.to(DEV), torch.empty(5, cfg["vocab_size"], device=DEV))
    ref = hh.float() @ w["lm_head.weight"].float().T
    assert (out.cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-5) * ref.abs().max()


def test_a_matrix_stored_in_32_bits_stays_32_bit_under_bfloat16():
    from yalm_b200.parts import HEADS
    rt = _rt(torch.bfloat16)
    head = HEADS["linear_head"]({"vocab_size": 300, "size": 88}, rt)
    w = torch.randn(300, 88) * (1 + 2 ** -12)                   # not representable in bfloat16
    head.bind({"weight": w})
    assert head.weight.dtype == torch.float32
    h = torch.randn(4, 88).to(torch.bfloat16)
    out = head.forward(h.to(DEV), torch.empty(4, 300, device=DEV))
    ref = h.double() @ w.double().T
    assert (out.double().cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()


# ---------------------------------------------------------------------------
# A toy mixer with state of its own, defined here: s <- decay * s + h_t per
# sequence, output W s.  It is registered, built into a model next to an
# attention layer, and stepped, without a change to the library's files.

def _register_toy():
    from yalm_b200.cache import CacheNeed
    from yalm_b200.config import LlamaConfig, PartSpec, register_architecture
    from yalm_b200.parts import MIXERS, register_mixer
    from yalm_b200.weights import TensorNeed
    if "toy_decay" in MIXERS:
        return

    @register_mixer("toy_decay")
    class ToyDecay:
        def __init__(self, params, rt):
            self.rt, self.D, self.decay = rt, int(params["size"]), float(params["decay"])

        def tensor_needs(self):
            return {"w": TensorNeed((self.D, self.D))}

        def bind(self, tensors):
            self.w = tensors["w"].to(self.rt.device, torch.float32)

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.D,), state_dtype=torch.float32)

        def forward(self, h, batch, stream, view, shared=False):
            out = torch.empty(batch.n_tokens, self.D, device=self.rt.device)
            t = 0
            for slot, n in zip(batch.slots, batch.q_lens):
                s = view.state[slot]
                for i in range(n):
                    s = self.decay * s + h[t].float()
                    out[t] = self.w @ s
                    t += 1
                view.state[slot] = s
            stream.add_tensor(out)

    class ToyConfig(LlamaConfig):
        def to_spec(self):
            spec = super().to_spec()
            toy = PartSpec("toy_decay", {"size": self.hidden_size, "decay": 0.5},
                           {"w": "model.layers.0.toy.weight"})
            layers = [spec.layers[0].with_parts(mixer=toy)] + spec.layers[1:]
            return dataclasses.replace(spec, layers=layers)

    register_architecture("ToyForCausalLM", ToyConfig)


def _plain_toy_forward(cfg, w, toks):
    T = len(toks)
    x = plain_embedding(w["model.embed_tokens.weight"], toks)
    h = plain_rmsnorm(x, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    s = torch.zeros(cfg["hidden_size"])
    y = torch.zeros_like(x)
    for t in range(T):
        s = 0.5 * s + h[t]
        y[t] = w["model.layers.0.toy.weight"].float() @ s
    x = x + y
    h = plain_rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + plain_swiglu(h, w["model.layers.0.mlp.gate_proj.weight"],
                         w["model.layers.0.mlp.up_proj.weight"], w["model.layers.0.mlp.down_proj.weight"])
    x = plain_block(x, cfg, w, 1, torch.arange(T))
    x = plain_rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return x @ w["lm_head.weight"].float().T


def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    _register_toy()
    cfg = dict(TINY_A, architectures=["ToyForCausalLM"])
    w = make_weights(cfg, 4)
    for k in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.0.self_attn.{k}.weight"]
    w["model.layers.0.toy.weight"] = (0.05 * torch.randn(64, 64)).to(torch.bfloat16)
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2)
    kinds = sorted(g["need"].kind for g in lm.engine.cache.groups)
    assert kinds == ["kv", "state"]                             # two groups, storage of their own
    ta, tb = random_tokens(30, 256, 1), random_tokens(12, 256, 2)
    ra, rb = _plain_toy_forward(cfg, w, ta), _plain_toy_forward(cfg, w, tb)
    sa, sb = lm.acquire(2)
    lg = lm.step([ta[:20], tb[:5]], [sa, sb], [[19], [4]])
    assert (lg[0].cpu() - ra[19]).abs().max() <= 1e-5 * ra.abs().max()
    assert (lg[1].cpu() - rb[4]).abs().max() <= 1e-5 * rb.abs().max()
    for p in range(5, 12):                                      # token by token, state carried
        lg = lm.step([[ta[15 + p]], [tb[p]]], [sa, sb], [[0], [0]])
        assert (lg[0].cpu() - ra[15 + p]).abs().max() <= 1e-5 * ra.abs().max()
        assert (lg[1].cpu() - rb[p]).abs().max() <= 1e-5 * rb.abs().max()
    lm.release([sa, sb])
    (sc,) = lm.acquire(1)                                       # a used slot: its state starts at zero
    lg = lm.step([tb], [sc], [[11]])
    assert (lg[0].cpu() - rb[11]).abs().max() <= 1e-5 * rb.abs().max()


def test_a_layer_named_twice_and_a_layer_reading_anothers_cache():
    """run_order [0, 1, 0]: layer 0 runs twice with a cache per run; then
    [0, 1, 1<-reads 1]: the third run reuses the second run's keys and values."""
    from yalm_b200.cache import Cache
    from yalm_b200.config import RunEntry, config_from_dict
    from yalm_b200.engine.step import Engine
    from yalm_b200.parts import Model, Runtime
    cfg = TINY_A
    w = make_weights(cfg, 0)
    toks = random_tokens(40, 256, 3)
    spec = config_from_dict(cfg).to_spec()
    rt = Runtime(torch.float32, DEV)
    m = Model(dataclasses.replace(spec, run_order=[RunEntry(0), RunEntry(1), RunEntry(0)]), rt)
    m.bind(dict(w))
    assert sorted(k[0] for k in m.cache_needs()) == [0, 1, 2]
    eng = Engine(m, 1, 128)
    s = eng.acquire(1)
    ref = plain_forward(cfg, w, toks, run_order=[0, 1, 0])
    lg = eng.step([toks[:25]], s, [[24]])
    assert (lg[0].cpu() - ref[24]).abs().max() <= 1e-5 * ref.abs().max()
    for p in range(25, 40):
        lg = eng.step([[toks[p]]], s, [[0]])
        assert (lg[0].cpu() - ref[p]).abs().max() <= 1e-5 * ref.abs().max(), p
    # sharing: the reader's keys/values are the owner's, so its own k/v projections are unused
    m2 = Model(dataclasses.replace(spec, run_order=[RunEntry(0), RunEntry(1), RunEntry(1, 1)]), rt)
    m2.bind(dict(w))
    assert sorted(k[0] for k in m2.cache_needs()) == [0, 1]
    eng2 = Engine(m2, 1, 128)
    s = eng2.acquire(1)
    whole = eng2.step([toks], s, [list(range(40))]).cpu()
    eng2.release(s)
    s = eng2.acquire(1)
    cut = eng2.step([toks[:30]], s, [[29]]).cpu()
    assert (cut[0] - whole[29]).abs().max() <= 1e-5 * whole.abs().max()
    for p in range(30, 40):
        lg = eng2.step([[toks[p]]], s, [[0]]).cpu()
        assert (lg[0] - whole[p]).abs().max() <= 1e-5 * whole.abs().max(), p
    assert (whole - plain_forward(cfg, w, toks, run_order=[0, 1, 1])).abs().max() > 1e-3


# ---------------------------------------------------------------------------
# Two more toy parts, again defined here only: a position encoding that does not
# rotate at all, and a feed-forward that routes each token to one of two experts
# (router logits in 32 bits).  They sit in layer 0 of a model whose layer 1 is the
# stock attention + SwiGLU.

def _register_toy_position_and_routing():
    from yalm_b200.config import LlamaConfig, PartSpec, register_architecture
    from yalm_b200.csrc import ops
    from yalm_b200.parts import FEED_FORWARDS, register_feed_forward, register_position
    from yalm_b200.weights import TensorNeed
    if "toy_top1" in FEED_FORWARDS:
        return

    @register_position("no_position")
    class NoPosition:
        """Keys and queries as they are: the rotary kernel with every frequency zero
        (it still converts, and writes the cache)."""

        def __init__(self, params, rt):
            self.hd = int(params["head_dim"])
            self.zero = torch.zeros(self.hd // 2, device=rt.device)

        def rotate_and_store(self, qkv, n_partials, batch, view, q_out, kv_step, H, G,
                             write_cache=True):
            ops.rope_store(qkv, n_partials, self.zero, batch, q_out, kv_step, view.k, view.v,
                           view.slot_pos, H, G, self.hd, view.capacity, write_cache, pages=view.pages)

    @register_feed_forward("toy_top1")
    class ToyTop1:
        def __init__(self, params, rt):
            self.rt, self.D, self.F, self.E = rt, params["size"], params["ffn"], params["experts"]

        def tensor_needs(self):
            n = {"router": TensorNeed((self.E, self.D))}
            for e in range(self.E):
                n[f"gate{e}"] = TensorNeed((self.F, self.D))
                n[f"up{e}"] = TensorNeed((self.F, self.D))
                n[f"down{e}"] = TensorNeed((self.D, self.F))
            return n

        def bind(self, tensors):
            self.w = {k: v.to(self.rt.device, torch.float32) for k, v in tensors.items()}

        def forward(self, h, batch, stream):
            hf = h.float()
            choice = (hf @ self.w["router"].T).argmax(-1)          # router logits in 32 bits
            out = torch.zeros_like(hf)
            for e in range(self.E):
                rows = (choice == e).nonzero()[:, 0]
                if rows.numel():
                    x = hf[rows]
                    g, u = x @ self.w[f"gate{e}"].T, x @ self.w[f"up{e}"].T
                    out[rows] = (torch.nn.functional.silu(g) * u) @ self.w[f"down{e}"].T
            stream.add_tensor(out)

    class ToyRoutedConfig(LlamaConfig):
        def to_spec(self):
            spec = super().to_spec()
            l0 = spec.layers[0]
            mixer = dataclasses.replace(l0.part("mixer"), params=dict(
                l0.part("mixer").params, position=PartSpec("no_position", {"head_dim": self.head_dim})))
            names = {"router": "model.layers.0.moe.router.weight"}
            for e in range(2):
                for k in ("gate", "up", "down"):
                    names[f"{k}{e}"] = f"model.layers.0.moe.experts.{e}.{k}.weight"
            ffn = PartSpec("toy_top1", {"size": self.hidden_size, "ffn": 40, "experts": 2}, names)
            return dataclasses.replace(spec, layers=[l0.with_parts(mixer=mixer, feed_forward=ffn)]
                                       + spec.layers[1:])

    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)


def test_toy_position_encoding_and_routed_feed_forward():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    _register_toy_position_and_routing()
    cfg = dict(TINY_A, architectures=["ToyRoutedForCausalLM"])
    w = make_weights(cfg, 6)
    for k in ("gate_proj", "up_proj", "down_proj"):
        del w[f"model.layers.0.mlp.{k}.weight"]
    g = torch.Generator().manual_seed(9)
    w["model.layers.0.moe.router.weight"] = torch.randn(2, 64, generator=g).to(torch.bfloat16)
    for e in range(2):
        w[f"model.layers.0.moe.experts.{e}.gate.weight"] = (0.1 * torch.randn(40, 64, generator=g)).to(torch.bfloat16)
        w[f"model.layers.0.moe.experts.{e}.up.weight"] = (0.1 * torch.randn(40, 64, generator=g)).to(torch.bfloat16)
        w[f"model.layers.0.moe.experts.{e}.down.weight"] = (0.1 * torch.randn(64, 40, generator=g)).to(torch.bfloat16)

    def plain(toks):
        T = len(toks)
        H, G, hd, eps = 4, 2, 16, cfg["rms_norm_eps"]
        x = plain_embedding(w["model.embed_tokens.weight"], toks)
        h = plain_rmsnorm(x, w["model.layers.0.input_layernorm.weight"], eps)
        q = (h @ w["model.layers.0.self_attn.q_proj.weight"].float().T).view(T, H, hd)
        k = (h @ w["model.layers.0.self_attn.k_proj.weight"].float().T).view(T, G, hd)
        v = (h @ w["model.layers.0.self_attn.v_proj.weight"].float().T).view(T, G, hd)
        a = plain_attention(q, k, v, None).reshape(T, H * hd)          # no rotation
        x = x + a @ w["model.layers.0.self_attn.o_proj.weight"].float().T
        h = plain_rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], eps)
        choice = (h @ w["model.layers.0.moe.router.weight"].float().T).argmax(-1)
        y = torch.zeros_like(x)
        for t in range(T):
            e = int(choice[t])
            y[t] = plain_swiglu(h[t:t + 1], w[f"model.layers.0.moe.experts.{e}.gate.weight"],
                                w[f"model.layers.0.moe.experts.{e}.up.weight"],
                                w[f"model.layers.0.moe.experts.{e}.down.weight"])[0]
        x = plain_block(x + y, cfg, w, 1, torch.arange(T))
        x = plain_rmsnorm(x, w["model.norm.weight"], eps)
        return x @ w["lm_head.weight"].float().T, choice

    toks = random_tokens(50, 256, 12)
    ref, choice = plain(toks)
    assert 5 < int(choice.sum()) < 45                               # both experts are used
    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=1)
    s = lm.acquire(1)
    lg = lm.step([toks[:35]], s, [list(range(35))]).cpu()
    assert (lg - ref[:35]).abs().max() <= 1e-5 * ref.abs().max()
    for p in range(35, 50):
        lg = lm.step([[toks[p]]], s, [[0]]).cpu()
        assert (lg[0] - ref[p]).abs().max() <= 1e-5 * ref.abs().max(), p


# ---------------------------------------------------------------------------
# Two more arrangements that only this file defines: a block with four norms (one
# before and one after each of mixer and feed-forward), and a mixer that asks the cache
# for keys/values AND a state of its own (attention plus a decaying sum).

def _register_sandwich_and_kv_state():
    from yalm_b200.cache import CacheNeed
    from yalm_b200.config import LayerSpec, LlamaConfig, PartSpec, register_architecture
    from yalm_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, ResidualStream, make_part,
                                 register_block, register_mixer)
    from yalm_b200.weights import TensorNeed
    if "sandwich" in BLOCKS:
        return

    @register_block("sandwich")
    class SandwichBlock:
        NAMES = ("pre_mixer_norm", "mixer", "post_mixer_norm", "pre_ffn_norm", "feed_forward",
                 "post_ffn_norm")

        def __init__(self, layer_spec, rt):
            self.rt, self.spec = rt, layer_spec
            table = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS}
            self.p = {n: make_part(table.get(n, NORMS), layer_spec.part(n), rt) for n in self.NAMES}

        def parts(self):
            return [(self.p[n], self.spec.part(n)) for n in self.NAMES]

        def mixers(self):
            return {"mixer": self.p["mixer"]}

        def _branch(self, stream, pre, run, post):
            h = self.p[pre](stream)
            side = ResidualStream(self.rt, torch.zeros_like(stream.x))
            later = run(h, side)
            side.resolve()
            stream.add_tensor(self.p[post](side, name=post))
            return later

        def forward(self, stream, batch, views, shared=False):
            later = self._branch(stream, "pre_mixer_norm",
                                 lambda h, side: self.p["mixer"].forward(h, batch, side, views["mixer"], shared=shared),
                                 "post_mixer_norm")
            self._branch(stream, "pre_ffn_norm",
                         lambda h, side: self.p["feed_forward"].forward(h, batch, side), "post_ffn_norm")
            return later

    @register_mixer("toy_kv_state")
    class AttentionPlusDecay:
        def __init__(self, params, rt):
            self.rt, self.D = rt, int(params["hidden_size"])
            self.attn = MIXERS["gqa_attention"](params, rt)

        def tensor_needs(self):
            return dict(self.attn.tensor_needs(), s=TensorNeed((self.D, self.D)))

        def bind(self, tensors):
            self.attn.bind({k: v for k, v in tensors.items() if k != "s"})
            self.ws = tensors["s"].to(self.rt.device, torch.float32)

        def cache_need(self):
            return {"kv": self.attn.cache_need(),
                    "state": CacheNeed("state", state_shape=(self.D,), state_dtype=torch.float32)}

        def forward(self, h, batch, stream, view, shared=False):
            later = self.attn.forward(h, batch, stream, view["kv"], shared=shared)
            out = torch.empty(batch.n_tokens, self.D, device=self.rt.device)
            t = 0
            for slot, n in zip(batch.slots, batch.q_lens):
                s = view["state"].state[slot]
                for _ in range(n):
                    s = 0.5 * s + h[t].float()
                    out[t] = self.ws @ s
                    t += 1
                view["state"].state[slot] = s
            stream.add_tensor(out)
            return later

    class SandwichConfig(LlamaConfig):
        def to_spec(self):
            spec = super().to_spec()
            norm = lambda n: PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps},
                                      {"weight": n})
            l0 = spec.layers[0]
            mixer = dataclasses.replace(l0.part("mixer"), kind="toy_kv_state",
                                        tensors=dict(l0.part("mixer").tensors, s="model.layers.0.decay.weight"))
            layer0 = LayerSpec("sandwich", {
                "pre_mixer_norm": l0.part("mixer_norm"), "mixer": mixer,
                "post_mixer_norm": norm("model.layers.0.post_mixer_norm.weight"),
                "pre_ffn_norm": l0.part("feed_forward_norm"), "feed_forward": l0.part("feed_forward"),
                "post_ffn_norm": norm("model.layers.0.post_ffn_norm.weight")})
            return dataclasses.replace(spec, layers=[layer0] + spec.layers[1:])

    register_architecture("SandwichForCausalLM", SandwichConfig)


def test_a_block_with_four_norms_and_a_mixer_with_keys_values_and_a_state():
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    _register_sandwich_and_kv_state()
    cfg = dict(TINY_C, architectures=["SandwichForCausalLM"])       # window 40: the kv part is a ring
    D, H, G, hd, eps = cfg["hidden_size"], 6, 2, 48, cfg["rms_norm_eps"]
    w = make_weights(cfg, 8)
    g = torch.Generator().manual_seed(3)
    w["model.layers.0.decay.weight"] = (0.05 * torch.randn(D, D, generator=g)).to(torch.bfloat16)
    w["model.layers.0.post_mixer_norm.weight"] = 1.0 + 0.1 * torch.randn(D, generator=g)
    w["model.layers.0.post_ffn_norm.weight"] = 1.0 + 0.1 * torch.randn(D, generator=g)

    def plain(toks):
        T = len(toks)
        p = "model.layers.0"
        x = plain_embedding(w["model.embed_tokens.weight"], toks)
        h = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps)
        inv = plain_inv_freq(hd, cfg["rope_theta"], None)
        pos = torch.arange(T)
        q = plain_rope((h @ w[f"{p}.self_attn.q_proj.weight"].float().T).view(T, H, hd), pos, inv)
        k = plain_rope((h @ w[f"{p}.self_attn.k_proj.weight"].float().T).view(T, G, hd), pos, inv)
        v = (h @ w[f"{p}.self_attn.v_proj.weight"].float().T).view(T, G, hd)
        y = plain_attention(q, k, v, cfg["sliding_window"]).reshape(T, H * hd) @ \
            w[f"{p}.self_attn.o_proj.weight"].float().T
        s = torch.zeros(D)
        for t in range(T):
            s = 0.5 * s + h[t]
            y[t] += w[f"{p}.decay.weight"].float() @ s
        x = x + plain_rmsnorm(y, w[f"{p}.post_mixer_norm.weight"], eps)
        h = plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
        y = plain_swiglu(h, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                         w[f"{p}.mlp.down_proj.weight"])
        x = x + plain_rmsnorm(y, w[f"{p}.post_ffn_norm.weight"], eps)
        x = plain_block(x, cfg, w, 1, pos)
        return plain_rmsnorm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].float().T

    lm = LM(config_from_dict(cfg), dict(w), dtype="float32", max_batch=2)
    kinds = sorted(g_["need"].kind for g_ in lm.engine.cache.groups)
    assert kinds == ["kv", "state"]
    assert sorted(k[2] for k in lm.model.cache_needs() if k[0] == 0) == ["kv", "state"]
    ta, tb = random_tokens(90, cfg["vocab_size"], 1), random_tokens(33, cfg["vocab_size"], 2)
    ra, rb = plain(ta), plain(tb)
    sa, sb = lm.acquire(2)
    lg = lm.step([ta[:60], tb[:20]], [sa, sb], [[59], [19]]).cpu()
    assert (lg[0] - ra[59]).abs().max() <= 1e-5 * ra.abs().max()
    assert (lg[1] - rb[19]).abs().max() <= 1e-5 * rb.abs().max()
    for p in range(20, 33):                                     # past the ring of 40 for request a
        lg = lm.step([[ta[40 + p]], [tb[p]]], [sa, sb], [[0], [0]]).cpu()
        assert (lg[0] - ra[40 + p]).abs().max() <= 1e-5 * ra.abs().max(), p
        assert (lg[1] - rb[p]).abs().max() <= 1e-5 * rb.abs().max(), p
    lm.release([sa, sb])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_reader_of_a_windowed_cache_sees_the_old_rows_when_a_prompt_is_cut(dtype):
    """Run order [0, 1, 2, 2<-2] on a ring of 32 rows: the last entry reads entry 2's
    keys and values.  A prompt given as 30 + 25 + 1 tokens makes the second portion land
    on a full ring; the owner's ring write must wait until the reader has run, or the
    reader's first tokens would find their oldest keys replaced.  Whole and cut agree."""
    from yalm_b200.config import RunEntry, config_from_dict
    from yalm_b200.engine.step import Engine
    from yalm_b200.parts import Model, Runtime
    from helpers import TINY_B, TOL
    cfg = dict(TINY_B, tie_word_embeddings=False)
    w = make_weights(cfg, 21)
    toks = random_tokens(56, cfg["vocab_size"], 4)
    spec = config_from_dict(cfg).to_spec()
    rt = Runtime({"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], DEV)
    m = Model(dataclasses.replace(spec, run_order=[RunEntry(0), RunEntry(1), RunEntry(2),
                                                   RunEntry(2, 2)]), rt)
    m.bind(dict(w))
    eng = Engine(m, 1, 96)
    s = eng.acquire(1)
    whole = eng.step([toks], s, [list(range(56))]).cpu()
    eng.release(s)
    s = eng.acquire(1)
    cut = torch.cat([eng.step([toks[a:b]], s, [list(range(b - a))]).cpu()
                     for a, b in ((0, 30), (30, 55), (55, 56))])
    tol = 2e-5 if dtype == "float32" else TOL[dtype]
    assert float((cut - whole).abs().max() / whole.abs().max()) <= tol
    rt.check_status()
