"""Typed configuration of the Llama / Mistral dense decoder, read from the
architecture's own ``config.json`` keys.

Key mapping and defaults follow the reference's packer (convert.py:22-56:
``head_dim`` defaults to ``hidden_size // num_attention_heads``,
``num_key_value_heads`` to ``num_attention_heads``, ``rope_theta`` to 10000.0,
biases must be off, ``hidden_act`` is checked).  Three keys the reference
drops are honoured here: ``rope_scaling`` (llama3 rule), ``sliding_window``
and ``tie_word_embeddings``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Any, Dict, List, Optional

from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


class ConfigError(ValueError):
    """A config.json that this library cannot serve; the message names the key."""


@dataclass(frozen=True)
class RopeScaling:
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        kind = d.get("rope_type", d.get("type", "default"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(
                f"rope_scaling.rope_type={kind!r} is not supported "
                f"(supported: 'default', 'llama3')")
        try:
            return RopeScaling(
                rope_type="llama3",
                factor=float(d["factor"]),
                low_freq_factor=float(d["low_freq_factor"]),
                high_freq_factor=float(d["high_freq_factor"]),
                original_max_position_embeddings=int(d["original_max_position_embeddings"]),
            )
        except KeyError as e:
            raise ConfigError(f"rope_scaling (llama3) lacks the key {e.args[0]!r}") from None


_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "vocab_size", "max_position_embeddings",
             "rms_norm_eps")


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    sliding_window: Optional[int] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    bos_token_id: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)
    torch_dtype: Optional[str] = None

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks the keys {missing}")
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        heads = int(d["num_attention_heads"])
        hidden = int(d["hidden_size"])
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"hidden_size={hidden} is not a multiple of "
                    f"num_attention_heads={heads} and head_dim is not given")
            head_dim = hidden // heads
        kv = d.get("num_key_value_heads")
        kv = heads if kv is None else int(kv)
        if d.get("attention_bias", False) or d.get("mlp_bias", False):
            raise ConfigError("attention_bias / mlp_bias are not supported")
        if float(d.get("partial_rotary_factor", 1.0)) != 1.0:
            raise ConfigError("partial_rotary_factor != 1 is not supported")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (only 'silu')")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: List[int] = []
        elif isinstance(eos, (list, tuple)):
            eos_ids = [int(t) for t in eos]
        else:
            eos_ids = [int(eos)]
        window = d.get("sliding_window")
        cfg = cls(
            architecture=str(archs[0]),
            hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=int(head_dim),
            vocab_size=int(d["vocab_size"]),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            sliding_window=None if window is None else int(window),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=act,
            bos_token_id=d.get("bos_token_id"),
            eos_token_ids=eos_ids,
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple "
                f"of num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary pairs")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"sliding_window must be positive, got {self.sliding_window}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    # ---- writing (random-weights mode writes a model folder) ------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else asdict(self.rope_scaling),
            "sliding_window": self.sliding_window,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.torch_dtype is not None:
            d["torch_dtype"] = self.torch_dtype
        return d

    def with_window(self, n: int) -> "LlamaConfig":
        """The same model with its attention bounded to the last ``n`` positions where
        the checkpoint sets no window (or a longer one): the role of the reference's
        ``-T n``, whose cache is a ring of n rows (model.cpp:28-32, infer.cu:1160-1165),
        here as a pure window without its two sink tokens."""
        n = int(n)
        if n <= 0:
            raise ConfigError(f"a window must be positive, got {n}")
        own = self.sliding_window
        return replace(self, sliding_window=n if own is None else min(own, n))

    def ignorable_tensor(self, name: str) -> bool:
        """Checkpoint tensors that this architecture does not read and that are no
        error: the rotary frequency buffers some exporters save, and a copy of the
        head when the embeddings are tied."""
        return name.endswith("rotary_emb.inv_freq") or (self.tie_word_embeddings
                                                        and name == "lm_head.weight")

    # ---- the architecture as a list of parts -----------------------------
    def to_spec(self) -> ModelSpec:
        """Tensor names are the checkpoint's own (the left column of the
        reference's rename table, convert.py:171-201)."""
        norm = lambda name: PartSpec(
            "rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps},
            {"weight": name})
        position = PartSpec("rope", {
            "head_dim": self.head_dim,
            "theta": self.rope_theta,
            "scaling": None if self.rope_scaling is None else asdict(self.rope_scaling),
        })
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "window": self.sliding_window,
                "position": position,
            }, {
                "q": f"{p}.self_attn.q_proj.weight",
                "k": f"{p}.self_attn.k_proj.weight",
                "v": f"{p}.self_attn.v_proj.weight",
                "o": f"{p}.self_attn.o_proj.weight",
            })
            ffn = PartSpec("swiglu", {
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
            }, {
                "gate": f"{p}.mlp.gate_proj.weight",
                "up": f"{p}.mlp.up_proj.weight",
                "down": f"{p}.mlp.down_proj.weight",
            })
            layers.append(LayerSpec("prenorm", {
                "mixer_norm": norm(f"{p}.input_layernorm.weight"), "mixer": mixer,
                "feed_forward_norm": norm(f"{p}.post_attention_layernorm.weight"),
                "feed_forward": ffn}))
        head_tensors = ({"weight": "model.embed_tokens.weight"} if self.tie_word_embeddings
                        else {"weight": "lm_head.weight"})
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding",
                               {"vocab_size": self.vocab_size, "size": self.hidden_size},
                               {"weight": "model.embed_tokens.weight"}),
            layers=layers,
            run_order=[RunEntry(i) for i in range(self.num_hidden_layers)],
            final_norm=norm("model.norm.weight"),
            head=PartSpec("linear_head",
                          {"vocab_size": self.vocab_size, "size": self.hidden_size,
                           "tied": self.tie_word_embeddings},
                          head_tensors),
            stop_token_ids=list(self.eos_token_ids),
            bos_token_id=self.bos_token_id,
        )
        spec.validate()
        return spec
