"""yalm_b200: a small inference library for the Llama / Mistral dense decoder
on one NVIDIA B200 (sm_100a): model folder in, logits or generated tokens out.

    from yalm_b200 import LM
    lm = LM.from_pretrained("model_dir", dtype="bfloat16")
    lm.generate([[1, 2, 3]], max_new_tokens=16, temperature=0.0)
"""

__all__ = ["LM", "Completion", "tensor_needs_of"]


def __getattr__(name):
    if name in ("LM", "tensor_needs_of"):
        from .engine import lm
        return getattr(lm, name)
    if name == "Completion":
        from .engine.generate import Completion
        return Completion
    raise AttributeError(name)
