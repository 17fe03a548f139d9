"""The generation loop's decisions, driven by a scripted backend (no GPU)."""
import pytest

from yalm_b200.engine.generate import plan_batches, run_generation


class Scripted:
    """Sequence i of a request continues with script[i][0], script[i][1], ..."""

    def __init__(self, scripts, max_batch=2, context=64):
        self.scripts = scripts
        self.max_batch = max_batch
        self.context = context
        self.log = []
        self.live = 0
        self.peak = 0

    def begin(self, prompts, keys):
        self.live += len(prompts)
        self.peak = max(self.peak, self.live)
        self.log.append(("begin", list(keys), [len(p) for p in prompts]))
        return {"keys": list(keys), "n": [0] * len(keys)}, [self._next(k, 0) for k in keys]

    def _next(self, key, i):
        s = self.scripts[key]
        return s[i] if i < len(s) else 999

    def decode(self, handle, active, tokens):
        self.log.append(("decode", list(active), list(tokens)))
        out = []
        for j in active:
            handle["n"][j] += 1
            out.append(self._next(handle["keys"][j], handle["n"][j]))
        return out

    def end(self, handle):
        self.live -= len(handle["keys"])
        self.log.append(("end", handle["keys"]))


def test_batches_follow_request_order():
    assert plan_batches(5, 2) == [[0, 1], [2, 3], [4]]
    assert plan_batches(0, 4) == []
    with pytest.raises(ValueError):
        plan_batches(3, 0)


def test_stop_tokens_end_a_sequence_and_are_part_of_the_output():
    b = Scripted({0: [5, 6, 2, 7], 1: [2], 2: [8, 8, 8, 8, 8]}, max_batch=2)
    out = run_generation(b, [[1, 4], [1], [1, 1, 1]], max_new_tokens=4, stop_ids=[2])
    assert out[0].tokens == [5, 6, 2] and out[0].finish_reason == "stop"
    assert out[1].tokens == [2] and out[1].finish_reason == "stop"
    assert out[2].tokens == [8, 8, 8, 8] and out[2].finish_reason == "length"
    # the shorter request left the batch: later steps carry only the survivor
    decodes = [e for e in b.log if e[0] == "decode"]
    assert decodes[0] == ("decode", [0], [5]) and decodes[1] == ("decode", [0], [6])
    # the second batch starts only after the first gave its slots back
    kinds = [e[0] for e in b.log]
    assert kinds.index("end") < len(kinds) - 1 - kinds[::-1].index("begin")
    assert b.peak == 2 and b.live == 0


def test_the_stop_token_is_never_forwarded():
    b = Scripted({0: [2]})
    run_generation(b, [[3, 3]], max_new_tokens=8, stop_ids=[2])
    assert not [e for e in b.log if e[0] == "decode"]


def test_length_and_context_limits():
    b = Scripted({0: list(range(10, 40))}, context=8)
    out = run_generation(b, [[1, 1, 1, 1, 1]], max_new_tokens=-1)
    # 5 prompt positions; tokens 1..3 can still be forwarded (positions 5,6,7), the 4th cannot
    assert out[0].finish_reason == "context" and len(out[0].tokens) == 4
    out = run_generation(Scripted({0: [9] * 5}), [[1]], max_new_tokens=0)
    assert out[0].tokens == [] and out[0].finish_reason == "length"
    with pytest.raises(ValueError, match="empty"):
        run_generation(Scripted({0: []}), [[]], 1)
    with pytest.raises(ValueError, match="context"):
        run_generation(Scripted({0: []}, context=2), [[1, 2, 3]], 1)


def test_slots_are_given_back_when_the_backend_fails():
    class Failing(Scripted):
        def decode(self, handle, active, tokens):
            raise RuntimeError("boom")
    b = Failing({0: [5, 5]})
    with pytest.raises(RuntimeError, match="boom"):
        run_generation(b, [[1]], 4)
    assert b.live == 0


def test_on_token_sees_every_token_with_its_request():
    seen = []
    b = Scripted({0: [5, 2], 1: [6, 7, 2], 2: [2]}, max_batch=2)
    run_generation(b, [[1], [1], [1]], 8, stop_ids=[2], on_token=lambda i, t: seen.append((i, t)))
    assert sorted(seen) == [(0, 2), (0, 5), (1, 2), (1, 6), (1, 7), (2, 2)]
