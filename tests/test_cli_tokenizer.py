"""Command-line parsing and the tokenizer (no GPU)."""
import json

import pytest

from yalm_b200.__main__ import parse
from yalm_b200.tokenizer import Tokenizer


def test_options_follow_the_reference_letters():
    o = parse(["dir", "-m", "perp", "-T", "512", "-i", "hello", "-t", "0.5", "-n", "7", "-l", "3"])
    assert (o["model"], o["mode"], o["context"], o["prompt"]) == ("dir", "perplexity", 512, "hello")
    assert (o["temperature"], o["n"], o["line"]) == (0.5, 7, 3)
    assert parse(["dir", "-m", "c", "--tokens", "1,2;3"])["mode"] == "completion"
    d = parse(["dir", "-i", "x"])
    assert d["temperature"] == 1.0 and d["n"] is None and d["device"] == "cuda"
    for bad in (["dir", "-m", "bogus", "-i", "x"], ["dir", "-i"], ["dir", "-q", "1"], [],
                ["dir", "-d", "cpu", "-i", "x"]):
        with pytest.raises(SystemExit):
            parse(bad)


def test_greedy_longest_match_with_byte_fallback(tmp_path):
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    for b in range(256):
        vocab[f"<0x{b:02X}>"] = 3 + b
    for i, p in enumerate(["▁the", "▁", "the", "t", "he", "▁cat", "cat", "s"]):
        vocab[p] = 259 + i
    (tmp_path / "tokenizer.json").write_text(json.dumps(
        {"model": {"vocab": vocab, "byte_fallback": True},
         "added_tokens": [{"id": 267, "content": "<|eot_id|>"}]}))
    tk = Tokenizer.from_dir(str(tmp_path), 300, 1, [2])
    assert tk.byte_start == 3 and tk.eot_id == 267 and tk.stop_ids == [2, 267]
    ids = tk.encode("the cats!", bos=True)
    assert ids == [1, 261, 264, 266, 3 + ord("!")]            # "the", " cat", "s", byte fallback
    assert tk.decode(ids[1:], prev=1) == "the cats!"
    assert tk.decode_one(1, 259) == b"the"                     # the space after BOS is stripped
    assert tk.decode_one(5, 259) == b" the"
    assert tk.encode("", bos=False) == []
    assert Tokenizer.from_dir(str(tmp_path / "none"), 10, 1, [2]) is None


def test_byte_level_vocabularies_are_mapped_back_to_bytes(tmp_path):
    vocab = {"Ġhello": 0, "hello": 1, "Ċ": 2, "!": 3}     # Ġ = space, Ċ = newline
    (tmp_path / "tokenizer.json").write_text(json.dumps({"model": {"vocab": vocab}, "added_tokens": []}))
    tk = Tokenizer.from_dir(str(tmp_path), 4, None, [])
    assert tk.pieces == [b" hello", b"hello", b"\n", b"!"]
    assert tk.encode("hello hello\n!", bos=True) == [1, 0, 2, 3]
