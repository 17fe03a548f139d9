"""The byte and flop counts that bench.py divides by time, against the figures worked out
by hand for the Mistral-7B-v0.2 shapes: 14.22 GB of weights per decode step plus 128 KiB
per cached position, 29.7 TFLOP for a 2,048-token prompt."""
import os
import sys
from types import SimpleNamespace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
from yalm_b200.config import config_from_dict  # noqa: E402


def _model_without_device(cfg_dict):
    import torch
    from yalm_b200.parts import Model, Runtime
    cfg = config_from_dict(dict(cfg_dict))
    return cfg, SimpleNamespace(config=cfg, model=Model(cfg.to_spec(), Runtime.shapes_only(torch.float16)))


def test_decode_bytes_and_prefill_flops():
    cfg, lm = _model_without_device(bench.MISTRAL_7B)
    weights_only = bench.decode_bytes(lm, [])
    assert abs(weights_only - 14.22e9) / 14.22e9 < 0.01
    per_position = bench.decode_bytes(lm, [1]) - weights_only - cfg.hidden_size * 2
    assert per_position == 128 * 1024
    b64 = bench.decode_bytes(lm, [1056] * 64)
    assert abs(b64 - 23.08e9) / 23.08e9 < 0.01
    assert abs(bench.prefill_flops(lm, 2048) - 29.7e12) / 29.7e12 < 0.01
    # under a window only the ring is read
    _, v01 = _model_without_device(bench.WORKLOADS["mistral-7b-v0.1"][0])
    assert bench.decode_bytes(v01, [6000]) == bench.decode_bytes(v01, [4096])
    # a tied head: the table is read whole once, as the head
    _, l1b = _model_without_device(bench.LLAMA32_1B)
    assert abs(bench.decode_bytes(l1b, []) - 2.47e9) / 2.47e9 < 0.01


def test_more_than_one_gpu_is_refused(capsys):
    sys.argv = ["bench.py", "--gpus", "2"]
    assert bench.main() == 2
    assert "one GPU" in capsys.readouterr().out
    sys.argv = ["bench.py", "--impl", "reference"]
    assert bench.main() == 0
    assert '"unavailable"' in capsys.readouterr().out


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    import json
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"gpu": "B200", "peaks": {"hbm_gbs": 6900.5, "bf16_tflops": 1610, "bf16_tflops_sustained": 1400.0}}))
    pk = bench.peaks()
    assert pk == {"hbm_gbs": 6900.5, "bf16_tflops": 1610.0, "bf16_tflops_sustained": 1400.0, "source": "measured"}
    (tmp_path / "MEASURED_PEAKS.json").write_text("{not json")
    assert bench.peaks()["source"] == "fallback"
