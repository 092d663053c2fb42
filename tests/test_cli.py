"""The command line without a GPU: model folders from a configuration and a seed, model description."""
from __future__ import annotations

import json
import os
import subprocess
import sys

from helpers import ROOT, TINY_E


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "inferctl"), *args], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_random_then_models(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_E))
    out = _run("random", "--config", str(cfg), "--seed", "3", "--out", str(tmp_path / "m"), "--float32-vectors")
    assert out["architecture"] == "Qwen2ForCausalLM"
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    info = _run("models", "--model", str(tmp_path / "m"))
    assert info["config"]["hidden_size"] == 96 and info["tensors"] == 3 * 12 + 3
    assert [g["window"] for g in info["cache_groups"]] == [None, 40]
