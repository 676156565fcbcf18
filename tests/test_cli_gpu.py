"""The roost command line as a user runs it."""
import json
import subprocess
import sys

import pytest

from tests import helpers as H
from tests.conftest import ROOT, TINY
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def roost(*args):
    return subprocess.run([sys.executable, str(ROOT / "bin" / "roost"), *args], capture_output=True, text=True, timeout=300)


def test_generate_doctor_and_usage_errors(tiny_model_dirs, tmp_path):
    model_dir = tiny_model_dirs["A"]
    prompt = H.random_ids(12, TINY["A"]["config"]["vocab_size"], 3)
    r = roost("generate", "--model", str(model_dir), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
              "--max-output-tokens", "6", "--ignore-eos", "--attention-blocks", "8", "--max-sequences", "2")
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    cfg, w = plain.load_model_dir(model_dir)
    assert out["token_ids"] == plain.greedy(cfg, w, prompt, 6) and out["finish_reason"] == "length" and out["prompt_tokens"] == 12
    (tmp_path / "prompts.txt").write_text("1 2 3\n4,5,6,7\n")
    r = roost("generate", "--model", str(model_dir), "--prompt-file", str(tmp_path / "prompts.txt"), "--max-output-tokens", "3",
              "--temperature", "0.7", "--top-p", "0.9", "--top-k", "20", "--seed", "5", "--attention-blocks", "8")
    assert r.returncode == 0 and len(r.stdout.strip().splitlines()) == 2
    r = roost("doctor", "--model", str(model_dir))
    assert r.returncode == 0 and "ok   weights" in r.stdout and "ok   gpu" in r.stdout
    r = roost("doctor", "--model", str(tmp_path))
    assert r.returncode == 1 and "FAIL" in r.stdout
    for bad in (["generate", "--model", "x", "--bogus", "1"], ["generate", "--model"], ["generate", "--model", "a", "--model", "b"],
                ["serve"], [], ["generate", "--model", "x"], ["generate", "--model", "x", "--prompt-ids", "1", "--max-output-tokens", "many"]):
        r = roost(*bad)
        assert r.returncode == 2 and "usage" in r.stderr, bad
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(TINY["B"]["config"]))
    r = roost("random-weights", "--config", str(cfg_path), "--out", str(tmp_path / "m"), "--seed", "4", "--std", "0.05")
    assert r.returncode == 0 and (tmp_path / "m" / "model.safetensors").exists() and (tmp_path / "m" / "config.json").exists()
