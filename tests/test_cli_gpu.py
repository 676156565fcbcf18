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
    # penalties change the greedy tokens; logprobs and alternatives come with the line (the first alternative of a greedy
    # token without penalties is the token itself)
    r = roost("generate", "--model", str(model_dir), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-output-tokens", "6",
              "--ignore-eos", "--attention-blocks", "8", "--logprobs", "--top-logprobs", "2")
    assert r.returncode == 0, r.stderr
    with_lp = json.loads(r.stdout.strip().splitlines()[-1])
    assert with_lp["token_ids"] == out["token_ids"] and len(with_lp["logprobs"]) == 6 and all(lp <= 0 for lp in with_lp["logprobs"])
    assert [alts[0][0] for alts in with_lp["top_logprobs"]] == out["token_ids"] and all(len(alts) == 2 for alts in with_lp["top_logprobs"])
    logits = plain.forward_logits(cfg, w, prompt)[-1].tolist()
    assert abs(with_lp["logprobs"][0] - plain.logprob_at(logits, out["token_ids"][0])) < 1e-4
    r = roost("generate", "--model", str(model_dir), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-output-tokens", "6",
              "--ignore-eos", "--attention-blocks", "8", "--repetition-penalty", "5", "--frequency-penalty", "2", "--presence-penalty", "2")
    assert r.returncode == 0, r.stderr
    penalised = json.loads(r.stdout.strip().splitlines()[-1])["token_ids"]
    assert len(set(penalised)) == 6 and not set(penalised) & set(prompt)       # so strong that no token comes twice, nor one of the prompt
    r = roost("doctor", "--model", str(model_dir))
    assert r.returncode == 0 and "ok   weights" in r.stdout and "ok   gpu" in r.stdout
    r = roost("bench", "--model", str(model_dir), "--batch", "3", "--prompt-tokens", "20", "--new-tokens", "5", "--attention-blocks", "16")
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["batch"] == 3 and line["prefill_tokens_per_s"] > 0 and line["decode_tokens_per_s"] > 0 and line["preemptions"] == 0
    r = roost("doctor", "--model", str(tmp_path))
    assert r.returncode == 1 and "FAIL" in r.stdout
    for bad in (["generate", "--model", "x", "--bogus", "1"], ["generate", "--model"], ["generate", "--model", "a", "--model", "b"],
                ["serve"], [], ["generate", "--model", "x"], ["generate", "--model", "x", "--prompt-ids", "1", "--max-output-tokens", "many"],
                ["generate", "--model", "x", "--prompt-ids", "1", "--top-logprobs", "3"],          # alternatives need --logprobs
                ["generate", "--model", "x", "--prompt-ids", "1", "--frequency-penalty", "2.5"],
                ["generate", "--model", "x", "--prompt-ids", "1", "--repetition-penalty", "0"]):
        r = roost(*bad)
        assert r.returncode == 2 and "usage" in r.stderr, bad
    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(TINY["B"]["config"]))
    r = roost("random-weights", "--config", str(cfg_path), "--out", str(tmp_path / "m"), "--seed", "4", "--std", "0.05")
    assert r.returncode == 0 and (tmp_path / "m" / "model.safetensors").exists() and (tmp_path / "m" / "config.json").exists()


def test_chat_console_keeps_the_conversation(tiny_model_dirs, tmp_path):
    """Token ids in and out; every turn's prompt is the conversation so far; /reset clears it; a turn that cannot fit is
    dropped with the refusal's name; with a tokenizer file a line is text and so is the reply."""
    import shutil
    model_dir = tiny_model_dirs["A"]
    V = TINY["A"]["config"]["vocab_size"]
    first, second = H.random_ids(9, V, 21), H.random_ids(4, V, 22)
    too_long = " ".join(map(str, H.random_ids(600, V, 23)))        # the model has 512 positions
    script = "\n".join([" ".join(map(str, first)), ",".join(map(str, second)), too_long, "/reset", " ".join(map(str, first)), "/exit"]) + "\n"
    args = [sys.executable, str(ROOT / "bin" / "roost"), "chat", "--model", str(model_dir), "--dtype", "float32", "--max-output-tokens", "5",
            "--ignore-eos", "--attention-blocks", "16"]
    r = subprocess.run(args, input=script, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = [ln[2:] if ln.startswith("> ") else ln for ln in r.stdout.splitlines()]
    replies = [ln for ln in lines if ln and ln[0].isdigit()]
    cfg, w = plain.load_model_dir(model_dir)
    a = plain.greedy(cfg, w, first, 5)
    b = plain.greedy(cfg, w, first + a + second, 5)
    assert [list(map(int, x.split())) for x in replies] == [a, b, a]
    assert any(ln.startswith("[") and "/reset" in ln for ln in lines) and "(conversation cleared)" in lines

    from tokenizers import Tokenizer, models, pre_tokenizers
    words = {f"w{i}": i for i in range(V)}
    tok = Tokenizer(models.WordLevel(words, unk_token="w0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    with_tok = tmp_path / "with_tokenizer"
    shutil.copytree(model_dir, with_tok)
    tok.save(str(with_tok / "tokenizer.json"))
    text = " ".join(f"w{i}" for i in first)
    r = subprocess.run(args[:4] + [str(with_tok)] + args[5:] + ["--template", "{message}"], input=text + "\n/exit\n", capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    reply = [ln[2:] for ln in r.stdout.splitlines() if ln.startswith("> w")]
    assert reply and reply[0].split() == [f"w{i}" for i in a]
    r = subprocess.run(args + ["--template", "no placeholder"], input="", capture_output=True, text=True, timeout=300)
    assert r.returncode == 2 and "usage" in r.stderr
