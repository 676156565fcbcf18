"""The engine on the reference's own tiny model: the weights its seeded generator draws for roost-tiny, and the eight
greedy tokens its tests pin for them.

The reference's model code cannot be run here (no .NET runtime on the image), so the anchors are the literals its
tests hold: FNV-1a digests of one generated slot (tests/Starlings.Roost.Models.Tiny.Tests/TinyWeightsTests.cs:53-54) and
the pinned generation for Prompt(18, 6) (tests/Starlings.Roost.Models.Tiny.Tests/RoostTinyTests.cs:16,260-293), every
step of which has a top-two gap above 1e-3 there. The weight folder is written by the product's ``random-weights
--mode reference``; the slot names are hashed into the values, so a wrong name or a wrong row order in the fused
gate_up slot moves every token.
"""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.weights.random_init import REFERENCE_TINY_SEED, reference_slot_values, reference_tensors, write_random_model
from tests import helpers as H
from tests.conftest import ROOT
from tests.plain import qwen3_plain as plain

PINNED = [57, 4, 41, 54, 132, 98, 231, 164]
ROOST_TINY = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=64, intermediate_size=128,
                  vocab_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=False, max_position_embeddings=512, torch_dtype="float32", hidden_act="silu")


def reference_prompt(length: int, salt: int) -> list[int]:
    """ids[i] = (37 i + 101 salt + 11) mod 256 (tests/Starlings.Roost.Models.Tiny.Tests/RoostTinyTests.cs:16)."""
    return [(37 * i + 101 * salt + 11) % 256 for i in range(length)]


@pytest.fixture(scope="module")
def roost_tiny_dir(tmp_path_factory):
    return write_random_model(tmp_path_factory.mktemp("roost_tiny"), ROOST_TINY, REFERENCE_TINY_SEED, mode="reference")


def test_the_products_generator_meets_the_references_digests_and_the_plain_generator():
    v = reference_slot_values(REFERENCE_TINY_SEED, "l0.q_proj", (64, 64))
    f32 = v.astype(np.float32)
    assert plain.fnv1a64_bytes(f32.tobytes()) == 10427801740649689927
    bf16 = torch.from_numpy(f32).to(torch.bfloat16).view(torch.int16).numpy()
    assert plain.fnv1a64_bytes(bf16.tobytes()) == 6253068743922294065
    cfg, w = plain.roost_tiny_reference_model()
    ours = reference_tensors(ROOST_TINY)
    assert sorted(ours) == sorted(w)
    for name, want in w.items():
        assert torch.equal(ours[name].double(), want), name
    tied = reference_tensors(dict(ROOST_TINY, tie_word_embeddings=True))
    assert "lm_head.weight" not in tied and torch.equal(tied["model.embed_tokens.weight"], ours["model.embed_tokens.weight"])


BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("cut", ["whole", "portions of 5"])
def test_the_engine_generates_the_references_pinned_tokens(roost_tiny_dir, backend, cut):
    kind, dtype = backend
    model = H.make_model(roost_tiny_dir, dtype, kind)
    engine = RoostEngine(model, page_size=16, attention_blocks=40, max_sequences=4, max_tokens=64,
                         max_chunk_tokens=5 if cut != "whole" else None)
    prompt = reference_prompt(18, 6)
    got = engine.generate([prompt], GenerationOptions(max_output_tokens=8, ignore_eos=True))[0].token_ids
    if dtype == torch.float32:
        assert got == PINNED
        return
    # bfloat16: the first token, and every token while the history is still the pinned one and the plain implementation's
    # top two logits (on weights rounded to bfloat16) are further apart than a bfloat16 path can move them
    cfg, w = plain.load_model_dir(roost_tiny_dir)
    w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    assert got[0] == PINNED[0]
    seq = list(prompt)
    for tok in got:
        logits = plain.forward_logits(cfg, w, seq)[-1]
        top = logits.topk(2)
        if float(top.values[0] - top.values[1]) > 0.15:
            assert tok == int(top.indices[0])
        seq.append(tok)


@pytest.mark.gpu
def test_the_command_line_writes_the_references_weights_and_generates_its_tokens(tmp_path):
    def roost(*args):
        return subprocess.run([sys.executable, str(ROOT / "bin" / "roost"), *args], capture_output=True, text=True, timeout=300)

    (tmp_path / "config.json").write_text(json.dumps(ROOST_TINY))
    r = roost("random-weights", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "m"), "--mode", "reference")
    assert r.returncode == 0, r.stderr
    r = roost("generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt-ids", ",".join(map(str, reference_prompt(18, 6))),
              "--max-output-tokens", "8", "--ignore-eos", "--attention-blocks", "8", "--max-sequences", "2")
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["token_ids"] == PINNED
    r = roost("random-weights", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "n"), "--mode", "reference", "--std", "0.1")
    assert r.returncode == 2 and "usage" in r.stderr
