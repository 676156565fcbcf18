"""The plain implementation itself, against the constants the reference's own tests pin (it cannot be compared with
the reference's code: that is C# and no .NET SDK is in the image) and against hand cases of the sampler."""
import json
import math
from pathlib import Path

import numpy as np
import torch

from tests.plain import qwen3_plain as plain

GOLDEN = json.loads((Path(__file__).parent / "golden" / "roost_tiny_plain.json").read_text())
PINS = GOLDEN["reference_pins"]
SEED = 0x524F4F53540001


def test_weight_generator_digests():
    v = plain.tiny_weights(SEED, "l0.q_proj", (64, 64))
    assert plain.fnv1a64_bytes(v.astype("<f4").tobytes()) == PINS["digest_l0_q_proj_f32"]
    vb = plain.tiny_weights(SEED, "l0.q_proj", (64, 64), "BF16")
    bits = torch.from_numpy(vb).to(torch.bfloat16).view(torch.int16).numpy().astype("<i2").tobytes()
    assert plain.fnv1a64_bytes(bits) == PINS["digest_l0_q_proj_bf16"]
    norm = plain.tiny_weights(3, "l0.input_norm", (64,))
    assert 0.899 <= norm.min() and norm.max() <= 1.101
    assert np.abs(plain.tiny_weights(3, "l0.down", (64, 128))).max() <= 1.5 / math.sqrt(128)


def test_greedy_ids_of_roost_tiny_are_the_references():
    cfg, w = plain.roost_tiny_reference_model()
    prompt = GOLDEN["prompt"]
    assert prompt == [((i * 37) + (6 * 101) + 11) % 256 for i in range(18)]
    got = plain.greedy(cfg, w, prompt, 8)
    assert got == PINS["greedy_ids_prompt_18_6"] == GOLDEN["plain_greedy"]
    # no step is a near-tie, so the equality does not hinge on rounding
    seq = list(prompt)
    for t in got:
        top = plain.forward_logits(cfg, w, seq)[-1].topk(2).values
        assert float(top[0] - top[1]) > 1e-3
        seq.append(t)
    logits = plain.forward_logits(cfg, w, prompt)
    assert np.allclose(logits[-1].numpy(), GOLDEN["plain_last_row_logits"], rtol=0, atol=1e-12)
    assert np.allclose(logits[0][:16].numpy(), GOLDEN["plain_first_row_logits_head"], rtol=0, atol=1e-12)


def test_philox_known_answers():
    for counter, key, want in PINS["philox"]:
        assert list(plain.philox4x32_10(tuple(counter), tuple(key))) == want
    u = plain.philox_uniform(7, 3)
    assert 0 <= u < 1 and u * 2 ** 24 == int(u * 2 ** 24)


def test_causal_attention_sees_the_history_and_only_the_history():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 4, 8, generator=g, dtype=torch.float64) for _ in range(3))
    k, v = k[:, :2], v[:, :2]
    out = plain.causal_gqa_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0
    out2 = plain.causal_gqa_attention(q, k2, v2, 0.3)
    assert torch.equal(out[:5], out2[:5]) and not torch.allclose(out[5:], out2[5:])
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))          # the first query sees only its own key
    w3 = plain.causal_gqa_attention(q, k, v, 0.3, window=3)
    k3, v3 = k.clone(), v.clone()
    k3[:4], v3[:4] = 7, 7                                                    # keys the last queries cannot see with a window of 3
    assert torch.allclose(plain.causal_gqa_attention(q, k3, v3, 0.3, window=3)[6:], w3[6:])
    assert torch.equal(plain.causal_gqa_attention(q, k, v, 0.3, window=100), out)


def test_rope_and_norm_hand_cases():
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0]]], dtype=torch.float64)
    r = plain.rope_neox(x, [1], theta=10000.0)
    f1 = 10000.0 ** (-2.0 / 4)
    want = [math.cos(1.0), -math.sin(f1), math.sin(1.0), math.cos(f1)]
    assert np.allclose(r[0, 0].numpy(), want, atol=1e-15)
    assert torch.equal(plain.rope_neox(x, [0], 1e6), x)
    part = plain.rope_neox(torch.ones(1, 1, 6, dtype=torch.float64), [3], 10.0, rotary_dim=2)
    assert torch.equal(part[0, 0, 2:], torch.ones(4, dtype=torch.float64))
    y = plain.rms_norm(torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    assert np.allclose(y.numpy(), [[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]])
    assert np.allclose(plain.silu_and_mul(torch.tensor([0.0, 2.0]), torch.tensor([5.0, 3.0])).numpy(), [0.0, 2 / (1 + math.exp(-2)) * 3])


def test_sampler_hand_cases():
    # greedy: ties to the lowest index, NaN never chosen, nothing allowed gives -1 (tests/Starlings.Roost.Ops.Tests/SamplingTests.cs:38-66)
    assert plain.sample_row([1.0, 3.0, 3.0, 2.0], 0.0) == 1
    assert plain.sample_row([float("nan"), 2.0, float("-inf")], 0.0) == 1
    assert plain.sample_row([float("nan"), float("-inf")], 0.7) == -1
    z = [math.log(p) for p in (0.5, 0.2, 0.2, 0.1)]
    # top-k 1 and a tiny top-p both leave the best token whatever the draw
    for seed in range(5):
        assert plain.sample_row(z, 1.0, top_k=1, seed=seed) == 0
        assert plain.sample_row(z, 1.0, top_p=0.3, seed=seed) == 0
        assert plain.sample_row(z, 1.0, min_p=0.5, seed=seed) == 0
        # top-p 0.7 keeps the crossing token: {0, 1} (ties by lower index), never 2 or 3
        assert plain.sample_row(z, 1.0, top_p=0.7, seed=seed) in (0, 1)
    # the draw follows the cumulative masses in the sorted order
    counts = [0, 0, 0, 0]
    for off in range(4000):
        counts[plain.sample_row(z, 1.0, seed=11, offset=off)] += 1
    assert [round(c / 4000, 1) for c in counts] == [0.5, 0.2, 0.2, 0.1]
    # temperature sharpens
    hot = sum(plain.sample_row(z, 0.25, seed=3, offset=o) == 0 for o in range(500))
    assert hot > 450
    # same seed and offset, same token; the batch plays no part by construction
    assert plain.sample_row(z, 0.9, top_p=0.95, seed=5, offset=2) == plain.sample_row(z, 0.9, top_p=0.95, seed=5, offset=2)


def test_schedule_and_shared_cache_in_the_plain_model(tmp_path):
    from roost_b200.weights.random_init import write_random_model
    from tests.conftest import TINY_A
    write_random_model(tmp_path, TINY_A, seed=0, std=0.08)
    cfg, w = plain.load_model_dir(tmp_path)
    ids = list(range(3, 20))
    base = plain.forward_logits(cfg, w, ids)
    assert torch.equal(base, plain.forward_logits(cfg, w, ids, [(0, None), (1, None)]))
    twice = plain.forward_logits(cfg, w, ids, [(0, None), (1, None), (0, None)])
    shared = plain.forward_logits(cfg, w, ids, [(0, None), (1, None), (0, 0)])
    assert not torch.allclose(twice, base) and not torch.allclose(twice, shared)
