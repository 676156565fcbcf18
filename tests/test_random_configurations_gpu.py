"""Configurations drawn at random, beyond the fixed tiny ones: head counts and groups, head sizes from 16 to 256, widths
and vocabularies that are no power of two, one to three layers with a window in some, pages of 4 to 32 tokens, either
precision, with and without captured steps. Three to six requests of up to 700 tokens are fed in random portions with at
most four live at a time and just enough pages for the four longest, so pages are used again, and every logit of every
position is compared with the plain implementation. The seeds are a sample of a longer run of the same draws (thousands
of configurations), picked so that every attention kernel, a window that pages fall out of, and steps that split a
decoding row into several chunks all occur."""
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.engine.executor import StepExecutor
from roost_b200.weights.random_init import write_random_model
from tests import helpers as H
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def draw(seed: int):
    rng = random.Random(seed)
    nkv = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 4, 6, 8])
    d = rng.choice([16, 32, 48, 64, 64, 80, 96, 128, 128, 256])
    layers = rng.choice([1, 2, 3])
    hidden = rng.choice([40, 44, 64, 72, 96, 120, 136, 200])
    inter = rng.choice([64, 100, 128, 200, 256, 272, 384])
    vocab = rng.randrange(100, 700)
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=layers, hidden_size=hidden,
               num_attention_heads=nkv * group, num_key_value_heads=nkv, head_dim=d, intermediate_size=inter, vocab_size=vocab,
               rope_theta=rng.choice([1e4, 5e4, 1e6]), rms_norm_eps=rng.choice([1e-5, 1e-6]), tie_word_embeddings=rng.random() < 0.5,
               max_position_embeddings=4096, torch_dtype="bfloat16", hidden_act="silu")
    if rng.random() < 0.5:
        cfg["sliding_window"] = rng.choice([9, 24, 40, 48, 100, 200])
        cfg["layer_types"] = [rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)]
    page = rng.choice([4, 8, 16, 16, 32])
    dtype = rng.choice([torch.float32, torch.bfloat16])
    lens = [rng.choice([rng.randrange(10, 80), rng.randrange(80, 300), rng.randrange(300, 700)]) for _ in range(rng.randrange(3, 7))]
    graphs = rng.random() < 0.7
    return rng, cfg, page, dtype, lens, graphs


@pytest.mark.parametrize("seed", [1017, 1018, 1025, 1038, 1075, 1102, 1109, 1110, 1153, 1162, 1422, 1441, 1569, 1680, 1711, 1714])
def test_a_random_configuration_in_random_portions_and_batches(tmp_path, seed):
    rng, cfg, page, dtype, lens, graphs = draw(seed)
    write_random_model(tmp_path, cfg, seed=seed, std=rng.choice([0.05, 0.08]), norm_std=rng.choice([0.0, 0.1]))
    model = H.make_model(tmp_path, dtype, "gpu")
    need = sorted((-(-(n + 1) // page) for n in lens), reverse=True)
    ex = StepExecutor(model, page_size=page, num_pages=sum(need[:4]) + 2, max_requests=4, use_graphs=graphs)
    requests = {f"r{i}": H.random_ids(n, cfg["vocab_size"], seed * 31 + i) for i, n in enumerate(lens)}
    got = H.run_mixed(ex, requests, seed=seed, max_live=4, decode_tail=rng.choice([4, 8, 40]))
    model.rt.kernels.check_device_status()
    for rid, ids in requests.items():
        want = H.plain_logits(tmp_path, ids, dtype == torch.bfloat16)
        assert H.scaled_error(got[rid], want) <= H.bound_for(dtype), (rid, cfg, page, lens)
        if dtype == torch.bfloat16:
            assert H.rms_error(got[rid], want) <= H.BF16_RMS_BOUND, (rid, cfg, page, lens)
    ex.close()


@pytest.mark.parametrize("seed", [9006, 9007, 9012, 9043, 9139, 9142, 9144, 9230, 9232])
def test_a_random_configuration_through_the_entry_point(tmp_path, seed):
    """The same draws through ``RoostEngine.generate``: three to eleven requests, greedy and sampled (temperature, top-k,
    top-p, min-p, a seed each), under random limits of rows and tokens a step and with as few pages as the largest request
    needs or more, so that prompts are cut, requests wait, some are preempted and computed again, and decode steps are
    started ahead. Every token is the plain implementation's choice on the engine's own history, unless the plain top two
    (or the draw and the edge of its token's interval) are too close to call. The seeds are a sample of a run of some
    thousands; what differed there were draws between two tokens of equal probability to seven digits, or a kept set whose
    edge lay within 1e-4 of top-p or of the min-p floor."""
    rng, cfg, page, dtype, _, _ = draw(seed)
    V = cfg["vocab_size"]
    prompts = [H.random_ids(rng.choice([rng.randrange(1, 20), rng.randrange(20, 120), rng.randrange(120, 300)]), V, seed * 17 + i)
               for i in range(rng.randrange(3, 12))]
    opts = []
    for i in range(len(prompts)):
        new = rng.choice([1, 2, rng.randrange(3, 30), rng.randrange(30, 70)])
        if rng.random() < 0.4:
            opts.append(GenerationOptions(max_output_tokens=new, ignore_eos=True, temperature=rng.choice([0.5, 0.9, 1.3]), top_k=rng.choice([0, 0, 5, 40]),
                                          top_p=rng.choice([1.0, 0.9, 0.5]), min_p=rng.choice([0.0, 0.0, 0.05]), seed=seed * 100 + i))
        else:
            opts.append(GenerationOptions(max_output_tokens=new, ignore_eos=True))
    pages_of = [-(-(len(p) + o.max_output_tokens + 1) // page) for p, o in zip(prompts, opts)]
    biggest, total = max(pages_of), sum(pages_of)
    blocks = rng.choice([biggest + 1, biggest + 3, (biggest + total) // 2, total + 4])
    max_seq = rng.randrange(1, 7)
    max_tok = rng.choice([8, 16, 33, 64, 128, 256])
    chain = rng.random() < 0.7
    write_random_model(tmp_path, cfg, seed=seed, std=rng.choice([0.05, 0.08]), norm_std=rng.choice([0.0, 0.1]))
    model = H.make_model(tmp_path, dtype, "gpu")
    engine = RoostEngine(model, page_size=page, attention_blocks=blocks, max_sequences=max_seq, max_tokens=max_tok, chain_steps=chain)
    outs = engine.generate(prompts, opts)
    engine.check_device()
    pc, w = plain.load_model_dir(tmp_path)
    if dtype == torch.bfloat16:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    compared = 0
    for i, (p, o, out) in enumerate(zip(prompts, opts, outs)):
        assert out.finish_reason == "length" and len(out.token_ids) == o.max_output_tokens
        logits = plain.forward_logits(pc, w, list(p) + out.token_ids[:-1])
        for j, tok in enumerate(out.token_ids):
            row = logits[len(p) - 1 + j]
            if o.temperature:
                if dtype == torch.float32:
                    want, detail = plain.sample_row(row.tolist(), o.temperature, o.top_k, o.top_p, o.min_p, o.seed, j, return_detail=True)
                    if detail["margin"] > 1e-4:
                        assert tok == want, f"request {i}, token {j}: engine {tok}, plain sampler {want} (margin {detail['margin']:.2e})"
                        compared += 1
            else:
                top = row.topk(2)
                gap = float(top.values[0] - top.values[1])
                if gap > (1e-3 if dtype == torch.float32 else 0.15):
                    assert tok == int(top.indices[0]), f"request {i}, token {j}: engine {tok}, plain {int(top.indices[0])} (gap {gap:.3g})"
                    compared += 1
    assert compared > 20
    engine.executor.cache.check_invariants()
    assert all(pool.used_count == 0 for pool in engine.executor.cache.pools)       # every page and slot came back
