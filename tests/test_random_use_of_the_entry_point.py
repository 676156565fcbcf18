"""The request interface under random use, on the CPU stand-in for the kernels and on the device: requests are added
while others run, with priorities, deadlines, stop ids, penalties and logprobs; some are cancelled; rows and tokens a step,
the cap on a prompt's portion and the number of pages are drawn at random (few pages: requests wait, are preempted and
computed again). In half of the cases steps fail at random, before the forward pass or after the step has committed its
rows. Every finished request is the plain implementation's choice token by token on its own history, ends for the reason
and at the token it should, and every page, state slot, seed and slot of penalty counts comes back. The seeds are a sample
of longer runs of the same draws."""
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.sampling.sampler import Sampler
from roost_b200.weights.random_init import write_random_model
from tests import helpers as H
from tests.plain import qwen3_plain as plain
from tests.test_random_configurations_gpu import draw

BACKENDS = [pytest.param("gpu", marks=pytest.mark.gpu), "fake"]


@pytest.mark.parametrize("inject", [False, True], ids=["", "failing-steps"])
@pytest.mark.parametrize("seed", [40000, 40016, 40030, 40045, 50007])
@pytest.mark.parametrize("kind", BACKENDS)
def test_requests_added_cancelled_stopped_and_preempted_at_random(tmp_path, monkeypatch, kind, seed, inject):
    rng, cfg, page, dtype, _, _ = draw(seed)
    if kind == "fake":
        dtype = torch.float32
    eos = [rng.randrange(cfg["vocab_size"]) for _ in range(rng.choice([0, 1, 2]))]
    if eos:
        cfg["eos_token_id"] = eos
    V = cfg["vocab_size"]
    reqs = []
    for i in range(rng.randrange(3, 10)):
        kw = dict(max_output_tokens=rng.choice([1, 2, rng.randrange(3, 30), rng.randrange(30, 50)]), ignore_eos=rng.random() < 0.5)
        if rng.random() < 0.4:
            kw.update(temperature=rng.choice([0.5, 0.9, 1.3]), top_k=rng.choice([0, 0, 5, 40]), top_p=rng.choice([1.0, 0.9, 0.5]), seed=seed * 100 + i)
        if rng.random() < 0.3:
            kw.update(repetition_penalty=rng.choice([0.7, 1.3]), frequency_penalty=rng.choice([0.0, 0.5]), presence_penalty=rng.choice([0.0, 0.4]))
        if rng.random() < 0.3:
            kw.update(logprobs=True, top_logprobs=rng.choice([0, 2]))
        stops = tuple(rng.sample(range(V), rng.choice([0, 0, 3, 20])))
        prompt = H.random_ids(rng.choice([rng.randrange(1, 20), rng.randrange(20, 150)]), V, seed * 17 + i)
        reqs.append(dict(prompt=prompt, opts=GenerationOptions(**kw), stops=stops, priority=rng.choice([0, 0, 0, 1, 5]), deadline=rng.choice([None, None, 1.0, 2.0]),
                         at=rng.randrange(0, 40), cancel_at=rng.randrange(1, 80) if rng.random() < 0.2 else None))
    pages_of = [-(-(len(r["prompt"]) + r["opts"].max_output_tokens + 1) // page) for r in reqs]
    biggest, total = max(pages_of), sum(pages_of)
    blocks = rng.choice([biggest + 1, biggest + 3, (biggest + total) // 2, total + 4])
    max_seq = rng.randrange(1, 7)
    max_tok = rng.choice([8, 16, 33, 64, 128])
    chunk = rng.choice([None, None, 4, 16])
    chain = rng.random() < 0.7
    write_random_model(tmp_path, cfg, seed=seed, std=rng.choice([0.05, 0.08]), norm_std=rng.choice([0.0, 0.1]))
    model = H.make_model(tmp_path, dtype, kind)
    failures = random.Random(seed)
    if inject:
        forward, sample = model.forward, Sampler.__call__

        def failing_forward(batch, storage):
            if failures.random() < 0.03:
                raise RuntimeError("injected failure in the step")
            return forward(batch, storage)

        def failing_sampler(self, logits, rows):
            if failures.random() < 0.02:
                raise RuntimeError("injected failure after the step")
            return sample(self, logits, rows)

        model.forward = failing_forward
        monkeypatch.setattr(Sampler, "__call__", failing_sampler)
    engine = RoostEngine(model, page_size=page, attention_blocks=blocks, max_sequences=max_seq, max_tokens=max_tok, max_chunk_tokens=chunk, chain_steps=chain,
                         **({"device": "cpu"} if kind == "fake" else {}))
    ids, got, done, cancelled = {}, {}, {}, set()
    pending = sorted(range(len(reqs)), key=lambda i: reqs[i]["at"])
    step = 0
    while pending or engine.has_unfinished():
        while pending and reqs[pending[0]]["at"] <= step:
            i = pending.pop(0)
            r = reqs[i]
            ids[i] = engine.add_request(r["prompt"], r["opts"].sampling(), stop_token_ids=r["stops"], priority=r["priority"], deadline=r["deadline"])
            got[i] = []
        for i, rid in ids.items():
            if reqs[i]["cancel_at"] == step and i not in done and i not in cancelled:
                engine.cancel(rid)
                cancelled.add(i)
        by_id = {rid: i for i, rid in ids.items()}
        try:
            events = engine.step()
        except RuntimeError as e:
            assert inject and "injected" in str(e)
            events = []
        for e in events:
            i = by_id[e.request_id]
            assert i not in cancelled and i not in done, f"an event for request {i} after its end"
            if e.token is not None:
                got[i].append((e.token, e.logprob))
            if e.finish_reason is not None:
                done[i] = e.finish_reason
        step += 1
        assert step < 20000, "the engine does not come to an end"
    engine.check_device()
    engine.executor.cache.check_invariants()
    assert all(pool.used_count == 0 for pool in engine.executor.cache.pools)
    assert not engine.sampler._slots and (engine.sampler._counts is None or len(engine.sampler._free) == engine.sampler.max_requests)
    assert not engine._seeds
    pc, w = plain.load_model_dir(tmp_path)
    f32 = dtype == torch.float32
    if not f32:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    compared = 0
    for i, r in enumerate(reqs):
        if i in cancelled:
            continue
        o, sp, p = r["opts"], r["opts"].sampling(), r["prompt"]
        toks = [t for t, _ in got[i]]
        stops = set(r["stops"]) | (set() if o.ignore_eos else set(eos))       # ignore_eos: the model's stop ids only
        if done[i] == "stop":
            assert toks[-1] in stops and not any(t in stops for t in toks[:-1])
        else:
            assert done[i] == "length" and len(toks) == o.max_output_tokens and not any(t in stops for t in toks)
        logits = plain.forward_logits(pc, w, list(p) + toks[:-1])
        counts = {}
        for j, (tok, lp) in enumerate(got[i]):
            raw = logits[len(p) - 1 + j].tolist()
            z = plain.penalise_row(raw, counts, p, sp.repetition_penalty, sp.frequency_penalty, sp.presence_penalty) if sp.penalised else raw
            if sp.greedy:
                order = sorted(range(V), key=lambda v: (-z[v], v))
                if z[order[0]] - z[order[1]] > (1e-3 if f32 else 0.15):
                    assert tok == order[0], f"request {i}, token {j}: engine {tok}, plain {order[0]}"
                    compared += 1
            elif f32:
                want, detail = plain.sample_row(z, sp.temperature, sp.top_k, sp.top_p, sp.min_p, o.seed, j, return_detail=True)
                edge = {plain.sample_row(z, sp.temperature, sp.top_k, tp, sp.min_p, o.seed, j) for tp in (max(sp.top_p - 1e-4, 1e-6), min(sp.top_p + 1e-4, 1.0))}
                tie = tok in detail["prob"] and abs(detail["prob"][tok] - detail["prob"][want]) < 1e-4 * detail["prob"][want]
                if detail["margin"] > 1e-3 and edge == {want} and not (tok != want and tie):
                    assert tok == want, f"request {i}, token {j}: engine {tok}, plain sampler {want}"
                    compared += 1
            assert (lp is None) == (not sp.logprobs)
            if sp.logprobs:
                assert abs(lp - plain.logprob_at(raw, tok)) < (1e-4 if f32 else 0.15) * (1 + abs(lp))
            counts[tok] = counts.get(tok, 0) + 1
    assert compared > 0
    engine.executor.close()
