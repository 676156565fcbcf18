"""What the reference's sampler does beside the draw (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:10-46): repetition,
frequency and presence penalties before it, the chosen token's logprob and the most likely alternatives after it. The
plain functions by hand, the kernels against the plain functions, and the engine against both, token by token."""
import math

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.engine.request import RequestError, SamplingParameters
from tests import helpers as H
from tests.conftest import TINY
from tests.plain import qwen3_plain as plain

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]


@pytest.fixture(params=BACKENDS)
def backend(request):
    return request.param


# ------------------------------------------------------------------------------------------ the plain functions, by hand
def test_plain_penalties_by_hand():
    z = [2.0, -1.0, 0.5, 3.0, -4.0]
    # token 0 generated twice, token 1 once, token 2 in the prompt only, tokens 3 and 4 never seen
    got = plain.penalise_row(z, {0: 2, 1: 1}, [2], repetition=2.0, frequency=0.5, presence=0.25)
    assert got == [2.0 / 2 - 0.5 * 2 - 0.25, -1.0 * 2 - 0.5 - 0.25, 0.5 / 2, 3.0, -4.0]
    assert plain.penalise_row(z, {}, [], 1.0, 0.0, 0.0) == z
    # a negative frequency penalty rewards repetition; the prompt alone draws no frequency or presence penalty
    assert plain.penalise_row(z, {3: 3}, [3, 4], 1.0, -1.0, 0.0) == [2.0, -1.0, 0.5, 6.0, -4.0]


def test_plain_logprobs_by_hand():
    z = [math.log(0.5), math.log(0.25), float("nan"), math.log(0.25), float("-inf")]
    assert abs(plain.logprob_at(z, 0) - math.log(0.5)) < 1e-12 and abs(plain.logprob_at(z, 3) - math.log(0.25)) < 1e-12
    assert plain.logprob_at(z, -1) == -math.inf and plain.logprob_at(z, 4) == -math.inf
    ids, vals = plain.top_logprobs(z, 3)
    assert ids == [0, 1, 3] and [round(math.exp(v), 6) for v in vals] == [0.5, 0.25, 0.25]      # ties to the lower index, NaN skipped
    ids, vals = plain.top_logprobs([float("nan"), 1.0], 3)
    assert ids == [1, -1, -1] and vals[0] == 0.0 and vals[1:] == [-math.inf, -math.inf]


def test_options_are_range_checked():
    SamplingParameters(repetition_penalty=1.5, frequency_penalty=-2.0, presence_penalty=2.0, logprobs=True, top_logprobs=20).validate()
    for bad in (dict(repetition_penalty=0.0), dict(repetition_penalty=-1.0), dict(repetition_penalty=float("nan")), dict(frequency_penalty=2.5),
                dict(presence_penalty=-2.01), dict(presence_penalty=float("inf")), dict(logprobs=True, top_logprobs=21), dict(top_logprobs=-1),
                dict(top_logprobs=2)):                      # alternatives without logprobs
        with pytest.raises(RequestError):
            SamplingParameters(**bad).validate()
    assert SamplingParameters(frequency_penalty=0.1).penalised and not SamplingParameters().penalised
    go = GenerationOptions(repetition_penalty=1.2, logprobs=True, top_logprobs=4).sampling()
    assert (go.repetition_penalty, go.frequency_penalty, go.presence_penalty, go.logprobs, go.top_logprobs) == (1.2, 0.0, 0.0, True, 4)


# ------------------------------------------------------------------------------------------ the kernels against the plain functions
@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [131, 5000, 151936])
def test_penalty_kernels(kernels, vocab):
    g = torch.Generator().manual_seed(71)
    R, slots = 5, 4
    logits = torch.randn(R, vocab, generator=g) * 3
    counts = torch.zeros(slots, vocab, dtype=torch.int32).cuda()
    bits = torch.zeros(slots, (vocab + 31) // 32, dtype=torch.int32).cuda()
    outputs = {0: [7, 7, 3, vocab - 1, 7], 2: [0, 1, 1], 3: []}
    prompts = {0: [5, 7, 31, 32, vocab - 1], 2: [], 3: [9, 9, 64, 2]}
    for slot, ids in prompts.items():
        kernels.sample_prompt_bits(bits[slot], torch.tensor(ids, dtype=torch.int32).cuda())
    row_slot = [0, -1, 2, 3, 0]        # two rows may name the same slot; a row without penalties is copied
    ids_flat = [(s, t) for s, toks in outputs.items() for t in toks]
    kernels.sample_count_tokens(counts, torch.tensor([s for s, _ in ids_flat], dtype=torch.int32).cuda(),
                                torch.tensor([t for _, t in ids_flat], dtype=torch.int32).cuda())
    kernels.sample_count_tokens(counts, torch.tensor([-1, 2], dtype=torch.int32).cuda(), torch.tensor([4, -1], dtype=torch.int32).cuda())   # ignored
    assert counts[0, 7].item() == 3 and counts[2, 1].item() == 2 and int(counts.sum()) == len(ids_flat)
    rep = torch.tensor([1.7, 1.0, 0.8, 1.3, 1.0])
    pres = torch.tensor([0.4, 0.0, -0.5, 1.0, 0.25])
    freq = torch.tensor([0.3, 0.0, 0.1, 2.0, -0.2])
    got = kernels.sample_penalise(logits.cuda(), counts, bits, torch.tensor(row_slot, dtype=torch.int32).cuda(), rep.cuda(), pres.cuda(), freq.cuda()).cpu()
    # with a mask: slot 2 allows four tokens, the other slots all of them
    mask = torch.full_like(bits, -1)
    mask[2].zero_()
    kernels.sample_prompt_bits(mask[2], torch.tensor([0, 1, 33, vocab - 1], dtype=torch.int32).cuda())
    masked = kernels.sample_penalise(logits.cuda(), counts, bits, torch.tensor(row_slot, dtype=torch.int32).cuda(), rep.cuda(), pres.cuda(), freq.cuda(),
                                     mask).cpu()
    keep = torch.zeros(vocab, dtype=torch.bool)
    keep[[0, 1, 33, vocab - 1]] = True
    assert torch.equal(masked[2][keep], got[2][keep]) and bool(torch.isinf(masked[2][~keep]).all()) and bool((masked[2][~keep] < 0).all())
    assert torch.equal(masked[[0, 1, 3, 4]], got[[0, 1, 3, 4]])
    for r, slot in enumerate(row_slot):
        if slot < 0:
            assert torch.equal(got[r], logits[r])
            continue
        c = {}
        for t in outputs[slot]:
            c[t] = c.get(t, 0) + 1
        want = torch.tensor(plain.penalise_row(logits[r].tolist(), c, prompts[slot], float(rep[r]), float(freq[r]), float(pres[r])), dtype=torch.float64)
        assert float((got[r].double() - want).abs().max()) < 2e-6, r            # float32 operations against double ones
        changed = {v for v in range(vocab) if got[r, v] != logits[r, v]}
        assert changed <= set(c) | set(prompts[slot])                           # no other token is touched


@pytest.mark.gpu
@pytest.mark.parametrize("vocab,top", [(131, 5), (5000, 20), (151936, 3), (40, 0)])
def test_logprob_kernel(kernels, vocab, top):
    g = torch.Generator().manual_seed(72)
    R = 6
    logits = torch.randn(R, vocab, generator=g) * 4
    logits[1, 3] = float("nan")
    logits[1, 10] = float("-inf")
    logits[2, 5:9] = logits[2].max() + 1.0          # a tie at the top: the lower indices come first
    logits[3] = 0.5                                  # every token the same
    logits[4, 1:] = float("nan")                     # fewer non-NaN logits than alternatives asked for
    ids = torch.tensor([0, 10, 6, vocab - 1, 0, -1], dtype=torch.int32)
    lp, top_ids, top_vals = kernels.sample_logprobs(logits.cuda(), ids.cuda(), top)
    lp2, _, _ = kernels.sample_logprobs(logits.cuda(), ids.cuda(), top)
    assert torch.equal(lp, lp2), "the sums are not repeatable"
    lp, top_ids, top_vals = lp.cpu(), top_ids.cpu(), top_vals.cpu()
    for r in range(R):
        want = plain.logprob_at(logits[r].tolist(), int(ids[r]))
        assert (lp[r] == want) if math.isinf(want) else abs(float(lp[r]) - want) < 1e-4 * (1 + abs(want)), (r, float(lp[r]), want)
        if top:
            wi, wv = plain.top_logprobs(logits[r].tolist(), top)
            assert top_ids[r].tolist() == wi, r
            for a, b in zip(top_vals[r].tolist(), wv):
                assert (a == b) if math.isinf(b) else abs(a - b) < 1e-4 * (1 + abs(b)), (r, a, b)


# ------------------------------------------------------------------------------------------ the engine, token by token
def test_generation_with_penalties_and_logprobs_follows_the_plain_functions(tiny_model_dirs, backend):
    """Teacher-forced along the engine's own tokens. A request with penalties: at every step the plain logits of its
    history, penalised by the counts of the tokens it has generated and by its prompt, give its token (greedy, where the
    penalised top two are not a near-tie; sampled, where the draw is not at an interval's edge). Its logprob and its
    alternatives are the log-softmax of the raw logits. Requests without penalties run beside it in the same steps."""
    kind, dtype = backend
    t = TINY["B"]
    model = H.make_model(tiny_model_dirs["B"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=64, max_sequences=8, max_tokens=48)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 310 + n) for n in (5, 12, 21, 9)]
    opts = [GenerationOptions(max_output_tokens=24, ignore_eos=True, repetition_penalty=1.8, frequency_penalty=0.7, presence_penalty=0.5,
                              logprobs=True, top_logprobs=4),
            GenerationOptions(max_output_tokens=24, ignore_eos=True, temperature=0.9, top_p=0.95, seed=77, repetition_penalty=0.7,
                              frequency_penalty=-0.4, logprobs=True),
            GenerationOptions(max_output_tokens=24, ignore_eos=True),                                    # plain greedy beside them
            GenerationOptions(max_output_tokens=24, ignore_eos=True, logprobs=True, top_logprobs=2)]     # logprobs without penalties
    outs = engine.generate(prompts, opts)
    assert engine.chained_steps == 0     # steps of requests with penalties or logprobs are not started ahead
    cfg, w = plain.load_model_dir(tiny_model_dirs["B"])
    if dtype == torch.bfloat16:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    lp_bound = 1e-4 if dtype == torch.float32 else 0.15
    compared = 0
    for prompt, o, out in zip(prompts, opts, outs):
        sp = o.sampling()
        assert len(out.token_ids) == 24 and (out.logprobs is None) == (not sp.logprobs) and (out.top_logprobs is None) == (sp.top_logprobs == 0)
        seq, counts = list(prompt), {}
        for n, tok in enumerate(out.token_ids):
            raw = plain.forward_logits(cfg, w, seq)[-1].tolist()
            z = plain.penalise_row(raw, counts, prompt, sp.repetition_penalty, sp.frequency_penalty, sp.presence_penalty) if sp.penalised else raw
            if sp.greedy:
                order = sorted(range(V), key=lambda v: (-z[v], v))
                if z[order[0]] - z[order[1]] > (1e-3 if dtype == torch.float32 else 0.15):
                    assert tok == order[0], f"token {n}: engine {tok}, plain {order[0]}"
                    compared += 1
            elif dtype == torch.float32:
                want, detail = plain.sample_row(z, sp.temperature, sp.top_k, sp.top_p, sp.min_p, o.seed, n, return_detail=True)
                lo = plain.sample_row(z, sp.temperature, sp.top_k, max(sp.top_p - 1e-4, 1e-6), sp.min_p, o.seed, n)
                hi = plain.sample_row(z, sp.temperature, sp.top_k, min(sp.top_p + 1e-4, 1.0), sp.min_p, o.seed, n)
                if detail["margin"] > 1e-3 and lo == want == hi:
                    assert tok == want, f"token {n}: engine {tok}, plain {want}"
                    compared += 1
            if sp.logprobs:
                assert abs(out.logprobs[n] - plain.logprob_at(raw, tok)) < lp_bound * (1 + abs(out.logprobs[n])), n
            if sp.top_logprobs:
                wi, wv = plain.top_logprobs(raw, sp.top_logprobs)
                gi = [i for i, _ in out.top_logprobs[n]]
                gaps_clear = all(raw[a] - raw[b] > (1e-3 if dtype == torch.float32 else 0.15) for a, b in zip(wi, wi[1:]))
                if gaps_clear and (dtype == torch.float32 or raw[wi[-1]] - sorted(raw, reverse=True)[len(wi)] > 0.15):
                    assert gi == wi, n
                    assert all(abs(a - b) < lp_bound * (1 + abs(b)) for (_, a), b in zip(out.top_logprobs[n], wv)), n
            counts[tok] = counts.get(tok, 0) + 1
            seq.append(tok)
    assert compared >= (60 if dtype == torch.float32 else 30), compared
    # the penalties change what is generated, and a strong repetition penalty keeps the request off its own tokens
    bare = engine.generate(prompts[:1], [GenerationOptions(max_output_tokens=24, ignore_eos=True)])[0]
    assert bare.token_ids != outs[0].token_ids
    # every slot of counts came back
    assert not engine.sampler._slots and len(engine.sampler._free) == engine.sampler.max_requests


def test_a_token_mask_keeps_generation_inside_the_allowed_tokens(tiny_model_dirs, backend):
    """Greedy and sampled requests that allow a handful of tokens: every generated token is one of them and is the plain
    choice among them (penalties first, then the mask); the logprob is still that of the raw logits; a request beside
    them is not touched. A mask that names a token outside the vocabulary is refused at admission."""
    kind, dtype = backend
    t = TINY["B"]
    model = H.make_model(tiny_model_dirs["B"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=64, max_sequences=8, max_tokens=48)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 350 + n) for n in (7, 15, 11)]
    allowed = [(3, 31, 32, 33, V - 1, 100), tuple(range(40, 60)), None]
    opts = [GenerationOptions(max_output_tokens=16, ignore_eos=True, allowed_token_ids=allowed[0], frequency_penalty=1.5, logprobs=True),
            GenerationOptions(max_output_tokens=16, ignore_eos=True, temperature=1.0, seed=5, allowed_token_ids=allowed[1]),
            GenerationOptions(max_output_tokens=16, ignore_eos=True)]
    outs = engine.generate(prompts, opts)
    bare = engine.generate(prompts[2:], opts[2:])[0]
    assert outs[2].token_ids == bare.token_ids or dtype == torch.bfloat16
    cfg, w = plain.load_model_dir(tiny_model_dirs["B"])
    if dtype == torch.bfloat16:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    compared = 0
    for prompt, o, out, allow in zip(prompts[:2], opts[:2], outs[:2], allowed[:2]):
        assert set(out.token_ids) <= set(allow)
        sp = o.sampling()
        seq, counts = list(prompt), {}
        for n, tok in enumerate(out.token_ids):
            raw = plain.forward_logits(cfg, w, seq)[-1].tolist()
            z = plain.mask_row(plain.penalise_row(raw, counts, prompt, sp.repetition_penalty, sp.frequency_penalty, sp.presence_penalty), allow)
            if sp.greedy:
                order = sorted(allow, key=lambda v: (-z[v], v))
                if z[order[0]] - z[order[1]] > (1e-3 if dtype == torch.float32 else 0.15):
                    assert tok == order[0], f"token {n}: engine {tok}, plain {order[0]}"
                    compared += 1
                assert abs(out.logprobs[n] - plain.logprob_at(raw, tok)) < (1e-4 if dtype == torch.float32 else 0.15) * (1 + abs(out.logprobs[n]))
            elif dtype == torch.float32:
                want, detail = plain.sample_row(z, sp.temperature, sp.top_k, sp.top_p, sp.min_p, o.seed, n, return_detail=True)
                if detail["margin"] > 1e-3:
                    assert tok == want, f"token {n}: engine {tok}, plain {want}"
                    compared += 1
            counts[tok] = counts.get(tok, 0) + 1
            seq.append(tok)
    assert compared >= (20 if dtype == torch.float32 else 8), compared
    with pytest.raises(RequestError):
        engine.add_request(prompts[0], GenerationOptions(allowed_token_ids=(1, V)).sampling())
    with pytest.raises(RequestError):
        engine.add_request(prompts[0], GenerationOptions(allowed_token_ids=()).sampling())
    assert not engine.sampler._slots


def test_a_request_with_penalties_draws_the_same_tokens_alone_in_a_batch_and_after_preemption(tiny_model_dirs, backend):
    kind, dtype = backend
    if dtype != torch.float32:
        pytest.skip("compared token for token: float32 only")
    t = TINY["A"]
    model = H.make_model(tiny_model_dirs["A"], dtype, kind)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 330 + n) for n in (30, 28, 26)]
    opts = [GenerationOptions(max_output_tokens=30, ignore_eos=True, temperature=0.8, seed=900 + i, repetition_penalty=1.4, presence_penalty=0.6,
                              logprobs=True) for i in range(3)]
    roomy = RoostEngine(model, page_size=16, attention_blocks=64, max_sequences=4, max_tokens=64)
    want = roomy.generate(prompts, opts)
    alone = roomy.generate(prompts[1:2], opts[1:2])[0]
    assert alone.token_ids == want[1].token_ids and all(abs(a - b) < 1e-5 for a, b in zip(alone.logprobs, want[1].logprobs))
    tight = RoostEngine(model, page_size=16, attention_blocks=9, max_sequences=4, max_tokens=64)     # 144 tokens for 3 x ~60
    got = tight.generate(prompts, opts)
    assert tight.stats()["preemptions"] > 0, "the pool is too large for this test"
    assert [o.token_ids for o in got] == [o.token_ids for o in want]       # a recomputed request counts no token twice
    # a request that is cancelled gives its slot back
    rid = roomy.add_request(prompts[0], opts[0].sampling())
    for _ in range(3):
        roomy.step()
    assert rid in roomy.sampler._slots
    roomy.cancel(rid)
    assert rid not in roomy.sampler._slots and len(roomy.sampler._free) == roomy.sampler.max_requests


def test_more_requests_with_penalties_than_a_step_has_rows(tiny_model_dirs, backend):
    """A request keeps its counts from its first sampled token to its end, also while it waits: preempted, its pages
    gone, with requests that are ordered before it taking the step's rows. With two rows a step and pages for little more
    than one request, more than two requests hold counts at a time; the tokens are those of an engine with room for all."""
    kind, dtype = backend
    if dtype != torch.float32:
        pytest.skip("compared token for token: float32 only")
    model = H.make_model(tiny_model_dirs["A"], dtype, kind)
    V = TINY["A"]["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 370 + n) for n in (12, 19, 5, 9)]
    opts = [GenerationOptions(max_output_tokens=n, ignore_eos=True, repetition_penalty=1.3, frequency_penalty=0.5, temperature=t, seed=40 + i)
            for i, (n, t) in enumerate(zip((50, 40, 36, 30), (None, 0.8, None, 0.9)))]
    roomy = RoostEngine(model, page_size=16, attention_blocks=64, max_sequences=8, max_tokens=128)
    want = [o.token_ids for o in roomy.generate(prompts, opts)]
    tight = RoostEngine(model, page_size=16, attention_blocks=5, max_sequences=2, max_tokens=128)
    got = [o.token_ids for o in tight.generate(prompts, opts)]
    assert tight.stats()["preemptions"] > 0 and tight.sampler.max_requests > 2, "no request waited with counts of its own"
    assert got == want
    assert not tight.sampler._slots and len(tight.sampler._free) == tight.sampler.max_requests
