"""Text in and out through the entry point (stop strings, chat messages), sampled generation against the plain
sampler, and what the engine does when a step raises."""
import pytest
import torch

from roost_b200 import GenerationOptions, IncrementalDetokenizer, RoostEngine, StopMatcher, render_chat
from roost_b200.engine.request import RequestError
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


class LetterTokenizer:
    """One character a token: id i is chr(0x100 + i), so any id sequence is text and text is ids again."""

    def encode(self, text):
        return [ord(c) - 0x100 for c in text]

    def decode(self, ids):
        return "".join(chr(0x100 + i) for i in ids)


class ByteTokenizer:
    """A token is a byte; characters of several bytes end inside a token sequence now and then."""

    def encode(self, text):
        return list(text.encode())

    def decode(self, ids):
        return bytes(ids).decode("utf-8", errors="replace")


# ------------------------------------------------------------------------------------------ the matcher and the detokeniser alone
def test_stop_matcher_holds_back_partial_matches_and_prefers_the_earliest_then_longest():
    m = StopMatcher(["END", "ENDING", "xy"])
    out = []
    for piece in ["abE", "N", "x", "EN", "DI", "NG!"]:
        emit, matched = m.push(piece)
        out.append(emit)
        if matched:
            break
    # "abE" may begin END: the E waits; "ENx" is no stop: it is given out, the x waits (xy); "xEN" gives x out; ...
    # END is whole with "DI", but ENDING, which begins at the same place and would win, is still open: it is decided with "NG!"
    assert out == ["ab", "", "EN", "x", "", ""] and matched == "ENDING"
    assert m.flush() == "" and m.push("more") == ("", "ENDING")
    m = StopMatcher(["ab", "abc"])
    assert m.push("zab") == ("z", None)        # "abc" might still come, and at the same start the longest wins
    assert m.push("d") == ("", "ab")           # it did not
    m = StopMatcher(["ab", "abc"])
    assert m.push("zab") == ("z", None) and m.flush() == "" and m.matched == "ab"      # nor when the text ends there
    m = StopMatcher(["abc", "ab"])
    assert m.push("zabc") == ("z", "abc")      # same start: the longest
    m = StopMatcher(["abcd", "bc"])
    assert m.push("abc") == ("", None)         # "bc" is whole, but "abcd" begins before it and is still open
    assert m.push("d!") == ("", "abcd")
    m = StopMatcher(["abcd", "bc"])
    assert m.push("abc") == ("", None) and m.push("x") == ("a", "bc")
    m = StopMatcher(["stop"])
    assert m.push("no st") == ("no ", None) and m.flush() == "st"
    assert StopMatcher([]).push("anything") == ("anything", None)
    with pytest.raises(ValueError):
        StopMatcher([""])


def test_stop_matcher_decides_as_on_the_whole_text_however_it_is_cut():
    """Random texts over three letters, random stop strings that overlap and contain one another, random cuts: what is
    given out is the text before the earliest match of the whole text, and the match named is the longest that begins
    there, as if the text had come in one piece."""
    import random
    rng = random.Random(11)
    for _ in range(3000):
        stops = ["".join(rng.choice("abc") for _ in range(rng.randrange(1, 6))) for _ in range(rng.randrange(1, 5))]
        text = "".join(rng.choice("abc" if rng.random() < 0.8 else "xyz") for _ in range(rng.randrange(1, 40)))
        want = None
        for s in stops:
            at = text.find(s)
            if at >= 0 and (want is None or (at, -len(s)) < (want[0], -len(want[1]))):
                want = (at, s)
        cuts = sorted(rng.sample(range(1, len(text)), min(len(text) - 1, rng.randrange(0, 8)))) if len(text) > 1 else []
        m = StopMatcher(stops)
        got = ""
        for piece in (text[a:b] for a, b in zip([0] + cuts, cuts + [len(text)])):
            emit, matched = m.push(piece)
            got += emit
            if matched is not None:
                break
        got += m.flush()
        assert (got, m.matched) == ((text[: want[0]], want[1]) if want else (text, None)), (stops, text, cuts)


def test_stop_matcher_never_emits_a_prefix_of_the_match_whatever_the_cut():
    import random
    rng = random.Random(5)
    text = "the quick brown fox STOP jumps over STO the lazy STOP dog"
    for _ in range(200):
        cuts = sorted(rng.sample(range(1, len(text)), rng.randrange(1, 12)))
        pieces = [text[a:b] for a, b in zip([0] + cuts, cuts + [len(text)])]
        m = StopMatcher(["STOP", "lazy"])
        got = ""
        for p in pieces:
            emit, matched = m.push(p)
            got += emit
            assert "STOP" not in got
            if matched:
                break
        assert got == "the quick brown fox " and matched == "STOP"


def test_incremental_detokenizer_waits_for_the_bytes_of_a_character():
    tok = ByteTokenizer()
    d = IncrementalDetokenizer(tok)
    deltas = [d.push(b) for b in "aé€z".encode()]
    assert "".join(deltas) == "aé€z" and deltas[1] == "" and "�" not in "".join(deltas)
    d = IncrementalDetokenizer(tok)
    assert [d.push(b) for b in b"a\xe2\x82"] == ["a", "", ""] and d.flush() == "�"   # the end came inside a character


def test_render_chat():
    text = render_chat([{"role": "system", "content": "s"}, {"role": "user", "content": "hi"}])
    assert text == "<|im_start|>system\ns<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    for bad in ([], [{"role": "user"}], [{"role": "wizard", "content": "x"}], [{"role": "user", "content": 3}]):
        with pytest.raises(ValueError):
            render_chat(bad)


# ------------------------------------------------------------------------------------------ text through the engine
def test_stop_strings_end_a_completion_and_are_cut_from_it(tiny_model_dirs, backend):
    kind, dtype = backend
    t = TINY["A"]
    model = H.make_model(tiny_model_dirs["A"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=32, max_sequences=4, max_tokens=64)
    tok = LetterTokenizer()
    prompt = tok.decode(H.random_ids(9, 256, 21))
    opts = GenerationOptions(max_output_tokens=24, ignore_eos=True)
    free = engine.complete_text(tok, prompt, opts)
    assert free.finish_reason == "length" and len(free.text) == 24 and free.completion_tokens == 24 and free.prompt_tokens == 9
    assert tok.encode(free.text) == engine.generate([tok.encode(prompt)], opts)[0].token_ids
    # a stop string from the middle of that text, spanning three tokens; a decoy that shares its first two characters
    # comes first in the list and never matches
    at = next(i for i in range(6, 20) if free.text.find(free.text[i : i + 3]) == i)
    stop = free.text[at : at + 3]
    decoy = stop[:2] + chr(0x100 + (ord(stop[2]) - 0x100 + 1) % 256)
    updates = list(engine.stream_text(tok, prompt, opts, stop=[decoy, stop]))
    text = "".join(u.text for u in updates)
    last = updates[-1]
    assert text == free.text[:at] and last.finish_reason == "stop" and last.stop_string == stop
    assert last.completion_tokens == at + 3                      # generation went on exactly until the match was whole
    assert all(u.finish_reason is None for u in updates[:-1])
    assert not engine.has_unfinished()                           # the request was cancelled
    assert all(p.free_count == p.capacity for p in engine.executor.cache.pools)
    # a stop string that never comes changes nothing but what is held back while it might
    never = engine.complete_text(tok, prompt, opts, stop=[free.text[-1] + "ĀĀĀ"])
    assert never.text == free.text and never.finish_reason == "length"
    # a stop token ends the text too, and is no part of it
    stop_id = tok.encode(free.text)[5]
    first = tok.encode(free.text).index(stop_id)
    by_token = engine.complete_text(tok, prompt, GenerationOptions(max_output_tokens=24, stop_token_ids=(stop_id,)))
    assert by_token.finish_reason == "stop" and by_token.text == free.text[:first] and by_token.stop_string is None
    with pytest.raises(RequestError):
        engine.complete_text(tok, "", opts)


def test_chat_renders_the_messages_and_stops_at_the_end_of_turn(tiny_model_dirs, backend):
    kind, dtype = backend
    t = TINY["A"]
    model = H.make_model(tiny_model_dirs["A"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=32, max_sequences=4, max_tokens=64)

    class Tok(LetterTokenizer):
        """Letters as above; every other character of the turn format maps into the vocabulary by its code."""

        def encode(self, text):
            return [(ord(c) - 0x100) if ord(c) >= 0x100 else ord(c) for c in text]

    tok = Tok()
    messages = [{"role": "user", "content": tok.decode([3, 1, 4, 1, 5])}]
    opts = GenerationOptions(max_output_tokens=12, ignore_eos=True)
    reply = engine.chat(tok, messages, opts)
    want = engine.generate([tok.encode(render_chat(messages))], opts)[0].token_ids
    assert reply.text == LetterTokenizer().decode(want) and reply.finish_reason == "length"
    cut = reply.text[4:6]
    stopped = engine.chat(tok, messages, opts, stop=[cut])
    assert stopped.text == reply.text[: reply.text.find(cut)] and stopped.finish_reason == "stop" and stopped.stop_string == cut


# ------------------------------------------------------------------------------------------ sampled generation against the plain sampler
def test_sampled_tokens_are_the_plain_samplers_for_the_same_seed_and_count(tiny_model_dirs, backend):
    """Teacher-forced along the engine's own tokens: at every step the plain sampler, fed the plain logits of the
    history with the request's seed and the number of tokens generated so far as the Philox offset, draws the engine's
    token, wherever its draw is not within 1e-3 of the kept mass from an edge of the token's interval and the kept set
    does not hinge on a near-tie at the top-p cut. A wrong offset (counted from one, or per step instead of per request)
    moves every draw."""
    kind, dtype = backend
    if dtype != torch.float32:
        pytest.skip("compared draw for draw: float32 only")
    t = TINY["B"]
    model = H.make_model(tiny_model_dirs["B"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=64, max_sequences=8, max_tokens=48)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 190 + n) for n in (3, 17, 40)]
    settings = [dict(temperature=0.8, top_p=0.9), dict(temperature=1.3, top_k=30), dict(temperature=0.6, top_p=0.95, min_p=0.02)]
    opts = [GenerationOptions(max_output_tokens=20, seed=4000 + i, ignore_eos=True, **s) for i, s in enumerate(settings)]
    outs = engine.generate(prompts, opts)
    cfg, w = plain.load_model_dir(tiny_model_dirs["B"])
    compared = 0
    for prompt, o, out in zip(prompts, opts, outs):
        seq = list(prompt)
        for n, tok in enumerate(out.token_ids):
            logits = plain.forward_logits(cfg, w, seq)[-1]
            sp = o.sampling()
            want, detail = plain.sample_row(logits.tolist(), sp.temperature, sp.top_k, sp.top_p, sp.min_p, o.seed, n, return_detail=True)
            # the same draw with the cut moved by a hair: if the kept set changes, the cut is a near-tie and proves nothing
            lo = plain.sample_row(logits.tolist(), sp.temperature, sp.top_k, max(sp.top_p - 1e-4, 1e-6), sp.min_p * (1 + 1e-3), o.seed, n)
            hi = plain.sample_row(logits.tolist(), sp.temperature, sp.top_k, min(sp.top_p + 1e-4, 1.0), sp.min_p * (1 - 1e-3), o.seed, n)
            if detail["margin"] > 1e-3 and lo == want == hi:
                assert tok == want, f"token {n}: engine {tok}, plain {want} (margin {detail['margin']:.2e})"
                compared += 1
            seq.append(tok)
    assert compared >= 40, compared


# ------------------------------------------------------------------------------------------ a step that raises
def test_a_step_that_raises_leaves_the_engine_usable_and_the_tokens_unchanged(tiny_model_dirs):
    """The forward pass raises once in the middle of a generation (as a kernel error would): the error reaches the
    caller, nothing of the failed plan is applied, and the generation, carried on, gives the tokens of an undisturbed
    run. The same when the failure comes after the step function has committed its rows (the status check that follows
    the tokens): those requests are recomputed."""
    t = TINY["A"]
    model = H.make_model(tiny_model_dirs["A"], torch.float32, "fake")
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 60 + n) for n in (21, 9, 14)]
    opts = GenerationOptions(max_output_tokens=10, ignore_eos=True)
    want = [o.token_ids for o in RoostEngine(model, page_size=16, attention_blocks=32, max_sequences=4, max_tokens=16).generate(prompts, opts)]

    for fail_after_commit in (False, True):
        engine = RoostEngine(model, page_size=16, attention_blocks=32, max_sequences=4, max_tokens=16)
        rids = [engine.add_request(p, opts.sampling()) for p in prompts]
        got = {r: [] for r in rids}
        calls = {"n": 0}
        if fail_after_commit:
            orig = engine.sampler.__call__

            def flaky(logits, rows, orig=engine.sampler):
                calls["n"] += 1
                if calls["n"] == 4:
                    raise RuntimeError("injected failure after the step")
                return type(orig).__call__(orig, logits, rows)

            engine.sampler = flaky
        else:
            orig_forward = model.forward

            def flaky_forward(batch, storage):
                calls["n"] += 1
                if calls["n"] == 4:
                    raise RuntimeError("injected failure in the step")
                return orig_forward(batch, storage)

            model.forward = flaky_forward
        raised = 0
        try:
            for _ in range(200):
                if not engine.has_unfinished():
                    break
                try:
                    events = engine.step()
                except RuntimeError as e:
                    assert "injected" in str(e)
                    raised += 1
                    engine.executor.cache.check_invariants()
                    continue
                for e in events:
                    if e.token is not None:
                        got[e.request_id].append(e.token)
        finally:
            model.forward = type(model).forward.__get__(model)
        assert raised == 1
        assert [got[r] for r in rids] == want
        assert all(p.free_count == p.capacity for p in engine.executor.cache.pools)
