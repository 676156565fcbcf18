"""Shared test helpers: building an executor over a backend, trace drivers, comparison metrics."""
from __future__ import annotations

import random

import torch

from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.engine.model import Model, parameter_declarations, read_model_config
from roost_b200.parts import Runtime
from roost_b200.weights import loader
from tests.plain import qwen3_plain as plain


def make_model(model_dir, dtype, backend: str):
    """backend "gpu": the real kernel library on cuda:0; "fake": tests/fake_kernels on the CPU."""
    arch, cfg, _ = read_model_config(model_dir)
    tied = cfg.tie_word_embeddings
    if tied is None:
        tied = not loader.checkpoint_has(model_dir, "lm_head.weight")
    spec = arch.to_spec(cfg, tied)
    if backend == "gpu":
        from roost_b200.kernels import library
        rt = Runtime(dtype, "cuda", library.load())
    else:
        from tests.fake_kernels import FakeKernels
        rt = Runtime(dtype, "cpu", FakeKernels())
    model = Model(spec, rt)
    allow = ("lm_head.weight",) if spec.tie_embeddings else ()
    model.load(loader.load_checkpoint(model_dir, parameter_declarations(spec), spec.weight_names, allow_unexpected=allow))
    return model


def plain_logits(model_dir, ids, bf16: bool, schedule=None) -> torch.Tensor:
    cfg, w = plain.load_model_dir(model_dir)
    if bf16:  # the engine keeps matrices in bfloat16; vectors stay as they are stored
        w = {k: (v.to(torch.bfloat16).to(torch.float64) if v.dim() >= 2 else v) for k, v in w.items()}
    return plain.forward_logits(cfg, w, ids, schedule)


def scaled_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """The reference's metric: worst |got - want| / (1 + |want|) over a block of logits
    (tests/Starlings.Roost.Models.Tiny.Tests/RoostTinyTests.cs:18-29)."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    return float(((got - want).abs() / (1 + want.abs())).max())


# Bounds. float32: the reference holds its float32 model to 1e-5 against a double implementation
# (tests/Starlings.Roost.Models.Tiny.Tests/Support/Tolerances.cs:10); device sums run in float32, so 2e-5.
# bfloat16: every op output is rounded to 8 bits of mantissa (up to 2^-8 relative each); a token passes through about a
# dozen roundings a layer, which add like a random walk: about 1 % of the logits' size is the expected error and, as
# the worst of tens of thousands of logits, three to four times that (measured on the tiny models: 1.4e-2 to 3.7e-2,
# growing with the number of logits compared). Two bounds therefore: the worst scaled error below 2^-4, and the
# root-mean-square error below 2^-6 of the logits' root mean square, which a misplaced key or page breaks at once
# (such faults move logits by tens of percent) and which does not grow with the sample size.
FP32_BOUND = 2e-5
BF16_BOUND = 2.0 ** -4
BF16_RMS_BOUND = 2.0 ** -6


def rms_error(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())


def bound_for(dtype) -> float:
    return FP32_BOUND if dtype == torch.float32 else BF16_BOUND


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def run_whole(ex: StepExecutor, rid, ids) -> torch.Tensor:
    out = ex.step([StepEntry(rid, list(ids), list(range(len(ids))))])
    ex.finish(rid)
    return out


def run_tail_decoded(ex: StepExecutor, rid, ids, tail: int = 32) -> torch.Tensor:
    """All but the last ``tail`` tokens in one step, then one token a step."""
    n = len(ids)
    head = max(1, n - tail)
    outs = [ex.step([StepEntry(rid, list(ids[:head]), list(range(head)))])]
    for i in range(head, n):
        outs.append(ex.step([StepEntry(rid, [ids[i]], [0])]))
    ex.finish(rid)
    return torch.cat(outs)


def run_portions(ex: StepExecutor, rid, ids, sizes) -> torch.Tensor:
    """Portions of changing size (cycled), down to two tokens."""
    outs, at, i = [], 0, 0
    while at < len(ids):
        n = min(sizes[i % len(sizes)], len(ids) - at)
        outs.append(ex.step([StepEntry(rid, list(ids[at : at + n]), list(range(n)))]))
        at += n
        i += 1
    ex.finish(rid)
    return torch.cat(outs)


def run_mixed(ex: StepExecutor, requests: dict, seed: int, max_live: int = 4, decode_tail: int = 8):
    """Replays several requests with up to ``max_live`` live at a time: each request is fed in random portions, its
    last ``decode_tail`` tokens one by one, beside whatever the other live requests bring in the same step. A request
    that ends gives its pages back and the next one starts at once, so pages are used again. Returns {id: logits}."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}
    outs = {rid: [] for rid in requests}
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0]
        entries, ended = [], []
        chosen = [rid for rid in live if rng.random() < 0.8] or [next(iter(live))]
        for rid in chosen:
            ids, at = live[rid]
            left = len(ids) - at
            n = 1 if left <= decode_tail else min(left - decode_tail, rng.choice([2, 3, 5, 7, 16, 33]))
            if n == 1 and left > decode_tail:
                n = min(2, left)
            entries.append(StepEntry(rid, list(ids[at : at + n]), list(range(n))))
            live[rid][1] = at + n
        logits = ex.step(entries)
        at = 0
        for e in entries:
            n = len(e.tokens)
            outs[e.request_id].append(logits[at : at + n])
            at += n
            if live[e.request_id][1] == len(live[e.request_id][0]):
                ended.append(e.request_id)
        for rid in ended:
            ex.finish(rid)
            del live[rid]
        ex.cache.check_invariants()
    return {rid: torch.cat(v) for rid, v in outs.items()}
