"""Generation through the entry point, each part alone, run orders that name a layer twice or share a cache, and a toy
mixer with state of its own that is registered, built and stepped without a change to the framework's files."""
import math
from dataclasses import dataclass

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.config.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, RunEntry)
from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.engine.model import Model, parameter_declarations
from roost_b200.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheNeed, Linear, Mixer, ParamDecl, Runtime, register_mixer)
from roost_b200.weights import loader
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


def runtime(backend) -> Runtime:
    kind, dtype = backend
    if kind == "gpu":
        from roost_b200.kernels import library
        return Runtime(dtype, "cuda", library.load())
    from tests.fake_kernels import FakeKernels
    return Runtime(dtype, "cpu", FakeKernels())


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tiny_model_dirs, backend, name):
    kind, dtype = backend
    t = TINY[name]
    model = H.make_model(tiny_model_dirs[name], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=64, max_sequences=4, max_tokens=24)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 70 + n) for n in (7, 19, 33)]
    outs = engine.generate(prompts, GenerationOptions(max_output_tokens=16, ignore_eos=True))
    cfg, w = plain.load_model_dir(tiny_model_dirs[name])
    if dtype == torch.bfloat16:
        w = {k: (v.to(torch.bfloat16).double() if v.dim() >= 2 else v) for k, v in w.items()}
    for prompt, out in zip(prompts, outs):
        assert out.finish_reason == "length" and len(out.token_ids) == 16 and out.prompt_tokens == len(prompt)
        # teacher-forced comparison: at every step the engine's token is the plain implementation's choice for the
        # engine's own history, unless the plain top two are a near-tie
        seq = list(prompt)
        for tok in out.token_ids:
            logits = plain.forward_logits(cfg, w, seq)[-1]
            top = logits.topk(2)
            gap = float(top.values[0] - top.values[1])
            if gap > (1e-3 if dtype == torch.float32 else 0.15):
                assert tok == int(top.indices[0]), f"step {len(seq) - len(prompt)}: engine {tok}, plain {int(top.indices[0])} (gap {gap:.3g})"
            seq.append(tok)
    assert engine.executor.cache.pools[0].free_count == 64       # every page came back
    if kind == "gpu":
        # decode steps replayed captured graphs, most of them with tables made while the step before was still running
        assert engine.executor.graph_replays > 0 and engine.executor.prepared_replays > 0
    # the same prompts one at a time give the same tokens as the batch did
    alone = [engine.generate([p], GenerationOptions(max_output_tokens=16, ignore_eos=True))[0].token_ids for p in prompts]
    if dtype == torch.float32:
        assert alone == [o.token_ids for o in outs]


def test_sampled_generation_is_seeded_and_stops(tiny_model_dirs, backend):
    kind, dtype = backend
    t = TINY["B"]
    model = H.make_model(tiny_model_dirs["B"], dtype, kind)
    engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=64, max_sequences=8, max_tokens=64)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 90 + n) for n in (1, 4, 17, 40, 64)]
    opts = [GenerationOptions(max_output_tokens=24, temperature=0.8, top_p=0.9, seed=1000 + i) for i in range(5)]
    a = engine.generate(prompts, opts)
    b = engine.generate(prompts, opts)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]
    # every token is the plain sampler's choice on the plain logits of the engine's own history, with the request's seed
    # and the number of tokens generated so far as the offset, unless the draw falls within 1e-4 of the kept mass from an
    # edge of the token's interval (a counter that started at 1, or a seed of another row, would show at once)
    cfg, w = plain.load_model_dir(tiny_model_dirs["B"])
    if dtype == torch.float32:
        compared = 0
        for i, (prompt, out) in enumerate(zip(prompts, a)):
            seq = list(prompt)
            for j, tok in enumerate(out.token_ids):
                logits = plain.forward_logits(cfg, w, seq)[-1]
                want, detail = plain.sample_row(logits.tolist(), 0.8, 0, 0.9, 0.0, 1000 + i, j, return_detail=True)
                if detail["margin"] > 1e-4:
                    assert tok == want, f"request {i}, token {j}: engine {tok}, plain {want} (margin {detail['margin']:.2e})"
                    compared += 1
                seq.append(tok)
        assert compared >= 0.8 * sum(len(o.token_ids) for o in a), compared
    c = engine.generate(prompts[2:3], opts[2:3])                 # alone: the draw does not depend on the batch
    if dtype == torch.float32:
        assert c[0].token_ids == a[2].token_ids
    other = engine.generate(prompts[2:3], [GenerationOptions(max_output_tokens=24, temperature=0.8, top_p=0.9, seed=5)])
    assert other[0].token_ids != a[2].token_ids
    # the model's stop ids (eos_token_id of config.json) end a request with "stop" unless ignored
    assert all(o.finish_reason in ("stop", "length") for o in a)
    for o in a:
        if o.finish_reason == "stop":
            assert o.token_ids[-1] in (5, 7) and not any(x in (5, 7) for x in o.token_ids[:-1])
    stop = a[3].token_ids[2]
    s = engine.generate(prompts[3:4], [GenerationOptions(max_output_tokens=24, temperature=0.8, top_p=0.9, seed=1003, stop_token_ids=(stop,))])
    assert s[0].finish_reason == "stop" and s[0].token_ids == a[3].token_ids[: a[3].token_ids.index(stop) + 1]
    updates = list(engine.stream_completion(prompts[1], GenerationOptions(max_output_tokens=5, ignore_eos=True)))
    assert [u.completion_tokens for u in updates] == [1, 2, 3, 4, 5] and updates[-1].finish_reason == "length"


def test_generation_with_preemption_gives_the_same_tokens(tiny_model_dirs, backend):
    kind, dtype = backend
    if dtype != torch.float32:
        pytest.skip("compared token for token: float32 only")
    t = TINY["A"]
    model = H.make_model(tiny_model_dirs["A"], dtype, kind)
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 30 + n) for n in (30, 28, 26)]
    opt = GenerationOptions(max_output_tokens=30, ignore_eos=True)
    roomy = RoostEngine(model, page_size=16, attention_blocks=64, max_sequences=4, max_tokens=64)
    want = [o.token_ids for o in roomy.generate(prompts, opt)]
    tight = RoostEngine(model, page_size=16, attention_blocks=9, max_sequences=4, max_tokens=64)   # 144 tokens for 3 x ~60
    got = [o.token_ids for o in tight.generate(prompts, opt)]
    assert tight.stats()["preemptions"] > 0, "the pool is too large for this test"
    assert got == want
    tight.executor.cache.check_invariants()


# ------------------------------------------------------------------------------------------ each part alone
def test_norm_part_alone(backend):
    rt = runtime(backend)
    norm = NORMS.build(NormSpec(size=72, eps=1e-5), rt)
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.1 * torch.randn(72, generator=g)
    x = torch.randn(5, 72, generator=g).to(rt.dtype)
    res = torch.randn(5, 72, generator=g).to(rt.dtype)
    norm.load({"weight": w.to(rt.device)})
    y = norm(x.to(rt.device))
    want = plain.rms_norm(x.double(), w.double(), 1e-5)
    assert H.scaled_error(y, want) < (2e-6 if rt.full_precision else 2 ** -7)
    y2, r2 = norm.add_norm(x.to(rt.device), res.to(rt.device).clone())
    s = (x.float() + res.float()).to(rt.dtype)
    assert torch.equal(r2.cpu(), s)
    assert H.scaled_error(y2, plain.rms_norm(s.double(), w.double(), 1e-5)) < (2e-6 if rt.full_precision else 2 ** -7)


def test_feed_forward_part_alone(backend):
    rt = runtime(backend)
    spec = GatedMlpSpec(hidden=40, intermediate=104)
    ff = FEED_FORWARDS.build(spec, rt)
    g = torch.Generator().manual_seed(1)
    gate_up = (torch.randn(208, 40, generator=g) * 0.2).to(rt.dtype)
    down = (torch.randn(40, 104, generator=g) * 0.2).to(rt.dtype)
    ff.load({"gate_up": gate_up.to(rt.device), "down": down.to(rt.device)})
    x = torch.randn(9, 40, generator=g).to(rt.dtype)
    want = plain.swiglu_mlp(x.double(), gate_up[:104].double(), gate_up[104:].double(), down.double())
    assert H.scaled_error(ff(x.to(rt.device), None), want) < (5e-6 if rt.full_precision else 2 ** -5)
    assert FEED_FORWARDS.get("gated_mlp").parameters(spec)["gate_up"].row_splits == (104, 104)
    with pytest.raises(ValueError, match="activation"):
        FEED_FORWARDS.build(GatedMlpSpec(hidden=8, intermediate=8, activation="gelu"), rt)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [3, 40, 300])
def test_feed_forward_part_on_the_interleaved_layout(rows):
    """An intermediate size of a multiple of 128 stores gate and up in blocks of 128; few rows take the product split over
    clusters, more the library product and the SiLU kernel, many the fused tensor-core product (made to here: by its own
    rule it starts at larger products). All are the same function."""
    rt = runtime(("gpu", torch.bfloat16))
    spec = GatedMlpSpec(hidden=136, intermediate=256)
    g = torch.Generator().manual_seed(2)
    gate_up = (torch.randn(512, 136, generator=g) * 0.1).to(rt.dtype)
    down = (torch.randn(136, 256, generator=g) * 0.1).to(rt.dtype)
    x = torch.randn(rows, 136, generator=g).to(rt.dtype)
    want = plain.swiglu_mlp(x.double(), gate_up[:256].double(), gate_up[256:].double(), down.double())
    outs = []
    for work in (None, 0.0):
        ff = FEED_FORWARDS.build(spec, rt)
        assert ff.interleave == 128
        if work is not None:
            ff.fused_min_work = work
        ff.load({"gate_up": gate_up.to(rt.device), "down": down.to(rt.device)})
        outs.append(ff(x.to(rt.device), None))
        assert H.scaled_error(outs[-1], want) < 2 ** -5
    if rows < 256:
        assert torch.equal(outs[0], outs[1])      # the threshold moves nothing below the fused product's rows


def attention_spec(window=None, position=True):
    return AttentionSpec(hidden=48, num_heads=6, num_kv_heads=2, head_dim=16, scale=0.25, window=window,
                         qk_norm=NormSpec(size=16, eps=1e-6), position=PositionSpec(rotary_dim=16, theta=1e4) if position else None)


@pytest.mark.parametrize("window", [None, 9])
def test_attention_mixer_alone_whole_and_in_portions(backend, window):
    """The mixer as a one-part model: pages, rotation and window through the step function, against the plain mixer."""
    rt = runtime(backend)
    spec = attention_spec(window)
    mixer = MIXERS.build(spec, rt)
    g = torch.Generator().manual_seed(2)
    qkv = (torch.randn(160, 48, generator=g) * 0.3).to(rt.dtype)
    out = (torch.randn(48, 96, generator=g) * 0.2).to(rt.dtype)
    qn, kn = 1 + 0.1 * torch.randn(16, generator=g), 1 + 0.1 * torch.randn(16, generator=g)
    mixer.load({"qkv": qkv.to(rt.device), "out": out.to(rt.device), "q_norm": qn.to(rt.device), "k_norm": kn.to(rt.device)})
    assert mixer.cache_need() == CacheNeed("paged", kv_heads=2, head_dim=16, window=window)
    T = 37
    x = torch.randn(T, 48, generator=g).to(rt.dtype)
    w = {"q_proj.weight": qkv[:96].double(), "k_proj.weight": qkv[96:128].double(), "v_proj.weight": qkv[128:].double(),
         "o_proj.weight": out.double(), "q_norm.weight": qn.double(), "k_norm.weight": kn.double()}
    cfg = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4)
    want, _ = plain.attention_mixer(x.double(), list(range(T)), w, "", cfg, window)

    from roost_b200.cache.manager import CacheManager, build_groups
    from roost_b200.cache.storage import CacheStorage
    from roost_b200.engine.batch import BatchBuilder
    groups = build_groups([mixer.cache_need()], page_size=4)
    cm = CacheManager(groups, [12, 2])
    storage = CacheStorage(groups, [12, 2], rt.dtype, rt.device)
    builder = BatchBuilder(rt.device, cm)
    outs, at = [], 0
    for n in (11, 2, 24):
        rc = cm.extend("r", at + n)
        batch = builder.build([(rc, at, [0] * n, [])], vocab=1)
        outs.append(mixer(x[at : at + n].to(rt.device), batch, storage.view(0)))
        at += n
        cm.commit("r", at)
    assert H.scaled_error(torch.cat(outs), want) < (5e-6 if rt.full_precision else 2 ** -5)


def test_parts_refuse_sizes_no_kernel_serves(backend):
    rt = runtime(backend)
    with pytest.raises(ValueError, match="multiple"):
        MIXERS.build(AttentionSpec(hidden=8, num_heads=3, num_kv_heads=2, head_dim=16, scale=1.0), rt)
    with pytest.raises(ValueError, match="head_dim"):
        MIXERS.build(AttentionSpec(hidden=8, num_heads=2, num_kv_heads=1, head_dim=1024, scale=1.0), rt)
    with pytest.raises(KeyError, match="registered"):
        MIXERS.build(MixerSpec(kind="nonesuch"), rt)
    with pytest.raises(ValueError):
        NORMS.build(NormSpec(size=8, eps=0.0), rt)


# ------------------------------------------------------------------------------------------ run order as data
@pytest.mark.parametrize("schedule", [[(0, None), (1, None), (0, None)], [(0, None), (1, None), (0, 0), (1, 1)], [(1, None), (0, None)]])
def test_a_layer_may_run_twice_or_read_another_runs_cache(tiny_model_dirs, backend, schedule):
    kind, dtype = backend
    from dataclasses import replace
    model_dir = tiny_model_dirs["A"]
    base = H.make_model(model_dir, dtype, kind)
    spec = replace(base.spec, schedule=tuple(RunEntry(b, r) for b, r in schedule))
    model = Model(spec, base.rt)
    allow = ("lm_head.weight",)
    model.load(loader.load_checkpoint(model_dir, parameter_declarations(spec), spec.weight_names, allow_unexpected=allow))
    ex = StepExecutor(model, page_size=16, num_pages=16, max_requests=2)
    owners = [i for i, (_, r) in enumerate(schedule) if r is None]
    assert ex.groups[0].runs == tuple(owners)                    # a run that reads another's cache keeps none
    ids = H.random_ids(41, 256, 5)
    want = H.plain_logits(model_dir, ids, bf16=dtype == torch.bfloat16, schedule=schedule)
    got = H.run_portions(ex, "r", ids, [17, 2, 9])
    assert H.scaled_error(got, want) < H.bound_for(dtype)
    got = H.run_tail_decoded(ex, "r", ids, tail=8)
    assert H.scaled_error(got, want) < H.bound_for(dtype)


# ------------------------------------------------------------------------------------------ a toy mixer with state of its own
@dataclass(frozen=True)
class ToyStateSpec(MixerSpec):
    kind: str = "toy_running_mean"
    hidden: int = 0
    decay: float = 0.5


class ToyRunningMean(Mixer):
    """state <- decay * state + (1 - decay) * (x W^T), token by token; the output is the state. The state is one
    vector per live request, kept in a slot of the cache manager's fixed-size state group between steps."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.proj = Linear(rt, spec.hidden, spec.hidden)

    @classmethod
    def parameters(cls, spec):
        return {"proj": ParamDecl(shape=(spec.hidden, spec.hidden))}

    def load(self, params):
        self.proj.load(params["proj"])

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.spec.hidden,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache=True):
        u = self.proj(x).float()
        out = torch.empty_like(u)
        slots = batch.groups[cache.group].state_slots.tolist()
        at = 0
        for b, n in enumerate(batch.row_counts):
            s = cache.state[slots[b]].clone()
            for i in range(n):
                s = self.spec.decay * s + (1 - self.spec.decay) * u[at + i]
                out[at + i] = s
            cache.state[slots[b]] = s
            at += n
        return out.to(x.dtype)


class ToyRunningMeanOnDevice(ToyRunningMean):
    """The same mixer written over the step's device tables alone (``token_row``, ``positions``, ``q_indptr``,
    ``state_slots``): no value is read on the host and the launches do not depend on the rows, so the mixer may say
    ``state_capturable`` and its model's steps are captured and replayed like any other's. The scan over a row's tokens
    is a product with a [T, T] matrix of decay powers between tokens of the same row."""
    state_capturable = True

    def __call__(self, x, batch, cache, write_cache=True):
        d = self.spec.decay
        u = self.proj(x).float()                                           # [T, H]
        tables = batch.groups[cache.group]
        row = batch.token_row.long()
        pos = batch.positions.float()
        first = batch.q_indptr[:-1].long().clamp(max=max(batch.num_tokens - 1, 0))
        idx = torch.arange(batch.num_tokens, device=u.device)
        same = (row[:, None] == row[None, :]) & (idx[None, :] <= idx[:, None])
        # (a scalar base: a tensor made from a host value inside a captured step would be a copy from pageable memory)
        w = torch.where(same, (1 - d) * torch.pow(d, (pos[:, None] - pos[None, :]).clamp(min=0)), torch.zeros((), device=u.device))
        slots = tables.state_slots.long()
        before = cache.state.index_select(0, slots)                        # [B, H]
        carried = torch.pow(d, pos - pos[first][row] + 1)[:, None] * before[row]
        out = w @ u + carried
        last = (batch.q_indptr[1:].long() - 1).clamp(min=0)
        cache.state.index_copy_(0, slots, out.index_select(0, last))      # padding rows write the scratch slot
        return out.to(x.dtype)


def toy_plain(x, w, decay):
    u = x @ w.T
    s = torch.zeros(w.shape[0], dtype=torch.float64)
    out = []
    for t in range(x.shape[0]):
        s = decay * s + (1 - decay) * u[t]
        out.append(s)
    return torch.stack(out)


@pytest.mark.parametrize("written", ["as a loop over the rows", "over the device tables"])
def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped(backend, written):
    register_mixer("toy_running_mean", ToyRunningMean if written == "as a loop over the rows" else ToyRunningMeanOnDevice)
    rt = runtime(backend)
    H_, V, I = 32, 50, 48
    norm = NormSpec(size=H_, eps=1e-6)
    attn = AttentionSpec(hidden=H_, num_heads=2, num_kv_heads=1, head_dim=16, scale=0.25, qk_norm=None,
                         position=PositionSpec(rotary_dim=16, theta=100.0))
    ff = GatedMlpSpec(hidden=H_, intermediate=I)
    blocks = (BlockSpec(mixer=ToyStateSpec(hidden=H_, decay=0.75), feed_forward=ff, input_norm=norm, post_mixer_norm=norm),
              BlockSpec(mixer=attn, feed_forward=ff, input_norm=norm, post_mixer_norm=norm))
    spec = ModelSpec(architecture="ToyForTests", hidden=H_, vocab=V, blocks=blocks, schedule=(RunEntry(0), RunEntry(1), RunEntry(0)),
                     final_norm=norm, tie_embeddings=True, max_positions=0)
    model = Model(spec, rt)
    assert [n.kind if n else None for n in model.cache_needs] == ["state", "paged", "state"]
    g = torch.Generator().manual_seed(3)
    params = {}
    for scope, decl in parameter_declarations(spec).items():
        params[scope] = {k: (torch.ones(d.shape) if d.role == "vector" else torch.randn(d.shape, generator=g) * 0.2).to(rt.dtype) for k, d in decl.items()}
    model.load(params)
    ex = StepExecutor(model, page_size=4, num_pages=40, max_requests=3)
    assert [(g_.kind, g_.runs) for g_ in ex.groups] == [("paged", (1,)), ("state", (0, 2))]

    def plain_forward(ids):
        P = {s: {k: v.double() for k, v in p.items()} for s, p in params.items()}
        h = P["embed"]["table"][torch.tensor(ids)]
        pos = list(range(len(ids)))
        for bi in (0, 1, 0):
            x = plain.rms_norm(h, P[f"blocks.{bi}.input_norm"]["weight"], 1e-6)
            if bi == 0:
                mix = toy_plain(x, P["blocks.0.mixer"]["proj"], 0.75)
            else:
                qkv = P["blocks.1.mixer"]["qkv"]
                q = plain.rope_neox((x @ qkv[:32].T).reshape(-1, 2, 16), pos, 100.0)
                k = plain.rope_neox((x @ qkv[32:48].T).reshape(-1, 1, 16), pos, 100.0)
                v = (x @ qkv[48:].T).reshape(-1, 1, 16)
                mix = plain.causal_gqa_attention(q, k, v, 0.25).reshape(-1, 32) @ P["blocks.1.mixer"]["out"].T
            h = h + mix
            y = plain.rms_norm(h, P[f"blocks.{bi}.post_mixer_norm"]["weight"], 1e-6)
            gu = P[f"blocks.{bi}.feed_forward"]["gate_up"]
            h = h + plain.swiglu_mlp(y, gu[:I], gu[I:], P[f"blocks.{bi}.feed_forward"]["down"])
        return plain.rms_norm(h, P["final_norm"]["weight"], 1e-6) @ P["embed"]["table"].T

    a, b = H.random_ids(23, V, 1), H.random_ids(15, V, 2)
    bound = 2e-5 if rt.full_precision else H.BF16_BOUND
    got = H.run_mixed(ex, {"a": a, "b": b}, seed=3, max_live=2, decode_tail=4)
    assert H.scaled_error(got["a"], plain_forward(a)) < bound
    assert H.scaled_error(got["b"], plain_forward(b)) < bound
    # a slot that is used again starts from zero: the next request does not see the last one's state
    got = H.run_portions(ex, "c", b, [4, 2, 9])
    assert H.scaled_error(got, plain_forward(b)) < bound
    assert ex.cache.pools[1].free_count == 3
    # The mixer written as a Python loop keeps its model's steps eager; the one written over the device tables lets them
    # be captured: single-token steps replay a graph (the fresh slot is zeroed inside it, padding rows write the scratch
    # slot), three requests beside each other in the captured step of three rows, one of them ending early.
    captured = backend[0] == "gpu" and written == "over the device tables"
    assert ex.use_graphs == captured
    replays0 = ex.graph_replays
    got = H.run_tail_decoded(ex, "d", a, tail=12)
    assert H.scaled_error(got, plain_forward(a)) < bound
    seqs = {"x": a[:9], "y": b[:14], "z": a[5:17]}
    outs = {r: [] for r in seqs}
    for i in range(14):
        live = [r for r, ids in seqs.items() if i < len(ids)]
        logits = ex.step([StepEntry(r, [seqs[r][i]], [0]) for r in live])
        for r, row in zip(live, logits):
            outs[r].append(row)
        for r in live:
            if i == len(seqs[r]) - 1:
                ex.finish(r)
    for r, ids in seqs.items():
        assert H.scaled_error(torch.stack(outs[r]), plain_forward(ids)) < bound, r
    assert (ex.graph_replays - replays0 >= 15) == captured
    assert ex.cache.pools[1].free_count == 3


# ------------------------------------------------------------------------------------------ a toy mixer with a latent in pages
@dataclass(frozen=True)
class ToyLatentSpec(MixerSpec):
    kind: str = "toy_latent_mean"
    hidden: int = 0
    latent: int = 0
    window: int | None = None


class ToyLatentMean(Mixer):
    """Keeps ONE vector a token in the paged cache (c_t = x_t Wc^T, `latent` wide: a cache group of one plane) and gives
    out the mean of the cached vectors a token sees (all earlier ones and its own, or the last `window`), projected back:
    out_t = mean_s(c_s) Wo^T. Written with host loops over the step's tables, so its model's steps run eagerly."""
    capturable = False

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.down = Linear(rt, spec.latent, spec.hidden)
        self.up = Linear(rt, spec.hidden, spec.latent)

    @classmethod
    def parameters(cls, spec):
        return {"down": ParamDecl(shape=(spec.latent, spec.hidden)), "up": ParamDecl(shape=(spec.hidden, spec.latent))}

    def load(self, params):
        self.down.load(params["down"])
        self.up.load(params["up"])

    def cache_need(self):
        return CacheNeed("paged", kv_heads=1, head_dim=self.spec.latent, window=self.spec.window, planes=1)

    def __call__(self, x, batch, cache, write_cache=True):
        assert cache.v_pool is None and cache.k_pool.shape[1:] == (1, cache.page_size, self.spec.latent)
        tables = batch.groups[cache.group]
        c = self.down(x)
        pool = cache.k_pool.view(-1, self.spec.latent)                     # [pages * page_size, latent]: slot = page * page_size + offset
        if write_cache:
            pool[tables.slot_mapping.long()] = c
        indptr, pages = tables.kv_indptr.tolist(), tables.kv_indices.tolist()
        P, out, at = cache.page_size, [], 0
        for b, n in enumerate(batch.row_counts):
            kv_len = int(batch.kv_lens[b])
            mine = pages[indptr[b]:indptr[b + 1]]
            for i in range(n):
                pos = kv_len - n + i
                lo = max(0, pos - self.spec.window + 1) if self.spec.window else 0
                slots = [mine[j // P] * P + j % P for j in range(lo, pos + 1)]
                assert min(slots) >= 0, "a page the window has passed was read"
                out.append(pool[torch.tensor(slots, device=pool.device)].float().mean(0))
            at += n
        return self.up(torch.stack(out).to(x.dtype))


@pytest.mark.parametrize("window", [None, 6])
def test_a_toy_mixer_that_keeps_one_latent_vector_a_token_in_pages(backend, window):
    """A paged cache group need not hold keys and values: a mixer asks for one plane, gets pages, block tables and slots
    from the same cache manager (window release included) and shares nothing with the attention layer's group."""
    register_mixer("toy_latent_mean", ToyLatentMean)
    rt = runtime(backend)
    H_, V, I, L = 32, 40, 48, 24
    norm = NormSpec(size=H_, eps=1e-6)
    attn = AttentionSpec(hidden=H_, num_heads=2, num_kv_heads=1, head_dim=16, scale=0.25, qk_norm=None,
                         position=PositionSpec(rotary_dim=16, theta=100.0))
    ff = GatedMlpSpec(hidden=H_, intermediate=I)
    blocks = (BlockSpec(mixer=ToyLatentSpec(hidden=H_, latent=L, window=window), feed_forward=ff, input_norm=norm, post_mixer_norm=norm),
              BlockSpec(mixer=attn, feed_forward=ff, input_norm=norm, post_mixer_norm=norm))
    spec = ModelSpec(architecture="ToyLatentForTests", hidden=H_, vocab=V, blocks=blocks, schedule=(RunEntry(0), RunEntry(1)),
                     final_norm=norm, tie_embeddings=True, max_positions=0)
    model = Model(spec, rt)
    g = torch.Generator().manual_seed(13)
    params = {}
    for scope, decl in parameter_declarations(spec).items():
        params[scope] = {k: (torch.ones(d.shape) if d.role == "vector" else torch.randn(d.shape, generator=g) * 0.2).to(rt.dtype) for k, d in decl.items()}
    model.load(params)
    ex = StepExecutor(model, page_size=4, num_pages=24, max_requests=3)
    kinds = [(g_.kind, g_.planes if g_.kind == "paged" else 0, g_.window, g_.runs) for g_ in ex.groups]
    assert kinds[:2] == [("paged", 1, window, (0,)), ("paged", 2, None, (1,))] and not ex.use_graphs
    assert ex.storage.tensors[0].shape[:2] == (1, 1) and ex.storage.tensors[1].shape[:2] == (1, 2)

    def plain_forward(ids):
        P = {s_: {k: v.double() for k, v in p_.items()} for s_, p_ in params.items()}
        h = P["embed"]["table"][torch.tensor(ids)]
        pos = list(range(len(ids)))
        for bi in (0, 1):
            x = plain.rms_norm(h, P[f"blocks.{bi}.input_norm"]["weight"], 1e-6)
            if bi == 0:
                c = x @ P["blocks.0.mixer"]["down"].T
                if rt.dtype == torch.bfloat16:
                    c = c.to(torch.bfloat16).double()       # the cache holds the latent in the compute dtype
                means = torch.stack([c[max(0, t - window + 1) if window else 0 : t + 1].mean(0) for t in pos])
                mix = means @ P["blocks.0.mixer"]["up"].T
            else:
                qkv = P["blocks.1.mixer"]["qkv"]
                q = plain.rope_neox((x @ qkv[:32].T).reshape(-1, 2, 16), pos, 100.0)
                k = plain.rope_neox((x @ qkv[32:48].T).reshape(-1, 1, 16), pos, 100.0)
                v = (x @ qkv[48:].T).reshape(-1, 1, 16)
                mix = plain.causal_gqa_attention(q, k, v, 0.25).reshape(-1, 32) @ P["blocks.1.mixer"]["out"].T
            h = h + mix
            y = plain.rms_norm(h, P[f"blocks.{bi}.post_mixer_norm"]["weight"], 1e-6)
            gu = P[f"blocks.{bi}.feed_forward"]["gate_up"]
            h = h + plain.swiglu_mlp(y, gu[:I], gu[I:], P[f"blocks.{bi}.feed_forward"]["down"])
        return plain.rms_norm(h, P["final_norm"]["weight"], 1e-6) @ P["embed"]["table"].T

    a, b = H.random_ids(26, V, 5), H.random_ids(17, V, 6)
    bound = 2e-5 if rt.full_precision else H.BF16_BOUND
    free0 = [p.free_count for p in ex.cache.pools]
    got = H.run_mixed(ex, {"a": a, "b": b}, seed=7, max_live=2, decode_tail=5)
    assert H.scaled_error(got["a"], plain_forward(a)) < bound
    assert H.scaled_error(got["b"], plain_forward(b)) < bound
    got = H.run_portions(ex, "c", a, [5, 2, 11, 8])
    assert H.scaled_error(got, plain_forward(a)) < bound
    if window:
        # the latent group gives back the pages its window has passed while the request lives; the attention's group keeps all
        ex.step([StepEntry("w", a, [len(a) - 1])])
        held = ex.cache.get("w").tables
        assert sum(1 for p_ in held[0] if p_ >= 0) < sum(1 for p_ in held[1] if p_ >= 0) == -(-len(a) // 4)
        ex.finish("w")
    assert [p.free_count for p in ex.cache.pools] == free0
    ex.cache.check_invariants()


# ------------------------------------------------------------------------------------------ position encoding and block alone
def test_position_encoding_part_alone(backend):
    from roost_b200.parts import POSITIONS
    rt = runtime(backend)
    rope = POSITIONS.build(PositionSpec(kind="rope_neox", rotary_dim=48, theta=5e5, max_positions=77), rt)
    inv_freq, rot = rope.rotation()
    assert rot == 48 and inv_freq.dtype == torch.float64 and rope.max_positions == 77
    want = torch.pow(torch.tensor(5e5, dtype=torch.float64), -2.0 * torch.arange(24, dtype=torch.float64) / 48)
    assert torch.allclose(inv_freq.cpu(), want, rtol=0, atol=0)
    assert POSITIONS.build(PositionSpec(kind="none"), rt).rotation() == (None, 0)
    with pytest.raises(ValueError):
        POSITIONS.build(PositionSpec(kind="rope_neox", rotary_dim=7, theta=1e4), rt)
    # through the fused kernel: rotating x at position p equals the plain rotation (no norm, no cache write)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 3 * 64, generator=g).to(rt.dtype)
    positions = torch.tensor([0, 1, 17, 300, 76], dtype=torch.int32)
    got = rt.kernels.qk_norm_rope_cache(x.to(rt.device), 3, 0, 64, q_w=None, k_w=None, eps=1.0, inv_freq=inv_freq, rotary_dim=48,
                                        positions=positions.to(rt.device), write_kv=False)
    want_x = plain.rope_neox(x.double().reshape(5, 3, 64), positions.tolist(), 5e5, 48)
    assert H.scaled_error(got, want_x) < (4e-6 if rt.full_precision else 2 ** -6)


def test_block_arrangement_alone(backend, tiny_model_dirs):
    """One pre-norm block over the step function's tables: h' = h + mixer(norm1(h)); out = h' + ff(norm2(h'))."""
    from roost_b200.cache.manager import CacheManager, build_groups
    from roost_b200.cache.storage import CacheStorage
    from roost_b200.engine.batch import BatchBuilder
    rt = runtime(backend)
    norm = NormSpec(size=48, eps=1e-5)
    spec = BlockSpec(mixer=attention_spec(None), feed_forward=GatedMlpSpec(hidden=48, intermediate=80), input_norm=norm, post_mixer_norm=norm)
    block = BLOCKS.build(spec, rt)
    g = torch.Generator().manual_seed(5)
    P = {"input_norm": {"weight": 1 + 0.1 * torch.randn(48, generator=g)}, "post_mixer_norm": {"weight": 1 + 0.1 * torch.randn(48, generator=g)},
         # weights small enough that the block's output stays O(1): bfloat16 rounding is relative to the values' size
         "mixer": {"qkv": torch.randn(160, 48, generator=g) * 0.1, "out": torch.randn(48, 96, generator=g) * 0.1,
                   "q_norm": 1 + 0.1 * torch.randn(16, generator=g), "k_norm": 1 + 0.1 * torch.randn(16, generator=g)},
         "feed_forward": {"gate_up": torch.randn(160, 48, generator=g) * 0.1, "down": torch.randn(48, 80, generator=g) * 0.1}}
    P = {s: {k: (v.to(rt.dtype) if v.dim() == 2 else v) for k, v in p.items()} for s, p in P.items()}
    for name, part in block.sub_parts().items():
        part.load({k: v.to(rt.device) for k, v in P[name].items()})
    T = 21
    h = torch.randn(T, 48, generator=g).to(rt.dtype)
    D = {s: {k: v.double() for k, v in p.items()} for s, p in P.items()}
    x = plain.rms_norm(h.double(), D["input_norm"]["weight"], 1e-5)
    w = {"q_proj.weight": D["mixer"]["qkv"][:96], "k_proj.weight": D["mixer"]["qkv"][96:128], "v_proj.weight": D["mixer"]["qkv"][128:],
         "o_proj.weight": D["mixer"]["out"], "q_norm.weight": D["mixer"]["q_norm"], "k_norm.weight": D["mixer"]["k_norm"]}
    cfg = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4)
    mix, _ = plain.attention_mixer(x, list(range(T)), w, "", cfg, None)
    hm = h.double() + mix
    y = plain.rms_norm(hm, D["post_mixer_norm"]["weight"], 1e-5)
    want = hm + plain.swiglu_mlp(y, D["feed_forward"]["gate_up"][:80], D["feed_forward"]["gate_up"][80:], D["feed_forward"]["down"])

    groups = build_groups([block.mixer.cache_need()], page_size=8)
    cm = CacheManager(groups, [6, 2])
    storage = CacheStorage(groups, [6, 2], rt.dtype, rt.device)
    rc = cm.extend("r", T)
    batch = BatchBuilder(rt.device, cm).build([(rc, 0, [0] * T, [])], vocab=1)
    out, residual = block(h.to(rt.device), None, batch, storage.view(0))
    got = out.double().cpu() + residual.double().cpu()       # the block hands back the branch output and the stream it joins
    assert H.scaled_error(got, want) < (1e-5 if rt.full_precision else 2 ** -4)


# ------------------------------------------------------------------------------------------ a toy feed-forward with routing, a toy position encoding
@dataclass(frozen=True)
class ToyRoutedSpec:
    """Two (or more) small SwiGLU experts and a router that sends every token to the expert with the largest logit and
    scales the expert's output by the softmax weight of that logit."""
    kind: str = "toy_top1_experts"
    hidden: int = 0
    intermediate: int = 0
    experts: int = 2


class ToyTop1Experts:
    """Defined in the test only: registered, built, loaded and stepped through the package's interfaces."""
    capturable = False   # the routing below reads device values on the host: no CUDA graph for this model's decode steps

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.router = Linear(rt, spec.experts, spec.hidden)
        self.gate_up = [Linear(rt, 2 * spec.intermediate, spec.hidden) for _ in range(spec.experts)]
        self.down = [Linear(rt, spec.hidden, spec.intermediate) for _ in range(spec.experts)]

    @classmethod
    def parameters(cls, spec):
        decl = {"router": ParamDecl(shape=(spec.experts, spec.hidden))}
        for e in range(spec.experts):
            decl[f"gate_up_{e}"] = ParamDecl(shape=(2 * spec.intermediate, spec.hidden))
            decl[f"down_{e}"] = ParamDecl(shape=(spec.hidden, spec.intermediate))
        return decl

    def load(self, params):
        self.router.load(params["router"])
        for e in range(self.spec.experts):
            self.gate_up[e].load(params[f"gate_up_{e}"])
            self.down[e].load(params[f"down_{e}"])

    def __call__(self, x, batch=None):
        logits = self.router(x, out_dtype=torch.float32) if self.rt.full_precision else self.router(x).float()   # router logits in 32-bit
        weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros_like(x, dtype=torch.float32)
        I = self.spec.intermediate
        for e in range(self.spec.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                gu = self.gate_up[e](x[rows].contiguous()).float()
                act = (gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]).to(x.dtype)
                out[rows] = self.down[e](act).float() * weight[rows, None]
        return out.to(x.dtype)


@dataclass(frozen=True)
class ToyScaledRopeSpec:
    """NeoX rotation over part of the head with every frequency divided by a factor (positions stretched)."""
    kind: str = "toy_scaled_rope"
    rotary_dim: int = 0
    theta: float = 10000.0
    factor: float = 1.0
    max_positions: int = 0


class ToyScaledRope:
    def __init__(self, spec, rt):
        self.spec = spec
        self.max_positions = spec.max_positions
        i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / spec.rotary_dim) / spec.factor).to(rt.device)

    def rotation(self):
        return self.inv_freq, self.spec.rotary_dim


class ToyGridRope(ToyScaledRope):
    """Two position axes: a token at position p sits at (row p // 5, column p % 5) of a grid five wide; the first half of
    the frequencies turn with the row, the second half with the column. The angles are no longer position x frequency,
    so the encoding hands over the step's cosines and sines itself, made on the device from the step's positions."""

    def step_table(self, batch):
        pos = batch.positions.clamp(min=0).double()
        half = self.inv_freq.numel()
        axis = torch.where(torch.arange(half, device=pos.device) < half // 2, torch.div(pos, 5, rounding_mode="floor")[:, None], (pos % 5)[:, None])
        ang = axis * self.inv_freq[None, :]
        return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous()


@pytest.mark.parametrize("encoding", ["toy_scaled_rope", "toy_grid_rope"])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_are_registered_built_and_stepped(backend, encoding):
    """Generality of the parts: a feed-forward with routing and another position encoding, both defined here, go into a
    model beside the package's own parts without a change to the package, and every way of stepping agrees with a
    plain whole-sequence computation."""
    from roost_b200.parts import register_feed_forward, register_position
    register_feed_forward("toy_top1_experts", ToyTop1Experts)
    register_position("toy_scaled_rope", ToyScaledRope)
    register_position("toy_grid_rope", ToyGridRope)
    rt = runtime(backend)
    H_, V, I, E = 48, 61, 32, 3
    norm = NormSpec(size=H_, eps=1e-5)
    attn = AttentionSpec(hidden=H_, num_heads=3, num_kv_heads=1, head_dim=16, scale=0.25, qk_norm=NormSpec(size=16, eps=1e-5),
                         position=ToyScaledRopeSpec(kind=encoding, rotary_dim=8, theta=50.0, factor=4.0))
    blocks = (BlockSpec(mixer=attn, feed_forward=ToyRoutedSpec(hidden=H_, intermediate=I, experts=E), input_norm=norm, post_mixer_norm=norm),
              BlockSpec(mixer=attn, feed_forward=GatedMlpSpec(hidden=H_, intermediate=I), input_norm=norm, post_mixer_norm=norm))
    spec = ModelSpec(architecture="ToyRoutedForTests", hidden=H_, vocab=V, blocks=blocks, schedule=(RunEntry(0), RunEntry(1)),
                     final_norm=norm, tie_embeddings=True, max_positions=0)
    model = Model(spec, rt)
    g = torch.Generator().manual_seed(5)
    params = {}
    for scope, decl in parameter_declarations(spec).items():
        params[scope] = {k: (torch.ones(d.shape) + 0.1 * torch.randn(d.shape, generator=g) if d.role == "vector"
                             else torch.randn(d.shape, generator=g) * 0.25).to(rt.dtype) for k, d in decl.items()}
    # well separated router logits: a rounding difference must not send a token to another expert
    params["blocks.0.feed_forward"]["router"] = (torch.randn(E, H_, generator=g) * 2.0).to(rt.dtype)
    model.load(params)
    ex = StepExecutor(model, page_size=4, num_pages=48, max_requests=3)

    def rope(x, pos):   # the toy encoding, plainly: the first 8 elements of a head, frequencies divided by 4
        half = 4
        freq = torch.pow(torch.tensor(50.0, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / 8) / 4.0
        p64 = torch.tensor(pos, dtype=torch.float64)
        if encoding == "toy_grid_rope":   # two axes: the first two frequencies turn with p // 5, the last two with p % 5
            ang = torch.cat([torch.floor(p64 / 5)[:, None] * freq[None, :2], (p64 % 5)[:, None] * freq[None, 2:]], dim=1)
        else:
            ang = p64[:, None] * freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = x.clone()
        out[..., :half] = x[..., :half] * c - x[..., half:8] * s
        out[..., half:8] = x[..., half:8] * c + x[..., :half] * s
        return out

    def plain_forward(ids):
        P = {s: {k: v.double() for k, v in p.items()} for s, p in params.items()}
        h = P["embed"]["table"][torch.tensor(ids)]
        pos = list(range(len(ids)))
        margins = []
        for bi in (0, 1):
            x = plain.rms_norm(h, P[f"blocks.{bi}.input_norm"]["weight"], 1e-5)
            m = P[f"blocks.{bi}.mixer"]
            qkv = m["qkv"]
            q = rope(plain.rms_norm((x @ qkv[:48].T).reshape(-1, 3, 16), m["q_norm"], 1e-5), pos)
            k = rope(plain.rms_norm((x @ qkv[48:64].T).reshape(-1, 1, 16), m["k_norm"], 1e-5), pos)
            v = (x @ qkv[64:].T).reshape(-1, 1, 16)
            h = h + plain.causal_gqa_attention(q, k, v, 0.25).reshape(-1, 48) @ m["out"].T
            y = plain.rms_norm(h, P[f"blocks.{bi}.post_mixer_norm"]["weight"], 1e-5)
            f = P[f"blocks.{bi}.feed_forward"]
            if bi == 0:
                probs = torch.softmax(y @ f["router"].T, dim=-1)
                weight, choice = probs.max(dim=-1)
                top2 = probs.topk(2, dim=-1).values
                margins.append(float((top2[:, 0] - top2[:, 1]).min()))
                ff = torch.zeros_like(y)
                for t in range(y.shape[0]):
                    e = int(choice[t])
                    ff[t] = plain.swiglu_mlp(y[t : t + 1], f[f"gate_up_{e}"][:I], f[f"gate_up_{e}"][I:], f[f"down_{e}"])[0] * weight[t]
                h = h + ff
            else:
                h = h + plain.swiglu_mlp(y, f["gate_up"][:I], f["gate_up"][I:], f["down"])
        return plain.rms_norm(h, P["final_norm"]["weight"], 1e-5) @ P["embed"]["table"].T, min(margins)

    a, b = H.random_ids(21, V, 11), H.random_ids(14, V, 12)
    want_a, margin_a = plain_forward(a)
    want_b, margin_b = plain_forward(b)
    assert min(margin_a, margin_b) > 0.02, "the test's router must separate its experts clearly"
    bound = 2e-5 if rt.full_precision else H.BF16_BOUND
    got = H.run_mixed(ex, {"a": a, "b": b}, seed=4, max_live=2, decode_tail=3)
    assert H.scaled_error(got["a"], want_a) < bound
    assert H.scaled_error(got["b"], want_b) < bound
    got = H.run_portions(ex, "c", a, [5, 2, 14])
    assert H.scaled_error(got, want_a) < bound
    assert not ex.use_graphs and ex.graph_replays == 0


# ------------------------------------------------------------------------------------------ toy ends of a model
@dataclass(frozen=True)
class ToyScaledEmbeddingSpec:
    kind: str = "toy_scaled_table"
    vocab: int = 0
    hidden: int = 0
    scale: float = 1.0


@dataclass(frozen=True)
class ToyCappedHeadSpec:
    kind: str = "toy_capped_linear"
    vocab: int = 0
    hidden: int = 0
    cap: float = 30.0


def test_a_toy_embedding_and_a_toy_head_are_registered_built_and_stepped(backend):
    """The two ends of a model are parts like the others: an embedding that scales its rows and a head that caps its logits
    (cap * tanh(z / cap)), defined here, registered and run through the executor, the head tied to the toy embedding's
    table; nothing in the package changes."""
    from roost_b200.parts import Embedding, Head, register_embedding, register_head

    class ToyScaledEmbedding(Embedding):
        def __init__(self, spec, rt):
            self.spec, self.rt, self.table = spec, rt, None

        @classmethod
        def parameters(cls, spec):
            return {"table": ParamDecl(shape=(spec.vocab, spec.hidden))}

        def load(self, params):
            self.table = params["table"].to(self.rt.dtype).contiguous()

        def tied_weight(self):
            return self.table

        def __call__(self, ids, batch=None):
            return (self.rt.kernels.embedding(self.table, ids).float() * self.spec.scale).to(self.rt.dtype)

    class ToyCappedHead(Head):
        def __init__(self, spec, rt):
            self.spec, self.rt = spec, rt
            self.linear = Linear(rt, spec.vocab, spec.hidden)

        @classmethod
        def parameters(cls, spec):
            return {"weight": ParamDecl(shape=(spec.vocab, spec.hidden))}

        def load(self, params):
            self.linear.load(params["weight"])

        def __call__(self, final, batch=None):
            z = self.linear(final, out_dtype=torch.float32)
            return self.spec.cap * torch.tanh(z / self.spec.cap)

    register_embedding("toy_scaled_table", ToyScaledEmbedding)
    register_head("toy_capped_linear", ToyCappedHead)
    rt = runtime(backend)
    H_, V, I = 32, 70, 48
    norm = NormSpec(size=H_, eps=1e-6)
    attn = AttentionSpec(hidden=H_, num_heads=2, num_kv_heads=1, head_dim=16, scale=0.25, qk_norm=None,
                         position=PositionSpec(rotary_dim=16, theta=100.0))
    block = BlockSpec(mixer=attn, feed_forward=GatedMlpSpec(hidden=H_, intermediate=I), input_norm=norm, post_mixer_norm=norm)
    scale, cap = math.sqrt(H_), 4.0
    spec = ModelSpec(architecture="ToyEndsForTests", hidden=H_, vocab=V, blocks=(block,), schedule=(RunEntry(0),), final_norm=norm,
                     tie_embeddings=True, max_positions=0, embedding=ToyScaledEmbeddingSpec(vocab=V, hidden=H_, scale=scale),
                     head=ToyCappedHeadSpec(vocab=V, hidden=H_, cap=cap))
    model = Model(spec, rt)
    g = torch.Generator().manual_seed(8)
    params = {}
    for scope, decl in parameter_declarations(spec).items():
        params[scope] = {k: (torch.ones(d.shape) if d.role == "vector" else torch.randn(d.shape, generator=g) * 0.3).to(rt.dtype) for k, d in decl.items()}
    assert "lm_head" not in params
    model.load(params)
    ex = StepExecutor(model, page_size=4, num_pages=24, max_requests=2)

    def plain_forward(ids):
        P = {s_: {k: v.double() for k, v in p.items()} for s_, p in params.items()}
        h = P["embed"]["table"][torch.tensor(ids)] * scale
        if not rt.full_precision:
            h = h.to(torch.bfloat16).double()
        pos = list(range(len(ids)))
        x = plain.rms_norm(h, P["blocks.0.input_norm"]["weight"], 1e-6)
        qkv = P["blocks.0.mixer"]["qkv"]
        q = plain.rope_neox((x @ qkv[:32].T).reshape(-1, 2, 16), pos, 100.0)
        k = plain.rope_neox((x @ qkv[32:48].T).reshape(-1, 1, 16), pos, 100.0)
        v = (x @ qkv[48:].T).reshape(-1, 1, 16)
        h = h + plain.causal_gqa_attention(q, k, v, 0.25).reshape(-1, 32) @ P["blocks.0.mixer"]["out"].T
        y = plain.rms_norm(h, P["blocks.0.post_mixer_norm"]["weight"], 1e-6)
        gu = P["blocks.0.feed_forward"]["gate_up"]
        h = h + plain.swiglu_mlp(y, gu[:I], gu[I:], P["blocks.0.feed_forward"]["down"])
        z = plain.rms_norm(h, P["final_norm"]["weight"], 1e-6) @ P["embed"]["table"].T
        return cap * torch.tanh(z / cap)

    ids = H.random_ids(19, V, 5)
    want = plain_forward(ids)
    assert float(want.abs().max()) > 0.8 * cap, "the test's logits must reach the cap for the cap to show"
    bound = 2e-5 if rt.full_precision else H.BF16_BOUND
    assert H.scaled_error(H.run_whole(ex, "w", ids), want) < bound
    assert H.scaled_error(H.run_tail_decoded(ex, "t", ids, tail=8), want) < bound


@pytest.mark.gpu
def test_steps_started_before_the_last_tokens_were_read_give_the_same_tokens(tiny_model_dirs):
    """While every live request decodes, the engine starts the next step with the sampled tokens still on the device.
    Requests that end at different times (their rows of the running step are dropped), stop tokens, a request that
    arrives in the middle (the running step stands, the newcomer joins a step later) and one that is cancelled: the
    tokens are those of an engine that reads every step's tokens first."""
    t = TINY["B"]
    model = H.make_model(tiny_model_dirs["B"], torch.float32, "gpu")
    V = t["config"]["vocab_size"]
    prompts = [H.random_ids(n, V, 400 + n) for n in (5, 11, 17, 23, 9)]
    opts = [GenerationOptions(max_output_tokens=m, temperature=(0.9 if i % 2 else None), top_p=0.95, seed=60 + i)
            for i, m in enumerate((40, 9, 26, 14, 12))]
    results = []
    for chain in (True, False):
        engine = RoostEngine(model, page_size=t["page_size"], attention_blocks=96, max_sequences=8, max_tokens=64, chain_steps=chain)
        got = {}
        ids = [engine.add_request(p, o.sampling(), stop_token_ids=o.stop_token_ids) for p, o in zip(prompts[:3], opts[:3])]
        steps = 0
        while engine.has_unfinished():
            for e in engine.step():
                if e.token is not None:
                    got.setdefault(e.request_id, []).append(e.token)
            steps += 1
            if steps == 7:
                ids.append(engine.add_request(prompts[3], opts[3].sampling()))
            if steps == 12:
                ids.append(engine.add_request(prompts[4], opts[4].sampling()))
            if steps == 16:
                engine.cancel(ids[4])
        results.append([got.get(r, []) for r in ids[:4]])
        assert engine.executor.cache.pools[0].free_count == 96
        engine.executor.cache.check_invariants()
        if chain:
            assert engine.chained_steps > 10
        else:
            assert engine.chained_steps == 0
    assert results[0] == results[1]
    assert [len(x) for x in results[0]][1] == 9
