"""A whole architecture added from outside the package, without a change to the package's files: a made-up decoder for
this test (never a model of anyone's) with config.json keys, tensor names and an arrangement of its own. No head norms, a
rotation of half of each head, two blocks of weights of which the first runs twice, its second run reading the first run's
cache instead of keeping one, a window in the other block, an untied head. ``register_architecture`` is all it takes: the
random-weights mode writes its model folder, the loader reads the folder by the names the architecture gives (and says what
is missing by those names), the step function, the scheduler and the entry point run it, and the logits are those of the
plain parts put together by hand."""
import json
import math
from dataclasses import dataclass

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine, register_architecture
from roost_b200.config.reader import ConfigError, ConfigReader
from roost_b200.config.spec import AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec, PositionSpec, RunEntry
from roost_b200.engine.executor import StepExecutor
from roost_b200.weights.loader import WeightError
from roost_b200.weights.random_init import write_random_model
from roost_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
from tests import helpers as H
from tests.plain import qwen3_plain as plain

# What this file shows is host-side (the registry, the loader's names, the cache groups a run order asks for, the step
# function's and the scheduler's handling of a run that reads another run's cache): it runs on the CPU stand-in for the
# kernels. The kernels meet the same parts (no head norms, a partial rotation, windows, a run without a cache of its own)
# in the device tests of the parts and of the toy mixers.
BACKENDS = [pytest.param(("fake", torch.float32), id="cpu-fake")]


@dataclass(frozen=True)
class EchoConfig:
    width: int
    symbols: int
    heads: int
    shared_heads: int
    head_width: int
    turn: int                  # elements of a head that are rotated
    base: float
    inner: int
    eps: float
    order: tuple               # which block each run uses
    reads: tuple               # per run: the earlier run whose cache it reads, or None
    windows: tuple             # per block: keys a query sees, or None
    stop: tuple
    tie_word_embeddings = False

    @classmethod
    def read(cls, c: ConfigReader) -> "EchoConfig":
        order = tuple(c.opt_ints("order") or ())
        blocks = c.positive_int("blocks")
        if not order or any(not 0 <= b < blocks for b in order):
            raise ConfigError(f"{c.source}: key 'order' must name blocks 0..{blocks - 1}")
        reads = c.raw("reads") if c.has("reads") else [None] * len(order)
        windows = c.raw("windows") if c.has("windows") else [None] * blocks
        if len(reads) != len(order) or len(windows) != blocks:
            raise ConfigError(f"{c.source}: 'reads' has an entry a run and 'windows' an entry a block")
        return cls(width=c.positive_int("width"), symbols=c.positive_int("symbols"), heads=c.positive_int("heads"),
                   shared_heads=c.positive_int("shared_heads"), head_width=c.positive_int("head_width"), turn=c.required_int("turn"),
                   base=c.opt_float("base") or 10000.0, inner=c.positive_int("inner"), eps=c.opt_float("eps") or 1e-6, order=order,
                   reads=tuple(reads), windows=tuple(windows), stop=tuple(c.opt_ints("stop") or ()))

    def to_spec(self, tied=None) -> ModelSpec:
        norm = NormSpec(size=self.width, eps=self.eps)
        ff = GatedMlpSpec(hidden=self.width, intermediate=self.inner)
        blocks, names = [], {"embed": {"table": ("symbols.table",)}, "final_norm": {"weight": ("last.scale",)}, "lm_head": {"weight": ("last.readout",)}}
        for i, window in enumerate(self.windows):
            mixer = AttentionSpec(hidden=self.width, num_heads=self.heads, num_kv_heads=self.shared_heads, head_dim=self.head_width,
                                  scale=1.0 / math.sqrt(self.head_width), window=window, qk_norm=None,
                                  position=PositionSpec(rotary_dim=self.turn, theta=self.base))
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm))
            names[f"blocks.{i}.input_norm"] = {"weight": (f"b{i}.scale_in",)}
            names[f"blocks.{i}.post_mixer_norm"] = {"weight": (f"b{i}.scale_mid",)}
            names[f"blocks.{i}.mixer"] = {"qkv": (f"b{i}.ask", f"b{i}.keys", f"b{i}.vals"), "out": (f"b{i}.back",)}
            names[f"blocks.{i}.feed_forward"] = {"gate_up": (f"b{i}.gate", f"b{i}.lift"), "down": (f"b{i}.drop",)}
        return ModelSpec(architecture="EchoDecoderForTests", hidden=self.width, vocab=self.symbols, blocks=tuple(blocks),
                         schedule=tuple(RunEntry(block=b, reads_cache_of=r) for b, r in zip(self.order, self.reads)), final_norm=norm,
                         tie_embeddings=False, max_positions=0, stop_token_ids=self.stop, stored_dtype="float32", weight_names=names)


CONFIG = {"architectures": ["EchoDecoderForTests"], "width": 56, "symbols": 113, "heads": 6, "shared_heads": 2, "head_width": 32, "turn": 16,
          "base": 700.0, "inner": 72, "eps": 1e-5, "blocks": 2, "order": [0, 1, 0], "reads": [None, None, 0], "windows": [None, 11], "stop": [4]}


@pytest.fixture(scope="module")
def echo_dir(tmp_path_factory):
    register_architecture("EchoDecoderForTests", read_config=EchoConfig.read, to_spec=lambda cfg, tied=None: cfg.to_spec(tied))
    return write_random_model(tmp_path_factory.mktemp("echo"), CONFIG, seed=12, std=0.15, norm_std=0.1)


def stored_tensors(model_dir) -> dict:
    with SafetensorsFile(model_dir / "model.safetensors") as f:
        return {n: f.tensor(n) for n in f.names()}


def plain_logits(model_dir, ids, bf16):
    """The architecture's forward pass from the plain parts, whole sequence, no cache."""
    w = {n: t.double() for n, t in stored_tensors(model_dir).items()}
    if bf16:
        w = {n: (t.to(torch.bfloat16).double() if t.dim() >= 2 else t) for n, t in w.items()}
    c = CONFIG
    nq, nkv, d = c["heads"], c["shared_heads"], c["head_width"]
    h = w["symbols.table"][torch.tensor(ids)]
    pos = list(range(len(ids)))
    kept = {}
    for run, (b, reads) in enumerate(zip(c["order"], c["reads"])):
        x = plain.rms_norm(h, w[f"b{b}.scale_in"], c["eps"])
        q = plain.rope_neox((x @ w[f"b{b}.ask"].T).reshape(-1, nq, d), pos, c["base"], c["turn"])
        if reads is None:
            k = plain.rope_neox((x @ w[f"b{b}.keys"].T).reshape(-1, nkv, d), pos, c["base"], c["turn"])
            v = (x @ w[f"b{b}.vals"].T).reshape(-1, nkv, d)
            kept[run] = (k, v)
        else:
            k, v = kept[reads]
        mix = plain.causal_gqa_attention(q, k, v, 1 / math.sqrt(d), c["windows"][b]).reshape(len(ids), nq * d) @ w[f"b{b}.back"].T
        h = h + mix
        y = plain.rms_norm(h, w[f"b{b}.scale_mid"], c["eps"])
        h = h + plain.swiglu_mlp(y, w[f"b{b}.gate"], w[f"b{b}.lift"], w[f"b{b}.drop"])
    return plain.rms_norm(h, w["last.scale"], c["eps"]) @ w["last.readout"].T


def test_the_architecture_is_found_by_config_json_and_its_folder_is_written_and_read_by_its_own_names(echo_dir):
    names = set(stored_tensors(echo_dir))
    assert {"symbols.table", "b0.ask", "b1.vals", "b0.lift", "last.readout"} <= names and len(names) == 3 + 2 * 9
    model = H.make_model(echo_dir, torch.float32, "fake")
    assert model.spec.architecture == "EchoDecoderForTests" and len(model.blocks) == 2 and len(model.spec.schedule) == 3
    assert [n.kind if n else None for n in model.cache_needs] == ["paged", "paged", None]       # the third run keeps no cache
    # a folder that lacks a tensor says so by this architecture's name for it
    tensors = stored_tensors(echo_dir)
    broken = echo_dir.parent / "broken"
    broken.mkdir(exist_ok=True)
    (broken / "config.json").write_text(json.dumps(CONFIG))
    write_safetensors(broken / "model.safetensors", {n: t for n, t in tensors.items() if n != "b1.lift"})
    with pytest.raises(WeightError, match="b1.lift"):
        H.make_model(broken, torch.float32, "fake")
    with pytest.raises(ConfigError, match="order"):
        EchoConfig.read(ConfigReader(dict(CONFIG, order=[0, 2]), "config"))


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_step_function_runs_it_in_portions_and_batches(echo_dir, backend):
    kind, dtype = backend
    model = H.make_model(echo_dir, dtype, kind)
    ex = StepExecutor(model, page_size=4, num_pages=30, max_requests=3)
    assert [(g.kind, g.window, g.runs) for g in ex.groups if g.kind == "paged"] == [("paged", None, (0,)), ("paged", 11, (1,))]
    reqs = {"a": H.random_ids(41, CONFIG["symbols"], 1), "b": H.random_ids(23, CONFIG["symbols"], 2), "c": H.random_ids(30, CONFIG["symbols"], 3)}
    got = H.run_mixed(ex, reqs, seed=5, max_live=2, decode_tail=6)
    for rid, ids in reqs.items():
        assert H.scaled_error(got[rid], plain_logits(echo_dir, ids, dtype == torch.bfloat16)) < H.bound_for(dtype), rid
    whole = H.run_whole(ex, "w", reqs["a"])
    assert H.scaled_error(whole, plain_logits(echo_dir, reqs["a"], dtype == torch.bfloat16)) < H.bound_for(dtype)


@pytest.mark.parametrize("backend", BACKENDS)
def test_the_entry_point_generates_from_its_folder(echo_dir, backend):
    kind, dtype = backend
    model = H.make_model(echo_dir, dtype, kind)
    engine = RoostEngine(model, page_size=4, attention_blocks=24, max_sequences=3, max_tokens=16, **({"device": "cpu"} if kind == "fake" else {}))
    prompts = [H.random_ids(n, CONFIG["symbols"], 40 + n) for n in (19, 5, 11)]
    outs = engine.generate(prompts, GenerationOptions(max_output_tokens=12))
    for p, out in zip(prompts, outs):
        assert out.finish_reason in ("length", "stop") and (out.finish_reason == "length" or out.token_ids[-1] == 4)     # the config's stop id
        logits = plain_logits(echo_dir, list(p) + out.token_ids[:-1], dtype == torch.bfloat16)
        for j, tok in enumerate(out.token_ids):
            top = logits[len(p) - 1 + j].topk(2)
            if float(top.values[0] - top.values[1]) > (1e-3 if dtype == torch.float32 else 0.15):
                assert tok == int(top.indices[0]), (j, tok, int(top.indices[0]))
    assert all(pool.used_count == 0 for pool in engine.executor.cache.pools)
