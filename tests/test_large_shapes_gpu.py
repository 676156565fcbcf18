"""The engine at the layer sizes of real models (one or two layers of each, the full vocabulary), against the plain
implementation run in float64 on the GPU: head size 128, query width unequal to the hidden size, a vocabulary that is no
power of two, tied and untied heads. float32 must agree to 1e-4 relative and give the same greedy tokens for every way
of cutting the work; bfloat16 stays within the bounds stated in tests/helpers.py."""
import pytest
import torch

from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.random_init import write_random_model
from tests import helpers as H
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", rope_theta=1000000.0, rms_norm_eps=1e-6,
            vocab_size=151936, max_position_embeddings=40960, torch_dtype="bfloat16", head_dim=128, num_key_value_heads=8)
SHAPES = {
    "0.6b": dict(BASE, num_hidden_layers=2, hidden_size=1024, num_attention_heads=16, intermediate_size=3072, tie_word_embeddings=True),
    "8b": dict(BASE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(BASE, num_hidden_layers=1, hidden_size=5120, num_attention_heads=64, intermediate_size=25600, tie_word_embeddings=False),
}


V = BASE["vocab_size"]


class Big:
    """A model folder at one size, with the plain implementation's float64 weights kept on the GPU while the module's
    tests of that size run (the file stores bfloat16, so both of the engine's precisions see exactly these values)."""

    def __init__(self, name, model_dir):
        self.name, self.dir = name, model_dir
        self.cfg, w = plain.load_model_dir(model_dir)
        self.w = {k: v.cuda() for k, v in w.items()}

    def plain(self, ids, rows=None) -> torch.Tensor:
        out = plain.forward_logits(self.cfg, self.w, ids, rows=rows).cpu()
        torch.cuda.empty_cache()
        return out


@pytest.fixture(scope="module", params=list(SHAPES))
def big_model(request, tmp_path_factory):
    name = request.param
    d = tmp_path_factory.mktemp(f"big_{name}")
    write_random_model(d, SHAPES[name], seed=11, std=0.02, norm_std=0.05)
    b = Big(name, d)
    yield b
    b.w.clear()
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def big(big_model):
    ids = H.random_ids(80, V, seed=12)
    return big_model.name, big_model.dir, ids, big_model.plain(ids)


def compare(what, dtype, got, want):
    """float32: 1e-4 relative and the same greedy token wherever the plain top two are not a near-tie; bfloat16: the two
    bounds explained in test_layer_sizes_of_real_models."""
    got, want = got.cpu(), want.cpu()
    err, rms = H.scaled_error(got, want), H.rms_error(got, want)
    print(f"MEASURED {what} {dtype}: worst scaled error {err:.3e}, rms error {rms:.3e}")
    if dtype == torch.float32:
        assert err < 1e-4, f"{what}: {err}"
        top2 = want.topk(2, dim=-1).values
        clear = (top2[..., 0] - top2[..., 1]) > 1e-3
        assert torch.equal(got.argmax(-1)[clear], want.argmax(-1)[clear]), what
    else:
        assert err < 2.0 ** -3 and rms < H.BF16_RMS_BOUND, f"{what}: worst {err}, rms {rms}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_sizes_of_real_models(big, dtype):
    name, model_dir, ids, want = big
    model = H.make_model(model_dir, dtype, "gpu")
    ex = StepExecutor(model, page_size=16, num_pages=24, max_requests=4)
    whole = H.run_whole(ex, "w", ids).cpu()
    tail = H.run_tail_decoded(ex, "t", ids, tail=32).cpu()
    parts = H.run_portions(ex, "p", ids, [17, 2, 9, 3, 2, 31]).cpu()
    a, b = H.random_ids(40, 151936, 13), H.random_ids(25, 151936, 14)
    mixed = H.run_mixed(ex, {"m": ids, "a": a, "b": b}, seed=15, max_live=3, decode_tail=6)["m"].cpu()
    for what, got in (("whole", whole), ("tail decoded", tail), ("portions", parts), ("mixed", mixed)):
        err, rms = H.scaled_error(got, want), H.rms_error(got, want)
        print(f"MEASURED {name} {dtype} {what}: worst scaled error {err:.3e}, rms error {rms:.3e}")
        if dtype == torch.float32:
            assert err < 1e-4, f"{name} {what}: {err}"
            top2 = want.topk(2, dim=-1).values
            clear = (top2[:, 0] - top2[:, 1]) > 1e-3
            assert torch.equal(got.argmax(-1)[clear], want.argmax(-1)[clear])
        else:
            # twelve million logits are compared here, three hundred times more than on the tiny models: the worst of
            # that many roundings of the same size lies near six standard deviations instead of four (measured 2.9e-2 to
            # 6.8e-2 with a root-mean-square error of 0.9e-2 to 1.1e-2), so the worst-case bound is 2^-3 here; the
            # root-mean-square bound, which does not grow with the sample, stays 2^-6
            assert err < 2.0 ** -3 and rms < H.BF16_RMS_BOUND, f"{name} {what}: worst {err}, rms {rms}"
    if dtype == torch.float32:
        assert torch.equal(tail, whole) and torch.equal(parts, whole) and torch.equal(mixed, whole), \
            "the float32 kernels promise the same bits for every cut"
    assert all(p.free_count == p.capacity for p in ex.cache.pools)


# ------------------------------------------------------------------------------------------ the regimes the benchmark runs
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_of_2048_tokens_whole_and_replayed_from_its_captured_graph(big_model, dtype):
    """The benchmark's prefill: 2,048 tokens in one step. First with the logits of its last 64 positions (more logits
    than rows: that step runs eagerly), then three times with the last position's alone: the second such step is
    captured, the third replays the graph. At these sizes the step's feed-forward runs the fused tcgen05 product
    and, with 64 query heads, the attention takes two row groups a CTA."""
    model = H.make_model(big_model.dir, dtype, "gpu")
    ids = H.random_ids(2048, V, seed=21)
    want = big_model.plain(ids, rows=range(1984, 2048))
    ex = StepExecutor(model, page_size=16, num_pages=2048 // 16 + 4, max_requests=2)
    tail = ex.step([StepEntry("tail", ids, list(range(1984, 2048)))])
    ex.finish("tail")
    compare(f"{big_model.name} 2048 whole, last 64", dtype, tail, want)
    lasts = []
    for rep in range(3):
        lasts.append(ex.step([StepEntry(f"r{rep}", ids, [2047])]))
        ex.finish(f"r{rep}")
    assert ex.graph_replays >= 1 and (2048, 1) in {k[:2] for k in ex._graphs}, "the 2,048-token step was not replayed from a graph"
    for rep, got in enumerate(lasts):
        compare(f"{big_model.name} 2048 whole, run {rep}", dtype, got, want[-1:])
        assert torch.equal(got, lasts[0]), "the eager step, the capture's step and the replay give the same bits"
    if dtype == torch.float32:
        assert torch.equal(lasts[0], tail[-1:])
    model.rt.kernels.check_device_status()
    ex.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_512_tokens_beside_three_decoding_requests(big_model, dtype):
    """A serving step under a 512-token budget: three requests with 1,000 to 3,000 tokens behind them decode one token
    each beside a 509-token portion of a fourth request's prompt, four steps of the same sizes in a row (captured at the
    second, replayed after). The decode rows are split over several chunks and merged inside the mixed step."""
    model = H.make_model(big_model.dir, dtype, "gpu")
    lens = [1000, 2030, 3000]
    decoders = {f"d{i}": H.random_ids(n + 4, V, seed=30 + i) for i, n in enumerate(lens)}
    prompt = H.random_ids(4 * 509, V, seed=34)
    want_dec = {r: big_model.plain(ids, rows=range(len(ids) - 4, len(ids))) for r, ids in decoders.items()}
    want_prompt = big_model.plain(prompt, rows=[len(prompt) - 1])
    pages = sum(-(-(len(x) + 1) // 16) for x in list(decoders.values()) + [prompt]) + 4
    ex = StepExecutor(model, page_size=16, num_pages=pages, max_requests=8)
    ex.step([StepEntry(r, ids[:-4], []) for r, ids in decoders.items()])       # 6,030 tokens, three rows: eager
    got_dec = {r: [] for r in decoders}
    for i in range(4):
        entries = [StepEntry(r, [ids[len(ids) - 4 + i]], [0]) for r, ids in decoders.items()]
        entries.insert(1, StepEntry("p", prompt[i * 509 : (i + 1) * 509], [508] if i == 3 else []))
        out = ex.step(entries)
        rows = iter(out)
        for e in entries:
            if e.request_id == "p":
                if e.want:
                    compare(f"{big_model.name} portions: the prompt's last position", dtype, next(rows)[None], want_prompt)
            else:
                got_dec[e.request_id].append(next(rows))
    assert ex.graph_replays >= 2, "the mixed steps were not replayed from a captured graph"
    for r in decoders:
        compare(f"{big_model.name} portions: decoding request {r}", dtype, torch.stack(got_dec[r]), want_dec[r])
    model.rt.kernels.check_device_status()
    ex.close()


@pytest.mark.parametrize("requests", [9, 8])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_at_contexts_of_1000_to_4090_keys_through_captured_graphs(big_model, dtype, requests):
    """The benchmark's decode: requests with 1,000 to 4,074 tokens behind them decode 16 tokens each, every step's logits
    compared. Nine requests run the captured step of twelve rows (three of them padding) with chunks of 512 keys; eight
    run the step whose size class makes the split decode kernel take chunks of 1,024 keys and merge them in clusters. The contexts are prefilled
    two or three requests a step (up to 7,500 tokens a step: two row groups a CTA in the prefill attention)."""
    from roost_b200.engine.executor import graph_rows
    model = H.make_model(big_model.dir, dtype, "gpu")
    k = model.rt.kernels
    steps = 16
    contexts = [1000 + (4074 - 1000) * i // (requests - 1) for i in range(requests)]
    reqs = {f"q{i}": H.random_ids(n + steps, V, seed=40 + i) for i, n in enumerate(contexts)}
    want = torch.stack([big_model.plain(ids, rows=range(len(ids) - steps, len(ids))) for ids in reqs.values()], dim=1)   # [steps, requests, V]
    pages = sum(-(-len(x) // 16) for x in reqs.values()) + 4
    ex = StepExecutor(model, page_size=16, num_pages=pages, max_requests=16)
    names = list(reqs)
    at = 0
    while at < requests:                     # prefill: the longest with the shortest, so that a step stays near 7,500 tokens
        group = names[at : at + 3] if contexts[min(at + 2, requests - 1)] < 2500 else names[at : at + 2]
        ex.step([StepEntry(r, reqs[r][:-steps], []) for r in group])
        at += len(group)
    got = []
    for i in range(steps):
        got.append(ex.step([StepEntry(r, [ids[len(ids) - steps + i]], [0]) for r, ids in reqs.items()]))
    got = torch.stack(got)
    rows = graph_rows(requests)
    assert rows == (12 if requests == 9 else 8) and ex.graph_replays >= steps - 1 and {key[0] for key in ex._graphs if key[0] == key[1]} == {rows}
    if dtype == torch.bfloat16:
        # nine requests: chunks of 512 keys through partial results and the merge kernel; eight: chunks of 1,024 keys, each
        # row's four chunks merged by a cluster of four CTAs
        pools = ex.storage.tensors[0][0]
        assert k.decode_split_for(rows, 4096, pools[0], pools[1]) == ((512, 0) if requests == 9 else (1024, 4))
    compare(f"{big_model.name} decode of {requests} requests at {contexts[0]}..{contexts[-1] + steps} keys", dtype, got, want)
    k.check_device_status()
    assert all(ex.cache.get(r).tokens == len(ids) for r, ids in reqs.items())
    ex.close()
