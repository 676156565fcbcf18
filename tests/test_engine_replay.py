"""The engine against the plain implementation, for every way of cutting the work.

Each test runs twice: on the GPU with the real kernel library (marked gpu), in float32 and bfloat16, and on the CPU
with the stand-in kernels of tests/fake_kernels.py, which checks the host side (tables, pages, the step function's
bookkeeping) where no GPU is present.
"""
import pytest
import torch

from roost_b200.engine.executor import StepEntry, StepExecutor
from tests import helpers as H
from tests.conftest import TINY

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]


@pytest.fixture(params=BACKENDS)
def backend(request):
    return request.param


@pytest.fixture(params=["A", "B", "C", "D"])
def tiny(request, tiny_model_dirs):
    return request.param, tiny_model_dirs[request.param], TINY[request.param]


def make_executor(tiny, backend, num_pages):
    name, model_dir, t = tiny
    kind, dtype = backend
    model = H.make_model(model_dir, dtype, kind)
    if num_pages >= 40:   # "roomy" pools are sized in tokens, whatever the page size
        num_pages = max(num_pages, num_pages * 8 // t["page_size"])
    return StepExecutor(model, page_size=t["page_size"], num_pages=num_pages, max_requests=4), dtype


def check(got, model_dir, ids, dtype, what):
    want = H.plain_logits(model_dir, ids, bf16=dtype == torch.bfloat16)
    err = H.scaled_error(got, want)
    rms = H.rms_error(got, want)
    print(f"MEASURED {what} {dtype}: worst scaled error {err:.3e}, rms error {rms:.3e}")
    assert err < H.bound_for(dtype), f"{what}: worst scaled error {err}"
    if dtype == torch.bfloat16:
        assert rms < H.BF16_RMS_BOUND, f"{what}: rms error {rms}"
    if dtype == torch.float32:
        # greedy tokens agree wherever the plain implementation's top two logits are not a near-tie
        top2 = want.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 1e-3
        assert torch.equal(got.cpu().argmax(-1)[clear], want.argmax(-1)[clear])


@pytest.mark.parametrize("length", [7, 19, 33, 150])
def test_each_request_alone_and_whole(tiny, backend, length):
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=40)
    ids = H.random_ids(length, t["config"]["vocab_size"], seed=length)
    check(H.run_whole(ex, "r", ids), model_dir, ids, dtype, f"{name} whole {length}")
    ex.cache.check_invariants()
    assert ex.cache.pools[0].free_count == ex.cache.pools[0].capacity


def test_first_tokens_of_a_sequence(tiny, backend):
    """One token, then two: the shortest prompts, the first row of the first page."""
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=8)
    for n in (1, 2, 3):
        ids = H.random_ids(n, t["config"]["vocab_size"], seed=100 + n)
        check(H.run_whole(ex, f"r{n}", ids), model_dir, ids, dtype, f"{name} first {n}")
    ids = H.random_ids(5, t["config"]["vocab_size"], seed=9)
    check(H.run_tail_decoded(ex, "one-by-one", ids, tail=5), model_dir, ids, dtype, f"{name} from the first token on")


def test_most_in_one_step_then_last_32_one_by_one(tiny, backend):
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=40)
    ids = H.random_ids(97, t["config"]["vocab_size"], seed=2)
    check(H.run_tail_decoded(ex, "r", ids, tail=32), model_dir, ids, dtype, f"{name} tail decoded")


def test_portions_of_changing_size(tiny, backend):
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=40)
    ids = H.random_ids(131, t["config"]["vocab_size"], seed=3)
    for sizes in ([17, 2, 9, 3, 2, 31], [5], [2], [64, 2, 2, 63]):
        check(H.run_portions(ex, "r", ids, sizes), model_dir, ids, dtype, f"{name} portions {sizes}")


def test_long_decoding(tiny, backend):
    """A short prompt and then two hundred single-token steps: windows pass, pages fill and are crossed."""
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=40)
    ids = H.random_ids(4 + 200, t["config"]["vocab_size"], seed=4)
    check(H.run_tail_decoded(ex, "r", ids, tail=200), model_dir, ids, dtype, f"{name} long decoding")


def test_mixed_batches_with_pages_used_again(tiny, backend):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool so small that the pages a
    finished request gives back are taken by the next one."""
    name, model_dir, t = tiny
    lengths = [40, 23, 64, 17, 51, 9, 70, 33]
    P = t["page_size"]
    # the four largest neighbours that can be live together, in whole pages, and not one page more
    live_max = max(sum(-(-n // P) for n in lengths[i : i + 4]) for i in range(len(lengths)))
    num_pages = max(live_max, max(sum(sorted(-(-n // P) for n in lengths)[-4:]), live_max))
    ex, dtype = make_executor(tiny, backend, num_pages=num_pages)
    ex.storage.poison()      # every slot holds NaN until a request writes it: a read of a slot nobody wrote shows in the logits
    reqs = {f"q{i}": H.random_ids(n, t["config"]["vocab_size"], seed=50 + i) for i, n in enumerate(lengths)}
    taken = set()
    orig_extend = ex.cache.extend

    def spy(rid, total):
        rc = orig_extend(rid, total)
        taken.update((rid, p) for p in rc.tables[0])
        return rc

    ex.cache.extend = spy
    got = H.run_mixed(ex, reqs, seed=7)
    pages_by_request = {}
    for rid, p in taken:
        pages_by_request.setdefault(p, set()).add(rid)
    assert any(len(v) > 1 for v in pages_by_request.values()), "no page was used by two requests: the pool is too large for this test"
    for rid, ids in reqs.items():
        check(got[rid], model_dir, ids, dtype, f"{name} mixed {rid}")
    assert all(p.free_count == p.capacity for p in ex.cache.pools)


def test_cuts_agree_with_each_other(tiny, backend):
    """The same request whole, decoded and in portions: the three runs of the engine agree with each other far more
    tightly than with the plain implementation (in float32 to the last bit but for the reading order of pages)."""
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=40)
    ids = H.random_ids(90, t["config"]["vocab_size"], seed=5)
    whole = H.run_whole(ex, "w", ids)
    tail = H.run_tail_decoded(ex, "t", ids, tail=32)
    parts = H.run_portions(ex, "p", ids, [13, 2, 7])
    kind, _ = backend
    # the float32 kernels sum in an order that depends on the token alone (measured: identical bits); the CPU stand-in
    # uses torch's matrix products, which do not keep that promise
    # bfloat16: a whole prompt runs the prefill attention kernel and cuBLAS at one size, single tokens the split decode
    # kernel and cuBLAS at another, so two cuts differ by independent bfloat16 roundings, like each differs from the
    # plain implementation: the same two bounds apply
    bound = (1e-6 if kind == "gpu" else 1e-5) if dtype == torch.float32 else H.BF16_BOUND
    print(f"MEASURED {name} {dtype} cuts: tail {H.scaled_error(tail, whole):.3e} portions {H.scaled_error(parts, whole):.3e}")
    assert H.scaled_error(tail, whole) < bound
    assert H.scaled_error(parts, whole) < bound
    if dtype == torch.bfloat16:
        assert H.rms_error(tail, whole) < H.BF16_RMS_BOUND and H.rms_error(parts, whole) < H.BF16_RMS_BOUND


def test_a_step_that_does_not_fit_changes_nothing(tiny, backend):
    from roost_b200.cache.manager import OutOfPages
    name, model_dir, t = tiny
    ex, dtype = make_executor(tiny, backend, num_pages=4)
    P = t["page_size"]
    ids = H.random_ids(3 * P, t["config"]["vocab_size"], seed=6)
    ex.step([StepEntry("a", ids, [])])
    with pytest.raises(OutOfPages):
        ex.step([StepEntry("b", H.random_ids(2 * P, t["config"]["vocab_size"], seed=8), [0])])
    assert "b" not in ex.cache
    ex.cache.check_invariants()
    ex.finish("a")
    out = ex.step([StepEntry("b", ids[: 2 * P], [2 * P - 1])])
    assert out.shape == (1, t["config"]["vocab_size"])


@pytest.mark.gpu
@pytest.mark.parametrize("policy", ["stream", "split", "library"])
def test_every_small_product_kernel_serves_the_engine(tiny_model_dirs, policy):
    """Decode steps through each of the kernels a product of few rows can run on (the default picks by size)."""
    name, t = "B", TINY["B"]
    model = H.make_model(tiny_model_dirs[name], torch.bfloat16, "gpu")
    model.rt.small_gemm = policy
    ex = StepExecutor(model, page_size=t["page_size"], num_pages=40, max_requests=4)
    ids = H.random_ids(60, t["config"]["vocab_size"], seed=44)
    check(H.run_tail_decoded(ex, "r", ids, tail=32), tiny_model_dirs[name], ids, torch.bfloat16, f"{name} decode with {policy} products")
    assert model.rt.kernels.gemm_tcgen05_status() == 0


@pytest.mark.gpu
def test_a_long_step_makes_its_rotation_table_once_for_all_layers(tiny_model_dirs, monkeypatch):
    """The layers have an encoding each, but equal ones share their frequencies, and a step keeps its cosines and sines
    by them: one table a step, however many layers read it. A short step makes none."""
    from roost_b200.engine.batch import ROTATION_TABLE_MIN_TOKENS
    name, t = "B", TINY["B"]
    assert t["config"]["num_hidden_layers"] > 1
    model = H.make_model(tiny_model_dirs[name], torch.bfloat16, "gpu")
    k = model.rt.kernels
    made = []
    real = k.rope_table
    monkeypatch.setattr(k, "rope_table", lambda positions, inv_freq: (made.append(positions.numel()), real(positions, inv_freq))[1])
    ex = StepExecutor(model, page_size=t["page_size"], num_pages=40, max_requests=4, use_graphs=False)
    n = ROTATION_TABLE_MIN_TOKENS + 5
    ids = H.random_ids(n + 1, t["config"]["vocab_size"], seed=45)
    ex.step([StepEntry("r", ids[:n], [n - 1])])
    assert made == [n]
    ex.step([StepEntry("r", ids[n:], [0])])
    assert made == [n]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_captured_step_filled_up_with_padding_rows(tiny_model_dirs, dtype):
    """Eleven, then nine decoding requests are served by the captured step of twelve rows. The logits are those of an
    executor without graphs and of the plain implementation, and no byte of the cache outside the requests' own slots
    changes (a padding row writes nothing)."""
    from roost_b200.engine.executor import graph_rows
    name, t = "B", TINY["B"]
    V, P = t["config"]["vocab_size"], t["page_size"]
    model = H.make_model(tiny_model_dirs[name], dtype, "gpu")
    execs = [StepExecutor(model, page_size=P, num_pages=48, max_requests=16, use_graphs=g) for g in (True, False)]
    for ex in execs:
        for ten in ex.storage.tensors:
            ten.fill_(7.0)
    seqs = {f"r{i}": H.random_ids(3 + i, V, seed=300 + i) for i in range(11)}
    logits = []
    for ex in execs:
        got = []
        live = dict((k, list(v)) for k, v in seqs.items())
        ex.step([StepEntry(r, ids, []) for r, ids in live.items()])
        for step in range(10):
            if step == 5:
                for r in ("r2", "r7"):
                    ex.finish(r)
                    del live[r]
            nxt = {r: H.random_ids(1, V, seed=900 + 31 * step + i)[0] for i, r in enumerate(live)}
            got.append(ex.step([StepEntry(r, [tok], [0]) for r, tok in nxt.items()]))
            for r, tok in nxt.items():
                live[r].append(tok)
        logits.append(got)
        final = live
    graphs, eager = execs
    assert graph_rows(11) == graph_rows(9) == 12
    assert graphs.graph_replays >= 8 and set(k[0] for k in graphs._graphs) == {12}
    for a, b in zip(*logits):
        assert a.shape == b.shape and a.shape[0] in (11, 9)
        assert H.scaled_error(a, b) <= H.bound_for(dtype) / 4
    for r, row in zip(final, logits[0][-1]):
        want = H.plain_logits(tiny_model_dirs[name], final[r], dtype == torch.bfloat16)[-1]
        assert H.scaled_error(row, want) <= H.bound_for(dtype), r
    for a, b in zip(graphs.storage.tensors, eager.storage.tensors):
        if a.numel() == 0:
            continue   # the group of fixed-size state, which this architecture leaves empty
        untouched = b == 7.0
        assert untouched.any() and bool((a[untouched] == 7.0).all())
        assert H.scaled_error(a, b) <= H.bound_for(dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["B", "C"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_steps_of_prompt_portions_beside_decoded_tokens_replayed_from_captured_graphs(tiny_model_dirs, name, dtype):
    """The same sizes of mixed steps come again and again (a scheduler that fills a token budget): from their second
    coming on they are captured and replayed, filled up with padding rows and tokens. Every step's logits are those of
    an executor without graphs; the last ones are checked against the plain implementation; requests longer than the
    window, pages used again."""
    t = TINY[name]
    V, P = t["config"]["vocab_size"], t["page_size"]
    model = H.make_model(tiny_model_dirs[name], dtype, "gpu")
    pages = 4 * (-(-100 // P)) + 2
    execs = [StepExecutor(model, page_size=P, num_pages=pages, max_requests=8, use_graphs=g) for g in (True, False)]
    results = []
    for ex in execs:
        got, hist = [], {}
        for rep in range(4):
            a, b, c = (f"{x}{rep}" for x in "abc")
            hist[a] = H.random_ids(50 + rep, V, seed=10 * rep + 1)
            hist[b] = H.random_ids(21, V, seed=10 * rep + 2)
            ex.step([StepEntry(a, hist[a], []), StepEntry(b, hist[b], [])])                  # sizes differ from rep to rep: eager
            prompt = H.random_ids(37, V, seed=10 * rep + 3)
            hist[c] = []
            cuts = [(0, 13), (13, 27), (27, 37)]
            for lo, hi in cuts:                                                               # 2 decoded tokens beside a portion
                na, nb = H.random_ids(2, V, seed=100 * rep + lo)
                want_c = [hi - lo - 1] if hi == 37 else []
                got.append(ex.step([StepEntry(a, [na], [0]), StepEntry(c, prompt[lo:hi], want_c), StepEntry(b, [nb], [0])]))
                hist[a].append(na); hist[b].append(nb); hist[c] = prompt[:hi]
            final = {r: list(hist[r]) for r in (a, b, c)}
            for r in (a, b, c):
                ex.finish(r)
        results.append(got)
        ex.cache.check_invariants()
    graphs, eager = execs
    mixed_keys = [k for k in graphs._graphs if k[0] != k[1]]
    assert mixed_keys and graphs.graph_replays >= 4, (list(graphs._graphs), graphs.graph_replays)
    for i, (x, y) in enumerate(zip(*results)):
        assert x.shape == y.shape, i
        assert H.scaled_error(x, y) <= H.bound_for(dtype) / 4, i
    last = results[0][-1]      # rows: a's decoded token, c's last prompt token, b's decoded token
    order = list(final)        # a, b, c
    for row, r in zip(last, (order[0], order[2], order[1])):
        want = H.plain_logits(tiny_model_dirs[name], final[r], dtype == torch.bfloat16)[-1]
        assert H.scaled_error(row, want) <= H.bound_for(dtype), r
