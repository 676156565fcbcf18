"""Each kernel alone against a plain torch float64 restatement of the same op, at sizes other than the engine's
tiny models: widths and vocabularies that are no power of two, head sizes in steps of 16, odd group sizes."""
import functools
import math

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-6 if dtype == torch.float32 else 2.0 ** -7) * scale


def close(got, want, dtype, what, scale=1.0):
    err = float(((got.double().cpu() - want.double().cpu()).abs() / (1 + want.double().cpu().abs())).max())
    print(f"MEASURED {what} {dtype}: {err:.3e}")
    assert err < tol(dtype, scale), f"{what}: {err}"


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(80, 131), (1000, 50)])
def test_embedding(kernels, dtype, hidden, vocab):
    table = rand((vocab, hidden), dtype, 1)
    ids = torch.tensor([0, vocab - 1, 3, 3, vocab, -1, 7], dtype=torch.int32).cuda()
    out = kernels.embedding(table, ids)
    want = plain.embedding(table.cpu(), [0, vocab - 1, 3, 3, 0, 0, 7]).clone()
    want[4] = 0
    want[5] = 0  # an id outside the vocabulary gives a zero row on the device
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(5, 72, 1e-6), (33, 1000, 1e-5), (2, 5120, 1e-6)])
def test_rms_norm_and_fused_add(kernels, dtype, wdtype, rows, hidden, eps):
    x = rand((rows, hidden), dtype, 2, 3.0)
    res = rand((rows, hidden), dtype, 3, 2.0)
    w = (1 + 0.1 * torch.randn(hidden, generator=torch.Generator().manual_seed(4))).to(wdtype).cuda()
    close(kernels.rms_norm(x, w, eps), plain.rms_norm(x.double().cpu(), w.double().cpu(), eps), dtype, "rms_norm")
    sel = torch.tensor([rows - 1, 0], dtype=torch.int32).cuda()
    close(kernels.rms_norm(x, w, eps, sel), plain.rms_norm(x.double().cpu(), w.double().cpu(), eps)[[rows - 1, 0]], dtype, "rms_norm rows")
    s = (x.float() + res.float()).to(dtype)  # the sum is rounded once to the activation dtype
    res_in = res.clone()
    out = kernels.add_rms_norm(x, res_in, w, eps)
    assert torch.equal(res_in, s)
    close(out, plain.rms_norm(s.double().cpu(), w.double().cpu(), eps), dtype, "add_rms_norm")
    res_in2 = res.clone()
    out2 = kernels.add_rms_norm(x, res_in2, w, eps, sel)
    assert torch.equal(res_in2, res), "with gathered rows the residual stays as it is"
    close(out2, plain.rms_norm(s.double().cpu(), w.double().cpu(), eps)[[rows - 1, 0]], dtype, "add_rms_norm rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,inter", [(3, 100), (17, 1111)])
def test_silu_mul(kernels, dtype, tokens, inter):
    x = rand((tokens, 2 * inter), dtype, 5, 3.0)
    xd = x.double().cpu()
    close(kernels.silu_mul(x), plain.silu_and_mul(xd[:, :inter], xd[:, inter:]), dtype, "silu_mul")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 70, 50), (37, 129, 200), (130, 64, 1024), (64, 387, 96)])
def test_gemm_simt(kernels, dtype, m, n, k):
    a = rand((m, k), dtype, 6)
    w = rand((n, k), dtype, 7)
    want = a.double().cpu() @ w.double().cpu().T
    # float32: k additions into a running sum of size ~sqrt(k), each rounded to 2^-24 relative: an absolute error of
    # the order k * 2^-24 sqrt(...) at worst, against outputs that may be near zero; the bound is k * 2^-23.
    fp32_scale = k * 2.0 ** -23 / 2e-6
    close(kernels.gemm_simt(a, w), want, dtype, "gemm", scale=fp32_scale if dtype == torch.float32 else math.sqrt(k) / 8)
    if dtype == torch.bfloat16:
        close(kernels.gemm_simt(a, w, torch.float32), want, torch.float32, "gemm f32 out", scale=fp32_scale)
    # a row's bits do not depend on which other rows are in the product
    if m > 1:
        assert torch.equal(kernels.gemm_simt(a[m // 2 : m // 2 + 1].contiguous(), w), kernels.gemm_simt(a, w)[m // 2 : m // 2 + 1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(4, 2, 16, 16, 16), (6, 1, 32, 32, 8), (5, 5, 48, 32, 4), (8, 2, 128, 128, 16), (3, 1, 80, 80, 32)])
def test_qk_norm_rope_cache(kernels, dtype, nq, nkv, d, rot, page):
    T, pages = 11, 9
    eps, theta = 1e-5, 1e6
    qkv = rand((T, (nq + 2 * nkv) * d), dtype, 8, 2.0)
    qw = (1 + 0.1 * torch.randn(d, generator=torch.Generator().manual_seed(9))).to(dtype).cuda()
    kw = (1 + 0.1 * torch.randn(d, generator=torch.Generator().manual_seed(10))).to(dtype).cuda()
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 4095, 100000, 7, 8, 9], dtype=torch.int32).cuda()
    slots = torch.tensor([5, 30, 3, -1, 0, page * pages - 1, 17, 18, 19, 33, 34], dtype=torch.int32)  # distinct, below 36
    assert page * pages >= 36
    slots = slots.cuda()
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).cuda()
    kp = torch.full((pages, nkv, page, d), 7.0, dtype=dtype).cuda()
    vp = torch.full((pages, nkv, page, d), 7.0, dtype=dtype).cuda()
    q = kernels.qk_norm_rope_cache(qkv, nq, nkv, d, q_w=qw, k_w=kw, eps=eps, inv_freq=inv_freq, rotary_dim=rot, positions=positions,
                                   k_pool=kp, v_pool=vp, slot_mapping=slots, page_size=page)
    x = qkv.double().cpu()
    qq = x[:, : nq * d].reshape(T, nq, d)
    kk = x[:, nq * d : (nq + nkv) * d].reshape(T, nkv, d)
    vv = x[:, (nq + nkv) * d :].reshape(T, nkv, d)
    qq, kk = plain.qk_norm(qq, kk, qw.double().cpu(), kw.double().cpu(), eps)
    pos = positions.cpu().tolist()
    qq = plain.rope_neox(qq, pos, theta, rot)
    kk = plain.rope_neox(kk, pos, theta, rot)
    close(q, qq, dtype, "q normed and rotated", scale=2)
    want_k = torch.full((pages, nkv, page, d), 7.0, dtype=torch.float64)
    want_v = want_k.clone()
    for t, s in enumerate(slots.cpu().tolist()):
        if s >= 0:
            want_k[s // page, :, s % page, :] = kk[t]
            want_v[s // page, :, s % page, :] = vv[t]
    close(kp, want_k, dtype, "k pages", scale=2)
    assert torch.equal(vp.double().cpu(), want_v), "values are copied bit for bit, and no other slot is touched"
    kp2, vp2 = torch.full_like(kp, 7.0), torch.full_like(vp, 7.0)
    q_t = kernels.qk_norm_rope_cache(qkv, nq, nkv, d, q_w=qw, k_w=kw, eps=eps, inv_freq=inv_freq, rotary_dim=rot, positions=positions,
                                     k_pool=kp2, v_pool=vp2, slot_mapping=slots, page_size=page, cos_sin=kernels.rope_table(positions, inv_freq))
    assert torch.equal(q_t, q) and torch.equal(kp2, kp) and torch.equal(vp2, vp), "the step's table gives the same bits"
    # q only (a run that reads another run's cache), no norm, no rotation
    q2 = kernels.qk_norm_rope_cache(qkv[:, : nq * d].contiguous(), nq, nkv, d, q_w=None, k_w=None, eps=eps, inv_freq=None, rotary_dim=0,
                                    positions=positions, write_kv=False)
    assert torch.equal(q2.reshape(T, -1), qkv[:, : nq * d])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,nq,nkv,d,page,weights", [(64, 8, 2, 128, 16, "same"), (300, 5, 3, 64, 8, "float32"), (1100, 3, 1, 256, 32, "same"),
                                                     (1030, 4, 4, 128, 16, None), (70, 2, 1, 96, 16, "same"),
                                                     # head slots that share a warp's pass and take different branches: key
                                                     # heads beside value heads, a query head beside a key head, a value head
                                                     # and an empty slot
                                                     (150, 4, 2, 64, 16, "same"), (70, 5, 1, 64, 16, "float32"), (90, 3, 1, 128, 16, "same"),
                                                     # so many tokens that one part serves all the head slots of a token, and
                                                     # parts of several slots whose last is shorter
                                                     (9600, 2, 1, 128, 16, "same"), (2048, 7, 2, 128, 16, "same")])
def test_qk_norm_rope_cache_of_many_tokens(kernels, dtype, T, nq, nkv, d, page, weights):
    """Steps of many tokens (bfloat16 heads of 64, 128 or 256 take a kernel of their own): a token's head slots in one or
    several parts, some tokens skipped (slot -1), slots scattered over the pool, norm weights in either dtype or none."""
    eps, theta = 1e-6, 1e6
    g = torch.Generator().manual_seed(T + d)
    pages = -(-T // page) + 3
    qkv = rand((T, (nq + 2 * nkv) * d), dtype, T, 2.0)
    wdtype = torch.float32 if weights == "float32" else dtype
    qw = kw = None
    if weights is not None:
        qw = (1 + 0.1 * torch.randn(d, generator=g)).to(wdtype).cuda()
        kw = (1 + 0.1 * torch.randn(d, generator=g)).to(wdtype).cuda()
    positions = torch.randint(0, 200000, (T,), generator=g, dtype=torch.int32)
    positions[:3] = torch.tensor([0, 1, 131071], dtype=torch.int32)
    slots = torch.randperm(page * pages, generator=g)[:T].to(torch.int32)
    slots[torch.randperm(T, generator=g)[: T // 9]] = -1
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(d // 2, dtype=torch.float64) / d).cuda()
    kp = torch.full((pages, nkv, page, d), 7.0, dtype=dtype).cuda()
    vp = torch.full((pages, nkv, page, d), 7.0, dtype=dtype).cuda()
    q = kernels.qk_norm_rope_cache(qkv, nq, nkv, d, q_w=qw, k_w=kw, eps=eps, inv_freq=inv_freq, rotary_dim=d, positions=positions.cuda(),
                                   k_pool=kp, v_pool=vp, slot_mapping=slots.cuda(), page_size=page)
    x = qkv.double().cpu()
    qq = x[:, : nq * d].reshape(T, nq, d)
    kk = x[:, nq * d : (nq + nkv) * d].reshape(T, nkv, d)
    vv = x[:, (nq + nkv) * d :].reshape(T, nkv, d)
    if weights is not None:
        qq, kk = plain.qk_norm(qq, kk, qw.double().cpu(), kw.double().cpu(), eps)
    pos = positions.tolist()
    qq = plain.rope_neox(qq, pos, theta, d)
    kk = plain.rope_neox(kk, pos, theta, d)
    close(q, qq, dtype, "q normed and rotated", scale=2)
    want_k = torch.full((pages, nkv, page, d), 7.0, dtype=torch.float64)
    want_v = want_k.clone()
    for t, s_ in enumerate(slots.tolist()):
        if s_ >= 0:
            want_k[s_ // page, :, s_ % page, :] = kk[t]
            want_v[s_ // page, :, s_ % page, :] = vv[t]
    close(kp, want_k, dtype, "k pages", scale=2)
    assert torch.equal(vp.double().cpu(), want_v), "values are copied bit for bit, and no other slot is touched"
    untouched = want_k == 7.0
    assert torch.equal(kp.double().cpu()[untouched], want_k[untouched])
    # with the step's table of cosines and sines (computed once for all layers) the bits are the same
    kp2, vp2 = torch.full_like(kp, 7.0), torch.full_like(vp, 7.0)
    table = kernels.rope_table(positions.cuda(), inv_freq)
    q2 = kernels.qk_norm_rope_cache(qkv, nq, nkv, d, q_w=qw, k_w=kw, eps=eps, inv_freq=inv_freq, rotary_dim=d, positions=positions.cuda(),
                                    k_pool=kp2, v_pool=vp2, slot_mapping=slots.cuda(), page_size=page, cos_sin=table)
    assert torch.equal(q2, q) and torch.equal(kp2, kp) and torch.equal(vp2, vp)


def paged_reference(q, keys, values, positions, rows, scale, window):
    """q [T, nq, d]; keys/values: per row a [len, nkv, d] tensor; float64."""
    out = torch.zeros(q.shape[0], q.shape[1] * q.shape[2], dtype=torch.float64)
    group = q.shape[1] // keys[0].shape[1]
    for t in range(q.shape[0]):
        p, b = positions[t], rows[t]
        lo = max(0, p - window + 1) if window else 0
        k, v = keys[b][lo : p + 1], values[b][lo : p + 1]
        for h in range(q.shape[1]):
            s = (k[:, h // group] @ q[t, h]) * scale
            out[t, h * q.shape[2] : (h + 1) * q.shape[2]] = torch.softmax(s, 0) @ v[:, h // group]
    return out


def build_paged(keys, values, page, dtype, num_pages, seed):
    """Scatters per-row keys and values into shuffled pages; unused slots hold NaN so that a read of a slot that is
    not the row's shows."""
    nkv, d = keys[0].shape[1:]
    pool = torch.full((2, num_pages, nkv, page, d), float("nan"), dtype=dtype)   # keys then values, as the engine's cache holds them
    kp, vp = pool[0], pool[1]
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    indptr, indices = [0], []
    for k, v in zip(keys, values):
        n = k.shape[0]
        for pi in range(-(-n // page)):
            pg = order.pop()
            indices.append(pg)
            seg = slice(pi * page, min(n, (pi + 1) * page))
            kp[pg, :, : seg.stop - seg.start] = k[seg].transpose(0, 1).to(dtype)
            vp[pg, :, : seg.stop - seg.start] = v[seg].transpose(0, 1).to(dtype)
        indptr.append(len(indices))
    pool = pool.cuda()
    return pool[0], pool[1], torch.tensor(indptr, dtype=torch.int32).cuda(), torch.tensor(indices, dtype=torch.int32).cuda()


def release_passed_pages(kp, vp, indptr, indices, lens, news, window, page):
    """What the cache manager's commit leaves of a windowed request before a step: every page wholly below
    (tokens held before the step) - window has gone back to the pool, its block-table entry is -1 and, here, its
    slots hold NaN (the pool's next user may have written anything). Returns how many pages were released."""
    released = 0
    if not window:
        return 0
    table = indices.cpu().clone()
    ptr = indptr.cpu().tolist()
    for b, (n, m) in enumerate(zip(lens, news)):
        start = n - m
        gone = (start - window) // page if start > window else 0
        for i in range(gone):
            pg = int(table[ptr[b] + i])
            kp[pg] = float("nan")
            vp[pg] = float("nan")
            table[ptr[b] + i] = -1
            released += 1
    indices.copy_(table)
    return released


ATTN_SHAPES = [(4, 2, 16, 16), (6, 1, 32, 8), (8, 2, 128, 16), (5, 5, 48, 4), (14, 2, 64, 32), (3, 1, 80, 16), (2, 1, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("nq,nkv,d,page", ATTN_SHAPES)
def test_paged_attention_mixed_rows(kernels, dtype, window, nq, nkv, d, page):
    """Three rows in one launch: a whole prompt, a portion in the middle of a request, a single decoded token."""
    g = torch.Generator().manual_seed(11)
    lens = [45, 133, 300]           # keys each row holds after this step
    news = [45, 21, 1]              # queries each row brings (the last `news` positions)
    keys = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    values = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    positions, rows = [], []
    for b, (n, m) in enumerate(zip(lens, news)):
        positions += list(range(n - m, n))
        rows += [b] * m
    T = len(positions)
    q = (torch.randn(T, nq, d, generator=g) * 1.5).to(dtype)
    kp, vp, indptr, indices = build_paged(keys, values, page, dtype, num_pages=sum(-(-n // page) for n in lens) + 3, seed=12)
    if window:
        assert release_passed_pages(kp, vp, indptr, indices, lens, news, window, page) > 0
    scale = 1 / math.sqrt(d)
    out = kernels.paged_attention_generic(q.cuda(), kp, vp, torch.tensor(positions, dtype=torch.int32).cuda(),
                                          torch.tensor(rows, dtype=torch.int32).cuda(), indptr, indices, scale, window)
    want = paged_reference(q.double(), keys, values, positions, rows, scale, window)
    assert not torch.isnan(out).any(), "a slot outside the row's visible keys was read"
    # a dot product over head_dim and a softmax over hundreds of keys, each in 32-bit: four times the elementwise bound
    close(out, want, dtype, f"attention window={window}", scale=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["far key", "first key", "page edge", "window edge in", "window edge out"])
def test_paged_attention_finds_the_one_key_that_matters(kernels, dtype, case):
    """Random keys would hide a key that is skipped or read from the wrong slot. Here one key's score stands out by
    construction, so the output must be that key's value (or, for a key just outside the window, must not be)."""
    nq, nkv, d, page, n = 4, 2, 64, 16, 700
    window = None
    target = {"far key": 3, "first key": 0, "page edge": 16 * 20 - 1, "window edge in": n - 50, "window edge out": n - 51}[case]
    if case.startswith("window"):
        window = 50
    g = torch.Generator().manual_seed(13)
    keys = torch.randn(n, nkv, d, generator=g) * 0.1
    values = torch.randn(n, nkv, d, generator=g)
    q = torch.randn(1, nq, d, generator=g) * 0.1
    direction = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
    keys[target] = direction * 8.0
    q[0, :] = direction * 8.0                      # score 64 / sqrt(64) * ... = 8 * 8 / 8 = 8 at the target, ~0 elsewhere
    q = q * 2                                       # 16 at the target: exp(16) dwarfs 700 keys of exp(~0)
    keys_d, values_d = keys.to(dtype).double(), values.to(dtype).double()
    kp, vp, indptr, indices = build_paged([keys_d], [values_d], page, dtype, num_pages=-(-n // page) + 2, seed=14)
    out = kernels.paged_attention_generic(q.to(dtype).cuda(), kp, vp, torch.tensor([n - 1], dtype=torch.int32).cuda(),
                                          torch.tensor([0], dtype=torch.int32).cuda(), indptr, indices, 1 / math.sqrt(d), window)
    want = paged_reference(q.to(dtype).double(), [keys_d], [values_d], [n - 1], [0], 1 / math.sqrt(d), window)
    close(out, want, dtype, case, scale=4)
    got_v = out.double().cpu().reshape(nq, d)
    hit = (got_v - values_d[target][torch.arange(nq) // 2]).abs().max() < 0.05
    assert hit == (case != "window edge out"), f"{case}: output {'is' if hit else 'is not'} the target's value"


def test_argmax_ties_and_nan(kernels):
    V = 151936 // 8 + 3
    z = torch.randn(4, V)
    z[0, 77] = 50.0
    z[0, 9000] = 50.0          # a tie: the lower index wins
    z[1, 5] = float("nan")     # never chosen
    z[1, 6] = 40.0
    z[2] = float("nan")        # nothing to choose
    z[3, V - 1] = 60.0
    ids = kernels.argmax(z.cuda()).cpu().tolist()
    assert ids == [77, 6, -1, V - 1]
    # a vocabulary large enough for a row to be split over sixteen blocks: ties across spans, maxima at span edges,
    # a row of NaN, and the counters left clean for a second call with other values
    V = 151936
    span = (((V + 15) // 16) + 3) & ~3
    for seed in (1, 2):
        z = torch.randn(9, V, generator=torch.Generator().manual_seed(seed))
        z[0, 77] = 50.0
        z[0, 9 * span + 1] = 50.0      # the same value in a later span: the lower index wins
        z[1, 5] = float("nan")
        z[1, 3 * span] = 40.0          # first element of a span
        z[2] = float("nan")
        z[3, V - 1] = 60.0             # last element of the last span
        z[4, span - 1] = 45.0          # last element of the first span
        z[4, span] = 45.0
        z[5, 12 * span + 7] = 33.0
        want = []
        for r in range(9):
            row = z[r]
            ok = ~torch.isnan(row)
            want.append(int(torch.where(ok, row, torch.tensor(-float("inf"))).argmax()) if ok.any() else -1)
        assert want[:6] == [77, 3 * span, -1, V - 1, span - 1, 12 * span + 7]
        assert kernels.argmax(z.cuda()).cpu().tolist() == want


@pytest.mark.parametrize("vocab", [387, 5000, 151936, 200003])
def test_sampler_matches_the_plain_sampler(kernels, vocab):
    """Rows with different settings in one launch; a row is compared when the plain sampler's draw is not within
    1e-4 of the kept mass from an edge of the chosen token's interval. The sizes take both kernels: a block a row (the
    smallest, and the largest, whose eighth no longer fits a block's shared memory) and a cluster of eight a row."""
    g = torch.Generator().manual_seed(15)
    settings = [(0.0, 0, 1.0, 0.0), (1.0, 0, 1.0, 0.0), (0.8, 0, 0.9, 0.0), (0.7, 20, 1.0, 0.0), (1.3, 50, 0.8, 0.0),
                (1.0, 0, 1.0, 0.05), (0.9, 40, 0.95, 0.02), (0.5, 1, 1.0, 0.0), (2.0, 0, 0.5, 0.0), (1.0, 3, 0.2, 0.0)]
    rows = []
    for rep in range(4 if vocab < 100000 else 1):     # the plain sampler sorts a row in Python: one pass at the real vocabulary
        for s in settings:
            rows.append(s)
    R = len(rows)
    # at the real vocabulary a flatter row gives every token an interval of a few millionths of the mass, within the
    # margin below of its edges: the rows are made more peaked there so that most draws can be compared
    logits = torch.randn(R, vocab, generator=g) * (3 if vocab < 100000 else 6)
    logits[3, 10] = float("-inf")
    logits[4, 11] = float("nan")
    logits[5, 40:44] = logits[5, 40]            # ties in the middle of the order
    logits[1] = 1.25                            # every token the same: one bucket holds the whole row, the draw is a rank among ties
    logits[8, ::2] = 2.0                        # two values, half the row each
    logits[8, 1::2] = 1.0
    seeds = torch.arange(R, dtype=torch.int64) * 7919 + 12345
    offsets = torch.arange(R, dtype=torch.int64) % 5
    t = torch.tensor([r[0] for r in rows], dtype=torch.float32)
    k = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    p = torch.tensor([r[2] for r in rows], dtype=torch.float32)
    mp = torch.tensor([r[3] for r in rows], dtype=torch.float32)
    got = kernels.sample(logits.cuda(), t.cuda(), k.cuda(), p.cuda(), mp.cuda(), seeds.cuda(), offsets.cuda()).cpu().tolist()
    again = kernels.sample(logits.cuda(), t.cuda(), k.cuda(), p.cuda(), mp.cuda(), seeds.cuda(), offsets.cuda()).cpu().tolist()
    assert got == again, "the sampler is not repeatable"
    compared = 0
    for r in range(R):
        temp, tk, tp, m = rows[r]
        if temp <= 0:
            assert got[r] == plain.sample_row(logits[r].tolist(), 0.0)
            compared += 1
            continue
        want, detail = plain.sample_row(logits[r].tolist(), temp, tk, tp, m, int(seeds[r]), int(offsets[r]), return_detail=True)
        assert got[r] in detail["kept"] or detail["margin"] < 1e-4, f"row {r}: token {got[r]} is outside the kept set"
        if detail["margin"] > 1e-4:
            assert got[r] == want, f"row {r} {rows[r]}: got {got[r]}, want {want} (margin {detail['margin']:.2e})"
            compared += 1
    assert compared >= R * (0.8 if vocab < 100000 else 0.7), compared
    # a row's token does not depend on the batch it is in
    one = kernels.sample(logits[7:8].cuda(), t[7:8].cuda(), k[7:8].cuda(), p[7:8].cuda(), mp[7:8].cuda(), seeds[7:8].cuda(), offsets[7:8].cuda())
    assert one.cpu().tolist() == [got[7]]
    # nor on how many CTAs share a row: up to eight rows a launch take clusters of eight, more take clusters of four,
    # and every sum is a sum of integers
    def twice(x):
        return torch.cat([x, x]).cuda()
    both = kernels.sample(twice(logits[:8]), twice(t[:8]), twice(k[:8]), twice(p[:8]), twice(mp[:8]), twice(seeds[:8]), twice(offsets[:8])).cpu().tolist()
    few = kernels.sample(logits[:8].cuda(), t[:8].cuda(), k[:8].cuda(), p[:8].cuda(), mp[:8].cuda(), seeds[:8].cuda(), offsets[:8].cuda()).cpu().tolist()
    assert both[:8] == both[8:] == few == got[:8]


# ------------------------------------------------------------------------------------------ tensor-core attention (bfloat16)
def run_mma(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, chunk=None, tile_rows=None, cluster=0):
    from roost_b200.parts.attention_work import plan_attention
    nq, nkv = q.shape[1], kp.shape[1]
    starts = [n - m for n, m in zip(lens, news)]
    plan = plan_attention(starts, news, nq // nkv, window, chunk or kernels.decode_chunk, "cuda",
                          tile_rows or kernels.attention_prefill_tile_rows(nq, kp, vp), cluster)
    q_indptr = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32).cuda()
    kv_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    return kernels.attention_mma(q.cuda(), kp, vp, q_indptr, kv_lens, indptr, indices, plan, scale, window), plan


MMA_SHAPES = [(4, 2, 16, 16), (6, 1, 32, 8), (8, 2, 128, 16), (14, 2, 64, 32), (2, 1, 256, 16), (16, 1, 64, 16), (40, 2, 128, 16),
              (8, 2, 64, 32), (4, 1, 128, 64)]


@pytest.mark.parametrize("chunk", [512, 1024])
@pytest.mark.parametrize("window", [None, 37, 300])
@pytest.mark.parametrize("nq,nkv,d,page", MMA_SHAPES)
def test_attention_mma_mixed_rows(kernels, window, nq, nkv, d, page, chunk):
    """A whole prompt, a portion in the middle of a request, a two-token portion after a long history, single decoded
    tokens after short and long histories (several chunks of the split decode kernel, for both chunk sizes the engine
    uses), all in one launch. Under a window the pages the window has passed are gone (entry -1, slots NaN), as the cache
    manager leaves them."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(21)
    lens = [45, 233, 700, 19, 1000, 257, 2300]
    news = [45, 121, 2, 1, 1, 1, 1]
    keys = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    values = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    positions, rows = [], []
    for b, (n, m) in enumerate(zip(lens, news)):
        positions += list(range(n - m, n))
        rows += [b] * m
    q = (torch.randn(len(positions), nq, d, generator=g) * 1.5).to(dtype)
    kp, vp, indptr, indices = build_paged(keys, values, page, dtype, num_pages=sum(-(-n // page) for n in lens) + 5, seed=22)
    if window:
        assert release_passed_pages(kp, vp, indptr, indices, lens, news, window, page) > 0
    scale = 1 / math.sqrt(d)
    run = functools.partial(run_mma, chunk=chunk)      # every run below uses this test's chunk size

    out, plan = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window)
    assert plan.prefill_items > 0 and (nq // nkv > 16 or (plan.decode_items > 0 and (plan.merge_items > 0 or window is not None)))
    want = paged_reference(q.double(), keys, values, positions, rows, scale, window)
    assert not torch.isnan(out.float()).any(), "a slot outside the rows' visible keys was read"
    # the softmax weights are rounded to bfloat16 for the second product: 2^-8 of the values' size on top of the
    # output's own rounding (the reference's attention tolerance, 2^-7 rtol + 2^-8 max|V|, op-class-tolerances)
    close(out, want, dtype, f"attention_mma window={window}", scale=2)
    # the 32-bit kernel gives the same answer within the same bound
    generic = kernels.paged_attention_generic(q.cuda(), kp, vp, torch.tensor(positions, dtype=torch.int32).cuda(),
                                              torch.tensor(rows, dtype=torch.int32).cuda(), indptr, indices, scale, window)
    close(out, generic.double(), dtype, "attention_mma against the 32-bit kernel", scale=2)
    # the decode rows again through the cp.async kernel (where the copy-engine kernel served them above)
    kernels.attention_set_decode_tma(False)
    try:
        plain_copy, _ = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window)
    finally:
        kernels.attention_set_decode_tma(True)
    assert kernels.attention_status() == 0, "a bounded wait inside the decode kernel was given up"
    assert not torch.isnan(plain_copy.float()).any()
    close(plain_copy, want, dtype, f"attention_mma (cp.async decode) window={window}", scale=2)
    # the prompt portions again through the mma.sync kernel (where the tcgen05 kernel served them above)
    kernels.attention_set_prefill_tc(False)
    try:
        legacy, _ = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window)
    finally:
        kernels.attention_set_prefill_tc(True)
    assert kernels.attention_status() == 0, "a bounded wait inside an attention kernel was given up"
    assert not torch.isnan(legacy.float()).any()
    close(legacy, want, dtype, f"attention_mma (mma.sync prefill) window={window}", scale=2)
    group = nq // nkv
    tc_serves = d in (64, 128) and group & (group - 1) == 0 and page >= 16
    assert torch.equal(legacy, out) != tc_serves, "the tcgen05 kernel serves exactly these sizes (its tiles round differently)"
    if tc_serves:
        # two row groups a CTA (work items of 256 packed rows) compute every row as one group does
        both, both_plan = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, tile_rows=256)
        assert both_plan.prefill_items < plan.prefill_items
        assert torch.equal(both, out), "one and two row groups a CTA differ"
    if d <= 128:
        # work items of 128 packed rows (two row tiles a warp) compute every row with the same operations in the same order
        kernels.attention_set_prefill_tc(False)
        try:
            wide, wide_plan = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, tile_rows=128)
            narrow, narrow_plan = run(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, tile_rows=64)
        finally:
            kernels.attention_set_prefill_tc(True)
        assert wide_plan.prefill_items < narrow_plan.prefill_items or nq // nkv * max(news) <= 64
        assert torch.equal(wide, narrow), "64-row and 128-row prefill tiles differ"


@pytest.mark.parametrize("case", ["far key", "first key", "page edge", "chunk edge 511", "chunk edge 512", "chunk edge 1023", "chunk edge 1024",
                                  "window edge in", "window edge out"])
@pytest.mark.parametrize("queries", [1, 40])
@pytest.mark.parametrize("chunk", [512, 1024])
def test_attention_mma_finds_the_one_key_that_matters(kernels, case, queries, chunk):
    dtype = torch.bfloat16
    nq, nkv, d, page, n = 4, 2, 64, 16, 1300
    window = 50 if case.startswith("window") else None
    last = n - 1
    # the last and the first key of a chunk of the split decode kernel, for both chunk sizes the engine uses
    target = {"far key": 3, "first key": 0, "page edge": 16 * 20 - 1, "chunk edge 511": 511, "chunk edge 512": 512, "chunk edge 1023": 1023,
              "chunk edge 1024": 1024, "window edge in": last - 49, "window edge out": last - 50}[case]
    g = torch.Generator().manual_seed(23)
    keys = torch.randn(n, nkv, d, generator=g) * 0.1
    values = torch.randn(n, nkv, d, generator=g)
    q = torch.randn(queries, nq, d, generator=g) * 0.1
    direction = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
    keys[target] = direction * 8.0
    q[-1, :] = direction * 16.0
    keys_d, values_d = keys.to(dtype).double(), values.to(dtype).double()
    kp, vp, indptr, indices = build_paged([keys_d], [values_d], page, dtype, num_pages=-(-n // page) + 2, seed=24)
    if window:
        assert release_passed_pages(kp, vp, indptr, indices, [n], [queries], window, page) > 0
    out, _ = run_mma(kernels, q.to(dtype), kp, vp, [n], [queries], indptr, indices, 1 / math.sqrt(d), window, chunk=chunk)
    positions = list(range(n - queries, n))
    want = paged_reference(q.to(dtype).double(), [keys_d], [values_d], positions, [0] * queries, 1 / math.sqrt(d), window)
    close(out, want, dtype, f"{case} x{queries}", scale=4)
    got_v = out[-1].double().cpu().reshape(nq, d)
    hit = (got_v - values_d[target][torch.arange(nq) // 2]).abs().max() < 0.05
    assert hit == (case != "window edge out"), f"{case}: the last query's output {'is' if hit else 'is not'} the target's value"


@pytest.mark.parametrize("chunk", [512, 1024])
def test_attention_mma_rows_do_not_depend_on_the_batch(kernels, chunk):
    """A decode row alone and the same row among others: the same bits (for a given chunk size every sum's order is fixed)."""
    dtype = torch.bfloat16
    nq, nkv, d, page = 8, 2, 128, 16
    g = torch.Generator().manual_seed(25)
    lens = [900, 300, 2500]
    keys = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    values = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    q = torch.randn(3, nq, d, generator=g).to(dtype)
    kp, vp, indptr, indices = build_paged(keys, values, page, dtype, num_pages=300, seed=26)
    together, plan = run_mma(kernels, q, kp, vp, lens, [1, 1, 1], indptr, indices, 0.1, None, chunk=chunk)
    assert plan.merge_items >= 1
    alone, _ = run_mma(kernels, q[2:3], kp, vp, lens[2:], [1], torch.tensor([0, int(indptr[3] - indptr[2])], dtype=torch.int32).cuda(),
                       indices[int(indptr[2]):].contiguous(), 0.1, None, chunk=chunk)
    assert torch.equal(together[2:3], alone)
    # the two chunk sizes give the same row within rounding (a step's size class picks one of them)
    other, _ = run_mma(kernels, q, kp, vp, lens, [1, 1, 1], indptr, indices, 0.1, None, chunk=1536 - chunk)
    positions = [n - 1 for n in lens]
    want = paged_reference(q.double(), keys, values, positions, [0, 1, 2], 0.1, None)
    close(together, want, dtype, f"chunk {chunk}", scale=2)
    close(other, together.double(), dtype, "one chunk size against the other", scale=2)


@pytest.mark.parametrize("window", [None, 300])
@pytest.mark.parametrize("nq,nkv,d,page,chunk,cluster", [(8, 2, 128, 16, 512, 8), (32, 8, 128, 16, 1024, 4), (14, 2, 64, 32, 512, 8),
                                                        (4, 4, 64, 16, 1024, 2), (16, 1, 128, 64, 512, 4)])
def test_attention_decode_clusters_give_the_merge_kernels_bits(kernels, nq, nkv, d, page, chunk, cluster, window):
    """Split rows merged by thread-block clusters through distributed shared memory against the same rows through partial
    results in memory and the merge kernel: the same chunks, the same order of sums, the same bits. Rows of one chunk,
    of every chunk of the cluster, of a length that ends on a chunk's edge, rows of two tokens, and a prompt portion
    beside them (which the prefill kernel takes either way)."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(61)
    top = chunk * cluster
    lens = [top, 37, chunk, chunk + 1, top - 1, 2 * chunk - 5, 700, 90]
    news = [1, 1, 1, 2, 1, 1, 2, 60]
    keys = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    values = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
    positions, rows = [], []
    for b, (n, m) in enumerate(zip(lens, news)):
        positions += list(range(n - m, n))
        rows += [b] * m
    q = (torch.randn(len(positions), nq, d, generator=g) * 1.5).to(dtype)
    kp, vp, indptr, indices = build_paged(keys, values, page, dtype, num_pages=sum(-(-n // page) for n in lens) + 3, seed=62)
    if window:
        assert release_passed_pages(kp, vp, indptr, indices, lens, news, window, page) > 0
    scale = 1 / math.sqrt(d)
    assert kernels._lib.roost_attention_decode_cluster_supported(d, page, kp.shape[0], nkv, kp.data_ptr(), vp.data_ptr())
    plain_path, plan0 = run_mma(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, chunk=chunk)
    clustered, plan1 = run_mma(kernels, q, kp, vp, lens, news, indptr, indices, scale, window, chunk=chunk, cluster=cluster)
    assert kernels.attention_status() == 0
    assert (plan0.merge_items > 0 or window) and plan1.merge_items == 0 and plan1.cluster_chunks == cluster   # a window may leave every row one chunk
    assert plan1.decode_items == cluster * sum(1 for m in news if m * (nq // nkv) <= 16)
    assert not torch.isnan(clustered.float()).any()
    assert torch.equal(clustered, plain_path)
    want = paged_reference(q.double(), keys, values, positions, rows, scale, window)
    close(clustered, want, dtype, f"clustered decode window={window}", scale=2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 272, 96), (1, 256, 64), (77, 18992, 1024), (2048, 6144, 4096), (513, 512, 12288)])
def test_gemm_tcgen05(kernels, m, n, k):
    """TMA + tcgen05 product: tiles that end inside m, n and k (zero-filled by the TMA unit), one row, many tiles a CTA."""
    a = rand((m, k), torch.bfloat16, 41)
    w = rand((n, k), torch.bfloat16, 42)
    want = a.double().cpu() @ w.double().cpu().T
    got = kernels.gemm_tcgen05(a, w)
    assert kernels.gemm_tcgen05_status() == 0, "a bounded wait inside the kernel was given up"
    close(got, want, torch.bfloat16, "gemm_tcgen05", scale=math.sqrt(k) / 8)
    got32 = kernels.gemm_tcgen05(a, w, torch.float32)
    assert kernels.gemm_tcgen05_status() == 0
    # the tensor cores add products with less than full 32-bit rounding: the same bound as the library product shows
    lib = torch.mm(a, w.t(), out_dtype=torch.float32) if hasattr(torch, "mm") else None
    err = float(((got32.double().cpu() - want).abs() / (1 + want.abs())).max())
    err_lib = float(((lib.double().cpu() - want).abs() / (1 + want.abs())).max())
    print(f"MEASURED gemm_tcgen05 f32 out: {err:.3e} (cuBLAS {err_lib:.3e})")
    assert err < max(2 * err_lib, k * 2.0 ** -23)
    assert not kernels.gemm_tcgen05_supported(m, n, k + 4, k + 4, k + 4)


@pytest.mark.parametrize("m,inter,k", [(64, 128, 64), (200, 384, 96), (2048, 12288, 4096)])
def test_gemm_tcgen05_swiglu(kernels, m, inter, k):
    a = rand((m, k), torch.bfloat16, 43)
    gate = rand((inter, k), torch.bfloat16, 44, 1 / math.sqrt(k))
    up = rand((inter, k), torch.bfloat16, 45, 1 / math.sqrt(k))
    w = torch.stack([gate.reshape(inter // 128, 128, k), up.reshape(inter // 128, 128, k)], dim=1).reshape(2 * inter, k).contiguous()
    got = kernels.gemm_tcgen05_swiglu(a, w)
    assert kernels.gemm_tcgen05_status() == 0
    ad = a.double().cpu()
    want = plain.silu_and_mul(ad @ gate.double().cpu().T, ad @ up.double().cpu().T)
    close(got, want, torch.bfloat16, "gemm_tcgen05_swiglu")
    # the unfused pair on the same interleaved layout
    two = kernels.silu_mul(torch.matmul(a, w.t()), 128)
    close(two, want, torch.bfloat16, "library product + silu_mul on the interleaved layout", scale=2)


@pytest.mark.parametrize("m,inter,k", [(1, 128, 256), (8, 384, 200), (8, 12288, 4096), (16, 3072, 1024), (23, 1280, 2560)])
def test_gemm_split_swiglu(kernels, m, inter, k):
    """The k-split product with the activation on the summed accumulators: gate and up of an output in two accumulators
    that share x, both summed over the cluster before silu(gate) * up; repeatable and independent of the batch."""
    assert kernels.gemm_split_swiglu_supported(m, 2 * inter, k, k, k)
    a = rand((m, k), torch.bfloat16, 56)
    gate = rand((inter, k), torch.bfloat16, 57, 1 / math.sqrt(k))
    up = rand((inter, k), torch.bfloat16, 58, 1 / math.sqrt(k))
    w = torch.stack([gate.reshape(inter // 128, 128, k), up.reshape(inter // 128, 128, k)], dim=1).reshape(2 * inter, k).contiguous()
    got = kernels.gemm_split_swiglu(a, w)
    assert kernels.gemm_tcgen05_status() == 0, "a bounded wait inside the kernel was given up"
    ad = a.double().cpu()
    want = plain.silu_and_mul(ad @ gate.double().cpu().T, ad @ up.double().cpu().T)
    close(got, want, torch.bfloat16, "gemm_split_swiglu")
    assert torch.equal(kernels.gemm_split_swiglu(a, w), got), "the product is not repeatable"
    r = m // 2
    assert torch.equal(kernels.gemm_split_swiglu(a[r : r + 1].contiguous(), w), got[r : r + 1]), "a row depends on its batch"
    assert not kernels.gemm_split_swiglu_supported(33, 2 * inter, k, k, k) and not kernels.gemm_split_swiglu_supported(m, 2 * inter + 128, k, k, k)
    assert not kernels.gemm_split_swiglu_supported(m, 2 * 25600, 5120, 5120, 5120)      # too many tiles for clusters that all run at once


@pytest.mark.parametrize("m,inter,k", [(1, 128, 64), (8, 384, 96), (8, 12288, 4096), (16, 3072, 1024), (23, 1280, 2560)])
def test_gemm_stream_swiglu(kernels, m, inter, k):
    """The weight-streaming product with the activation on its accumulators: gate and up of an output in one row of tensor
    memory, tiles shared by neighbouring CTAs fixed up before the activation, repeatable and independent of the batch."""
    assert kernels.gemm_stream_swiglu_supported(m, 2 * inter, k, k, k)
    a = rand((m, k), torch.bfloat16, 53)
    gate = rand((inter, k), torch.bfloat16, 54, 1 / math.sqrt(k))
    up = rand((inter, k), torch.bfloat16, 55, 1 / math.sqrt(k))
    w = torch.stack([gate.reshape(inter // 128, 128, k), up.reshape(inter // 128, 128, k)], dim=1).reshape(2 * inter, k).contiguous()
    got = kernels.gemm_stream_swiglu(a, w)
    assert kernels.gemm_tcgen05_status() == 0, "a bounded wait inside the kernel was given up"
    assert int(kernels._stream_ws[1].abs().sum()) == 0, "a flag was left raised"
    ad = a.double().cpu()
    want = plain.silu_and_mul(ad @ gate.double().cpu().T, ad @ up.double().cpu().T)
    close(got, want, torch.bfloat16, "gemm_stream_swiglu")
    assert torch.equal(kernels.gemm_stream_swiglu(a, w), got), "the product is not repeatable"
    r = m // 2
    assert torch.equal(kernels.gemm_stream_swiglu(a[r : r + 1].contiguous(), w), got[r : r + 1]), "a row depends on its batch"
    assert not kernels.gemm_stream_swiglu_supported(33, 2 * inter, k, k, k) and not kernels.gemm_stream_swiglu_supported(m, 2 * inter + 128, k, k, k)


@pytest.mark.parametrize("m,n,k", [(8, 128, 256), (17, 272, 200), (1, 6144, 4096), (8, 4096, 12288), (64, 2048, 512), (33, 4096, 4096), (5, 1000, 1024),
                                   (16, 5120, 25600)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_split(kernels, m, n, k, out_dtype):
    """The product of decode steps with k split over a thread-block cluster a tile and the partial sums added up in CTA
    order through distributed shared memory: clusters of 2 to 8 (and of 6), a k whose last block is part empty, a last
    tile that is part empty, every padding of the rows of x; the same bits on every run and for every batch."""
    assert kernels.gemm_split_supported(m, n, k, k, k)
    a = rand((m, k), torch.bfloat16, 53)
    w = rand((n, k), torch.bfloat16, 54)
    want = a.double().cpu() @ w.double().cpu().T
    got = kernels.gemm_split(a, w, out_dtype)
    assert kernels.gemm_tcgen05_status() == 0, "a bounded wait inside the kernel was given up"
    if out_dtype == torch.float32:
        lib = torch.mm(a, w.t(), out_dtype=torch.float32)
        err = float(((got.double().cpu() - want).abs() / (1 + want.abs())).max())
        err_lib = float(((lib.double().cpu() - want).abs() / (1 + want.abs())).max())
        assert err < max(2 * err_lib, k * 2.0 ** -23), f"{err} against the library's {err_lib}"
    else:
        close(got, want, torch.bfloat16, "gemm_split", scale=math.sqrt(k) / 8)
    assert torch.equal(kernels.gemm_split(a, w, out_dtype), got), "the product is not repeatable"
    r = m // 2
    assert torch.equal(kernels.gemm_split(a[r : r + 1].contiguous(), w, out_dtype), got[r : r + 1]), "a row depends on its batch"
    # too many rows of x; a row stride that is no multiple of 8; too few blocks of k to split; too many tiles for clusters
    assert not kernels.gemm_split_supported(65, n, k, k, k) and not kernels.gemm_split_supported(m, n, k + 4, k + 4, k + 4)
    assert not kernels.gemm_split_supported(m, n, 64, 64, 64) and not kernels.gemm_split_supported(m, 151936, 4096, 4096, 4096)


@pytest.mark.parametrize("m,n,k", [(8, 128, 64), (17, 272, 96), (1, 6144, 4096), (8, 4096, 12288), (64, 2048, 512), (33, 4096, 4096), (5, 151936, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_stream(kernels, m, n, k, out_dtype):
    """The weight-streaming product of decode steps: equal ranges of (128 rows x 64 k) units per CTA, tiles shared by
    neighbouring CTAs fixed up in CTA order, flags left at zero, the same bits on every run and for every batch."""
    assert kernels.gemm_stream_supported(m, n, k, k, k)
    a = rand((m, k), torch.bfloat16, 51)
    w = rand((n, k), torch.bfloat16, 52)
    want = a.double().cpu() @ w.double().cpu().T
    got = kernels.gemm_stream(a, w, out_dtype)
    assert kernels.gemm_tcgen05_status() == 0, "a bounded wait inside the kernel was given up"
    assert int(kernels._stream_ws[1].abs().sum()) == 0, "a flag was left raised"
    if out_dtype == torch.float32:
        lib = torch.mm(a, w.t(), out_dtype=torch.float32)
        err = float(((got.double().cpu() - want).abs() / (1 + want.abs())).max())
        err_lib = float(((lib.double().cpu() - want).abs() / (1 + want.abs())).max())
        assert err < max(2 * err_lib, k * 2.0 ** -23), f"{err} against the library's {err_lib}"
    else:
        close(got, want, torch.bfloat16, "gemm_stream", scale=math.sqrt(k) / 8)
    assert torch.equal(kernels.gemm_stream(a, w, out_dtype), got), "the product is not repeatable"
    r = m // 2
    assert torch.equal(kernels.gemm_stream(a[r : r + 1].contiguous(), w, out_dtype), got[r : r + 1]), "a row depends on its batch"
    assert not kernels.gemm_stream_supported(65, n, k, k, k) and not kernels.gemm_stream_supported(m, n, k + 4, k + 4, k + 4)
