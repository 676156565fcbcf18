"""Plain, slow implementation of the dense Qwen3 decoder: whole sequences, no cache, no pages.

It rests on the formulas of starlinghq/roost's reference ops (its C# model code cannot be compiled in an
image without a .NET SDK); every function cites the file and lines of the reference that define the
formula. Nothing here is shared with the product path under ``roost_b200/``: the tests compare the two.

All arithmetic is float64 unless ``dtype`` says otherwise; weights are taken as given (the caller rounds
them to bfloat16 first when the engine under test stores bfloat16).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------------------------------
# weights on disk (a reader of its own: the product's reader is under test)
# --------------------------------------------------------------------------------------------------
_ST_DTYPES = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F64": (torch.float64, 8),
              "I64": (torch.int64, 8), "I32": (torch.int32, 4)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw little-endian data
    (src/Starlings.Roost.Worker/Weights/SafetensorsHeader.cs:89-172)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _ST_DTYPES[meta["dtype"]]
        a, b = meta["data_offsets"]
        buf = bytearray(raw[8 + n + a : 8 + n + b])
        t = torch.frombuffer(buf, dtype=dt).reshape(meta["shape"]) if b > a else torch.empty(meta["shape"], dtype=dt)
        out[name] = t.clone()
    return out


def load_model_dir(model_dir, round_to_bf16: bool = False) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor as float64 (optionally rounded to bfloat16 first)."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    w = read_safetensors(model_dir / "model.safetensors")
    out = {}
    for k, v in w.items():
        if round_to_bf16:
            v = v.to(torch.bfloat16)
        out[k] = v.to(F64)
    return cfg, out


# --------------------------------------------------------------------------------------------------
# parts, one function each
# --------------------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """h0[t,:] = table[ids[t],:], no scaling (src/Starlings.Roost.Ops/CpuOps.cs:441-458)."""
    ids = torch.as_tensor(ids, dtype=torch.long, device=table.device)
    if ((ids < 0) | (ids >= table.shape[0])).any():
        raise ValueError("token id outside the vocabulary")
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i / sqrt(mean(x^2) + eps) * w_i, the weight as stored
    (src/Starlings.Roost.Ops/CpuOps.cs:87-101)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * inv * weight


def qk_norm(q: torch.Tensor, k: torch.Tensor, q_weight, k_weight, eps: float):
    """RMS norm over head_dim of every query head and every key head, one weight vector shared by the
    heads; values are not normed (src/Starlings.Roost.Ops/CpuOps.cs:65-85). q: [T, nq, d], k: [T, nkv, d]."""
    return rms_norm(q, q_weight, eps), rms_norm(k, k_weight, eps)


def rope_neox(x: torch.Tensor, positions, theta: float, rotary_dim: int | None = None) -> torch.Tensor:
    """NeoX rotation: f_i = theta^(-2i/R), angle = pos * f_i, the pair (i, i + R/2) becomes
    (x1 cos - x2 sin, x2 cos + x1 sin); elements at and beyond R are unchanged
    (src/Starlings.Roost.Ops/CpuOps.cs:111-177). x: [T, heads, d]."""
    d = x.shape[-1]
    rot = d if rotary_dim is None else rotary_dim
    half = rot // 2
    pos = torch.as_tensor(positions, dtype=F64, device=x.device)
    i = torch.arange(half, dtype=F64, device=x.device)
    freq = torch.pow(torch.tensor(float(theta), dtype=F64, device=x.device), -2.0 * i / rot)
    ang = pos[:, None] * freq[None, :]
    c = torch.cos(ang)[:, None, :].to(x.dtype)
    s = torch.sin(ang)[:, None, :].to(x.dtype)
    x1 = x[..., :half]
    x2 = x[..., half:rot]
    out = x.clone()
    out[..., :half] = x1 * c - x2 * s
    out[..., half:rot] = x2 * c + x1 * s
    return out


def causal_gqa_attention(q, k, v, scale: float, window: int | None = None) -> torch.Tensor:
    """Whole-sequence causal attention. Query i sees keys j <= i and, with a window of W keys that includes
    the query's own, j > i - W (the reference's WindowLeft is W - 1); query head h reads key/value head
    h // (nq // nkv); score = q.k * scale; softmax; weighted sum of v
    (src/Starlings.Roost.Ops/CpuOps.cs:181-298). q: [T, nq, d], k, v: [T, nkv, d] -> [T, nq, d]."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.zeros_like(q)
    idx = torch.arange(T, device=q.device)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= idx[None, :] > (idx[:, None] - window)
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """act = gate / (1 + exp(-gate)) * up (src/Starlings.Roost.Ops/CpuOps.cs:355-368,
    src/Starlings.Roost.Ops/CpuElements.cs:223)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def swiglu_mlp(y, gate_w, up_w, down_w) -> torch.Tensor:
    """down(silu(y Wg^T) * (y Wu^T)), weights stored [out, in], no bias
    (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:51-53)."""
    return silu_and_mul(y @ gate_w.T, y @ up_w.T) @ down_w.T


def attention_mixer(x, positions, w: dict, prefix: str, cfg: dict, window: int | None, kv_from=None):
    """q/k/v projections (no bias), per-head QK norm before the rotation, rotation of q and k, attention,
    output projection (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:41-48). Returns (output, (k, v)); with
    ``kv_from`` the keys and values of another layer are read and none are computed."""
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    q = (x @ w[prefix + "q_proj.weight"].T).reshape(T, nq, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    q = rope_neox(q, positions, theta)
    if kv_from is None:
        k = (x @ w[prefix + "k_proj.weight"].T).reshape(T, nkv, d)
        v = (x @ w[prefix + "v_proj.weight"].T).reshape(T, nkv, d)
        k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
        k = rope_neox(k, positions, theta)
    else:
        k, v = kv_from
    o = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return o.reshape(T, nq * d) @ w[prefix + "o_proj.weight"].T, (k, v)


def layer_windows(cfg: dict) -> list[int | None]:
    """Which layers use the sliding window: ``layer_types`` when present, else with ``use_sliding_window``
    the layers at or above ``max_window_layers``
    (evidence/pipeline/onboarding/Starlings.Roost.Onboarding/ConfigInspector.cs:266-318)."""
    L = cfg["num_hidden_layers"]
    win = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is not None:
        return [win if t == "sliding_attention" else None for t in types]
    if win is not None and cfg.get("use_sliding_window"):
        first = cfg.get("max_window_layers", L)
        return [win if i >= first else None for i in range(L)]
    return [None] * L


def normalise_config(cfg: dict) -> dict:
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    cfg.setdefault("rms_norm_eps", 1e-6)
    cfg.setdefault("rope_theta", 10000.0)
    if cfg.get("rope_parameters") and "rope_theta" in cfg["rope_parameters"]:
        cfg["rope_theta"] = cfg["rope_parameters"]["rope_theta"]
    return cfg


def forward_logits(cfg: dict, w: dict[str, torch.Tensor], ids, schedule=None, rows=None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence (or, with ``rows``, at those positions only: the
    final norm and the head are per position, so the other positions' logits need not be formed)
    (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:39-56; the shape of the reference's TinyReference,
    tests/Starlings.Roost.Models.Tiny.Tests/Support/TinyReference.cs:22-102).

    ``schedule`` is a list of (layer, reads_cache_of) entries in running order; ``reads_cache_of`` is None
    for a run that computes its own keys and values, or the index of an earlier entry whose keys and
    values it reads. The default is every layer once, in order."""
    cfg = normalise_config(cfg)
    eps = cfg["rms_norm_eps"]
    wins = layer_windows(cfg)
    T = len(ids)
    positions = list(range(T))
    h = embedding(w["model.embed_tokens.weight"], ids)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, reads in schedule:
        p = f"model.layers.{layer}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        mix, kv = attention_mixer(x, positions, w, p + "self_attn.", cfg, wins[layer],
                                  kv_from=None if reads is None else kvs[reads])
        kvs.append(kv)
        h = h + mix
        y = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu_mlp(y, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long, device=h.device)]
    final = rms_norm(h, w["model.norm.weight"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w and not cfg.get("tie_word_embeddings", False) else w["model.embed_tokens.weight"]
    return final @ head.T


def greedy(cfg, w, prompt, n: int, schedule=None) -> list[int]:
    """n greedy tokens; ties to the lowest index (src/Starlings.Roost.Ops/CpuOps.cs:603-626)."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        logits = forward_logits(cfg, w, seq, schedule)[-1]
        t = int(torch.argmax(logits))  # torch.argmax returns the first maximum
        out.append(t)
        seq.append(t)
    return out


# --------------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------------
_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_U32 = 0xFFFFFFFF


def philox4x32_10(counter, key):
    """Ten rounds over a four-word counter and a two-word key (src/Starlings.Roost.Ops/CpuPhilox.cs:15-33)."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> 32, p0 & _U32
        hi1, lo1 = p1 >> 32, p1 & _U32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _U32, lo1, (hi0 ^ c3 ^ k1) & _U32, lo0
        k0 = (k0 + _W0) & _U32
        k1 = (k1 + _W1) & _U32
    return c0, c1, c2, c3


def philox_uniform(seed: int, offset: int) -> float:
    """counter = (offset low, offset high, 0, 0), key = (seed low, seed high); first word's top 24 bits
    times 2^-24 (src/Starlings.Roost.Ops/CpuPhilox.cs:39-43)."""
    r0 = philox4x32_10((offset & _U32, (offset >> 32) & _U32, 0, 0), (seed & _U32, (seed >> 32) & _U32))[0]
    return (r0 >> 8) * (1.0 / 16777216.0)


def sample_row(logits, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
               seed: int = 0, offset: int = 0, return_detail: bool = False):
    """One row of the reference sampler in double (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:279-370):
    NaN and -inf are removed; temperature <= 0 is the highest logit, ties to the lowest index; else
    p = softmax((z - max)/T), ordered by p descending then index ascending; top-k keeps the first k;
    top-p keeps the shortest prefix whose mass reaches top_p times the kept total (the crossing token
    stays); min-p drops p < min_p * p_max; the draw picks the first token whose running mass exceeds
    u times the kept mass."""
    z = np.asarray(logits, dtype=np.float64)
    allowed = [v for v in range(len(z)) if not (math.isnan(z[v]) or z[v] == -math.inf)]
    if not allowed:
        return -1
    if temperature <= 0:
        best = allowed[0]
        for v in allowed[1:]:
            if z[v] > z[best]:
                best = v
        return best
    mx = max(z[v] for v in allowed)
    prob = {v: math.exp((z[v] - mx) / temperature) for v in allowed}
    total = 0.0
    for v in allowed:
        total += prob[v]
    for v in allowed:
        prob[v] /= total
    order = sorted(allowed, key=lambda v: (-prob[v], v))
    keep = len(order)
    if 0 < top_k < keep:
        keep = top_k
    if top_p < 1.0:
        tot = sum(prob[v] for v in order[:keep])
        cum = 0.0
        cut = keep
        for i in range(keep):
            cum += prob[order[i]]
            if cum >= top_p * tot:
                cut = i + 1
                break
        keep = cut
    if min_p > 0.0:
        floor = min_p * prob[order[0]]
        cut = keep
        for i in range(keep):
            if prob[order[i]] < floor:
                cut = i
                break
        keep = max(1, cut)
    mass = 0.0
    for v in order[:keep]:
        mass += prob[v]
    u = philox_uniform(seed, offset)
    target = u * mass
    run = 0.0
    chosen = order[keep - 1]
    margin = math.inf
    found = False
    for i in range(keep):
        prev = run
        run += prob[order[i]]
        if not found and run > target:
            chosen = order[i]
            found = True
            margin = min(run - target, target - prev) / mass
    if return_detail:
        # margin: how far (as a share of the kept mass) the draw is from the edges of the chosen token's interval
        return chosen, {"kept": order[:keep], "margin": margin, "u": u, "prob": prob}
    return chosen


def penalise_row(logits, counts: dict, prompt_tokens, repetition: float = 1.0, frequency: float = 0.0, presence: float = 0.0):
    """The reference's penalties on one row, in double (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:195-237; vLLM's
    order, :13-17): with c the token's count in the generated output and seen = c > 0 or the token is in the prompt, a seen
    logit x becomes x / repetition if it is above 0 and x * repetition otherwise; then x - frequency * c; then, when
    c > 0, x - presence."""
    z = [float(x) for x in logits]
    prompt = set(prompt_tokens)
    for v in range(len(z)):
        c = counts.get(v, 0)
        x = z[v]
        if c > 0 or v in prompt:
            x = x / repetition if x > 0 else x * repetition
        x -= frequency * c
        if c > 0:
            x -= presence
        z[v] = x
    return z


def mask_row(logits, allowed_token_ids):
    """Tokens outside the mask are removed before the softmax, after the penalties
    (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:18-19,240-262): here they become -inf, which the sampler never draws."""
    allowed = set(allowed_token_ids)
    return [x if v in allowed else -math.inf for v, x in enumerate(logits)]


def log_norm(logits):
    """(max, log of the sum of exp(x - max)) over the non-NaN raw logits (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:516-537)."""
    mx = -math.inf
    for x in logits:
        if x > mx:
            mx = x
    total = 0.0
    for x in logits:
        if not math.isnan(x):
            total += math.exp(x - mx)
    return mx, math.log(total) if total > 0 else -math.inf


def logprob_at(logits, token: int) -> float:
    """The log-softmax of the raw logits at a token; -inf for token -1 (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:166-170,566-567)."""
    if token < 0:
        return -math.inf
    mx, lse = log_norm(logits)
    return float(logits[token]) - mx - lse


def top_logprobs(logits, k: int):
    """The k highest raw logits, ties to the lower index, NaN skipped, with their log-softmax; missing entries are id -1
    and -inf (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:569-603)."""
    mx, lse = log_norm(logits)
    order = sorted((v for v in range(len(logits)) if not math.isnan(logits[v])), key=lambda v: (-logits[v], v))[:k]
    ids = order + [-1] * (k - len(order))
    return ids, [float(logits[v]) - mx - lse if v >= 0 else -math.inf for v in ids]


# --------------------------------------------------------------------------------------------------
# the reference's seeded weight generator (for the pinned greedy ids of roost-tiny)
# --------------------------------------------------------------------------------------------------
_MASK64 = (1 << 64) - 1


def fnv1a64_chars(name: str) -> int:
    h = 14695981039346656037
    for ch in name:
        h = ((h ^ ord(ch)) * 1099511628211) & _MASK64
    return h


def fnv1a64_bytes(data: bytes) -> int:
    h = 14695981039346656037
    for b in data:
        h = ((h ^ b) * 1099511628211) & _MASK64
    return h


def tiny_weights(model_seed: int, slot: str, shape: tuple[int, ...], dtype: str = "F32") -> np.ndarray:
    """state = seed ^ FNV-1a(slot name); SplitMix64; u = (x >> 11) 2^-53; value = offset + (2u - 1) amp with
    (offset, amp) = (1, 0.1) for names ending in "norm", (0, 1) for "embed", (0, 1.5/sqrt(last dim)) else;
    rounded to the slot's dtype (src/Starlings.Roost.Models.Tiny/TinyWeights.cs:22-32,45-78,155-162)."""
    n = int(np.prod(shape))
    if slot.endswith("norm"):
        amp, off = 0.1, 1.0
    elif slot == "embed":
        amp, off = 1.0, 0.0
    else:
        amp, off = 1.5 / math.sqrt(shape[-1]), 0.0
    state = (model_seed ^ fnv1a64_chars(slot)) & _MASK64
    # vectorised SplitMix64: state_i = state + (i+1) * golden
    idx = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(state) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    vals = (off + (2.0 * u - 1.0) * amp).astype(np.float32)
    if dtype == "BF16":
        vals = torch.from_numpy(vals).to(torch.bfloat16).to(torch.float32).numpy()
    return vals.reshape(shape)


def roost_tiny_reference_model():
    """config dict and float64 weights of the reference's roost-tiny
    (src/Starlings.Roost.Models.Tiny/TinyConfig.cs:63-66, RoostTiny.cs:14-57)."""
    seed = 0x524F4F53540001
    cfg = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=64,
               intermediate_size=128, vocab_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512,
               torch_dtype="float32")
    H, I, V, Q, KV, d = 64, 128, 256, 64, 32, 16
    w = {}

    def gen(slot, shape):
        return torch.from_numpy(tiny_weights(seed, slot, shape)).to(F64)

    w["model.embed_tokens.weight"] = gen("embed", (V, H))
    for i in range(4):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = gen(f"l{i}.input_norm", (H,))
        w[p + "self_attn.q_proj.weight"] = gen(f"l{i}.q_proj", (Q, H))
        w[p + "self_attn.k_proj.weight"] = gen(f"l{i}.k_proj", (KV, H))
        w[p + "self_attn.v_proj.weight"] = gen(f"l{i}.v_proj", (KV, H))
        w[p + "self_attn.q_norm.weight"] = gen(f"l{i}.q_norm", (d,))
        w[p + "self_attn.k_norm.weight"] = gen(f"l{i}.k_norm", (d,))
        w[p + "self_attn.o_proj.weight"] = gen(f"l{i}.o_proj", (H, Q))
        w[p + "post_attention_layernorm.weight"] = gen(f"l{i}.post_norm", (H,))
        gu = gen(f"l{i}.gate_up", (2 * I, H))
        w[p + "mlp.gate_proj.weight"] = gu[:I].clone()
        w[p + "mlp.up_proj.weight"] = gu[I:].clone()
        w[p + "mlp.down_proj.weight"] = gen(f"l{i}.down", (H, I))
    w["model.norm.weight"] = gen("final_norm", (H,))
    w["lm_head.weight"] = gen("lm_head", (V, H))
    return cfg, w
