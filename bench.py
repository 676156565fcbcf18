"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers L] [--impl reference]
    python bench.py --sizes 0.6b|8b|32b          the same line at another model's layer sizes
    python bench.py --workload serving --sizes 0.6b [--requests 32] [--budget 512] [--new-tokens 256] [--max-prompt 2048]

Prints ONE JSON line. ``value`` is decoded tokens per second over K timed decode steps of ``--batch`` requests
that each hold ``--context`` tokens, timed on the device with CUDA events; ``e2e`` is the same through the
Python entry point (``RoostEngine.step``: host token ids in from pinned memory, sampled ids back to the host,
every step). ``prefill`` is one 2,048-token prompt; ``roofline`` the decode step's bytes (every weight once and
the live requests' cache) over its time against the measured copy bandwidth; ``points`` decode at batch 1 and
64 at the same context, at batch 1, 8 and 64 with 1,024-token contexts and at batch 1 and 8 with 16,384-token contexts
(tokens a second; ``points_detail`` has each point's step time and roofline fraction); ``other_sizes`` the same figures at the Qwen3-0.6B and -32B layer sizes and
the 0.6B serving workload. After every timed region the kernels' status words are read: a bounded wait given up inside
it fails the run instead of printing a fast, wrong number. Weights are seeded random values, token ids seeded uniform-random, and the contexts of the device-timed
decode runs are filled with random keys and values instead of being prefilled (their values do not change the
work of a decode step); the e2e run prefills its contexts for real through the engine.

``--workload serving`` prints another line instead: concurrent requests whose prompts are cut into portions under a
token budget and mixed with the decoding of the others, by wall clock through the Python entry point.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
                torch_dtype="bfloat16")
# layer sizes of the other two models the baseline names; every key a config.json of the architecture has
QWEN3_0_6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                  intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                 intermediate_size=25600)
SIZES = {"0.6b": QWEN3_0_6B, "8b": QWEN3_8B, "32b": QWEN3_32B}
PAGE = 16
E2E_SETTLE_S = 10.0   # idle seconds between the untimed prefill of the end-to-end run and its warm-up steps
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.samples = []
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                try:
                    self.samples.append((float(parts[0]), float(parts[1]), parts[3:7]))
                except ValueError:
                    pass

    def summary(self) -> dict:
        if not getattr(self, "samples", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(s[0] for s in self.samples), "sm_max_mhz": max(s[1] for s in self.samples),
                "reasons": reasons, "samples": len(self.samples)}


def build_model(layers: int, dtype, seed: int = 0, sizes: dict = QWEN3_8B):
    import torch

    from roost_b200.config.qwen3 import Qwen3Config
    from roost_b200.engine.model import Model
    from roost_b200.kernels import library
    from roost_b200.parts import Runtime
    from roost_b200.weights.random_init import random_parameters
    cfg = dict(sizes, num_hidden_layers=layers)
    spec = Qwen3Config.from_dict(cfg).to_spec(bool(cfg["tie_word_embeddings"]))
    model = Model(spec, Runtime(dtype, "cuda", library.load()))
    model.load(random_parameters(spec, seed, torch.device("cuda"), dtype, std=0.02))
    return model, cfg


def matrix_bytes(cfg: dict) -> int:
    """Bytes of every weight a decode step reads once: the layers' matrices and norms, the head (the embedding is read
    a row per token)."""
    H, I, V, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    per_layer = (Q + 2 * KV) * H + H * Q + 2 * I * H + H * I + 2 * H + 2 * d
    return 2 * (cfg["num_hidden_layers"] * per_layer + V * H + H)


def kv_bytes_per_token(cfg: dict) -> int:
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, T: int) -> float:
    H, I, V, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d
    per_layer = 2.0 * T * ((Q + 2 * KV) * H + H * Q + 2 * I * H + H * I) + 4.0 * T * T / 2 * Q
    return cfg["num_hidden_layers"] * per_layer + 2.0 * V * H


def fill_context(executor, request_ids, context: int, seed: int = 1):
    """Gives every request ``context`` tokens of cache filled with random keys and values."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    for t, grp in zip(executor.storage.tensors, executor.groups):
        if grp.kind == "paged":
            for i in range(t.shape[0]):
                t[i].copy_(torch.randn(t[i].shape, generator=g, device="cuda", dtype=torch.float32) * 0.5)
    for rid in request_ids:
        executor.cache.extend(rid, context)
        executor.cache.commit(rid, context)


def timed_decode(model, batch: int, context: int, steps: int, warmup: int):
    """K decode steps on the device: step function and greedy choice, no host read inside the timed region."""
    import torch

    from roost_b200.engine.executor import StepEntry, StepExecutor
    pages = batch * (-(-(context + steps + warmup + 2) // PAGE)) + 8
    ex = StepExecutor(model, page_size=PAGE, num_pages=pages, max_requests=max(batch, 1))
    rids = [f"d{i}" for i in range(batch)]
    start = context - (steps + warmup)
    fill_context(ex, rids, start)
    gen = torch.Generator().manual_seed(7)
    tokens = torch.randint(0, model.spec.vocab, (steps + warmup, batch), generator=gen).tolist()
    k = model.rt.kernels

    def one(i):
        logits = ex.step([StepEntry(r, [tokens[i][b]], [0]) for b, r in enumerate(rids)])
        return k.argmax(logits)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0, library0 = k.launches, k.library_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches, library_launches = k.launches - launches0, k.library_launches - library0
    k.check_device_status()   # a bounded wait given up inside the timed region would make the figure a fast, wrong one: fail instead
    ex.close()
    del ex
    gc.collect()
    torch.cuda.empty_cache()
    return batch / (ms / 1e3), ms, (launches, library_launches), clocks.summary()


def timed_prefill(model, tokens_n: int, warmup: int = 3, iters: int = 6):
    import torch

    from roost_b200.engine.executor import StepEntry, StepExecutor
    ex = StepExecutor(model, page_size=PAGE, num_pages=-(-tokens_n // PAGE) + 2, max_requests=2)
    gen = torch.Generator().manual_seed(11)
    ids = torch.randint(0, model.spec.vocab, (tokens_n,), generator=gen).tolist()
    times = []
    for i in range(warmup + iters):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ex.step([StepEntry("p", ids, [tokens_n - 1])])
        e1.record()
        torch.cuda.synchronize()
        ex.finish("p")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    model.rt.kernels.check_device_status()
    ex.close()
    del ex
    gc.collect()
    torch.cuda.empty_cache()
    return min(times)


def timed_e2e(model, batch: int, context: int, steps: int, warmup: int):
    """The same decode through the Python entry point: every step plans, uploads the step's tables from pinned host
    memory, runs, samples on the device and reads the sampled ids back to the host."""
    import torch

    from roost_b200 import GenerationOptions, RoostEngine
    pages = batch * (-(-(context + 2) // PAGE)) + 8
    engine = RoostEngine(model, page_size=PAGE, attention_blocks=pages, max_sequences=max(batch, 1), max_tokens=2048)
    gen = torch.Generator().manual_seed(13)
    # requests that finish their prompt first decode while the others still prefill: leave room for those tokens so
    # that every request stays live, within the context, through the timed steps
    prefill_steps = -(-batch * context // 2048) + 1
    prompt_len = context - (steps + warmup + prefill_steps)
    opts = GenerationOptions(max_output_tokens=4 * (steps + warmup + prefill_steps), ignore_eos=True).sampling()
    for b in range(batch):
        engine.add_request(torch.randint(0, model.spec.vocab, (prompt_len,), generator=gen).tolist(), opts)
    # prefill (untimed): run engine steps until every request decodes
    while any(s.computed < s.prompt_len for s in engine.scheduler.sequences()) or \
            any(s.generated == 0 for s in engine.scheduler.sequences()):
        engine.step()
    # After some seconds of load (always after this prefill, at about 750 W) the device runs the same decode step about
    # 3 % slower (4.68 against 4.55 ms), the SM and memory clocks reading the same; some seconds of idling bring the
    # faster state back. The device-timed figure above is taken at the start of the process, so this one lets the
    # device idle before its warm-up steps too.
    torch.cuda.synchronize()
    time.sleep(E2E_SETTLE_S)
    for _ in range(warmup - 1):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    h2d = d2h = 0
    for _ in range(steps):
        events = engine.step()
        assert len(events) == batch, "a request left the batch inside the timed region"
        produced += sum(1 for e in events if e.token is not None)
        h2d += engine.executor.last_upload_bytes
        d2h += 4 * (len(events) + 4)     # the sampled ids and the kernels' four status words, one pinned copy
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    engine.check_device()
    engine.executor.close()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return produced / dt, h2d // steps, d2h // steps


def timed_serving(model, requests: int, budget: int, new_tokens: int, max_prompt: int, seed: int = 17) -> dict:
    """The serving workload: ``requests`` concurrent requests with prompt lengths uniform in [16, max_prompt], prompts
    cut into portions under a ``budget`` of tokens a step and mixed with the decoding of the others, ``new_tokens``
    greedy tokens each, through the Python entry point (host token ids in, sampled ids out, every step). Wall clock
    from the first step to the last, after two untimed passes of the same requests through the same engine (a server
    that has been up for a while: its allocator is warm and the steps whose sizes come again are captured)."""
    import torch

    from roost_b200 import GenerationOptions, RoostEngine
    gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(16, max_prompt + 1, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, model.spec.vocab, (n,), generator=gen).tolist() for n in lengths]
    pages = sum(-(-(n + new_tokens + 1) // PAGE) for n in lengths) + 8
    opts = GenerationOptions(max_output_tokens=new_tokens, ignore_eos=True).sampling()
    out = {}
    engine = RoostEngine(model, page_size=PAGE, attention_blocks=pages, max_sequences=requests, max_tokens=budget)
    for timed in (False, False, True):
        replays0 = engine.executor.prepared_replays
        steps0 = engine.steps
        for p in prompts:
            engine.add_request(p, opts)
        kinds = {"mixed": [0, 0.0, 0], "decode": [0, 0.0, 0]}     # steps, seconds, tokens run
        produced = 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.has_unfinished():
            t1 = time.perf_counter()
            events = engine.step()
            plan = engine.last_plan
            if plan is None or not plan.rows:
                continue
            kind = kinds["decode" if all(r.count == 1 for r in plan.rows) else "mixed"]
            kind[0] += 1
            kind[1] += time.perf_counter() - t1
            kind[2] += plan.num_tokens
            produced += sum(1 for e in events if e.token is not None)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        engine.check_device()
        stats = engine.stats()
        stats["steps"] -= steps0
        replays = engine.executor.prepared_replays - replays0
        if timed:
            out = {"seconds": round(dt, 3), "output_tokens": produced, "prompt_tokens": sum(lengths),
                   "output_tokens_per_s": round(produced / dt, 1), "total_tokens_per_s": round((produced + sum(lengths)) / dt, 1),
                   "steps": stats["steps"], "preemptions": stats["preemptions"], "prepared_replays": replays,
                   "mixed_steps": kinds["mixed"][0], "mixed_ms_per_step": round(kinds["mixed"][1] / max(kinds["mixed"][0], 1) * 1e3, 3),
                   "mixed_tokens_per_step": round(kinds["mixed"][2] / max(kinds["mixed"][0], 1), 1),
                   "decode_steps": kinds["decode"][0], "decode_ms_per_step": round(kinds["decode"][1] / max(kinds["decode"][0], 1) * 1e3, 3),
                   "decode_rows_per_step": round(kinds["decode"][2] / max(kinds["decode"][0], 1), 1),
                   "captured_steps": len(engine.executor._graphs)}
    engine.executor.close()
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


def serving_main(args) -> int:
    import torch
    sizes = SIZES[args.sizes]
    layers = args.layers if args.layers else sizes["num_hidden_layers"]
    model, cfg = build_model(layers, torch.bfloat16, sizes=sizes)
    with ClockSampler() as clocks:
        r = timed_serving(model, args.requests, args.budget, args.new_tokens, args.max_prompt)
    line = {"metric": f"serving output tokens/s ({args.requests} concurrent requests, prompts 16..{args.max_prompt}, {args.budget}-token step budget, "
                      f"{args.new_tokens} new tokens each), Qwen3-{args.sizes.upper()} layer sizes",
            "value": r["output_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "impl": "ours",
            "data": "synthetic: seeded random weights N(0, 0.02), seeded uniform-random prompts, greedy decoding, wall clock through RoostEngine.step",
            "config": {"model": f"qwen3-{args.sizes}-shapes", "layers": layers, "layers_of_config": sizes["num_hidden_layers"],
                       "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                       "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": PAGE,
                       "requests": args.requests, "budget": args.budget, "new_tokens": args.new_tokens, "max_prompt": args.max_prompt},
            "serving": r, "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


def reference_arm() -> int:
    print(json.dumps({"impl": "reference", "unavailable": "starlinghq/roost is a C#/.NET 10 program with no Python package "
                      "(pip install of the reference's source tree finds no setup.py or pyproject.toml) and no .NET SDK or runtime is on this image"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="layers built (default: all the layers of --sizes)")
    ap.add_argument("--sizes", default="8b", choices=sorted(SIZES), help="whose layer sizes: Qwen3-0.6B, -8B (the headline) or -32B")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="decode: the headline line; serving: concurrent requests with chunked prefill mixed with decoding")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--budget", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--point-batches", default="1,64", help="batch sizes of the extra decode points (the 32B configuration names 1, 8 and 32)")
    ap.add_argument("--point-contexts", default="1024", help="further context lengths of the decode points (the 8B configuration starts at 1,024)")
    ap.add_argument("--point-context-batches", default="1,8,64", help="batch sizes measured at each of --point-contexts")
    ap.add_argument("--point-long-contexts", default="16384", help="long context lengths of the decode points, measured at --point-long-batches")
    ap.add_argument("--point-long-batches", default="1,8", help="batch sizes at --point-long-contexts (batch 8 at 16,384 keys holds 19 GB of keys and values)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-other-sizes", action="store_true", help="leave out the 0.6B and 32B figures that the 8B line carries")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not served")
        return 2
    warmup = max(args.warmup, 3)
    if args.workload == "serving":
        return serving_main(args)

    import torch
    pk, pk_kind = peaks()
    sizes = SIZES[args.sizes]
    args.layers = args.layers or sizes["num_hidden_layers"]
    model, cfg = build_model(args.layers, torch.bfloat16, sizes=sizes)
    tps, ms, launches, clocks = timed_decode(model, args.batch, args.context, args.steps, warmup)
    roof = decode_roofline(cfg, args.batch, args.context, ms, pk)
    # (the same settling as before the end-to-end run: the contexts' prefill at full power leaves the device for some
    # seconds in a state in which every kernel runs a few percent slower, at unchanged clock readings)
    time.sleep(E2E_SETTLE_S)
    pre_ms = timed_prefill(model, args.prefill_tokens)
    points, detail = {}, {}
    if not args.skip_points:
        # the rest of the metric at these sizes: the other batches at this context, every batch at 1,024 tokens, and a
        # long context, where the attention kernel's share of the step is largest
        todo = [(b, args.context) for b in _ints(args.point_batches)] + [(b, c) for c in _ints(args.point_contexts) for b in _ints(args.point_context_batches)]
        todo += [(b, c) for c in _ints(args.point_long_contexts) for b in _ints(args.point_long_batches)]
        for b, c in todo:
            name = f"decode_b{b}" + ("" if c == args.context else f"_ctx{c}")
            p_tps, p_ms, _, _ = timed_decode(model, b, c, max(8, args.steps // 2), warmup)
            points[name] = round(p_tps, 1)
            detail[name] = {"ms_per_step": round(p_ms, 4), "roofline_frac": decode_roofline(cfg, b, c, p_ms, pk)["frac"]}
    e2e = None
    if not args.skip_e2e:
        v, bi, bo = timed_e2e(model, args.batch, args.context, args.steps, warmup)
        e2e = {"value": round(v, 1), "unit": "tokens/s", "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo,
               "settle_s_after_prefill": E2E_SETTLE_S}
    line = {
        "metric": f"decode tokens/s (batch {args.batch}, context {args.context}), Qwen3-{args.sizes.upper()} layer sizes", "value": round(tps, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "ours",
        "data": "synthetic: seeded random weights N(0, 0.02), seeded uniform-random token ids, device-timed decode contexts filled with random keys/values",
        "config": {"model": f"qwen3-{args.sizes}-shapes", "global_batch": args.batch, "seq_len": args.context, "parallelism": "single-gpu",
                   "layers": args.layers, "layers_of_config": sizes["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": PAGE,
                   "l2": "inputs larger than L2: each step streams all weights (>10 GB) from HBM", "peaks": pk_kind},
        "prefill": dict(prefill_record(cfg, args.prefill_tokens, pre_ms, pk), settle_s=E2E_SETTLE_S),
        "roofline": roof,
        "points": points, "points_detail": detail, "clocks": clocks,
        # kernels of this repository's library launched inside the timed region, and the cuBLAS products beside them
        "gpu_launches": launches[0], "library_launches": launches[1],
    }
    if e2e is not None:
        line["e2e"] = e2e
    del model
    gc.collect()
    torch.cuda.empty_cache()
    if args.sizes == "8b" and not args.skip_other_sizes:
        # the baseline's other two configurations, each measured the same way (device-timed decode, one prefill), and the
        # serving workload of the smallest; the largest last, alone on the device (its weights are 65 GB)
        line["other_sizes"] = {name: other_sizes_record(name, args, warmup, pk) for name in ("0.6b", "32b")}
    print(json.dumps(line))
    return 0


def _ints(text: str) -> list:
    return [int(x) for x in text.split(",") if x.strip()]


def decode_roofline(cfg: dict, batch: int, context: int, ms: float, pk: dict) -> dict:
    """The decode step against the copy bandwidth: the bytes it has to read (every weight once, the live requests' keys
    and values) over its time."""
    achieved = (matrix_bytes(cfg) + batch * context * kv_bytes_per_token(cfg)) / (ms / 1e3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)}


def prefill_record(cfg: dict, tokens: int, ms: float, pk: dict) -> dict:
    """``frac`` is against the burst rate of a cuBLAS product timed alone; ``frac_sustained`` against the rate of a
    seconds-long loop under the power cap (the state a 36-layer step is in)."""
    rate = prefill_flops(cfg, tokens) / (ms / 1e3)
    rec = {"value": round(tokens / (ms / 1e3), 1), "tokens": tokens, "ms": round(ms, 3), "frac": round(rate / (pk["bf16_tflops"] * 1e12), 4)}
    if pk.get("bf16_tflops_sustained"):
        rec["frac_sustained"] = round(rate / (pk["bf16_tflops_sustained"] * 1e12), 4)
    return rec


def other_sizes_record(name: str, args, warmup: int, pk: dict) -> dict:
    import torch
    sizes = SIZES[name]
    model, cfg = build_model(sizes["num_hidden_layers"], torch.bfloat16, sizes=sizes)
    steps = max(8, args.steps // 2)
    rec = {"layers": sizes["num_hidden_layers"]}
    for b in (1, 8, 32 if name == "32b" else 64):
        tps, ms, _, _ = timed_decode(model, b, args.context, steps, warmup)
        rec[f"decode_b{b}"] = {"value": round(tps, 1), "ms_per_step": round(ms, 4), "roofline_frac": decode_roofline(cfg, b, args.context, ms, pk)["frac"]}
    rec["prefill"] = prefill_record(cfg, args.prefill_tokens, timed_prefill(model, args.prefill_tokens, warmup=2, iters=3), pk)
    if name == "0.6b":
        r = timed_serving(model, args.requests, args.budget, args.new_tokens, args.max_prompt)
        rec["serving"] = {k: r[k] for k in ("output_tokens_per_s", "total_tokens_per_s", "steps", "mixed_ms_per_step", "decode_ms_per_step", "preemptions")}
    del model
    gc.collect()
    torch.cuda.empty_cache()
    return rec


if __name__ == "__main__":
    sys.exit(main())
