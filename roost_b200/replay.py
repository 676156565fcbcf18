"""Trace replay over the engine's own step function (see ``bin/trace_run``).

The reference's closest tools are its test runner that feeds given tokens per sequence per step
(tests/Starlings.Roost.Models.Tiny.Tests/Support/TinyRunner.cs:75-141) and its planner replay
(src/Starlings.Roost.Engine/Scheduling/PlannerReplay.cs:54-94); it has no standalone replay program.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

REPLAY_PAGE_SIZE = 16   # divides 64, the granule --max-tokens is counted in
MAX_LIVE_REQUESTS = 16


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token traces through the engine's step function and dump logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each request rounded up to a multiple of 64")
    ap.add_argument("--page-size", type=int, default=REPLAY_PAGE_SIZE)
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")

    import torch
    from .engine.executor import StepEntry, StepExecutor
    from .engine.model import load_model

    dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, dtype, device="cuda")
    executor = StepExecutor(model, page_size=args.page_size, max_tokens=args.max_tokens, max_requests=MAX_LIVE_REQUESTS)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], list(e["tokens"]), list(e.get("want", []))) for e in rec.get("entries", [])]
        if entries:
            logits = executor.step(entries)
            if logits.shape[0] > 0:
                logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4").tofile(out_dir / f"{step}.f32")
            model.rt.kernels.check_device_status()   # a kernel that gave up a bounded wait makes the step an error, not a file
        for rid in rec.get("end", []):
            executor.finish(rid)
        print(f"done {step}", flush=True)
    return 0
