"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from the files it writes."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.conftest import ROOT, TINY

pytestmark = pytest.mark.gpu


class TraceRun:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out_dir = Path(out_dir)
        self.proc = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                                      "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                                     stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step_no = 0

    def step(self, entries, end=()):
        rec = {"step": self.step_no, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step_no}", f"trace_run answered {line!r}"
        f = self.out_dir / f"{self.step_no}.f32"
        self.step_no += 1
        wanted = sum(len(w) for _, _, w in entries)
        if wanted == 0:
            assert not f.exists()
            return None
        return torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(wanted, -1))

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_replays_whole_decoded_and_mixed(tiny_model_dirs, tmp_path, name, dtype):
    model_dir, t = tiny_model_dirs[name], TINY[name]
    V = t["config"]["vocab_size"]
    tdtype = torch.float32 if dtype == "float32" else torch.bfloat16
    a, b, c = H.random_ids(70, V, 21), H.random_ids(45, V, 22), H.random_ids(100, V, 23)
    want = {k: H.plain_logits(model_dir, ids, bf16=dtype == "bfloat16") for k, ids in (("a", a), ("b", b), ("c", c))}
    # a and b live together (128 + 64 tokens of pages), then c takes the pages a gave back: 192 tokens in all
    run = TraceRun(model_dir, dtype, tmp_path, max_tokens=192)
    try:
        got_a = [run.step([("a", a[:38], list(range(38)))])]
        got_b = [run.step([("b", b[:2], [0, 1]), ("a", a[38:40], [0, 1])])]
        got_a.append(got_b[0][2:]); got_b[0] = got_b[0][:2]
        assert run.step([("b", b[2:30], [])]) is None            # a step that wants nothing writes no file
        out = run.step([("a", a[40:41], [0]), ("b", b[30:45], [14])], end=["b"])
        got_a.append(out[:1]); last_b = out[1:]
        for i in range(41, 70):
            got_a.append(run.step([("a", a[i : i + 1], [0])], end=["a"] if i == 69 else []))
        got_c = run.step([("c", c, list(range(100)))], end=["c"])
    finally:
        run.close()
    bound = H.bound_for(tdtype)
    assert H.scaled_error(torch.cat(got_a), want["a"]) < bound
    if dtype == "bfloat16":
        assert H.rms_error(torch.cat(got_a), want["a"]) < H.BF16_RMS_BOUND
        assert H.rms_error(got_c, want["c"]) < H.BF16_RMS_BOUND
    assert H.scaled_error(got_b[0], want["b"][:2]) < bound
    assert H.scaled_error(last_b, want["b"][44:45]) < bound
    assert H.scaled_error(got_c, want["c"]) < bound
