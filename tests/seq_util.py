"""Drive bin/trace_run (the product's own entry: registry -> scheduler -> sequence-batch engine) from the tests."""
from __future__ import annotations

import json
import subprocess
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


def run_trace(model_dir, steps, dtype="float32", max_tokens=2048, page=None, residual=False, vocab=None, extra=()):
    """steps: [{"entries": [{"id", "tokens", "want"}], "end": [...]}].  Returns (logits per step, residual per step):
    logits[i] is [wanted rows, vocab] (None when nothing was wanted)."""
    out = tempfile.mkdtemp(prefix="kllm_trace_")
    cmd = [str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)]
    if page:
        cmd += ["--page", str(page)]
    if residual:
        cmd += ["--residual"]
    cmd += list(extra)
    text = "".join(json.dumps({"step": i, "entries": s["entries"], "end": s.get("end", [])}) + "\n"
                   for i, s in enumerate(steps))
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, f"trace_run exit {r.returncode}\n{r.stderr[-3000:]}"
    done = [ln for ln in r.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(steps))], r.stdout[-2000:]
    if vocab is None:
        vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab"]
    logits, resid = [], []
    for i, s in enumerate(steps):
        n = sum(len(e.get("want", [])) for e in s["entries"])
        f = Path(out) / f"{i}.f32"
        logits.append(np.fromfile(f, dtype="<f4").reshape(n, vocab) if n else None)
        assert n or not f.exists()
        rf = Path(out) / f"{i}.residual.f32"
        resid.append(np.fromfile(rf, dtype="<f4") if residual else None)
    return logits, resid


def whole(rid, tokens, want=None, end=True):
    return {"entries": [{"id": rid, "tokens": list(tokens), "want": list(range(len(tokens))) if want is None else want}],
            "end": [rid] if end else []}


def rel_err(got, ref):
    """Root-mean-square difference of the rows (mean over the vocabulary taken off), relative to the reference's own
    spread: the largest over the rows."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    spread = (ref - ref.mean(-1, keepdims=True)).std()
    return float(np.sqrt((d ** 2).mean(-1)).max() / spread)
