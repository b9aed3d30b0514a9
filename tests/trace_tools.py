"""Building step traces for ``bin/trace_run`` and reading back what it writes."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round64(n: int) -> int:
    return -(-n // 64) * 64


class TraceBuilder:
    """Collects steps, remembers which (request, position) each written row is,
    and tracks the most tokens that live requests hold (each rounded up to 64)."""

    def __init__(self):
        self.steps = []          # json records
        self.rows = {}           # step -> list of (request id, absolute position)
        self.held = {}           # live request id -> tokens held
        self.peak = 0

    def step(self, entries, end=()):
        """entries: list of (rid, tokens, want places).  Positions follow from what
        the request already holds."""
        k = len(self.steps)
        rec = {"step": k, "entries": [], "end": list(end)}
        rows = []
        for rid, tokens, want in entries:
            start = self.held.get(rid, 0)
            rec["entries"].append({"id": rid, "tokens": [int(t) for t in tokens], "want": [int(w) for w in want]})
            rows.extend((rid, start + int(w)) for w in want)
            self.held[rid] = start + len(tokens)
        self.peak = max(self.peak, sum(round64(v) for v in self.held.values()))
        for rid in end:
            self.held.pop(rid, None)
        if rows:
            self.rows[k] = rows
        self.steps.append(rec)
        return k


def run_trace(model_dir: str, dtype: str, builder: TraceBuilder, out_dir: str, vocab: int,
              max_tokens: int = 0, timeout: float = 600.0, trace_file: str = ""):
    """Run bin/trace_run on the trace, feeding a step only after the previous
    ``done`` line (or handing it the whole trace as ``--trace FILE``).  Returns
    {(rid, position): logits row}, read from the ``step_<k>.npy`` files by the program's
    own ``index.json``; the raw ``<k>.f32`` files must hold the same numbers, and the
    index must name the rows that the trace asked for."""
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or builder.peak)]
    if trace_file:
        with open(trace_file, "w") as f:
            f.writelines(json.dumps(rec) + "\n" for rec in builder.steps)
        done = subprocess.run(cmd + ["--trace", trace_file], stdin=subprocess.DEVNULL, capture_output=True,
                              text=True, timeout=timeout)
        assert done.returncode == 0, done.stderr[-2000:]
        assert done.stdout.split("\n")[:-1] == [f"done {rec['step']}" for rec in builder.steps]
    else:
        proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        try:
            for rec in builder.steps:
                proc.stdin.write(json.dumps(rec) + "\n")
                proc.stdin.flush()
                line = proc.stdout.readline()
                assert line.strip() == f"done {rec['step']}", f"trace_run answered {line!r} to step {rec['step']}"
            proc.stdin.close()
            rc = proc.wait(timeout=timeout)
        finally:
            if proc.poll() is None:
                proc.kill()
        assert rc == 0, f"trace_run exited with {rc}"
    with open(os.path.join(out_dir, "index.json")) as f:
        index = json.load(f)
    assert index["vocab"] == vocab
    listed = {}
    for r in index["rows"]:
        listed.setdefault(r["step"], []).append((r["row"], r["request"], r["position"]))
    assert sorted(listed) == sorted(builder.rows), "the index lists other steps than the trace wanted logits in"
    out = {}
    for k, rows in builder.rows.items():
        assert [(rid, pos) for _, rid, pos in sorted(listed[k])] == rows, f"index of step {k}"
        arr = np.load(os.path.join(out_dir, f"step_{k}.npy"))
        assert arr.dtype == np.dtype("<f4") and arr.shape == (len(rows), vocab) and arr.flags.c_contiguous
        raw = np.fromfile(os.path.join(out_dir, f"{k}.f32"), dtype="<f4").reshape(len(rows), vocab)
        assert np.array_equal(raw, arr, equal_nan=True)
        for i, key in enumerate(rows):
            assert key not in out, f"row {key} written twice"
            out[key] = arr[i]
    return out


def portions(total: int, sizes):
    """Cut ``total`` tokens into portions of the given sizes, cycling through them."""
    out, i, done = [], 0, 0
    while done < total:
        n = min(sizes[i % len(sizes)], total - done)
        out.append(n)
        done += n
        i += 1
    return out


def run_on_engine(eng, builder: TraceBuilder):
    """The same trace through an ``Engine`` of this process (its step function, cache
    manager and kernels), without the replay program.  Returns {(rid, position): row}."""
    from kllm_b200.engine import StepEntry
    live, out = {}, {}
    for rec in builder.steps:
        entries = []
        for e in rec["entries"]:
            if e["id"] not in live:
                live[e["id"]] = eng.cache.open()
            entries.append(StepEntry(live[e["id"]], e["tokens"], e["want"]))
        logits = eng.step(entries)
        if logits is not None:
            arr = logits.cpu().numpy()
            for i, key in enumerate(builder.rows[rec["step"]]):
                assert key not in out, f"row {key} written twice"
                out[key] = arr[i]
        for rid in rec["end"]:
            eng.cache.close(live.pop(rid))
    return out
