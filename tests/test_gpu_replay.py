"""Trace replay through bin/trace_run against the plain implementation.

For each tiny configuration and each dtype ONE trace_run process replays the same
requests in four ways, under request ids of their own:
  w: each request alone and whole, one step;
  d: most of it in one step and the last 32 tokens one by one;
  p: in portions of changing size, down to two tokens (and one);
  m: mixed, up to four live requests, portions of some beside single tokens of
     others, requests ending and new ones starting so that pages are used again.
The pool is as small as the trace allows (--max-tokens = the peak the trace
reaches), so the ways w, d and p reuse the pages of the requests before them too.
Every logits row of every way is compared with the plain implementation, and the
four ways are compared with EACH OTHER: the same (request, position) must give the
same logits however the tokens were cut and whatever ran beside them, beyond the
rounding of sums whose order depends on the step's size (the library's float32
products choose their kernel by the row count; the decode attention cuts a context
into more or fewer key ranges).  The bound on that difference is far below the
tolerance against the plain implementation, so a drift inside that tolerance shows.
One configuration hands the program its trace as ``--trace FILE``, the other feeds
standard input step by step.
"""
import numpy as np
import pytest

from helpers import CROSS_TOL, assert_close, make_weights, note_cross, plain_logits, prompts_for, write_model_dir
from trace_tools import TraceBuilder, portions, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 31, 64, 128, 90], "B": [1, 3, 40, 100, 128, 200, 256, 77]}
SIZES = {"A": [7, 2, 13, 3, 1, 29], "B": [13, 2, 64, 1, 5, 37]}


def build_trace(seqs, sizes, seed):
    tb = TraceBuilder()
    # w: whole
    for i, ids in enumerate(seqs):
        tb.step([(f"w{i}", ids, range(len(ids)))], end=[f"w{i}"])
    # d: most in one step, the last 32 one by one
    for i, ids in enumerate(seqs):
        head = max(0, len(ids) - 32)
        rid = f"d{i}"
        if head:
            tb.step([(rid, ids[:head], range(head))])
        for t in range(head, len(ids)):
            tb.step([(rid, [ids[t]], [0])], end=[rid] if t == len(ids) - 1 else [])
    # p: portions of changing size
    for i, ids in enumerate(seqs):
        rid, pos = f"p{i}", 0
        cuts = portions(len(ids), sizes[i % len(sizes):] + sizes[:i % len(sizes)])
        for j, n in enumerate(cuts):
            tb.step([(rid, ids[pos:pos + n], range(n))], end=[rid] if j == len(cuts) - 1 else [])
            pos += n
    # m: mixed, up to four live
    rng = np.random.default_rng(seed)
    queue = list(range(len(seqs)))
    live = {}       # index -> tokens fed
    while queue or live:
        while queue and len(live) < 4:
            live[queue.pop(0)] = 0
        chosen = [i for i in live if rng.random() < 0.75] or [next(iter(live))]
        entries, ended = [], []
        for i in chosen:
            ids, fed = seqs[i], live[i]
            left = len(ids) - fed
            tail = left <= min(32, len(ids) // 2)          # the end of a request goes token by token
            n = 1 if tail else int(min(left, rng.choice(sizes)))
            entries.append((f"m{i}", ids[fed:fed + n], range(n)))
            live[i] = fed + n
            if live[i] == len(ids):
                ended.append(i)
        tb.step(entries, end=[f"m{i}" for i in ended])
        for i in ended:
            del live[i]
    return tb


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_all_ways(tmp_path, name, dtype):
    cfg, w = make_weights(name, dtype)
    d = write_model_dir(str(tmp_path / "model"), cfg, w)
    seqs = prompts_for(cfg, LENGTHS[name], seed=3)
    tb = build_trace(seqs, SIZES[name], seed=5)
    total = sum(len(s) for s in seqs)
    assert tb.peak < total, "the pool must be smaller than what the mixed phase feeds, or no page is reused"
    got = run_trace(d, dtype, tb, str(tmp_path / "out"), cfg["vocab_size"],
                    trace_file=str(tmp_path / "trace.jsonl") if name == "A" else "")
    for i, ids in enumerate(seqs):
        want = plain_logits(w, cfg, ids, dtype)
        rows = {way: np.stack([got[(f"{way}{i}", p)] for p in range(len(ids))]) for way in "wdpm"}
        for way in "wdpm":
            assert_close(rows[way], want, dtype, f"{name} {dtype} request {i} (len {len(ids)}) way {way}")
        scale = float(np.abs(want).max())
        for way in "dpm":
            diff = float(np.abs(rows[way].astype(np.float64) - rows["w"]).max()) / scale
            note_cross(dtype, diff, f"{name} request {i} way {way} against whole")
            assert diff <= CROSS_TOL[dtype], (
                f"{name} {dtype} request {i}: way {way} differs from the whole run by {diff:.3e} of the "
                f"largest logit (bound {CROSS_TOL[dtype]:.0e})")
