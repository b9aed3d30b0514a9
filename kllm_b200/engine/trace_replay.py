"""Trace replay: feed given token ids through a model step by step and write the
logits.  It samples nothing.  It drives the engine's own model, step function,
cache manager and kernels, the ones that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--trace FILE]

Steps come on standard input (or from ``--trace FILE``), one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step are one batch.  ``end``: requests that
are finished after this step; their pages are given back.  For a step in which
something is wanted, ``<out>/<step>.f32`` holds the logits [wanted, vocab] as
little-endian float32 in the order of the entries and of ``want``; the same array is
written as ``<out>/step_<step>.npy`` (format 1.0, ``<f4``, C order: what the reference's
reader takes, engine/npy/npy.go:22-82, and its dumps use, tools/gen_reference.py:65-119).
When the input ends ``<out>/index.json`` lists every written row: step, row, request
id and the row's position in its request.  After every step a line ``done <step>`` is
printed and flushed.  The cache pool is sized for
``--max-tokens`` tokens (each request's count rounded up to whole pages), so pages
are used again.  The reference checks logits step by step in a Go test
(engine/oracle/oracle.go:47-137); it has no program that writes them.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--trace", default="", help="read the steps from this file instead of standard input")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0 or args.page_size <= 0 or 64 % args.page_size:
        print("error: --max-tokens must be positive and --page-size must divide 64", file=sys.stderr)
        return 2

    import numpy as np
    import torch
    from .. import kernels
    from .engine import Engine, Options
    from .step import StepEntry
    from ..config.base import load_config

    os.makedirs(args.out, exist_ok=True)
    cfg = load_config(args.model)
    max_pos = getattr(cfg, "max_position_embeddings", args.max_tokens)
    pages = -(-args.max_tokens // args.page_size)
    eng = Engine(args.model, Options(device=args.device, dtype=args.dtype, max_seq=max_pos,
                                     block_size=args.page_size, num_blocks=pages,
                                     max_step_tokens=max(args.max_tokens, 1), max_batch=8))
    live = {}
    held = {}       # request id -> tokens fed so far (the position of its next token)
    index = []
    source = open(args.trace, "r", encoding="utf-8") if args.trace else sys.stdin
    with torch.no_grad():
        for line in source:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            step = rec["step"]
            entries = []
            for e in rec.get("entries", []):
                rid = e["id"]
                if rid not in live:
                    live[rid] = eng.cache.open()
                entries.append(StepEntry(live[rid], [int(t) for t in e["tokens"]],
                                         [int(w) for w in e.get("want", [])]))
            if entries:
                logits = eng.runner.run(entries)
                rows = []
                for e, rec_e in zip(entries, rec["entries"]):
                    start = held.get(rec_e["id"], 0)
                    rows.extend((rec_e["id"], start + w) for w in e.want)
                    held[rec_e["id"]] = start + len(e.tokens)
                if logits is not None:
                    arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f"{step}.f32.part")
                    arr.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
                    with open(tmp, "wb") as f:
                        np.save(f, np.ascontiguousarray(arr))
                    os.replace(tmp, os.path.join(args.out, f"step_{step}.npy"))
                    index.extend({"step": step, "row": i, "request": rid, "position": pos}
                                 for i, (rid, pos) in enumerate(rows))
            for rid in rec.get("end", []):
                if rid in live:
                    eng.cache.close(live.pop(rid))
                    held.pop(rid, None)
            torch.cuda.synchronize()
            kernels.check_status(eng.device)
            print(f"done {step}", flush=True)
    if args.trace:
        source.close()
    with open(os.path.join(args.out, "index.json"), "w", encoding="utf-8") as f:
        json.dump({"vocab": eng.runner.vocab, "dtype": args.dtype, "rows": index}, f)
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
