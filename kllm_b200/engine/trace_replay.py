"""Trace replay: feed given token ids through a model step by step and write the
logits.  It samples nothing.  It drives the engine's own model, step function,
cache manager and kernels, the ones that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step are one batch.  ``end``: requests that
are finished after this step; their pages are given back.  For a step in which
something is wanted, ``<out>/<step>.f32`` holds the logits [wanted, vocab] as
little-endian float32 in the order of the entries and of ``want``.  After every
step a line ``done <step>`` is printed and flushed.  The cache pool is sized for
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
    with torch.no_grad():
        for line in sys.stdin:
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
                if logits is not None:
                    arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f"{step}.f32.part")
                    arr.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            for rid in rec.get("end", []):
                if rid in live:
                    eng.cache.close(live.pop(rid))
            torch.cuda.synchronize()
            kernels.check_status(eng.device)
            print(f"done {step}", flush=True)
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
