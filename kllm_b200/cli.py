"""``generate``: the command line, in the manner of the reference's cmd/generate
(cmd/generate/main.go:14-51): same option names and meanings where it has them,
same two output lines.

    generate --model DIR --ids "1 17 42 100 7" --steps 16 --max-seq 256 --device 0

``--backend`` named the CUDA backend library there; here the kernels are built
from source on first use, and the option names the folder where the built
libraries are kept.  Added: ``--temperature``, ``--seed``, ``--dtype``,
``--block-size``, ``--num-blocks``, ``--cache-gb``, ``--max-step-tokens``, and ``--random-config``
to write a random-weights model folder first.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _ids(text: str):
    out = []
    for f in text.split():
        try:
            out.append(int(f))
        except ValueError:
            raise SystemExit(f'error: bad token id "{f}"')
    return out


def _go_list(xs) -> str:
    return "[" + " ".join(str(int(x)) for x in xs) + "]"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", default="", help="folder for the built CUDA kernel libraries")
    ap.add_argument("--model", default="testmodels/tiny-llama", help="checkpoint directory (config.json + safetensors)")
    ap.add_argument("--device", type=int, default=0, help="CUDA device index")
    ap.add_argument("--ids", default="1 17 42 100 7", help="space-separated prompt token ids")
    ap.add_argument("--steps", type=int, default=16, help="max new tokens")
    ap.add_argument("--max-seq", type=int, default=256, help="KV capacity in tokens")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy; >0: sample from softmax(z/T)")
    ap.add_argument("--seed", type=int, default=0, help="sampler seed")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--num-blocks", type=int, default=0,
                    help="cache pages (0: from --cache-gb, else 4 * max-seq / block-size)")
    ap.add_argument("--cache-gb", type=float, default=0.0,
                    help="device memory for the paged cache in GB; sizes the pool when --num-blocks is 0")
    ap.add_argument("--max-step-tokens", type=int, default=0, help="token budget of one step (0: max-seq)")
    ap.add_argument("--random-config", default="", help="a config.json: write random weights for it into --model first")
    ap.add_argument("--random-seed", type=int, default=0, help="seed of --random-config")
    args = ap.parse_args(argv)

    if args.backend:
        os.environ["KLLM_B200_BUILD_DIR"] = args.backend
    prompt = _ids(args.ids)
    try:
        if args.random_config:
            import torch
            from .weights import write_random_model
            with open(args.random_config, "r", encoding="utf-8") as f:
                cfg = json.load(f)
            write_random_model(args.model, cfg, args.random_seed,
                               dtype=torch.float32 if args.dtype == "float32" else torch.bfloat16)
        from .engine import Engine, Options
        eng = Engine(args.model, Options(device=args.device, max_seq=args.max_seq, dtype=args.dtype,
                                         block_size=args.block_size, num_blocks=args.num_blocks,
                                         cache_bytes=int(args.cache_gb * 1e9),
                                         max_step_tokens=args.max_step_tokens))
        try:
            out = eng.generate(prompt, max_new_tokens=args.steps, temperature=args.temperature, seed=args.seed)
        finally:
            eng.close()
    except Exception as e:  # one line, like the reference's "error: ..."
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(f"prompt:    {_go_list(prompt)}\ngenerated: {_go_list(out)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
