#!/usr/bin/env python3
"""Throughput of the engine on one GPU: decoded tokens a second.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

Default run: the layer sizes of TinyLlama-1.1B (22 layers, hidden 2048, 32 heads
over 4 kv heads of 64, feed-forward 5632, vocabulary 32000) with random bfloat16
weights, 8 requests decoding at a context of 2048 tokens.  A "step" is one decode
step of the whole batch.  One JSON line is printed:

  value      decoded tokens a second, K steps between two CUDA events on the
             launching stream (device time, after W warm-up steps)
  e2e        the same through the public Python API (Scheduler.step): every step
             copies its inputs from pinned host memory and reads its tokens back
  prefill    one prompt of 2048 tokens in one step, with the fraction of the
             bfloat16 tensor peak that its flops reach
  roofline   the decode step against HBM bandwidth: every weight once plus the
             cache of the live requests, over the step's time
  points     decode at batch 1 and at batch 64, and BASELINE.json's stated decode
             workload: batch 8, prompts of 512 tokens, 256 tokens generated each, all of
             them timed
  points_fp32  the float32 path of this engine on the same model (decode at batch 8,
             the 2048-token prompt): the reference computes in float32 only, so this is
             the arm to hold against it at equal precision
  spread     the K-step region is timed several times over; ``value`` is the median,
             ``spread`` the fastest and slowest repeat

Weights are random and token ids synthetic (there is neither a checkpoint nor a
dataset here).  Every decode step reads about 2.4 GB, far more than the 126 MB of
L2, so nothing is flushed between steps.  ``--impl reference`` runs the reference's
own CUDA backend (float32, built unmodified by baseline/build_reference.py) through
its C ABI for the same metric and sizes, or says why it cannot.

``--shape`` picks the layer sizes of another Llama (with ``--layers`` for fewer of
them) and ``--prefill-tokens`` another prompt length: measurements at further sizes,
printed in the same form but not the bench line; their weights are drawn on the device.
``--workload llama2-7b-mixed`` runs BASELINE.json's continuous-batching workload (32
requests, prompt lengths uniform in [128, 3072], 128 new tokens each) through the
scheduler and prints a record of its own.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TINYLLAMA = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 22, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 4,
    "head_dim": 64, "intermediate_size": 5632, "vocab_size": 32000, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 2048, "tie_word_embeddings": False,
}
SHAPES = {
    "tinyllama-1.1b": TINYLLAMA,
    "llama2-7b": dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                      num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32000,
                      max_position_embeddings=4096),
    "llama3-8b": dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
                      rope_theta=500000.0, max_position_embeddings=8192),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        if "bf16_tflops_sustained" in d:
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        return out
    except Exception:
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.rows = []
        self.proc = None
        exe = shutil.which("nvidia-smi")
        if exe:
            self.proc = subprocess.Popen([exe, f"--id={device}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6] or [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        mhz = sorted(int(float(r[0])) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(float(rows[0][1])), "reasons": reasons,
                "samples": len(rows)}


def model_bytes_and_flops(cfg, layers):
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (qd + 2 * kd) + qd * d + 3 * d * f           # matrix elements of one layer
    return per_layer, per_layer * layers + v * d                   # head counted once, embedding rows negligible


def reference_arm(args):
    """--impl reference: the reference's own CUDA backend, float32, through its C ABI
    (baseline/reference_arm.py), same metric and sizes; one JSON line."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    import reference_arm as ra
    why = ra.available()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: the reference runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.shape != "tinyllama-1.1b" or args.prefill_tokens != 2048:
        print("bench.py: the reference arm measures the default shape and prompt length only")
        return 2
    cfg = dict(TINYLLAMA)
    layers_full = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or layers_full
    B, ctx, K, W = args.batch, args.context, args.steps, max(3, args.warmup)
    points = not args.no_points and args.only == "all"
    ref = ra.Reference(cfg, max_seqs=max(B, 64 if points else B), max_seq=ctx)
    clocks = ClockSampler(0)
    t0 = time.time()
    ms = ref.decode_run(B, ctx, K, W)
    t1 = time.time()
    time.sleep(0.15)
    clocks.stop()
    out = {"impl": "reference", "metric": "decode tok/s at batch 8 (TinyLlama 1.1B shape, context 2048)",
           "value": round(B / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
           "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "fp32", "data": "synthetic token ids, random weights",
           "config": {"model": "TinyLlama-1.1B shape", "global_batch": B, "seq_len": ctx, "parallelism": "single GPU",
                      "layers": cfg["num_hidden_layers"], "layers_of_config": layers_full, "page_size": 16,
                      "how": "reference backend (backend/*.cu, unmodified) through its C ABI te_forward_batch; "
                             "wall clock around the synchronous call, logits to the host every step as it does"},
           "clocks": clocks.summary(t0, t1),
           "e2e": {"value": round(B / (ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4),
                   "h2d_bytes_per_step": B * 4 * 3 + B * ref.blocks_per_seq * 4,
                   "d2h_bytes_per_step": B * cfg["vocab_size"] * 4}}
    if points:
        pms = ref.prefill_run(2048)
        out["prefill"] = {"value": round(2048 / (pms * 1e-3), 1), "tokens": 2048, "ms": round(pms, 3)}
        out["points"] = {f"decode_b{b}": round(b / (ref.decode_run(b, ctx, max(8, K // 4), 3) * 1e-3), 1) for b in (1, 64)}
    print(json.dumps(out))
    return 0


def print_timeline(rows, dev_ms):
    """The instrumented kernels of the last step, in time order: for each the phases
    between its marks (mean over the recorded CTAs, microseconds) and how long after the
    previous instrumented kernel's end it ended."""
    if not rows:
        print("no instrumented kernel ran")
        return
    # the last step: walk back from the newest row until the gap between two kernels is
    # larger than any inside a step (the host's work between steps)
    last = [rows[-1]]
    for r in reversed(rows[:-1]):
        if last[0]["start"] - r["end"] > 400_000 or r["start"] > last[0]["start"]:
            break
        last.insert(0, r)
    t0 = last[0]["start"]
    print(f"decode step of {dev_ms * 1e3:.0f} us (device time); {len(last)} instrumented kernels in the last step; "
          "times in us")
    prev_end = None
    for r in last:
        marks = [m for m in r["marks"]]
        n = max(int((m > 0).sum()) for m in marks)
        phases = []
        for i in range(1, n):
            d = [(m[i] - m[i - 1]) / 1e3 for m in marks if m[i] > 0 and m[i - 1] > 0]
            phases.append(f"{sum(d) / len(d):5.2f}" if d else "    -")
        since = f"{(r['end'] - prev_end) / 1e3:6.2f}" if prev_end is not None else "     -"
        print(f"  {r['kernel']:<36s} start {(r['start'] - t0) / 1e3:8.2f}  end {(r['end'] - t0) / 1e3:8.2f}  "
              f"after previous end {since}  phases {' '.join(phases)}")
        prev_end = r["end"]


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--shape", default="tinyllama-1.1b", choices=sorted(SHAPES),
                    help="layer sizes; other than the default it is a measurement at further sizes, not the bench line")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the whole line is measured on the true 32-bit path (not the bench line)")
    ap.add_argument("--repeats", type=int, default=0, help="how often the K-step region is timed (0: 5, or 3 for K > 40)")
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="length of the timed prompt")
    ap.add_argument("--no-points", action="store_true", help="skip the further points and the prefill")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "attention", "products"],
                    help="decode: the batch's decode run alone; prefill: the 2048-token prompt alone (partial "
                         "records for profiling small cases, not the bench line); attention: the tcgen05 attention "
                         "kernels of prompt portions alone, both forms, at a few shapes; products: the "
                         "weight-streaming products of small steps alone, at --rows rows")
    ap.add_argument("--rows", type=int, default=8, help="rows of X for --only products (1 to 16)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--timeline", action="store_true",
                    help="decode run with the instrumented kernel builds; prints where the last step's time went, "
                         "kernel by kernel (not a bench line)")
    ap.add_argument("--workload", default="", choices=["", "llama2-7b-mixed"],
                    help="llama2-7b-mixed: 32 requests, prompts uniform in [128, 3072], 128 new tokens each, through "
                         "the scheduler (a record of its own, not the bench line)")
    args = ap.parse_args()
    if args.timeline:
        os.environ["KLLM_B200_TIMELINE"] = "1"
        args.only = "decode"

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.only == "decode":
        args.no_points = True

    import torch
    from kllm_b200 import kernels
    from kllm_b200.engine import Engine, Options, Scheduler, StepEntry
    from kllm_b200.weights import write_random_model

    if args.workload:
        return mixed_workload(args)
    if args.only == "attention":
        return attention_forms()
    if args.only == "products":
        return streaming_products(args.rows, args.dtype)

    cfg = dict(SHAPES[args.shape])
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context, args.prefill_tokens)
    layers_full = cfg["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg["num_hidden_layers"] = layers
    B, ctx, K, W = args.batch, args.context, args.steps, args.warmup
    R = args.repeats or (5 if K <= 40 else 3)
    shape_name = {"tinyllama-1.1b": "TinyLlama 1.1B shape", "llama2-7b": "Llama-2 7B shape",
                  "llama3-8b": "Llama-3 8B shape"}[args.shape]
    pk = peaks()
    page = 64
    default_line = args.shape == "tinyllama-1.1b" and args.dtype == "bfloat16"
    full = default_line and not args.no_points            # the further points of the bench line
    max_b = max(B, 64 if full else B)

    def options(dtype, batch_limit):
        pages = max(batch_limit * (-(-ctx // page)), -(-args.prefill_tokens // page)) + 8
        return Options(dtype=dtype, max_seq=max(ctx, args.prefill_tokens), block_size=page, num_blocks=pages,
                       max_batch=batch_limit, max_step_tokens=max(args.prefill_tokens, batch_limit),
                       cuda_graphs=not args.no_graphs)

    tmp = None
    if args.shape == "tinyllama-1.1b":
        # the default model goes through the random-weights mode's folder and the loader
        tmp = tempfile.mkdtemp(prefix="kllm_b200_bench_")
        t_w = time.time()
        write_random_model(tmp, cfg, seed=4, dtype=torch.bfloat16)
        print(f"[bench] random weights written in {time.time() - t_w:.1f} s", file=sys.stderr, flush=True)

    def make_engine(dtype, batch_limit):
        if tmp is not None:
            return Engine(tmp, options(dtype, batch_limit))
        return Engine(None, options(dtype, batch_limit), config=cfg, random_seed=4)    # drawn on the device

    g = torch.Generator().manual_seed(1)

    def prompts(n, length):
        return torch.randint(0, cfg["vocab_size"], (n, length), generator=g).tolist()

    def decode_run(eng, batch, steps, warm, repeats, sample_clocks=False):
        """Prefill ``batch`` requests and decode them together so that the furthest one
        ends at context ``ctx``.  Prompts are prefilled one a step while earlier requests
        already decode, so the requests' contexts differ by up to ``batch`` tokens (times
        the portions of a prompt longer than a step's budget); all of them stay live
        through every timed region.  The region of ``steps`` decode steps is timed
        ``repeats`` times, each time by CUDA events on the launching stream (device time)
        and by the wall clock around the same calls of the public API with a synchronise
        on both sides (end to end: every step copies its inputs from pinned host memory
        and the host reads the step's tokens).  Returns a dict."""
        portions = -(-ctx // eng.runner.max_step_tokens)       # steps that one prompt's prefill takes
        total = repeats * steps + warm + batch * portions + 2
        plen = ctx - total
        if plen < 1:
            raise SystemExit(f"bench.py: {repeats} x {steps} steps do not fit a context of {ctx}")
        sched = Scheduler(eng)
        for p in prompts(batch, plen):
            sched.submit(p, total)
        while any(r.fed < len(r.prompt) for r in list(sched.running) + list(sched.waiting)):
            sched.step()
        assert len(sched.running) == batch
        for _ in range(warm):
            sched.step()
        torch.cuda.synchronize()
        clocks = ClockSampler(eng.options.device) if sample_clocks else None
        if clocks:
            time.sleep(0.1)                                    # let the sampler's first rows arrive
        dev, e2e, launches = [], [], 0
        cached_mid = 0
        t0 = time.time()
        for rep in range(repeats):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            l0 = kernels.launches
            w0 = time.perf_counter()
            ev0.record()
            for _ in range(steps):
                sched.step()
            ev1.record()
            torch.cuda.synchronize()
            w1 = time.perf_counter()
            dev.append(ev0.elapsed_time(ev1) / steps)
            e2e.append((w1 - w0) * 1e3 / steps)
            launches = (kernels.launches - l0) // steps
            assert len(sched.running) == batch, "a request ended inside the timed region"
            if rep == repeats // 2:
                cached_mid = sum(r.cache.length for r in sched.running) - batch * steps // 2
            if clocks and time.time() - t0 < 0.3 and rep == repeats - 1:
                time.sleep(0.3 - (time.time() - t0))           # a few more samples of a very short run
        t1 = time.time()
        csum = None
        if clocks:
            time.sleep(0.1)
            clocks.stop()
            csum = clocks.summary(t0, t1)
        h2d = eng.runner.last_h2d_bytes
        sched.stop()
        i = sorted(range(repeats), key=lambda j: dev[j])[repeats // 2]     # the median repeat
        return {"dev_ms": dev[i], "e2e_ms": median(e2e), "dev_all": dev, "launches": launches, "h2d": h2d,
                "d2h": batch * 4, "clocks": csum, "cached": cached_mid}

    def decode_512_run(eng, batch=8, plen=512, new=256):
        """BASELINE.json's decode workload: ``batch`` prompts of 512 tokens, 256 tokens
        generated each; every decode step is timed (device time between two events)."""
        times = []
        for _ in range(2):                                   # the first pass warms up (graphs of the batch sizes)
            sched = Scheduler(eng)
            for p in prompts(batch, plen):
                sched.submit(p, new)
            while any(r.fed < len(r.prompt) for r in list(sched.running) + list(sched.waiting)):
                sched.step()
            torch.cuda.synchronize()
            d0 = sched.metrics.decode_tokens
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            sched.run()
            ev1.record()
            torch.cuda.synchronize()
            times.append((sched.metrics.decode_tokens - d0) / (ev0.elapsed_time(ev1) * 1e-3))
        return round(times[-1], 1)

    def prefill_run(eng, T=args.prefill_tokens):
        ids = prompts(1, T)[0]
        times = []
        for _ in range(7):                                  # the first two are warm-up (library set-up, first use of a route)
            req = eng.cache.open()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            eng.runner.run([StepEntry(req, ids, [T - 1])])
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
            eng.cache.close(req)
        times = times[2:]
        ms = median(times)
        per_layer, _ = model_bytes_and_flops(cfg, layers)
        qd = cfg["num_attention_heads"] * cfg["head_dim"]
        flops = 2 * T * (per_layer * layers) + 2 * cfg["vocab_size"] * cfg["hidden_size"] \
            + 2 * T * T * qd * layers          # causal attention: QK^T and PV over half the square
        out = {"value": round(T / (ms * 1e-3), 1), "tokens": T, "ms": round(ms, 3),
               "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "spread_ms": [round(min(times), 3), round(max(times), 3)]}
        if eng.dtype != torch.bfloat16:
            out["frac_of"] = "bf16 tensor peak (the float32 path does not use tensor cores)"
        return out

    def roofline(eng, run, batch):
        _, weight_elems = model_bytes_and_flops(cfg, layers)
        esize = 2 if eng.dtype == torch.bfloat16 else 4
        step_bytes = esize * weight_elems + run["cached"] * eng.cache.bytes_per_token_full()
        achieved = step_bytes / (run["dev_ms"] * 1e-3) / 1e9
        return step_bytes, {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                            "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes,
                            "mean_context": run["cached"] // batch}

    try:
        eng = make_engine(args.dtype, max_b)
        if args.only == "prefill":
            with torch.no_grad():
                print(json.dumps({"partial": "prefill only", "layers": layers, "prefill": prefill_run(eng)}))
            return 0
        if args.timeline:
            with torch.no_grad():
                run = decode_run(eng, B, K, W, 1)
            print_timeline(kernels.timeline(), run["dev_ms"])
            return 0

        with torch.no_grad():
            run = decode_run(eng, B, K, W, R, sample_clocks=True)
            step_bytes, roof = roofline(eng, run, B)
            dt = "bf16" if args.dtype == "bfloat16" else "fp32"
            out = {
                "metric": f"decode tok/s at batch {B} ({shape_name}, context {ctx})",
                "value": round(B / (run["dev_ms"] * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
                "ms_per_step": round(run["dev_ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": dt, "data": "synthetic token ids, random weights (seed 4)",
                "config": {"model": shape_name.replace("TinyLlama 1.1B", "TinyLlama-1.1B"), "global_batch": B,
                           "seq_len": ctx, "parallelism": "single GPU",
                           "layers": layers, "layers_of_config": layers_full, "hidden": cfg["hidden_size"],
                           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                           "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                           "vocab": cfg["vocab_size"], "page_size": page,
                           "l2": f"step reads {step_bytes / 1e9:.1f} GB > 126 MB L2, no flush",
                           "peaks": pk["source"], "repeats": R,
                           "timing": "median of the repeats of K steps; CUDA events, wall clock for e2e"},
                "spread": {"repeats": R, "min_ms": round(min(run["dev_all"]), 4), "max_ms": round(max(run["dev_all"]), 4)},
                "clocks": run["clocks"],
                "e2e": {"value": round(B / (run["e2e_ms"] * 1e-3), 1), "unit": "tokens/s",
                        "ms_per_step": round(run["e2e_ms"], 4),
                        "h2d_bytes_per_step": run["h2d"], "d2h_bytes_per_step": run["d2h"]},
                "gpu_launches": run["launches"] * K,
                "roofline": roof,
            }
            if not args.no_points:
                out["prefill"] = prefill_run(eng)
            if full:
                pts = {}
                for b in (1, 64):
                    pts[f"decode_b{b}"] = round(b / (decode_run(eng, b, K, 3, R)["dev_ms"] * 1e-3), 1)
                pts["decode_b8_ctx512"] = decode_512_run(eng)
                out["points"] = pts
                # the same model on the float32 path: what to hold against the reference, which
                # has no other precision
                eng.close()
                del eng
                torch.cuda.empty_cache()
                eng = make_engine("float32", B)
                r32 = decode_run(eng, B, K, 3, R)
                _, roof32 = roofline(eng, r32, B)
                out["points_fp32"] = {"decode_b8": round(B / (r32["dev_ms"] * 1e-3), 1),
                                      "decode_b8_ms_per_step": round(r32["dev_ms"], 4),
                                      "decode_b8_e2e": round(B / (r32["e2e_ms"] * 1e-3), 1),
                                      "decode_b8_hbm_frac": roof32["frac"],
                                      "prefill": prefill_run(eng)}
                out["precision"] = ("value and e2e are bfloat16; the reference arm computes in float32, its only "
                                    "precision: points_fp32 is this engine at that precision")
        print(json.dumps(out))
        return 0
    finally:
        if tmp is not None:
            shutil.rmtree(tmp, ignore_errors=True)


def attention_forms():
    """The two tcgen05 attention kernels of prompt portions (probabilities through shared
    memory / kept in tensor memory) alone, on random caches: microseconds per call and
    TFLOP/s of the causal work, by CUDA events over calls on alternating caches larger than
    L2 in sum.  One JSON record."""
    import math
    import torch
    from kllm_b200 import kernels
    dev, page, layers, reps = "cuda", 64, 6, 10
    rows = []
    for n_req, per, H, G, hd in ((1, 2048, 32, 4, 64), (1, 8192, 32, 4, 64), (8, 512, 32, 4, 64), (1, 512, 32, 4, 64),
                                 (1, 2048, 32, 8, 128), (1, 8192, 32, 8, 128), (1, 8192, 32, 32, 128)):
        T = n_req * per
        n_pages = n_req * (-(-per // page))
        caches = [(torch.randn(n_pages, G, page, hd, device=dev).bfloat16(),
                   torch.randn(n_pages, G, page, hd, device=dev).bfloat16()) for _ in range(layers)]
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(n_req, -1).contiguous()
        q = torch.randn(T, H * hd, device=dev).bfloat16()
        out = torch.empty_like(q)
        q_start = torch.arange(0, T + 1, per, dtype=torch.int32, device=dev)
        start_pos = torch.zeros(n_req, dtype=torch.int32, device=dev)
        rec = {"portions": n_req, "tokens_each": per, "heads": H, "kv_heads": G, "head_dim": hd}
        for form in ("smem", "tmem"):
            def call(i):
                kernels.attention_prefill_tcgen05(out, q, caches[i][0], caches[i][1], q_start, start_pos, table, n_req,
                                                  H, G, hd, 0, 1.0 / math.sqrt(hd), probabilities=form)
            for i in range(layers):
                call(i)
            torch.cuda.synchronize()
            kernels.check_status(dev)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for _ in range(reps):
                for i in range(layers):
                    call(i)
            ev1.record()
            torch.cuda.synchronize()
            us = ev0.elapsed_time(ev1) / (reps * layers) * 1e3
            rec[form] = {"us": round(us, 1), "tflops": round(2.0 * per * per * H * hd * n_req / us / 1e6, 1)}
        rows.append(rec)
        del caches
    print(json.dumps({"partial": "tcgen05 attention of prompt portions, both forms", "rows": rows}))
    return 0


def streaming_products(rows: int, dtype: str = "bfloat16"):
    """The weight-streaming products of steps of up to 16 tokens (csrc/skinny_gemm.cu; with
    ``--dtype float32`` csrc/skinny_gemm_f32.cu, up to 8 rows, TinyLlama's shapes) alone:
    microseconds per call and TB/s of weight bytes at ``rows`` rows of X, by CUDA events
    over 24 calls replayed as a graph on weights that rotate through more than L2 holds.
    One JSON record."""
    import torch
    from kllm_b200 import kernels
    dev = "cuda"
    torch.manual_seed(0)
    wt = torch.float32 if dtype == "float32" else torch.bfloat16
    esize = 4 if dtype == "float32" else 2
    cases = [("head 32000 x 2048", 32000, 2048, "norm", "f32"), ("head 128256 x 4096", 128256, 4096, "norm", "f32"),
             ("gate/up 2 x 14336 x 4096", 14336, 4096, "norm", "swiglu"),
             ("gate/up 2 x 5632 x 2048", 5632, 2048, "norm", "swiglu"), ("QKV 6144 x 4096", 6144, 4096, "norm", "bf16"),
             ("QKV 2560 x 2048", 2560, 2048, "norm", "bf16"), ("down 2048 x 5632", 2048, 5632, "x", "add"),
             ("down slice 4096 x 7168", 4096, 7168, "x", "add"), ("O 4096 x 4096", 4096, 4096, "x", "add"),
             ("O 2048 x 2048", 2048, 2048, "x", "add")]
    if dtype == "float32":
        cases = [c for c in cases if c[2] in (2048, 5632) and c[1] != 32000] + [("head 32000 x 2048", 32000, 2048, "norm", "f32")]
    out = []
    for name, N, K, pro, epi in cases:
        mats = 2 if epi == "swiglu" else 1
        copies = int(400e6 // (N * K * esize * mats)) + 1
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(wt) for _ in range(copies)]
        w2 = [(torch.randn(N, K, device=dev) * 0.02).to(wt) for _ in range(copies)] if mats == 2 else None
        xf = torch.randn(rows, K, device=dev)
        gain = torch.ones(K, device=dev)
        xb = xf.to(wt)
        if epi in ("bf16", "f32"):
            epi = "store"
        acc = torch.zeros(rows, N, device=dev)
        turn = [0]

        def call():
            j = turn[0] % copies
            turn[0] += 1
            if pro == "norm":
                kernels.skinny_gemm(ws[j], x_f32=xf, gain=gain, eps=1e-5, weight_up=w2[j] if w2 else None, epilogue=epi)
            else:
                kernels.skinny_gemm(ws[j], x=xb, epilogue="add", out=acc)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream), torch.cuda.graph(graph, stream=stream):
            for _ in range(24):
                call()
        times = []
        for _ in range(8):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            graph.replay()
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1) / 24 * 1e3)
        us = sorted(times)[len(times) // 2]
        out.append({"product": name, "us": round(us, 1), "tb_per_s": round(N * K * esize * mats / us / 1e6, 2)})
        del ws, w2
    print(json.dumps({"partial": f"weight-streaming products alone, {rows} rows, {dtype}", "rows": out}))
    return 0


def mixed_workload(args):
    """BASELINE.json's continuous-batching workload at the layer sizes of Llama-2 7B: 32
    requests, prompt lengths uniform in [128, 3072] (seeded), 128 new tokens each, greedy,
    through ``Scheduler.run``'s loop; random bfloat16 weights drawn on the device.  Prints one
    JSON record: generated tokens a second over the whole run (wall clock, prefill included),
    steps, preemptions, the pages' high-water mark, and for the steps that held single tokens
    only their device time against the bytes they had to read (weights once, the cache of the
    live requests)."""
    import torch
    from kllm_b200.engine import Engine, Options, Scheduler
    cfg = dict(SHAPES["llama2-7b"])
    layers_full = cfg["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    n_req, new = 32, 128
    rng = torch.Generator().manual_seed(5)
    lengths = torch.randint(128, 3073, (n_req,), generator=rng).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=rng).tolist() for n in lengths]
    page = 64
    pages = sum(-(-(n + new) // page) for n in lengths) + 8
    eng = Engine(None, Options(dtype="bfloat16", max_seq=3072 + new, block_size=page, num_blocks=pages, max_batch=n_req,
                               max_step_tokens=4096), config=cfg, random_seed=5)
    _, weight_elems = model_bytes_and_flops(cfg, layers)
    per_token = eng.cache.bytes_per_token_full()

    def run_once(record):
        sched = Scheduler(eng)
        reqs = [sched.submit(p, new) for p in prompts]
        marks = []
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((ev, None))
        while sched.waiting or sched.running or sched._inflight:
            before = sched.metrics.steps
            live = [r for r in sched.running]
            sched.step()
            if record and sched.metrics.steps > before:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                prefill = sched.metrics.prefill_tokens
                marks.append((ev, (prefill, sum(r.cache.length for r in sched.running if r.cache is not None),
                                   len(sched.running))))
        torch.cuda.synchronize()
        wall = time.perf_counter() - w0
        assert all(r.status == "finished" and len(r.generated) == new for r in reqs)
        return sched, wall, marks

    with torch.no_grad():
        run_once(False)                                  # warm-up: library set-up, graphs of the batch sizes
        clocks = ClockSampler(0)
        t0 = time.time()
        sched, wall, marks = run_once(True)
        t1 = time.time()
        time.sleep(0.15)
        clocks.stop()
    # steps whose entries were all single tokens: no prefill token was added by them
    dec_ms, dec_bytes, dec_steps = 0.0, 0, 0
    prev_prefill = 0
    for (e0, _), (e1, info) in zip(marks, marks[1:]):
        prefill, cached, live = info
        if prefill == prev_prefill and live > 0:
            dec_ms += e0.elapsed_time(e1)
            dec_bytes += 2 * weight_elems + cached * per_token
            dec_steps += 1
        prev_prefill = prefill
    m = sched.metrics
    out = {"workload": "llama2-7b-mixed", "metric": "generated tok/s, 32 requests, prompts U[128,3072], 128 new tokens each",
           "value": round(n_req * new / wall, 1), "unit": "tokens/s", "wall_s": round(wall, 3), "dtype": "bf16",
           "data": "synthetic token ids (seed 5), random weights drawn on the device (seed 5)",
           "config": {"model": "Llama-2 7B shape", "layers": layers, "layers_of_config": layers_full,
                      "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                      "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                      "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "requests": n_req,
                      "prompt_tokens": sum(lengths), "new_tokens_each": new, "page_size": page, "pages": pages,
                      "max_batch": n_req, "max_step_tokens": 4096, "peaks": pk["source"]},
           "steps": m.steps, "prefill_tokens": m.prefill_tokens, "decode_tokens": m.decode_tokens,
           "preemptions": m.preemptions, "pages_high_water": m.pages_high_water,
           "prompt_tokens_per_s": round(sum(lengths) / wall, 1),
           "decode_only_steps": {"steps": dec_steps, "ms_per_step": round(dec_ms / max(1, dec_steps), 3),
                                 "hbm_gbs": round(dec_bytes / max(1e-9, dec_ms * 1e-3) / 1e9, 1),
                                 "hbm_frac": round(dec_bytes / max(1e-9, dec_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
           "clocks": clocks.summary(t0, t1)}
    print(json.dumps(out))
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
