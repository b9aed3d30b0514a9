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
  points     decode at batch 1 and at batch 64

Weights are random and token ids synthetic (there is neither a checkpoint nor a
dataset here).  Every decode step reads about 2.4 GB, far more than the 126 MB of
L2, so nothing is flushed between steps.  ``--impl reference`` runs the reference's
own CUDA backend (float32, built unmodified by baseline/build_reference.py) through
its C ABI for the same metric and sizes, or says why it cannot.

``--shape`` picks the layer sizes of another Llama (with ``--layers`` for fewer of
them) and ``--prefill-tokens`` another prompt length: measurements at further sizes,
printed in the same form but not the bench line.
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
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="length of the timed prompt")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="decode: the batch's decode run alone; prefill: the 2048-token prompt alone (partial "
                         "records for profiling small cases, not the bench line)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--timeline", action="store_true",
                    help="decode run with the instrumented kernel builds; prints where the last step's time went, "
                         "kernel by kernel (not a bench line)")
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
    from kllm_b200.engine import Engine, Options, Scheduler
    from kllm_b200.weights import write_random_model

    cfg = dict(SHAPES[args.shape])
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], args.context, args.prefill_tokens)
    layers_full = cfg["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg["num_hidden_layers"] = layers
    B, ctx, K, W = args.batch, args.context, args.steps, args.warmup
    shape_name = {"tinyllama-1.1b": "TinyLlama 1.1B shape", "llama2-7b": "Llama-2 7B shape",
                  "llama3-8b": "Llama-3 8B shape"}[args.shape]
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="kllm_b200_bench_")
    try:
        t_w = time.time()
        write_random_model(tmp, cfg, seed=4, dtype=torch.bfloat16)
        print(f"[bench] random weights written in {time.time() - t_w:.1f} s", file=sys.stderr, flush=True)
        page = 64
        max_b = max(B, 64 if not args.no_points else B)
        pages = max(max_b * (-(-ctx // page)), -(-args.prefill_tokens // page)) + 8
        eng = Engine(tmp, Options(dtype="bfloat16", max_seq=max(ctx, args.prefill_tokens), block_size=page, num_blocks=pages,
                                  max_batch=max_b, max_step_tokens=max(args.prefill_tokens, max_b),
                                  cuda_graphs=not args.no_graphs))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    g = torch.Generator().manual_seed(1)

    def prompts(n, length):
        return torch.randint(0, cfg["vocab_size"], (n, length), generator=g).tolist()

    def decode_run(batch, steps, warm, sample_clocks=False):
        """Prefill ``batch`` requests and decode them together so that the furthest
        one ends at context ``ctx``.  Prompts are prefilled one a step while earlier
        requests already decode, so the requests' contexts differ by up to ``batch``
        tokens (times the portions of a prompt longer than a step's budget); all of them stay live through both timed regions.  Returns (device ms
        per step, e2e ms per step, launches, h2d, d2h, clocks, cached tokens in the
        middle of the device-timed region)."""
        portions = -(-ctx // eng.runner.max_step_tokens)       # steps that one prompt's prefill takes
        total = 2 * (steps + warm) + batch * portions + 2
        plen = ctx - total
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
        # device-timed
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = kernels.launches
        t0 = time.time()
        ev0.record()
        for _ in range(steps):
            sched.step()
        ev1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        dev_ms = ev0.elapsed_time(ev1) / steps
        launches = (kernels.launches - l0) // steps
        assert len(sched.running) == batch, "a request ended inside the timed region"
        cached = sum(r.cache.length for r in sched.running) - batch * steps // 2
        # end to end: wall clock around the public API, synchronised on both sides
        for _ in range(warm):
            sched.step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            sched.step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - w0) * 1e3 / steps
        t2 = time.time()
        csum = None
        if clocks:
            time.sleep(0.15)
            clocks.stop()
            csum = clocks.summary(t0, t2)          # both timed regions: device-timed and end-to-end
        assert len(sched.running) == batch, "a request ended inside the timed region"
        h2d = eng.runner.last_h2d_bytes
        sched.stop()
        return dev_ms, e2e_ms, launches, h2d, batch * 4, csum, cached

    def prefill_run(T=args.prefill_tokens):
        from kllm_b200.engine import StepEntry
        ids = prompts(1, T)[0]
        times = []
        for _ in range(4):
            req = eng.cache.open()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            eng.runner.run([StepEntry(req, ids, [T - 1])])
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
            eng.cache.close(req)
        ms = min(times[1:])
        per_layer, _ = model_bytes_and_flops(cfg, layers)
        qd = cfg["num_attention_heads"] * cfg["head_dim"]
        flops = 2 * T * (per_layer * layers) + 2 * cfg["vocab_size"] * cfg["hidden_size"] \
            + 2 * T * T * qd * layers          # causal attention: QK^T and PV over half the square
        return {"value": round(T / (ms * 1e-3), 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    if args.only == "prefill":
        with torch.no_grad():
            print(json.dumps({"partial": "prefill only", "layers": layers, "prefill": prefill_run()}))
        return 0

    if args.timeline:
        with torch.no_grad():
            dev_ms = decode_run(B, K, W)[0]
        print_timeline(kernels.timeline(), dev_ms)
        return 0

    with torch.no_grad():
        dev_ms, e2e_ms, launches, h2d, d2h, clocks, cached = decode_run(B, K, W, sample_clocks=True)
        per_layer, weight_elems = model_bytes_and_flops(cfg, layers)
        kv_bytes = cached * eng.cache.bytes_per_token_full()
        step_bytes = 2 * weight_elems + kv_bytes
        achieved = step_bytes / (dev_ms * 1e-3) / 1e9
        out = {
            "metric": f"decode tok/s at batch {B} ({shape_name}, context {ctx})",
            "value": round(B / (dev_ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic token ids, random weights (seed 4)",
            "config": {"model": shape_name.replace("TinyLlama 1.1B", "TinyLlama-1.1B"), "global_batch": B, "seq_len": ctx, "parallelism": "single GPU",
                       "layers": layers, "layers_of_config": layers_full, "hidden": cfg["hidden_size"],
                       "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                       "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                       "vocab": cfg["vocab_size"], "page_size": 64,
                       "l2": f"step reads {step_bytes / 1e9:.1f} GB > 126 MB L2, no flush",
                       "peaks": pk["source"]},
            "clocks": clocks,
            "e2e": {"value": round(B / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches * K,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes,
                         "mean_context": cached // B},
        }
        if not args.no_points:
            out["prefill"] = prefill_run()
            pts = {}
            for b in (1, 64):
                dms = decode_run(b, max(8, K // 2), 3)[0]
                pts[f"decode_b{b}"] = round(b / (dms * 1e-3), 1)
            out["points"] = pts
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
