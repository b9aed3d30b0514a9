"""Generation through the Python entry point, the command line and the scheduler:
greedy and temperature, alone and batched, long decoding, the first tokens of a
sequence, pages running out."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import TOL, assert_close, make_weights, plain_logits, prompts_for, write_model_dir
from plain import llama_plain as plain
from plain import sampling_plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def check_choices(w, cfg, dtype, prompt, generated, temperature=0.0, seed=0, rid=0, eos=()):
    """Every generated token is what the plain implementation would choose from
    the same history, up to the rounding allowed between engine and plain."""
    ids = list(prompt) + list(generated)
    logits = plain_logits(w, cfg, ids[:-1], dtype)
    slack = TOL[dtype] * np.abs(logits).max()
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        if temperature <= 0:
            assert row[tok] >= row.max() - 2 * slack, f"token {i}: {tok} is not the maximum"
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 2 * slack:           # no near tie: the choice is forced
                assert tok == plain.argmax_first(row), f"token {i}"
        else:
            u = sampling_plain.uniform(seed, rid, i)
            cdf = np.cumsum(plain.temperature_probs(row, temperature))
            lo = cdf[tok - 1] if tok else 0.0
            eps = 4 * slack / temperature + 1e-5         # how far rounding can move a CDF edge
            assert lo - eps <= u <= cdf[tok] + eps, f"draw {i}: token {tok} does not bracket u={u}"
        if i < len(generated) - 1:
            assert tok not in eos, "generation went on after EOS"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_through_the_entry_point(tmp_path, name, dtype):
    import kllm_b200
    cfg, w = make_weights(name, dtype)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = prompts_for(cfg, [5, 17, 31, 64] if name == "A" else [1, 3, 40, 100], seed=1)
    steps = 16 if name == "A" else 24
    outs = kllm_b200.generate(d, prompts, steps=steps, max_seq=cfg["max_position_embeddings"], dtype=dtype)
    eos = (cfg["eos_token_id"],) if "eos_token_id" in cfg else ()
    for p, out in zip(prompts, outs):
        assert 1 <= len(out) <= steps and (len(out) == steps or out[-1] in eos)
        check_choices(w, cfg, dtype, p, out, eos=eos)
    solo = kllm_b200.generate(d, prompts[2], steps=steps, max_seq=cfg["max_position_embeddings"], dtype=dtype)
    if dtype == "float32":
        assert solo == outs[2]                      # batching is invisible
        assert solo == plain.greedy_generate(w, cfg, prompts[2], steps, eos=set(eos))


def test_temperature_is_reproducible_and_independent_of_batching(tmp_path):
    from kllm_b200.engine import Engine, Options, Scheduler
    cfg, w = make_weights("B")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = prompts_for(cfg, [1, 3, 40, 100, 128, 200], seed=3)
    eng = Engine(d, Options(dtype="float32", max_seq=256, num_blocks=80, max_batch=4, max_step_tokens=64))
    runs = []
    for order in (range(6), reversed(range(6))):          # different batch compositions
        sched = Scheduler(eng)
        reqs = {}
        for i in order:
            reqs[i] = sched.submit(prompts[i], 24, temperature=0.8, seed=1234)
            reqs[i].rid = 100 + i                          # the draw is keyed by the request id
        sched.run()
        runs.append({i: r.generated for i, r in reqs.items()})
        assert eng.cache.free_pages() == [80]
    assert runs[0] == runs[1]
    for i, p in enumerate(prompts):
        check_choices(w, cfg, "float32", p, runs[0][i], temperature=0.8, seed=1234, rid=100 + i, eos=(511,))
    other = Scheduler(eng)
    r = other.submit(prompts[3], 24, temperature=0.8, seed=99)
    r.rid = 103
    other.run()
    assert r.generated != runs[0][3]                      # another seed, other draws
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_draws_are_valid_in_both_dtypes(tmp_path, dtype):
    import kllm_b200
    cfg, w = make_weights("A", dtype)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    p = prompts_for(cfg, [9], seed=8)[0]
    out = kllm_b200.generate(d, p, steps=20, max_seq=128, dtype=dtype, temperature=1.3, seed=5)
    check_choices(w, cfg, dtype, p, out, temperature=1.3, seed=5, rid=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    """One token of prompt, then token by token to the end of the position range."""
    from kllm_b200.engine import Engine, Options, StepEntry
    cfg, w = make_weights("B", dtype)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    ids = prompts_for(cfg, [256], seed=11)[0]
    eng = Engine(d, Options(dtype=dtype, max_seq=256, block_size=16, num_blocks=16, max_batch=2))
    req = eng.cache.open()
    rows = [eng.step([StepEntry(req, [t], [0])])[0].float().cpu().numpy() for t in ids]
    want = plain_logits(w, cfg, ids, dtype)
    assert_close(np.stack(rows[:4]), want[:4], dtype, "the first tokens of a sequence")
    assert_close(np.stack(rows), want, dtype, "256 tokens one by one")
    from kllm_b200.engine import StepError
    with pytest.raises(StepError, match="sequence limit"):
        eng.step([StepEntry(req, [1], [0])])              # position 256 does not exist
    assert req.length == 256
    eng.close()


def test_scheduler_on_the_gpu_with_pages_running_out(tmp_path):
    """So few pages that requests are preempted and recomputed; tokens equal the
    solo runs all the same."""
    from kllm_b200.engine import Engine, Options, Scheduler
    cfg, w = make_weights("A")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = prompts_for(cfg, [30, 25, 40, 12, 33], seed=21)
    eng = Engine(d, Options(dtype="float32", max_seq=128, block_size=4, num_blocks=28, max_batch=4,
                            max_step_tokens=24))
    sched = Scheduler(eng)
    reqs = [sched.submit(p, 30) for p in prompts]
    sched.run()
    assert sched.metrics.preemptions >= 1
    solo = Scheduler(eng)
    for p, r in zip(prompts, reqs):
        s = solo.submit(p, 30)
        solo.run()
        assert r.status == "finished" and r.generated == s.generated
    eng.cache.audit()
    assert eng.cache.free_pages() == [28]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pipelined_loop_equals_the_plain_loop_when_requests_end_early(tmp_path, dtype):
    """The scheduler launches a step before it has read the tokens of the step before.
    With an EOS id that requests really produce (taken from a first run), a request's end
    is seen one step late: the token of the step in flight is dropped and the other
    requests go on.  Tokens, ends and the pool equal the plain loop's."""
    from kllm_b200.engine import Engine, Options, Scheduler
    cfg, w = make_weights("A", dtype)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    prompts = prompts_for(cfg, [7, 19, 3, 30, 11], seed=31)
    eng = Engine(d, Options(dtype=dtype, max_seq=128, block_size=4, num_blocks=96, max_batch=4, max_step_tokens=32))

    def run(pipelined, eos=(), max_new=24):
        sched = Scheduler(eng, eos_token_ids=list(eos), pipelined=pipelined)
        reqs = [sched.submit(p, max_new if i != 1 else 5) for i, p in enumerate(prompts)]   # one ends on its count
        sched.run()
        assert all(r.status == "finished" for r in reqs)
        eng.cache.audit()
        assert eng.cache.free_pages() == [96]
        return [r.generated for r in reqs]

    free = run(False)
    assert run(True) == free
    eos = free[0][6]                                   # what request 0 says as its 7th token
    plain_loop, piped = run(False, [eos]), run(True, [eos])
    assert piped == plain_loop
    assert plain_loop[0][-1] == eos and len(plain_loop[0]) <= 7
    for got, full in zip(plain_loop, free):
        cut = full.index(eos) + 1 if eos in full else len(full)
        assert got == full[:cut]
    eng.close()


def test_command_line(tmp_path):
    cfg, w = make_weights("A")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "generate"), "--model", d, "--ids", "1 17 42 100 7",
           "--steps", "6", "--max-seq", "64", "--dtype", "float32"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert lines[0] == "prompt:    [1 17 42 100 7]"
    assert lines[1].startswith("generated: [") and lines[1].endswith("]")
    toks = [int(t) for t in lines[1][len("generated: ["):-1].split()]
    assert toks == plain.greedy_generate(w, cfg, [1, 17, 42, 100, 7], 6)
    bad = subprocess.run(cmd[:4] + ["--ids", "1 x 3"], capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and 'bad token id "x"' in bad.stderr
    # random-weights mode from the command line
    cfgfile = tmp_path / "cfg.json"
    import json
    cfgfile.write_text(json.dumps(cfg))
    rnd = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "generate"), "--model", str(tmp_path / "r"),
                          "--random-config", str(cfgfile), "--random-seed", "3", "--steps", "4"],
                         capture_output=True, text=True, timeout=300)
    assert rnd.returncode == 0, rnd.stderr
    assert os.path.exists(tmp_path / "r" / "model.safetensors") and "generated: [" in rnd.stdout
    # the cache sized from a byte budget: 2 layers x (k, v) x 2 kv heads x 16 slots x 16 dims x 4 bytes = 8 KiB a page
    sized = subprocess.run(cmd + ["--cache-gb", "0.0001"], capture_output=True, text=True, timeout=300)
    assert sized.returncode == 0, sized.stderr
    assert sized.stdout == out.stdout              # 12 pages hold the 11 tokens; same tokens as with the default pool
    small = subprocess.run(cmd + ["--cache-gb", "0.000001"], capture_output=True, text=True, timeout=300)
    assert small.returncode != 0 and "holds no page" in small.stderr


def test_cache_pool_from_a_byte_budget(tmp_path):
    from kllm_b200.engine import Engine, Options
    cfg, w = make_weights("B", "bfloat16")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    eng = Engine(d, Options(dtype="bfloat16", max_seq=64, block_size=16, cache_bytes=100_000))
    per = 3 * 2 * 1 * 16 * 32 * 2                  # layers x (k, v) x kv heads x slots x dims x bytes
    assert eng.cache.bytes_per_page() == per and eng.cache.num_pages == 100_000 // per == 16
    assert eng.cache.groups[0].storage.numel() * 2 == 16 * per
    out = eng.generate(prompts_for(cfg, [20], seed=4)[0], max_new_tokens=5)
    assert len(out) >= 1
    eng.close()


def test_a_captured_decode_graph_survives_a_larger_batch(tmp_path):
    """Decode graphs hold the addresses of the buffers they were recorded with.  A step of
    2 requests is captured, then a step of 70 requests runs (more tokens than any scratch
    buffer sized for the small step), then the 2-request graph is replayed: its logits must
    still be those of the plain implementation, and the large step's too."""
    from kllm_b200.engine import Engine, Options, StepEntry
    cfg, w = make_weights("B", "bfloat16")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    eng = Engine(d, Options(dtype="bfloat16", max_seq=64, block_size=16, num_blocks=4 * 72, max_batch=72,
                            max_step_tokens=512))
    seqs = prompts_for(cfg, [40, 23] + [5] * 70, seed=11)
    want = [plain_logits(w, cfg, ids, "bfloat16") for ids in seqs[:3]]
    small = [eng.cache.open() for _ in range(2)]
    eng.step([StepEntry(r, ids[:-4], []) for r, ids in zip(small, seqs)])
    rows = {0: [], 1: []}

    def decode_small(k):
        out = eng.step([StepEntry(r, [ids[len(ids) - 4 + k]], [0]) for r, ids in zip(small, seqs)]).cpu().numpy()
        for i in range(2):
            rows[i].append(out[i])

    decode_small(0)                     # eager run and capture of the 2-request step
    decode_small(1)                     # replay
    assert 2 in eng.runner.graphs and eng.runner.graphs[2].graph is not None
    many = [eng.cache.open() for _ in range(70)]
    eng.step([StepEntry(r, ids[:-1], []) for r, ids in zip(many[:35], seqs[2:37])])
    eng.step([StepEntry(r, ids[:-1], []) for r, ids in zip(many[35:], seqs[37:])])
    big = eng.step([StepEntry(r, ids[-1:], [0]) for r, ids in zip(many, seqs[2:])]).cpu().numpy()
    assert_close(big[0], want[2][-1], "bfloat16", "first request of the 70-request step")
    decode_small(2)                     # the old graph again, after the scratch grew
    decode_small(3)
    for i in range(2):
        assert_close(np.stack(rows[i]), want[i][-4:], "bfloat16", f"request {i} decoded by the replayed graph")
    for r in small + many:
        eng.cache.close(r)
    eng.cache.audit()
    eng.close()


def test_sequence_logits_stay_valid_over_the_next_step(tmp_path):
    """``Sequence_.forward`` hands out the caller's own tensor: the logits of step t are
    unchanged after step t + 1 has replayed the same decode graph."""
    from kllm_b200.engine import Engine, Options
    cfg, w = make_weights("A", "float32")
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    eng = Engine(d, Options(dtype="float32", max_seq=64))
    ids = prompts_for(cfg, [12], seed=2)[0]
    want = plain_logits(w, cfg, ids, "float32")
    seq = eng.new_sequence()
    seq.forward(ids[:8])
    kept = [seq.forward([t]) for t in ids[8:]]        # four single-token steps: eager, capture, replays
    for i, row in enumerate(kept):
        assert_close(row.cpu().numpy(), want[8 + i], "float32", f"kept logits of step {i}")
    seq.release()
    eng.close()
