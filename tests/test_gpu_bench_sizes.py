"""The engine against the plain implementation at the layer sizes that bench.py
measures: two layers of TinyLlama-1.1B's sizes (width 2048, 32 heads over 4 kv heads
of 64, feed-forward 5632, vocabulary 32000) and two layers of Llama-3-8B's (width
4096, 32 heads over 8 kv heads of 128, feed-forward 14336; the vocabulary is cut down
to 16032 rows and the position limit to 768, which the configuration says).

At these sizes the product takes routes that the tiny configurations never reach:
the tcgen05 attention of prompt portions, the tcgen05 gate/up product with the
activation in its epilogue, the weight-streaming products with a 2048- or 4096-wide
norm prologue, the down projection in column slices (width 14336), one and two token
tiles per weight tile (batch 4 and 12), captured decode steps with many key ranges.
Each route is checked alone in test_gpu_kernels.py; here they are checked together,
inside the engine, in every way of cutting the work:

  w    every request alone and whole, one step
  p    portions of 7 / 384 / 2 / 64 tokens
  d1   the longest request: most of it in one step, its last 32 tokens one by one
  d4   four requests, their last 32 tokens decoded together (batch 4)
  d12  three copies of each request, the last 32 tokens decoded together (batch 12)
  m    mixed steps as the scheduler orders them: single tokens of decoding requests
       first, then portions of prompts

In float32 the yardstick is the float64 formula, in bfloat16 the same formula with
the engine's roundings (helpers.plain_logits).  The reference checks its own engine
this way against recorded logits (engine/e2e/e2e_test.go:80-92, 178-251).
"""
import numpy as np
import pytest

from helpers import assert_close, plain_logits, write_model_dir
from trace_tools import TraceBuilder, portions, run_on_engine

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 768, "tie_word_embeddings": False}
SHAPES = {
    # name: (config, seed, factor on the q and k projections, page size)
    "tinyllama": (dict(BASE, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                       intermediate_size=5632, vocab_size=32000, rope_theta=10000.0), 4, 1.5, 64),
    "llama3-8b": (dict(BASE, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       intermediate_size=14336, vocab_size=16032, rope_theta=500000.0), 6, 1.0, 16),
}
LENGTHS = [700, 150, 70, 33]
CUTS = [7, 384, 2, 64]


def big_weights(cfg, seed, qk_boost):
    """N(0, 0.02) matrices and N(1, 0.05) gains, drawn in float32 (these models have up to
    half a billion elements); q and k scaled so that attention is far from uniform."""
    rng = np.random.default_rng(seed)
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd, nh, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]

    def mat(r, c, s=0.02):
        return rng.standard_normal((r, c), dtype=np.float32) * np.float32(s)

    def gain():
        return (1.0 + 0.05 * rng.standard_normal(d, dtype=np.float32)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(v, d), "lm_head.weight": mat(v, d), "model.norm.weight": gain()}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[p + ".self_attn.q_proj.weight"] = mat(nh * hd, d, 0.02 * qk_boost)
        w[p + ".self_attn.k_proj.weight"] = mat(nkv * hd, d, 0.02 * qk_boost)
        w[p + ".self_attn.v_proj.weight"] = mat(nkv * hd, d)
        w[p + ".self_attn.o_proj.weight"] = mat(d, nh * hd)
        w[p + ".mlp.gate_proj.weight"] = mat(f, d)
        w[p + ".mlp.up_proj.weight"] = mat(f, d)
        w[p + ".mlp.down_proj.weight"] = mat(d, f)
        w[p + ".input_layernorm.weight"] = gain()
        w[p + ".post_attention_layernorm.weight"] = gain()
    return w


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request, tmp_path_factory):
    cfg, seed, boost, page = SHAPES[request.param]
    w = big_weights(cfg, seed, boost)
    d = write_model_dir(str(tmp_path_factory.mktemp(request.param) / "model"), cfg, w)
    rng = np.random.default_rng(seed + 100)
    seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in LENGTHS]
    return {"name": request.param, "cfg": cfg, "weights": w, "dir": d, "seqs": seqs, "page": page, "plain": {}}


def build_trace(seqs):
    tb = TraceBuilder()
    marks = {}
    # w: whole
    marks["w"] = len(tb.steps)
    for i, ids in enumerate(seqs):
        tb.step([(f"w{i}", ids, range(len(ids)))], end=[f"w{i}"])
    # p: portions
    marks["p"] = len(tb.steps)
    for i, ids in enumerate(seqs):
        pos, cuts = 0, portions(len(ids), CUTS[i:] + CUTS[:i])
        for j, n in enumerate(cuts):
            tb.step([(f"p{i}", ids[pos:pos + n], range(n))], end=[f"p{i}"] if j == len(cuts) - 1 else [])
            pos += n
    # d1: the longest request alone, its last 32 tokens one by one
    marks["d1"] = len(tb.steps)
    ids = seqs[0]
    tb.step([("d1_0", ids[:-32], range(len(ids) - 32))])
    for t in range(len(ids) - 32, len(ids)):
        tb.step([("d1_0", [ids[t]], [0])], end=["d1_0"] if t == len(ids) - 1 else [])
    # d4 and d12: the last 32 tokens of 4 and of 12 requests decoded together
    for way, copies in (("d4", 1), ("d12", 3)):
        marks[way] = len(tb.steps)
        names = [(f"{way}_{i}_{c}", seqs[i]) for c in range(copies) for i in range(len(seqs))]
        for c in range(copies):       # the heads of four requests as one step of portions
            tb.step([(rid, ids[:-32], range(len(ids) - 32)) for rid, ids in names[c * 4:(c + 1) * 4]])
        for k in range(32, 0, -1):
            tb.step([(rid, [ids[len(ids) - k]], [0]) for rid, ids in names],
                    end=[rid for rid, _ in names] if k == 1 else [])
    # m: decoding requests first, then portions, as the scheduler orders a step
    marks["m"] = len(tb.steps)
    a, b, c, d = seqs
    tb.step([("m1", b[:-3], range(len(b) - 3))])
    tb.step([("m2", c[:-2], range(len(c) - 2))])
    tb.step([("m1", b[-3:-2], [0]), ("m2", c[-2:-1], [0]), ("m0", a[:300], range(300)), ("m3", d, range(len(d)))],
            end=["m3"])
    tb.step([("m1", b[-2:-1], [0]), ("m2", c[-1:], [0]), ("m0", a[300:698], range(398))], end=["m2"])
    tb.step([("m1", b[-1:], [0]), ("m0", a[698:], range(2))], end=["m1", "m0"])
    return tb, marks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_at_bench_sizes(shape, dtype, monkeypatch):
    from kllm_b200 import kernels
    from kllm_b200.engine import Engine, Options
    cfg, seqs, page = shape["cfg"], shape["seqs"], shape["page"]
    calls = []
    for name in ("attention_prefill_tcgen05", "attention_decode_fused", "attention_decode", "gemm", "skinny_gemm"):
        real = getattr(kernels, name)

        def spy(*a, _n=name, _r=real, **k):
            calls.append((_n, k.get("epilogue"), tuple(a[0].shape)))
            return _r(*a, **k)
        monkeypatch.setattr(kernels, name, spy)
    tb, marks = build_trace(seqs)
    eng = Engine(shape["dir"], Options(dtype=dtype, max_seq=768, block_size=page, num_blocks=12 * (768 // page),
                                       max_batch=12, max_step_tokens=1024))
    got = run_on_engine(eng, tb)
    eng.cache.audit()
    assert not eng.cache.live
    eng.close()

    if dtype == "bfloat16":
        names = {c[0] for c in calls}
        assert "attention_prefill_tcgen05" in names, "portions did not take the tcgen05 attention"
        assert ("gemm", "swiglu") in {c[:2] for c in calls}, "the 700-token step did not take the tcgen05 gate/up product"
        assert "attention_decode_fused" in names and "skinny_gemm" in names, "decode steps did not take the fused route"
        assert "attention_decode" in names, "the single tokens of a mixed step did not take the decode attention"
        widths = {c[2][1] for c in calls if c[0] == "skinny_gemm"}
        if cfg["intermediate_size"] > 11000:
            assert any(k < cfg["intermediate_size"] and k != cfg["hidden_size"] for k in widths), \
                "the down projection was not taken in column slices"

    if dtype not in shape["plain"]:
        shape["plain"][dtype] = [plain_logits(shape["weights"], cfg, ids, dtype) for ids in seqs]
    want = shape["plain"][dtype]

    def check(rid, i, lo, hi, what):
        rows = np.stack([got[(rid, p)] for p in range(lo, hi)])
        assert_close(rows, want[i][lo:hi], dtype, f"{shape['name']} {dtype} {what} request {i} (len {len(seqs[i])})")

    for i, ids in enumerate(seqs):
        n = len(ids)
        check(f"w{i}", i, 0, n, "whole")
        check(f"p{i}", i, 0, n, "portions")
        check(f"d4_{i}_0", i, 0, n, "last 32 at batch 4")
        for c in range(3):
            check(f"d12_{i}_{c}", i, 0, n, f"last 32 at batch 12 (copy {c})")
    check("d1_0", 0, 0, len(seqs[0]), "last 32 at batch 1")
    check("m0", 0, 0, len(seqs[0]), "mixed")
    check("m1", 1, 0, len(seqs[1]), "mixed")
    check("m2", 2, 0, len(seqs[2]), "mixed")
    check("m3", 3, 0, len(seqs[3]), "mixed")


def test_float32_decode_logits_do_not_depend_on_the_batch_bit_for_bit(shape):
    """The float32 path's decode steps run kernels of this repository only (for up to 8 tokens a
    step), and each of them sums a row in an order that depends on that row alone.  So a request
    that is decoded alone and the same request decoded beside three others (its prompt prefilled
    alone both times, so that the caches hold the same bits) must give the same logits bit for
    bit, not merely within a tolerance."""
    from kllm_b200.engine import Engine, Options, StepEntry
    cfg, seqs, page = shape["cfg"], shape["seqs"], shape["page"]
    eng = Engine(shape["dir"], Options(dtype="float32", max_seq=768, block_size=page, num_blocks=4 * (768 // page),
                                       max_batch=4, max_step_tokens=1024))
    runs = []
    for together in (False, True):
        reqs = [eng.cache.open() for _ in seqs]
        for r, ids in zip(reqs, seqs):
            eng.step([StepEntry(r, ids[:-8], [])])              # every prompt alone, the same steps in both runs
        rows = []
        for k in range(8, 0, -1):
            entries = [StepEntry(r, [ids[len(ids) - k]], [0]) for r, ids in zip(reqs, seqs)]
            if together:
                rows.append(eng.step(entries)[0].cpu().numpy())
            else:
                rows.append(eng.step(entries[:1])[0].cpu().numpy())
                for e in entries[1:]:
                    eng.step([e])
        runs.append(np.stack(rows))
        for r in reqs:
            eng.cache.close(r)
    eng.close()
    assert np.array_equal(runs[0], runs[1]), (
        f"{shape['name']}: float32 logits of a request decoded alone and in a batch of 4 differ by "
        f"{np.abs(runs[0] - runs[1]).max():.3e}")
    want = plain_logits(shape["weights"], cfg, seqs[0], "float32") if "float32" not in shape["plain"] else shape["plain"]["float32"][0]
    assert_close(runs[0], want[-8:], "float32", f"{shape['name']} float32 last 8 tokens alone")
