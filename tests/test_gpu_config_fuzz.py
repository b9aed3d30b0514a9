"""Configurations drawn at random (seeded): sizes that are no power of two, head sizes
the tensor-core kernels do not take, odd vocabularies, every group width.  Each model runs
a whole prompt, its last tokens one by one, and three requests decoding side by side, in
float32 and bfloat16, against the plain implementation.  A size that a kernel does not
take must show as an error when the engine is built or stepped, never as a wrong logit;
the sizes drawn here are all meant to run."""
import numpy as np
import pytest

from helpers import assert_close, plain_logits, write_model_dir
from plain import llama_plain as plain

pytestmark = pytest.mark.gpu

HEAD_DIMS = [6, 8, 10, 16, 18, 24, 32, 34, 40, 48, 64, 72, 80, 96, 112, 128, 144, 200, 256]
HIDDEN = [24, 40, 56, 64, 72, 88, 100, 128, 136, 200, 256, 264, 328, 384]
INTER = [24, 50, 96, 100, 172, 173, 256, 333, 384, 640, 700]
VOCAB = [97, 257, 512, 1001, 2053, 5003]


def draw(seed: int) -> dict:
    rng = np.random.default_rng(1000 + seed)
    n_kv = int(rng.choice([1, 2, 3, 4, 5]))
    group = int(rng.choice([1, 2, 3, 4, 6, 8]))
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": int(rng.integers(1, 4)), "hidden_size": int(rng.choice(HIDDEN)),
        "num_attention_heads": n_kv * group, "num_key_value_heads": n_kv,
        "head_dim": int(rng.choice(HEAD_DIMS)), "intermediate_size": int(rng.choice(INTER)),
        "vocab_size": int(rng.choice(VOCAB)), "rope_theta": float(rng.choice([1e4, 5e5, 1e6])),
        "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-6])), "max_position_embeddings": 256,
        "tie_word_embeddings": bool(rng.integers(0, 2)),
    }


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(24))
def test_drawn_configuration(tmp_path, seed, dtype):
    from kllm_b200.engine import Engine, Options, StepEntry
    cfg = draw(seed)
    w = plain.random_weights(cfg, seed, gain_std=0.1, std=0.05)
    # attention far from uniform, as sharp as in helpers.make_weights: a score's spread grows
    # with the width (q and k are sums over it), so the factor shrinks with the root of it
    boost = (3.0 if dtype == "float32" else 2.0) * (64.0 / cfg["hidden_size"]) ** 0.5
    for k in list(w):
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = (w[k] * boost).astype(np.float32)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    rng = np.random.default_rng(seed)
    page = int(rng.choice([16, 32, 64]))
    eng = Engine(d, Options(dtype=dtype, max_seq=256, block_size=page, num_blocks=1024 // page, max_batch=4))
    what = f"drawn {seed} {dtype} {cfg['num_attention_heads']}/{cfg['num_key_value_heads']}x{cfg['head_dim']} " \
           f"d{cfg['hidden_size']} f{cfg['intermediate_size']} V{cfg['vocab_size']} pages of {page}"

    # a whole prompt, logits everywhere
    ids = rng.integers(0, cfg["vocab_size"], size=int(rng.integers(40, 150))).tolist()
    want = plain_logits(w, cfg, ids, dtype)
    req = eng.cache.open()
    got = eng.step([StepEntry(req, ids, list(range(len(ids))))]).cpu().numpy()
    eng.cache.close(req)
    assert_close(got, want, dtype, what + " whole")

    # most of it in one step, the last 6 tokens one by one
    req = eng.cache.open()
    cut = len(ids) - 6
    eng.step([StepEntry(req, ids[:cut], [])])
    for i in range(cut, len(ids)):
        got = eng.step([StepEntry(req, [ids[i]], [0])]).cpu().numpy()
        assert_close(got, want[i:i + 1], dtype, what + f" token {i} alone")
    eng.cache.close(req)

    # three requests of different lengths decoding side by side
    seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in (9, 33, 70)]
    wants = [plain_logits(w, cfg, s, dtype) for s in seqs]
    reqs = [eng.cache.open() for _ in seqs]
    eng.step([StepEntry(r, s[:-4], []) for r, s in zip(reqs, seqs)])
    for back in range(4, 0, -1):
        got = eng.step([StepEntry(r, [s[-back]], [0]) for r, s in zip(reqs, seqs)]).cpu().numpy()
        for j, (s, wj) in enumerate(zip(seqs, wants)):
            assert_close(got[j:j + 1], wj[len(s) - back:len(s) - back + 1], dtype, what + f" batch of 3, request {j}")
    for r in reqs:
        eng.cache.close(r)
    eng.cache.audit()
    eng.close()
