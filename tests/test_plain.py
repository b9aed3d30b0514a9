"""The plain implementation itself: against the reference project's own numpy
forward (outputs committed under tests/golden/), and its parts against each other."""
import json
import os

import numpy as np

from plain import llama_plain as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_numpy_forward.npz")


def load_golden():
    z = np.load(GOLDEN)
    cfg = json.loads(bytes(z["config_json"]).decode())
    w = {k[2:]: z[k] for k in z.files if k.startswith("w/")}
    return z, cfg, w


def test_plain_matches_reference_numpy_forward():
    z, cfg, w = load_golden()
    n_layers = cfg["num_hidden_layers"]
    for i in range(2):
        ids = z[f"p{i}/ids"].tolist()
        logits, hidden = plain.forward(w, cfg, ids, return_hidden=True)
        # the reference computes in float32: 1e-6 is its rounding, not ours
        assert np.abs(logits[-1] - z[f"p{i}/last_logits"]).max() < 1e-6
        assert np.abs(logits[-1] - z[f"p{i}/last_logits_two_portions"]).max() < 1e-6
        # reference list: embedding, output of layers 0..L-2, final norm (HF layout)
        for j in range(n_layers):
            assert np.abs(hidden[j] - z[f"p{i}/hidden_{j}"]).max() < 1e-6, j
        assert np.abs(hidden[n_layers + 1] - z[f"p{i}/hidden_{n_layers}"]).max() < 1e-6


def test_prefix_property():
    """Logits at position t depend on tokens 0..t only."""
    _, cfg, w = load_golden()
    ids = [3, 9, 27, 33, 1, 0, 47, 12, 12, 5]
    full = plain.forward(w, cfg, ids)
    for t in (1, 4, 9):
        part = plain.forward(w, cfg, ids[:t + 1])
        assert np.abs(part[-1] - full[t]).max() < 1e-12


def test_window_equals_full_when_wide_and_differs_when_narrow():
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((12, 4 * 8)), rng.standard_normal((12, 2 * 8)), rng.standard_normal((12, 2 * 8)))
    full = plain.attention(q, k, v, 4, 2, 8)
    assert np.allclose(full, plain.attention(q, k, v, 4, 2, 8, window=12))
    narrow = plain.attention(q, k, v, 4, 2, 8, window=3)
    assert np.allclose(narrow[:3], full[:3]) and not np.allclose(narrow[5:], full[5:])
    # window 1: every token sees itself only
    assert np.allclose(plain.attention(q, k, v, 4, 2, 8, window=1).reshape(12, 4, 8),
                       np.repeat(v.reshape(12, 2, 8), 2, axis=1))


def test_rope_is_a_rotation_and_relative():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((6, 2 * 16))
    pos = np.array([0, 1, 5, 17, 100, 1000])
    y = plain.rope(x, pos, 2, 16, 10000.0)
    assert np.allclose(np.linalg.norm(x.reshape(6, 2, 16), axis=-1), np.linalg.norm(y.reshape(6, 2, 16), axis=-1))
    assert np.allclose(y[0], x[0])
    a = plain.rope(x[:1], [7], 2, 16, 5e5)[0, :16] @ plain.rope(x[1:2], [3], 2, 16, 5e5)[0, :16]
    b = plain.rope(x[:1], [107], 2, 16, 5e5)[0, :16] @ plain.rope(x[1:2], [103], 2, 16, 5e5)[0, :16]
    assert abs(a - b) < 1e-9


def test_argmax_first_and_round_bf16():
    assert plain.argmax_first(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    assert plain.argmax_first(np.array([-1.0, -1.0])) == 0
    import torch
    a = np.random.default_rng(2).standard_normal(1000).astype(np.float32) * 3
    assert np.array_equal(plain.round_bf16(a), torch.from_numpy(a).to(torch.bfloat16).float().numpy())


def test_greedy_stops_at_eos():
    _, cfg, w = load_golden()
    out = plain.greedy_generate(w, cfg, [1, 2, 3], 6)
    assert len(out) == 6
    out2 = plain.greedy_generate(w, cfg, [1, 2, 3], 6, eos={out[2]})
    assert out2 == out[:out.index(out[2]) + 1]
