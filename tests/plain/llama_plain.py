"""Plain, slow Llama forward pass in numpy float64: the yardstick of the tests.

Whole sequences, no cache, no paging, one function for each part.  Nothing in
this file is imported by the product package and nothing of the product package
is imported here.  Every function restates a formula of the reference project
(Kartikeya-trivedi/KLLM) and cites it as ``path:line`` inside that project.

Weights arrive as a ``dict`` of tensor name -> numpy array (any float dtype);
they are widened to float64 before use, so the only rounding left is float64's.
The comparison of this file with the reference's own numpy forward
(``tools/gen_reference_numpy_moe.py``) is recorded under ``tests/golden/``.
"""
from __future__ import annotations

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def embed(table, ids):
    """x[t, :] = E[ids[t], :], no scaling for Llama (backend/model.cu:89-95, 1056-1058)."""
    return f64(table)[np.asarray(ids, dtype=np.int64)]


def rmsnorm(x, gain, eps):
    """out = x * rsqrt(mean(x^2) + eps) * w, the gain used as it is stored
    (backend/model.cu:101-122; tools/gen_reference_numpy_moe.py:28-30)."""
    x = f64(x)
    scale = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x * scale * f64(gain)


def rope(x, positions, n_heads, head_dim, theta):
    """rotate_half rotary embedding: pair (j, j + hd/2) turns by p * theta^(-2j/hd)
    (backend/model.cu:170-184; tools/gen_reference_numpy_moe.py:33-45)."""
    x = f64(x)
    t = x.shape[0]
    half = head_dim // 2
    j = np.arange(half, dtype=np.float64)
    freq = float(theta) ** (-2.0 * j / head_dim)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    cos = np.cos(ang)[:, None, :]
    sin = np.sin(ang)[:, None, :]
    xh = x.reshape(t, n_heads, head_dim)
    a, b = xh[:, :, :half], xh[:, :, half:]
    out = np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)
    return out.reshape(t, n_heads * head_dim)


def attention(q, k, v, n_heads, n_kv_heads, head_dim, window=None, scale=None, rnd_p=None):
    """Causal grouped-query attention of a whole sequence.

    Per (token t, head h): kv head g = h // (H/G); keys 0..t (or the last
    ``window`` of them); score = (q . k) * 1/sqrt(hd); max-subtracted softmax;
    weighted sum of values (backend/model.cu:343-408, scale at :1063-1064, window
    start at :361-362; tools/gen_reference_numpy_moe.py:103-118).  ``rnd_p`` rounds
    the unnormalised probabilities exp(s - max) before they meet the values, as an
    engine does that feeds them to a reduced-precision matrix unit; the sum that
    divides is taken of the unrounded ones.
    """
    q, k, v = f64(q), f64(k), f64(v)
    t = q.shape[0]
    if scale is None:
        scale = 1.0 / np.sqrt(float(head_dim))
    group = n_heads // n_kv_heads
    out = np.zeros((t, n_heads * head_dim), dtype=np.float64)
    pos = np.arange(t)
    mask = pos[:, None] >= pos[None, :]
    if window is not None and window > 0:
        mask &= pos[None, :] > (pos[:, None] - window)
    for h in range(n_heads):
        g = h // group
        qh = q[:, h * head_dim:(h + 1) * head_dim]
        kh = k[:, g * head_dim:(g + 1) * head_dim]
        vh = v[:, g * head_dim:(g + 1) * head_dim]
        sc = (qh @ kh.T) * scale
        sc = np.where(mask, sc, -np.inf)
        sc = sc - sc.max(axis=1, keepdims=True)
        p = np.exp(sc)
        total = p.sum(axis=1, keepdims=True)
        if rnd_p is not None:
            p = rnd_p(p)
        out[:, h * head_dim:(h + 1) * head_dim] = (p @ vh) / total
    return out


def silu(x):
    """x / (1 + exp(-x)) (backend/model.cu:477-483; tools/gen_reference_numpy_moe.py:48-49)."""
    return x / (1.0 + np.exp(-x))


def swiglu(x, w_gate, w_up, w_down, rnd=None):
    """down( silu(x Wg^T) * (x Wu^T) ) (backend/model.cu:1112-1115)."""
    rnd = rnd or (lambda a: a)
    x = f64(x)
    g = x @ f64(w_gate).T              # gate, up and the result are float32 in the
    u = x @ f64(w_up).T                # engine; only the activation's output is stored
    return rnd(silu(g) * u) @ f64(w_down).T


def _same(a):
    return a


def attention_block(x, w, prefix, cfg, positions, rnd=_same):
    """q, k, v projections without bias, rotary on q and k, attention, output
    projection (backend/model.cu:1090-1104).  ``rnd`` rounds what a reduced-precision
    engine stores between its kernels (identity for the exact yardstick)."""
    hd, nh, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    q = rnd(x @ f64(w[prefix + ".self_attn.q_proj.weight"]).T)
    k = rnd(x @ f64(w[prefix + ".self_attn.k_proj.weight"]).T)
    v = rnd(x @ f64(w[prefix + ".self_attn.v_proj.weight"]).T)
    q = rnd(rope(q, positions, nh, hd, cfg["rope_theta"]))
    k = rnd(rope(k, positions, nkv, hd, cfg["rope_theta"]))
    a = rnd(attention(q, k, v, nh, nkv, hd, window=cfg.get("sliding_window"),
                      rnd_p=None if rnd is _same else rnd))
    return a @ f64(w[prefix + ".self_attn.o_proj.weight"]).T     # float32 into the residual stream


def decoder_layer(x, w, layer, cfg, positions, rnd=_same):
    """Pre-norm block: x += attn(norm(x)); x += mlp(norm(x)).  The reference adds
    the feed-forward's output inside the next norm kernel, which is the same sum
    (backend/model.cu:1067-1118)."""
    prefix = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    xn = rnd(rmsnorm(x, w[prefix + ".input_layernorm.weight"], eps))
    x = x + attention_block(xn, w, prefix, cfg, positions, rnd)
    xn = rnd(rmsnorm(x, w[prefix + ".post_attention_layernorm.weight"], eps))
    x = x + swiglu(xn, w[prefix + ".mlp.gate_proj.weight"], w[prefix + ".mlp.up_proj.weight"],
                   w[prefix + ".mlp.down_proj.weight"], rnd)
    return x


def normalise_config(cfg):
    """Defaults as the reference applies them (models/config.go:107-119)."""
    c = dict(cfg)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-6)
    if not c.get("num_key_value_heads"):
        c["num_key_value_heads"] = c["num_attention_heads"]
    if not c.get("head_dim"):
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    return c


def forward(w, cfg, ids, return_hidden=False, rnd=_same):
    """Logits [T, V] in float64 at every position of one whole sequence
    (backend/model.cu:1056-1188; the reference keeps only the last row, :1184-1188).
    With ``rnd=round_act_bf16`` every tensor that a bfloat16 engine stores between
    two kernels is rounded to bfloat16 (the residual stream and the logits are not).

    ``lm_head.weight`` falls back to the embedding table when the configuration
    ties them (the reference resolves tying offline, tools/convert_hf.py:81-82).
    """
    cfg = normalise_config(cfg)
    positions = np.arange(len(ids))
    x = embed(w["model.embed_tokens.weight"], ids)
    hidden = [x.copy()]
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, positions, rnd)
        hidden.append(x.copy())
    xn = rnd(rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    hidden.append(xn.copy())
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    logits = xn @ f64(head).T
    if return_hidden:
        return logits, hidden
    return logits


def argmax_first(row):
    """First index of the maximum, strict '>' (engine/engine.go:216-224)."""
    best, best_val = 0, row[0]
    for i in range(1, len(row)):
        if row[i] > best_val:
            best, best_val = i, row[i]
    return best


def greedy_generate(w, cfg, prompt, steps, eos=None):
    """Greedy loop by whole-sequence recomputation; the EOS token is emitted and
    ends the loop (engine/engine.go:192-213)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        nxt = argmax_first(forward(w, cfg, ids)[-1])
        out.append(nxt)
        ids.append(nxt)
        if eos is not None and nxt in eos:
            break
    return out


def temperature_probs(row, temperature):
    """softmax(z / tau) (docs/theory/02-autoregressive-decoding.md:122-124)."""
    z = f64(row) / float(temperature)
    z = z - z.max()
    p = np.exp(z)
    return p / p.sum()


# ---- tensor helpers for tests ------------------------------------------------

def round_bf16(a):
    """Round float32 values to the nearest bfloat16 (ties to even), return float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bias = ((bits >> 16) & 1) + 0x7FFF
    out = (((bits + bias) >> 16) << 16).astype(np.uint32)
    return out.view(np.float32).reshape(a.shape)


def round_act_bf16(a):
    """float64 activations as a bfloat16 tensor would hold them."""
    return round_bf16(np.asarray(a, dtype=np.float32)).astype(np.float64)


def random_weights(cfg, seed, gain_std=0.0, std=0.02):
    """A weight dict for a Llama configuration: matrices N(0, std), gains
    N(1, gain_std).  Independent of the product's random-weights mode."""
    cfg = normalise_config(cfg)
    rng = np.random.default_rng(seed)
    d, f, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd, nh, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]

    def mat(r, c):
        return (rng.standard_normal((r, c)) * std).astype(np.float32)

    def gain():
        return (1.0 + gain_std * rng.standard_normal(d)).astype(np.float32)

    w = {"model.embed_tokens.weight": mat(v, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[p + ".self_attn.q_proj.weight"] = mat(nh * hd, d)
        w[p + ".self_attn.k_proj.weight"] = mat(nkv * hd, d)
        w[p + ".self_attn.v_proj.weight"] = mat(nkv * hd, d)
        w[p + ".self_attn.o_proj.weight"] = mat(d, nh * hd)
        w[p + ".mlp.gate_proj.weight"] = mat(f, d)
        w[p + ".mlp.up_proj.weight"] = mat(f, d)
        w[p + ".mlp.down_proj.weight"] = mat(d, f)
        w[p + ".input_layernorm.weight"] = gain()
        w[p + ".post_attention_layernorm.weight"] = gain()
    w["model.norm.weight"] = gain()
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(v, d)
    return w
