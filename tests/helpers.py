"""Shared by the tests: the two tiny configurations, model folders made in a
temporary place, and the comparison of engine logits with the plain implementation."""
from __future__ import annotations

import json
import os

import numpy as np

from plain import llama_plain as plain

# Two configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 172, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 128, "tie_word_embeddings": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True,
    "eos_token_id": 511,
}
TINY = {"A": (TINY_A, 0, 0.0), "B": (TINY_B, 2, 0.1)}   # config, seed, spread of the gains


QK_BOOST = {"float32": 3.0, "bfloat16": 2.0}


def make_weights(name: str, dtype: str = "float32", qk_boost: float = 0.0):
    """Random weights of a tiny configuration.  The q and k projections are scaled
    up so that attention is far from uniform and a wrong position, key or page
    changes the logits by much more than rounding does.  How far: sharp attention
    also amplifies the honest rounding of bfloat16 activations (measured on the
    3-layer configuration: up to 2.1e-2 of the logit range at a factor of 3, under
    1e-2 at 2), so models for bfloat16 runs are a little less sharp than those for
    float32 runs; the tolerance is the same for both factors."""
    qk_boost = qk_boost or QK_BOOST[dtype]
    cfg, seed, gain_std = TINY[name]
    w = plain.random_weights(cfg, seed, gain_std=gain_std, std=0.05)
    for k in list(w):
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = (w[k] * qk_boost).astype(np.float32)
    return cfg, w


def write_model_dir(path: str, cfg: dict, weights: dict, bf16: bool = False) -> str:
    """A model folder from numpy weights, written with the safetensors library
    (not with the product's writer)."""
    import torch
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = {}
    for k, v in weights.items():
        t = torch.from_numpy(np.ascontiguousarray(v))
        if bf16 and v.ndim == 2:
            t = t.to(torch.bfloat16)
        tensors[k] = t
    save_file(tensors, os.path.join(path, "model.safetensors"))
    return path


def rounded_weights(weights: dict) -> dict:
    """What a bfloat16 engine holds: matrices rounded to bfloat16, gains in float32."""
    return {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in weights.items()}


def prompts_for(cfg: dict, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


# Largest |engine - plain| allowed, as a fraction of the largest |logit| of the
# sequence.  float32: float32 sums against float64 ones; measured 1e-6 to 3e-6 on
# these models.  bfloat16: the plain implementation runs with the same rounded
# weights and rounds to bfloat16 wherever the engine stores a bfloat16 tensor
# (``plain_logits``), so what is left is the order of float32 sums and roundings
# that flip at a tie; measured 4e-3 to 7.6e-3 on the tiny models and 9.8e-3 on two
# layers of TinyLlama-1.1B's sizes (700 tokens, test_gpu_bench_sizes.py).
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def plain_logits(weights: dict, cfg: dict, ids, dtype: str) -> np.ndarray:
    """The yardstick for an engine of the given dtype, at every position of ``ids``."""
    if dtype == "float32":
        return plain.forward(weights, cfg, ids)
    return plain.forward(rounded_weights(weights), cfg, ids, rnd=plain.round_act_bf16)


WORST = {}      # dtype -> (largest error / tolerance seen in this run, where)

# Largest difference between two runs of the same (request, position) that were cut or
# batched differently, as a fraction of the sequence's largest |logit|.  float32: sums
# of the same numbers in another order (about 2^-24 per rounding; measured up to 2.1e-6
# = 35 ulp of the largest logit over two or three layers).  bfloat16: a sum that rounds
# the other way flips a stored activation by one bfloat16 step (2^-8), which then runs
# through the rest of the model; measured up to 7.0e-3.
CROSS_TOL = {"float32": 4e-6, "bfloat16": 1e-2}
CROSS = {}      # dtype -> (largest such difference seen in this run, where)


def note_cross(dtype: str, diff: float, what: str) -> None:
    if diff > CROSS.get(dtype, (0.0, ""))[0]:
        CROSS[dtype] = (diff, what)


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str = ""):
    scale = max(1e-6, float(np.abs(want).max()))
    err = float(np.abs(got.astype(np.float64) - want).max())
    ratio = err / (TOL[dtype] * scale)
    if ratio > WORST.get(dtype, (0.0, ""))[0]:
        WORST[dtype] = (ratio, what)
    assert err <= TOL[dtype] * scale, (
        f"{what}: max |diff| {err:.3e} exceeds {TOL[dtype]:.0e} * {scale:.3e} "
        f"(first bad row {int(np.argmax(np.abs(got - want).max(axis=-1)))})")
