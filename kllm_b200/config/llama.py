"""``LlamaConfig``: the keys of a Llama ``config.json`` as the engine reads them.

Keys and defaults follow the reference's ``HFConfig`` (models/config.go:15-49,
102-125): ``rope_theta`` 10000, ``rms_norm_eps`` 1e-6, no EOS; ``num_key_value_heads``
falls back to ``num_attention_heads`` and ``head_dim`` to ``hidden_size /
num_attention_heads``; the transformers-5 ``rope_parameters`` block is folded in and
a ``rope_type`` other than "default" is refused (:58-99).  Beyond the reference:
``tie_word_embeddings`` is read (the reference resolves tying offline,
tools/convert_hf.py:81-82), ``eos_token_id`` may be a list, a non-null
``rope_scaling`` is an error instead of being ignored, and biases are refused here
rather than in an offline converter (tools/convert_hf.py:94-100).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Tuple

from .base import ConfigError, ModelConfig, take_float, take_int


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...]
    model_type: str = "llama"

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        hidden = take_int(d, "hidden_size", minimum=1)
        layers = take_int(d, "num_hidden_layers", minimum=1)
        heads = take_int(d, "num_attention_heads", minimum=1)
        vocab = take_int(d, "vocab_size", minimum=1)
        inter = take_int(d, "intermediate_size", minimum=1)
        kv_heads = take_int(d, "num_key_value_heads", default=0, minimum=0) or heads
        head_dim = take_int(d, "head_dim", default=0, minimum=0)
        if head_dim == 0:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary embedding")
        max_pos = take_int(d, "max_position_embeddings", minimum=1)
        theta = take_float(d, "rope_theta", default=10000.0)
        theta = _fold_rope_parameters(d.get("rope_parameters"), theta)
        if d.get("rope_scaling") is not None:
            rs = d["rope_scaling"]
            kind = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {kind!r} is not supported (plain rotary only)")
        if theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        eps = take_float(d, "rms_norm_eps", default=1e-6)
        if eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported for Llama (silu only)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"config.json: {key}=true is not supported (projections carry no bias)")
        eos = d.get("eos_token_id", None)
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, list):
            eos_ids = tuple(int(e) for e in eos if int(e) >= 0)
        else:
            eos_ids = (int(eos),) if int(eos) >= 0 else ()
        return cls(
            architecture=d["architectures"][0], vocab_size=vocab, hidden_size=hidden,
            intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, max_position_embeddings=max_pos,
            rope_theta=theta, rms_norm_eps=eps,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids, model_type=str(d.get("model_type", "llama")))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        eos = d.pop("eos_token_ids")
        if len(eos) == 1:
            d["eos_token_id"] = eos[0]
        elif len(eos) > 1:
            d["eos_token_id"] = list(eos)
        d["hidden_act"] = "silu"
        return d


def _fold_rope_parameters(rp, theta: float) -> float:
    """``rope_parameters: {"rope_theta": ..., "rope_type": ...}`` (models/config.go:58-99)."""
    if rp is None:
        return theta
    if not isinstance(rp, dict):
        raise ConfigError(f"config.json: unrecognized rope_parameters shape: {rp!r}")
    if "full_attention" in rp or "sliding_attention" in rp:
        raise ConfigError("config.json: per-layer-type rope_parameters belong to another architecture")
    kind = rp.get("rope_type", "default")
    if kind not in ("", "default", None):
        raise ConfigError(f"config.json: rope_parameters rope_type {kind!r} not supported (no rope scaling)")
    t = rp.get("rope_theta")
    if t is None:
        return theta
    if isinstance(t, bool) or not isinstance(t, (int, float)) or t <= 0:
        raise ConfigError(f"config.json: unrecognized rope_parameters shape: {rp!r}")
    return float(t)
