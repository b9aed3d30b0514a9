"""The Llama architecture (``LlamaForCausalLM``) as a ``ModelSpec``.

Dense decoder as the reference runs it with arch 0 and no experts
(backend/model.cu:1067-1124, 1181-1188): pre-norm RMSNorm, grouped-query attention
with rotate-half rotary embedding and no bias, SwiGLU feed-forward, final RMSNorm,
head tied to the embedding or not.  Tensor names are the checkpoint's own
(backend/model.cu:873-892).  This file holds no sizes and no kernels: it only
translates ``LlamaConfig`` into part descriptions.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.llama import LlamaConfig
from ..parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    d = cfg.hidden_size
    norm = {"width": d, "eps": cfg.rms_norm_eps}
    rotary = PartSpec("rotary", "", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        blocks.append(BlockSpec(
            kind="pre_norm", prefix=p,
            mixer=PartSpec("paged_attention", p + ".self_attn", {
                "hidden": d, "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                "window": None, "position": rotary}),
            feed_forward=PartSpec("gated_mlp", p + ".mlp", {
                "hidden": d, "intermediate": cfg.intermediate_size, "activation": "silu"}),
            mixer_norm=PartSpec("rmsnorm", p + ".input_layernorm", dict(norm)),
            ff_norm=PartSpec("rmsnorm", p + ".post_attention_layernorm", dict(norm))))
    return ModelSpec(
        hidden_size=d, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", "model.embed_tokens", {"vocab": cfg.vocab_size, "width": d}),
        blocks=blocks,
        schedule=[LayerCall(block=i, cache=i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", "model.norm", dict(norm)),
        head=PartSpec("linear_head", "lm_head", {
            "vocab": cfg.vocab_size, "width": d,
            "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec)
