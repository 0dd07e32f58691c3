"""Dense Qwen3 put together from the parts, and its registration.

Per layer (src/model/arch/qwen3.hpp:272-312): pre-norm residual block of
grouped-query attention with per-head q/k RMSNorm before rotation, and a SwiGLU
feed-forward; a final RMSNorm and a head that is the embedding when
`tie_word_embeddings` (a stored lm_head is then ignored, as the reference drops
it: src/model/arch/hf_config.hpp:300-335).  Tensor names are Hugging Face's
(src/model/arch/qwen3.hpp:140-153).
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts import (Attention, GatedMLP, LogitsHead, PreNormBlock, RMSNorm, RotaryEmbedding, TokenEmbedding)
from ..registry import register_architecture
from .model import Model


def build_qwen3(cfg: Qwen3Config) -> Model:
    rope = RotaryEmbedding(cfg.head_dim, cfg.rope_theta, yarn=cfg.rope_scaling)
    blocks = []
    for _ in range(cfg.num_hidden_layers):
        attention = Attention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                              position_encoding=rope, qk_norm_eps=cfg.rms_norm_eps, window=None)
        blocks.append(PreNormBlock(RMSNorm(cfg.hidden_size, cfg.rms_norm_eps), attention,
                                   RMSNorm(cfg.hidden_size, cfg.rms_norm_eps),
                                   GatedMLP(cfg.hidden_size, cfg.intermediate_size, "silu")))
    embedding = TokenEmbedding(cfg.vocab_size, cfg.hidden_size)
    head = LogitsHead(RMSNorm(cfg.hidden_size, cfg.rms_norm_eps), cfg.vocab_size, cfg.hidden_size,
                      tied_to=embedding if cfg.tie_word_embeddings else None)
    return Model(embedding=embedding, blocks=blocks, head=head, vocab_size=cfg.vocab_size,
                 max_positions=cfg.max_position_embeddings,
                 ignorable=("lm_head.weight",) if cfg.tie_word_embeddings else (),
                 eos_ids=cfg.eos_ids)


register_architecture(("Qwen3ForCausalLM", "qwen3"), Qwen3Config, build_qwen3)
