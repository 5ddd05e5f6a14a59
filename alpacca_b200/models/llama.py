"""The Llama-style dense decoder, put together from the parts.

Pre-norm blocks of grouped-query attention with rotary positions and a SwiGLU
feed-forward, a final RMSNorm and a tied or untied head: the graph of
alpacca/model.py:469-518.  Tensor names follow config.json-style checkpoints
(the reference reads the same tensors under GGUF names, alpacca/model.py:295-322):

    model.embed_tokens.weight                      token_embd.weight
    model.layers.N.input_layernorm.weight          blk.N.attn_norm.weight
    model.layers.N.self_attn.{q,k,v,o}_proj.weight blk.N.attn_{q,k,v,output}.weight
    model.layers.N.post_attention_layernorm.weight blk.N.ffn_norm.weight
    model.layers.N.mlp.{gate,up,down}_proj.weight  blk.N.ffn_{gate,up,down}.weight
    model.norm.weight                              output_norm.weight
    lm_head.weight (absent when tied)              output.weight
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..engine.model import DecoderSpec
from ..parts import (Attention, BuildOptions, PreNormBlock, RMSNorm, RotaryEncoding, SwiGLU, TokenEmbedding,
                     VocabHead)


@register_architecture("LlamaForCausalLM", LlamaConfig)
def build_llama(cfg: LlamaConfig, opts: BuildOptions) -> DecoderSpec:
    E, H, K, D = cfg.hidden_size, cfg.num_attention_heads, cfg.n_kv_heads, cfg.head_size
    rope = RotaryEncoding(opts, D, cfg.n_rot, cfg.rope_theta, cfg.rope_pairing, cfg.rope_scaling,
                          max_positions=min(opts.max_positions, cfg.max_position_embeddings))
    embedding = TokenEmbedding(opts, cfg.vocab_size, E, "model.embed_tokens")
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(PreNormBlock(
            RMSNorm(opts, E, cfg.rms_norm_eps, f"{p}.input_layernorm"),
            Attention(opts, E, H, K, D, rope, f"{p}.self_attn", qkv_bias=cfg.attention_bias,
                      out_bias=cfg.attention_bias),
            RMSNorm(opts, E, cfg.rms_norm_eps, f"{p}.post_attention_layernorm"),
            SwiGLU(opts, E, cfg.intermediate_size, f"{p}.mlp", bias=cfg.mlp_bias)))
    return DecoderSpec(
        embedding=embedding, layers=layers,
        final_norm=RMSNorm(opts, E, cfg.rms_norm_eps, "model.norm"),
        head=VocabHead(opts, cfg.vocab_size, E, "lm_head",
                       tied_to=embedding if cfg.tie_word_embeddings else None),
        stop_token_ids=cfg.stop_token_ids, vocab_size=cfg.vocab_size)
