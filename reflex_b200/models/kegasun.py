"""Kegasun as data: its typed config turned into a `ModelSpec`.

The design: the token embedding times a scale, plus a hashed bigram row (the
previous token is part of a sequence's state), plus a sinusoidal position
vector; pre-norm layers with layer norms (a weight, no bias), whose mixer is a
latent attention (low-rank query and key/value latents, only the key/value
latent cached, a sliding window, a sink in the softmax's denominator, a
per-head output gate) or an mLSTM (matrix memory, exponential gates kept
stable by a running maximum), and whose feed-forward is a gated dense one
(SiLU), a mixture of experts (squared ReLU, top-k routing, weights from the
softmax over the chosen logits) or absent; the model's layer norm, then an
untied head.  Tensor names are the checkpoint's; the right columns of
`*_NAMES` are the only place they occur.
"""

from __future__ import annotations

from ..config.kegasun import KegasunConfig
from ..config.registry import register_architecture
from ..config.spec import (
    EmbeddingTermSpec,
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
)

LATENT_NAMES = (
    ("q_down", "mix.dq"), ("q_norm", "mix.dq.norm"), ("q_up", "mix.uq"),
    ("kv_down", "mix.dkv"), ("kv_norm", "mix.dkv.norm"), ("k_up", "mix.uk"), ("v_up", "mix.uv"),
    ("sink", "mix.sink"), ("gate", "mix.g"), ("o_proj", "mix.o"),
)
MLSTM_NAMES = (
    ("q_proj", "mix.q"), ("k_proj", "mix.k"), ("v_proj", "mix.v"), ("gate", "mix.g"),
    ("o_proj", "mix.o"), ("norm", "mix.norm"), ("i_proj", "mix.i"), ("i_bias", "mix.i.b"),
    ("f_proj", "mix.f"), ("f_bias", "mix.f.b"),
)
DENSE_NAMES = (("gate_proj", "mlp.gate"), ("up_proj", "mlp.up"), ("down_proj", "mlp.down"))
MOE_NAMES = (("router", "mlp.router"), ("router_bias", "mlp.router.b"),
             ("expert_up", "mlp.e{expert}.up"), ("expert_down", "mlp.e{expert}.down"))
BLOCK_NAMES = (("mixer_norm", "norm1"), ("feed_forward_norm", "norm2"))

SINUSOID_BASE = 10000.0  # fixed by the design


def build_kegasun_spec(cfg: KegasunConfig) -> ModelSpec:
    eps, W = cfg.norm_eps, cfg.width
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type == "latent_attention":
            mixer = MixerSpec(
                "latent_attention", hidden_size=W, num_heads=m["heads"], num_kv_heads=1,
                head_dim=m["dim"], v_head_dim=m["vdim"], scale=float(m["scale"]),
                window=int(m["mask"]["size"]), names=LATENT_NAMES,
                params=(("q_rank", int(m["q_rank"])), ("kv_rank", int(m["kv_rank"])), ("eps", eps),
                        ("sink", True), ("gate", "head")))
        else:
            mixer = MixerSpec(
                "mlstm", hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                scale=float(m["dim"]) ** -0.5, names=MLSTM_NAMES,
                params=(("gate_cap", float(m["gate_cap"])), ("eps", eps)))
        ffn = None
        if l.mlp is not None and l.mlp["kind"] == "dense":
            ffn = FeedForwardSpec("swiglu", hidden_size=W, intermediate_size=int(l.mlp["ff"]),
                                  names=DENSE_NAMES)
        elif l.mlp is not None:
            ffn = FeedForwardSpec(
                "moe", hidden_size=W, intermediate_size=int(l.mlp["expert"]["ff"]), names=MOE_NAMES,
                params=(("experts", int(l.mlp["router"]["experts"])), ("top", int(l.mlp["router"]["top"])),
                        ("activation", "relu2"), ("router_bias", True)))
        layers.append(LayerSpec(
            block="prenorm", prefix=f"l{i}.", mixer=mixer, feed_forward=ffn,
            mixer_norm=NormSpec("layernorm", W, eps),
            feed_forward_norm=NormSpec("layernorm", W, eps) if ffn is not None else None,
            names=BLOCK_NAMES))
    terms = []
    if cfg.bigram is not None:
        terms.append(EmbeddingTermSpec(
            "bigram_hash", W, names=(("table", "bigram"),),
            params=(("buckets", cfg.bigram["buckets"]), ("mul_prev", cfg.bigram["mul_prev"]),
                    ("mul_cur", cfg.bigram["mul_cur"]), ("vocab", cfg.vocab))))
    terms.append(EmbeddingTermSpec("sinusoidal", W, params=(("base", SINUSOID_BASE),)))
    return ModelSpec(
        architecture="kegasun", vocab_size=cfg.vocab, hidden_size=W, layers=layers,
        final_norm=NormSpec("layernorm", W, eps), tie_word_embeddings=False,
        max_positions=cfg.max_positions, embedding_name="embed", final_norm_name="final.norm",
        head_name="head", embedding_scale=cfg.embedding_scale, embedding_terms=tuple(terms))


KEGASUN = register_architecture(("Kegasun", "kegasun"), KegasunConfig.from_dict, build_kegasun_spec)
