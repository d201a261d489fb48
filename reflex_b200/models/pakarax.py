"""Pakarax as data: its typed config turned into a `ModelSpec`.

The design: a token embedding; layers in which one RMS norm feeds the mixer
and the feed-forward side by side (x += mixer(n) + ff(n)).  The mixer is two
mixers side by side on the same input, their outputs each RMS-normed with a
weight of its own and averaged: an attention with biases, a short causal
convolution on q, k and v, a query temperature that grows with the logarithm
of the position, a per-head linear distance penalty on the scores and a sink
in the softmax's denominator; and a gated linear recurrence (a gelu branch, a
convolved branch, block-diagonal gates, decay exp(-8 r softplus(lam))).  The
feed-forward is the clamped gated form, dense or as a mixture of experts with
sigmoid scores that weight the experts' inputs and a gated shared expert.  A
stretch of layers may run several times with the same weights; each pass has
its own cache entries and starts from a mix of the stream with the embedding
output.  The model's RMS norm, the head, a scale and a tanh cap on the logits.
Tensor names are the checkpoint's; the right columns of `*_NAMES` are the only
place they occur.
"""

from __future__ import annotations

from ..config.pakarax import PakaraxConfig
from ..config.registry import register_architecture
from ..config.spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, RunEntry

LEFT_NAMES = (
    ("q_proj", "q"), ("q_bias", "q.b"), ("k_proj", "k"), ("k_bias", "k.b"), ("v_proj", "v"), ("v_bias", "v.b"),
    ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"), ("sink", "sink"),
    ("o_proj", "o"), ("o_bias", "o.b"),
)
RIGHT_NAMES = (
    ("y_proj", "y"), ("y_bias", "y.b"), ("x_proj", "x"), ("x_bias", "x.b"), ("conv", "conv"),
    ("conv_bias", "conv.b"), ("gate_a", "ra"), ("gate_a_bias", "ra.b"), ("gate_i", "ri"),
    ("gate_i_bias", "ri.b"), ("lam", "lam"), ("o_proj", "o"),
)
PAIR_NAMES = (tuple((f"left/{r}", f"mix.left.{n}") for r, n in LEFT_NAMES)
              + tuple((f"right/{r}", f"mix.right.{n}") for r, n in RIGHT_NAMES)
              + (("left_out", "mix.left.out"), ("right_out", "mix.right.out")))
DENSE_NAMES = (("gate_proj", "mlp.gate"), ("up_proj", "mlp.up"), ("down_proj", "mlp.down"))
MOE_NAMES = (("router", "mlp.router"), ("expert_gate", "mlp.e{expert}.gate"), ("expert_up", "mlp.e{expert}.up"),
             ("expert_down", "mlp.e{expert}.down"), ("shared_gate", "mlp.shared.gate"),
             ("shared_up", "mlp.shared.up"), ("shared_down", "mlp.shared.down"), ("shared_sg", "mlp.shared.sg"))
BLOCK_NAMES = (("mixer_norm", "norm1"),)

# fixed by the design
GLU_ALPHA = 1.702            # g * sigmoid(1.702 g) in every feed-forward
DECAY_SCALE = 8.0            # log a = -8 r softplus(lam)
SLOPE_EXPONENT = 8.0         # distance slope of head h: 2^(-8 (h + 1) / heads)


def build_pakarax_spec(cfg: PakaraxConfig) -> ModelSpec:
    eps, W = cfg.norm_eps, cfg.width
    layers = []
    for i, l in enumerate(cfg.layers):
        a, r = l.mixer["left"], l.mixer["right"]
        temp = a.get("q_temp") or {}
        left = MixerSpec(
            "conv_attention", hidden_size=W, num_heads=int(a["heads"]), num_kv_heads=int(a["kv_heads"]),
            head_dim=int(a["dim"]), v_head_dim=int(a["vdim"]), scale=float(a["scale"]), window=None,
            params=(("taps", int(a["conv"])), ("bias", True), ("sink", True),
                    ("temp_coef", float(temp.get("coef", 0.0))), ("temp_every", int(temp.get("every", 1))),
                    ("distance_slope_exponent", SLOPE_EXPONENT)))
        right = MixerSpec(
            "rglru", hidden_size=W,
            params=(("width", int(r["width"])), ("blocks", int(r["blocks"])), ("taps", int(r["conv"])),
                    ("decay_scale", DECAY_SCALE)))
        mixer = MixerSpec("pair", hidden_size=W, names=PAIR_NAMES,
                          params=(("left", left), ("right", right), ("eps", eps)))
        ffn = None
        if l.mlp is not None and l.mlp["kind"] == "dense":
            ffn = FeedForwardSpec("glu_clamped", hidden_size=W, intermediate_size=int(l.mlp["ff"]),
                                  names=DENSE_NAMES,
                                  params=(("alpha", GLU_ALPHA), ("limit", float(l.mlp["limit"]))))
        elif l.mlp is not None:
            shared = l.mlp.get("shared")
            ffn = FeedForwardSpec(
                "moe", hidden_size=W, intermediate_size=int(l.mlp["expert"]["ff"]), names=MOE_NAMES,
                params=(("experts", int(l.mlp["router"]["experts"])), ("top", int(l.mlp["router"]["top"])),
                        ("activation", "glu_clamped"), ("alpha", GLU_ALPHA),
                        ("limit", float(l.mlp["expert"]["limit"])), ("scores", "sigmoid"),
                        ("weight_input", True), ("router_bias", False),
                        ("shared_ff", int(shared["ff"]) if shared else 0),
                        ("shared_limit", float(shared["limit"]) if shared else 0.0)))
        layers.append(LayerSpec(
            block="parallel", prefix=f"l{i}.", mixer=mixer, feed_forward=ffn,
            mixer_norm=NormSpec("rmsnorm", W, eps), feed_forward_norm=None, names=BLOCK_NAMES))
    # the order of the runs: a looped stretch names its layers once per pass, every
    # run with a cache entry of its own, every pass starting from the stream mix
    n = len(layers)
    order = []
    if cfg.loop is None:
        runs = [(i, False) for i in range(n)]
    else:
        start, stop, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
        runs = [(i, False) for i in range(start)]
        for _ in range(times):
            runs += [(i, i == start) for i in range(start, stop)]
        runs += [(i, False) for i in range(stop, n)]
    for entry, (layer, first) in enumerate(runs):
        order.append(RunEntry(layer, entry, True, mixes_input=first))
    return ModelSpec(
        architecture="pakarax", vocab_size=cfg.vocab, hidden_size=W, layers=layers,
        final_norm=NormSpec("rmsnorm", W, eps), tie_word_embeddings=False,
        max_positions=cfg.max_positions, embedding_name="embed", final_norm_name="final.norm",
        head_name="head", run_order=order, logit_scale=cfg.logit_scale, logit_softcap=cfg.logit_softcap,
        stream_mix_name="loop.in" if cfg.loop is not None else None)


PAKARAX = register_architecture(("Pakarax", "pakarax"), PakaraxConfig.from_dict, build_pakarax_spec)
