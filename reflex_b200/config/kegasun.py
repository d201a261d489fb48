"""Typed configuration of the Kegasun design, read from config.json.

config.json keys: `architecture` ("Kegasun"), `vocab`, `width`, `norm.eps`,
`embedding` (`scale`; optional `bigram` with `buckets`, `mul_prev`,
`mul_cur`), and `layers`, a list whose entries give `type` (the mixer:
"latent_attention" or "mlstm"), `mixer` (its sizes) and `mlp` (the
feed-forward: `kind` "dense" with `ff`, or "moe" with `expert.ff`,
`router.experts`, `router.top`; null for a layer without one).  Every size and
every constant that differs between models comes from here; what the design
fixes (the sinusoid's base, the mLSTM's denominator guard) lives in the parts.
Missing or ill-typed keys are reported together, by name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import CheckpointError

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale", "mask"),
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
}


@dataclass
class KegasunLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class KegasunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: Optional[Dict[str, int]]
    layers: List[KegasunLayer] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    # the design fixes no longest context; the cache bounds it
    max_positions: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "KegasunConfig":
        problems: List[str] = []

        def need(d, key, types, where):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None or isinstance(v, bool) or not isinstance(v, types):
                problems.append(f"{where}{key}")
                return None
            return v

        vocab = need(cfg, "vocab", int, "")
        width = need(cfg, "width", int, "")
        norm = cfg.get("norm") if isinstance(cfg.get("norm"), dict) else {}
        eps = need(norm, "eps", (int, float), "norm.")
        emb = cfg.get("embedding") if isinstance(cfg.get("embedding"), dict) else {}
        scale = need(emb, "scale", (int, float), "embedding.")
        bigram = emb.get("bigram")
        if bigram is not None:
            for k in ("buckets", "mul_prev", "mul_cur"):
                need(bigram, k, int, "embedding.bigram.")
        layers_in = cfg.get("layers")
        layers: List[KegasunLayer] = []
        if not isinstance(layers_in, list) or not layers_in:
            problems.append("layers")
            layers_in = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]."
            kind = need(l, "type", str, where)
            mixer = l.get("mixer") if isinstance(l, dict) and isinstance(l.get("mixer"), dict) else None
            if mixer is None:
                problems.append(where + "mixer")
                continue
            if kind not in MIXER_KEYS:
                if kind is not None:
                    problems.append(f"{where}type={kind!r} (known: {sorted(MIXER_KEYS)})")
                continue
            for k in MIXER_KEYS[kind]:
                if k == "mask":
                    need(mixer.get("mask"), "size", int, where + "mixer.mask.")
                else:
                    need(mixer, k, (int, float) if k in ("scale", "gate_cap") else int, where + "mixer.")
            mlp = l.get("mlp")
            if mlp is not None:
                mk = need(mlp, "kind", str, where + "mlp.")
                if mk == "dense":
                    need(mlp, "ff", int, where + "mlp.")
                elif mk == "moe":
                    need(mlp.get("expert"), "ff", int, where + "mlp.expert.")
                    need(mlp.get("router"), "experts", int, where + "mlp.router.")
                    need(mlp.get("router"), "top", int, where + "mlp.router.")
                elif mk is not None:
                    problems.append(f"{where}mlp.kind={mk!r} (known: dense, moe)")
            layers.append(KegasunLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        if problems:
            raise CheckpointError("config.json: missing or ill-typed keys: " + ", ".join(problems))
        out = cls(vocab=vocab, width=width, norm_eps=float(eps), embedding_scale=float(scale),
                  bigram=None if bigram is None else {k: int(bigram[k]) for k in ("buckets", "mul_prev", "mul_cur")},
                  layers=layers, torch_dtype=str(cfg.get("torch_dtype", "bfloat16")),
                  max_positions=int(cfg.get("max_positions", 1 << 20)), raw=dict(cfg))
        out.validate()
        return out

    def validate(self) -> None:
        def bad(msg: str) -> None:
            raise CheckpointError(f"config.json: {msg}")

        if self.vocab <= 0 or self.width <= 0:
            bad("vocab and width must be positive")
        if not (self.norm_eps > 0):
            bad("norm.eps must be positive")
        if self.bigram is not None and self.bigram["buckets"] <= 0:
            bad("embedding.bigram.buckets must be positive")
        for i, l in enumerate(self.layers):
            m = l.mixer
            for k in ("heads", "dim", "vdim"):
                if m[k] <= 0:
                    bad(f"layers[{i}].mixer.{k} must be positive")
            if l.type == "latent_attention":
                if m["q_rank"] <= 0 or m["kv_rank"] <= 0 or m["mask"]["size"] <= 0:
                    bad(f"layers[{i}].mixer: q_rank, kv_rank and mask.size must be positive")
            if l.type == "mlstm" and not (m["gate_cap"] > 0):
                bad(f"layers[{i}].mixer.gate_cap must be positive")
            if l.mlp is not None and l.mlp["kind"] == "moe":
                r = l.mlp["router"]
                if not (0 < r["top"] <= r["experts"]):
                    bad(f"layers[{i}].mlp.router: top must be between 1 and experts")

    def to_dict(self) -> Dict[str, Any]:
        out = dict(self.raw)
        out.update({
            "architecture": "Kegasun", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "embedding": dict({"scale": self.embedding_scale},
                              **({"bigram": dict(self.bigram)} if self.bigram else {})),
            "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers],
        })
        return out
