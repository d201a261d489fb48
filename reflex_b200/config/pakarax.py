"""Typed configuration of the Pakarax design, read from config.json.

config.json keys: `architecture` ("Pakarax"), `vocab`, `width`, `norm.eps`,
optional `logit_scale` and `logit_softcap`, optional `loop` (`start`, `stop`,
`times`: layers start .. stop - 1 run `times` times in a row with the same
weights), and `layers`, a list whose entries give `type` (the mixer:
"parallel", an attention and a gated recurrence side by side), `mixer` (its
sizes: `left` with `heads`, `kv_heads`, `dim`, `vdim`, `conv`, `scale` and an
optional `q_temp` {`coef`, `every`}; `right` with `width`, `blocks`, `conv`)
and `mlp` (the feed-forward: `kind` "dense" with `ff` and `limit`, or "moe"
with `expert` {`ff`, `limit`}, `router` {`experts`, `top`} and an optional
`shared` {`ff`, `limit`}; null for a layer without one).  Every size and every
constant that differs between models comes from here; what the design fixes
lives in the architecture module.  Missing or ill-typed keys are reported
together, by name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..errors import CheckpointError

NUM = (int, float)


@dataclass
class PakaraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class PakaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    loop: Optional[Dict[str, int]] = None
    layers: List[PakaraxLayer] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    # the design fixes no longest context; the cache bounds it
    max_positions: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "PakaraxConfig":
        problems: List[str] = []

        def need(d, key, types, where):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None or isinstance(v, bool) or not isinstance(v, types):
                problems.append(f"{where}{key}")
                return None
            return v

        def optional(d, key, types, where, default):
            if not isinstance(d, dict) or d.get(key) is None:
                return default
            return need(d, key, types, where)

        vocab = need(cfg, "vocab", int, "")
        width = need(cfg, "width", int, "")
        norm = cfg.get("norm") if isinstance(cfg.get("norm"), dict) else {}
        eps = need(norm, "eps", NUM, "norm.")
        logit_scale = optional(cfg, "logit_scale", NUM, "", 1.0)
        logit_softcap = optional(cfg, "logit_softcap", NUM, "", 0.0)
        loop = cfg.get("loop")
        if loop is not None:
            for k in ("start", "stop", "times"):
                need(loop, k, int, "loop.")
        layers_in = cfg.get("layers")
        layers: List[PakaraxLayer] = []
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
            if kind != "parallel":
                if kind is not None:
                    problems.append(f"{where}type={kind!r} (known: parallel)")
                continue
            left, right = mixer.get("left"), mixer.get("right")
            for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                need(left, k, int, where + "mixer.left.")
            need(left, "scale", NUM, where + "mixer.left.")
            if isinstance(left, dict) and left.get("q_temp") is not None:
                need(left["q_temp"], "coef", NUM, where + "mixer.left.q_temp.")
                need(left["q_temp"], "every", int, where + "mixer.left.q_temp.")
            for k in ("width", "blocks", "conv"):
                need(right, k, int, where + "mixer.right.")
            mlp = l.get("mlp")
            if mlp is not None:
                mk = need(mlp, "kind", str, where + "mlp.")
                if mk == "dense":
                    need(mlp, "ff", int, where + "mlp.")
                    need(mlp, "limit", NUM, where + "mlp.")
                elif mk == "moe":
                    need(mlp.get("expert"), "ff", int, where + "mlp.expert.")
                    need(mlp.get("expert"), "limit", NUM, where + "mlp.expert.")
                    need(mlp.get("router"), "experts", int, where + "mlp.router.")
                    need(mlp.get("router"), "top", int, where + "mlp.router.")
                    if mlp.get("shared") is not None:
                        need(mlp["shared"], "ff", int, where + "mlp.shared.")
                        need(mlp["shared"], "limit", NUM, where + "mlp.shared.")
                elif mk is not None:
                    problems.append(f"{where}mlp.kind={mk!r} (known: dense, moe)")
            layers.append(PakaraxLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        if problems:
            raise CheckpointError("config.json: missing or ill-typed keys: " + ", ".join(problems))
        out = cls(vocab=vocab, width=width, norm_eps=float(eps), logit_scale=float(logit_scale),
                  logit_softcap=float(logit_softcap),
                  loop=None if loop is None else {k: int(loop[k]) for k in ("start", "stop", "times")},
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
        if self.logit_softcap < 0:
            bad("logit_softcap must not be negative")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp["start"] < lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                bad("loop: 0 <= start < stop <= number of layers and times >= 1 are needed")
        for i, l in enumerate(self.layers):
            left, right = l.mixer["left"], l.mixer["right"]
            for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                if left[k] <= 0:
                    bad(f"layers[{i}].mixer.left.{k} must be positive")
            if left["heads"] % left["kv_heads"]:
                bad(f"layers[{i}].mixer.left: heads must be a multiple of kv_heads")
            if left.get("q_temp") is not None and left["q_temp"]["every"] <= 0:
                bad(f"layers[{i}].mixer.left.q_temp.every must be positive")
            for k in ("width", "blocks", "conv"):
                if right[k] <= 0:
                    bad(f"layers[{i}].mixer.right.{k} must be positive")
            if right["width"] % right["blocks"]:
                bad(f"layers[{i}].mixer.right: width must be a multiple of blocks")
            if l.mlp is not None and l.mlp["kind"] == "moe":
                r = l.mlp["router"]
                if not (0 < r["top"] <= r["experts"]):
                    bad(f"layers[{i}].mlp.router: top must be between 1 and experts")

    def to_dict(self) -> Dict[str, Any]:
        out = dict(self.raw)
        out.update({
            "architecture": "Pakarax", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
            "logit_softcap": self.logit_softcap,
            "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers],
        })
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out
