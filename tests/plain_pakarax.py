"""A plain, slow implementation of the Pakarax design, for tests.

Whole sequences, no cache, one function per mechanism, NumPy in double
precision; it shares no code with `reflex_b200`.  Linear weights are [out, in]
and applied as y = x W^T.

The design: a token embedding; layers in which one RMS norm feeds a mixer and
a feed-forward side by side (x += mixer(n) + ff(n)); the mixer is itself two
mixers side by side, an attention (biases, a short causal convolution on q, k
and v, a query temperature that grows with the logarithm of the position, a
per-head linear distance penalty on the scores, a sink in the softmax's
denominator) and a gated linear recurrence (two branches, a short convolution,
block-diagonal gates, a decay a = exp(-8 r softplus(lam))), each RMS-normed
and averaged; the feed-forward is a clamped gated one, dense or a mixture of
experts with sigmoid scores that weight the experts' inputs and a gated shared
expert; a stretch of layers may run several times with the same weights, each
pass starting from a mix of the stream with the embedding output; the model's
norm, the head, a scale and a tanh cap on the logits.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

F = np.float64


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        b, e = ent["data_offsets"]
        raw = blob[b:e]
        if ent["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif ent["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif ent["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {ent['dtype']} of {name}")
        out[name] = arr.astype(F).reshape(ent["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ------------------------------------------------------------------ elements
def rms_norm(x: np.ndarray, w, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(u: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros
    before the sequence's start; the last tap meets the current token."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), u], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y if bias is None else y + bias


# -------------------------------------------------------------------- mixers
def query_temperature(positions: np.ndarray, coef: float, every: int) -> np.ndarray:
    return 1.0 + coef * np.log(np.floor((positions + 1) / every) + 1.0)


def distance_slopes(heads: int) -> np.ndarray:
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F)


def conv_attention(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict) -> np.ndarray:
    """The attention half of the mixer: h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"])
    k = causal_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"])
    v = causal_conv(h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"])
    pos = np.arange(T)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(pos, temp["coef"], temp["every"])[:, None]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    slopes = distance_slopes(H)
    out = np.zeros((T, H, dv), dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        sink = w[p + "sink"][hd]
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, hd]) * m["scale"] - slopes[hd] * (i - pos[:i + 1])
            mx = max(s.max(), sink)
            e = np.exp(s - mx)
            out[i, hd] = (e[:, None] * v[:i + 1, g]).sum(axis=0) / (e.sum() + math.exp(sink - mx))
    return out.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def gated_recurrence(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict) -> np.ndarray:
    """The recurrent half of the mixer: h [T, width] -> [T, width]."""
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, B, W // B)
    r = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    i = sigmoid(np.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    a = np.exp(-8.0 * r * softplus(w[p + "lam"]))
    S = np.zeros(W, dtype=F)
    out = np.zeros((T, W), dtype=F)
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * (i[t] * u[t])
        out[t] = S
    return (out * y) @ w[p + "o"].T


def pair_mixer(h, w, p, m, eps):
    left = rms_norm(conv_attention(h, w, p + "left.", m["left"]), w[p + "left.out"], eps)
    right = rms_norm(gated_recurrence(h, w, p + "right.", m["right"]), w[p + "right.out"], eps)
    return 0.5 * (left + right)


# ------------------------------------------------------------- feed-forwards
def clamped_glu(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def moe_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(h @ w[p + "router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for ex in np.argsort(-s[t], kind="stable")[:top]:
            out[t] += clamped_glu(s[t, ex] * h[t:t + 1], w, f"{p}e{ex}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + sigmoid(h @ w[p + "shared.sg"].T) * clamped_glu(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# --------------------------------------------------------------------- model
def run_order(cfg: dict) -> List[tuple]:
    """(layer, first of a pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], layers_out=None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives
    the residual stream after every layer run."""
    tokens = np.asarray(tokens, dtype=np.int64)
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][tokens]
    x = x0
    for i, first in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T
        hn = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        delta = pair_mixer(hn, w, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            delta = delta + (clamped_glu(hn, w, p + "mlp.", mlp["limit"]) if mlp["kind"] == "dense"
                             else moe_ff(hn, w, p + "mlp.", mlp))
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.copy())
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z
