"""A plain, slow implementation of the Kegasun design, for tests.

Whole sequences, no cache, one function per mechanism, NumPy in double
precision; it shares no code with `reflex_b200`.  Linear weights are [out, in]
and applied as y = x W^T.

The design: token embedding times a scale, plus a hashed bigram row, plus a
sinusoidal position vector; pre-norm layers (layer norm with a weight and no
bias) whose mixer is either a latent attention (queries and keys/values through
low-rank latents, a sliding window, a per-head sink in the softmax's
denominator, a per-head output gate) or an mLSTM (matrix memory with
exponential gates and a running maximum); a feed-forward that is either a
gated dense one (SiLU) or a mixture of experts (squared ReLU, top-k routing);
the model's norm, then the head.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, Sequence

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


# ----------------------------------------------------------------- embedding
def bigram_rows(tokens: np.ndarray, buckets: int, mul_prev: int, mul_cur: int) -> np.ndarray:
    """Row of the bigram table for every position: a hash of (previous token,
    token); the first token of a sequence takes the extra last row."""
    rows = np.empty(len(tokens), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (tokens[:-1] * mul_prev + tokens[1:] * mul_cur) % buckets
    return rows


def sinusoid(positions: np.ndarray, width: int) -> np.ndarray:
    """Entry 2i is sin(p * 10000^(-2i/width)), entry 2i + 1 the cosine of the same angle."""
    out = np.zeros((len(positions), width), dtype=F)
    for i in range((width + 1) // 2):
        ang = positions.astype(F) * (10000.0 ** (-2.0 * i / width))
        out[:, 2 * i] = np.sin(ang)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] = np.cos(ang)
    return out


def embed(cfg: dict, w: Dict[str, np.ndarray], tokens: np.ndarray) -> np.ndarray:
    e = cfg["embedding"]
    x = w["embed"][tokens] * e["scale"]
    b = e.get("bigram")
    if b:
        x = x + w["bigram"][bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x + sinusoid(np.arange(len(tokens)), cfg["width"])


# --------------------------------------------------------------------- norms
def layer_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_norm(x: np.ndarray, w, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# -------------------------------------------------------------------- mixers
def latent_attention(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    """h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ w[p + "g"].T)  # [T, H]
    size = m["mask"]["size"]
    out = np.zeros((T, H, dv), dtype=F)
    for hd in range(H):
        sink = w[p + "sink"][hd]
        for i in range(T):
            lo = max(0, i - size + 1)
            s = (k[lo:i + 1, hd] @ q[i, hd]) * m["scale"]
            mx = max(s.max(), sink)
            e = np.exp(s - mx)
            out[i, hd] = (e[:, None] * v[lo:i + 1, hd]).sum(axis=0) / (e.sum() + math.exp(sink - mx))
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def log_sigmoid(z):
    return np.minimum(z, 0.0) - np.log1p(np.exp(-np.abs(z)))


def mlstm(h: np.ndarray, w: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    ig = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)  # [T, H]
    fg = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = np.zeros((T, H, dv), dtype=F)
    for hd in range(H):
        S = np.zeros((d, dv), dtype=F)
        n = np.zeros(d, dtype=F)
        mx = 0.0
        for t in range(T):
            m_new = max(fg[t, hd] + mx, ig[t, hd])
            a, b = math.exp(fg[t, hd] + mx - m_new), math.exp(ig[t, hd] - m_new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            o[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-mx)) + 1e-6)
    o = o / np.sqrt((o * o).mean(axis=-1, keepdims=True) + eps)
    o = o.reshape(T, H * dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    g = h @ w[p + "gate"].T
    return ((g * sigmoid(g)) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        e = np.exp(z[t, chosen] - z[t, chosen].max())
        e = e / e.sum()
        for wt, ex in zip(e, chosen):
            a = np.maximum(h[t] @ w[f"{p}e{ex}.up"].T, 0.0) ** 2
            out[t] += wt * (a @ w[f"{p}e{ex}.down"].T)
    return out


# --------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], layers_out=None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives
    the residual stream after every layer."""
    tokens = np.asarray(tokens, dtype=np.int64)
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        hn = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            x = x + latent_attention(hn, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            x = x + mlstm(hn, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp:
            hn = layer_norm(x, w[p + "norm2"], eps)
            x = x + (dense_ff(hn, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(hn, w, p + "mlp.", mlp))
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
