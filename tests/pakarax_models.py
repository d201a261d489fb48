"""Tiny Pakarax models for tests: configurations that differ in every size and
option, and weights reshaped so that a fault shows.

Random N(0, 0.02) weights would hide most faults: attention scores would be
nearly equal, the recurrence's gates nearly constant, router scores all near a
half, and no logit anywhere near its cap.  `sharpen` scales groups of tensors
so that scores spread over several units (a few keys dominate each softmax, so
the distance penalty, the temperature and the sink show), the gates swing, the
decay covers its whole range, routers choose decisively, the clamps of the
feed-forwards bite, and the largest logits reach the cap's bend.
"""

from __future__ import annotations

import os
import tempfile
from typing import Dict, Tuple

import numpy as np


def pair(heads, kv_heads, dim, vdim, taps, scale, temp, width, blocks, rtaps):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps, "scale": scale}
    if temp is not None:
        left["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": rtaps}}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def model(vocab, width, eps, logit_scale, cap, loop, layers):
    out = {"architecture": "Pakarax", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "logit_scale": logit_scale, "layers": [dict(l, mlp=m) for l, m in layers]}
    if cap is not None:
        out["logit_softcap"] = cap
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# A: the first two of three layers run twice; grouped heads, values wider than keys
# (heads stored 32 wide), a temperature that steps every 7 positions, every kind of
# feed-forward, a layer without one
PAK_A = model(97, 64, 1e-5, 0.5, 12.0, (0, 2, 2), [
    (pair(4, 2, 16, 24, 3, 0.3, (0.3, 7), 48, 3, 2), dense(96, 1.0)),
    (pair(4, 2, 16, 24, 3, 0.3, (0.3, 7), 48, 3, 2), moe(5, 2, 24, 1.5, (40, 0.8))),
    (pair(4, 2, 16, 24, 3, 0.3, (0.3, 7), 48, 3, 2), None),
])
# B: no loop and no cap; one key/value head for six query heads, no convolution on the
# attention's side (one tap: no state), no temperature; one gate block; every expert chosen,
# no shared expert
PAK_B = model(130, 72, 1e-6, 1.0, None, None, [
    (pair(6, 1, 8, 8, 1, 0.5, None, 72, 1, 4), moe(3, 3, 40, 2.0)),
    (pair(2, 2, 32, 16, 2, 0.25, (0.5, 64), 24, 4, 1), dense(80, 0.7)),
])
# C: a width that is no multiple of 8, heads of 40 and 20 (stored 48 wide), the middle layer
# alone runs three times, five taps, one expert of eight
PAK_C = model(61, 100, 1e-5, 2.0, 30.0, (1, 2, 3), [
    (pair(3, 3, 40, 20, 4, 0.2, (0.2, 64), 50, 5, 3), dense(52, 1.0)),
    (pair(3, 3, 40, 20, 5, 0.2, (0.2, 33), 50, 5, 3), moe(8, 1, 16, 1.0, (24, 1.5))),
    (pair(1, 1, 12, 12, 2, 0.3, (1.0, 1), 10, 1, 2), None),
])
# D: heads of 64 (the decode kernel takes their pages by TMA), a loop of one pass (the mix
# still runs once), many experts
PAK_D = model(200, 128, 1e-5, 0.25, 8.0, (0, 1, 1), [
    (pair(8, 2, 64, 64, 2, 0.125, (0.3, 128), 128, 4, 2), moe(33, 4, 32, 1.0, (64, 1.0))),
    (pair(8, 2, 64, 64, 2, 0.125, (0.3, 128), 128, 4, 2), dense(256, 1.2)),
])
# E: keys of 128 and values of 96, the whole model runs twice, long filters
PAK_E = model(77, 96, 1e-5, 1.5, 20.0, (0, 2, 2), [
    (pair(2, 1, 128, 96, 2, 0.09, (0.4, 50), 24, 2, 5), dense(40, 1.0)),
    (pair(2, 1, 128, 96, 2, 0.09, (0.4, 50), 24, 2, 5), moe(1, 1, 20, 1.0)),
])

ALL = {"A": PAK_A, "B": PAK_B, "C": PAK_C, "D": PAK_D, "E": PAK_E}

# tensor-name suffix -> factor (the longest matching suffix counts)
SHARP = (("left.q", 10.0), ("left.k", 10.0), ("left.v", 6.0), ("left.o", 12.0), ("left.sink", 5.0),
         ("right.x", 8.0), ("right.y", 8.0), ("right.ra", 30.0), ("right.ri", 30.0), ("right.o", 12.0),
         ("right.lam", 6.0), ("mlp.router", 40.0), (".gate", 10.0), (".up", 10.0), (".down", 8.0),
         ("shared.sg", 40.0), ("embed", 25.0), ("head", 8.0), ("loop.in", 5.0))

_FOLDERS: Dict[Tuple[str, int, str, bool], str] = {}


def factor(name: str) -> float:
    best, f = -1, 1.0
    for suffix, value in SHARP:
        if name.endswith(suffix) and len(suffix) > best:
            best, f = len(suffix), value
    return f


def model_folder(name: str, seed: int = 3, dtype: str = "float32", sharp: bool = True) -> str:
    """A model folder with the framework's random weights, sharpened; made once."""
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors

    key = (name, seed, dtype, sharp)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"rfx_pak_{name}_")
        write_random_model(ALL[name], seed, d, dtype)
        if sharp:
            path = os.path.join(d, "model.safetensors")
            f = SafetensorsFile(path)
            tensors = [(k, f.tensor(k).clone()) for k in f.keys()]
            f.close()
            write_safetensors(path, [(k, (t.float() * factor(k)).to(t.dtype)) for k, t in tensors])
        _FOLDERS[key] = d
    return _FOLDERS[key]


def tokens(n: int, vocab: int, seed: int):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]
