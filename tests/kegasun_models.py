"""Tiny Kegasun models for tests: configurations that differ in every size and
option, and weights reshaped so that a fault shows.

Random N(0, 0.02) weights would hide most faults: attention scores would be
nearly equal (every key moves the output by 1/n), gates and router logits
nearly constant, and every layer's output tiny beside the position vector.
`sharpen` scales groups of tensors so that scores spread over several units
(a few keys dominate each softmax, so a key wrongly in or out of a window
shows), sinks matter, the mLSTM's gates swing, routers choose decisively, and
the layers' outputs are of the residual's size.
"""

from __future__ import annotations

import os
import tempfile
from typing import Dict, Tuple

import numpy as np


def latent(heads, dim, vdim, q_rank, kv_rank, window, scale):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "mask": {"size": window}, "scale": scale}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, eps, scale, bigram, layers):
    return {"architecture": "Kegasun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1],
                                                    "mul_cur": bigram[2]}},
            "layers": [dict(l, mlp=m) for l, m in layers]}


# A: a window shorter than a page, value size other than key size, two latent
# layers of one shape (one cache group), a layer that is its mixer alone
KEG_A = model(97, 64, 1e-5, 2.0, (53, 31, 3), [
    (latent(4, 16, 24, 24, 32, 5, 0.3), moe(5, 2, 24)),
    (mlstm(2, 16, 40, 8.0), dense(96)),
    (latent(4, 16, 24, 24, 32, 5, 0.3), None),
])
# B: one head, a value size of two column slices, every expert chosen, one expert
# of eight chosen, a window longer than a page, latents of the tensor-core sizes
KEG_B = model(130, 72, 1e-6, 1.0, (1000, 7, 11), [
    (mlstm(1, 24, 72, 15.0), moe(3, 3, 40)),
    (latent(6, 8, 8, 16, 64, 70, 0.5), dense(80)),
    (latent(1, 32, 16, 40, 128, 200, 0.25), moe(8, 1, 16)),
])
# C: a width that is no multiple of 8 (no 16-byte unit fits a bfloat16 row), a
# latent of 40 (no tensor-core attention takes it), a window of exactly a page,
# a tiny bigram table, an mLSTM last and alone
KEG_C = model(61, 100, 1e-5, 4.0, (7, 1000003, 999983), [
    (latent(3, 12, 20, 20, 40, 64, 0.2), dense(52)),
    (mlstm(3, 8, 8, 5.0), None),
])
# D: many heads over a 64-wide latent, a window of two pages and one
KEG_D = model(200, 128, 1e-5, 3.0, (211, 5, 9), [
    (latent(12, 16, 16, 32, 64, 129, 0.25), moe(33, 4, 32)),
    (mlstm(4, 32, 32, 10.0), dense(256)),
])

# E: awkward sizes throughout: five heads of 10, values of 6, a latent of 48, a window of 33,
# an mLSTM whose values are no multiple of four and span two column slices, one expert
# of one, a dense width that is no multiple of 8
KEG_E = model(77, 88, 1e-5, 1.5, (19, 3, 5), [
    (latent(5, 10, 6, 12, 48, 33, 0.31), moe(1, 1, 20)),
    (mlstm(3, 10, 70, 6.0), dense(36)),
    (latent(5, 10, 6, 12, 48, 33, 0.31), dense(36)),
])
# F: a latent of 192 (three 64-column boxes), key sizes of 200 and 300 in the mLSTM (the
# widest register form, and the shared-memory form), a window longer than the prompts
KEG_F = model(90, 96, 1e-5, 2.5, (64, 9, 1), [
    (mlstm(2, 200, 16, 9.0), None),
    (latent(2, 64, 32, 48, 192, 1000, 0.125), moe(4, 2, 48)),
    (mlstm(1, 300, 8, 20.0), dense(64)),
])

# G: no attention at all (the cache then holds state only)
KEG_G = model(50, 48, 1e-5, 1.0, (31, 2, 3), [
    (mlstm(2, 12, 24, 7.0), moe(4, 2, 16)),
    (mlstm(3, 16, 16, 11.0), None),
])

ALL = {"A": KEG_A, "B": KEG_B, "C": KEG_C, "D": KEG_D, "E": KEG_E, "F": KEG_F, "G": KEG_G}

# tensor-name suffix -> factor
SHARP = (("mix.uq", 14.0), ("mix.uk", 14.0), ("mix.sink", 5.0), ("mix.i", 25.0), ("mix.f", 25.0),
         ("mix.i.b", 3.0), ("mix.f.b", 6.0), ("mlp.router", 40.0), ("mlp.router.b", 2.0),
         (".up", 8.0), (".down", 8.0), ("mlp.gate", 8.0), ("mix.o", 12.0), ("mix.uv", 6.0),
         ("mix.v", 6.0), ("mix.k", 6.0), ("mix.q", 6.0), ("mix.g", 10.0), ("embed", 25.0), ("bigram", 25.0),
         ("head", 6.0))

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
        d = tempfile.mkdtemp(prefix=f"rfx_keg_{name}_")
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
