"""Kegasun without a GPU: configuration, the model description built from it,
tensor names, the random-weights writer and the loader's one error; and the
plain implementation against itself (the attention over the cached latents with
the query folded through the key up-projection equals the direct form)."""

import copy
import json
import os

import numpy as np
import pytest

import kegasun_models as km
import plain_kegasun as pk


def test_config_to_model_description():
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.cache.specs import KVSpec, StateSpec
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.engine.model import expected_tensors

    typed, spec = spec_from_config_dict(km.KEG_A)
    assert spec.architecture == "kegasun" and spec.vocab_size == 97 and spec.hidden_size == 64
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "mlstm", "latent_attention"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == ["moe", "swiglu", None]
    assert spec.layers[0].mixer.window == 5 and spec.layers[0].mixer.value_dim == 24
    assert [t.kind for t in spec.embedding_terms] == ["bigram_hash", "sinusoidal"]
    names = expected_tensors(spec)
    for n in ("embed", "bigram", "l0.norm1", "l0.norm2", "l0.mix.dq.norm", "l0.mix.sink", "l0.mlp.e4.down",
              "l0.mlp.router.b", "l1.mix.i.b", "l1.mix.norm", "l1.mlp.gate", "l2.norm1", "final.norm", "head"):
        assert n in names, n
    assert "l2.norm2" not in names and "l0.mlp.e5.up" not in names
    assert names["bigram"][1].shape == (54, 64) and names["l0.mix.uk"][1].shape == (64, 32)
    assert names["l1.mix.i"][1].shape == (2, 64) and names["l0.mix.g"][1].shape == (4, 64)
    assert typed.to_dict()["layers"][0]["mixer"]["mask"]["size"] == 5


def test_config_problems_are_named_together():
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.errors import CheckpointError

    bad = copy.deepcopy(km.KEG_B)
    del bad["width"]
    del bad["layers"][1]["mixer"]["kv_rank"]
    bad["layers"][0]["mlp"]["router"]["top"] = "two"
    with pytest.raises(CheckpointError) as e:
        spec_from_config_dict(bad)
    for piece in ("width", "layers[1].mixer.kv_rank", "layers[0].mlp.router.top"):
        assert piece in str(e.value)
    worse = copy.deepcopy(km.KEG_B)
    worse["layers"][2]["type"] = "conv"
    with pytest.raises(CheckpointError):
        spec_from_config_dict(worse)
    over = copy.deepcopy(km.KEG_B)
    over["layers"][0]["mlp"]["router"]["top"] = 4
    with pytest.raises(CheckpointError):
        spec_from_config_dict(over)


def test_random_model_folder_and_the_loaders_one_error(tmp_path):
    from reflex_b200.errors import CheckpointError
    from reflex_b200.weights import SafetensorsFile, write_safetensors
    from reflex_b200.weights.loader import check_names_and_shapes, load_spec
    from reflex_b200.weights.safetensors_io import Checkpoint

    d = km.model_folder("C")
    with open(os.path.join(d, "config.json")) as f:
        assert json.load(f)["architecture"] == "Kegasun"
    _typed, spec = load_spec(d)
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = [(k, f.tensor(k).clone()) for k in f.keys() if k != "l0.mix.sink"]
    f.close()
    tensors = [(k, t[:-1].clone() if k == "bigram" else t) for k, t in tensors] + [("l1.norm2", tensors[0][1])]
    bad = str(tmp_path)
    with open(os.path.join(bad, "config.json"), "w") as out, open(os.path.join(d, "config.json")) as src:
        out.write(src.read())
    write_safetensors(os.path.join(bad, "model.safetensors"), tensors)
    ck = Checkpoint(bad)
    with pytest.raises(CheckpointError) as e:
        check_names_and_shapes(spec, ck)
    ck.close()
    for piece in ("l0.mix.sink", "l1.norm2", "bigram"):
        assert piece in str(e.value)


def test_plain_latent_attention_equals_its_form_over_the_latents():
    """Scores (W_uk^T q) . c and values W_uv (sum p c): what the kernels compute."""
    cfg, w = pk.read_model(km.model_folder("A"))
    m, p, eps = cfg["layers"][0]["mixer"], "l0.mix.", cfg["norm"]["eps"]
    rng = np.random.default_rng(0)
    h = rng.standard_normal((23, cfg["width"]))
    direct = pk.latent_attention(h, w, p, m, eps)
    T, H, d, dv, kr = 23, m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    cq = pk.rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d)
    c = pk.rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    uk, uv = w[p + "uk"].reshape(H, d, kr), w[p + "uv"].reshape(H, dv, kr)
    gate = pk.sigmoid(h @ w[p + "g"].T)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        qa = q[:, hd] @ uk[hd]  # [T, kv_rank]
        for i in range(T):
            lo = max(0, i - m["mask"]["size"] + 1)
            s = (c[lo:i + 1] @ qa[i]) * m["scale"]
            mx = max(s.max(), w[p + "sink"][hd])
            e = np.exp(s - mx)
            o = (e[:, None] * c[lo:i + 1]).sum(0) / (e.sum() + np.exp(w[p + "sink"][hd] - mx))
            out[i, hd] = (uv[hd] @ o) * gate[i, hd]
    assert np.abs(out.reshape(T, -1) @ w[p + "o"].T - direct).max() < 1e-9


def test_plain_mlstm_stays_finite_and_its_maximum_starts_at_zero():
    cfg, w = pk.read_model(km.model_folder("B"))
    rng = np.random.default_rng(1)
    h = rng.standard_normal((400, cfg["width"])) * 3
    out = pk.mlstm(h, w, "l0.mix.", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    assert np.isfinite(out).all() and np.abs(out).max() > 1e-3


def test_state_and_cache_needs():
    """An mLSTM asks for fixed-size state, a latent attention for one shared
    key/value head of kv_rank elements with its window, the bigram term for one
    word a sequence."""
    import torch

    from reflex_b200 import models  # noqa: F401
    from reflex_b200.cache.specs import KVSpec, StateSpec
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.engine.model import CausalLM

    _t, spec = spec_from_config_dict(km.KEG_A)
    lm = CausalLM(spec, torch.float32, "cpu")
    needs = lm.cache_entry_specs()
    assert needs[0] == needs[2] == KVSpec(1, 32, 5, shared_kv=True)
    assert needs[1] == StateSpec((2, 16 * 40 + 16 + 1), "float32")
    assert needs[-1] == StateSpec((1,), "int32")
    assert lm.capturable
