"""Pakarax without a GPU: configuration, the model description built from it
(run order of a looped stretch, cache entries, tensor names), the
random-weights writer and the loader's one error; the plain implementation
against itself; and that the test models' weights make every mechanism show."""

import copy
import json
import os

import numpy as np
import pytest

import pakarax_models as pm
import plain_pakarax as pp


def test_config_to_model_description():
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.engine.model import expected_tensors

    typed, spec = spec_from_config_dict(pm.PAK_A)
    assert spec.architecture == "pakarax" and spec.vocab_size == 97 and spec.hidden_size == 64
    assert [l.block for l in spec.layers] == ["parallel"] * 3
    assert [l.mixer.kind for l in spec.layers] == ["pair"] * 3
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["glu_clamped", "moe", None]
    left, right = spec.layers[0].mixer.param("left"), spec.layers[0].mixer.param("right")
    assert (left.kind, left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim) == \
        ("conv_attention", 4, 2, 16, 24)
    assert left.param("taps") == 3 and left.param("temp_every") == 7 and left.window is None
    assert (right.kind, right.param("width"), right.param("blocks"), right.param("taps")) == ("rglru", 48, 3, 2)
    # layers 0 and 1 twice, then layer 2; a cache entry per run; each pass starts from the mix
    assert [(r.layer, r.cache, r.mixes_input) for r in spec.run_order] == \
        [(0, 0, True), (1, 1, False), (0, 2, True), (1, 3, False), (2, 4, False)]
    assert spec.logit_scale == 0.5 and spec.logit_softcap == 12.0 and spec.stream_mix_name == "loop.in"
    names = expected_tensors(spec)
    for n in ("embed", "loop.in", "l0.norm1", "l0.mix.left.q.b", "l0.mix.left.k.conv", "l0.mix.left.sink",
              "l0.mix.left.o.b", "l0.mix.left.out", "l0.mix.right.ra.b", "l0.mix.right.lam", "l0.mix.right.out",
              "l0.mlp.gate", "l1.mlp.e4.gate", "l1.mlp.router", "l1.mlp.shared.sg", "l2.norm1", "final.norm", "head"):
        assert n in names, n
    for n in ("l0.norm2", "l1.mlp.e5.up", "l2.mlp.gate", "l1.mlp.router.b", "l0.mix.right.o.b"):
        assert n not in names, n
    assert names["loop.in"][1].shape == (64, 128) and names["l0.mix.left.v"][1].shape == (48, 64)
    assert names["l0.mix.left.q.conv"][1].shape == (64, 3) and names["l0.mix.right.ra"][1].shape == (3, 16, 16)
    assert names["l1.mlp.shared.sg"][1].shape == (1, 64) and names["l0.mix.left.o"][1].shape == (64, 96)
    assert typed.to_dict()["loop"] == {"start": 0, "stop": 2, "times": 2}


def test_models_without_a_loop_a_cap_a_temperature_or_a_shared_expert():
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.engine.model import expected_tensors

    _typed, spec = spec_from_config_dict(pm.PAK_B)
    assert spec.stream_mix_name is None and spec.logit_softcap == 0.0
    assert not any(r.mixes_input for r in spec.run_order) and len(spec.run_order) == 2
    names = expected_tensors(spec)
    assert "loop.in" not in names and "l0.mlp.shared.gate" not in names and "l0.mlp.e2.gate" in names
    assert spec.layers[0].mixer.param("left").param("temp_coef") == 0.0
    _typed, spec = spec_from_config_dict(pm.PAK_C)  # the middle layer three times, between two others
    assert [(r.layer, r.mixes_input) for r in spec.run_order] == \
        [(0, False), (1, True), (1, True), (1, True), (2, False)]
    assert sorted(spec.cache_entries()) == [0, 1, 2, 3, 4]


def test_what_the_mixers_ask_of_the_cache():
    import torch

    from reflex_b200 import models  # noqa: F401
    from reflex_b200.cache.specs import KVSpec, StateSpec
    from reflex_b200.cache.store import Cache
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.engine.model import CausalLM

    _typed, spec = spec_from_config_dict(pm.PAK_A)
    model = CausalLM(spec, torch.float32, "cpu")
    entries = model.cache_entry_specs()
    # keys and values 32 wide (values of 24 beside keys of 16), the three projections' last two
    # rows, and the recurrence's [last input | S]
    assert entries[0] == (KVSpec(2, 32, None), StateSpec((2, 4 * 16 + 2 * 16 + 2 * 24), "float32"),
                          StateSpec((2 * 48,), "float32"))
    _typed, spec_b = spec_from_config_dict(pm.PAK_B)
    assert CausalLM(spec_b, torch.float32, "cpu").cache_entry_specs()[0] == \
        (KVSpec(1, 16, None), StateSpec((4 * 72,), "float32"))  # one tap: the attention keeps no state
    cache = Cache(entries, 256, 1 << 20, torch.float32, None)
    assert cache.has(0) == "parts" and cache.has(4) == "parts" and cache.has(7) is None
    assert len(cache.kv_groups) == 1 and len(cache.kv_groups[0].entries) == 5  # one group for all five runs
    s = cache.take_slot()
    cache.reserve([(s, 70)])
    cache.commit([(s, 70)])
    assert cache.tokens_held() == 128
    cache.give_slot(s)
    assert cache.tokens_held() == 0


def test_config_problems_are_named_together():
    from reflex_b200 import models  # noqa: F401
    from reflex_b200.config.registry import spec_from_config_dict
    from reflex_b200.errors import CheckpointError

    bad = copy.deepcopy(pm.PAK_A)
    del bad["width"]
    del bad["layers"][1]["mixer"]["left"]["kv_heads"]
    bad["layers"][0]["mlp"]["limit"] = "one"
    bad["layers"][1]["mlp"]["router"]["top"] = "two"
    del bad["loop"]["times"]
    with pytest.raises(CheckpointError) as e:
        spec_from_config_dict(bad)
    for piece in ("width", "layers[1].mixer.left.kv_heads", "layers[0].mlp.limit", "layers[1].mlp.router.top",
                  "loop.times"):
        assert piece in str(e.value)
    for change in (lambda c: c["layers"][2].update(type="serial"),
                   lambda c: c["layers"][1]["mlp"]["router"].update(top=6),
                   lambda c: c["loop"].update(stop=4),
                   lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5),
                   lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3)):
        worse = copy.deepcopy(pm.PAK_A)
        change(worse)
        with pytest.raises(CheckpointError):
            spec_from_config_dict(worse)


def test_random_weights_writer_and_the_loaders_one_error(tmp_path):
    import torch

    from reflex_b200.errors import CheckpointError
    from reflex_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    from reflex_b200.weights.loader import check_names_and_shapes, load_spec
    from reflex_b200.weights.safetensors_io import Checkpoint

    d = str(tmp_path / "m")
    write_random_model(pm.PAK_C, 7, d, "bfloat16")
    _typed, spec = load_spec(d)
    ck = Checkpoint(d)
    check_names_and_shapes(spec, ck)
    ck.close()
    cfg, w = pp.read_model(d)
    assert cfg["loop"] == {"start": 1, "stop": 2, "times": 3} and w["loop.in"].shape == (100, 200)
    assert pp.forward(cfg, w, [1, 2, 3]).shape == (3, 61)
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    f.close()
    del tensors["l1.mlp.shared.sg"]
    tensors["l0.mix.right.lam"] = torch.zeros(49)
    tensors["l2.mlp.gate"] = torch.zeros(3, 3)
    write_safetensors(path, list(tensors.items()))
    ck = Checkpoint(d)
    with pytest.raises(CheckpointError) as e:
        check_names_and_shapes(spec, ck)
    ck.close()
    for piece in ("l1.mlp.shared.sg", "l0.mix.right.lam", "l2.mlp.gate"):
        assert piece in str(e.value)


# ------------------------------------------------- the plain implementation
def test_plain_convolution_taps_and_start():
    u = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    w = np.array([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]])
    y = pp.causal_conv(u, w)
    # the last tap meets the current token, the first one the token two back; zeros before the start
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    assert y[:, 1].tolist() == [20.0, 40.0, 60.0, 80.0, 100.0]
    assert np.array_equal(pp.causal_conv(u, w[:, 2:]), u * w[:, 2])  # one tap: no look back


def test_plain_recurrence_limits():
    """Gates pinned open or shut: S follows its closed forms."""
    W = 4
    w = {"y": np.zeros((W, 3)), "y.b": np.full(W, 50.0), "x": np.zeros((W, 3)), "x.b": np.full(W, 2.0),
         "conv": np.ones((W, 1)), "conv.b": np.zeros(W), "ra": np.zeros((1, W, W)), "ri": np.zeros((1, W, W)),
         "ra.b": np.full((1, W), -50.0), "ri.b": np.full((1, W), 50.0), "lam": np.zeros(W), "o": np.eye(W)}
    h = np.zeros((5, 3))
    m = {"width": W, "blocks": 1, "conv": 1}
    # r = 0: a = 1, the step sqrt(1 - a^2) = 0: nothing ever enters S
    assert np.abs(pp.gated_recurrence(h, w, "", m)).max() < 1e-9
    # r = 1: a = exp(-8 ln 2) = 2^-8; S_t -> sqrt(1 - a^2) u / (1 - a); gelu(50) = 50
    w["ra.b"] = np.full((1, W), 50.0)
    out = pp.gated_recurrence(h, w, "", m)
    a = 2.0 ** -8
    want = [50.0 * 2.0 * np.sqrt(1 - a * a) * (1 - a ** (t + 1)) / (1 - a) for t in range(5)]
    assert np.abs(out[:, 0] - want).max() < 1e-9


def test_plain_temperature_and_slopes():
    t = pp.query_temperature(np.array([0, 5, 6, 12, 13]), 0.5, 7)
    assert np.allclose(t, [1.0, 1.0, 1 + 0.5 * np.log(2), 1 + 0.5 * np.log(2), 1 + 0.5 * np.log(3)])
    assert np.allclose(pp.distance_slopes(4), [0.25, 0.0625, 0.015625, 0.00390625])


@pytest.mark.parametrize("name", sorted(pm.ALL))
def test_every_mechanism_shows_in_the_test_models(name):
    """With one mechanism changed a little (the plain model's own config or
    weights), the logits move by far more than the tests' tolerance: a fault
    in it would be seen."""
    cfg, w = pp.read_model(pm.model_folder(name))
    toks = pm.tokens(140 if name == "D" else 90, cfg["vocab"], 11)  # past D's first temperature step
    base = pp.forward(cfg, w, toks)
    size = np.abs(base).max()

    def moved(cfg2, w2, since=0):
        other = pp.forward(cfg2, w2, toks)
        return np.abs(other - base)[since:].max() / size

    changes = []
    c = copy.deepcopy(cfg)  # a cap a little higher
    if c.get("logit_softcap"):
        c["logit_softcap"] *= 1.5
        changes.append(("cap", moved(c, w)))
    for li, layer in enumerate(cfg["layers"]):
        left = layer["mixer"]["left"]
        if left.get("q_temp"):
            c = copy.deepcopy(cfg)
            c["layers"][li]["mixer"]["left"]["q_temp"]["every"] += 1
            changes.append((f"l{li} temperature", moved(c, w)))
        w2 = dict(w)  # the sinks a little larger
        w2[f"l{li}.mix.left.sink"] = w[f"l{li}.mix.left.sink"] + 0.5
        changes.append((f"l{li} sink", moved(cfg, w2)))
        w2 = dict(w)  # the first token's influence through the recurrence's decay
        w2[f"l{li}.mix.right.lam"] = w[f"l{li}.mix.right.lam"] + 0.3
        changes.append((f"l{li} decay", moved(cfg, w2)))
        if left["conv"] > 1:
            w2 = dict(w)  # the oldest tap
            w2[f"l{li}.mix.left.k.conv"] = w[f"l{li}.mix.left.k.conv"].copy()
            w2[f"l{li}.mix.left.k.conv"][:, 0] += 0.2
            changes.append((f"l{li} oldest tap", moved(cfg, w2)))
        mlp = layer.get("mlp")
        if mlp:
            c = copy.deepcopy(cfg)
            if mlp["kind"] == "dense":
                c["layers"][li]["mlp"]["limit"] *= 0.8
            else:
                c["layers"][li]["mlp"]["expert"]["limit"] *= 0.8
            changes.append((f"l{li} clamp", moved(c, w)))
    for what, m in changes:
        assert m > 2e-3, (what, m)


def test_the_distance_penalty_is_not_a_bias_on_the_key_alone():
    """With a sink, taking slope * (i - j) off the scores differs from adding
    slope * j: the plain model tells the two apart."""
    cfg, w = pp.read_model(pm.model_folder("A"))
    m = cfg["layers"][0]["mixer"]["left"]
    rng = np.random.default_rng(0)
    h = rng.standard_normal((40, cfg["width"]))
    out = pp.conv_attention(h, w, "l0.mix.left.", m)
    real = pp.distance_slopes
    try:
        pp.distance_slopes = lambda heads: np.zeros(heads)
        flat = pp.conv_attention(h, w, "l0.mix.left.", m)
    finally:
        pp.distance_slopes = real
    assert np.abs(out - flat).max() > 0.05 * np.abs(out).max()
