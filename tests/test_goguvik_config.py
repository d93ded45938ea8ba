"""Goguvik on the CPU: its config.json, the model spec made from it, its tensor names, and the plain
statement's own mechanisms on cases whose answer is known."""

import copy
import math

import pytest
import torch

import plain_goguvik as plain
from tiny_goguvik import TINY_G, make_goguvik_folder

from starter_b200.config import ConfigError, GoguvikConfig, config_from_dict
from starter_b200.engine.model import expected_tensors


def test_the_architecture_is_found_by_either_key():
    raw = copy.deepcopy(TINY_G["GA"])
    assert isinstance(config_from_dict(raw), GoguvikConfig)
    raw["architectures"] = [raw.pop("architecture")]
    assert isinstance(config_from_dict(raw), GoguvikConfig)
    with pytest.raises(ConfigError):
        config_from_dict({"vocab": 3})


def test_every_size_and_constant_comes_from_the_config():
    spec = config_from_dict(TINY_G["GC"]).to_model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.streams, len(spec.layers)) == (300, 80, 2, 3)
    first, middle, last = (layer.mixer for layer in spec.layers)
    assert (first.num_heads, first.num_kv_heads, first.head_dim, first.value_dim) == (6, 1, 24, 16)
    assert (first.scale, first.lambda_init, first.norm_eps) == (0.15, 0.28, 1e-6)
    assert (first.q_temperature.coef, first.q_temperature.every) == (0.35, 48)
    assert middle.q_temperature is None and (middle.num_heads, middle.head_dim, middle.value_dim) == (2, 32, 32)
    assert first.own_kv and middle.own_kv and not last.own_kv
    assert spec.layers[2].feed_forward.intermediate_size == 64
    assert spec.layers[0].feed_forward.activation == "gelu_tanh"
    assert spec.tie_embeddings


def test_a_shared_layer_reads_its_source_layers_cache_entry():
    spec = config_from_dict(TINY_G["GA"]).to_model_spec()
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == \
        [(0, 0, True), (1, 0, False), (2, 2, True), (3, 0, False)]
    names = expected_tensors(spec)
    assert "l0.mix.k" in names and "l0.mix.v.b" in names
    assert not any(n.startswith(("l1.mix.k", "l1.mix.v", "l3.mix.k", "l3.mix.v")) for n in names)
    # the layer without a feed-forward has one sublayer: no second norm, no second connection
    assert "l2.hc1.mix" in names and not any(n.startswith(("l2.mlp", "l2.norm2", "l2.hc2")) for n in names)
    assert tuple(names["l0.hc1.mix"].shape) == (3, 3) and tuple(names["l0.norm1.alpha"].shape) == ()
    assert tuple(names["l0.mix.q"].shape) == (4 * 2 * 16, 64) and tuple(names["l0.mix.v"].shape) == (2 * 24, 64)
    assert tuple(names["l0.mix.g"].shape) == (4 * 24, 64) and tuple(names["l0.mix.o"].shape) == (64, 4 * 24)
    assert "final.norm.alpha" in names and "lm_head" not in names


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim differs"),
    (lambda c: c["layers"][0].update(type="recurrent"), "attention"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(rope=1e4), "does not define"),
    (lambda c: c.pop("streams"), "streams"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_a_config_that_asks_for_something_else_is_refused(change, text):
    raw = copy.deepcopy(TINY_G["GA"])
    change(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_the_config_survives_writing_and_reading(tmp_path):
    folder = make_goguvik_folder(tmp_path, "GC", seed=3)
    cfg, w = plain.read_model_folder(folder)
    again = config_from_dict(cfg)
    assert again.to_model_spec() == config_from_dict(TINY_G["GC"]).to_model_spec()
    assert set(w) == set(expected_tensors(again.to_model_spec()))


def test_tensors_of_an_absent_second_sublayer_may_be_stored_and_are_not_read(tmp_path):
    from starter_b200.weights.loader import WeightError, check_names

    spec = config_from_dict(TINY_G["GA"]).to_model_spec()
    assert "l2.norm2.alpha" in spec.ignored_tensors and "l2.hc2.mix" in spec.ignored_tensors
    wanted = expected_tensors(spec)
    stored = {n: (torch.bfloat16, tuple(p.shape)) for n, p in wanted.items()}
    stored["l2.hc2.mix"] = (torch.bfloat16, (3, 3))
    assert check_names(wanted, stored, spec.ignored_tensors)[1] == []
    stored["l2.hc3.mix"] = (torch.bfloat16, (3, 3))
    assert check_names(wanted, stored, spec.ignored_tensors)[1] == ["l2.hc3.mix"]
    assert WeightError


# ------------------------------------------------------------------ the plain statement itself

def test_plain_streams_with_identity_mixing_are_a_residual_sum():
    t = torch.randn(5, 3, 7, dtype=torch.float64)
    y = torch.randn(5, 7, dtype=torch.float64)
    new = plain.plain_stream_write(t, y, torch.eye(3, dtype=torch.float64), torch.tensor([1.0, 0.0, 2.0], dtype=torch.float64))
    assert torch.allclose(new[:, 0], t[:, 0] + y) and torch.allclose(new[:, 1], t[:, 1]) and torch.allclose(new[:, 2], t[:, 2] + 2 * y)
    # rows of the matrix are source streams, columns destinations: the entry [0, 2] copies stream 0 into stream 2
    mix = torch.zeros(3, 3, dtype=torch.float64)
    mix[0, 2] = 1.0
    moved = plain.plain_stream_write(t, torch.zeros_like(y), mix, torch.zeros(3, dtype=torch.float64))
    assert torch.allclose(moved[:, 2], t[:, 0]) and float(moved[:, :2].abs().max()) == 0.0


def test_plain_temperature_steps_where_the_quotient_does():
    p = torch.arange(20, dtype=torch.float64)
    got = plain.plain_query_temperature(p, 0.5, 8)
    assert torch.all(got[:7] == 1.0)                                  # (p + 1) / 8 < 1
    assert torch.allclose(got[7:15], torch.tensor(1.0 + 0.5 * math.log(2.0), dtype=torch.float64))
    assert torch.allclose(got[15:], torch.tensor(1.0 + 0.5 * math.log(3.0), dtype=torch.float64))


def test_plain_differential_head_with_equal_maps_is_a_normed_single_map():
    torch.manual_seed(0)
    q, k = torch.randn(6, 4, dtype=torch.float64), torch.randn(6, 4, dtype=torch.float64)
    v = torch.randn(6, 5, dtype=torch.float64)
    pos = torch.arange(6)
    out = plain.plain_differential_head(q, q, k, k, v, 0.5, 0.25, 0.2, 0.0, pos)
    single = plain.plain_softmax_map(q, k, 0.5, pos) @ v
    want = single / single.pow(2).mean(-1, keepdim=True).sqrt() * 0.8     # (1 - 0.25) cancels in the norm
    assert torch.allclose(out, want)
    assert torch.allclose(out[0], v[0] / v[0].pow(2).mean().sqrt() * 0.8)   # the first token sees itself


def test_plain_gelu_is_the_tanh_form():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.5, 3.0], dtype=torch.float64)
    assert torch.allclose(plain.plain_gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
