"""Kesedra's configuration on the CPU: what config.json means, what is refused, the run order of layers
that share a latent, tensor names, and the plain statement on cases whose answer is known."""

import copy
import math

import pytest
import torch

import plain_kesedra as plain
from tiny_kesedra import K_A, K_B, K_C, TINY_K


def spec_of(raw):
    from starter_b200.config import config_from_dict

    return config_from_dict(raw).to_model_spec()


def test_every_size_and_constant_comes_from_the_config():
    spec = spec_of(K_A)
    assert spec.architecture == "Kesedra" and spec.vocab_size == 200 and spec.hidden_size == 64
    assert spec.embedding_scale == 6.0 and not spec.tie_embeddings and spec.lm_head_name == "head"
    first, second, third, fourth = spec.layers
    assert first.mixer.kind == "wkv" and (first.mixer.num_heads, first.mixer.head_dim, first.mixer.decay_rank) == (2, 16, 8)
    assert first.feed_forward.kind == "dense_biased" and first.feed_forward.intermediate_size == 96
    m = second.mixer
    assert (m.num_heads, m.head_dim, m.rot_dim, m.value_dim, m.q_rank, m.kv_rank) == (3, 16, 8, 24, 24, 32)
    assert m.window == 10 and m.scale == 0.2 and m.position.base == 100.0 and m.position.dims == 8 and m.own_kv
    ff = second.feed_forward
    assert (ff.kind, ff.experts, ff.top, ff.intermediate_size, ff.limit) == ("routed_experts", 5, 2, 24, 1.0)
    assert third.arrangement == "sandwich_mixer_only" and "feed_forward" not in third.parts
    assert not fourth.mixer.own_kv and fourth.mixer.window == 64
    assert all(layer.norm1.unit_offset and layer.norm1.eps == 1e-5 for layer in spec.layers)
    assert spec.final_norm.unit_offset


def test_run_order_of_layers_that_share_a_latent():
    order = spec_of(K_A).schedule
    assert [(e.layer, e.cache, e.writes_cache) for e in order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    order = spec_of(K_C).schedule
    assert [(e.cache, e.writes_cache) for e in order] == [(0, True), (1, True), (1, False), (3, True)]


def test_tensor_names():
    from starter_b200.engine.model import expected_tensors

    names = expected_tensors(spec_of(K_A))
    for name, shape in {"embed": (200, 64), "head": (200, 64), "final.norm": (64,), "l0.mix.mu.w": (64,),
                        "l0.mix.w1": (8, 64), "l0.mix.w2": (32, 8), "l0.mix.u": (2, 16), "l0.mlp.up.b": (96,),
                        "l1.mix.dkv": (40, 64), "l1.mix.uq": (72, 24), "l1.mix.dq.norm": (24,),
                        "l1.mlp.e4.down": (64, 24), "l1.mlp.router.b": (5,), "l1.norm2b": (64,),
                        "l3.mix.uv": (32, 32)}.items():
        assert tuple(names[name].shape) == shape, name
    assert "l3.mix.dkv" not in names and "l2.norm2" not in names and "l2.mlp.up" not in names
    assert "lm_head" not in names


def test_the_decay_rank_comes_from_the_checkpoint_when_the_config_leaves_it_out():
    from starter_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(K_B)
    del raw["layers"][1]["mixer"]["decay_rank"]
    config = config_from_dict(raw)
    with pytest.raises(ConfigError, match="decay"):
        config.to_model_spec()
    filled = config.with_tensor_shapes({"l1.mix.w1": (12, 96), "l0.mix.dq": (40, 96)})
    assert filled.to_model_spec().layers[1].mixer.decay_rank == 12
    with pytest.raises(ConfigError, match="rows"):
        config_from_dict(K_B).with_tensor_shapes({"l1.mix.w1": (5, 96)})


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "mixers"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 2), "does not define"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 0), "caches no latent"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "earlier"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_rank", 16), "kv_rank differs"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 10), "even and at most"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top=6"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "gated"), "feed-forwards"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c["norm"].__setitem__("kind", "layer"), "does not define"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "positive"),
])
def test_what_is_refused(change, message):
    from starter_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(K_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_round_trip():
    from starter_b200.config import config_from_dict

    for raw in TINY_K.values():
        config = config_from_dict(raw)
        assert config_from_dict(config.to_dict()) == config


# ------------------------------------------------------------------------------ the plain statement

def test_plain_rotation_keeps_lengths_and_turns_pairs():
    x = torch.zeros(3, 6, dtype=torch.float64)
    x[:, 0] = 1.0
    x[:, 5] = 7.0
    out = plain.rotate_interleaved(x, torch.tensor([0, 1, 2]), 100.0, 4)
    assert torch.allclose(out[0], x[0])
    assert math.isclose(out[1, 0].item(), math.cos(1.0)) and math.isclose(out[1, 1].item(), math.sin(1.0))
    assert torch.equal(out[:, 4:], x[:, 4:])          # entries from `dims` on pass unchanged
    assert torch.allclose(out.norm(dim=1), x.norm(dim=1))


def test_plain_recurrence_by_hand():
    # one head, one channel: S_t = w S_(t-1) + k v, o_t = r (S_(t-1) + u k v)
    r = torch.tensor([1.0, 2.0, 1.0], dtype=torch.float64).reshape(3, 1, 1)
    k = torch.tensor([1.0, 1.0, 0.0], dtype=torch.float64).reshape(3, 1, 1)
    v = torch.tensor([3.0, 5.0, 9.0], dtype=torch.float64).reshape(3, 1, 1)
    w = torch.full((3, 1, 1), 0.5, dtype=torch.float64)
    u = torch.tensor([[2.0]], dtype=torch.float64)
    out = plain.wkv_recurrence(r, k, v, w, u).flatten().tolist()
    assert out == [6.0, 2.0 * (3.0 + 10.0), 0.5 * 3.0 + 5.0]


def test_plain_routing_by_hand():
    w = {"x.router": torch.eye(4, dtype=torch.float64), "x.router.b": torch.tensor([0.0, 0.0, 0.0, 2.5], dtype=torch.float64)}
    h = torch.tensor([[3.0, 1.0, 2.0, 0.0]], dtype=torch.float64)
    index, weight = plain.route(h, w, "x.", 2)
    assert index.tolist() == [[0, 3]]
    assert torch.allclose(weight, torch.softmax(torch.tensor([[3.0, 2.5]], dtype=torch.float64), dim=-1))


def test_plain_window_by_hand():
    # values that name their position: a query with uniform scores sees exactly the last `size` tokens
    m = dict(heads=1, dim=2, rot_dim=2, vdim=1, q_rank=2, kv_rank=2, scale=1.0, mask=dict(size=3), rot=dict(base=10.0, dims=2))
    z = torch.zeros
    w = {"dq": z(2, 2, dtype=torch.float64), "dq.norm": torch.ones(2, dtype=torch.float64),
         "uq": z(4, 2, dtype=torch.float64), "uk": z(2, 2, dtype=torch.float64),
         "uv": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    c = torch.stack([torch.arange(6, dtype=torch.float64), z(6, dtype=torch.float64)], dim=1)
    out = plain.latent_attention(z(6, 2, dtype=torch.float64), w, "", m, 1e-6, (c, z(6, 2, dtype=torch.float64)))
    assert torch.allclose(out.flatten(), torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=torch.float64))
