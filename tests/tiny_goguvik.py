"""Tiny Goguvik configurations for the tests: they differ in every size and option."""

import os

import torch


def _mixer(heads, kv_heads, dim, vdim, scale, diff, temp=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if temp is not None:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, ff):
    return dict(type="attention", mixer=mixer, mlp=dict(kind="dense", ff=ff) if ff else None)


# three streams; value rows shorter than key rows; a layer without a feed-forward; a shared layer right
# behind its source and one further on; a temperature that steps every 8 positions
G_A = dict(architecture="Goguvik", vocab=200, width=64, streams=3, norm=dict(eps=1e-5), layers=[
    _layer(_mixer(4, 2, 16, 24, 0.2, 0.25, (0.5, 8)), 96),
    _layer(_mixer(4, 2, 16, 24, 0.2, 0.25, (0.5, 8), kv_from=0), 96),
    _layer(_mixer(4, 2, 16, 24, 0.3, 0.4, (0.25, 8)), None),
    _layer(_mixer(4, 2, 16, 24, 0.3, 0.4, (0.25, 8), kv_from=0), 80),
])

# one stream; as many key/value heads as query heads; value rows longer than key rows; no shared
# layers; a temperature that steps every 5 positions; an odd vocabulary
G_B = dict(architecture="Goguvik", vocab=131, width=96, streams=1, norm=dict(eps=1e-6), layers=[
    _layer(_mixer(3, 3, 8, 40, 0.35, 0.1, (1.0, 5)), 160),
    _layer(_mixer(3, 3, 8, 40, 0.35, 0.1, (1.0, 5)), 160),
])

# two streams; one key/value head for six query heads; key rows of 48; layers that differ in their
# head counts; no temperature in the middle layer; a shared layer whose source is two layers back
G_C = dict(architecture="Goguvik", vocab=300, width=80, streams=2, norm=dict(eps=1e-6), layers=[
    _layer(_mixer(6, 1, 24, 16, 0.15, 0.28, (0.35, 48)), 112),
    _layer(_mixer(2, 2, 32, 32, 0.125, 0.2), 112),
    _layer(_mixer(6, 1, 24, 16, 0.15, 0.28, (0.35, 48), kv_from=0), 64),
])

# sizes the tensor-core prompt kernel takes (key rows of 32 and 64, value rows of 32 and 64), so that
# whole prompts and portions run on it and single tokens on the other kernel, over the same cache
G_D = dict(architecture="Goguvik", vocab=257, width=128, streams=2, norm=dict(eps=1e-6), layers=[
    _layer(_mixer(4, 2, 16, 32, 0.25, 0.2, (0.4, 16)), 192),
    _layer(_mixer(4, 2, 16, 32, 0.25, 0.2, (0.4, 16), kv_from=0), 192),
    _layer(_mixer(2, 1, 32, 64, 0.18, 0.35, (0.4, 16)), 192),
])

TINY_G = {"GA": G_A, "GB": G_B, "GC": G_C, "GD": G_D}


def make_goguvik_folder(tmp_path, name, seed=0, dtype=torch.float32):
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    path = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    write_model_folder(path, config_from_dict(TINY_G[name]), seed, dtype)
    # The library draws matrices from N(0, 0.02): with those every score is near 0, every softmax near
    # uniform and every tanh near linear, and a wrong key or a lost stream would hardly show.  Larger
    # matrices give scores of order one and norms that bend.
    from safetensors.torch import load_file, save_file

    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for key, value in tensors.items():
        if value.dim() == 2 and ".hc" not in key:
            factor = 25.0 if key == "embed" else 16.0 if key.endswith((".q", ".k")) else 4.0
            tensors[key] = (value.float() * factor).to(value.dtype)
        elif key.endswith(".mix"):          # near the identity, so that streams neither die out nor blow up
            tensors[key] = (torch.eye(value.shape[0]) * 0.8 + (value.float() - 0.25)).to(value.dtype)
        elif key.endswith((".in", ".out")) and ".hc" in key:
            tensors[key] = (value.float() + 0.6).to(value.dtype)
    save_file(tensors, file, metadata={"format": "pt"})
    return path
