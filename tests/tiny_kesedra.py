"""Tiny Kesedra configurations for the tests: they differ in every size, constant and layer order."""

import os

import torch


def wkv(heads, dim, rank, mlp):
    return dict(type="wkv", mixer=dict(heads=heads, dim=dim, decay_rank=rank), mlp=mlp)


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base, mlp, dims=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
             mask=dict(size=window), rot=dict(base=base, dims=rot_dim if dims is None else dims))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


# recurrence first; a window of 10; a layer without a feed-forward; a shared latent two layers on with
# other heads and a window that ends on a page border; experts of 24 (no multiple of 16)
K_A = dict(architecture="Kesedra", vocab=200, width=64, embedding=dict(scale=6.0), norm=dict(eps=1e-5), layers=[
    wkv(2, 16, 8, dense(96)),
    latent(3, 16, 8, 24, 24, 32, 0.2, 10, 100.0, moe(5, 2, 24, 1.0)),
    wkv(4, 8, 4, None),
    latent(2, 8, 8, 16, 16, 32, 0.3, 64, 100.0, dense(80), kv_from=1),
])

# attention first, one head, only half of the rotated part turned, a window of 3; one expert of three and
# all three of three; one recurrent head of 48 channels; a window longer than any test sequence; an odd vocabulary
K_B = dict(architecture="Kesedra", vocab=131, width=96, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=[
    latent(1, 24, 16, 8, 40, 48, 0.15, 3, 10000.0, moe(3, 1, 32, 2.5), dims=8),
    wkv(1, 48, 12, moe(3, 3, 16, 0.7)),
    latent(5, 8, 4, 8, 8, 16, 0.35, 500, 50.0, None),
])

# sizes the tensor-core tiles take (multiples of 16), recurrent heads of 64 and 128 channels, windows of 65
# and 64 around a page border, a shared latent right behind its source
K_C = dict(architecture="Kesedra", vocab=257, width=128, embedding=dict(scale=11.0), norm=dict(eps=1e-5), layers=[
    wkv(2, 64, 16, dense(192)),
    latent(4, 32, 32, 32, 64, 64, 0.125, 65, 10000.0, moe(8, 2, 64, 1.5)),
    latent(4, 32, 32, 64, 32, 64, 0.125, 64, 10000.0, moe(8, 3, 32, 1.5), kv_from=1),
    wkv(1, 128, 16, dense(64)),
])

TINY_K = {"KA": K_A, "KB": K_B, "KC": K_C}


def make_kesedra_folder(tmp_path, name, seed=0, dtype=torch.float32):
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    path = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    write_model_folder(path, config_from_dict(TINY_K[name]), seed, dtype)
    # The library draws matrices from N(0, 0.02): with those every score is near 0, every softmax near
    # uniform, every clamp idle and every decay the same, and a wrong key, a lost state or a window that is
    # one token off would hardly show.  Larger matrices give scores of order one, experts that reach their
    # limits and routers that decide; decay offsets spread from short to long memory.
    from safetensors.torch import load_file, save_file

    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for key, value in tensors.items():
        v = value.float()
        if key == "embed":
            v = v * (150.0 / TINY_K[name]["embedding"]["scale"])      # rows of about 3 a channel once scaled
        elif key.endswith((".uq", ".uk")):
            v = v * 12.0
        elif key.endswith(".router"):
            v = v * 40.0
        elif key.endswith(".w0"):
            v = torch.linspace(-5.0, 0.5, v.numel()).reshape(v.shape) + v
        elif key.endswith((".mix.k", ".mix.v", ".mix.r")):
            v = v * 6.0
        elif key.endswith(".u"):
            v = v * 5.0
        elif value.dim() == 2:
            v = v * 4.0
        elif key.endswith(".b"):
            v = v * 10.0
        tensors[key] = v.to(value.dtype)
    save_file(tensors, file, metadata={"format": "pt"})
    if name == "KB":
        # this folder leaves the rank of the decay matrices to the checkpoint's shapes
        import json

        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as handle:
            raw = json.load(handle)
        for layer in raw["layers"]:
            layer["mixer"].pop("decay_rank", None)
        with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as handle:
            json.dump(raw, handle, indent=1, sort_keys=True)
    return path
