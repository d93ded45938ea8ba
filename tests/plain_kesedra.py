"""A plain statement of the Kesedra decoder: whole sequences, no cache, no batches, float64, one
function per mechanism.  It shares no code with the package and is slow on purpose.

The design: an embedding times a constant; layers ``x + post_norm(sublayer(pre_norm(x)))`` with RMS
norms whose gain is stored around zero; two mixers (a linear recurrence with a per-channel decay
that depends on the token, and attention over a low-rank latent with a shared rotated key part and a
sliding window, which may read the latent another layer cached); two feed-forwards (dense with
squared relu and biases, and a routed mixture of small clamped gated experts); a final norm and a
separate output head.
"""

import json
import math
import os

import torch

F = torch.float64


def read_model_folder(path):
    """(config dict, {name: float64 tensor})."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as handle:
        cfg = json.load(handle)
    weights = {k: v.to(F) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, weights


# ------------------------------------------------------------------------------------------ norms

def rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The layer norms and the final norm: the stored weight is the gain minus one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain_gain(x, w, eps):
    """The norms inside the latent attention: the stored weight is the gain."""
    return rms(x, eps) * w


# ------------------------------------------------------------------------------------------ rotation

def rotate_interleaved(x, positions, base, dims):
    """Turns the first ``dims`` entries of the last dimension of ``x`` ``[T, ..., D]``: entry ``2i``
    with entry ``2i + 1`` by the angle ``p * base ** (-2i / dims)``."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(F)[:, None] * freq[None, :]                # [T, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().reshape(shape), angle.sin().reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


# ------------------------------------------------------------------------------------------ recurrence

def shifted(h):
    """Every row's predecessor; zeros before the first."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def wkv_decay(mix_w, w, p):
    """Per head and key channel, in (0, 1): ``exp(-exp(w2 tanh(w1 m) + w0))``."""
    return torch.exp(-torch.exp(torch.tanh(mix_w @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))


def wkv_recurrence(r, k, v, decay, u):
    """``[T, H, D]`` each, ``u`` ``[H, D]``.  Token by token with a state ``S`` ``[H, D(key), D(value)]``
    that starts at zero: the output reads the state before this token plus this token's own
    ``k v^T`` weighted by ``u``; then the state decays per key channel and takes ``k v^T``."""
    T, H, D = r.shape
    S = torch.zeros(H, D, D, dtype=F)
    out = torch.zeros(T, H, D, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    return out


def wkv_mixer(h, w, p, m, eps):
    """``h`` ``[T, width]``: the normed input of one sequence from its first token on."""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    prev = shifted(h)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).reshape(T, H, D)
    k = (mix["k"] @ w[p + "k"].T).reshape(T, H, D)
    v = (mix["v"] @ w[p + "v"].T).reshape(T, H, D)
    g = mix["g"] @ w[p + "g"].T
    gate = g * torch.sigmoid(g)
    decay = wkv_decay(mix["w"], w, p).reshape(T, H, D)
    o = wkv_recurrence(r, k, v, decay, w[p + "u"])
    o = rms(o, eps).reshape(T, H * D) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ latent attention

def latent_of(h, w, p, m, eps, positions):
    """What a layer with its own down-projection caches for ``h``: the normed latent ``[T, kv_rank]``
    and the rotated key part ``[T, rot_dim]`` that all heads share."""
    down = h @ w[p + "dkv"].T
    c = norm_plain_gain(down[:, : m["kv_rank"]], w[p + "dkv.norm"], eps)
    shared = rotate_interleaved(down[:, m["kv_rank"]:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, shared


def latent_attention(h, w, p, m, eps, latent):
    """``latent`` = (c, shared rotated key part), this layer's own or another layer's."""
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    c, shared = latent
    cq = norm_plain_gain(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    q_plain = q[:, :, :D]
    q_turned = rotate_interleaved(q[:, :, D:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    value = (c @ w[p + "uv"].T).reshape(T, H, V)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain)
              + torch.einsum("thr,sr->hts", q_turned, shared)) * m["scale"]
    i = positions[:, None]
    j = positions[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~seen[None], -math.inf)
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shv->thv", weights, value).reshape(T, H * V)
    return out @ w[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forwards

def dense_feed_forward(h, w, p):
    a = torch.relu(h @ w[p + "up"].T + w[p + "up.b"])
    return (a * a) @ w[p + "down"].T + w[p + "down.b"]


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, top):
    """(indices ``[T, top]``, weights ``[T, top]``): the largest logits, softmax over those alone."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    best = torch.topk(z, top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def routed_feed_forward(h, w, p, mlp, chosen=None):
    """``chosen`` (``[T, top]``): use these experts instead of the largest logits (their weights are still
    the softmax over their own logits); for comparisons in which a near-tie may fall either way."""
    index, weight = route(h, w, p, mlp["router"]["top"])
    if chosen is not None:
        z = h @ w[p + "router"].T + w[p + "router.b"]
        index = torch.as_tensor(chosen).long()
        weight = torch.softmax(z.gather(1, index), dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(index[t].tolist(), weight[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


# ------------------------------------------------------------------------------------------ the model

def forward(cfg, w, tokens, layers_out=None, routes=None):
    """Logits ``[T, vocab]`` of one sequence from its first token; ``layers_out`` (a list) receives the
    residual stream after every layer; ``routes`` ({layer: ``[T, top]``}) fixes the experts of routed layers."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = norm_around_zero(x, w[p + "norm1"], eps)
        if layer["type"] == "wkv":
            y = wkv_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                latents[i] = latent_of(h, w, p + "mix.", m, eps, positions)
                source = i
            y = latent_attention(h, w, p + "mix.", m, eps, latents[source])
        else:
            raise ValueError(layer["type"])
        x = x + norm_around_zero(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_around_zero(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = dense_feed_forward(h, w, p + "mlp.")
            else:
                y = routed_feed_forward(h, w, p + "mlp.", mlp, None if routes is None else routes.get(i))
            x = x + norm_around_zero(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T


def generate(cfg, w, prompt, n):
    """Greedy continuation: ``n`` tokens, each the largest logit (the lowest index among equals)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
