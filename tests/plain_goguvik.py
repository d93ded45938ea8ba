"""A plain, slow statement of the Goguvik decoder: whole sequences, no cache, one function per mechanism.

It shares no code with ``starter_b200``: it reads ``config.json`` and ``model.safetensors`` with the
``json`` module and the ``safetensors`` package and computes with torch on the CPU, in float64 by
default (the oracle both number formats of the engine are held against).

Notation.  A token has S residual streams r[0..S-1], each a vector of the model's width, all equal to
its embedding at first.  A sublayer f with read weights a[S], write weights c[S] and a mixing matrix
M[S, S] (row = from, column = to) and the norm N does

    u = sum_s a[s] r[s];   y = f(N(u));   r'[t] = sum_s M[s, t] r[s] + c[t] y      (all t from the old r)

N is Dynamic Tanh: N(u) = tanh(alpha u) * w + b.  The mixer is differential attention: per query head
two maps over the same values, out = A1 V - lambda A2 V, divided by its root mean square over the
value size, times (1 - lambda0); lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + lambda0; the query at
position p is first scaled by 1 + coef ln(floor((p + 1) / every) + 1); the heads are gated by
sigmoid(G h) and projected.  A layer with ``kv_from`` attends over that earlier layer's keys and
values.  The feed-forward is D(gelu_tanh(Gt h) * (U h)).  The logits are E N_final(sum_s r[s]).
"""

from __future__ import annotations

import json
import math
import os

import torch


def read_model_folder(path, dtype=torch.float64):
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as handle:
        cfg = json.load(handle)
    weights = {k: v.to(dtype) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, weights


# --------------------------------------------------------------------------- mechanisms

def plain_dynamic_tanh(x, alpha, weight, bias):
    return torch.tanh(alpha * x) * weight + bias


def plain_gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def plain_gated_feed_forward(h, gate, up, down):
    return (plain_gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def plain_stream_read(streams, read):
    """``streams`` [T, S, W]; the weighted sum over S."""
    return torch.einsum("s,tsw->tw", read, streams)


def plain_stream_write(streams, y, mix, out):
    """Every new stream from the values before the update: new[t] = sum_s mix[s, t] old[s] + out[t] y."""
    return torch.einsum("sk,tsw->tkw", mix, streams) + out[None, :, None] * y[:, None, :]


def plain_query_temperature(positions, coef, every):
    return 1.0 + coef * torch.log(torch.floor((positions + 1) / every) + 1.0)


def plain_lambda(lq1, lk1, lq2, lk2, lambda0):
    return torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + lambda0


def plain_softmax_map(q, k, scale, q_positions, window=None):
    """Weights [Tq, Tk] of one map: the query at position p sees keys 0..p (the last ``window`` of
    them, when a window is given); ``k`` holds the keys of positions 0..Tk-1."""
    scores = (q @ k.T) * scale
    key_pos = torch.arange(k.shape[0])
    seen = key_pos[None, :] <= q_positions[:, None]
    if window is not None:
        seen &= key_pos[None, :] > q_positions[:, None] - window
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)


def plain_differential_head(q1, q2, k1, k2, v, scale, lam, lambda0, eps, q_positions, window=None):
    """One query head: [Tq, vdim]."""
    a1 = plain_softmax_map(q1, k1, scale, q_positions, window) @ v
    a2 = plain_softmax_map(q2, k2, scale, q_positions, window) @ v
    o = a1 - lam * a2
    o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
    return o * (1.0 - lambda0)


def plain_differential_attention(h, w, prefix, m, eps, kv, positions):
    """The whole mixer on ``h`` [T, W]; ``kv`` is ``(k, v)`` of an earlier layer or None; returns the
    output and the ``(k, v)`` it used."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    count = h.shape[0]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(count, heads, 2, dim)
    if kv is None:
        k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(count, groups, 2, dim)
        v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(count, groups, vdim)
    else:
        k, v = kv
    temp = m.get("q_temp")
    if temp:
        q = q * plain_query_temperature(positions.to(h.dtype), temp["coef"], temp["every"])[:, None, None, None]
    lam = plain_lambda(w[prefix + "lq1"], w[prefix + "lk1"], w[prefix + "lq2"], w[prefix + "lk2"], m["diff"])
    outs = []
    for head in range(heads):
        g = head // (heads // groups)
        outs.append(plain_differential_head(q[:, head, 0], q[:, head, 1], k[:, g, 0], k[:, g, 1], v[:, g],
                                            m["scale"], lam, m["diff"], eps, positions))
    o = torch.cat(outs, dim=-1) * torch.sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T + w[prefix + "o.b"], (k, v)


# --------------------------------------------------------------------------- the model

def plain_forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence."""
    dtype = w["embed"].dtype
    count = len(tokens)
    positions = torch.arange(count)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    streams = x[:, None, :].repeat(1, cfg["streams"], 1)
    eps = cfg["norm"]["eps"]
    kept = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        u = plain_stream_read(streams, w[p + "hc1.in"])
        n = plain_dynamic_tanh(u, w[p + "norm1.alpha"], w[p + "norm1"], w[p + "norm1.b"])
        source = m.get("kv_from")
        y, kv = plain_differential_attention(n, w, p + "mix.", m, eps, kept[source] if source is not None else None,
                                             positions)
        if source is None:
            kept[i] = kv
        streams = plain_stream_write(streams, y, w[p + "hc1.mix"], w[p + "hc1.out"])
        if layer.get("mlp"):
            u = plain_stream_read(streams, w[p + "hc2.in"])
            n = plain_dynamic_tanh(u, w[p + "norm2.alpha"], w[p + "norm2"], w[p + "norm2.b"])
            y = plain_gated_feed_forward(n, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
            streams = plain_stream_write(streams, y, w[p + "hc2.mix"], w[p + "hc2.out"])
        after.append(streams.sum(dim=1))
    final = plain_dynamic_tanh(streams.sum(dim=1), w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
    logits = (final @ w["embed"].T).to(dtype)
    return (logits, after) if return_layers else logits


def plain_generate(cfg, w, prompt, max_new_tokens):
    """Greedy continuation, the whole sequence computed anew for every token."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        token = int(torch.argmax(plain_forward(cfg, w, seq)[-1]))
        out.append(token)
        seq.append(token)
    return out
