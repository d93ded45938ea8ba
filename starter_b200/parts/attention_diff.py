"""Differential attention over the paged cache: two softmax maps per head, subtracted.

One step of it: one stacked product gives ``[q | gate | k | v]``; ``ops.diff_prepare`` adds the
biases, scales the queries by their temperature and files keys and values at each token's own
position; the attention kernel forms both maps over the cached keys, ``a1 - lambda * a2``, the
head's unit norm, the factor ``1 - lambda_init`` and the sigmoid gate; the output projection
follows.  A whole prompt, a later chunk and a single token are the same code: every query is told
its absolute position.

A layer whose spec says ``own_kv = False`` has no key and value projections: the run order gives it
the cache entry of the layer whose keys and values it uses (``writes_cache`` false), and it only
projects queries and the gate.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.layout import KVNeed
from .base import ParamSpec, Part, bytes_of


class DifferentialAttention(Part):
    #: the output projection's bias can be left to whoever adds the output to the residual stream
    can_defer_bias = True

    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads")
        if 2 * spec.head_dim > ops.DIFF_MAX_ROW or spec.value_dim > ops.DIFF_MAX_ROW:
            raise ValueError(f"2 * head_dim = {2 * spec.head_dim} and value_dim = {spec.value_dim} must be at "
                             f"most {ops.DIFF_MAX_ROW}")
        if position is not None or spec.position is not None:
            raise ValueError("differential attention here takes no rotation")
        self.q_size = spec.num_heads * 2 * spec.head_dim
        self.gate_size = spec.num_heads * spec.value_dim if spec.gated else 0
        self.k_size = spec.num_kv_heads * 2 * spec.head_dim
        self.v_size = spec.num_kv_heads * spec.value_dim
        self.out_size = spec.num_heads * spec.value_dim
        self.deferred_bias = None
        self.lam = None

    # what this mixer keeps per sequence: a key row of both maps and a value row per key/value head
    def kv_need(self):
        if not self.spec.own_kv:
            return None
        return KVNeed(self.spec.num_kv_heads, 2 * self.spec.head_dim, self.spec.window, self.spec.value_dim)

    def state_need(self):
        return None

    def param_specs(self):
        s = self.spec
        out = {"q": ParamSpec((self.q_size, s.hidden_size)), "o": ParamSpec((s.hidden_size, self.out_size))}
        if s.gated:
            out["g"] = ParamSpec((self.gate_size, s.hidden_size))
        if s.own_kv:
            out["k"] = ParamSpec((self.k_size, s.hidden_size))
            out["v"] = ParamSpec((self.v_size, s.hidden_size))
        if s.bias:
            out["q_bias"] = ParamSpec((self.q_size,), "bias32")
            out["o_bias"] = ParamSpec((s.hidden_size,), "bias32")
            if s.own_kv:
                out["k_bias"] = ParamSpec((self.k_size,), "bias32")
                out["v_bias"] = ParamSpec((self.v_size,), "bias32")
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = ParamSpec((s.head_dim,), "vector32")
        return out

    def set_params(self, params):
        s = self.spec
        # one product instead of up to four: [q | gate | k | v]; every output is the same dot product
        rows = [params["q"]] + ([params["g"]] if s.gated else []) + ([params["k"], params["v"]] if s.own_kv else [])
        self.weight = torch.cat(rows, dim=0).contiguous()
        self.o = params["o"].contiguous()
        self.bias = None
        if s.bias:
            dev = params["q_bias"].device
            parts = [params["q_bias"].float()]
            if s.gated:
                parts.append(torch.zeros(self.gate_size, dtype=torch.float32, device=dev))
            if s.own_kv:
                parts += [params["k_bias"].float(), params["v_bias"].float()]
            self.bias = torch.cat(parts).contiguous()
            self.deferred_bias = params["o_bias"].float().contiguous()
        # a single lambda serves every head of the layer; it is formed in float32, as its vectors are
        f = lambda name: params[name].float()  # noqa: E731
        lam = torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum())
        self.lam = float(lam.item()) + float(s.lambda_init)
        self._lambda_vectors = [params[n] for n in ("lq1", "lk1", "lq2", "lk2")]

    def prepare(self, max_position: int) -> bool:
        return False

    def __call__(self, x, ctx, entry, writes_cache=True, defer_bias=False):
        s = self.spec
        if writes_cache and not s.own_kv:
            raise ValueError("a differential attention without key and value projections cannot fill a cache entry")
        cache = ctx.cache
        keys, values = cache.entry_pages(entry)
        weight, bias = self.weight, self.bias
        if s.own_kv and not writes_cache:             # its own projections exist but another entry is read
            weight = weight[: self.q_size + self.gate_size]
            bias = bias[: self.q_size + self.gate_size] if bias is not None else None
        proj = ops.linear(x, weight, status=ctx.status)
        temp = (s.q_temperature.coef, s.q_temperature.every) if s.q_temperature is not None else None
        q = ops.diff_prepare(proj, bias, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, self.gate_size,
                             temp, ctx.tok_pos, ctx.tok_slot, cache.block_table, keys, values,
                             write_cache=writes_cache)
        gate = proj[:, self.q_size:self.q_size + self.gate_size] if s.gated else None
        a = ops.diff_attention_step(q, gate, keys, values, cache.block_table, ctx, s.num_heads, s.num_kv_heads,
                                    s.head_dim, s.value_dim, s.scale, self.lam, 1.0 - s.lambda_init, s.norm_eps,
                                    s.window)
        y = ops.linear(a, self.o, status=ctx.status)
        if self.deferred_bias is not None and not defer_bias:
            y = ops.add_bias(y, self.deferred_bias)
        return y

    def weight_bytes(self):
        return bytes_of(self.weight, self.o, self.bias, self.deferred_bias)
