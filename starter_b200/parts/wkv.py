"""A linear recurrence with a matrix state per head and a token-dependent decay (the time mixing of the
RWKV family), with its state in the cache's per-sequence slots.

One step of it: ``ops.token_shift`` forms the five mixes of each token's input with its predecessor's
(the predecessor of a portion's first token is what the sequence left in its slot); receptance, key,
value and gate are projections of their mixes; the decay goes through two small matrices with a tanh
between them, comes back in float32 and becomes ``exp(-exp(. + w0))`` there; ``ops.wkv_scan`` walks the tokens each sequence brings, from the
state in its slot and back into it, and applies the head norm, the gain and the gate; the output
projection follows.  A whole prompt, a later portion and a single token are the same code, and a step
captured in a CUDA graph too: everything the kernels need is in the step's device arrays.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.layout import StateNeed
from .base import ParamSpec, Part, bytes_of

SHIFTS = ("r", "k", "v", "g", "w")


class WkvMixer(Part):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if position is not None:
            raise ValueError("the recurrent mixer takes no position part")
        self.inner = spec.num_heads * spec.head_dim

    def kv_need(self):
        return None

    def state_need(self):
        """Per sequence: the last token's mixer input, then every head's state (32-bit, zero at the start)."""
        s = self.spec
        return StateNeed((s.hidden_size + s.num_heads * s.head_dim * s.head_dim,), "float32")

    def param_specs(self):
        s = self.spec
        out = {f"mu_{name}": ParamSpec((s.hidden_size,), "shift") for name in SHIFTS}
        for name in ("r", "k", "v", "g"):
            out[name] = ParamSpec((self.inner, s.hidden_size))
        out["w1"] = ParamSpec((s.decay_rank, s.hidden_size))
        out["w2"] = ParamSpec((self.inner, s.decay_rank))
        out["w0"] = ParamSpec((self.inner,), "vector32")
        out["u"] = ParamSpec((s.num_heads, s.head_dim), "vector32")
        out["norm"] = ParamSpec((self.inner,), "gain32")
        out["o"] = ParamSpec((s.hidden_size, self.inner))
        return out

    def set_params(self, params):
        self.mu = torch.stack([params[f"mu_{name}"].float() for name in SHIFTS]).contiguous()
        self.r, self.k, self.v, self.g = (params[n].contiguous() for n in ("r", "k", "v", "g"))
        self.w1, self.w2, self.o = params["w1"].contiguous(), params["w2"].contiguous(), params["o"].contiguous()
        self.w0 = params["w0"].float().contiguous()
        self.u = params["u"].float().contiguous()
        self.gain = params["norm"].float().contiguous()

    def prepare(self, max_position: int) -> bool:
        return False

    def __call__(self, x, ctx, entry, writes_cache=True):
        s = self.spec
        state = ctx.cache.entry_state(entry)
        if state is None or not writes_cache:
            raise ValueError("the recurrent mixer needs a state of its own in the cache")
        mixes = ops.token_shift(x, state, self.mu, ctx.tok_slot)
        r = ops.linear(mixes[0], self.r, status=ctx.status)
        k = ops.linear(mixes[1], self.k, status=ctx.status)
        v = ops.linear(mixes[2], self.v, status=ctx.status)
        g = ops.linear(mixes[3], self.g, status=ctx.status)
        inner = ops.bias_act(ops.linear(mixes[4], self.w1, status=ctx.status), None, "tanh")
        decay = ops.bias_act(ops.linear(inner, self.w2, out_float=True, status=ctx.status), self.w0, "decay")
        o = ops.wkv_scan(r, k, v, decay, self.u, g, self.gain, state, x, ctx.seq_slot,
                         ctx.seq_q_start, ctx.seq_q_len, s.num_heads, s.head_dim, s.norm_eps)
        return ops.linear(o, self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.mu, self.r, self.k, self.v, self.g, self.w1, self.w2, self.w0, self.u, self.gain, self.o)
