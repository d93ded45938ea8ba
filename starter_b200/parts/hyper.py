"""Hyper-connections: several residual streams per token, and how a sublayer reads and writes them.

A token has ``S`` streams ``x_1 .. x_S`` (float32 ``[tokens, S, hidden]``), all equal to its embedding
at the start.  A sublayer with this part's ``in`` ``[S]``, ``out`` ``[S]`` and ``mix`` ``[S, S]``
(indexed ``[from, to]``) reads ``u = sum_s in[s] * x_s``, computes ``y = sublayer(norm(u))`` and
writes every stream from the values before the update: ``x_t = sum_s mix[s, t] * x_s + out[t] * y``.  The
model's output is the sum of the streams.

The update that closes a sublayer and the read (and norm) that opens the next are one kernel
(``ops.hyper_step``), as the residual sum and the norm after it are one kernel for a single stream:
a sublayer's output stays ``Pending`` until the next read, or the model's end, applies it.
"""

from __future__ import annotations

from dataclasses import dataclass

from .. import ops
from .base import ParamSpec, Part, bytes_of


@dataclass
class Pending:
    """A sublayer's output not yet written to the streams, with the connection that will write it and
    a bias (float32 ``[hidden]`` or None) still to be added to the output."""

    value: object
    connection: object
    bias: object = None

    def for_kernel(self):
        c = self.connection
        return self.value, c.mix, c.out, self.bias


class HyperConnection(Part):
    def param_specs(self):
        s = self.spec.streams
        return {"in": ParamSpec((s,), "stream_weight"), "out": ParamSpec((s,), "stream_weight"),
                "mix": ParamSpec((s, s), "stream_weight")}

    def set_params(self, params):
        self.read = params["in"].contiguous()
        self.out = params["out"].contiguous()
        self.mix = params["mix"].contiguous()

    def open(self, streams, pending, norm, dtype):
        """Apply ``pending`` (a ``Pending`` or None) to ``streams`` in place and return this sublayer's
        normed input ``[tokens, hidden]`` in ``dtype``."""
        before = pending.for_kernel() if pending is not None else None
        fused = getattr(norm, "parameters", None)
        if fused is not None:
            return ops.hyper_step(streams, dtype, before, self.read, fused())
        return norm(ops.hyper_step(streams, dtype, before, self.read, None))

    def weight_bytes(self):
        return bytes_of(self.read, self.out, self.mix)


def close_rows(streams, pending, rows, norm, dtype):
    """The model's end for the rows asked for: the last pending update, the sum of the streams and the
    final norm, without touching ``streams``."""
    before = pending.for_kernel() if pending is not None else None
    fused = getattr(norm, "parameters", None)
    if fused is not None:
        return ops.hyper_step(streams, dtype, before, None, fused(), rows=rows)
    return norm(ops.hyper_step(streams, dtype, before, None, None, rows=rows))


class HyperPreNormBlock:
    """``y1 = mixer(norm1(read1(x)))`` written through connection 1, then the same with the
    feed-forward through connection 2.  ``residual`` is the streams tensor; ``pending`` a ``Pending``."""

    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm",
                "connection1": "connection", "connection2": "connection"}

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.norm1 = parts["norm1"]
        self.norm2 = parts.get("norm2")
        self.connection1 = parts["connection1"]
        self.connection2 = parts.get("connection2")

    def parts(self) -> dict:
        return dict(self._parts)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        dtype = self.mixer.dtype
        n = self.connection1.open(residual, pending, self.norm1, dtype)
        if getattr(self.mixer, "can_defer_bias", False):
            # the output projection's bias is added where the output is written to the streams
            a = self.mixer(n, ctx, entry, writes_cache, defer_bias=True)
            pending = Pending(a, self.connection1, self.mixer.deferred_bias)
        else:
            pending = Pending(self.mixer(n, ctx, entry, writes_cache), self.connection1)
        if self.feed_forward is None:
            return residual, pending
        m = self.connection2.open(residual, pending, self.norm2, dtype)
        return residual, Pending(self.feed_forward(m, ctx), self.connection2)


class HyperMixerOnlyBlock(HyperPreNormBlock):
    """The same layer without a feed-forward (and so without a second norm and connection)."""

    FAMILIES = {"mixer": "mixer", "norm1": "norm", "connection1": "connection"}
