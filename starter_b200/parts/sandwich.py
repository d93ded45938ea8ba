"""Layers with a norm in front of AND behind each sublayer, around a residual stream kept in float32:
``x <- x + norm1b(mixer(norm1(x)))``, then ``x <- x + norm2b(feed_forward(norm2(x)))``.

The sum that closes one sublayer and the norm that opens the next are one kernel
(``ops.residual_norm``), as the residual sum and the norm after it are one kernel for the pre-norm
block: a sublayer's output stays ``Unsummed`` (with the norm that is to be applied to it, and a bias a
part left for the kernel to add) until the next sublayer, or the model's end, takes it.
"""

from __future__ import annotations

from dataclasses import dataclass

from .. import ops


@dataclass
class Unsummed:
    """A sublayer's output not yet normed and added onto the residual stream."""

    value: object
    norm: object          # the norm behind the sublayer (its ``weight`` is the float32 gain, its spec has eps)
    bias: object = None

    def for_kernel(self):
        return self.value, self.norm.weight, self.bias, self.norm.spec.eps


def open_sublayer(residual, pending, norm, dtype):
    """Add ``pending`` (an ``Unsummed`` or None) onto ``residual`` in place and return ``norm`` of the sum in
    ``dtype``."""
    return ops.residual_norm(residual, dtype, norm.spec.eps, pending.for_kernel() if pending is not None else None,
                             norm.weight)


def close_rows32(residual, pending, rows, norm, dtype):
    """The model's end for the rows asked for: the last open sum and the final norm, without touching
    ``residual``."""
    return ops.residual_norm(residual, dtype, norm.spec.eps, pending.for_kernel() if pending is not None else None,
                             norm.weight, rows=rows)


class SandwichBlock:
    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm1b": "norm",
                "norm2": "norm", "norm2b": "norm"}
    #: what the model makes the residual stream of: float32 rows from ``ops.embedding32``
    residual_kind = "float32"

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.norm1, self.norm1b = parts["norm1"], parts["norm1b"]
        self.norm2, self.norm2b = parts.get("norm2"), parts.get("norm2b")
        for norm in (self.norm1, self.norm1b, self.norm2, self.norm2b):
            if norm is not None and getattr(norm.spec, "kind", None) != "rmsnorm":
                raise ValueError("the sandwich arrangement fuses RMS norms; got " + repr(norm.spec))

    def parts(self) -> dict:
        return dict(self._parts)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        dtype = self.mixer.dtype
        n = open_sublayer(residual, pending, self.norm1, dtype)
        pending = Unsummed(self.mixer(n, ctx, entry, writes_cache), self.norm1b)
        if self.feed_forward is None:
            return residual, pending
        m = open_sublayer(residual, pending, self.norm2, dtype)
        if getattr(self.feed_forward, "can_defer_bias", False):
            y = self.feed_forward(m, ctx, defer_bias=True)
            return residual, Unsummed(y, self.norm2b, self.feed_forward.deferred_bias)
        return residual, Unsummed(self.feed_forward(m, ctx), self.norm2b)


class SandwichMixerOnlyBlock(SandwichBlock):
    """The same layer without a feed-forward (and so without the second pair of norms)."""

    FAMILIES = {"mixer": "mixer", "norm1": "norm", "norm1b": "norm"}
