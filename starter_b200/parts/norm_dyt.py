"""Dynamic Tanh in a norm's place: ``tanh(alpha * x) * weight + bias``, no mean and no variance."""

from __future__ import annotations

from .. import ops
from .base import ParamSpec, Part, bytes_of


class DynamicTanh(Part):
    """A member of the norm family (``__call__``, ``add``, ``add_rows`` as ``RMSNorm`` has them), so a
    single-stream block can use it; a block over several streams hands its parameters
    (``parameters()``) to the kernel that also reads the streams.  All three parameters are float32."""

    def param_specs(self):
        return {"weight": ParamSpec((self.spec.size,), "gain32"), "alpha": ParamSpec((), "slope"),
                "bias": ParamSpec((self.spec.size,), "bias32")}

    def set_params(self, params):
        self.weight = params["weight"].contiguous()
        self.alpha = params["alpha"].reshape(1).contiguous()
        self.bias = params["bias"].contiguous()

    def parameters(self):
        return self.alpha, self.weight, self.bias

    def __call__(self, x):
        return ops.dynamic_tanh(x, self.alpha, self.weight, self.bias)

    def add(self, residual, delta):
        if delta is None or delta is ops.ADDED:
            return ops.dynamic_tanh(residual, self.alpha, self.weight, self.bias)
        return ops.dynamic_tanh(residual, self.alpha, self.weight, self.bias, delta=delta)

    def add_rows(self, residual, delta, rows):
        if delta is ops.ADDED:
            delta = None
        return ops.dynamic_tanh(residual, self.alpha, self.weight, self.bias, delta=delta, rows=rows)

    def weight_bytes(self):
        return bytes_of(self.weight, self.alpha, self.bias)
