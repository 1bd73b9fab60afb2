"""RMSNorm over the float32 residual stream.

y = x / sqrt(mean(x^2) + eps) * gain, eps inside the root, no mean subtraction, gain used as
is (src/DotLLM.Cpu/Kernels/RmsNorm.cs:22-51).  The fused form adds a pending branch output
to the stream first, as the reference's fused_add_rmsnorm does
(native/kernels/fused_add_rmsnorm.cu:9-72).
"""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, WeightSpec, register_norm


class RmsNorm(Norm):
    """params: ``eps``; optional ``gain_init`` for the random-weights mode; optional ``offset``: the stored
    tensor is the gain minus this number (1.0: a gain kept around zero, y = rms(x) * (1 + w); the sum is
    taken once, in float32, when the weights are bound); optional ``tensor``: the local name of the stored
    tensor (default "weight"; "" when the prefix is the whole name)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset", 0.0))
        self.tensor_name = str(params.get("tensor", "weight"))
        self.gain = None

    def weight_specs(self):
        default = ("ones",) if self.offset == 0.0 else ("normal", 0.1)
        return {self.tensor_name: WeightSpec((self.hidden_size,), "precise",
                                             tuple(self.params.get("gain_init", default)))}

    def bind(self, tensors):
        stored = tensors[self.tensor_name]
        self.gain = stored if self.offset == 0.0 else (stored + self.offset).contiguous()

    def branch(self, data):
        return ops.NormedBranch(data, self.gain, self.eps)

    def weight_bytes(self):
        return self.gain.numel() * self.gain.element_size()

    fuses_products = True

    def forward(self, x):
        return ops.add_rmsnorm(x, None, self.gain, self.eps, self.runtime.dtype)

    def add_forward(self, residual, delta, lazy=False):
        return ops.add_rmsnorm(residual, delta, self.gain, self.eps, self.runtime.dtype, lazy=lazy)


register_norm("rmsnorm", RmsNorm)
