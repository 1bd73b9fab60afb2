"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)).

src/DotLLM.Models/Architectures/TransformerModel.cs:342-382 with the activation of
src/DotLLM.Cpu/Kernels/FusedOps.cs:33-78.  Gate and up are stacked into one matrix when the
weights are bound, so one product feeds the gating kernel.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .attention import BRANCH_DTYPE
from .base import FeedForward, WeightSpec, register_feed_forward


class GatedFeedForward(FeedForward):
    """params: ``intermediate_size``; ``activation``: "silu" (the fused products gate with it), or one of
    ``ops.GATINGS`` ("gelu_tanh", "clamped_sigmoid" with ``limit`` and ``alpha``), which gate in a kernel of
    their own behind the gate/up product; optional ``tensors``: the local names of the gate, up and down
    matrices (default the HuggingFace ones)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in ops.GATINGS:
            raise ConfigError(f"gated feed-forward: unsupported activation {self.activation!r}; known: {sorted(ops.GATINGS)}")
        self.limit = float(params.get("limit", 0.0))
        self.alpha = float(params.get("alpha", 1.0))
        names = params.get("tensors") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        self.gate_name, self.up_name, self.down_name = (str(n) for n in names)
        self.takes_scaled_rows = self.activation == "silu"      # x goes straight into the gate/up product
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {self.gate_name: WeightSpec((i, h)),
                self.up_name: WeightSpec((i, h)),
                self.down_name: WeightSpec((h, i))}

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.gate_name], tensors[self.up_name]], dim=0).contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x):
        gated = ops.gated_linear(x, self.w_gate_up, resident=True, kind=self.activation, limit=self.limit, alpha=self.alpha)
        return ops.linear(gated, self.w_down, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_feed_forward("gated_mlp", GatedFeedForward)
