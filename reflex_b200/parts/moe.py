"""Mixture-of-experts feed-forward with top-k routing.

Router logits z = W_r x (+ b), 32-bit; the `top` experts with the largest
logits are chosen (ties: the lower index) and weighted by the softmax over the
chosen logits only; an expert is W_down act(W_up x) without biases, act the
square of relu ("relu2") or silu; the output is the weighted sum of the chosen
experts' outputs, summed in the order of their rank in 32-bit, so a row's
result does not depend on what else is in the batch.  The experts' matrices
are stacked at load: up [experts, ff, hidden], down [experts, hidden, ff].
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import FeedForwardSpec
from .registry import TensorInfo, register_feed_forward


@register_feed_forward("moe")
class MixtureOfExperts:
    capturable = True  # routing stays on the device: ids and weights are read by the expert kernels

    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.experts = int(spec.param("experts"))
        self.top = int(spec.param("top"))
        self.activation = str(spec.param("activation", "relu2"))
        self.router = self.router_bias = self.up = self.down = None

    @classmethod
    def tensor_specs(cls, spec: FeedForwardSpec) -> Dict[str, TensorInfo]:
        H, I, E = spec.hidden_size, spec.intermediate_size, int(spec.param("experts"))
        out = {"router": TensorInfo((E, H), "matrix")}
        if spec.param("router_bias", False):
            out["router_bias"] = TensorInfo((E,), "bias")
        for e in range(E):  # role#index: the checkpoint names every expert's tensors
            out[f"expert_up#{e}"] = TensorInfo((I, H), "matrix")
            out[f"expert_down#{e}"] = TensorInfo((H, I), "matrix")
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        self.router = dev(tensors["router"]).contiguous()
        b = tensors.get("router_bias")
        self.router_bias = None if b is None else b.to(device=self.device, dtype=torch.float32).contiguous()
        self.up = torch.stack([dev(tensors[f"expert_up#{e}"]) for e in range(self.experts)]).contiguous()
        self.down = torch.stack([dev(tensors[f"expert_down#{e}"]) for e in range(self.experts)]).contiguous()

    def forward(self, x, residual=None):
        logits = ops.linear(x, self.router, out_dtype=torch.float32)
        ids, wts = ops.moe_route(logits, self.router_bias, self.top)
        ops.prof_mark("moe_router")
        out = ops.moe_experts(x, self.up, self.down, ids, wts, self.activation)
        ops.prof_mark("moe_experts")
        return out
