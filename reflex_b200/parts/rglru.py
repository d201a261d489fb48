"""A recurrent block around a real-gated linear recurrence.

With h the mixer's input [rows, hidden], `width` channels in `blocks` equal
parts:
  y = gelu_tanh(W_y h + b_y)
  u = conv(W_x h + b_x) + c       one filter a channel over the last `taps`
                                  tokens, zeros before the start
  r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)      per part b,
                                  A_b and I_b square matrices [out, in]
  log a = -c_decay * r * softplus(lam),  a = exp(log a)
  S_t = a S_(t-1) + sqrt(1 - a^2) * (i * u)        S = 0 before the first token
  out = W_o (S * y)
Per sequence the state is the last taps - 1 rows of W_x h + b_x and S, 32-bit,
one vector of the cache's state group.  Both projections are one product whose
result stays 32-bit; the convolution, the gates (their products too), the
decay and the recurrence are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import MixerSpec
from ..errors import InvalidInput
from .registry import TensorInfo, register_mixer


@register_mixer("rglru")
class GatedLinearRecurrence:
    capturable = True  # sequences' slots and rows are read from device memory

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.width = int(spec.param("width"))
        self.blocks = int(spec.param("blocks"))
        self.taps = int(spec.param("taps", 1))
        self.decay_scale = float(spec.param("decay_scale", 8.0))
        if self.width % self.blocks:
            raise InvalidInput("rglru: width must be a multiple of blocks")
        self.yx = self.y_bias = self.x_bias = self.filters = self.conv_bias = None
        self.gates = self.gates_lo = self.gate_a_bias = self.gate_i_bias = self.lam = self.o = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, Wr, B = spec.hidden_size, int(spec.param("width")), int(spec.param("blocks"))
        taps, K = int(spec.param("taps", 1)), int(spec.param("width")) // int(spec.param("blocks"))
        return {
            "y_proj": TensorInfo((Wr, W), "matrix"), "y_bias": TensorInfo((Wr,), "bias"),
            "x_proj": TensorInfo((Wr, W), "matrix"), "x_bias": TensorInfo((Wr,), "bias"),
            "conv": TensorInfo((Wr, taps), "filter"), "conv_bias": TensorInfo((Wr,), "bias"),
            "gate_a": TensorInfo((B, K, K), "matrix"), "gate_a_bias": TensorInfo((B, K), "bias"),
            "gate_i": TensorInfo((B, K, K), "matrix"), "gate_i_bias": TensorInfo((B, K), "bias"),
            "lam": TensorInfo((Wr,), "bias"), "o_proj": TensorInfo((W, Wr), "matrix"),
        }

    def cache_spec(self) -> StateSpec:
        # [the last taps - 1 inputs of the convolution | S]
        return StateSpec((self.taps * self.width,), "float32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.yx = torch.cat([dev(tensors["y_proj"]), dev(tensors["x_proj"])], dim=0).contiguous()
        self.y_bias, self.x_bias = f32(tensors["y_bias"]), f32(tensors["x_bias"])
        self.filters, self.conv_bias = f32(tensors["conv"]).t().contiguous(), f32(tensors["conv_bias"])  # [taps, width]
        # a part's two gate matrices stacked, [blocks, 2K, K], 32-bit: one per-part product gives both
        self.gates = torch.cat([f32(tensors["gate_a"]), f32(tensors["gate_i"])], dim=1).contiguous()
        # the same in bfloat16 for prompts, where the product runs on the tensor cores with 32-bit
        # sums: exact for weights stored in bfloat16, u rounded once (a convolution's output)
        self.gates_lo = self.gates.to(torch.bfloat16) if self.dtype == torch.bfloat16 else None
        self.gate_a_bias = f32(tensors["gate_a_bias"]).reshape(-1)
        self.gate_i_bias = f32(tensors["gate_i_bias"]).reshape(-1)
        self.lam = f32(tensors["lam"])
        self.o = dev(tensors["o_proj"]).contiguous()

    def input_weight(self):
        """The matrix of the mixer's first product, for a caller that stacks it with
        others of the same input; `adopt_input_weight` hands back this mixer's rows of
        the stacked matrix, so that the weights are held once."""
        return self.yx

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.yx = rows

    def forward(self, x, ctx, proj=None):
        """`proj` = (float32 rows, first column): the first product, already made by
        the caller as part of a stacked one."""
        batch, state, Wr = ctx.batch, ctx.state, self.width
        if proj is None:
            proj, y0 = ops.linear(x, self.yx, out_dtype=torch.float32), 0  # [rows, y | x]
            ops.prof_mark("qkv_gemm")
        else:
            proj, y0 = proj
        x0 = y0 + Wr
        many = self.gates_lo is not None and x.shape[0] > ops.HEADS_LINEAR_MAX_ROWS
        u = ops.short_conv(proj, x0, Wr, self.x_bias, self.filters, self.conv_bias,
                           state if self.taps > 1 else None, batch, also_bf16=many)
        ops.prof_mark("conv_post")
        if many:
            u, u_lo = u
            gates = ops.heads_linear(u_lo, self.gates_lo, out_dtype=torch.float32)
        else:
            gates = ops.heads_linear(u, self.gates)  # [rows, blocks * 2K], 32-bit
        ops.prof_mark("rglru_gates")
        # the recurrence's kernel also stores the convolution's new last inputs (it runs after it)
        act = ops.rglru_scan(u, gates, self.gate_a_bias, self.gate_i_bias, self.lam, self.decay_scale, proj, y0,
                             self.y_bias, state, (self.taps - 1) * Wr, batch, self.blocks, self.dtype,
                             max_rows=batch.max_new, conv_tail=(x0, self.x_bias, self.taps, 0))
        ops.prof_mark("rglru_scan")
        out = ops.linear(act, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
