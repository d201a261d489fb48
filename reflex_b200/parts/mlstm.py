"""mLSTM: a matrix memory per head with exponential gates.

With h the mixer's input, per head: q = W_q h * scale, k = W_k h, v = W_v h,
log input gate i = cap tanh((W_i h + b_i) / cap), log forget gate
f = logsigmoid(cap tanh((W_f h + b_f) / cap)), and with a running maximum m
(zero at a sequence's start):
  m_t = max(f_t + m_{t-1}, i_t)
  S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T
  n_t = e^(f_t + m_{t-1} - m_t) n_{t-1} + e^(i_t - m_t) k_t
  o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
then each head's o over its root mean square, times a weight, times
sigmoid(W_g h), then W_o.  (S, n, m) is the sequence's state, 32-bit, carried
from step to step in the cache's state group.  All six projections are one
product whose result stays 32-bit; the recurrence and everything after it up
to the output projection's input are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import MixerSpec
from .registry import TensorInfo, register_mixer

DENOMINATOR_GUARD = 1e-6  # fixed by the design (the kernel holds the same constant)


@register_mixer("mlstm")
class MLSTM:
    capturable = True  # sequences' slots and rows are read from device memory
    supports_fused_residual = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.cap = float(spec.param("gate_cap"))
        self.eps = float(spec.param("eps"))
        self.stacked = self.o = self.norm = self.bias_i = self.bias_f = None
        H, d, dv = spec.num_heads, spec.head_dim, spec.value_dim
        # columns of the stacked product: q, k, v, output gate, i, f
        self.q_off, self.k_off, self.v_off = 0, H * d, 2 * H * d
        self.g_off = 2 * H * d + H * dv
        self.i_off = self.g_off + H * dv
        self.f_off = self.i_off + H

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, H, d, dv = spec.hidden_size, spec.num_heads, spec.head_dim, spec.value_dim
        return {
            "q_proj": TensorInfo((H * d, W), "matrix"), "k_proj": TensorInfo((H * d, W), "matrix"),
            "v_proj": TensorInfo((H * dv, W), "matrix"), "gate": TensorInfo((H * dv, W), "matrix"),
            "o_proj": TensorInfo((W, H * dv), "matrix"), "norm": TensorInfo((H * dv,), "norm"),
            "i_proj": TensorInfo((H, W), "matrix"), "i_bias": TensorInfo((H,), "bias"),
            "f_proj": TensorInfo((H, W), "matrix"), "f_bias": TensorInfo((H,), "bias"),
        }

    def cache_spec(self) -> StateSpec:
        s = self.spec
        return StateSpec((s.num_heads, ops.mlstm_state_floats(s.head_dim, s.value_dim)), "float32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.stacked = torch.cat([dev(tensors[k]) for k in
                                  ("q_proj", "k_proj", "v_proj", "gate", "i_proj", "f_proj")], dim=0).contiguous()
        self.o = dev(tensors["o_proj"]).contiguous()
        self.norm = f32(tensors["norm"])
        self.bias_i, self.bias_f = f32(tensors["i_bias"]), f32(tensors["f_bias"])

    def forward(self, x, ctx, residual=None):
        s = self.spec
        H, d, dv = s.num_heads, s.head_dim, s.value_dim
        proj = ops.linear(x, self.stacked, out_dtype=torch.float32)
        ops.prof_mark("qkv_gemm")
        num, den = ops.mlstm_scan(proj, (self.q_off, self.k_off, self.v_off, self.i_off, self.f_off),
                                  self.bias_i, self.bias_f, self.cap, s.scale, ctx.batch, ctx.state, H, d, dv,
                                  max_rows=ctx.batch.max_new)
        ops.prof_mark("mlstm_scan")
        o = ops.mlstm_out(num, den, proj, self.g_off, self.norm, self.eps, H, dv, self.dtype)
        ops.prof_mark("mlstm_out")
        if residual is not None:
            fused = ops.linear_residual(o, self.o, residual[0], residual[1])
            if fused is not None:
                ops.prof_mark("o_proj")
                return None if fused is ops.ADDED else fused
        out = ops.linear(o, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
