"""Grouped-query attention whose q, k and v pass a short causal convolution,
with a query temperature, a linear distance bias and a sink.

With h the mixer's input [rows, hidden]:
  q = conv(W_q h + b_q), k = conv(W_k h + b_k), v = conv(W_v h + b_v)
      one filter a channel over the last `taps` tokens, zeros before the start
  q_p <- q_p * (1 + coef * ln(floor((p + 1) / every) + 1))          position p
  s_ij = (q_i . k_j) * scale - slope_h * (i - j)   for j <= i (and in the window)
      slope_h = 2^(-e (h + 1) / heads) for head h
  p = exp(s) / (sum_j exp(s_ij) + exp(sink_h))     the sink has no key and no value
  out = W_o concat_h(sum_j p_ij v_j) + b_o
There is no rotation: positions enter through the temperature and the bias
alone.  The convolved k and v are what the paged cache holds; the last
taps - 1 projected rows of q, k and v are a state of fixed size beside it.
Key and value heads may differ in size: both are stored `pad` wide (the larger
of the two, rounded up to 16, zeros beyond), q and the output projection's
columns are padded alike, and one attention kernel serves both.  Projections
leave the product as 32-bit values; convolution, temperature, scores and
softmax are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import KVSpec, StateSpec
from ..config.spec import MixerSpec
from ..errors import InvalidInput
from .registry import TensorInfo, register_mixer


@register_mixer("conv_attention")
class ConvAttention:
    capturable = True  # positions, slots and the page table are read from device memory

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        if spec.num_heads % spec.num_kv_heads:
            raise InvalidInput("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.taps = int(spec.param("taps", 1))
        self.has_bias = bool(spec.param("bias", False))
        self.has_sink = bool(spec.param("sink", False))
        self.temp_coef = float(spec.param("temp_coef", 0.0))
        self.temp_every = int(spec.param("temp_every", 1))
        H, G, d, dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        self.channels = H * d + G * (d + dv)
        self.pad = (max(d, dv) + 15) // 16 * 16
        e = spec.param("distance_slope_exponent")
        self.slopes = None
        if e is not None:
            self.slopes = torch.tensor([2.0 ** (-float(e) * (h + 1) / H) for h in range(H)],
                                       dtype=torch.float32, device=device)
        self.qkv = self.bias = self.filters = self.sink = self.o = self.o_bias = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, H, G, d, dv = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        taps = int(spec.param("taps", 1))
        out = {
            "q_proj": TensorInfo((H * d, W), "matrix"), "k_proj": TensorInfo((G * d, W), "matrix"),
            "v_proj": TensorInfo((G * dv, W), "matrix"), "o_proj": TensorInfo((W, H * dv), "matrix"),
            "q_conv": TensorInfo((H * d, taps), "filter"), "k_conv": TensorInfo((G * d, taps), "filter"),
            "v_conv": TensorInfo((G * dv, taps), "filter"),
        }
        if spec.param("bias", False):
            out.update({"q_bias": TensorInfo((H * d,), "bias"), "k_bias": TensorInfo((G * d,), "bias"),
                        "v_bias": TensorInfo((G * dv,), "bias"), "o_bias": TensorInfo((W,), "bias")})
        if spec.param("sink", False):
            out["sink"] = TensorInfo((H,), "bias")
        return out

    def cache_spec(self):
        kv = KVSpec(self.spec.num_kv_heads, self.pad, self.spec.window)
        if self.taps <= 1:
            return kv
        return (kv, StateSpec((self.taps - 1, self.channels), "float32"))

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        H, dv, pad = s.num_heads, s.value_dim, self.pad

        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.qkv = torch.cat([dev(tensors[k]) for k in ("q_proj", "k_proj", "v_proj")], dim=0).contiguous()
        # transposed, [taps, channels]: neighbouring channels' taps side by side
        self.filters = torch.cat([f32(tensors[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()
        if self.has_bias:
            self.bias = torch.cat([f32(tensors[k]) for k in ("q_bias", "k_bias", "v_bias")]).contiguous()
            self.o_bias = f32(tensors["o_bias"])
        self.sink = f32(tensors["sink"]) if self.has_sink else None
        o = dev(tensors["o_proj"])
        if pad != dv:  # the attention's heads come out `pad` wide: zero columns for what lies beyond the values
            wide = torch.zeros((o.shape[0], H, pad), dtype=o.dtype, device=o.device)
            wide[:, :, :dv] = o.view(o.shape[0], H, dv)
            o = wide.view(o.shape[0], H * pad)
        self.o = o.contiguous()

    def input_weight(self):
        """The matrix of the mixer's first product, for a caller that stacks it with
        others of the same input; `adopt_input_weight` hands back this mixer's rows of
        the stacked matrix, so that the weights are held once."""
        return self.qkv

    def adopt_input_weight(self, rows: torch.Tensor) -> None:
        self.qkv = rows

    def forward(self, x, ctx, proj=None):
        """-> (W_o attention, b_o): the output projection's bias is left to the
        caller's next kernel (None when the mixer has none).  `proj` = (float32
        rows, first column): the first product, already made by the caller as part
        of a stacked one."""
        s = self.spec
        kv, batch = ctx.kv, ctx.batch
        state = ctx.state if self.taps > 1 else None
        state2d = state.view(state.shape[0], -1) if state is not None else None
        if proj is None:
            proj, col0 = ops.linear(x, self.qkv, out_dtype=torch.float32), 0
            ops.prof_mark("qkv_gemm")
        else:
            proj, col0 = proj
        q = ops.conv_qkv_post(proj, self.bias, self.filters, state2d, batch, kv.k_pages, kv.v_pages,
                              kv.page_table, kv.page_size, s.num_heads, s.num_kv_heads, s.head_dim,
                              s.value_dim, self.pad, self.temp_coef, self.temp_every, ctx.writes_cache,
                              self.dtype, col0=col0)
        if state2d is not None:
            ops.conv_state_update(proj, col0, self.channels, self.bias, self.taps, state2d, batch)
        ops.prof_mark("conv_post")
        attn = ops.attention(q, kv.k_pages, kv.v_pages, kv.page_table, kv.page_size, batch, s.num_heads,
                             s.num_kv_heads, self.pad, s.window, s.scale, sink=self.sink, slopes=self.slopes)
        ops.prof_mark("attn")
        out = ops.linear(attn, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out, self.o_bias
