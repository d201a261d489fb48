"""Latent attention: queries and keys/values through low-rank latents, only
the key/value latent cached.

With h the mixer's input [rows, hidden]:
  c_q = RMSNorm(W_dq h),  q = W_uq c_q             per head `head_dim` elements
  c   = RMSNorm(W_dkv h)                           `kv_rank` elements, cached
  k_j = W_uk c_j,  v_j = W_uv c_j                  per head, never materialised
  s_ij = (q_i . k_j) * scale  for 0 <= i - j < window
  p = exp(s) / (sum_j exp(s_ij) + exp(sink_h))     the sink has no key and no value
  out = W_o concat_h( sigmoid(W_g h)_h * sum_j p_ij v_j )
There is no position encoding.  Since k_j = W_uk c_j, the score is
(W_uk,h^T q_i) . c_j and the weighted values are W_uv,h (sum_j p_ij c_j): the
attention runs over the cached latents themselves as one shared key/value head
of `kv_rank` elements (keys and values are the same rows of the cache), with
the query folded through W_uk before it and W_uv applied after it, head by
head.  Norms, scores, the softmax and the gates are 32-bit.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.specs import KVSpec
from ..config.spec import MixerSpec
from .registry import TensorInfo, register_mixer


@register_mixer("latent_attention")
class LatentAttention:
    capturable = True  # positions, slots and the page table are read from device memory
    supports_fused_residual = True

    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.q_rank = int(spec.param("q_rank"))
        self.kv_rank = int(spec.param("kv_rank"))
        self.eps = float(spec.param("eps"))
        self.has_sink = bool(spec.param("sink", False))
        self.has_gate = spec.param("gate") == "head"
        self.down = self.q_up = self.k_absorb = self.v_up = self.o = None
        self.q_norm = self.kv_norm = self.sink = None

    @classmethod
    def tensor_specs(cls, spec: MixerSpec) -> Dict[str, TensorInfo]:
        W, H, d, dv = spec.hidden_size, spec.num_heads, spec.head_dim, spec.value_dim
        qr, kr = int(spec.param("q_rank")), int(spec.param("kv_rank"))
        out = {
            "q_down": TensorInfo((qr, W), "matrix"), "q_norm": TensorInfo((qr,), "norm"),
            "q_up": TensorInfo((H * d, qr), "matrix"),
            "kv_down": TensorInfo((kr, W), "matrix"), "kv_norm": TensorInfo((kr,), "norm"),
            "k_up": TensorInfo((H * d, kr), "matrix"), "v_up": TensorInfo((H * dv, kr), "matrix"),
            "o_proj": TensorInfo((W, H * dv), "matrix"),
        }
        if spec.param("sink", False):
            out["sink"] = TensorInfo((H,), "bias")
        if spec.param("gate") == "head":
            out["gate"] = TensorInfo((H, W), "matrix")
        return out

    def cache_spec(self) -> KVSpec:
        # one latent a position serves as key and as value
        return KVSpec(1, self.kv_rank, self.spec.window, shared_kv=True)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        H, d, dv = s.num_heads, s.head_dim, s.value_dim

        def dev(t):
            return t.to(device=self.device, dtype=self.dtype)

        def f32(t):
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        parts = [dev(tensors["q_down"]), dev(tensors["kv_down"])]
        if self.has_gate:
            parts.append(dev(tensors["gate"]))
        self.down = torch.cat(parts, dim=0).contiguous()  # one product for both latents and the gates
        self.q_up = dev(tensors["q_up"]).contiguous()
        # W_uk per head, transposed: [H, kv_rank, dim], so that q_h -> W_uk,h^T q_h is a per-head product
        self.k_absorb = dev(tensors["k_up"]).view(H, d, self.kv_rank).transpose(1, 2).contiguous()
        self.v_up = dev(tensors["v_up"]).view(H, dv, self.kv_rank).contiguous()
        self.o = dev(tensors["o_proj"]).contiguous()
        self.q_norm, self.kv_norm = f32(tensors["q_norm"]), f32(tensors["kv_norm"])
        self.sink = f32(tensors["sink"]) if self.has_sink else None

    def forward(self, x, ctx, residual=None):
        s = self.spec
        kv, batch = ctx.kv, ctx.batch
        H = s.num_heads
        proj = ops.linear(x, self.down, out_dtype=torch.float32)
        ops.prof_mark("qkv_gemm")
        cq, gate = ops.latent_post(proj, self.q_norm, self.kv_norm, self.eps, batch.row_pos, batch.row_slot,
                                   kv.k_pages, kv.page_table, kv.page_size, self.q_rank, self.kv_rank,
                                   H if self.has_gate else 0, ctx.writes_cache, self.dtype)
        ops.prof_mark("latent_post")
        q = ops.linear(cq, self.q_up)
        ops.prof_mark("q_up")
        qa = ops.heads_linear(q, self.k_absorb)  # [rows, H * kv_rank]
        ops.prof_mark("q_absorb")
        attn = ops.attention(qa, kv.k_pages, kv.k_pages, kv.page_table, kv.page_size, batch, H, 1,
                             self.kv_rank, s.window, s.scale, sink=self.sink)
        ops.prof_mark("attn")
        vals = ops.heads_linear(attn, self.v_up, scale=gate if self.has_gate else None)
        ops.prof_mark("v_up")
        if residual is not None:
            fused = ops.linear_residual(vals, self.o, residual[0], residual[1])
            if fused is not None:
                ops.prof_mark("o_proj")
                return None if fused is ops.ADDED else fused
        out = ops.linear(vals, self.o, out_dtype=torch.float32)
        ops.prof_mark("o_proj")
        return out
