"""Terms added to the token embedding before the first layer.

A term is registered under the `kind` its `EmbeddingTermSpec` names and has
the parts' usual face (`tensor_specs`, `bind`, `capturable`) plus
`state_spec() -> StateSpec | None` (what it keeps per sequence between steps)
and `add(hidden, batch, state)`, which adds itself to the 32-bit rows in place.

"bigram_hash": a table row chosen by a hash of (previous token, token),
row = (prev * mul_prev + token * mul_cur) mod buckets, and the table's extra
last row at a sequence's first position.  The previous token of a step's first
row is the sequence's state (one int32 a slot), written by the step before.

"sinusoidal": entry 2i gets sin(p * base^(-2i / width)), entry 2i + 1 the
cosine of the same angle, p the row's position.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..cache.specs import StateSpec
from ..config.spec import EmbeddingTermSpec
from .registry import EMBEDDING_TERMS, TensorInfo, register_embedding_term  # noqa: F401


@register_embedding_term("bigram_hash")
class BigramHash:
    capturable = True  # tokens, positions and slots are read from device memory

    def __init__(self, spec: EmbeddingTermSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.buckets = int(spec.param("buckets"))
        self.mul_prev = int(spec.param("mul_prev"))
        self.mul_cur = int(spec.param("mul_cur"))
        self.vocab = int(spec.param("vocab"))
        self.table: Optional[torch.Tensor] = None

    @classmethod
    def tensor_specs(cls, spec: EmbeddingTermSpec) -> Dict[str, TensorInfo]:
        return {"table": TensorInfo((int(spec.param("buckets")) + 1, spec.hidden_size), "table")}

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), "int32")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors["table"].to(device=self.device, dtype=self.dtype).contiguous()

    def add(self, hidden: torch.Tensor, batch, state: torch.Tensor) -> None:
        ops.bigram_add(hidden, self.table, batch, state, self.mul_prev, self.mul_cur, self.vocab)


@register_embedding_term("sinusoidal")
class Sinusoidal:
    capturable = True

    def __init__(self, spec: EmbeddingTermSpec, dtype: torch.dtype, device):
        self.spec = spec
        H = spec.hidden_size
        base = float(spec.param("base", 10000.0))
        # base^(-2i / H) in double precision, once; the kernel takes the angle and
        # its sine and cosine in double too
        i = torch.arange((H + 1) // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / H).to(device)

    @classmethod
    def tensor_specs(cls, spec: EmbeddingTermSpec) -> Dict[str, TensorInfo]:
        return {}

    def state_spec(self) -> None:
        return None

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def add(self, hidden: torch.Tensor, batch, state) -> None:
        ops.sinusoid_add(hidden, batch.row_pos, self.inv_freq)
