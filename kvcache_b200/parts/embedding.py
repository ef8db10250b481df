"""Parts that act on the embedded rows before the first layer."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, EmbeddingPart, LayerContext, StateSpec


class HashedBigramEmbedding(EmbeddingPart):
    """h[r] += table[b(r)], b = (previous token * mul_prev + token * mul_cur) mod buckets; a request's first token takes
    the table's last row (number `buckets`).  The previous token of a row that opens a step's portion is the request's
    state (one int32 per request, written by the step that ran the token before)."""

    def __init__(self, width: int, buckets: int, mul_prev: int, mul_cur: int, vocab_size: int, table_name: str, dtype: str):
        self.width, self.buckets, self.mul_prev, self.mul_cur = width, int(buckets), int(mul_prev), int(mul_cur)
        self.vocab_size = vocab_size
        self.table_name = table_name
        self.dtype = TORCH_DTYPES[dtype]
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.table_name: TensorSpec((self.buckets + 1, self.width))}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.table = tensors[self.table_name].to(self.dtype).to(device).contiguous()

    def state_spec(self):
        return {"previous_token": StateSpec((), "int32")}

    def forward(self, h: torch.Tensor, ctx: LayerContext) -> None:
        ctx.kernels.bigram_embed(self.table, ctx.batch, ctx.state["previous_token"], h, self.buckets, self.mul_prev,
                                 self.mul_cur, self.vocab_size)
