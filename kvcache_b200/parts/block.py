"""The arrangement of parts in one layer: pre-norm residual block
(reference order: apps/qwen_serve.cu:101-116)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, Block, FeedForward, LayerContext, Mixer, Norm


class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += ffn(norm2(h)).

    Each add is folded into the norm that follows it, so the block takes the
    previous layer's delta as `pending` and hands its own feed-forward delta on.
    """

    def __init__(self, width: int, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, dtype: str):
        self.width = width
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.dtype = TORCH_DTYPES[dtype]

    def _parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def init_kinds(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for part in self._parts():
            out.update(part.init_kinds())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        for part in self._parts():
            part.bind(tensors, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self._parts())

    def supports_fold(self, kernels, num_rows: int) -> bool:
        return (self.mixer.supports_fold(self.norm1, kernels, num_rows)
                and self.ffn.supports_fold(self.norm2, kernels, num_rows))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, ctx: LayerContext) -> None:
        self.mixer.forward_folded(h, h16, self.norm1, ctx)
        self.ffn.forward_folded(h, h16, self.norm2, ctx)

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], ctx: LayerContext) -> Optional[torch.Tensor]:
        T = h.shape[0]
        x = ctx.workspace.buffer("block.normed", (T, self.width), self.dtype)
        self.norm1.add_norm(h, pending, x, ctx)
        delta = self.mixer.forward(x, ctx)
        self.norm2.add_norm(h, delta, x, ctx)
        return self.ffn.forward(x, ctx)


class SandwichBlock(Block):
    """h += post1(mixer(pre1(h))); h += post2(ffn(pre2(h))): a norm before and after each sublayer.

    The normalisation of a sublayer's result and its add are folded into the norm that follows (one launch computes
    both sums of squares), so the block takes the layer before's `NormedDelta` as `pending` and hands its own on.
    `ffn` may be None: the layer then ends after its mixer.
    """

    def __init__(self, width: int, pre1: Norm, mixer: Mixer, post1: Norm, pre2: Optional[Norm], ffn: Optional[FeedForward],
                 post2: Optional[Norm], dtype: str):
        if (ffn is None) != (pre2 is None) or (ffn is None) != (post2 is None):
            raise ValueError("a feed-forward comes with its two norms, or none of the three is given")
        self.width = width
        self.pre1, self.mixer, self.post1, self.pre2, self.ffn, self.post2 = pre1, mixer, post1, pre2, ffn, post2
        self.dtype = TORCH_DTYPES[dtype]

    def _parts(self):
        return tuple(p for p in (self.pre1, self.mixer, self.post1, self.pre2, self.ffn, self.post2) if p is not None)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def init_kinds(self) -> Dict[str, str]:
        out: Dict[str, str] = {}
        for part in self._parts():
            out.update(part.init_kinds())
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        for part in self._parts():
            part.bind(tensors, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self._parts())

    def forward(self, h: torch.Tensor, pending, ctx: LayerContext):
        from .base import NormedDelta
        T = h.shape[0]
        x = ctx.workspace.buffer("block.normed", (T, self.width), self.dtype)
        self.pre1.add_norm(h, pending, x, ctx)
        delta = NormedDelta(self.mixer.forward(x, ctx), self.post1)
        if self.ffn is None:
            return delta
        self.pre2.add_norm(h, delta, x, ctx)
        return NormedDelta(self.ffn.forward(x, ctx), self.post2)
