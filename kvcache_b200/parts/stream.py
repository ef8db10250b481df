"""Parts that act on the residual stream between layers."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, NormedDelta, StreamPart


class LoopEntry(StreamPart):
    """What a pass over a run of layers does on entering it: h = Win [h; x0] + step[t], with x0 the embedding output
    and t the number of the pass.  The passes share Win ([width, 2 width], h's half first) and the table of steps
    ([passes, width])."""
    needs_embedding = True

    def __init__(self, width: int, passes: int, in_name: str, step_name: str, dtype: str):
        self.width, self.passes = width, passes
        self.in_name, self.step_name = in_name, step_name
        self.dtype = TORCH_DTYPES[dtype]
        self.w_in: Optional[torch.Tensor] = None
        self.steps: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.in_name: TensorSpec((self.width, 2 * self.width)), self.step_name: TensorSpec((self.passes, self.width))}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.w_in = tensors[self.in_name].to(self.dtype).to(device).contiguous()
        self.steps = tensors[self.step_name].to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return self.w_in.numel() * self.w_in.element_size() + 4 * self.width

    def forward(self, h: torch.Tensor, pending, ctx: LayerContext, argument: int):
        T = h.shape[0]
        k = ctx.kernels
        both = ctx.workspace.buffer("loop.both", (T, 2 * self.width), self.dtype)
        post = pending.post.fold_params() if isinstance(pending, NormedDelta) else None
        if isinstance(pending, NormedDelta) and post is None:
            raise ValueError("the pending delta's norm cannot be applied before the add")
        delta = pending.delta if isinstance(pending, NormedDelta) else pending
        # h += the pending delta; both = [h | x0] in the compute type; then the product writes the new h over the old.
        k.norm_add_rmsnorm(h, delta, post[0] if post else None, post[1] if post else 0.0, None, 0.0, both, None, ctx.embedded)
        k.linear(both, self.w_in, h, self.steps[argument])
        return None
