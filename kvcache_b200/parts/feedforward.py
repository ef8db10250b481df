"""Dense gated feed-forward (reference: apps/qwen_serve.cu:112-116, src/qwen_kernels.cu:102-105)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Sequence

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, FeedForward, LayerContext


class GatedMLP(FeedForward):
    """delta = (act(x Wg^T) * (x Wu^T)) Wd^T with act = silu; no biases."""

    def __init__(self, hidden: int, intermediate: int, *, activation: str, prefix: str, dtype: str,
                 names: Sequence[str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """`names`: what the gate, up and down matrices are called after `prefix` in the checkpoint."""
        self.names = tuple(names)
        if activation != "silu":
            raise ValueError(f"activation '{activation}' is not supported by the gated feed-forward kernel")
        self.hidden, self.intermediate = hidden, intermediate
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.interleaved = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p = self.prefix
        gate, up, down = self.names
        return {
            f"{p}{gate}": TensorSpec((self.intermediate, self.hidden)),
            f"{p}{up}": TensorSpec((self.intermediate, self.hidden)),
            f"{p}{down}": TensorSpec((self.hidden, self.intermediate)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p = self.prefix
        gate, up = tensors[f"{p}{self.names[0]}"], tensors[f"{p}{self.names[1]}"]
        # One projection for gate and up.  When the width allows, rows are interleaved in eights (gate rows
        # 8 b .. 8 b + 7, then the up rows of the same indices) so that a kernel's thread holds both values
        # of an index and can write the activation without a second pass.
        self.interleaved = self.intermediate % 8 == 0
        if self.interleaved:
            both = torch.stack([gate.view(-1, 8, self.hidden), up.view(-1, 8, self.hidden)], dim=1).reshape(-1, self.hidden)
        else:
            both = torch.cat([gate, up], dim=0)
        self.w_gate_up = both.to(self.dtype).to(device).contiguous()
        self.w_down = tensors[f"{p}{self.names[2]}"].to(self.dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def supports_fold(self, norm, kernels, num_rows: int) -> bool:
        can = getattr(kernels, "can_fold", None)
        return (can is not None and self.interleaved and norm.fold_params() is not None
                and can(self.dtype, num_rows, self.hidden, 2 * self.intermediate)
                and can(self.dtype, num_rows, self.intermediate, self.hidden))

    def forward_folded(self, h: torch.Tensor, h16: torch.Tensor, norm, ctx: LayerContext) -> None:
        T = h.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        weight, eps = norm.fold_params()
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.norm_gate_up_act(h16, self.w_gate_up, weight, eps, act)
        k.linear_into_residual(act, self.w_down, h, h16)


    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        act = ws.buffer("ffn.act", (T, self.intermediate), self.dtype)
        k.gate_up_act(x, self.w_gate_up, act, ws, self.interleaved)
        delta = ws.buffer("ffn.delta", (T, self.hidden), self.dtype)
        k.linear(act, self.w_down, delta)
        return delta


class RoutedMLP(FeedForward):
    """A mixture of small feed-forwards: delta = sum over the `top` experts e with the largest router logits of
    w_e * Wdown_e act(Wup_e x), the weights w being the softmax over the chosen logits only; no biases.

    The router's logits are float32 (from the rows in the compute type).  The experts' matrices are stacked
    ([experts, ff, hidden] and [experts, hidden, ff]) so that one grouped product serves all of them; which rows go to
    which expert is decided on the device, and the launches do not depend on it.
    """

    def __init__(self, hidden: int, expert_ff: int, experts: int, top: int, *, activation: str, prefix: str, dtype: str,
                 router_name: str = "router", expert_names: Sequence[str] = ("e{e}.up", "e{e}.down")):
        if activation != "relu2":
            raise ValueError(f"activation '{activation}' is not supported by the routed feed-forward kernels")
        if not 1 <= top <= experts:
            raise ValueError(f"top {top} of {experts} experts")
        self.hidden, self.expert_ff, self.experts, self.top = hidden, expert_ff, experts, top
        self.activation = activation
        self.prefix, self.router_name, self.expert_names = prefix, router_name, tuple(expert_names)
        self.dtype = TORCH_DTYPES[dtype]
        self.w_router: Optional[torch.Tensor] = None
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _expert(self, which: int, e: int) -> str:
        return self.prefix + self.expert_names[which].format(e=e)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.router_name: TensorSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            specs[self._expert(0, e)] = TensorSpec((self.expert_ff, self.hidden))
            specs[self._expert(1, e)] = TensorSpec((self.hidden, self.expert_ff))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        self.w_router = tensors[self.prefix + self.router_name].to(self.dtype).to(device).contiguous()
        self.w_up = torch.stack([tensors[self._expert(0, e)] for e in range(self.experts)]).to(self.dtype).to(device).contiguous()
        self.w_down = torch.stack([tensors[self._expert(1, e)] for e in range(self.experts)]).to(self.dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        """Bytes one row reads: the router and its `top` experts (a step of many rows reads up to all experts)."""
        size = self.w_up.element_size()
        return (self.w_router.numel() + self.top * 2 * self.expert_ff * self.hidden) * size

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T = x.shape[0]
        k, ws = ctx.kernels, ctx.workspace
        logits = ws.buffer("moe.logits", (T, self.experts), torch.float32)
        k.linear(x, self.w_router, logits)
        chosen = ws.buffer("moe.chosen", (T, self.top), torch.int32)
        share = ws.buffer("moe.share", (T, self.top), torch.float32)
        k.route_top(logits, chosen, share)
        delta = ws.buffer("ffn.delta", (T, self.hidden), self.dtype)
        k.routed_experts(x, self.w_up, self.w_down, chosen, share, delta, self.activation, ws)
        return delta
