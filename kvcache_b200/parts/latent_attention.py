"""Latent attention: keys and values of all heads are expanded from one small latent per token, and only the
latent (with one rotated key part that all heads share) is cached.

With h the mixer's input, per token:
    cq = norm(Wdq h),  q = Wuq cq                      per head [dim unrotated | rot_dim rotated]
    [c_raw | kr] = Wdkv h,  c = norm(c_raw)            c: kv_rank, kr: rot_dim, rotated by the position, not normed
    per head: k = Wuk c, v = Wuv c
    score(i, j) = scale * (q_i[:dim] . k_j + R_i(q_i[dim:]) . R_j(kr_j)),  j <= i;  softmax over j
    out = Wo (concat_heads(sum_j p_ij v_j) * sigmoid(Wg h))

This part never expands a cached token.  Since k_j = Wuk c_j, the unrotated score is (Wuk^T q_i[:dim]) . c_j: the
query is taken into the latent's space once (a product per head with Wuk^T), attention then runs with one shared
"key" row [c_j | R_j(kr_j)] of kv_rank + rot_dim numbers per token, whose first kv_rank numbers are also the "value",
and the head's result sum_j p_ij c_j goes through Wuv afterwards.  The cache entry is one key head of that width and
no value pool (`PagedKVSpec.value_dim == 0`); a step reads kv_rank + rot_dim numbers per cached token, whatever the
number of heads.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import TensorSpec
from .base import TORCH_DTYPES, LayerContext, Mixer, PagedKVSpec, PositionEncoding


class LatentAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, *,
                 scale: float, eps: float, position: PositionEncoding, prefix: str, dtype: str, window: Optional[int] = None):
        self.hidden, self.num_heads = hidden, num_heads
        self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank = dim, rot_dim, vdim, kv_rank, q_rank
        self.scale, self.eps = float(scale), float(eps)
        self.position = position
        self.window = window
        self.prefix = prefix
        self.dtype = TORCH_DTYPES[dtype]
        self.q_head = dim + rot_dim                 # a head's query as the checkpoint lays it out
        self.key_dim = kv_rank + rot_dim            # a cached row, and a head's query after it was taken to the latent's space
        self.gate_col = q_rank + kv_rank + rot_dim  # where the gate starts in the fused projection's rows
        self.w_in: Optional[torch.Tensor] = None
        self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.q_norm = self.kv_norm = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        p, H = self.prefix, self.num_heads
        return {
            f"{p}dq": TensorSpec((self.q_rank, self.hidden)),
            f"{p}dq.norm": TensorSpec((self.q_rank,)),
            f"{p}uq": TensorSpec((H * self.q_head, self.q_rank)),
            f"{p}dkv": TensorSpec((self.kv_rank + self.rot_dim, self.hidden)),
            f"{p}dkv.norm": TensorSpec((self.kv_rank,)),
            f"{p}uk": TensorSpec((H * self.dim, self.kv_rank)),
            f"{p}uv": TensorSpec((H * self.vdim, self.kv_rank)),
            f"{p}g": TensorSpec((H * self.vdim, self.hidden)),
            f"{p}o": TensorSpec((self.hidden, H * self.vdim)),
        }

    def init_kinds(self) -> Dict[str, str]:
        return {f"{self.prefix}dq.norm": "ones_plus_normal", f"{self.prefix}dkv.norm": "ones_plus_normal"}

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        p, H = self.prefix, self.num_heads
        place = lambda t: t.to(self.dtype).to(device).contiguous()
        # One product for everything that reads the mixer's input: rows [query latent | key/value latent | shared key part | gate].
        self.w_in = place(torch.cat([tensors[f"{p}dq"], tensors[f"{p}dkv"], tensors[f"{p}g"]], dim=0))
        self.w_uq = place(tensors[f"{p}uq"])
        # [H, kv_rank, dim]: the transposed key expansion, which takes a head's unrotated query to the latent's space.
        self.w_uk_t = place(tensors[f"{p}uk"].view(H, self.dim, self.kv_rank).transpose(1, 2))
        self.w_uv = place(tensors[f"{p}uv"].view(H, self.vdim, self.kv_rank))
        self.w_o = place(tensors[f"{p}o"])
        self.q_norm = tensors[f"{p}dq.norm"].to(torch.float32).to(device).contiguous()
        self.kv_norm = tensors[f"{p}dkv.norm"].to(torch.float32).to(device).contiguous()
        self.position.bind(tensors, device)

    def weight_bytes(self) -> int:
        mats = (self.w_in, self.w_uq, self.w_uk_t, self.w_uv, self.w_o)
        return sum(m.numel() * m.element_size() for m in mats) + 4 * (self.q_rank + self.kv_rank)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(1, self.key_dim, self.window, value_dim=0)

    def step_planners(self, kernels):
        planner = getattr(kernels, "latent_attention_planner", None)
        return () if planner is None else (planner(self.num_heads, self.key_dim, self.kv_rank),)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        T, H = x.shape[0], self.num_heads
        k, ws = ctx.kernels, ctx.workspace
        rotation = self.position.rotation()
        proj = ws.buffer("latent.proj", (T, self.w_in.shape[0]), self.dtype)
        k.linear(x, self.w_in, proj)
        cq = ws.buffer("latent.cq", (T, self.q_rank), self.dtype)
        k.latent_norm_rope_append(proj, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps,
                                  rotation.cos, rotation.sin, ctx.batch, ctx.kv, cq)
        q = ws.buffer("latent.q", (T, H * self.q_head), self.dtype)
        k.linear(cq, self.w_uq, q)
        q_lat = ws.buffer("latent.q_lat", (T, H * self.key_dim), self.dtype)
        k.head_linear(q, self.w_uk_t, q_lat, rotate=(rotation.cos, rotation.sin, ctx.batch.positions))
        o_lat = ws.buffer("latent.o_lat", (T, H * self.kv_rank), self.dtype)
        k.latent_attention(q_lat, ctx.batch, ctx.kv, o_lat, H, self.kv_rank, self.scale, ws)
        o = ws.buffer("latent.o", (T, H * self.vdim), self.dtype)
        k.head_linear(o_lat, self.w_uv, o, gate=(proj, self.gate_col))
        delta = ws.buffer("attn.delta", (T, self.hidden), self.dtype)
        k.linear(o, self.w_o, delta)
        return delta
