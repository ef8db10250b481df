"""Plain, slow implementation of the Kakipel decoder: whole sequences, no cache, one function
for each mechanism, float64 by default.  It shares no code with `kvcache_b200` (it reads the
model folder with the `safetensors` package and `json`) and states every formula directly:
per-head keys and values are expanded from the latent, never absorbed into the queries.

The design, in this file's notation.  W = width, residual stream x[T, W].

* norm(v; w) = v / sqrt(mean(v^2) + eps) * w.
* layer: x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))) (the second line only if the layer has a feed-forward).
* latent attention: cq = norm(Wdq h; dq.norm), q = Wuq cq, per head [dim | rot_dim];
  [c_raw | kr] = Wdkv h, c = norm(c_raw; dkv.norm); per head k = Wuk c, v = Wuv c;
  score(i, j) = scale * (q_i[:dim] . k_j + R_i(q_i[dim:]) . R_j(kr_j)) for j <= i, softmax over j,
  o = concat_heads(sum_j p_ij v_j) * sigmoid(Wg h), out = Wo o.
* rotation R_p: dimension t pairs with t + dims/2, angle p * f_t, with the frequencies
  blended between f_t and f_t / factor by a ramp over t, and cos and sin scaled by 0.1 ln(factor) + 1.
* dense feed-forward: Wdown (silu(Wgate h) * (Wup h)).
* routed feed-forward: z = Wrouter h; the `top` largest z, weights softmax over those; sum_e w_e Wdown_e relu(Wup_e h)^2.
* looped layers start..stop-1 run `times` times; before pass t: x = Win [x; x0] + step[t], x0 the embedding output.
* logits = head norm(x; final.norm).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        config = json.load(fh)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return x @ weight.t()


def rotation_frequencies(rot: dict, dtype=torch.float64) -> (torch.Tensor, float):
    """Frequencies f_t, t < dims/2, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * t / dims) for t in range(half)], dtype=dtype)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((t - lo) / max(hi - lo, 0.001), 0.0), 1.0) for t in range(half)], dtype=dtype)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x[T, ..., D]: the first rot.dims dimensions of the last axis are rotated, the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, mag = rotation_frequencies(rot, x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = (torch.cos(angle) * mag).view(shape), (torch.sin(angle) * mag).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T)
    cq = rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = linear(cq, w[p + "uq"]).view(T, H, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], pos, m["rot"])
    down = linear(h, w[p + "dkv"])
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, rank:], pos, m["rot"])                       # one for all heads
    k_plain = linear(c, w[p + "uk"]).view(T, H, dim)
    v = linear(c, w[p + "uv"]).view(T, H, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * vdim)
    out = out * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(out, w[p + "o"])


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = linear(h, w[p + "gate"])
    return linear(g * torch.sigmoid(g) * linear(h, w[p + "up"]), w[p + "down"])


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = linear(h, w[p + "router"])
    best, which = torch.topk(z, top, dim=-1)
    share = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for r in range(h.shape[0]):
        for s in range(top):
            e = int(which[r, s])
            a = torch.relu(linear(h[r:r + 1], w[f"{p}e{e}.up"])) ** 2
            out[r] += share[r, s] * linear(a, w[f"{p}e{e}.down"])[0]
    return out


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, spec: dict, eps: float) -> torch.Tensor:
    p = f"l{i}."
    if spec["type"] != "latent_attention":
        raise ValueError(f"unknown mixer '{spec['type']}'")
    mixed = latent_attention(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    x = x + rms_norm(mixed, w[p + "norm1b"], eps)
    mlp = spec.get("mlp")
    if mlp is None:
        return x
    h = rms_norm(x, w[p + "norm2"], eps)
    y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, w, p + "mlp.", mlp)
    return x + rms_norm(y, w[p + "norm2b"], eps)


def layer_runs(config: dict) -> List[tuple]:
    """[(layer, pass or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def residual_streams(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> List[torch.Tensor]:
    """The residual stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x0 = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    x, out = x0, []
    for i, t, first in layer_runs(config):
        if first:
            x = linear(torch.cat([x, x0], dim=-1), w["loop.in"]) + w["loop.step"][t]
        x = layer(x, w, i, config["layers"][i], eps)
        out.append(x)
    return out


def logits_of(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    x = residual_streams(config, w, tokens)[-1]
    return linear(rms_norm(x, w["final.norm"], float(config["norm"]["eps"])), w["head"])


def greedy_generate(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    """Recomputes the whole sequence for every new token."""
    tokens, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(torch.argmax(logits_of(config, w, tokens)[-1]))
        tokens.append(nxt)
        out.append(nxt)
    return out
