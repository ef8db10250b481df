"""Plain, slow implementation of the Libulorn decoder: whole sequences, no cache, token-by-token recurrences, one
function for each mechanism, float64 by default.  It shares no code with `kvcache_b200` (it reads the model folder
with the `safetensors` package and `json`) and states every formula directly.

The design, in this file's notation.  W = width, residual stream x[T, W]; unit(v) = v / sqrt(mean(v^2) + eps).

* embedding: x_t = embed[tok_t] + bigram[b_t], b_0 = buckets (the table's last row), b_t = (tok_{t-1} mul_prev +
  tok_t mul_cur) mod buckets.
* layer: x += unit(mixer(x)) * norm1; x += unit(ff(x)) * norm2 (the second line only if the layer has a feed-forward);
  the sublayers read x as it is.
* windowed attention with grouped keys: q, k, v = Wq h, Wk h, Wv h; per head q and k are unit(.) * weight over their
  `dim` numbers, then rotated (first `dims` numbers of a head, t pairs with t + dims/2, angle p f_t, the frequencies
  stretched piecewise by wavelength); score(i, j) = scale q_i . k_j for 0 <= i - j < window, softmax over j;
  head h's sum of values is multiplied by sigmoid(Wg h)_h; out = Wo concat.
* gated linear attention: q = Wq h / sqrt(dim), k = Wk h, v = Wv h, a = sigmoid(Wa2 (Wa1 h) + b)^(1/tau) per key
  channel; S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; out = Wo (concat_heads(unit(o) * norm) * silu(Wg h)).
* the parallel mixer: left_scale * attention + right_scale * gated linear attention, both reading the same h.
* matrix memory with exponential gates: q = Wq h / sqrt(dim), k, v; per head i_t = cap tanh((Wi h + bi) / cap),
  f_t = logsigmoid(cap tanh((Wf h + bf) / cap)); m_t = max(f_t + m_{t-1}, i_t), m_{-1} = 0;
  S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T, n_t the same with k_t alone;
  o_t = S_t^T q_t / (max(|n_t . q_t|, e^{-m_t}) + 1e-6); out = Wo (concat_heads(unit(o)) * norm * sigmoid(Wg h)).
* feed-forward: p = softmax(Wrouter h) over all experts; the `top` largest p, weights p themselves;
  expert(h) = Wdown (g sigmoid(1.702 g) (u + 1)), g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit);
  a shared expert of the same form (its own size and limit) is added for every token.
* logits = head (unit(x) * final.norm).
"""
from __future__ import annotations

import contextlib
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


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


_ROUND_TO: Optional[torch.dtype] = None


@contextlib.contextmanager
def rounding(dtype: torch.dtype = torch.bfloat16):
    """Within the block every matrix product rounds its input rows and its result to `dtype` (the arithmetic stays as
    wide as the weights): what rounding alone does to a position's logits, which is what a reduced-precision run of the
    engine may be held to where a position is badly conditioned."""
    global _ROUND_TO
    saved, _ROUND_TO = _ROUND_TO, dtype
    try:
        yield
    finally:
        _ROUND_TO = saved


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if _ROUND_TO is None:
        return x @ weight.t()
    return (x.to(_ROUND_TO).to(weight.dtype) @ weight.t()).to(_ROUND_TO).to(weight.dtype)


# ---- embedding --------------------------------------------------------------------------------------------------------
def bigram_rows(tokens: Sequence[int], bigram: dict) -> List[int]:
    buckets, mul_prev, mul_cur = int(bigram["buckets"]), int(bigram["mul_prev"]), int(bigram["mul_cur"])
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embed(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    x = w["embed"][list(tokens)].clone()
    bigram = (config.get("embedding") or {}).get("bigram")
    if bigram:
        x = x + w["bigram"][bigram_rows(tokens, bigram)]
    return x


# ---- rotation ---------------------------------------------------------------------------------------------------------
def rotation_frequencies(rot: dict) -> torch.Tensor:
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    s = rot.get("scaling")
    for t in range(dims // 2):
        f = base ** (-2.0 * t / dims)
        if s:
            factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                blend = (original / wavelength - low) / (high - low)
                f = (1.0 - blend) * f / factor + blend * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, D]: the first rot.dims numbers of each head rotated by the row's position."""
    dims = int(rot["dims"])
    half = dims // 2
    angle = positions.to(torch.float64)[:, None] * rotation_frequencies(rot)[None, :]
    c, s = torch.cos(angle)[:, None, :].to(x.dtype), torch.sin(angle)[:, None, :].to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- mixers -----------------------------------------------------------------------------------------------------------
def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = linear(h, w[p + "q"]).view(T, H, D)
    k = linear(h, w[p + "k"]).view(T, G, D)
    v = linear(h, w[p + "v"]).view(T, G, Dv)
    q = unit(q, eps) * w[p + "q.norm"]
    k = unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    gate = torch.sigmoid(linear(h, w[p + "g"]))                      # [T, H]
    window = int(m["mask"]["size"]) if m.get("mask") else None
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for head in range(H):
            g = head // (H // G)
            score = (k[lo:i + 1, g] @ q[i, head]) * float(m["scale"])
            out[i, head] = torch.softmax(score, dim=0) @ v[lo:i + 1, g]
    out = out * gate[:, :, None]
    return linear(out.reshape(T, H * Dv), w[p + "o"])


def gated_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = linear(h, w[p + "q"]).view(T, H, D) / math.sqrt(D)
    k = linear(h, w[p + "k"]).view(T, H, D)
    v = linear(h, w[p + "v"]).view(T, H, Dv)
    z = linear(linear(h, w[p + "a1"]), w[p + "a2"]) + w[p + "a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / float(m["tau"])).view(T, H, D)
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit(o, eps) * w[p + "norm"]
    gate = linear(h, w[p + "g"])
    o = o.reshape(T, H * Dv) * (gate * torch.sigmoid(gate))
    return linear(o, w[p + "o"])


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = window_attention(h, w, p + "left.", m["left"], eps)
    right = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def matrix_memory(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = linear(h, w[p + "q"]).view(T, H, D) / math.sqrt(D)
    k = linear(h, w[p + "k"]).view(T, H, D)
    v = linear(h, w[p + "v"]).view(T, H, Dv)
    gi = cap * torch.tanh((linear(h, w[p + "i"]) + w[p + "i.b"]) / cap)                                   # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((linear(h, w[p + "f"]) + w[p + "f.b"]) / cap))
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        denom = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / denom[:, None]
    o = unit(o, eps).reshape(T, H * Dv) * w[p + "norm"] * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(o, w[p + "o"])


# ---- feed-forward -----------------------------------------------------------------------------------------------------
def clamped_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(linear(h, w[p + "gate"]), max=limit)
    u = torch.clamp(linear(h, w[p + "up"]), min=-limit, max=limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict):
    """(chosen experts [T, top], their weights [T, top]): the largest softmax scores over all experts, as they are."""
    scores = torch.softmax(linear(h, w[p + "router"]), dim=-1)
    weight, chosen = torch.topk(scores, int(mlp["router"]["top"]), dim=-1)
    return chosen, weight


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    chosen, weight = route(h, w, p, mlp)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s in range(chosen.shape[1]):
            e = int(chosen[t, s])
            out[t] += weight[t, s] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# ---- the model --------------------------------------------------------------------------------------------------------
def mixer_of(layer: dict):
    return {"parallel": parallel_mixer, "mlstm": matrix_memory}[layer["type"]]


def residual_streams(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> List[torch.Tensor]:
    """The residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = embed(config, w, tokens)
    out = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        x = x + unit(mixer_of(layer)(x, w, p + "mix.", layer["mixer"], eps), eps) * w[p + "norm1"]
        if layer.get("mlp"):
            x = x + unit(feed_forward(x, w, p + "mlp.", layer["mlp"]), eps) * w[p + "norm2"]
        out.append(x)
    return out


def logits_of(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    eps = float(config["norm"]["eps"])
    x = residual_streams(config, w, tokens)[-1]
    return linear(unit(x, eps) * w["final.norm"], w["head"])


def greedy_generate(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> List[int]:
    tokens, out = list(prompt), []
    for _ in range(new_tokens):
        out.append(int(torch.argmax(logits_of(config, w, tokens)[-1])))
        tokens.append(out[-1])
    return out
