"""Tiny Libulorn configurations for the tests: they differ from one another in every size, in the order and kinds of
layers, in windows, rotation and gate constants; sizes that tend to coincide or to be 1 (one key/value head, as many as
query heads, values as wide as keys, one expert chosen, all chosen, no shared expert, a layer without feed-forward, a
window of one page, of two tokens, none at all, whole-head rotation, none, a model of one kind of layer only, no pair
table) each occur somewhere."""
from __future__ import annotations

import copy
import os

import torch


def _attention(heads, kv_heads, dim, vdim, scale, window, rot):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        out["mask"] = {"size": window}
    if rot is not None:
        base, dims, scaling = rot
        out["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            out["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def _parallel(left, right, left_scale, right_scale):
    heads, dim, vdim, tau, rank = right
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                          "right": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}}


def _memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# A: memory layer first, then two different parallel layers (two windows: two cache groups), a layer without feed-forward.
LIB_A = {
    "architecture": "Libulorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        _layer(_memory(2, 24, 16, 8.0), _moe(5, 2, 24, 1.5, (40, 0.75))),
        _layer(_parallel(_attention(4, 2, 16, 24, 0.3, 11, (10000.0, 8, (4.0, 1.0, 4.0, 32))), (3, 8, 16, 4.0, 6), 1.3, 0.7), _moe(5, 2, 24, 1.5, (40, 0.75))),
        _layer(_parallel(_attention(4, 2, 16, 24, 0.3, 16, (10000.0, 8, (4.0, 1.0, 4.0, 32))), (3, 8, 16, 4.0, 6), 0.6, 1.1), None),
    ],
}
# B: one key/value head, values as wide as keys, whole-head plain rotation, one expert chosen and no shared expert, a window
# of two tokens; then all experts chosen; a memory layer with one head.
LIB_B = {
    "architecture": "Libulorn", "vocab": 331, "width": 96, "norm": {"eps": 3e-5},
    "embedding": {"bigram": {"buckets": 50, "mul_prev": 1, "mul_cur": 1000003}},
    "layers": [
        _layer(_parallel(_attention(3, 1, 32, 32, 0.2, 2, (500.0, 32, None)), (1, 40, 24, 9.0, 3), 1.0, 1.0), _moe(3, 1, 40, 0.5)),
        _layer(_memory(1, 40, 72, 2.5), _moe(4, 4, 16, 3.0, (16, 3.0))),
        _layer(_parallel(_attention(2, 2, 24, 8, 0.25, None, None), (2, 16, 40, 1.0, 16), 2.0, 0.25), _moe(3, 1, 40, 0.5)),
    ],
}
# C: only memory layers, no pair table (no cache pages at all), sizes that are no power of two.
LIB_C = {
    "architecture": "Libulorn", "vocab": 150, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_memory(3, 12, 20, 12.0), _moe(2, 1, 56, 2.0, (24, 1.0))),
        _layer(_memory(5, 8, 8, 1.0), None),
    ],
}
# D: only parallel layers, five query heads per key/value head group of one, windows across several pages, slow decay.
LIB_D = {
    "architecture": "Libulorn", "vocab": 500, "width": 120, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 1, "mul_prev": 7, "mul_cur": 3}},
    "layers": [
        _layer(_parallel(_attention(5, 5, 24, 40, 0.125, 37, (300000.0, 12, (2.5, 2.0, 8.0, 64))), (2, 48, 24, 32.0, 8), 1.0, 0.5), _moe(9, 3, 40, 1.0, (72, 4.0))),
        _layer(_parallel(_attention(10, 2, 8, 16, 0.35, 37, (300000.0, 8, (2.5, 2.0, 8.0, 64))), (4, 16, 8, 2.0, 4), 0.9, 1.2), _moe(9, 3, 40, 1.0, (72, 4.0))),
    ],
}
# E: sizes in steps of 16 as real models have them - keys of 64 beside values of 128 (in bfloat16 the keys are cached as
# wide as the values and the layer runs on the tensor-core attention kernels), a window that crosses pages.
LIB_E = {
    "architecture": "Libulorn", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 211, "mul_prev": 17, "mul_cur": 3}},
    "layers": [
        _layer(_parallel(_attention(4, 2, 64, 128, 0.125, 40, (50000.0, 32, (8.0, 1.0, 4.0, 256))), (2, 32, 64, 8.0, 8), 1.1, 0.8), _moe(4, 2, 32, 2.0, (64, 1.5))),
        _layer(_memory(2, 32, 64, 10.0), _moe(4, 2, 32, 2.0, (64, 1.5))),
    ],
}
CONFIGS = {"A": LIB_A, "B": LIB_B, "C": LIB_C, "D": LIB_D, "E": LIB_E}
PAGE_SIZE = {"A": 8, "B": 16, "C": 16, "D": 4, "E": 16}


def config_dict(name: str, **changes) -> dict:
    out = copy.deepcopy(CONFIGS[name])
    out.update(changes)
    return out


def make_libulorn_folder(tmp_path, name: str, seed: int = 0, dtype=torch.float32, sharpen: float = 1.0, std: float = 0.08,
                         all_experts: bool = False) -> str:
    """A random-weights folder for configuration `name`.  `sharpen` multiplies every attention's score scale, so that the
    softmax picks out single keys and a wrong or missing key shows in the logits.  `all_experts`: every routed layer
    chooses all its experts - for comparisons in bfloat16, where rounding may turn a close call between two experts the
    other way than the plain implementation's float64 does."""
    import kvcache_b200  # registers the architectures  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    data = config_dict(name, initializer_range=std)
    for layer in data["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= sharpen
        if all_experts and layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    folder = os.path.join(str(tmp_path), f"lib_{name}_{seed}_{sharpen}_{int(all_experts)}")
    write_random_model(folder, config_from_dict(data), seed, dtype)
    return folder
