"""Tiny Kakipel configurations for the tests: they differ from one another in every size, in the order and kinds of
layers, in the looped run and in the rotation's constants; sizes that tend to coincide (head count 1, one expert
chosen, all experts chosen, key rank equal to nothing else, one pass) each occur somewhere."""
from __future__ import annotations

import copy
import os

import torch


def _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None, dims=None):
    rot = {"base": base, "dims": dims or rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "rot": rot}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


DENSE = lambda ff: {"kind": "dense", "ff": ff}
MOE = lambda experts, top, ff: {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}

# P: three heads, a looped pair of layers at the start, a layer without feed-forward, ramp-scaled rotation.
KAKI_P = {
    "architecture": "Kakipel", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(3, 16, 8, 24, 40, 32, 0.3, 10000.0, (4.0, 64, 16.0, 2.0)), DENSE(96)),
        _layer(_mixer(3, 16, 8, 24, 40, 32, 0.3, 10000.0, (4.0, 64, 16.0, 2.0)), MOE(5, 2, 24)),
        _layer(_mixer(3, 16, 8, 24, 40, 32, 0.3, 10000.0, (4.0, 64, 16.0, 2.0)), None),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
# Q: one head, no loop, plain rotation (no scaling) with other constants in every layer, one expert chosen / all chosen.
KAKI_Q = {
    "architecture": "Kakipel", "vocab": 331, "width": 96, "norm": {"eps": 3e-5},
    "layers": [
        _layer(_mixer(1, 24, 16, 40, 56, 48, 0.2, 500.0), MOE(3, 1, 40)),
        _layer(_mixer(1, 32, 12, 16, 20, 24, 0.25, 80000.0, (8.0, 32, 8.0, 1.0)), MOE(4, 4, 16)),
        _layer(_mixer(2, 8, 4, 8, 12, 16, 0.4, 100.0), DENSE(72)),
        _layer(_mixer(1, 24, 16, 40, 56, 48, 0.2, 500.0), DENSE(200)),
    ],
    "loop": None,
}
# R: five heads, sizes that are no power of two, one layer looped three times in the middle, the last layers after it.
KAKI_R = {
    "architecture": "Kakipel", "vocab": 500, "width": 120, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_mixer(5, 48, 16, 32, 72, 56, 0.125, 300000.0, (2.5, 128, 24.0, 1.5)), MOE(9, 3, 40)),
        _layer(_mixer(5, 48, 16, 32, 72, 56, 0.125, 300000.0, (2.5, 128, 24.0, 1.5)), DENSE(136)),
        _layer(_mixer(5, 48, 16, 32, 72, 56, 0.125, 300000.0, (2.5, 128, 24.0, 1.5)), MOE(9, 3, 40)),
    ],
    "loop": {"start": 1, "stop": 2, "times": 3},
}
# S: the whole model is one looped run with a single pass; rotation that turns fewer dimensions than the rotated part has.
KAKI_S = {
    "architecture": "Kakipel", "vocab": 150, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(4, 8, 16, 8, 24, 8, 0.35, 3000.0, (3.0, 48, 4.0, 0.5), dims=12), DENSE(40)),
        _layer(_mixer(2, 16, 8, 32, 16, 40, 0.3, 3000.0), MOE(2, 1, 56)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 1},
}
CONFIGS = {"P": KAKI_P, "Q": KAKI_Q, "R": KAKI_R, "S": KAKI_S}
PAGE_SIZE = {"P": 8, "Q": 16, "R": 16, "S": 4}


def config_dict(name: str, **changes) -> dict:
    out = copy.deepcopy(CONFIGS[name])
    out.update(changes)
    return out


def make_kakipel_folder(tmp_path, name: str, seed: int = 0, dtype=torch.float32, sharpen: float = 1.0, std: float = 0.08,
                        all_experts: bool = False) -> str:
    """A random-weights folder for configuration `name`.  `sharpen` multiplies every mixer's score scale, so that the
    softmax picks out single keys and a wrong or missing key shows in the logits.  `all_experts`: every routed layer
    chooses all its experts - for comparisons in bfloat16, where rounding may turn a close call between two experts the
    other way than the plain implementation's float64 does, which changes a position's logits by far more than rounding
    (the choice itself is held to the plain implementation in float32 and at kernel level)."""
    import kvcache_b200  # registers the architectures  # noqa: F401
    from kvcache_b200.config import config_from_dict
    from kvcache_b200.weights import write_random_model
    data = config_dict(name, initializer_range=std)
    for layer in data["layers"]:
        layer["mixer"]["scale"] *= sharpen
        if all_experts and layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    folder = os.path.join(str(tmp_path), f"kaki_{name}_{seed}_{sharpen}_{int(all_experts)}")
    write_random_model(folder, config_from_dict(data), seed, dtype)
    return folder
